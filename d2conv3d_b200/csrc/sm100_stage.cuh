// Operand staging kernels shared by the tensor-core forward and backward.
#pragma once

#include <cuda_fp16.h>

#include "sm100_ptx.cuh"

namespace d2c {
namespace {

// round-to-nearest fp32 -> fp16 with saturation to the largest finite half (|x| > 65504 is clamped)
__device__ __forceinline__ uint32_t pack_f16x2_sat(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.satfinite.f16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}

// x [B][C][Vin] fp32 -> x_cl [B][Vin][C] fp16 (channels-last).  Block: 64 channels x 32 voxels.
static __global__ void __launch_bounds__(256)
stage_input_cl_f16_kernel(int C, long long Vin, const float* __restrict__ x, __half* __restrict__ x_cl) {
  __shared__ float tile[64][33];
  const int b = blockIdx.z, c0 = blockIdx.y * 64;
  const long long v0 = (long long)blockIdx.x * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 8 warps
  for (int cc = ty; cc < 64; cc += 8) {
    const long long v = v0 + tx;
    tile[cc][tx] = (v < Vin && c0 + cc < C) ? __ldg(x + ((long long)b * C + c0 + cc) * Vin + v) : 0.f;
  }
  __syncthreads();
  for (int vv = ty; vv < 32; vv += 8) {
    const long long v = v0 + vv;
    if (v < Vin && c0 + 2 * tx + 1 < C) {
      const uint32_t pk = pack_f16x2_sat(tile[2 * tx][vv], tile[2 * tx + 1][vv]);
      *reinterpret_cast<uint32_t*>(x_cl + ((long long)b * Vin + v) * C + c0 + 2 * tx) = pk;
    }
  }
}

// x [B][C][Vin] fp32 -> x_cl [B][Vin][C] fp32 (channels-last) for the fp32-parity mode.  Infinities are
// replaced by the largest finite float: the gather multiplies stand-in corners by zero weights, which must
// give zero.
static __global__ void __launch_bounds__(256)
stage_input_cl_f32_kernel(int C, long long Vin, const float* __restrict__ x, float* __restrict__ x_cl) {
  __shared__ float tile[64][33];
  const int b = blockIdx.z, c0 = blockIdx.y * 64;
  const long long v0 = (long long)blockIdx.x * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;   // 8 warps
  for (int cc = ty; cc < 64; cc += 8) {
    const long long v = v0 + tx;
    float f = (v < Vin && c0 + cc < C) ? __ldg(x + ((long long)b * C + c0 + cc) * Vin + v) : 0.f;
    if (isinf(f)) f = copysignf(3.402823466e+38f, f);
    tile[cc][tx] = f;
  }
  __syncthreads();
  for (int vv = ty; vv < 32; vv += 8) {
    const long long v = v0 + vv;
    if (v < Vin && c0 + 2 * tx + 1 < C)
      *reinterpret_cast<float2*>(x_cl + ((long long)b * Vin + v) * C + c0 + 2 * tx) =
          make_float2(tile[2 * tx][vv], tile[2 * tx + 1][vv]);
  }
}

}  // namespace
}  // namespace d2c
