// Shared-memory tile kernels for the common depthwise case: 3x3x3 kernel, stride 1, dilation 1,
// padding 1, channel multiplier 1 (the ir-CSN bottleneck conv).  HBM-bound by design: a block stages a
// (ZC+2) x (YC+2) x (W+2) zero-bordered slab of ONE channel of ONE clip in shared memory with coalesced
// row loads, so every input element is read from global memory once (plus the slab halo) and the inner
// loop has no bounds checks; each thread then produces strips of 4 outputs along x from a 3x3x6 register
// window (54 shared-memory reads for 108 MACs).
//   forward:         out = conv(x, w) + bias
//   input gradient:  grad_x = conv(grad_out, w flipped)        (same kernel, flip = 1)
//   weight gradient: dW[c, t] = sum_{b, v} grad_out[b, c, v] * x[b, c, v + delta_t]   (27 accumulators/thread)
// Reference: ops/fast-depthwise-conv3d/csrc/grouped_conv3d.cu:22-276.
#pragma once

#include "d2c_common.cuh"

namespace d2c {
namespace {

struct DwTilePlan {
  int ZC, YC, tz, ty;
  size_t smem_conv, smem_wgrad;
};

inline bool dw_tile_plan(const Geom& g, size_t esize, DwTilePlan* p) {
  if (!(g.kd == 3 && g.kh == 3 && g.kw == 3 && g.sd == 1 && g.sh == 1 && g.sw == 1 && g.dd == 1 && g.dh == 1 &&
        g.dw == 1 && g.pd == 1 && g.ph == 1 && g.pw == 1 && g.Cout == g.Cin))
    return false;
  auto slab = [&](int zc, int yc) { return (size_t)(zc + 2) * (yc + 2) * (g.W + 2) * esize; };
  auto both = [&](int zc, int yc) { return slab(zc, yc) + (size_t)zc * yc * g.W * esize; };
  const size_t budget = 100 * 1024;     // two blocks per SM
  int ZC = g.D, YC = g.H;
  while (both(ZC, YC) > budget && ZC > 2) ZC = (ZC + 1) / 2;
  while (both(ZC, YC) > budget && YC > 4) YC = (YC + 1) / 2;
  if (both(ZC, YC) > 200 * 1024) return false;
  p->ZC = ZC; p->YC = YC;
  p->tz = (g.D + ZC - 1) / ZC; p->ty = (g.H + YC - 1) / YC;
  p->smem_conv = slab(ZC, YC);
  p->smem_wgrad = both(ZC, YC);
  if ((long long)g.B * g.Cin * p->tz * p->ty > 0x7fffffffLL) return false;
  return true;
}

template <typename T, typename A>
__device__ __forceinline__ A dwt_ld(const T* p);
template <> __device__ __forceinline__ float dwt_ld<float, float>(const float* p) { return __ldg(p); }
template <> __device__ __forceinline__ double dwt_ld<double, double>(const double* p) { return __ldg(p); }
template <> __device__ __forceinline__ float dwt_ld<__half, float>(const __half* p) { return __half2float(__ldg(p)); }
template <typename T, typename A> __device__ __forceinline__ T dwt_st(A a) { return (T)a; }
template <> __device__ __forceinline__ __half dwt_st<__half, float>(float a) { return __float2half_rn(a); }

// Stages the zero-bordered slab [z0-1, z0+ZC] x [y0-1, y0+YC] x [-1, W] of one channel plane.
template <typename T, typename A>
__device__ __forceinline__ void dwt_load_slab(const Geom& g, const T* __restrict__ src, int z0, int y0, int ZC, int YC,
                                              A* __restrict__ xs) {
  const int W2 = g.W + 2, Y2 = YC + 2, rows = (ZC + 2) * Y2;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int r = warp; r < rows; r += nwarps) {
    const int fz = r / Y2, fy = r - fz * Y2;
    const int z = z0 - 1 + fz, y = y0 - 1 + fy;
    const bool ok = z >= 0 && z < g.D && y >= 0 && y < g.H;
    const T* rp = src + ((long long)z * g.H + y) * g.W;
    A* dp = xs + (long long)r * W2;
    for (int fx = lane; fx < W2; fx += 32) {
      const int x = fx - 1;
      dp[fx] = (ok && x >= 0 && x < g.W) ? dwt_ld<T, A>(rp + x) : (A)0;
    }
  }
}

template <typename T, typename A>
__global__ void __launch_bounds__(256)
dw_tile_conv_kernel(Geom g, int ZC, int YC, int tz, int ty, const T* __restrict__ in, const T* __restrict__ w,
                    const T* __restrict__ bias, T* __restrict__ out, int flip) {
  extern __shared__ __align__(16) unsigned char dwt_smem[];
  A* xs = reinterpret_cast<A*>(dwt_smem);
  int blk = blockIdx.x;
  const int iy = blk % ty; blk /= ty;
  const int iz = blk % tz; blk /= tz;
  const int c = blk % g.Cin, b = blk / g.Cin;
  const int z0 = iz * ZC, y0 = iy * YC, W2 = g.W + 2, Y2 = YC + 2;
  const long long plane = ((long long)b * g.Cin + c) * g.Vin;
  dwt_load_slab<T, A>(g, in + plane, z0, y0, ZC, YC, xs);
  A wk[27];
#pragma unroll
  for (int t = 0; t < 27; ++t) wk[t] = dwt_ld<T, A>(w + (long long)c * 27 + (flip ? 26 - t : t));
  const A bb = bias ? dwt_ld<T, A>(bias + c) : (A)0;
  __syncthreads();
  const int nsx = (g.W + 3) / 4, nstrips = ZC * YC * nsx;
  for (int s = threadIdx.x; s < nstrips; s += blockDim.x) {
    const int sx = s % nsx, yy = (s / nsx) % YC, zz = s / (nsx * YC);
    const int z = z0 + zz, y = y0 + yy, x0 = sx * 4;
    if (z >= g.D || y >= g.H) continue;
    A acc[4] = {bb, bb, bb, bb};
#pragma unroll
    for (int kz = 0; kz < 3; ++kz)
#pragma unroll
      for (int ky = 0; ky < 3; ++ky) {
        const A* row = xs + ((long long)(zz + kz) * Y2 + (yy + ky)) * W2 + x0;   // column q <-> input x = x0+q-1
        A v[6];
#pragma unroll
        for (int q = 0; q < 6; ++q) v[q] = (x0 + q < W2) ? row[q] : (A)0;
#pragma unroll
        for (int kx = 0; kx < 3; ++kx) {
          const A wv = wk[(kz * 3 + ky) * 3 + kx];
#pragma unroll
          for (int i = 0; i < 4; ++i) acc[i] += wv * v[i + kx];
        }
      }
    T* op = out + plane + ((long long)z * g.H + y) * g.W + x0;
#pragma unroll
    for (int i = 0; i < 4; ++i)
      if (x0 + i < g.W) op[i] = dwt_st<T, A>(acc[i]);
  }
}

// One block per (channel, slab tile, slice of clips); 27 accumulators per thread, block reduction, then one
// atomic per tap into partial[Cout][27] (accumulator type, zeroed beforehand).
template <typename T, typename A>
__global__ void __launch_bounds__(256)
dw_tile_wgrad_kernel(Geom g, int ZC, int YC, int tz, int ty, int clips_per_block, const T* __restrict__ gy,
                     const T* __restrict__ x, A* __restrict__ partial) {
  extern __shared__ __align__(16) unsigned char dwt_smem[];
  const int W2 = g.W + 2, Y2 = YC + 2;
  A* xs = reinterpret_cast<A*>(dwt_smem);
  A* gs = xs + (long long)(ZC + 2) * Y2 * W2;
  int blk = blockIdx.x;
  const int iy = blk % ty; blk /= ty;
  const int iz = blk % tz; blk /= tz;
  const int c = blk % g.Cin, bs = blk / g.Cin;
  const int z0 = iz * ZC, y0 = iy * YC;
  const int bbeg = bs * clips_per_block, bend = min(g.B, bbeg + clips_per_block);
  A acc[27];
#pragma unroll
  for (int t = 0; t < 27; ++t) acc[t] = (A)0;
  const int nsx = (g.W + 3) / 4, nstrips = ZC * YC * nsx;
  for (int b = bbeg; b < bend; ++b) {
    const long long plane = ((long long)b * g.Cin + c) * g.Vin;
    __syncthreads();
    dwt_load_slab<T, A>(g, x + plane, z0, y0, ZC, YC, xs);
    for (int e = threadIdx.x; e < ZC * YC * g.W; e += blockDim.x) {
      const int xx = e % g.W, yy = (e / g.W) % YC, zz = e / (g.W * YC);
      const int z = z0 + zz, y = y0 + yy;
      gs[e] = (z < g.D && y < g.H) ? dwt_ld<T, A>(gy + plane + ((long long)z * g.H + y) * g.W + xx) : (A)0;
    }
    __syncthreads();
    for (int s = threadIdx.x; s < nstrips; s += blockDim.x) {
      const int sx = s % nsx, yy = (s / nsx) % YC, zz = s / (nsx * YC);
      const int x0 = sx * 4;
      A g4[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) g4[i] = (x0 + i < g.W) ? gs[((long long)zz * YC + yy) * g.W + x0 + i] : (A)0;
#pragma unroll
      for (int kz = 0; kz < 3; ++kz)
#pragma unroll
        for (int ky = 0; ky < 3; ++ky) {
          const A* row = xs + ((long long)(zz + kz) * Y2 + (yy + ky)) * W2 + x0;
          A v[6];
#pragma unroll
          for (int q = 0; q < 6; ++q) v[q] = (x0 + q < W2) ? row[q] : (A)0;
#pragma unroll
          for (int kx = 0; kx < 3; ++kx) {
            A sacc = (A)0;
#pragma unroll
            for (int i = 0; i < 4; ++i) sacc += g4[i] * v[i + kx];
            acc[(kz * 3 + ky) * 3 + kx] += sacc;
          }
        }
    }
  }
  __syncthreads();
  A* red = xs;    // reuse the slab: [8 warps][27]
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int t = 0; t < 27; ++t) {
    A sv = acc[t];
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) sv += __shfl_xor_sync(0xffffffffu, sv, o);
    if (lane == 0) red[warp * 27 + t] = sv;
  }
  __syncthreads();
  if (threadIdx.x < 27) {
    A sv = (A)0;
    for (int wp = 0; wp < (int)(blockDim.x >> 5); ++wp) sv += red[wp * 27 + threadIdx.x];
    atomicAdd(partial + (long long)c * 27 + threadIdx.x, sv);
  }
}

template <typename T, typename A>
int dw_tile_conv(const Geom& g, const DwTilePlan& p, const T* in, const T* w, const T* bias, T* out, int flip,
                 cudaStream_t st) {
  D2C_CUDA_TRY(cudaFuncSetAttribute(dw_tile_conv_kernel<T, A>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)p.smem_conv));
  const unsigned blocks = (unsigned)((long long)g.B * g.Cin * p.tz * p.ty);
  dw_tile_conv_kernel<T, A><<<blocks, 256, p.smem_conv, st>>>(g, p.ZC, p.YC, p.tz, p.ty, in, w, bias, out, flip);
  D2C_LAUNCH_CHECK();
  return D2C_OK;
}

template <typename T, typename A>
int dw_tile_wgrad(const Geom& g, const DwTilePlan& p, const T* gy, const T* x, A* partial, cudaStream_t st) {
  D2C_CUDA_TRY(cudaFuncSetAttribute(dw_tile_wgrad_kernel<T, A>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)p.smem_wgrad));
  // enough (channel, tile, clip-slice) blocks for a few waves
  const long long per_slice = (long long)g.Cin * p.tz * p.ty;
  long long slices = (148LL * 6 + per_slice - 1) / per_slice;
  if (slices > g.B) slices = g.B;
  if (slices < 1) slices = 1;
  const int cpb = (int)((g.B + slices - 1) / slices);
  const unsigned blocks = (unsigned)(per_slice * ((g.B + cpb - 1) / cpb));
  dw_tile_wgrad_kernel<T, A><<<blocks, 256, p.smem_wgrad, st>>>(g, p.ZC, p.YC, p.tz, p.ty, cpb, gy, x, partial);
  D2C_LAUNCH_CHECK();
  return D2C_OK;
}

}  // namespace
}  // namespace d2c
