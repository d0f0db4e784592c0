// Sampling-coordinate records and the gather producer shared by the tensor-core forward, the
// weight-gradient and the sampling-gradient kernels.
//
// A record is the float4 {z, y, x, mask} of one (clip, offset group, tap, output voxel): the sampling
// position exactly as the reference forms it (integer base converted once + offset, one fp add;
// csrc/ops/dconv3d_gpu.cu:192-194 -- or the dilation-field synthesis of utils/grid.py:97) and the
// modulation value (1 when there is no mask).  They are computed ONCE per call by
// coord_records_kernel; consumers re-derive floor corners / validity / weights from (z, y, x) with the
// same make_sample() as every other kernel, so integer corners stay bit-identical across tiers while the
// integer div/mod and the strided offset reads leave the inner loops.
// Layout: [B][G][K][V] float4, i.e. the 128 records of a voxel tile of one (group, tap) are 2 KB contiguous.
#pragma once

#include "d2c_common.cuh"
#include "sm100_ptx.cuh"

namespace d2c {
namespace {

template <typename Coords>
static __global__ void __launch_bounds__(256)
coord_records_kernel(Geom g, Coords coords, const float* __restrict__ mask, float4* __restrict__ recs) {
  const int v = blockIdx.x * 256 + threadIdx.x;
  if (v >= g.V) return;
  const int tap = blockIdx.y % g.K, grp = blockIdx.y / g.K, b = blockIdx.z;
  int bz, by, bx;
  voxel_tap_base(g, v, tap, bz, by, bx);
  float z, y, x;
  coords.get(g, b, grp, tap, v, bz, by, bx, z, y, x);
  const long long i = (((long long)b * g.G + grp) * g.K + tap) * g.V + v;
  const float m = mask ? __ldg(mask + i) : 1.f;
  recs[i] = make_float4(z, y, x, m);
}

template <typename Coords>
static int launch_coord_records(const Geom& g, const Coords& coords, const float* mask, float4* recs,
                                cudaStream_t st) {
  dim3 grid((unsigned)((g.V + 255) / 256), (unsigned)(g.G * g.K), (unsigned)g.B);
  if (grid.y > 65535 || grid.z > 65535) return D2C_ERR_TOO_LARGE;
  coord_records_kernel<Coords><<<grid, 256, 0, st>>>(g, coords, mask, recs);
  D2C_LAUNCH_CHECK();
  return D2C_OK;
}

inline size_t coord_records_bytes(const Geom& g) {
  return align_up((size_t)g.B * g.G * g.K * g.V * sizeof(float4), 256);
}

// Element strides of the channels-last staging of x within one clip.
struct ClStrides {
  int dz, dy, dx;   // H*W*Cin, W*Cin, Cin
};

// One A-tile item: the 8 channels [ch0, ch0+8) of the modulated trilinear sample described by `rec`,
// packed to bf16 and stored (16 bytes) at shared-memory address `dst`.
//   xb: channels-last bf16 staging of the clip ([Vin][Cin]).
// Corners outside the volume (or a position failing the forward's early-out) are not loaded.
__device__ __forceinline__ void produce_item_rec(const Geom& g, const __nv_bfloat16* __restrict__ xb, ClStrides cs,
                                                 float4 rec, int ch0, uint32_t dst) {
  const Sample<float> s = make_sample(g, rec.x, rec.y, rec.z);
  float a[8];
  sample_weights(s, a);
  const unsigned valid = s.inside ? s.valid : 0u;
  const int off0 = ((s.z0 * g.H + s.y0) * g.W + s.x0) * g.Cin + ch0;
  uint4 c[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const int off = off0 + (j >> 2) * cs.dz + ((j >> 1) & 1) * cs.dy + (j & 1) * cs.dx;
    c[j] = ((valid >> j) & 1u) ? ptx::ldg_nc_v4(xb + off) : make_uint4(0u, 0u, 0u, 0u);
  }
  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) {   // corner order 000..111, fma chain as the reference's interpolation
    acc[0] = fmaf(ptx::bf16_lo(c[j].x), a[j], acc[0]);
    acc[1] = fmaf(ptx::bf16_hi(c[j].x), a[j], acc[1]);
    acc[2] = fmaf(ptx::bf16_lo(c[j].y), a[j], acc[2]);
    acc[3] = fmaf(ptx::bf16_hi(c[j].y), a[j], acc[3]);
    acc[4] = fmaf(ptx::bf16_lo(c[j].z), a[j], acc[4]);
    acc[5] = fmaf(ptx::bf16_hi(c[j].z), a[j], acc[5]);
    acc[6] = fmaf(ptx::bf16_lo(c[j].w), a[j], acc[6]);
    acc[7] = fmaf(ptx::bf16_hi(c[j].w), a[j], acc[7]);
  }
  const float m = rec.w;
  uint4 out;
  out.x = ptx::pack_bf16x2(m * acc[0], m * acc[1]);
  out.y = ptx::pack_bf16x2(m * acc[2], m * acc[3]);
  out.z = ptx::pack_bf16x2(m * acc[4], m * acc[5]);
  out.w = ptx::pack_bf16x2(m * acc[6], m * acc[7]);
  ptx::sts_v4(dst, out);
}

// Records of the kRows rows (r0, r0+kStride, ...) a gather thread owns in the tile starting at voxel v0.
// Rows past the end of the clip get {0,0,0,0}: a valid position with modulation 0, i.e. a zero row.
template <int kRows, int kStride>
__device__ __forceinline__ void load_row_records(const float4* __restrict__ recs, const Geom& g, int b, int grp,
                                                 int tap, int v0, int r0, float4 (&out)[kRows]) {
  const float4* p = recs + (((long long)b * g.G + grp) * g.K + tap) * g.V;
#pragma unroll
  for (int i = 0; i < kRows; ++i) {
    const int v = v0 + r0 + kStride * i;
    out[i] = (v < g.V) ? __ldg(p + v) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

}  // namespace
}  // namespace d2c
