// Sampling records and the gather producer shared by the tensor-core forward, the weight-gradient and
// the sampling-gradient kernels.
//
// Everything that depends only on (clip, offset group, tap, output voxel) -- the sampling position exactly
// as the reference forms it (integer base converted once + offset, one fp add; csrc/ops/dconv3d_gpu.cu:192-194,
// or the dilation-field synthesis of utils/grid.py:97), its floor corners, which corners are readable, the
// eight trilinear weights and the modulation value -- is computed ONCE per call by sample_records_kernel with
// the same make_sample() as every other kernel (so integer corners stay bit-identical across tiers), and the
// inner loops of the consumers contain no integer division, no strided offset read and no weight arithmetic.
//
// Two record streams, both [B][G][K][V]:
//   pos  float4 {z, y, x, mask}                                    -> sampling-gradient kernel
//   gat  3 x uint4 (48 B): {voff, steps, -, -}, w0..w3, w4..w7      -> gather producers (forward, dW)
//        voff  = element offset (no channel term) of the CLAMPED corner 000 inside the clip's channels-last
//                staging: per axis the floor index if it is inside the volume, else the ceil index if that is,
//                else 0
//        steps = bit 0/1/2 set when the x/y/z neighbour (+1) exists AND the floor index is inside, i.e. when
//                corner 1 of that axis is a different, readable voxel; otherwise both corners of the axis read
//                the same (readable) voxel
//        wj    = half2 {a_j*mask, a_j*mask}: trilinear weight x modulation, rounded to fp16, duplicated; ZERO
//                for every corner that does not contribute to the forward sample.  In the fp32-parity mode
//                the same 48 bytes hold {voff, steps, w0, w1}, w2..w5, {w6, w7, -, -} with fp32 weights.
//   so a producer issues 8 unconditional loads of readable addresses and lets the zero weights discard the
//   stand-ins (the staging is kept finite, so 0 x stand-in = 0): no predicate, no zero-fill.
#pragma once

#include <cuda_fp16.h>

#include "d2c_common.cuh"
#include "sm100_ptx.cuh"

namespace d2c {
namespace {

__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }
__device__ __forceinline__ __half2 bits_h2(uint32_t u) { return *reinterpret_cast<__half2*>(&u); }

// kShared: the coordinates do not depend on the offset group (dilation field): a thread serves one (voxel, tap)
// and all groups, computing the position, corners and weights once and applying each group's modulation.
template <typename Coords, bool kShared>
static __global__ void __launch_bounds__(256)
sample_records_kernel(Geom g, Coords coords, const float* __restrict__ mask, long long mask_bstride, int mask_act,
                      float4* __restrict__ pos, uint4* __restrict__ gat, int f32_weights) {
  const int v = blockIdx.x * 256 + threadIdx.x;
  if (v >= g.V) return;
  const int tap = kShared ? blockIdx.y : blockIdx.y % g.K, b = blockIdx.z;
  const int grp_beg = kShared ? 0 : blockIdx.y / g.K, grp_end = kShared ? g.G : grp_beg + 1;
  int bz, by, bx;
  voxel_tap_base(g, v, tap, bz, by, bx);
  float z, y, x;
  coords.get(g, b, grp_beg, tap, v, bz, by, bx, z, y, x);
  const Sample<float> s = make_sample(g, z, y, x);
  float a[8];
  sample_weights(s, a);
  const unsigned valid = s.inside ? s.valid : 0u;
  int cz, cy, cx;
  unsigned steps = 0;
  {
    const bool z0ok = s.z0 >= 0 && s.z0 < g.D, z1ok = s.z0 + 1 >= 0 && s.z0 + 1 < g.D;
    const bool y0ok = s.y0 >= 0 && s.y0 < g.H, y1ok = s.y0 + 1 >= 0 && s.y0 + 1 < g.H;
    const bool x0ok = s.x0 >= 0 && s.x0 < g.W, x1ok = s.x0 + 1 >= 0 && s.x0 + 1 < g.W;
    cz = z0ok ? s.z0 : (z1ok ? s.z0 + 1 : 0);
    cy = y0ok ? s.y0 : (y1ok ? s.y0 + 1 : 0);
    cx = x0ok ? s.x0 : (x1ok ? s.x0 + 1 : 0);
    steps = (x0ok && x1ok ? 1u : 0u) | (y0ok && y1ok ? 2u : 0u) | (z0ok && z1ok ? 4u : 0u);
  }
  const int voff = ((cz * g.H + cy) * g.W + cx) * g.Cin;
  for (int grp = grp_beg; grp < grp_end; ++grp) {
    const long long i = (((long long)b * g.G + grp) * g.K + tap) * g.V + v;
    // the mask as the op receives it, or the predictor's logits read in place and activated here
    const float m = mask ? mask_act_value(mask_act, __ldg(mask + (mask_bstride ? (long long)b * mask_bstride +
                                                          ((long long)grp * g.K + tap) * g.V + v : i)))
                         : 1.f;
    if (pos) pos[i] = make_float4(z, y, x, m);
    if (gat) {
      uint4* o = gat + 3 * i;
      if (f32_weights) {
        // fp32-parity mode: the 48 bytes hold the eight products a_j*mask in fp32
        uint32_t f[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) f[j] = ((valid >> j) & 1u) ? __float_as_uint(a[j] * m) : 0u;
        o[0] = make_uint4((uint32_t)voff, steps, f[0], f[1]);
        o[1] = make_uint4(f[2], f[3], f[4], f[5]);
        o[2] = make_uint4(f[6], f[7], 0u, 0u);
      } else {
        uint32_t w[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) w[j] = ((valid >> j) & 1u) ? h2_bits(__float2half2_rn(a[j] * m)) : 0u;
        o[0] = make_uint4((uint32_t)voff, steps, 0u, 0u);
        o[1] = make_uint4(w[0], w[1], w[2], w[3]);
        o[2] = make_uint4(w[4], w[5], w[6], w[7]);
      }
    }
  }
}

template <typename Coords>
struct CoordsSharedAcrossGroups { static constexpr bool value = false; };
template <typename T>
struct CoordsSharedAcrossGroups<FieldCoords<T>> { static constexpr bool value = true; };

template <typename Coords>
static int launch_sample_records(const Geom& g, const Coords& coords, const float* mask, const HeadCfg& head, float4* pos,
                                 uint4* gat, cudaStream_t st, bool f32_weights = false) {
  constexpr bool kShared = CoordsSharedAcrossGroups<Coords>::value;
  dim3 grid((unsigned)((g.V + 255) / 256), (unsigned)(kShared ? g.K : g.G * g.K), (unsigned)g.B);
  if (grid.y > 65535 || grid.z > 65535) return D2C_ERR_TOO_LARGE;
  sample_records_kernel<Coords, kShared><<<grid, 256, 0, st>>>(g, coords, mask, head.mask_bstride, head.mask_act, pos, gat,
                                                              f32_weights ? 1 : 0);
  D2C_LAUNCH_CHECK();
  return D2C_OK;
}

inline size_t pos_records_bytes(const Geom& g) {
  return align_up((size_t)g.B * g.G * g.K * g.V * sizeof(float4), 256);
}
inline size_t gather_records_bytes(const Geom& g) {
  return align_up((size_t)g.B * g.G * g.K * g.V * 3 * sizeof(uint4), 256);
}

// Element strides of the channels-last staging of x within one clip.
struct ClStrides {
  int dz, dy, dx;   // H*W*Cin, W*Cin, Cin
};

// One A-tile item = the 8 channels [ch0, ch0+8) of one modulated trilinear sample, blended in packed fp16
// (the weights already carry the modulation), converted to bf16 and stored (16 bytes) in the swizzled A tile.
// The work is split in two so that a producer can put the corners of several items in flight before the first
// blend: load_corners issues the 8 corner loads of one item (all unconditional, see the record format above),
// blend_store consumes them.   xb_ch: channels-last fp16 staging of the clip, advanced to the item's channel.
__device__ __forceinline__ void load_corners(const __half* __restrict__ xb_ch, ClStrides cs, uint32_t voff,
                                             uint32_t steps, uint4 (&c)[8]) {
  const int dx = (steps & 1u) ? cs.dx : 0, dy = (steps & 2u) ? cs.dy : 0, dz = (steps & 4u) ? cs.dz : 0;
  const __half* p0 = xb_ch + voff;
  const __half* p1 = p0 + dz;
  c[0] = ptx::ldg_nc_v4(p0);
  c[1] = ptx::ldg_nc_v4(p0 + dx);
  c[2] = ptx::ldg_nc_v4(p0 + dy);
  c[3] = ptx::ldg_nc_v4(p0 + dy + dx);
  c[4] = ptx::ldg_nc_v4(p1);
  c[5] = ptx::ldg_nc_v4(p1 + dx);
  c[6] = ptx::ldg_nc_v4(p1 + dy);
  c[7] = ptx::ldg_nc_v4(p1 + dy + dx);
}

// Returns the 16 bytes it stored (a caller that also keeps the samples for the backward writes them to global).
__device__ __forceinline__ uint4 blend_store(const uint4 (&c)[8], uint4 w03, uint4 w47, uint32_t dst) {
  const uint32_t w[8] = {w03.x, w03.y, w03.z, w03.w, w47.x, w47.y, w47.z, w47.w};
  __half2 acc[4];
#pragma unroll
  for (int e = 0; e < 4; ++e) acc[e] = __float2half2_rn(0.f);
#pragma unroll
  for (int j = 0; j < 8; ++j) {   // corner order 000..111, as the reference's interpolation chain
    const __half2 wj = bits_h2(w[j]);
    acc[0] = __hfma2(bits_h2(c[j].x), wj, acc[0]);
    acc[1] = __hfma2(bits_h2(c[j].y), wj, acc[1]);
    acc[2] = __hfma2(bits_h2(c[j].z), wj, acc[2]);
    acc[3] = __hfma2(bits_h2(c[j].w), wj, acc[3]);
  }
  uint4 out;
  float2 f;
  f = __half22float2(acc[0]); out.x = ptx::pack_bf16x2(f.x, f.y);
  f = __half22float2(acc[1]); out.y = ptx::pack_bf16x2(f.x, f.y);
  f = __half22float2(acc[2]); out.z = ptx::pack_bf16x2(f.x, f.y);
  f = __half22float2(acc[3]); out.w = ptx::pack_bf16x2(f.x, f.y);
  ptx::sts_v4(dst, out);
  return out;
}

// ---- fp32-parity mode ("bf16x3"): fp32 staging, fp32 blend, bf16 hi/lo split -------------------------------
// One item = 4 channels (16 bytes of fp32) of one sample.  The blended value v is written twice into the
// 128-byte A row of a 32-channel unit: hi = bf16(v) at channel column c, lo = bf16(v - hi) at column 32 + c,
// so that the MMA issuer can form a_hi*b_hi + a_lo*b_hi + a_hi*b_lo from K sub-blocks of ONE tile pair.
__device__ __forceinline__ void load_corners_f32(const float* __restrict__ xb_ch, ClStrides cs, uint32_t voff,
                                                 uint32_t steps, uint4 (&c)[8]) {
  const int dx = (steps & 1u) ? cs.dx : 0, dy = (steps & 2u) ? cs.dy : 0, dz = (steps & 4u) ? cs.dz : 0;
  const float* p0 = xb_ch + voff;
  const float* p1 = p0 + dz;
  c[0] = ptx::ldg_nc_v4(p0);
  c[1] = ptx::ldg_nc_v4(p0 + dx);
  c[2] = ptx::ldg_nc_v4(p0 + dy);
  c[3] = ptx::ldg_nc_v4(p0 + dy + dx);
  c[4] = ptx::ldg_nc_v4(p1);
  c[5] = ptx::ldg_nc_v4(p1 + dx);
  c[6] = ptx::ldg_nc_v4(p1 + dy);
  c[7] = ptx::ldg_nc_v4(p1 + dy + dx);
}

// w: the eight fp32 products a_j*mask (corner order 000..111, the reference's interpolation chain).
// dst_hi / dst_lo: shared-memory addresses of the 8-byte hi and lo slots of this item.
// Returns {hi (8 bytes), lo (8 bytes)} as stored.
__device__ __forceinline__ uint4 blend_split_store(const uint4 (&c)[8], const float (&w)[8], uint32_t dst_hi,
                                                   uint32_t dst_lo) {
  float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    v[0] = __fmaf_rn(__uint_as_float(c[j].x), w[j], v[0]);
    v[1] = __fmaf_rn(__uint_as_float(c[j].y), w[j], v[1]);
    v[2] = __fmaf_rn(__uint_as_float(c[j].z), w[j], v[2]);
    v[3] = __fmaf_rn(__uint_as_float(c[j].w), w[j], v[3]);
  }
  const uint32_t h01 = ptx::pack_bf16x2(v[0], v[1]), h23 = ptx::pack_bf16x2(v[2], v[3]);
  const uint32_t l01 = ptx::pack_bf16x2(v[0] - ptx::bf16_lo(h01), v[1] - ptx::bf16_hi(h01));
  const uint32_t l23 = ptx::pack_bf16x2(v[2] - ptx::bf16_lo(h23), v[3] - ptx::bf16_hi(h23));
  ptx::sts_v2(dst_hi, make_uint2(h01, h23));
  ptx::sts_v2(dst_lo, make_uint2(l01, l23));
  return make_uint4(h01, h23, l01, l23);
}

// The same item written with ONE 16-byte store per lane: lanes 2i and 2i+1 of a warp hold neighbouring 4-channel
// items of the same row, so the even lane takes both hi halves (one 16-byte chunk of the row's hi part) and the odd
// lane both lo halves.  dst_chunk: shared-memory address of the 16-byte chunk THIS lane writes (hi chunk for an even
// lane, lo chunk for an odd one).  Returns the 16 bytes stored.  Two 8-byte stores per lane cost 2.6x the
// shared-memory wavefronts of this form (bank conflicts between the half-chunks of different rows).
__device__ __forceinline__ uint4 blend_split_store16(const uint4 (&c)[8], const float (&w)[8], uint32_t dst_chunk,
                                                     bool odd_lane) {
  float v[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    v[0] = __fmaf_rn(__uint_as_float(c[j].x), w[j], v[0]);
    v[1] = __fmaf_rn(__uint_as_float(c[j].y), w[j], v[1]);
    v[2] = __fmaf_rn(__uint_as_float(c[j].z), w[j], v[2]);
    v[3] = __fmaf_rn(__uint_as_float(c[j].w), w[j], v[3]);
  }
  const uint32_t h01 = ptx::pack_bf16x2(v[0], v[1]), h23 = ptx::pack_bf16x2(v[2], v[3]);
  const uint32_t l01 = ptx::pack_bf16x2(v[0] - ptx::bf16_lo(h01), v[1] - ptx::bf16_hi(h01));
  const uint32_t l23 = ptx::pack_bf16x2(v[2] - ptx::bf16_lo(h23), v[3] - ptx::bf16_hi(h23));
  // even lane gives its lo and receives the odd lane's hi; the odd lane the other way round
  const uint32_t t0 = __shfl_xor_sync(0xffffffffu, odd_lane ? h01 : l01, 1);
  const uint32_t t1 = __shfl_xor_sync(0xffffffffu, odd_lane ? h23 : l23, 1);
  const uint4 out = odd_lane ? make_uint4(t0, t1, l01, l23) : make_uint4(h01, h23, t0, t1);
  ptx::sts_v4(dst_chunk, out);
  return out;
}

}  // namespace
}  // namespace d2c
