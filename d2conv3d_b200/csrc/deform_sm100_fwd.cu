// Fused modulated-deformable conv3d forward for sm_100a: trilinear gather -> shared
// memory A tile -> tcgen05.mma (bf16 operands, fp32 accumulate in tensor memory) ->
// bias epilogue.  No column matrix is ever written to global memory.
//
// Replaces the reference's deformable_im2col_gpu_kernel + cuBLAS gemmStridedBatched +
// out.add_(bias) (csrc/ops/dconv3d_gpu.cu:111-203, :334-352, :555-557).
//
// GEMM view: M = output voxels (tiles of 128 consecutive voxels of one clip), N = Cout
// (whole, <= 512, in tensor memory), K = Cin*27 walked as slices of 64 input channels of
// one (offset group, tap).  All channels of a slice share their 8 trilinear corners, so
// with the input staged channels-last in bf16 each corner of a slice is ONE contiguous
// 128-byte line.
//
// Per CTA (persistent over tiles), 14 warps:
//   warps 0-3   epilogue: tcgen05.ld the 128 x N accumulator, add bias, store NCDHW
//   warp  4     one thread issues tcgen05.mma and the commits that free the stages
//   warp  5     one thread streams pre-swizzled weight slices with cp.async.bulk
//   warps 6-13  gather producers: coordinates, 8 corner loads (16 B per thread),
//               fp32 blend, modulation, bf16 pack, swizzled st.shared of the A tile
// Stage hand-off is by mbarriers; every wait is bounded (sm100_ptx.cuh).
#include "deform_sm100.h"
#include "sm100_ptx.cuh"
#include "sm100_stage.cuh"

namespace d2c {

namespace {

constexpr int kBM = 128;            // voxels per tile (UMMA M)
constexpr int kBK = 64;             // channels per K slice (128 bytes of bf16: one swizzle row)
constexpr int kAStages = 4;
constexpr int kAStageBytes = kBM * kBK * 2;   // 16 KB
constexpr int kMaxN = 512;
constexpr int kThreads = 448;
constexpr int kEpiWarps = 4, kMmaWarp = 4, kLoadWarp = 5, kGatherWarp0 = 6, kGatherWarps = 8;
constexpr int kGatherThreads = kGatherWarps * 32;
constexpr int kSmemLimit = 227 * 1024;

__device__ int g_sm100_status = 0;   // sticky: set when a bounded wait gave up

struct FwdParams {
  Geom g;
  const __nv_bfloat16* x_cl;   // [B][Vin][Cin] bf16 (channels-last staging of x)
  const __nv_bfloat16* w_sw;   // [S][N rows x 128 B], rows swizzled exactly as the smem B tile
  const float* mask;           // [B, G*K, V] or nullptr
  const float* bias;           // [Cout] or nullptr
  float* y;                    // [B, Cout, V]
  int N;                       // Cout
  int nh;                      // K slices per (group, tap) = cpg / 64
  int S;                       // slices per tile = G * K * nh
  int tiles_per_clip, n_tiles;
  int b_stages, b_stage_bytes;
  int tmem_cols;
};

struct SmemLayout {
  // offsets from the 1024-aligned base
  int a_off, b_off, bar_off, total;
};

__host__ __device__ inline SmemLayout smem_layout(int b_stages, int b_stage_bytes) {
  SmemLayout L;
  L.a_off = 0;
  L.b_off = kAStages * kAStageBytes;
  L.bar_off = L.b_off + b_stages * b_stage_bytes;
  L.total = L.bar_off + 256;
  return L;
}

// One A-tile item: voxel row r, 16-byte chunk j (8 channels).
template <typename Coords>
__device__ __forceinline__ void produce_item(const FwdParams& p, const Coords& coords, int b, int v, int grp,
                                             int tap, int ch0, uint32_t dst) {
  const Geom& g = p.g;
  float a[8];
  long long idx[8];
  float m = 0.f;
  if (v < g.V) {
    int bz, by, bx;
    voxel_tap_base(g, v, tap, bz, by, bx);
    float z, y, x;
    coords.get(g, b, grp, tap, v, bz, by, bx, z, y, x);
    const Sample<float> s = make_sample(g, z, y, x);
    sample_weights(s, a);
    m = p.mask ? __ldg(p.mask + (((long long)b * g.G + grp) * g.K + tap) * g.V + v) : 1.f;
    const unsigned valid = s.inside ? s.valid : 0u;
    // invalid corners: weight 0 and a clamped (always readable) address
    const int zc[2] = {min(max(s.z0, 0), g.D - 1), min(max(s.z0 + 1, 0), g.D - 1)};
    const int yc[2] = {min(max(s.y0, 0), g.H - 1), min(max(s.y0 + 1, 0), g.H - 1)};
    const int xc[2] = {min(max(s.x0, 0), g.W - 1), min(max(s.x0 + 1, 0), g.W - 1)};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (!((valid >> j) & 1u)) a[j] = 0.f;
      idx[j] = ((((long long)b * g.D + zc[j >> 2]) * g.H + yc[(j >> 1) & 1]) * g.W + xc[j & 1]) * g.Cin + ch0;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 8; ++j) { a[j] = 0.f; idx[j] = ch0; }
  }
  uint4 c[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) c[j] = ptx::ldg_nc_v4(p.x_cl + idx[j]);
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
  uint4 out;
  out.x = ptx::pack_bf16x2(m * acc[0], m * acc[1]);
  out.y = ptx::pack_bf16x2(m * acc[2], m * acc[3]);
  out.z = ptx::pack_bf16x2(m * acc[4], m * acc[5]);
  out.w = ptx::pack_bf16x2(m * acc[6], m * acc[7]);
  ptx::sts_v4(dst, out);
}

template <typename Coords>
__global__ void __launch_bounds__(kThreads, 1)
fwd_sm100_kernel(const FwdParams p, const Coords coords) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const SmemLayout L = smem_layout(p.b_stages, p.b_stage_bytes);
  const uint32_t a_base = base + L.a_off, b_base = base + L.b_off, bar_base = base + L.bar_off;
  // barrier slots (8 bytes each)
  auto a_full = [&](int s) { return bar_base + 8u * s; };
  auto a_empty = [&](int s) { return bar_base + 8u * (kAStages + s); };
  auto b_full = [&](int s) { return bar_base + 8u * (2 * kAStages + s); };
  auto b_empty = [&](int s) { return bar_base + 8u * (2 * kAStages + 4 + s); };
  const uint32_t acc_full = bar_base + 8u * (2 * kAStages + 8);
  const uint32_t acc_empty = bar_base + 8u * (2 * kAStages + 9);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + L.bar_off + 8 * (2 * kAStages + 10));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + L.bar_off + 8 * (2 * kAStages + 10) + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const Geom& g = p.g;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kAStages; ++s) { ptx::mbar_init(a_full(s), kGatherWarps); ptx::mbar_init(a_empty(s), 1); }
    for (int s = 0; s < p.b_stages; ++s) { ptx::mbar_init(b_full(s), 1); ptx::mbar_init(b_empty(s), 1); }
    ptx::mbar_init(acc_full, 1);
    ptx::mbar_init(acc_empty, kEpiWarps);
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == 0) {
    __syncwarp();
    ptx::tmem_alloc(ptx::smem_u32((const void*)tmem_slot), (uint32_t)p.tmem_cols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp < kEpiWarps) {
    // ===================== epilogue =====================
    int it = 0;
    for (int tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x, ++it) {
      const int b = tile / p.tiles_per_clip, v0 = (tile % p.tiles_per_clip) * kBM;
      if (!ptx::mbar_wait(acc_full, it & 1, abort_flag)) break;
      ptx::tc_fence_after();
      const int v = v0 + warp * 32 + lane;
      float* yb = p.y + (long long)b * g.Cout * g.V + v;
      for (int c0 = 0; c0 < p.N; c0 += 32) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, r);
        ptx::tmem_ld_wait();
        if (v < g.V) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const float bb = p.bias ? __ldg(p.bias + c0 + j) : 0.f;
            yb[(long long)(c0 + j) * g.V] = __uint_as_float(r[j]) + bb;
          }
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(acc_empty);
    }
  } else if (warp == kMmaWarp) {
    // ===================== MMA issuer =====================
    if (lane == 0) {
      int it = 0;          // tile iteration of this CTA
      uint32_t ka = 0, kb = 0;   // running slice counters (A ring, B ring)
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < p.n_tiles; tile += gridDim.x, ++it) {
        if (!ptx::mbar_wait(acc_empty, (it & 1) ^ 1, abort_flag)) break;
        ptx::tc_fence_after();
        for (int s = 0; s < p.S; ++s, ++ka, ++kb) {
          const int sa = ka % kAStages, sb = kb % p.b_stages;
          if (!ptx::mbar_wait(a_full(sa), (ka / kAStages) & 1, abort_flag)) { ok = false; break; }
          if (!ptx::mbar_wait(b_full(sb), (kb / p.b_stages) & 1, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint64_t adesc = ptx::umma_desc_kmajor_sw128(a_base + sa * kAStageBytes);
#pragma unroll
          for (int k = 0; k < kBK / 16; ++k) {
            for (int n0 = 0; n0 < p.N; n0 += 256) {
              const int nc = min(256, p.N - n0);
              const uint64_t bdesc = ptx::umma_desc_kmajor_sw128(b_base + sb * p.b_stage_bytes + n0 * 128);
              ptx::umma_bf16(tmem_base + (uint32_t)n0, adesc + (uint64_t)(2 * k), bdesc + (uint64_t)(2 * k),
                             ptx::umma_idesc_bf16_f32(kBM, nc), (s > 0 || k > 0) ? 1u : 0u);
            }
          }
          ptx::umma_commit(a_empty(sa));
          ptx::umma_commit(b_empty(sb));
        }
        if (ok) ptx::umma_commit(acc_full);
      }
    }
  } else if (warp == kLoadWarp) {
    // ===================== weight-slice loader =====================
    if (lane == 0) {
      uint32_t kb = 0;
      bool ok = true;
      for (int tile = blockIdx.x; ok && tile < p.n_tiles; tile += gridDim.x) {
        for (int s = 0; s < p.S; ++s, ++kb) {
          const int sb = kb % p.b_stages;
          if (!ptx::mbar_wait(b_empty(sb), ((kb / p.b_stages) & 1) ^ 1, abort_flag)) { ok = false; break; }
          ptx::mbar_arrive_expect_tx(b_full(sb), (uint32_t)p.b_stage_bytes);
          const uint8_t* src = reinterpret_cast<const uint8_t*>(p.w_sw) + (long long)s * p.b_stage_bytes;
          const uint32_t dst = b_base + sb * p.b_stage_bytes;
          for (int off = 0; off < p.b_stage_bytes; off += 32768) {
            const int n = min(32768, p.b_stage_bytes - off);
            ptx::bulk_g2s(dst + off, src + off, (uint32_t)n, b_full(sb));
          }
        }
      }
      // never leave with a bulk copy in flight: wait (bounded) for the last copies issued
      const uint32_t issued = kb;
      for (uint32_t q = (issued > (uint32_t)p.b_stages ? issued - p.b_stages : 0); q < issued; ++q) {
        const int sb = q % p.b_stages;
        const uint32_t parity = (q / p.b_stages) & 1;
        const long long t0 = clock64();
        while (!ptx::mbar_try_wait(b_full(sb), parity)) {
          if (clock64() - t0 > ptx::kWaitBudgetCycles) break;
        }
      }
    }
  } else {
    // ===================== gather producers =====================
    const int t = threadIdx.x - kGatherWarp0 * 32;
    const int j = t & 7;             // 16-byte chunk (8 channels) of the 128-byte row
    const int r0 = t >> 3;           // rows r0, r0+32, r0+64, r0+96
    uint32_t ka = 0;
    bool ok = true;
    for (int tile = blockIdx.x; ok && tile < p.n_tiles; tile += gridDim.x) {
      const int b = tile / p.tiles_per_clip, v0 = (tile % p.tiles_per_clip) * kBM;
      for (int s = 0; s < p.S; ++s, ++ka) {
        const int sa = ka % kAStages;
        const int h = s % p.nh, gt = s / p.nh, tap = gt % g.K, grp = gt / g.K;
        const int ch0 = grp * g.cpg + h * kBK + j * 8;
        if (!ptx::mbar_wait(a_empty(sa), ((ka / kAStages) & 1) ^ 1, abort_flag)) { ok = false; break; }
        const uint32_t stage = a_base + sa * kAStageBytes;
#pragma unroll
        for (int i = 0; i < kBM / 32; ++i) {
          const int r = r0 + 32 * i;
          const uint32_t dst = stage + (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((j ^ (r & 7)) << 4));
          produce_item(p, coords, b, v0 + r, grp, tap, ch0, dst);
        }
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(a_full(sa));
      }
    }
  }

  // ---- teardown ----
  ptx::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicExch(&g_sm100_status, 1);
  if (warp == 0) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

// ---- staging kernels -------------------------------------------------------------------------

// w [Cout][Cin][K] fp32 (weight groups == 1) -> w_sw [S][Cout rows x 128 B] bf16, slice
// s = (grp*K + tap)*nh + h holding channels grp*cpg + h*64 .. +63, each row's 16-byte
// chunks XOR-swizzled by (row & 7) -- the byte image of the shared-memory B tile.
__global__ void __launch_bounds__(64)
stage_weight_sw128_kernel(int Cout, int Cin, int K, int cpg, int nh, const float* __restrict__ w,
                          __nv_bfloat16* __restrict__ w_sw) {
  extern __shared__ float wrow[];   // [64 channels][K]
  const int co = blockIdx.x, cblk = blockIdx.y;      // cblk: 64-channel block of Cin
  const int c0 = cblk * 64;
  const float* src = w + ((long long)co * Cin + c0) * K;
  for (int i = threadIdx.x; i < 64 * K; i += 64) wrow[i] = __ldg(src + i);
  __syncthreads();
  const int grp = c0 / cpg, h = (c0 % cpg) / 64;
  // thread -> (tap group, chunk): 8 chunks per tap
  for (int item = threadIdx.x; item < K * 8; item += 64) {
    const int tap = item >> 3, jj = item & 7;
    uint4 out;
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = wrow[(jj * 8 + e) * K + tap];
    out.x = ptx::pack_bf16x2(v[0], v[1]); out.y = ptx::pack_bf16x2(v[2], v[3]);
    out.z = ptx::pack_bf16x2(v[4], v[5]); out.w = ptx::pack_bf16x2(v[6], v[7]);
    const long long s = ((long long)grp * K + tap) * nh + h;
    uint8_t* dst = reinterpret_cast<uint8_t*>(w_sw) + s * (long long)Cout * 128 + (long long)(co >> 3) * 1024 +
                   (co & 7) * 128 + ((jj ^ (co & 7)) << 4);
    *reinterpret_cast<uint4*>(dst) = out;
  }
}

struct Plan {
  int nh, S, tiles_per_clip, n_tiles, b_stages, b_stage_bytes, tmem_cols, smem_bytes;
  size_t x_cl_bytes, w_sw_bytes;
};

bool make_plan(const Geom& g, Plan* pl) {
  if (g.groups != 1) return false;
  if (g.cpg % kBK != 0) return false;
  if (g.Cout % 64 != 0 || g.Cout > kMaxN) return false;
  if ((long long)g.B * g.Vin * g.Cin > 0x7fffffffLL * 8) return false;
  pl->nh = g.cpg / kBK;
  pl->S = g.G * g.K * pl->nh;
  pl->tiles_per_clip = (g.V + kBM - 1) / kBM;
  pl->n_tiles = pl->tiles_per_clip * g.B;
  pl->b_stage_bytes = g.Cout * 128;
  int nb = (kSmemLimit - 1024 - 256 - kAStages * kAStageBytes) / pl->b_stage_bytes;
  if (nb > 4) nb = 4;
  if (nb < 2) return false;
  pl->b_stages = nb;
  int cols = 32;
  while (cols < g.Cout) cols <<= 1;
  pl->tmem_cols = cols;
  pl->smem_bytes = smem_layout(pl->b_stages, pl->b_stage_bytes).total + 1024;
  pl->x_cl_bytes = align_up((size_t)g.B * g.Vin * g.Cin * 2, 256);
  pl->w_sw_bytes = align_up((size_t)pl->S * pl->b_stage_bytes, 256);
  return true;
}

template <typename Coords>
int run_fwd(const Geom& g, const Coords& coords, const float* x, const float* mask, const float* w,
            const float* bias, float* y, void* ws, cudaStream_t st) {
  Plan pl;
  if (!make_plan(g, &pl)) return D2C_ERR_MODE;
  __nv_bfloat16* x_cl = reinterpret_cast<__nv_bfloat16*>(ws);
  __nv_bfloat16* w_sw = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<uint8_t*>(ws) + pl.x_cl_bytes);

  prof_mark(st, "fwd_stage_operands");
  {
    dim3 grid((unsigned)((g.Vin + 31) / 32), (unsigned)((g.Cin + 63) / 64), (unsigned)g.B);
    stage_input_cl_bf16_kernel<<<grid, 256, 0, st>>>(g.Cin, g.Vin, x, x_cl);
    D2C_LAUNCH_CHECK();
    dim3 wgrid((unsigned)g.Cout, (unsigned)(g.Cin / 64));
    stage_weight_sw128_kernel<<<wgrid, 64, 64 * g.K * sizeof(float), st>>>(g.Cout, g.Cin, g.K, g.cpg, pl.nh, w, w_sw);
    D2C_LAUNCH_CHECK();
  }

  FwdParams p;
  p.g = g; p.x_cl = x_cl; p.w_sw = w_sw; p.mask = mask; p.bias = bias; p.y = y;
  p.N = g.Cout; p.nh = pl.nh; p.S = pl.S; p.tiles_per_clip = pl.tiles_per_clip; p.n_tiles = pl.n_tiles;
  p.b_stages = pl.b_stages; p.b_stage_bytes = pl.b_stage_bytes; p.tmem_cols = pl.tmem_cols;

  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    D2C_CUDA_TRY(cudaGetDevice(&dev));
    D2C_CUDA_TRY(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
  }
  D2C_CUDA_TRY(cudaFuncSetAttribute(fwd_sm100_kernel<Coords>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    pl.smem_bytes));
  const int grid = pl.n_tiles < sm_count ? pl.n_tiles : sm_count;
  prof_mark(st, "fwd_sm100_fused");
  fwd_sm100_kernel<Coords><<<grid, kThreads, pl.smem_bytes, st>>>(p, coords);
  D2C_LAUNCH_CHECK();
  prof_mark(st, nullptr);
  return D2C_OK;
}

// =====================================================================================================
// Weight gradient as an implicit GEMM over voxels that consumes the SAME sampled tile as the forward:
//   dW[(slice, c), co] = sum_{b, v} sample[b, v, (slice, c)] * grad_out[b, co, v]
// (reference: re-im2col + cuBLAS gemmStridedBatched + sum over the batch, csrc/ops/dconv3d_gpu.cu:1037-1088).
//
// One CTA owns a PAIR of K slices (2 x 64 channels = the 128 rows of the accumulator) and a contiguous
// range of voxel tiles; its accumulator [128 x Cout] fp32 lives in tensor memory for the whole range.
//   A operand: the two sampled [128 voxels x 64 ch] tiles, read MN-major (M = channel is the contiguous
//              dimension, K = voxel): byte-identical to the forward's K-major A tile.
//   B operand: grad_out as bf16 [co rows x 64 voxels], K-major, staged per 64-voxel block.
// The partial results of different voxel ranges are combined with vector reductions into a [S*64, Cout]
// fp32 buffer that a last kernel permutes into the [Cout, Cin, kd, kh, kw] layout of grad_weight.
// =====================================================================================================

constexpr int kDwAStages = 2;
constexpr int kDwAStageBytes = 2 * kAStageBytes;     // two slices
constexpr int kDwBStages = 2;
constexpr int kDwChunkBytes = 256 * 128;             // one 256-row (co) x 64-voxel image

struct DwParams {
  FwdParams f;               // g, x_cl, mask used by the gather producers
  const uint8_t* gyk_img;    // [n_tiles][2 voxel blocks][NCH][32 KB]
  float* dws;                // [S*64][Cout] fp32, zero-initialised
  int n_pairs, nsplit, tiles_per_split, NCH, b_stage_bytes;
};

// grad_out [B][Cout][V] fp32 -> per (tile, 64-voxel block, 256-co chunk) images: 256 rows (co) x 128 B
// (64 voxels, bf16), chunks XOR-swizzled by (row & 7).  Voxels past the clip are zero.
__global__ void __launch_bounds__(256)
stage_gy_kmajor_kernel(int Cout, int V, int tiles_per_clip, int NCH, const float* __restrict__ gy,
                       uint8_t* __restrict__ img) {
  const int tile = blockIdx.x, coblk = blockIdx.y;        // coblk: 64 rows of co
  const int b = tile / tiles_per_clip, v0 = (tile % tiles_per_clip) * kBM;
  for (int e = threadIdx.x; e < 64 * 16; e += 256) {
    const int rl = e >> 4, q = e & 15;                    // row within block, 8-voxel chunk (0..15)
    const int co = coblk * 64 + rl;
    if (co >= Cout) continue;
    const int v = v0 + q * 8;
    float f[8];
    const float* src = gy + ((long long)b * Cout + co) * V;
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = (v + i < V) ? __ldg(src + v + i) : 0.f;
    uint4 o;
    o.x = ptx::pack_bf16x2(f[0], f[1]); o.y = ptx::pack_bf16x2(f[2], f[3]);
    o.z = ptx::pack_bf16x2(f[4], f[5]); o.w = ptx::pack_bf16x2(f[6], f[7]);
    const int kblk = q >> 3, j = q & 7, chunk = co >> 8, row = co & 255;
    uint8_t* dst = img + (((long long)tile * 2 + kblk) * NCH + chunk) * kDwChunkBytes + (row >> 3) * 1024 +
                   (row & 7) * 128 + ((j ^ (row & 7)) << 4);
    *reinterpret_cast<uint4*>(dst) = o;
  }
}

template <typename Coords>
__global__ void __launch_bounds__(kThreads, 1)
dw_sm100_kernel(const DwParams p, const Coords coords) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t a_base = base, b_base = base + kDwAStages * kDwAStageBytes;
  const int bar_off = kDwAStages * kDwAStageBytes + kDwBStages * p.b_stage_bytes;
  const uint32_t bar_base = base + bar_off;
  auto a_full = [&](int s) { return bar_base + 8u * s; };
  auto a_empty = [&](int s) { return bar_base + 8u * (2 + s); };
  auto b_full = [&](int s) { return bar_base + 8u * (4 + s); };
  auto b_empty = [&](int s) { return bar_base + 8u * (6 + s); };
  const uint32_t acc_full = bar_base + 8u * 8;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + bar_off + 8 * 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + bar_off + 8 * 9 + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const FwdParams& f = p.f;
  const Geom& g = f.g;
  const int pair = blockIdx.x % p.n_pairs, split = blockIdx.x / p.n_pairs;
  const int tile_beg = split * p.tiles_per_split;
  const int tile_end = min(f.n_tiles, tile_beg + p.tiles_per_split);
  const int n_my_tiles = tile_end - tile_beg;          // may be <= 0 for a trailing split

  if (threadIdx.x == 0) {
    for (int s = 0; s < kDwAStages; ++s) { ptx::mbar_init(a_full(s), kGatherWarps); ptx::mbar_init(a_empty(s), 1); }
    for (int s = 0; s < kDwBStages; ++s) { ptx::mbar_init(b_full(s), 1); ptx::mbar_init(b_empty(s), 1); }
    ptx::mbar_init(acc_full, 1);
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  if (warp == 0) {
    __syncwarp();
    ptx::tmem_alloc(ptx::smem_u32((const void*)tmem_slot), (uint32_t)f.tmem_cols);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (n_my_tiles > 0) {
    if (warp < kEpiWarps) {
      // ---- epilogue (once): accumulator rows (slice_local*64 + c) x columns co -> dws, vector reductions
      if (ptx::mbar_wait(acc_full, 0, abort_flag)) {
        ptx::tc_fence_after();
        const int m = warp * 32 + lane;
        const int s = 2 * pair + (m >> 6);
        float* row = p.dws + ((long long)s * 64 + (m & 63)) * f.N;
        for (int c0 = 0; c0 < f.N; c0 += 32) {
          uint32_t r[32];
          ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, r);
          ptx::tmem_ld_wait();
          if (s < f.S) {
#pragma unroll
            for (int i = 0; i < 8; ++i)
              asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(row + c0 + 4 * i),
                           "f"(__uint_as_float(r[4 * i])), "f"(__uint_as_float(r[4 * i + 1])),
                           "f"(__uint_as_float(r[4 * i + 2])), "f"(__uint_as_float(r[4 * i + 3]))
                           : "memory");
          }
        }
        ptx::tc_fence_before();
      }
    } else if (warp == kMmaWarp) {
      if (lane == 0) {
        uint32_t kb = 0;
        bool ok = true;
        for (int t = 0; ok && t < n_my_tiles; ++t) {
          const int sa = t % kDwAStages;
          if (!ptx::mbar_wait(a_full(sa), (t / kDwAStages) & 1, abort_flag)) break;
          for (int kblk = 0; kblk < 2; ++kblk, ++kb) {
            const int sb = kb % kDwBStages;
            if (!ptx::mbar_wait(b_full(sb), (kb / kDwBStages) & 1, abort_flag)) { ok = false; break; }
            ptx::tc_fence_after();
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
              // A: 16 voxels starting at voxel kblk*64 + k4*16 -> two 8-row groups of 1024 bytes
              const uint64_t adesc = ptx::umma_desc_mnmajor_sw128(
                  a_base + sa * kDwAStageBytes + (kblk * 8 + k4 * 2) * 1024, kAStageBytes, 1024);
              for (int n0 = 0; n0 < f.N; n0 += 256) {
                const int nc = min(256, f.N - n0);
                const uint64_t bdesc =
                    ptx::umma_desc_kmajor_sw128(b_base + sb * p.b_stage_bytes + (n0 >> 8) * kDwChunkBytes) +
                    (uint64_t)(2 * k4);
                ptx::umma_bf16(tmem_base + (uint32_t)n0, adesc, bdesc,
                               ptx::umma_idesc_bf16_f32(kBM, nc) | (1u << 15) /* A is MN-major */,
                               (t > 0 || kblk > 0 || k4 > 0) ? 1u : 0u);
              }
            }
            ptx::umma_commit(b_empty(sb));
          }
          if (ok) ptx::umma_commit(a_empty(sa));
        }
        if (ok) ptx::umma_commit(acc_full);
      }
    } else if (warp == kLoadWarp) {
      if (lane == 0) {
        uint32_t kb = 0;
        bool ok = true;
        for (int t = 0; ok && t < n_my_tiles; ++t) {
          for (int kblk = 0; kblk < 2; ++kblk, ++kb) {
            const int sb = kb % kDwBStages;
            if (!ptx::mbar_wait(b_empty(sb), ((kb / kDwBStages) & 1) ^ 1, abort_flag)) { ok = false; break; }
            ptx::mbar_arrive_expect_tx(b_full(sb), (uint32_t)p.b_stage_bytes);
            const uint8_t* src = p.gyk_img + ((long long)(tile_beg + t) * 2 + kblk) * p.b_stage_bytes;
            for (int off = 0; off < p.b_stage_bytes; off += 32768)
              ptx::bulk_g2s(b_base + sb * p.b_stage_bytes + off, src + off, 32768u, b_full(sb));
          }
        }
        const uint32_t issued = kb;
        for (uint32_t q = (issued > (uint32_t)kDwBStages ? issued - kDwBStages : 0); q < issued; ++q) {
          const long long t0 = clock64();
          while (!ptx::mbar_try_wait(b_full(q % kDwBStages), (q / kDwBStages) & 1))
            if (clock64() - t0 > ptx::kWaitBudgetCycles) break;
        }
      }
    } else {
      // ---- gather producers: the forward's producer, two slices per stage
      const int tt = threadIdx.x - kGatherWarp0 * 32;
      const int j = tt & 7, r0 = tt >> 3;
      bool ok = true;
      for (int t = 0; ok && t < n_my_tiles; ++t) {
        const int tile = tile_beg + t;
        const int b = tile / f.tiles_per_clip, v0 = (tile % f.tiles_per_clip) * kBM;
        const int sa = t % kDwAStages;
        if (!ptx::mbar_wait(a_empty(sa), ((t / kDwAStages) & 1) ^ 1, abort_flag)) break;
        for (int sl = 0; sl < 2; ++sl) {
          const int s = min(2 * pair + sl, f.S - 1);      // an odd last slice is produced twice, second copy unused
          const int h = s % f.nh, gt = s / f.nh, tap = gt % g.K, grp = gt / g.K;
          const int ch0 = grp * g.cpg + h * kBK + j * 8;
          const uint32_t stage = a_base + sa * kDwAStageBytes + sl * kAStageBytes;
#pragma unroll
          for (int i = 0; i < kBM / 32; ++i) {
            const int r = r0 + 32 * i;
            const uint32_t dst = stage + (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((j ^ (r & 7)) << 4));
            produce_item(f, coords, b, v0 + r, grp, tap, ch0, dst);
          }
        }
        ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(a_full(sa));
      }
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) atomicExch(&g_sm100_status, 1);
  if (warp == 0) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, (uint32_t)f.tmem_cols);
  }
}

// dws [(slice, c)][co] -> grad_w [co][cin][tap]   (cin = grp*cpg + h*64 + c)
__global__ void __launch_bounds__(256)
unstage_dw_kernel(int Cout, int Cin, int K, int cpg, int nh, int S, const float* __restrict__ dws,
                  float* __restrict__ grad_w) {
  __shared__ float tile[32][33];
  const int r0 = blockIdx.x * 32, co0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int rr = ty; rr < 32; rr += 8) {
    const int r = r0 + rr;
    tile[rr][tx] = (r < S * 64 && co0 + tx < Cout) ? __ldg(dws + (long long)r * Cout + co0 + tx) : 0.f;
  }
  __syncthreads();
  for (int cc = ty; cc < 32; cc += 8) {
    const int r = r0 + tx, co = co0 + cc;
    if (r < S * 64 && co < Cout) {
      const int c = r & 63, s = r >> 6;
      const int h = s % nh, gt = s / nh, tap = gt % K, grp = gt / K;
      grad_w[((long long)co * Cin + grp * cpg + h * 64 + c) * K + tap] = tile[tx][cc];
    }
  }
}

struct DwPlan {
  int n_pairs, nsplit, tiles_per_split, NCH, b_stage_bytes, smem_bytes;
  size_t gyk_bytes, dws_bytes;
};

bool make_dw_plan(const Geom& g, const Plan& pl, int sm_count, DwPlan* dp) {
  dp->n_pairs = (pl.S + 1) / 2;
  dp->NCH = (g.Cout + 255) / 256;
  dp->b_stage_bytes = dp->NCH * kDwChunkBytes;
  dp->smem_bytes = kDwAStages * kDwAStageBytes + kDwBStages * dp->b_stage_bytes + 256 + 1024;
  if (dp->smem_bytes > kSmemLimit) return false;
  // enough (pair, voxel-range) work items for ~3 waves, but at least 8 tiles per item
  int nsplit = (3 * sm_count + dp->n_pairs - 1) / dp->n_pairs;
  const int max_split = (pl.n_tiles + 7) / 8;
  if (nsplit > max_split) nsplit = max_split;
  if (nsplit < 1) nsplit = 1;
  dp->tiles_per_split = (pl.n_tiles + nsplit - 1) / nsplit;
  dp->nsplit = (pl.n_tiles + dp->tiles_per_split - 1) / dp->tiles_per_split;
  dp->gyk_bytes = align_up((size_t)pl.n_tiles * 2 * dp->b_stage_bytes, 256);
  dp->dws_bytes = align_up((size_t)pl.S * 64 * g.Cout * 4, 256);
  return true;
}

template <typename Coords>
int run_dw(const Geom& g, const Coords& coords, const float* gy, const __nv_bfloat16* x_cl, const float* mask,
           float* grad_w, void* ws, cudaStream_t st) {
  Plan pl;
  if (!make_plan(g, &pl)) return D2C_ERR_MODE;
  static int sm_count = 0;
  if (sm_count == 0) {
    int dev = 0;
    D2C_CUDA_TRY(cudaGetDevice(&dev));
    D2C_CUDA_TRY(cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, dev));
  }
  DwPlan dp;
  if (!make_dw_plan(g, pl, sm_count, &dp)) return D2C_ERR_MODE;
  uint8_t* gyk = reinterpret_cast<uint8_t*>(ws);
  float* dws = reinterpret_cast<float*>(gyk + dp.gyk_bytes);

  prof_mark(st, "bwd_dw_stage");
  D2C_CUDA_TRY(cudaMemsetAsync(dws, 0, (size_t)pl.S * 64 * g.Cout * 4, st));
  stage_gy_kmajor_kernel<<<dim3((unsigned)pl.n_tiles, (unsigned)((g.Cout + 63) / 64)), 256, 0, st>>>(
      g.Cout, g.V, pl.tiles_per_clip, dp.NCH, gy, gyk);
  D2C_LAUNCH_CHECK();

  DwParams p;
  p.f.g = g; p.f.x_cl = x_cl; p.f.w_sw = nullptr; p.f.mask = mask; p.f.bias = nullptr; p.f.y = nullptr;
  p.f.N = g.Cout; p.f.nh = pl.nh; p.f.S = pl.S; p.f.tiles_per_clip = pl.tiles_per_clip; p.f.n_tiles = pl.n_tiles;
  p.f.b_stages = 0; p.f.b_stage_bytes = 0; p.f.tmem_cols = pl.tmem_cols;
  p.gyk_img = gyk; p.dws = dws;
  p.n_pairs = dp.n_pairs; p.nsplit = dp.nsplit; p.tiles_per_split = dp.tiles_per_split; p.NCH = dp.NCH;
  p.b_stage_bytes = dp.b_stage_bytes;
  D2C_CUDA_TRY(cudaFuncSetAttribute(dw_sm100_kernel<Coords>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    dp.smem_bytes));
  prof_mark(st, "bwd_dw_sm100");
  dw_sm100_kernel<Coords><<<dp.n_pairs * dp.nsplit, kThreads, dp.smem_bytes, st>>>(p, coords);
  D2C_LAUNCH_CHECK();
  prof_mark(st, "bwd_dw_unstage");
  unstage_dw_kernel<<<dim3((unsigned)((pl.S * 64 + 31) / 32), (unsigned)((g.Cout + 31) / 32)), 256, 0, st>>>(
      g.Cout, g.Cin, g.K, g.cpg, pl.nh, pl.S, dws, grad_w);
  D2C_LAUNCH_CHECK();
  return D2C_OK;
}

}  // namespace

size_t sm100_dw_workspace(const Geom& g) {
  Plan pl;
  DwPlan dp;
  if (!make_plan(g, &pl) || !make_dw_plan(g, pl, 148, &dp)) return 0;
  return dp.gyk_bytes + dp.dws_bytes;
}

int sm100_dw_offsets(const Geom& g, const float* offset, const float* gy, const void* x_cl, const float* mask,
                     float* grad_w, void* ws, cudaStream_t st) {
  OffsetCoords<float> oc{offset};
  return run_dw(g, oc, gy, reinterpret_cast<const __nv_bfloat16*>(x_cl), mask, grad_w, ws, st);
}

int sm100_dw_field(const Geom& g, const FieldCoords<float>& fc, const float* gy, const void* x_cl,
                   const float* mask, float* grad_w, void* ws, cudaStream_t st) {
  return run_dw(g, fc, gy, reinterpret_cast<const __nv_bfloat16*>(x_cl), mask, grad_w, ws, st);
}

bool sm100_fwd_supported(const Geom& g, int dtype, int math_mode) {
  if (dtype != D2C_F32) return false;
  if (math_mode != D2C_MATH_BF16) return false;
  if (g.K * 64 * (int)sizeof(float) > 48 * 1024) return false;   // weight staging kernel's smem
  Plan pl;
  return make_plan(g, &pl);
}

size_t sm100_fwd_workspace(const Geom& g, int dtype, int math_mode) {
  if (!sm100_fwd_supported(g, dtype, math_mode)) return 0;
  Plan pl;
  make_plan(g, &pl);
  return pl.x_cl_bytes + pl.w_sw_bytes;
}

int sm100_fwd_offsets(const Geom& g, int /*math_mode*/, const float* x, const float* offset, const float* mask,
                      const float* w, const float* bias, float* y, void* ws, cudaStream_t st) {
  OffsetCoords<float> oc{offset};
  return run_fwd(g, oc, x, mask, w, bias, y, ws, st);
}

int sm100_fwd_field(const Geom& g, int /*math_mode*/, const FieldCoords<float>& fc, const float* x,
                    const float* mask, const float* w, const float* bias, float* y, void* ws, cudaStream_t st) {
  return run_fwd(g, fc, x, mask, w, bias, y, ws, st);
}

int sm100_device_status() {
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_sm100_status, sizeof(int)) != cudaSuccess) return -1;
  return v;
}

}  // namespace d2c
