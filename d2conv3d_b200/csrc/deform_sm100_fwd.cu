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
// with the input staged channels-last each corner of a slice is ONE contiguous 128-byte
// (fp16 staging) or 256-byte (fp32 staging) line.
//
// Work decomposition: the (tile, slice) units are cut into one contiguous range per CTA
// (stream-K), so 203 tiles do not run as two ragged waves on 148 SMs.  A CTA whose range
// covers a whole tile stores it; partial tiles are combined with fp32 reductions into the
// zero-initialised output.
//
// Per CTA, 23 warps:
//   warps 0-3   epilogue: tcgen05.ld the 128 x N accumulator, add bias, store / reduce NCDHW
//   warp  4     one thread issues tcgen05.mma and the commits that free the stages
//   warp  5     one thread streams pre-swizzled weight slices with cp.async.bulk
//   warps 6-21  gather producers: unit header + gather record from the shared-memory record ring, 8
//               unconditional corner loads (16 B) for each of the thread's two rows in flight at once, blend
//               with pre-modulated weights, bf16 pack, swizzled st.shared of the A tile
//   warp  22    one thread bulk-copies each unit's gather records into the record ring and writes the unit
//               header (staging offset of the slice, valid rows), so the producers do no index arithmetic
// Stage hand-off is by mbarriers; every wait is bounded (sm100_ptx.cuh).
//
// Two math modes share the kernel (template parameter): single-pass bf16 (64-channel units, fp16 staging) and
// the fp32-parity split "bf16x3" (32-channel units, fp32 staging, rows [hi | lo], three K-sub-block products).
#include "deform_sm100.h"
#include "sm100_gather.cuh"
#include "sm100_ptx.cuh"
#include "sm100_stage.cuh"

#include <cstdio>
#include <cstdlib>

namespace d2c {

namespace {

constexpr int kBM = 128;            // voxels per tile (UMMA M)
constexpr int kBK = 64;             // channels per K slice (128 bytes of bf16: one swizzle row)
constexpr int kAStages = 4;
constexpr int kAStageBytes = kBM * kBK * 2;   // 16 KB
constexpr int kMaxN = 512;
constexpr int kThreads = (6 + 16 + 1) * 32;   // 4 epilogue + MMA + weight loader + 16 gather + record loader warps
constexpr int kEpiWarps = 4, kMmaWarp = 4, kLoadWarp = 5, kGatherWarp0 = 6, kGatherWarps = 16, kRecWarp = 22;
constexpr int kRStages = 4;                       // gather-record ring: one stage = the records of a unit's 128 rows
constexpr int kRecBytes = kBM * 48;               // 6 KB of records ...
constexpr int kRStageBytes = kRecBytes + 16;      // ... + unit header {int64 x_cl element offset of the slice, int rows}
constexpr int kRowStride = kGatherWarps * 4;          // 8 threads per row -> rows handled per pass
constexpr int kRowsPerThread = kBM / kRowStride;
constexpr int kSmemLimit = 227 * 1024;
constexpr int kMinUnitsPerCta = 16;

struct FwdParams {
  Geom g;
  const void* x_cl;            // [B][Vin][Cin] channels-last staging of x: fp16 (bf16 mode) or fp32 (bf16x3 mode)
  const uint8_t* w_sw;         // [S][N rows x 128 B], rows swizzled exactly as the smem B tile
  const uint4* recs;           // [B][G][K][V] gather records (3 x uint4 each, sm100_gather.cuh)
  const float* bias;           // [Cout] or nullptr
  float* y;                    // [B, Cout, V]
  ClStrides cs;
  int N;                       // Cout
  int nh;                      // K slices per (group, tap) = cpg / 64
  int S;                       // slices per tile = G * K * nh
  int tiles_per_clip, n_tiles;
  long long n_units;           // n_tiles * S
  int b_stages, b_stage_bytes;
  int tmem_cols;
};

__device__ __forceinline__ void cta_unit_range(long long n_units, long long& beg, long long& end) {
  beg = n_units * blockIdx.x / gridDim.x;
  end = n_units * (blockIdx.x + 1) / gridDim.x;
}

// kX3 = 0: math mode bf16 (a unit is 64 channels of one tap, one bf16 operand pair).
// kX3 = 1: math mode bf16x3, the fp32-parity mode: a unit is 32 channels; the A row holds [hi(32) | lo(32)] of
//          the fp32 blend, the weight row [hi(32) | lo(32)] of the fp32 weight, and the issuer forms
//          a_hi*b_hi + a_lo*b_hi + a_hi*b_lo from the 16-channel K sub-blocks of the same two tiles.
// kDual = 1 (single-pass mode only): 32 channels per offset group, a 64-channel unit spans two groups.
template <int kX3, int kDual>
__global__ void __launch_bounds__(kThreads, 1)
fwd_sm100_kernel(const FwdParams p) {
  constexpr int kUnitCh = kX3 ? 32 : 64;
  constexpr int kRStage = (1 + kDual) * kRecBytes + 16;      // record set(s) + unit header
  constexpr int hdr_off = (1 + kDual) * kRecBytes;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const int rec_off = kAStages * kAStageBytes + p.b_stages * p.b_stage_bytes;
  const int bar_off = rec_off + kRStages * kRStage;
  const uint32_t a_base = base, b_base = base + kAStages * kAStageBytes, rec_base = base + rec_off,
                 bar_base = base + bar_off;
  auto a_full = [&](int s) { return bar_base + 8u * s; };
  auto a_empty = [&](int s) { return bar_base + 8u * (kAStages + s); };
  auto b_full = [&](int s) { return bar_base + 8u * (2 * kAStages + s); };
  auto b_empty = [&](int s) { return bar_base + 8u * (2 * kAStages + 4 + s); };
  const uint32_t acc_full = bar_base + 8u * (2 * kAStages + 8);
  const uint32_t acc_empty = bar_base + 8u * (2 * kAStages + 9);
  auto r_full = [&](int s) { return bar_base + 8u * (2 * kAStages + 11 + s); };
  auto r_empty = [&](int s) { return bar_base + 8u * (2 * kAStages + 11 + kRStages + s); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + bar_off + 8 * (2 * kAStages + 10));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + bar_off + 8 * (2 * kAStages + 10) + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const Geom& g = p.g;
  long long u_beg, u_end;
  cta_unit_range(p.n_units, u_beg, u_end);

  if (threadIdx.x == 0) {
    for (int s = 0; s < kAStages; ++s) { ptx::mbar_init(a_full(s), kGatherWarps); ptx::mbar_init(a_empty(s), 1); }
    for (int s = 0; s < p.b_stages; ++s) { ptx::mbar_init(b_full(s), 1); ptx::mbar_init(b_empty(s), 1); }
    for (int s = 0; s < kRStages; ++s) { ptx::mbar_init(r_full(s), 1); ptx::mbar_init(r_empty(s), kGatherWarps); }
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
    // ===================== epilogue: one pass per tile segment =====================
    int seg = 0;
    for (long long u = u_beg; u < u_end; ++seg) {
      const int tile = (int)(u / p.S), s_beg = (int)(u % p.S);
      const int s_end = (int)min((long long)p.S, s_beg + (u_end - u));
      u += s_end - s_beg;
      const bool whole = (s_beg == 0 && s_end == p.S);
      const int b = tile / p.tiles_per_clip, v0 = (tile % p.tiles_per_clip) * kBM;
      if (!ptx::mbar_wait(acc_full, seg & 1, abort_flag, 2000)) break;
      ptx::tc_fence_after();
      const int v = v0 + warp * 32 + lane;
      float* yb = p.y + (long long)b * g.Cout * g.V + v;
      for (int c0 = 0; c0 < p.N; c0 += 32) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, r);
        ptx::tmem_ld_wait();
        if (v < g.V) {
          if (whole) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float bb = p.bias ? __ldg(p.bias + c0 + j) : 0.f;
              yb[(long long)(c0 + j) * g.V] = __uint_as_float(r[j]) + bb;
            }
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const float bb = (p.bias && s_beg == 0) ? __ldg(p.bias + c0 + j) : 0.f;
              atomicAdd(yb + (long long)(c0 + j) * g.V, __uint_as_float(r[j]) + bb);
            }
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
      int seg = 0;
      uint32_t k = 0;           // units consumed so far (A and B rings advance together)
      bool ok = true;
      for (long long u = u_beg; ok && u < u_end; ++seg) {
        const int s_beg = (int)(u % p.S);
        const int s_end = (int)min((long long)p.S, s_beg + (u_end - u));
        u += s_end - s_beg;
        if (!ptx::mbar_wait(acc_empty, (seg & 1) ^ 1, abort_flag)) break;
        ptx::tc_fence_after();
        for (int s = s_beg; s < s_end; ++s, ++k) {
          const int sa = k % kAStages, sb = k % p.b_stages;
          if (!ptx::mbar_wait(a_full(sa), (k / kAStages) & 1, abort_flag)) { ok = false; break; }
          if (!ptx::mbar_wait(b_full(sb), (k / p.b_stages) & 1, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint64_t adesc = ptx::umma_desc_kmajor_sw128(a_base + sa * kAStageBytes);
          // K sub-blocks (16 channels = 32 bytes) of the A and B rows that meet in each MMA
          constexpr int kSteps = kX3 ? 6 : 4;
          constexpr int ka_[6] = {0, 1, kX3 ? 2 : 2, kX3 ? 3 : 3, 0, 1};   // bf16: (k,k); x3: hi*hi, lo*hi, hi*lo
          constexpr int kb_[6] = {0, 1, kX3 ? 0 : 2, kX3 ? 1 : 3, 2, 3};
#pragma unroll
          for (int kk = 0; kk < kSteps; ++kk) {
            for (int n0 = 0; n0 < p.N; n0 += 256) {
              const int nc = min(256, p.N - n0);
              const uint64_t bdesc = ptx::umma_desc_kmajor_sw128(b_base + sb * p.b_stage_bytes + n0 * 128);
              ptx::umma_bf16(tmem_base + (uint32_t)n0, adesc + (uint64_t)(2 * ka_[kk]),
                             bdesc + (uint64_t)(2 * kb_[kk]), ptx::umma_idesc_bf16_f32(kBM, nc),
                             (s > s_beg || kk > 0) ? 1u : 0u);
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
      uint32_t k = 0;
      for (long long u = u_beg; u < u_end; ++u, ++k) {
        const int s = (int)(u % p.S), sb = k % p.b_stages;
        if (!ptx::mbar_wait(b_empty(sb), ((k / p.b_stages) & 1) ^ 1, abort_flag, 200)) break;
        ptx::mbar_arrive_expect_tx(b_full(sb), (uint32_t)p.b_stage_bytes);
        const uint8_t* src = p.w_sw + (long long)s * p.b_stage_bytes;
        const uint32_t dst = b_base + sb * p.b_stage_bytes;
        for (int off = 0; off < p.b_stage_bytes; off += 32768)
          ptx::bulk_g2s(dst + off, src + off, (uint32_t)min(32768, p.b_stage_bytes - off), b_full(sb));
      }
      // never leave with a bulk copy in flight: wait (bounded) for the last copies issued
      const uint32_t issued = k;
      for (uint32_t q = (issued > (uint32_t)p.b_stages ? issued - p.b_stages : 0); q < issued; ++q) {
        const long long t0 = clock64();
        while (!ptx::mbar_try_wait(b_full(q % p.b_stages), (q / p.b_stages) & 1))
          if (clock64() - t0 > ptx::kWaitBudgetCycles) break;
      }
    }
  } else if (warp == kRecWarp) {
    // ===================== gather-record loader =====================
    // The records of a unit's rows are one contiguous run of the [B][G][K][V] stream: one bulk copy per unit,
    // kRStages units ahead of the gather warps, so the producers read them from shared memory.
    if (lane == 0) {
      uint32_t k = 0;
      for (long long u = u_beg; u < u_end; ++u, ++k) {
        const int tile = (int)(u / p.S), s = (int)(u % p.S);
        const int b = tile / p.tiles_per_clip, v0 = (tile % p.tiles_per_clip) * kBM;
        const int gt = s / p.nh, tap = gt % g.K, grp = gt / g.K;      // dual: grp is the index of a group PAIR
        const int sr = k % kRStages;
        if (!ptx::mbar_wait(r_empty(sr), ((k / kRStages) & 1) ^ 1, abort_flag, 200)) break;
        const int rows = min(kBM, g.V - v0), h = s % p.nh;
        // unit header for the gather warps (no index arithmetic there); ordered before their reads by the
        // release of the arrive below and the acquire of their wait
        uint8_t* hdr = base_ptr + rec_off + sr * kRStage + hdr_off;
        *reinterpret_cast<long long*>(hdr) =
            (long long)b * g.Vin * g.Cin + grp * (kDual ? 2 * g.cpg : g.cpg) + h * kUnitCh;
        *reinterpret_cast<int*>(hdr + 8) = rows;
        const uint32_t bytes = (uint32_t)rows * 48u;
        ptx::mbar_arrive_expect_tx(r_full(sr), bytes * (uint32_t)(1 + kDual));
#pragma unroll
        for (int set = 0; set <= kDual; ++set) {
          const int og = kDual ? 2 * grp + set : grp;      // offset group whose records fill this set
          ptx::bulk_g2s(rec_base + sr * kRStage + set * kRecBytes,
                        p.recs + 3 * ((((long long)b * g.G + og) * g.K + tap) * g.V + v0), bytes, r_full(sr));
        }
      }
      const uint32_t issued = k;
      for (uint32_t q = (issued > (uint32_t)kRStages ? issued - kRStages : 0); q < issued; ++q) {
        const long long t0 = clock64();
        while (!ptx::mbar_try_wait(r_full(q % kRStages), (q / kRStages) & 1))
          if (clock64() - t0 > ptx::kWaitBudgetCycles) break;
      }
    }
  } else {
    // ===================== gather producers =====================
    const int t = threadIdx.x - kGatherWarp0 * 32;
    const int j = t & 7;             // 16-byte chunk (8 channels) of the 128-byte row
    const int r0 = t >> 3;           // rows r0, r0+kRowStride, ...
    uint32_t row_dst[kRowsPerThread];
#pragma unroll
    for (int i = 0; i < kRowsPerThread; ++i) {
      const int r = r0 + kRowStride * i;
      row_dst[i] = (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((j ^ (r & 7)) << 4));
    }
    uint32_t k = 0;
    const uint32_t n_my_units = (uint32_t)(u_end - u_beg);
    for (; k < n_my_units; ++k) {
      const int sr = k % kRStages, sa = k % kAStages;
      if (!ptx::mbar_wait(r_full(sr), (k / kRStages) & 1, abort_flag)) break;
      const uint8_t* rec_base_ptr = base_ptr + rec_off + sr * kRStage;
      const long long xoff = *reinterpret_cast<const long long*>(rec_base_ptr + hdr_off);
      const int rows = *reinterpret_cast<const int*>(rec_base_ptr + hdr_off + 8);
      // dual: 16-byte chunks 4-7 of a row (channels 32-63 of the unit) belong to the second offset group
      const uint8_t* rec_stage = rec_base_ptr + ((kDual && j >= 4) ? kRecBytes : 0);
      // every corner of every row this thread owns goes in flight before the first blend
      uint4 c[kRowsPerThread][8];
#pragma unroll
      for (int i = 0; i < kRowsPerThread; ++i) {
        const int r = r0 + kRowStride * i;
        uint2 head = make_uint2(0u, 0u);
        if (r < rows) head = *reinterpret_cast<const uint2*>(rec_stage + r * 48);
        if constexpr (kX3)
          load_corners_f32(reinterpret_cast<const float*>(p.x_cl) + xoff + j * 4, p.cs, head.x, head.y, c[i]);
        else
          load_corners(reinterpret_cast<const __half*>(p.x_cl) + xoff + j * 8, p.cs, head.x, head.y, c[i]);
      }
      if (!ptx::mbar_wait(a_empty(sa), ((k / kAStages) & 1) ^ 1, abort_flag)) break;
      const uint32_t stage = a_base + sa * kAStageBytes;
#pragma unroll
      for (int i = 0; i < kRowsPerThread; ++i) {
        const int r = r0 + kRowStride * i;
        if constexpr (kX3) {
          float w[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};   // rows past the clip end: stage bytes are stale
          if (r < rows) {
            const uint2 w01 = *reinterpret_cast<const uint2*>(rec_stage + r * 48 + 8);
            const uint4 w25 = *reinterpret_cast<const uint4*>(rec_stage + r * 48 + 16);
            const uint2 w67 = *reinterpret_cast<const uint2*>(rec_stage + r * 48 + 32);
            w[0] = __uint_as_float(w01.x); w[1] = __uint_as_float(w01.y);
            w[2] = __uint_as_float(w25.x); w[3] = __uint_as_float(w25.y);
            w[4] = __uint_as_float(w25.z); w[5] = __uint_as_float(w25.w);
            w[6] = __uint_as_float(w67.x); w[7] = __uint_as_float(w67.y);
          }
          // item j = channels 4j..4j+3: hi in 16-byte chunk j/2 (half j&1), lo in chunk 4 + j/2
          const uint32_t row_base = stage + (uint32_t)((r >> 3) * 1024 + (r & 7) * 128) + (uint32_t)((j & 1) * 8);
          blend_split_store(c[i], w, row_base + ((((j >> 1)) ^ (r & 7)) << 4),
                            row_base + (((4 + (j >> 1)) ^ (r & 7)) << 4));
        } else {
          uint4 w03 = make_uint4(0u, 0u, 0u, 0u), w47 = w03;   // rows past the clip end: stage bytes are stale
          if (r < rows) {
            w03 = *reinterpret_cast<const uint4*>(rec_stage + r * 48 + 16);
            w47 = *reinterpret_cast<const uint4*>(rec_stage + r * 48 + 32);
          }
          blend_store(c[i], w03, w47, stage + row_dst[i]);
        }
      }
      ptx::fence_proxy_async_smem();
      __syncwarp();
      if (lane == 0) {
        ptx::mbar_arrive(a_full(sa));
        ptx::mbar_arrive(r_empty(sr));
      }
    }
  }

  // ---- teardown ----
  ptx::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) ptx::report_device_timeout();
  if (warp == 0) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

#include "deform_sm100_fwd_v2.cuh"
#include "deform_sm100_fwd_pair.cuh"

// ---- staging kernels -------------------------------------------------------------------------

// w [Cout][Cin][K] fp32 (weight groups == 1) -> w_sw [S][Cout rows x 128 B] bf16, slice
// s = (grp*K + tap)*nh + h holding channels grp*cpg + h*64 .. +63, each row's 16-byte
// chunks XOR-swizzled by (row & 7) -- the byte image of the shared-memory B tile.
__global__ void __launch_bounds__(64)
stage_weight_sw128_kernel(int Cout, int Cin, int K, int cpg, int nh, const float* __restrict__ w,
                          uint8_t* __restrict__ w_sw) {
  extern __shared__ float wrow[];   // [64 channels][K]
  const int co = blockIdx.x, cblk = blockIdx.y;      // cblk: 64-channel block of Cin
  const int c0 = cblk * 64;
  const float* src = w + ((long long)co * Cin + c0) * K;
  for (int i = threadIdx.x; i < 64 * K; i += 64) wrow[i] = __ldg(src + i);
  __syncthreads();
  const int grp = c0 / cpg, h = (c0 % cpg) / 64;
  for (int item = threadIdx.x; item < K * 8; item += 64) {
    const int tap = item >> 3, jj = item & 7;
    uint4 out;
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = wrow[(jj * 8 + e) * K + tap];
    out.x = ptx::pack_bf16x2(v[0], v[1]); out.y = ptx::pack_bf16x2(v[2], v[3]);
    out.z = ptx::pack_bf16x2(v[4], v[5]); out.w = ptx::pack_bf16x2(v[6], v[7]);
    const long long s = ((long long)grp * K + tap) * nh + h;
    uint8_t* dst = w_sw + s * (long long)Cout * 128 + (long long)(co >> 3) * 1024 + (co & 7) * 128 +
                   ((jj ^ (co & 7)) << 4);
    *reinterpret_cast<uint4*>(dst) = out;
  }
}

// bf16x3 mode: slice s = (grp*K + tap)*nh + h with nh = cpg/32 holds 32 channels; each row is
// [hi(32 ch) | lo(32 ch)] where hi = bf16(w), lo = bf16(w - hi); same swizzle.
__global__ void __launch_bounds__(64)
stage_weight_sw128_x3_kernel(int Cout, int Cin, int K, int cpg, int nh, const float* __restrict__ w,
                             uint8_t* __restrict__ w_sw) {
  extern __shared__ float wrow[];   // [32 channels][K]
  const int co = blockIdx.x, cblk = blockIdx.y;      // cblk: 32-channel block of Cin
  const int c0 = cblk * 32;
  const float* src = w + ((long long)co * Cin + c0) * K;
  for (int i = threadIdx.x; i < 32 * K; i += 64) wrow[i] = __ldg(src + i);
  __syncthreads();
  const int grp = c0 / cpg, h = (c0 % cpg) / 32;
  for (int item = threadIdx.x; item < K * 8; item += 64) {
    const int tap = item >> 3, jj = item & 7;        // jj < 4: hi of channels 8jj.., jj >= 4: lo of channels 8(jj-4)..
    const int cb = (jj & 3) * 8;
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float f = wrow[(cb + e) * K + tap];
      const float hi = ptx::bf16_lo(ptx::pack_bf16x2(f, 0.f));
      v[e] = (jj < 4) ? f : f - hi;
    }
    uint4 out;
    out.x = ptx::pack_bf16x2(v[0], v[1]); out.y = ptx::pack_bf16x2(v[2], v[3]);
    out.z = ptx::pack_bf16x2(v[4], v[5]); out.w = ptx::pack_bf16x2(v[6], v[7]);
    const long long s = ((long long)grp * K + tap) * nh + h;
    uint8_t* dst = w_sw + s * (long long)Cout * 128 + (long long)(co >> 3) * 1024 + (co & 7) * 128 +
                   ((jj ^ (co & 7)) << 4);
    *reinterpret_cast<uint4*>(dst) = out;
  }
}

struct Plan {
  int nh, S, tiles_per_clip, n_tiles, b_stages, b_stage_bytes, tmem_cols, smem_bytes, dual, r_stage_bytes;
  size_t x_cl_bytes, w_sw_bytes, rec_bytes;
};

bool make_plan(const Geom& g, bool x3, Plan* pl) {
  if (g.groups != 1) return false;
  // a unit must lie inside one offset group -- or, single-pass mode with 32 channels per group, span exactly two
  const bool dual = !x3 && g.cpg == 32 && g.G % 2 == 0;
  if (!dual && g.cpg % (x3 ? 32 : kBK) != 0) return false;
  pl->dual = dual ? 1 : 0;
  pl->r_stage_bytes = (1 + pl->dual) * kRecBytes + 16;
  if (g.Cout % 64 != 0 || g.Cout > kMaxN) return false;
  if (g.Vin * g.Cin > 0x7fffffffLL) return false;                 // 32-bit element offsets within a clip
  if (g.K * 64 * (int)sizeof(float) > 48 * 1024) return false;    // weight staging kernel's smem
  pl->nh = dual ? 1 : g.cpg / (x3 ? 32 : kBK);
  pl->S = (dual ? g.G / 2 : g.G) * g.K * pl->nh;
  pl->tiles_per_clip = (g.V + kBM - 1) / kBM;
  pl->n_tiles = pl->tiles_per_clip * g.B;
  pl->b_stage_bytes = g.Cout * 128;
  int nb = (kSmemLimit - 1024 - 256 - kAStages * kAStageBytes - kRStages * pl->r_stage_bytes) / pl->b_stage_bytes;
  if (nb > 4) nb = 4;
  if (nb < 2) return false;
  pl->b_stages = nb;
  int cols = 32;
  while (cols < g.Cout) cols <<= 1;
  pl->tmem_cols = cols;
  pl->smem_bytes = kAStages * kAStageBytes + pl->b_stages * pl->b_stage_bytes + kRStages * pl->r_stage_bytes + 256 + 1024;
  pl->x_cl_bytes = align_up((size_t)g.B * g.Vin * g.Cin * (x3 ? 4 : 2), 256);
  pl->w_sw_bytes = align_up((size_t)pl->S * pl->b_stage_bytes, 256);
  pl->rec_bytes = gather_records_bytes(g);
  return true;
}

// Which variant serves this shape in this math mode: bf16 mode takes the single-pass kernel where it applies
// and otherwise the (more exact) split kernel, e.g. for 32 channels per offset group; auto / bf16x3 take the
// split kernel only.  Returns false when the tensor-core tier does not apply.
bool pick_variant(const Geom& g, int math_mode, bool* x3, Plan* pl) {
  if (math_mode == D2C_MATH_FP32) return false;
  if (math_mode == D2C_MATH_BF16 && make_plan(g, false, pl)) { *x3 = false; return true; }
  if (make_plan(g, true, pl)) { *x3 = true; return true; }
  return false;
}

template <typename Coords>
int run_fwd(const Geom& g, int math_mode, const Coords& coords, const float* x, const float* mask, const float* w,
            const float* bias, float* y, void* ws, cudaStream_t st) {
  bool x3 = false;
  Plan pl;
  if (!pick_variant(g, math_mode, &x3, &pl)) return D2C_ERR_MODE;
  uint8_t* wsp = reinterpret_cast<uint8_t*>(ws);
  void* x_cl = wsp; wsp += pl.x_cl_bytes;
  uint8_t* w_sw = wsp; wsp += pl.w_sw_bytes;
  uint4* recs = reinterpret_cast<uint4*>(wsp);
  int sm_count = 0, rc;
  if ((rc = device_sm_count(&sm_count))) return rc;
  ptx::bind_status_sink();

  const long long n_units = (long long)pl.n_tiles * pl.S;
  long long grid = n_units / kMinUnitsPerCta;
  if (grid > sm_count) grid = sm_count;
  if (grid < 1) grid = 1;
  bool whole_tiles_only = (pl.n_tiles % grid == 0);

  // CTA pairs (deform_sm100_fwd_pair.cuh) whenever there are at least two tiles and the device can co-schedule
  // clusters of 2 with this kernel's shared memory.  Opt-in (D2C_SM100_PAIR=1): measured slower than the
  // single-CTA kernel so far.
  const int n_tile_pairs = (pl.n_tiles + 1) / 2;
  const long long n_pair_units = (long long)n_tile_pairs * pl.S;
  int pair_b_stages = (kSmemLimit - 1024 - 256 - kAStages * kAStageBytes - kRStages * kRStageBytes) / (pl.b_stage_bytes / 2);
  if (pair_b_stages > 4) pair_b_stages = 4;
  const int pair_smem = kAStages * kAStageBytes + pair_b_stages * (pl.b_stage_bytes / 2) + kRStages * kRStageBytes + 256 + 1024;
  long long pair_clusters = 0;
  {
    static int pair_enabled = -1;
    if (pair_enabled < 0) {
      const char* e = getenv("D2C_SM100_PAIR");
      pair_enabled = (e && e[0] == '1') ? 1 : 0;
    }
    if (pair_enabled && !x3 && !pl.dual && pl.n_tiles >= 2 && pair_b_stages >= 2) {
      D2C_CUDA_TRY(cudaFuncSetAttribute(pair::fwd_sm100_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, pair_smem));
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(2 * (unsigned)sm_count, 1, 1);
      cfg.blockDim = dim3(kThreads, 1, 1);
      cfg.dynamicSmemBytes = (size_t)pair_smem;
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
      cfg.attrs = &attr; cfg.numAttrs = 1;
      int max_clusters = 0;
      if (cudaOccupancyMaxActiveClusters(&max_clusters, pair::fwd_sm100_pair_kernel, &cfg) == cudaSuccess && max_clusters > 0) {
        pair_clusters = n_pair_units / kMinUnitsPerCta;
        if (pair_clusters > max_clusters) pair_clusters = max_clusters;
        if (pair_clusters < 1) pair_clusters = 1;
        whole_tiles_only = (n_tile_pairs % pair_clusters == 0);
      } else {
        (void)cudaGetLastError();
      }
    }
  }

  prof_mark(st, "fwd_stage_operands");
  {
    dim3 sgrid((unsigned)((g.Vin + 31) / 32), (unsigned)((g.Cin + 63) / 64), (unsigned)g.B);
    if (x3) {
      stage_input_cl_f32_kernel<<<sgrid, 256, 0, st>>>(g.Cin, g.Vin, x, reinterpret_cast<float*>(x_cl));
      D2C_LAUNCH_CHECK();
      dim3 wgrid((unsigned)g.Cout, (unsigned)(g.Cin / 32));
      stage_weight_sw128_x3_kernel<<<wgrid, 64, 32 * g.K * sizeof(float), st>>>(g.Cout, g.Cin, g.K, g.cpg, pl.nh, w, w_sw);
      D2C_LAUNCH_CHECK();
    } else {
      stage_input_cl_f16_kernel<<<sgrid, 256, 0, st>>>(g.Cin, g.Vin, x, reinterpret_cast<__half*>(x_cl));
      D2C_LAUNCH_CHECK();
      dim3 wgrid((unsigned)g.Cout, (unsigned)(g.Cin / 64));
      stage_weight_sw128_kernel<<<wgrid, 64, 64 * g.K * sizeof(float), st>>>(g.Cout, g.Cin, g.K,
                                                                              pl.dual ? 64 : g.cpg, pl.nh, w, w_sw);
      D2C_LAUNCH_CHECK();
    }
    if ((rc = launch_sample_records(g, coords, mask, nullptr, recs, st, x3))) return rc;
    if (!whole_tiles_only) D2C_CUDA_TRY(cudaMemsetAsync(y, 0, sizeof(float) * (size_t)g.B * g.Cout * g.V, st));
  }

  FwdParams p;
  p.g = g; p.x_cl = x_cl; p.w_sw = w_sw; p.recs = recs; p.bias = bias; p.y = y;
  p.cs.dz = g.H * g.W * g.Cin; p.cs.dy = g.W * g.Cin; p.cs.dx = g.Cin;
  p.N = g.Cout; p.nh = pl.nh; p.S = pl.S; p.tiles_per_clip = pl.tiles_per_clip; p.n_tiles = pl.n_tiles;
  p.n_units = n_units;
  p.b_stages = pl.b_stages; p.b_stage_bytes = pl.b_stage_bytes; p.tmem_cols = pl.tmem_cols;

  if (pair_clusters > 0) {
    pair::PairParams pp;
    pp.f = p;
    pp.n_tile_pairs = n_tile_pairs; pp.n_pair_units = n_pair_units;
    pp.b_stages = pair_b_stages; pp.b_half_bytes = pl.b_stage_bytes / 2;
    prof_mark(st, "fwd_sm100_pair");
    pair::fwd_sm100_pair_kernel<<<(unsigned)(2 * pair_clusters), kThreads, pair_smem, st>>>(pp);
    D2C_LAUNCH_CHECK();
    prof_mark(st, nullptr);
    return D2C_OK;
  }
  prof_mark(st, "fwd_sm100_fused");
  static int fwd_v = -1;
  if (fwd_v < 0) {
    const char* e = getenv("D2C_FWD_V");
    fwd_v = (e && e[0] == '1') ? 1 : 2;
  }
  if (fwd_v == 2) {
    auto kern = x3 ? fwd_sm100_v2_kernel<1, 0> : (pl.dual ? fwd_sm100_v2_kernel<0, 1> : fwd_sm100_v2_kernel<0, 0>);
    D2C_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, pl.smem_bytes));
    kern<<<(unsigned)grid, kThreads2, pl.smem_bytes, st>>>(p);
  } else if (x3) {
    D2C_CUDA_TRY(cudaFuncSetAttribute(fwd_sm100_kernel<1, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, pl.smem_bytes));
    fwd_sm100_kernel<1, 0><<<(unsigned)grid, kThreads, pl.smem_bytes, st>>>(p);
  } else if (pl.dual) {
    D2C_CUDA_TRY(cudaFuncSetAttribute(fwd_sm100_kernel<0, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, pl.smem_bytes));
    fwd_sm100_kernel<0, 1><<<(unsigned)grid, kThreads, pl.smem_bytes, st>>>(p);
  } else {
    D2C_CUDA_TRY(cudaFuncSetAttribute(fwd_sm100_kernel<0, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, pl.smem_bytes));
    fwd_sm100_kernel<0, 0><<<(unsigned)grid, kThreads, pl.smem_bytes, st>>>(p);
  }
  D2C_LAUNCH_CHECK();
  prof_mark(st, nullptr);
  return D2C_OK;
}

}  // namespace

bool sm100_fwd_supported(const Geom& g, int dtype, int math_mode) {
  if (dtype != D2C_F32) return false;
  bool x3;
  Plan pl;
  return pick_variant(g, math_mode, &x3, &pl);
}

size_t sm100_fwd_workspace(const Geom& g, int dtype, int math_mode) {
  if (!sm100_fwd_supported(g, dtype, math_mode)) return 0;
  bool x3;
  Plan pl;
  pick_variant(g, math_mode, &x3, &pl);
  return pl.x_cl_bytes + pl.w_sw_bytes + pl.rec_bytes;
}

int sm100_fwd_offsets(const Geom& g, int math_mode, const float* x, const float* offset, const float* mask,
                      const float* w, const float* bias, float* y, void* ws, cudaStream_t st) {
  OffsetCoords<float> oc{offset};
  return run_fwd(g, math_mode, oc, x, mask, w, bias, y, ws, st);
}

int sm100_fwd_field(const Geom& g, int math_mode, const FieldCoords<float>& fc, const float* x,
                    const float* mask, const float* w, const float* bias, float* y, void* ws, cudaStream_t st) {
  return run_fwd(g, math_mode, fc, x, mask, w, bias, y, ws, st);
}

// ---- wait-expiry self-test ------------------------------------------------------------------------
// One warp initialises an mbarrier that nobody will ever arrive on, waits on it with the product kernels' own
// bounded wait (a short budget instead of the default) and, when the wait gives up, reports exactly as they
// do.  No tensor memory, no bulk copy: nothing is left in flight.  The kernel returns normally.
namespace {
__global__ void __launch_bounds__(32) selftest_wait_expiry_kernel(long long budget_cycles) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int abort_flag;
  const uint32_t bar_addr = ptx::smem_u32(&bar);
  if (threadIdx.x == 0) {
    ptx::mbar_init(bar_addr, 1);
    abort_flag = 0;
    ptx::fence_mbar_init();
  }
  __syncwarp();
  const bool done = ptx::mbar_wait(bar_addr, 0, &abort_flag, 100, budget_cycles);
  __syncwarp();
  if (threadIdx.x == 0 && (!done || abort_flag)) ptx::report_device_timeout();
}
}  // namespace

int sm100_selftest_wait_expiry(long long budget_cycles, cudaStream_t st) {
  ptx::bind_status_sink();
  selftest_wait_expiry_kernel<<<1, 32, 0, st>>>(budget_cycles);
  D2C_LAUNCH_CHECK();
  return D2C_OK;
}

}  // namespace d2c
