// Weight gradient of the deformable conv3d for sm_100a as an implicit GEMM over voxels that consumes
// the SAME sampled tile as the forward:
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
// In the fp32-parity mode (template parameter) a CTA owns ONE slice whose bf16 hi and lo parts are the two
// A tiles, and grad_out arrives as a hi and a lo image per voxel block: all four products are accumulated.
// Gather records reach the 16 producer warps through a bulk-copied shared-memory ring with a unit header,
// exactly as in the forward.
#include "deform_sm100.h"
#include "sm100_gather.cuh"
#include "sm100_ptx.cuh"

#include <algorithm>

namespace d2c {

namespace {

constexpr int kBM = 128;
constexpr int kBK = 64;
constexpr int kTileBytes = kBM * kBK * 2;            // one sampled slice tile: 16 KB
constexpr int kAStages = 2;
constexpr int kAStageBytes = 2 * kTileBytes;         // two slices
constexpr int kBStages = 2;
constexpr int kChunkBytes = 256 * 128;               // one 256-row (co) x 64-voxel image
constexpr int kThreads = (6 + 16 + 1) * 32;   // 4 epilogue + MMA + grad_out loader + 16 gather + record loader warps
constexpr int kEpiWarps = 4, kMmaWarp = 4, kLoadWarp = 5, kGatherWarp0 = 6, kGatherWarps = 16, kRecWarp = 22;
constexpr int kRStages = 4;                       // gather-record ring, one stage per (tile, slice) half-unit
constexpr int kRecBytes = kBM * 48;               // 6 KB of records per set; a stage adds a 16-byte header
                                                  // {int64 x_cl element offset of the slice, int rows}
constexpr int kRowStride = kGatherWarps * 4;          // 8 threads per row -> rows handled per pass
constexpr int kRowsPerThread = kBM / kRowStride;
constexpr int kSmemLimit = 227 * 1024;

struct DwParams {
  Geom g;
  const void* x_cl;          // channels-last staging of x: fp16 (bf16 mode) or fp32 (bf16x3 mode)
  const uint4* recs;         // gather records (sm100_gather.cuh)
  const uint8_t* gyk_img;    // [n_tiles][2 voxel blocks][NCH][32 KB]
  float* dws;                // [S*64][Cout] fp32, zero-initialised
  ClStrides cs;
  int N, nh, S, tiles_per_clip, n_tiles, tmem_cols;
  int n_pairs, tiles_per_split, NCH, b_stage_bytes;
  int pairg;                 // bf16x3 only: 32 channels per offset group, a slice = two neighbouring groups
};

// grad_out [B][Cout][V] fp32 -> per (tile, 64-voxel block, 256-co chunk) images: 256 rows (co) x 128 B
// (64 voxels, bf16), chunks XOR-swizzled by (row & 7).  Voxels past the clip are zero.
// x3 = 1 (fp32-parity mode): every (tile, voxel block) holds two image groups, hi = bf16(gy) then
// lo = bf16(gy - hi), NCH chunks each.
// grad_bias (nullable) = grad_out summed over clips and voxels (reference dconv3d_gpu.cu:1329): this kernel reads
// every element of grad_out exactly once, so the 16 threads that share a row add their 128-voxel partial sum with
// one atomic (grad_bias zeroed before).
__global__ void __launch_bounds__(256)
stage_gy_kmajor_kernel(int Cout, int V, int tiles_per_clip, int NCH, int x3, const float* __restrict__ gy,
                       uint8_t* __restrict__ img, float* __restrict__ grad_bias) {
  const int tile = blockIdx.x, coblk = blockIdx.y;        // coblk: 64 rows of co
  const int b = tile / tiles_per_clip, v0 = (tile % tiles_per_clip) * kBM;
  for (int e = threadIdx.x; e < 64 * 16; e += 256) {      // Cout is a multiple of 64: no thread leaves the loop early
    const int rl = e >> 4, q = e & 15;                    // row within block, 8-voxel chunk (0..15)
    const int co = coblk * 64 + rl;
    const int v = v0 + q * 8;
    float f[8];
    const float* src = gy + ((long long)b * Cout + co) * V;
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] = (v + i < V) ? __ldg(src + v + i) : 0.f;
    if (grad_bias) {
      float sum = ((f[0] + f[1]) + (f[2] + f[3])) + ((f[4] + f[5]) + (f[6] + f[7]));
      sum += __shfl_xor_sync(0xffffffffu, sum, 1);
      sum += __shfl_xor_sync(0xffffffffu, sum, 2);
      sum += __shfl_xor_sync(0xffffffffu, sum, 4);
      sum += __shfl_xor_sync(0xffffffffu, sum, 8);
      if (q == 0) atomicAdd(grad_bias + co, sum);
    }
    uint4 o;
    o.x = ptx::pack_bf16x2(f[0], f[1]); o.y = ptx::pack_bf16x2(f[2], f[3]);
    o.z = ptx::pack_bf16x2(f[4], f[5]); o.w = ptx::pack_bf16x2(f[6], f[7]);
    const int kblk = q >> 3, j = q & 7, chunk = co >> 8, row = co & 255;
    const long long in_img = (long long)(row >> 3) * 1024 + (row & 7) * 128 + ((j ^ (row & 7)) << 4);
    if (!x3) {
      *reinterpret_cast<uint4*>(img + (((long long)tile * 2 + kblk) * NCH + chunk) * kChunkBytes + in_img) = o;
    } else {
      uint4 l;
      l.x = ptx::pack_bf16x2(f[0] - ptx::bf16_lo(o.x), f[1] - ptx::bf16_hi(o.x));
      l.y = ptx::pack_bf16x2(f[2] - ptx::bf16_lo(o.y), f[3] - ptx::bf16_hi(o.y));
      l.z = ptx::pack_bf16x2(f[4] - ptx::bf16_lo(o.z), f[5] - ptx::bf16_hi(o.z));
      l.w = ptx::pack_bf16x2(f[6] - ptx::bf16_lo(o.w), f[7] - ptx::bf16_hi(o.w));
      const long long grp0 = ((long long)tile * 2 + kblk) * 2;
      *reinterpret_cast<uint4*>(img + ((grp0 + 0) * NCH + chunk) * kChunkBytes + in_img) = o;
      *reinterpret_cast<uint4*>(img + ((grp0 + 1) * NCH + chunk) * kChunkBytes + in_img) = l;
    }
  }
}

// kX3 = 0 (bf16 mode): a CTA owns a PAIR of 64-channel slices, the accumulator rows are (slice of the pair, c).
// kX3 = 1 (bf16x3, fp32-parity mode): a CTA owns ONE slice; the two A tiles of a stage are the bf16 hi and lo
//   parts of the fp32 sampled tile (rows 0-63 / 64-127 of the accumulator), every voxel block of grad_out comes
//   as a hi image and a lo image and both are accumulated: (a_hi + a_lo)(g_hi + g_lo), all four products; the
//   two accumulator halves meet in the same dws rows through the epilogue's reductions.
// kDual = 1 (bf16 mode only): 32 channels per offset group; a 64-channel slice spans two neighbouring groups, a
//   record stage holds both groups' records and the 16-byte chunks 0-3 / 4-7 of a row use the first / second set.
template <int kX3, int kDual>
__global__ void __launch_bounds__(kThreads, 1)
dw_sm100_kernel(const DwParams p) {
  static_assert(!(kX3 && kDual), "the fp32-parity kernel's 32-channel half-units need no second record set");
  constexpr int kBSteps = kX3 ? 4 : 2;      // grad_out images per tile: voxel block x (hi, lo)
  constexpr int kRStage = (1 + kDual) * kRecBytes + 16;     // record set(s) + header
  constexpr int hdr_off = (1 + kDual) * kRecBytes;
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t a_base = base, b_base = base + kAStages * kAStageBytes;
  const int rec_off = kAStages * kAStageBytes + kBStages * p.b_stage_bytes;
  const int bar_off = rec_off + kRStages * kRStage;
  const uint32_t rec_base = base + rec_off, bar_base = base + bar_off;
  auto a_full = [&](int s) { return bar_base + 8u * s; };
  auto a_empty = [&](int s) { return bar_base + 8u * (2 + s); };
  auto b_full = [&](int s) { return bar_base + 8u * (4 + s); };
  auto b_empty = [&](int s) { return bar_base + 8u * (6 + s); };
  const uint32_t acc_full = bar_base + 8u * 8;
  auto r_full = [&](int s) { return bar_base + 8u * (10 + s); };
  auto r_empty = [&](int s) { return bar_base + 8u * (10 + kRStages + s); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + bar_off + 8 * 9);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + bar_off + 8 * 9 + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const Geom& g = p.g;
  const int pair = blockIdx.x % p.n_pairs, split = blockIdx.x / p.n_pairs;
  const int tile_beg = split * p.tiles_per_split;
  const int tile_end = min(p.n_tiles, tile_beg + p.tiles_per_split);
  const int n_my_tiles = tile_end - tile_beg;          // may be <= 0 for a trailing split

  if (threadIdx.x == 0) {
    for (int s = 0; s < kAStages; ++s) { ptx::mbar_init(a_full(s), kGatherWarps); ptx::mbar_init(a_empty(s), 1); }
    for (int s = 0; s < kBStages; ++s) { ptx::mbar_init(b_full(s), 1); ptx::mbar_init(b_empty(s), 1); }
    for (int s = 0; s < kRStages; ++s) { ptx::mbar_init(r_full(s), 1); ptx::mbar_init(r_empty(s), kGatherWarps); }
    ptx::mbar_init(acc_full, 1);
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

  if (n_my_tiles > 0) {
    if (warp < kEpiWarps) {
      // ---- epilogue (once): accumulator rows (slice_local*64 + c) x columns co -> dws, vector reductions
      if (ptx::mbar_wait(acc_full, 0, abort_flag)) {
        ptx::tc_fence_after();
        const int m = warp * 32 + lane;
        const int s = kX3 ? pair : 2 * pair + (m >> 6);
        float* row = p.dws + ((long long)s * 64 + (m & 63)) * p.N;
        for (int c0 = 0; c0 < p.N; c0 += 32) {
          uint32_t r[32];
          ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, r);
          ptx::tmem_ld_wait();
          if (s < p.S) {
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
          const int sa = t % kAStages;
          if (!ptx::mbar_wait(a_full(sa), (t / kAStages) & 1, abort_flag)) break;
          for (int step = 0; step < kBSteps; ++step, ++kb) {
            const int kblk = kX3 ? (step >> 1) : step;
            const int sb = kb % kBStages;
            if (!ptx::mbar_wait(b_full(sb), (kb / kBStages) & 1, abort_flag)) { ok = false; break; }
            ptx::tc_fence_after();
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
              // A: 16 voxels starting at voxel kblk*64 + k4*16 -> two 8-row groups of 1024 bytes;
              //    the second slice's tile (rows 64..127 of M) sits kTileBytes further (LBO)
              const uint64_t adesc = ptx::umma_desc_mnmajor_sw128(
                  a_base + sa * kAStageBytes + (kblk * 8 + k4 * 2) * 1024, kTileBytes, 1024);
              for (int n0 = 0; n0 < p.N; n0 += 256) {
                const int nc = min(256, p.N - n0);
                const uint64_t bdesc =
                    ptx::umma_desc_kmajor_sw128(b_base + sb * p.b_stage_bytes + (n0 >> 8) * kChunkBytes) +
                    (uint64_t)(2 * k4);
                ptx::umma_bf16(tmem_base + (uint32_t)n0, adesc, bdesc,
                               ptx::umma_idesc_bf16_f32(kBM, nc) | (1u << 15) /* A is MN-major */,
                               (t > 0 || step > 0 || k4 > 0) ? 1u : 0u);
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
          for (int step = 0; step < kBSteps; ++step, ++kb) {
            const int sb = kb % kBStages;
            if (!ptx::mbar_wait(b_empty(sb), ((kb / kBStages) & 1) ^ 1, abort_flag)) { ok = false; break; }
            ptx::mbar_arrive_expect_tx(b_full(sb), (uint32_t)p.b_stage_bytes);
            const uint8_t* src = p.gyk_img + ((long long)(tile_beg + t) * kBSteps + step) * p.b_stage_bytes;
            for (int off = 0; off < p.b_stage_bytes; off += 32768)
              ptx::bulk_g2s(b_base + sb * p.b_stage_bytes + off, src + off, 32768u, b_full(sb));
          }
        }
        const uint32_t issued = kb;
        for (uint32_t q = (issued > (uint32_t)kBStages ? issued - kBStages : 0); q < issued; ++q) {
          const long long t0 = clock64();
          while (!ptx::mbar_try_wait(b_full(q % kBStages), (q / kBStages) & 1))
            if (clock64() - t0 > ptx::kWaitBudgetCycles) break;
        }
      }
    } else if (warp == kRecWarp) {
      // ---- gather-record loader: half-units q = 2*t + sl (tile t of the range, slice sl of the pair); the
      //      records of a half-unit's rows are one contiguous run, copied kRStages half-units ahead together
      //      with a header that spares the gather warps all index arithmetic
      if (lane == 0) {
        const int nq = 2 * n_my_tiles;
        // The CTA's two half-units per tile always use the same slices: everything that depends only on the slice
        // (offset group, tap, channel offset) is computed once; the tile's clip and first voxel advance by counters.
        // This single thread's instruction latency sits between "stage free" and "copy issued" for every half-unit,
        // so the loop holds no integer division.
        long long ch_off[2];
        int tap_[2], grp_rec_[2];
#pragma unroll
        for (int sl = 0; sl < 2; ++sl) {
          // bf16: slice sl of the pair (an odd last slice is produced twice, second copy unused);
          // x3: channels [32 sl, 32 sl + 32) of the CTA's slice
          const int sidx = kX3 ? pair : min(2 * pair + sl, p.S - 1);
          const int h = sidx % p.nh, gt = sidx / p.nh, tap = gt % g.K, grp = gt / g.K;
          // slices of two 32-channel groups: the half-unit's channels belong to group 2 grp + sl
          const int cpg = p.pairg ? kBK : g.cpg;
          ch_off[sl] = (long long)grp * cpg + h * kBK + (kX3 ? sl * 32 : 0);
          tap_[sl] = tap;
          grp_rec_[sl] = kDual ? grp : (p.pairg ? 2 * grp + sl : grp);
        }
        int b = tile_beg / p.tiles_per_clip, v0 = (tile_beg % p.tiles_per_clip) * kBM;
        int q = 0;
        for (; q < nq; ++q) {
          const int sl = q & 1;
          const int sr = q & (kRStages - 1);
          if (!ptx::mbar_wait(r_empty(sr), ((q / kRStages) & 1) ^ 1, abort_flag, 200)) break;
          const int rows = min(kBM, g.V - v0);
          uint8_t* hdr = base_ptr + rec_off + sr * kRStage + hdr_off;
          *reinterpret_cast<long long*>(hdr) = (long long)b * g.Vin * g.Cin + ch_off[sl];
          *reinterpret_cast<int*>(hdr + 8) = rows;
          ptx::mbar_arrive_expect_tx(r_full(sr), (uint32_t)rows * 48u * (uint32_t)(1 + kDual));
#pragma unroll
          for (int set = 0; set <= kDual; ++set) {
            const int og = kDual ? 2 * grp_rec_[sl] + set : grp_rec_[sl];     // offset group whose records fill this set
            ptx::bulk_g2s(rec_base + sr * kRStage + set * kRecBytes,
                          p.recs + 3 * ((((long long)b * g.G + og) * g.K + tap_[sl]) * g.V + v0), (uint32_t)rows * 48u,
                          r_full(sr));
          }
          if (sl == 1) {                      // next tile of the range
            v0 += kBM;
            if (v0 >= p.tiles_per_clip * kBM) { v0 = 0; ++b; }
          }
        }
        const int issued = q;
        for (int w = (issued > kRStages ? issued - kRStages : 0); w < issued; ++w) {
          const long long t0 = clock64();
          while (!ptx::mbar_try_wait(r_full(w % kRStages), (w / kRStages) & 1))
            if (clock64() - t0 > ptx::kWaitBudgetCycles) break;
        }
      }
    } else {
      // ---- gather producers: the forward's producer, two slices per stage
      const int tt = threadIdx.x - kGatherWarp0 * 32;
      const int j = tt & 7, r0 = tt >> 3;
      uint32_t row_dst[kRowsPerThread];
#pragma unroll
      for (int i = 0; i < kRowsPerThread; ++i) {
        const int r = r0 + kRowStride * i;
        row_dst[i] = (uint32_t)((r >> 3) * 1024 + (r & 7) * 128 + ((j ^ (r & 7)) << 4));
      }
      const int nq = 2 * n_my_tiles;
      for (int q = 0; q < nq; ++q) {
        const int t = q >> 1, sl = q & 1, sa = t % kAStages, sr = q % kRStages;
        if (!ptx::mbar_wait(r_full(sr), (q / kRStages) & 1, abort_flag)) break;
        const uint8_t* rec_stage0 = base_ptr + rec_off + sr * kRStage;
        const long long xoff = *reinterpret_cast<const long long*>(rec_stage0 + hdr_off);
        const int rows = *reinterpret_cast<const int*>(rec_stage0 + hdr_off + 8);
        // dual: channels 32-63 of the slice (16-byte chunks 4-7) belong to the second offset group
        const uint8_t* rec_stage = rec_stage0 + ((kDual && j >= 4) ? kRecBytes : 0);
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
        if (sl == 0 && !ptx::mbar_wait(a_empty(sa), ((t / kAStages) & 1) ^ 1, abort_flag)) break;
        const uint32_t stage = a_base + sa * kAStageBytes + (kX3 ? 0 : sl * kTileBytes);
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
            // channels 32 sl + 4j .. + 3 of the slice: 16-byte chunk 4 sl + j/2, half j&1; hi tile, lo tile
            const uint32_t in_tile = (uint32_t)((r >> 3) * 1024 + (r & 7) * 128) +
                                     (uint32_t)((((4 * sl + (j >> 1)) ^ (r & 7)) << 4) + (j & 1) * 8);
            blend_split_store(c[i], w, stage + in_tile, stage + kTileBytes + in_tile);
          } else {
            uint4 w03 = make_uint4(0u, 0u, 0u, 0u), w47 = w03;   // rows past the clip end: stage bytes are stale
            if (r < rows) {
              w03 = *reinterpret_cast<const uint4*>(rec_stage + r * 48 + 16);
              w47 = *reinterpret_cast<const uint4*>(rec_stage + r * 48 + 32);
            }
            blend_store(c[i], w03, w47, stage + row_dst[i]);
          }
        }
        if (sl == 1) ptx::fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (sl == 1) ptx::mbar_arrive(a_full(sa));
          ptx::mbar_arrive(r_empty(sr));
        }
      }
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) ptx::report_device_timeout();
  if (warp == 0) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  }
}

// ---- weight gradient from the samples the forward kept ------------------------------------------------------
// When the forward of the same call pair wrote its blended A tiles to global memory (FwdParams::sav in
// deform_sm100_fwd.cu), nothing is gathered or blended again: the sampled operand arrives by bulk copy like
// grad_out does, and the kernel is a plain two-operand streaming GEMM.
//   ring granularity = one 64-voxel block: A stage = the block's 8 KB images of the CTA's slice pair
//     bf16 mode : [slice 0 | slice 1]                         16 KB, M = 128 rows (slice of the pair, channel)
//     bf16x3    : [hi s0 | hi s1 | lo s0 | lo s1]             32 KB; hi and lo are two M = 128 operands that
//                 accumulate into the SAME rows: a_hi*g_hi + a_lo*g_hi + a_hi*g_lo, three products, no lo*lo
//   B ring = 32 KB chunks (256 co rows x 64 voxels) of the grad_out images, in the order
//     (block, [hi, lo], chunk) -- the order stage_gy_kmajor_kernel writes them, so the q-th chunk of a CTA is
//     one linear step further.
constexpr int kSvThreads = 7 * 32;        // 4 epilogue warps, MMA issuer, grad_out loader, sample loader
constexpr int kSvLoadWarp = 5, kSvSampleWarp = 6;
constexpr int kSvBlkBytes = 8192;         // one 64-channel slice x 64 voxels
constexpr int kSvBStages = 5;
constexpr int kSvARingBytes = 64 * 1024;  // 4 stages of 16 KB (bf16) or 2 stages of 32 KB (bf16x3)

struct DwSavedParams {
  const uint8_t* sav;        // sample image, see FwdParams::sav
  const uint8_t* gyk_img;    // grad_out images of stage_gy_kmajor_kernel
  float* dws;                // [S*64][Cout] fp32, zero-initialised
  int N, S, NCH, n_pairs, n_tiles, tiles_per_split, tmem_cols;
};

template <int kX3>
__global__ void __launch_bounds__(kSvThreads, 1)
dw_saved_sm100_kernel(const DwSavedParams p) {
  constexpr int kAStage = (kX3 ? 4 : 2) * kSvBlkBytes;
  constexpr int kASt = kSvARingBytes / kAStage;
  constexpr int kParts = kX3 ? 2 : 1;                 // grad_out image groups per block: hi, lo
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const uint32_t a_base = base, b_base = base + kSvARingBytes;
  const int bar_off = kSvARingBytes + kSvBStages * kChunkBytes;
  const uint32_t bar_base = base + bar_off;
  auto a_full = [&](int s) { return bar_base + 8u * s; };
  auto a_empty = [&](int s) { return bar_base + 8u * (4 + s); };
  auto b_full = [&](int s) { return bar_base + 8u * (8 + s); };
  auto b_empty = [&](int s) { return bar_base + 8u * (8 + kSvBStages + s); };
  const uint32_t acc_full = bar_base + 8u * (8 + 2 * kSvBStages);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + bar_off + 8 * (9 + 2 * kSvBStages));
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + bar_off + 8 * (9 + 2 * kSvBStages) + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int pair = blockIdx.x % p.n_pairs, split = blockIdx.x / p.n_pairs;
  const int tile_beg = split * p.tiles_per_split;
  const int tile_end = min(p.n_tiles, tile_beg + p.tiles_per_split);
  const int n_blocks = 2 * (tile_end - tile_beg);      // 64-voxel blocks; may be <= 0 for a trailing split

  if (threadIdx.x == 0) {
    for (int s = 0; s < kASt; ++s) { ptx::mbar_init(a_full(s), 1); ptx::mbar_init(a_empty(s), 1); }
    for (int s = 0; s < kSvBStages; ++s) { ptx::mbar_init(b_full(s), 1); ptx::mbar_init(b_empty(s), 1); }
    ptx::mbar_init(acc_full, 1);
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

  if (n_blocks > 0) {
    if (warp < kEpiWarps) {
      // ---- epilogue (once): accumulator rows (slice of the pair, c) x columns co -> dws, vector reductions
      if (ptx::mbar_wait(acc_full, 0, abort_flag, 1000)) {
        ptx::tc_fence_after();
        const int m = warp * 32 + lane;
        const int s = 2 * pair + (m >> 6);
        float* row = p.dws + ((long long)s * 64 + (m & 63)) * p.N;
        for (int c0 = 0; c0 < p.N; c0 += 32) {
          uint32_t r[32];
          ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0, r);
          ptx::tmem_ld_wait();
          if (s < p.S) {
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
        int sb = 0;
        uint32_t phb = 0;
        bool ok = true;
        for (int kb = 0; ok && kb < n_blocks; ++kb) {
          const int sa = kb % kASt;
          if (!ptx::mbar_wait(a_full(sa), (kb / kASt) & 1, abort_flag)) break;
          const uint32_t a_stage = a_base + sa * kAStage;
          for (int part = 0; ok && part < kParts; ++part) {
            // the NCH chunks of this image group: wait for all of them, then walk the K steps with the column
            // ranges innermost, so that consecutive MMAs alternate between accumulators (back-to-back MMAs into
            // the same columns issue at 217 clocks, alternating ones at 139)
            int sbc[2] = {0, 0};
            uint64_t bdesc0[2] = {0, 0};
            uint32_t idesc[2] = {0, 0};
#pragma unroll
            for (int c = 0; c < 2; ++c) {             // NCH <= 2 (Cout <= 512); fixed bounds keep these in registers
              if (c < p.NCH && ok) {
                if (!ptx::mbar_wait(b_full(sb), phb, abort_flag)) { ok = false; }
                sbc[c] = sb;
                bdesc0[c] = ptx::umma_desc_kmajor_sw128(b_base + sb * kChunkBytes);
                idesc[c] = ptx::umma_idesc_bf16_f32(kBM, min(256, p.N - 256 * c)) | (1u << 15);   // A is MN-major
                if (++sb == kSvBStages) { sb = 0; phb ^= 1u; }
              }
            }
            if (!ok) break;
            ptx::tc_fence_after();
#pragma unroll
            for (int k4 = 0; k4 < 4; ++k4) {
              // A: 16 voxels from voxel k4*16 of the block = two 8-row groups of 1024 bytes (SBO); the second
              // slice of the pair (rows 64..127 of M) lies one 8 KB image further (LBO)
              const uint64_t a_hi = ptx::umma_desc_mnmajor_sw128(a_stage + k4 * 2048, kSvBlkBytes, 1024);
              const uint64_t a_lo = ptx::umma_desc_mnmajor_sw128(a_stage + 2 * kSvBlkBytes + k4 * 2048, kSvBlkBytes, 1024);
              const uint32_t acc = (kb > 0 || k4 > 0) ? 1u : 0u;
              if (!kX3 || part == 0) {
#pragma unroll
                for (int c = 0; c < 2; ++c)                                                  // a (a_hi) * g (g_hi)
                  if (c < p.NCH)
                    ptx::umma_bf16(tmem_base + (uint32_t)(256 * c), a_hi, bdesc0[c] + (uint64_t)(2 * k4), idesc[c], acc);
                if (kX3) {
#pragma unroll
                  for (int c = 0; c < 2; ++c)                                                // a_lo * g_hi
                    if (c < p.NCH)
                      ptx::umma_bf16(tmem_base + (uint32_t)(256 * c), a_lo, bdesc0[c] + (uint64_t)(2 * k4), idesc[c], 1u);
                }
              } else {
#pragma unroll
                for (int c = 0; c < 2; ++c)                                                  // a_hi * g_lo
                  if (c < p.NCH)
                    ptx::umma_bf16(tmem_base + (uint32_t)(256 * c), a_hi, bdesc0[c] + (uint64_t)(2 * k4), idesc[c], 1u);
              }
            }
#pragma unroll
            for (int c = 0; c < 2; ++c)
              if (c < p.NCH) ptx::umma_commit(b_empty(sbc[c]));
          }
          if (ok) ptx::umma_commit(a_empty(sa));
        }
        if (ok) ptx::umma_commit(acc_full);
      }
    } else if (warp == kSvLoadWarp) {
      // ---- grad_out chunks: one linear stream per CTA
      if (lane == 0) {
        const int cpb = kParts * p.NCH;                       // chunks per block
        const uint32_t nq = (uint32_t)n_blocks * (uint32_t)cpb;
        const uint8_t* src = p.gyk_img + (long long)tile_beg * 2 * cpb * kChunkBytes;
        uint32_t q = 0;
        int sb = 0, c = 0;
        uint32_t phb = 1;                                     // the wait for a FREE slot looks at the previous phase
        for (; q < nq; ++q) {
          if (!ptx::mbar_wait(b_empty(sb), phb, abort_flag, 100)) break;
          const uint32_t bytes = (uint32_t)min(256, p.N - 256 * c) * 128u;
          ptx::mbar_arrive_expect_tx(b_full(sb), bytes);
          ptx::bulk_g2s(b_base + sb * kChunkBytes, src, bytes, b_full(sb));
          src += kChunkBytes;
          if (++c == p.NCH) c = 0;
          if (++sb == kSvBStages) { sb = 0; phb ^= 1u; }
        }
        // never leave with a bulk copy in flight: wait (bounded) for the last copies issued
        for (uint32_t w = (q > (uint32_t)kSvBStages ? q - kSvBStages : 0); w < q; ++w) {
          const long long t0 = clock64();
          while (!ptx::mbar_try_wait(b_full(w % kSvBStages), (w / kSvBStages) & 1))
            if (clock64() - t0 > ptx::kWaitBudgetCycles) break;
        }
      }
    } else if (warp == kSvSampleWarp) {
      // ---- kept samples: the slice pair's images of every 64-voxel block of the range
      if (lane == 0) {
        const long long blk_stride = (long long)p.n_pairs * kAStage;   // bytes between consecutive blocks
        const uint8_t* src = p.sav + (long long)tile_beg * 2 * blk_stride + (long long)pair * kAStage;
        int kb = 0;
        const uint64_t pol_stream = ptx::l2_evict_first();    // every byte of the image is read exactly once
        for (; kb < n_blocks; ++kb) {
          const int sa = kb % kASt;
          if (!ptx::mbar_wait(a_empty(sa), ((kb / kASt) & 1) ^ 1, abort_flag, 100)) break;
          ptx::mbar_arrive_expect_tx(a_full(sa), (uint32_t)kAStage);
          ptx::bulk_g2s_hint(a_base + sa * kAStage, src, (uint32_t)kAStage, a_full(sa), pol_stream);
          src += blk_stride;
        }
        for (int w = (kb > kASt ? kb - kASt : 0); w < kb; ++w) {
          const long long t0 = clock64();
          while (!ptx::mbar_try_wait(a_full(w % kASt), (w / kASt) & 1))
            if (clock64() - t0 > ptx::kWaitBudgetCycles) break;
        }
      }
    }
  }
  ptx::tc_fence_before();
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) ptx::report_device_timeout();
  if (warp == 0) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
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
  bool pairg;
  int nh, S, tiles_per_clip, n_tiles, tmem_cols;
  int n_pairs, nsplit, tiles_per_split, NCH, b_stage_bytes, smem_bytes;
  size_t gyk_bytes, dws_bytes;
};

bool make_dw_plan(const Geom& g, int sm_count, bool x3, DwPlan* dp) {
  dp->pairg = g.cpg == 32 && g.G % 2 == 0;      // bf16 mode: two record sets per stage (kDual)
  if (g.groups != 1 || (g.cpg % kBK != 0 && !dp->pairg) || g.Cout % 64 != 0 || g.Cout > 512) return false;
  if (g.Vin * g.Cin > 0x7fffffffLL) return false;
  dp->nh = dp->pairg ? 1 : g.cpg / kBK;
  dp->S = dp->pairg ? (g.G / 2) * g.K : g.G * g.K * dp->nh;
  dp->tiles_per_clip = (g.V + kBM - 1) / kBM;
  dp->n_tiles = dp->tiles_per_clip * g.B;
  int cols = 32;
  while (cols < g.Cout) cols <<= 1;
  dp->tmem_cols = cols;
  dp->n_pairs = x3 ? dp->S : (dp->S + 1) / 2;
  dp->NCH = (g.Cout + 255) / 256;
  dp->b_stage_bytes = dp->NCH * kChunkBytes;
  const int r_stage = ((dp->pairg && !x3) ? 2 : 1) * kRecBytes + 16;
  dp->smem_bytes = kAStages * kAStageBytes + kBStages * dp->b_stage_bytes + kRStages * r_stage + 256 + 1024;
  if (dp->smem_bytes > kSmemLimit) return false;
  // enough (pair, voxel-range) work items for ~3 waves, but at least 8 tiles per item
  int nsplit = (3 * sm_count + dp->n_pairs - 1) / dp->n_pairs;
  const int max_split = (dp->n_tiles + 7) / 8;
  if (nsplit > max_split) nsplit = max_split;
  if (nsplit < 1) nsplit = 1;
  // The tensor cores add into their fp32 accumulator with truncation (a chain of n accumulating MMAs loses about
  // n * 2^-26 of the result), so the fp32-parity mode ends an accumulation chain after 40 tiles (640 MMAs, ~1e-5);
  // partial sums of different voxel ranges meet in `dws` through fp32 reductions anyway.
  if (x3) {
    const int min_split = (dp->n_tiles + 39) / 40;
    if (nsplit < min_split) nsplit = min_split;
  }
  dp->tiles_per_split = (dp->n_tiles + nsplit - 1) / nsplit;
  dp->nsplit = (dp->n_tiles + dp->tiles_per_split - 1) / dp->tiles_per_split;
  dp->gyk_bytes = align_up((size_t)dp->n_tiles * (x3 ? 4 : 2) * dp->b_stage_bytes, 256);
  dp->dws_bytes = align_up((size_t)dp->S * 64 * g.Cout * 4, 256);
  return true;
}

// Work split of the saved-samples kernel: (slice pair, voxel range) items, at least two waves of them, ranges of at
// least 8 tiles, the smallest count whose last wave is at least 95 % full (else the fullest); the fp32-parity mode ends an
// accumulation chain after 27 tiles (24 accumulating MMAs per tile and column range -> 648, see make_dw_plan).
void split_saved(const DwPlan& dp, int sm_count, bool x3, int* tiles_per_split, int* nsplit_out) {
  const int n_pairs = (dp.S + 1) / 2;
  const int chain_min = x3 ? (dp.n_tiles + 26) / 27 : 1;              // fewest ranges the chain cap allows
  const int size_max = std::max(1, dp.n_tiles / 8);                   // most ranges of at least 8 tiles
  const int lo = std::max(chain_min, std::min(size_max, (2 * sm_count + n_pairs - 1) / n_pairs));
  const int hi = std::max(lo, std::min(size_max, lo + 8));
  int best = lo;
  double best_eff = -1.0;
  for (int ns = lo; ns <= hi; ++ns) {
    const int tps = (dp.n_tiles + ns - 1) / ns;
    const long long ctas = (long long)((dp.n_tiles + tps - 1) / tps) * n_pairs;
    const long long waves = (ctas + sm_count - 1) / sm_count;
    const double eff = (double)ctas / (double)(waves * sm_count);
    if (eff > best_eff + 1e-9) { best_eff = eff; best = ns; }
    if (eff >= 0.95) break;      // full enough: every further range costs one more epilogue and pipeline fill per pair
  }
  *tiles_per_split = (dp.n_tiles + best - 1) / best;
  *nsplit_out = (dp.n_tiles + *tiles_per_split - 1) / *tiles_per_split;
}

constexpr int kSvSmemBytes = kSvARingBytes + kSvBStages * kChunkBytes + 256 + 1024;
static_assert(kSvSmemBytes <= kSmemLimit, "saved-samples kernel: shared memory");

}  // namespace

bool sm100_sample_image_plan(const Geom& g, bool x3, int* n_pairs, size_t* bytes) {
  DwPlan dp;
  if (!make_dw_plan(g, 148, x3, &dp)) return false;
  const int np = (dp.S + 1) / 2;
  // block indices travel as 31-bit words through the forward's unit header
  if ((long long)dp.n_tiles * np * 16 >= 0x7fffffffLL) return false;
  *n_pairs = np;
  *bytes = (size_t)dp.n_tiles * 2 * np * (x3 ? 4 : 2) * kSvBlkBytes;
  return true;
}

bool sm100_sample_cache_layout(const Geom& g, bool x3, int* n_pairs, SampleCacheLayout* lay) {
  size_t img = 0;
  if (!sm100_sample_image_plan(g, x3, n_pairs, &img)) return false;
  lay->image_bytes = align_up(img, 256);
  lay->x_cl_bytes = align_up((size_t)g.B * g.Vin * g.Cin * (x3 ? 4 : 2), 256);
  lay->pos_bytes = pos_records_bytes(g);
  return true;
}

size_t sm100_dw_workspace(const Geom& g, bool x3) {
  DwPlan dp;
  if (!make_dw_plan(g, 148, x3, &dp)) return 0;
  return dp.gyk_bytes + dp.dws_bytes;
}

int sm100_dw(const Geom& g, bool x3, const float* gy, const void* x_cl, const void* recs, float* grad_w,
             float* grad_bias, void* ws, cudaStream_t st, const void* sav) {
  int sm_count = 0;
  {
    const int rc = device_sm_count(&sm_count);
    if (rc) return rc;
  }
  ptx::bind_status_sink();
  DwPlan dp;
  if (!make_dw_plan(g, sm_count, x3, &dp)) return D2C_ERR_MODE;
  uint8_t* gyk = reinterpret_cast<uint8_t*>(ws);
  float* dws = reinterpret_cast<float*>(gyk + dp.gyk_bytes);

  prof_mark(st, "bwd_dw_stage");
  D2C_CUDA_TRY(cudaMemsetAsync(dws, 0, (size_t)dp.S * 64 * g.Cout * 4, st));
  stage_gy_kmajor_kernel<<<dim3((unsigned)dp.n_tiles, (unsigned)((g.Cout + 63) / 64)), 256, 0, st>>>(
      g.Cout, g.V, dp.tiles_per_clip, dp.NCH, x3 ? 1 : 0, gy, gyk, grad_bias);
  D2C_LAUNCH_CHECK();

  DwParams p;
  p.g = g; p.x_cl = x_cl; p.recs = reinterpret_cast<const uint4*>(recs);
  p.gyk_img = gyk; p.dws = dws;
  p.cs.dz = g.H * g.W * g.Cin; p.cs.dy = g.W * g.Cin; p.cs.dx = g.Cin;
  p.N = g.Cout; p.nh = dp.nh; p.S = dp.S; p.tiles_per_clip = dp.tiles_per_clip; p.n_tiles = dp.n_tiles;
  p.tmem_cols = dp.tmem_cols;
  p.n_pairs = dp.n_pairs; p.tiles_per_split = dp.tiles_per_split; p.NCH = dp.NCH; p.b_stage_bytes = dp.b_stage_bytes;
  p.pairg = dp.pairg ? 1 : 0;
  if (sav) {
    DwSavedParams sp;
    sp.sav = reinterpret_cast<const uint8_t*>(sav); sp.gyk_img = gyk; sp.dws = dws;
    sp.N = g.Cout; sp.S = dp.S; sp.NCH = dp.NCH; sp.n_pairs = (dp.S + 1) / 2; sp.n_tiles = dp.n_tiles;
    sp.tmem_cols = dp.tmem_cols;
    int nsplit = 1;
    split_saved(dp, sm_count, x3, &sp.tiles_per_split, &nsplit);
    prof_mark(st, "bwd_dw_sm100_saved");
    auto kern = x3 ? dw_saved_sm100_kernel<1> : dw_saved_sm100_kernel<0>;
    D2C_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSvSmemBytes));
    kern<<<sp.n_pairs * nsplit, kSvThreads, kSvSmemBytes, st>>>(sp);
    D2C_LAUNCH_CHECK();
  } else {
    prof_mark(st, "bwd_dw_sm100");
    auto kern = x3 ? dw_sm100_kernel<1, 0> : (dp.pairg ? dw_sm100_kernel<0, 1> : dw_sm100_kernel<0, 0>);
    D2C_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, dp.smem_bytes));
    kern<<<dp.n_pairs * dp.nsplit, kThreads, dp.smem_bytes, st>>>(p);
    D2C_LAUNCH_CHECK();
  }
  prof_mark(st, "bwd_dw_unstage");
  unstage_dw_kernel<<<dim3((unsigned)((dp.S * 64 + 31) / 32), (unsigned)((g.Cout + 31) / 32)), 256, 0, st>>>(
      g.Cout, g.Cin, g.K, dp.pairg ? kBK : g.cpg, dp.nh, dp.S, dws, grad_w);
  D2C_LAUNCH_CHECK();
  return D2C_OK;
}

}  // namespace d2c
