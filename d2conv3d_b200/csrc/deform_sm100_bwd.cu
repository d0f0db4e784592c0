// Tensor-core backward of the modulated deformable conv3d for sm_100a (data side):
//
//   (a) dcol_sm100_kernel   gradient columns dcol[b, v, (slice, c)] = sum_co grad_out[b, co, v] * W[co, c, tap]
//                           as a tcgen05 GEMM (bf16 operands, fp32 accumulate in TMEM), voxel-major
//                           rows so that the 64 channels of one (offset group, tap) slice are contiguous.
//                           Replaces the reference's cuBLAS call at csrc/ops/dconv3d_gpu.cu:981-999.
//   (b) sample_grad_kernel  one pass over dcol that produces grad_offset / grad_mask (8 corner dot-products
//                           per (voxel, group, tap), reduced over channels by warp shuffles) AND scatters
//                           grad_input with 16-byte vector reductions into a channels-last fp32 buffer.
//                           Replaces deformable_col2im_coord_gpu_kernel (:756-864) and
//                           deformable_col2im_gpu_kernel (:562-643).
//   (c) unstage_grad_input_kernel  channels-last fp32 -> NCDHW.
//
// The weight gradient is in deform_sm100_dw.cu; sampling positions come from the records of
// sm100_gather.cuh, computed once per backward call.
#include "deform_generic.cuh"   // grad_bias_kernel, bwd_slice_clips
#include <type_traits>

#include "deform_sm100.h"
#include "sm100_gather.cuh"
#include "sm100_ptx.cuh"
#include "sm100_stage.cuh"

namespace d2c {

namespace {

constexpr int kBM = 128;
constexpr int kABlockBytes = kBM * 128;       // one 64-wide K block of the grad_out tile: 16 KB
constexpr int kNBlock = 256;                  // dcol columns per accumulator (4 slices of 64 channels)
constexpr int kBStageBytes = kNBlock * 128;   // 32 KB
constexpr int kBStages = 3;
constexpr int kDcolEpiWarps = 8;              // warp w: TMEM lane quarter w%4, column half w/4
constexpr int kDcolMmaWarp = 8, kDcolLoadWarp = 9;
constexpr int kDcolThreads = 320;
constexpr int kSmemLimit = 227 * 1024;

// ---- staging ------------------------------------------------------------------------------------

// grad_out [B][Cout][V] fp32 -> per (tile, 64-wide co block) images of 128 rows (voxels) x 128 B (64 co,
// bf16), 16-byte chunks XOR-swizzled by (row & 7): the byte image of a K-major SW128 A tile.
// Rows past the end of the clip are zero.
// x3 = 1 (fp32-parity mode): a K block is 32 co and a row is [hi(32 co) | lo(32 co)], hi = bf16(g),
// lo = bf16(g - hi).
// x3 = 2 (fp32-parity mode, long contractions): K blocks of 64 co as in the single-pass mode, written twice: the hi
// parts as one image and the lo parts as a second image `lo_off` bytes further.
__device__ __forceinline__ float split_part(float f, bool lo) {
  return lo ? f - ptx::bf16_lo(ptx::pack_bf16x2(f, 0.f)) : f;
}

__global__ void __launch_bounds__(256)
stage_gy_img_kernel(int Cout, int V, int tiles_per_clip, int b0, int x3, const float* __restrict__ gy,
                    uint8_t* __restrict__ img, long long lo_off) {
  __shared__ float tile[64][129];
  const int tile_id = blockIdx.x, kb = blockIdx.y, KB = gridDim.y;
  const int bl = tile_id / tiles_per_clip, v0 = (tile_id % tiles_per_clip) * kBM;
  const int b = b0 + bl;
  const int nco = x3 == 1 ? 32 : 64;
  for (int e = threadIdx.x; e < nco * 128; e += 256) {
    const int co = e >> 7, r = e & 127, v = v0 + r;
    tile[co][r] = (v < V) ? __ldg(gy + ((long long)b * Cout + kb * nco + co) * V + v) : 0.f;
  }
  __syncthreads();
  uint8_t* dst = img + ((long long)tile_id * KB + kb) * kABlockBytes;
  for (int e = threadIdx.x; e < 128 * 8; e += 256) {
    const int r = e >> 3, j = e & 7;
    const bool lo = x3 == 1 && j >= 4;
    const int cb = x3 == 1 ? (j & 3) * 8 : j * 8;
    const long long at = (r >> 3) * 1024 + (r & 7) * 128 + ((j ^ (r & 7)) << 4);
    uint4 o;
    o.x = ptx::pack_bf16x2(split_part(tile[cb + 0][r], lo), split_part(tile[cb + 1][r], lo));
    o.y = ptx::pack_bf16x2(split_part(tile[cb + 2][r], lo), split_part(tile[cb + 3][r], lo));
    o.z = ptx::pack_bf16x2(split_part(tile[cb + 4][r], lo), split_part(tile[cb + 5][r], lo));
    o.w = ptx::pack_bf16x2(split_part(tile[cb + 6][r], lo), split_part(tile[cb + 7][r], lo));
    *reinterpret_cast<uint4*>(dst + at) = o;
    if (x3 == 2) {
      o.x = ptx::pack_bf16x2(split_part(tile[cb + 0][r], true), split_part(tile[cb + 1][r], true));
      o.y = ptx::pack_bf16x2(split_part(tile[cb + 2][r], true), split_part(tile[cb + 3][r], true));
      o.z = ptx::pack_bf16x2(split_part(tile[cb + 4][r], true), split_part(tile[cb + 5][r], true));
      o.w = ptx::pack_bf16x2(split_part(tile[cb + 6][r], true), split_part(tile[cb + 7][r], true));
      *reinterpret_cast<uint4*>(dst + lo_off + at) = o;
    }
  }
}

// W [Cout][Cin][K] fp32 -> per (N block of 4 slices, 64-wide co block) images of 256 rows x 128 B:
// row = slice_local*64 + c, 64 co (bf16) per row, swizzled as above (K-major SW128 B tile, K = co).
// Block = (64-wide co block kb, input channel cin): the 64 x K weights W[kb*64 + q][cin][0..K) are read
// as 64 contiguous runs of K floats into shared memory, then each tap's 64 co values are written as one
// 128-byte row (8 swizzled 16-byte chunks).
__global__ void __launch_bounds__(64)
stage_wt_img_kernel(int Cout, int Cin, int K, int cpg, int nh, int x3, const float* __restrict__ w,
                    uint8_t* __restrict__ img, long long lo_off) {
  extern __shared__ float wsm[];                    // [64 (x3: 32) co][K]
  const int kb = blockIdx.x, cin = blockIdx.y, KB = gridDim.x;
  const int nco = x3 == 1 ? 32 : 64;
  for (int i = threadIdx.x; i < nco * K; i += 64) {
    const int q = i / K, t = i - q * K;
    wsm[i] = __ldg(w + ((long long)(kb * nco + q) * Cin + cin) * K + t);
  }
  __syncthreads();
  const int grp = cin / cpg, h = (cin % cpg) / 64, c = cin & 63;
  for (int item = threadIdx.x; item < K * 8; item += 64) {
    const int tap = item >> 3, j = item & 7;
    const bool lo = x3 == 1 && j >= 4;
    const int cb = x3 == 1 ? (j & 3) * 8 : j * 8;
    float v[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) v[q] = split_part(wsm[(cb + q) * K + tap], lo);
    uint4 o;
    o.x = ptx::pack_bf16x2(v[0], v[1]); o.y = ptx::pack_bf16x2(v[2], v[3]);
    o.z = ptx::pack_bf16x2(v[4], v[5]); o.w = ptx::pack_bf16x2(v[6], v[7]);
    const int s = (grp * K + tap) * nh + h;
    const int nb = s >> 2, row = (s & 3) * 64 + c;
    uint8_t* dst = img + ((long long)nb * KB + kb) * kBStageBytes + (row >> 3) * 1024 + (row & 7) * 128 +
                   ((j ^ (row & 7)) << 4);
    *reinterpret_cast<uint4*>(dst) = o;
    if (x3 == 2) {
#pragma unroll
      for (int q = 0; q < 8; ++q) v[q] = split_part(wsm[(cb + q) * K + tap], true);
      o.x = ptx::pack_bf16x2(v[0], v[1]); o.y = ptx::pack_bf16x2(v[2], v[3]);
      o.z = ptx::pack_bf16x2(v[4], v[5]); o.w = ptx::pack_bf16x2(v[6], v[7]);
      *reinterpret_cast<uint4*>(dst + lo_off) = o;
    }
  }
}

// ---- (a) dcol GEMM ------------------------------------------------------------------------------
// Work units are (tile, 256-column block); each CTA takes one contiguous range of them, so the last wave
// is as full as the others.  Within a range the grad_out tile (A, up to 128 KB) is loaded once per tile
// segment; B blocks stream through a 3-stage ring; two accumulators alternate so that the store epilogue
// (8 warps) overlaps the next block's MMAs.

struct DcolParams {
  const uint8_t* gy_img;   // [n_tiles][KB][16 KB]
  const uint8_t* wt_img;   // [NB][KB][32 KB]
  float* dcol;             // [clips_in_chunk * V][NT]
  int V, NT, KB, NB;       // KB: K blocks (128-byte rows) contracted by this launch
  int KBT, kb0;            // K blocks per image (image stride) and first block of this launch
  int tiles_per_clip, n_tiles;
  long long n_units;       // n_tiles * NB
  int tmem_cols;
  long long gy_lo_off, wt_lo_off;   // dcol_sm100_split_kernel: byte offsets of the lo images
};

// Store epilogue shared by the gradient-column kernels: warp w serves TMEM lane quarter w % 4 and column half w / 4 of
// the block's accumulator (two accumulators alternate; their full / empty barriers are 8 bytes apart).
__device__ __forceinline__ void dcol_epilogue(const DcolParams& p, int warp, int lane, long long u_beg, long long u_end,
                                              uint32_t tmem_base, uint32_t acc_full0, uint32_t acc_empty0,
                                              volatile int* abort_flag) {
    // ---- epilogue: TMEM -> dcol (a thread owns one voxel row and a 128-column half of the block)
    const int quarter = warp & 3, half = warp >> 2;
    uint32_t q = 0;
    for (long long u = u_beg; u < u_end; ++u, ++q) {
      const int tile = (int)(u / p.NB), nb = (int)(u % p.NB);
      const int bl = tile / p.tiles_per_clip, v0 = (tile % p.tiles_per_clip) * kBM;
      const int v = v0 + quarter * 32 + lane;
      // dcol is slice-major: [clip][slice][voxel][64 channels]; a 256-column block is 4 slices
      const long long S = p.NT / 64;
      float* row = p.dcol + (((long long)bl * S + nb * 4) * p.V + v) * 64;
      const long long slice_stride = (long long)p.V * 64;
      const int acc = q & 1;
      const int ncols = min(kNBlock, p.NT - nb * kNBlock);
      // Lanes 2i / 2i+1 hold rows v, v+1 (256 bytes apart).  They swap every other 16-byte chunk so that
      // each store instruction has the pair write one full 32-byte sector of ONE row (first the even
      // lane's row, then the odd lane's) instead of two half sectors of two rows.
      const bool odd = lane & 1;
      const bool ok_even = (v - (odd ? 1 : 0)) < p.V, ok_odd = (v + (odd ? 0 : 1)) < p.V;
      auto chunk_ptr = [&](int c0) {   // this lane's first 16-byte slot of the even row in the 32-column chunk c0
        return reinterpret_cast<float4*>(row - (odd ? 64 : 0) + (c0 >> 6) * slice_stride + (c0 & 63) + (odd ? 4 : 0));
      };
      const int c_beg = half * 128, c_end = min(ncols, half * 128 + 128);
      if (!ptx::mbar_wait(acc_full0 + 8u * acc, (q >> 1) & 1, abort_flag)) break;
      ptx::tc_fence_after();
      for (int c0 = c_beg; c0 < c_end; c0 += 32) {
        uint32_t r[32];
        ptx::tmem_ld_32x32(tmem_base + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(acc * kNBlock + c0), r);
        ptx::tmem_ld_wait();
        float4* dst = chunk_ptr(c0);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          uint32_t send[4], recv[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) send[e] = odd ? r[8 * i + e] : r[8 * i + 4 + e];
#pragma unroll
          for (int e = 0; e < 4; ++e) recv[e] = __shfl_xor_sync(0xffffffffu, send[e], 1);
          float4 first, second;   // first: even row's chunk (2i + odd); second: odd row's chunk (2i + odd)
          if (odd) {
            first = make_float4(__uint_as_float(recv[0]), __uint_as_float(recv[1]), __uint_as_float(recv[2]),
                                __uint_as_float(recv[3]));
            second = make_float4(__uint_as_float(r[8 * i + 4]), __uint_as_float(r[8 * i + 5]),
                                 __uint_as_float(r[8 * i + 6]), __uint_as_float(r[8 * i + 7]));
          } else {
            first = make_float4(__uint_as_float(r[8 * i]), __uint_as_float(r[8 * i + 1]),
                                __uint_as_float(r[8 * i + 2]), __uint_as_float(r[8 * i + 3]));
            second = make_float4(__uint_as_float(recv[0]), __uint_as_float(recv[1]), __uint_as_float(recv[2]),
                                 __uint_as_float(recv[3]));
          }
          if (ok_even) dst[2 * i] = first;
          if (ok_odd) dst[2 * i + 16] = second;    // next row: + 64 floats
        }
      }
      ptx::tc_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(acc_empty0 + 8u * acc);
    }
}

// kX3 = 1 (fp32-parity mode): a K block is 32 co with rows [hi | lo] in both operands and the issuer forms
// g_hi*w_hi + g_lo*w_hi + g_hi*w_lo from the 16-wide K sub-blocks.  The whole grad_out tile must be resident
// (at most 8 blocks): Cout <= 256 in this mode; longer contractions run dcol_sm100_split_kernel below.
template <int kX3>
__global__ void __launch_bounds__(kDcolThreads, 1)
dcol_sm100_kernel(const DcolParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const int a_bytes = p.KB * kABlockBytes;
  const uint32_t a_base = base, b_base = base + a_bytes, bar_base = b_base + kBStages * kBStageBytes;
  auto b_full = [&](int s) { return bar_base + 8u * s; };
  auto b_empty = [&](int s) { return bar_base + 8u * (kBStages + s); };
  auto acc_full = [&](int a) { return bar_base + 8u * (2 * kBStages + a); };
  auto acc_empty = [&](int a) { return bar_base + 8u * (2 * kBStages + 2 + a); };
  const uint32_t a_full = bar_base + 8u * (2 * kBStages + 4), a_empty = bar_base + 8u * (2 * kBStages + 5);
  const int slot_off = a_bytes + kBStages * kBStageBytes + 8 * (2 * kBStages + 6);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + slot_off);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + slot_off + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long u_beg = p.n_units * blockIdx.x / gridDim.x, u_end = p.n_units * (blockIdx.x + 1) / gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kBStages; ++s) { ptx::mbar_init(b_full(s), 1); ptx::mbar_init(b_empty(s), 1); }
    for (int a = 0; a < 2; ++a) { ptx::mbar_init(acc_full(a), 1); ptx::mbar_init(acc_empty(a), kDcolEpiWarps); }
    ptx::mbar_init(a_full, 1);
    ptx::mbar_init(a_empty, 1);
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

  if (warp < kDcolEpiWarps) {
    dcol_epilogue(p, warp, lane, u_beg, u_end, tmem_base, acc_full(0), acc_empty(0), abort_flag);
  } else if (warp == kDcolMmaWarp) {
    if (lane == 0) {
      uint32_t q = 0, kbc = 0;
      int seg = 0;
      bool ok = true;
      for (long long u = u_beg; ok && u < u_end; ++seg) {
        const int nb_beg = (int)(u % p.NB);
        const int nb_end = (int)min((long long)p.NB, nb_beg + (u_end - u));
        u += nb_end - nb_beg;
        if (!ptx::mbar_wait(a_full, seg & 1, abort_flag)) break;
        ptx::tc_fence_after();
        for (int nb = nb_beg; ok && nb < nb_end; ++nb, ++q) {
          const int acc = q & 1;
          const int ncols = min(kNBlock, p.NT - nb * kNBlock);
          if (!ptx::mbar_wait(acc_empty(acc), ((q >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t idesc = ptx::umma_idesc_bf16_f32(kBM, ncols);
          for (int kb = 0; kb < p.KB; ++kb, ++kbc) {
            const int sb = kbc % kBStages;
            if (!ptx::mbar_wait(b_full(sb), (kbc / kBStages) & 1, abort_flag)) { ok = false; break; }
            ptx::tc_fence_after();
            const uint64_t adesc = ptx::umma_desc_kmajor_sw128(a_base + kb * kABlockBytes);
            const uint64_t bdesc = ptx::umma_desc_kmajor_sw128(b_base + sb * kBStageBytes);
            constexpr int kSteps = kX3 ? 6 : 4;     // K sub-blocks that meet: bf16 (k,k); x3 hi*hi, lo*hi, hi*lo
            constexpr int ka_[6] = {0, 1, 2, 3, 0, 1};
            constexpr int kb_[6] = {0, 1, kX3 ? 0 : 2, kX3 ? 1 : 3, 2, 3};
#pragma unroll
            for (int k = 0; k < kSteps; ++k)
              ptx::umma_bf16(tmem_base + (uint32_t)(acc * kNBlock), adesc + (uint64_t)(2 * ka_[k]),
                             bdesc + (uint64_t)(2 * kb_[k]), idesc, (kb > 0 || k > 0) ? 1u : 0u);
            ptx::umma_commit(b_empty(sb));
          }
          if (ok) ptx::umma_commit(acc_full(acc));
        }
        if (ok) ptx::umma_commit(a_empty);
      }
    }
  } else if (warp == kDcolLoadWarp) {
    if (lane == 0) {
      uint32_t kbc = 0;
      int seg = 0;
      bool ok = true;
      for (long long u = u_beg; ok && u < u_end; ++seg) {
        const int tile = (int)(u / p.NB), nb_beg = (int)(u % p.NB);
        const int nb_end = (int)min((long long)p.NB, nb_beg + (u_end - u));
        u += nb_end - nb_beg;
        if (!ptx::mbar_wait(a_empty, (seg & 1) ^ 1, abort_flag)) break;
        ptx::mbar_arrive_expect_tx(a_full, (uint32_t)a_bytes);
        const uint8_t* asrc = p.gy_img + ((long long)tile * p.KBT + p.kb0) * kABlockBytes;
        for (int off = 0; off < a_bytes; off += 32768)
          ptx::bulk_g2s(a_base + off, asrc + off, (uint32_t)min(32768, a_bytes - off), a_full);
        for (int nb = nb_beg; ok && nb < nb_end; ++nb) {
          const int ncols = min(kNBlock, p.NT - nb * kNBlock);
          for (int kb = 0; kb < p.KB; ++kb, ++kbc) {
            const int sb = kbc % kBStages;
            if (!ptx::mbar_wait(b_empty(sb), ((kbc / kBStages) & 1) ^ 1, abort_flag)) { ok = false; break; }
            ptx::mbar_arrive_expect_tx(b_full(sb), (uint32_t)(ncols * 128));
            ptx::bulk_g2s(b_base + sb * kBStageBytes, p.wt_img + ((long long)nb * p.KBT + p.kb0 + kb) * kBStageBytes,
                          (uint32_t)(ncols * 128), b_full(sb));
          }
        }
      }
      // drain: never exit with a bulk copy in flight
      const uint32_t issued = kbc;
      for (uint32_t qq = (issued > (uint32_t)kBStages ? issued - kBStages : 0); qq < issued; ++qq) {
        const long long t0 = clock64();
        while (!ptx::mbar_try_wait(b_full(qq % kBStages), (qq / kBStages) & 1))
          if (clock64() - t0 > ptx::kWaitBudgetCycles) break;
      }
      if (seg > 0) {
        const long long t0 = clock64();
        while (!ptx::mbar_try_wait(a_full, (seg - 1) & 1))
          if (clock64() - t0 > ptx::kWaitBudgetCycles) break;
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

// Fp32-parity contraction longer than the resident tile (Cout > 256) in ONE launch.  Operands come as separate hi and
// lo images of 64-wide K blocks.  The hi part of the grad_out tile stays resident (Cout/64 blocks of 16 KB); per
// (256-column block, K block) three ring entries arrive in this order
//     W_hi (up to 32 KB)   -> g_hi * w_hi
//     g_lo (16 KB)         -> g_lo * w_hi      (W_hi still in its stage)
//     W_lo (up to 32 KB)   -> g_hi * w_lo
// so every product accumulates into the block's accumulator before the epilogue stores it: the gradient columns are
// written once (two launches into two partial buffers wrote and re-read 1.4 GB more).  The lo part of the tile is
// re-streamed from L2 for every column block (+25 % bytes into shared memory).
__global__ void __launch_bounds__(kDcolThreads, 1)
dcol_sm100_split_kernel(const DcolParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - raw);
  const int a_bytes = p.KB * kABlockBytes;
  const uint32_t a_base = base, b_base = base + a_bytes, bar_base = b_base + kBStages * kBStageBytes;
  auto b_full = [&](int s) { return bar_base + 8u * s; };
  auto b_empty = [&](int s) { return bar_base + 8u * (kBStages + s); };
  auto acc_full = [&](int a) { return bar_base + 8u * (2 * kBStages + a); };
  auto acc_empty = [&](int a) { return bar_base + 8u * (2 * kBStages + 2 + a); };
  const uint32_t a_full = bar_base + 8u * (2 * kBStages + 4), a_empty = bar_base + 8u * (2 * kBStages + 5);
  const int slot_off = a_bytes + kBStages * kBStageBytes + 8 * (2 * kBStages + 6);
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(base_ptr + slot_off);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + slot_off + 4);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long u_beg = p.n_units * blockIdx.x / gridDim.x, u_end = p.n_units * (blockIdx.x + 1) / gridDim.x;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kBStages; ++s) { ptx::mbar_init(b_full(s), 1); ptx::mbar_init(b_empty(s), 1); }
    for (int a = 0; a < 2; ++a) { ptx::mbar_init(acc_full(a), 1); ptx::mbar_init(acc_empty(a), kDcolEpiWarps); }
    ptx::mbar_init(a_full, 1);
    ptx::mbar_init(a_empty, 1);
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

  if (warp < kDcolEpiWarps) {
    dcol_epilogue(p, warp, lane, u_beg, u_end, tmem_base, acc_full(0), acc_empty(0), abort_flag);
  } else if (warp == kDcolMmaWarp) {
    if (lane == 0) {
      uint32_t q = 0, e = 0;            // column blocks and ring entries consumed so far
      int seg = 0;
      bool ok = true;
      auto wait_entry = [&](uint32_t idx) {
        return ptx::mbar_wait(b_full(idx % kBStages), (idx / kBStages) & 1, abort_flag);
      };
      for (long long u = u_beg; ok && u < u_end; ++seg) {
        const int nb_beg = (int)(u % p.NB);
        const int nb_end = (int)min((long long)p.NB, nb_beg + (u_end - u));
        u += nb_end - nb_beg;
        if (!ptx::mbar_wait(a_full, seg & 1, abort_flag)) break;
        ptx::tc_fence_after();
        for (int nb = nb_beg; ok && nb < nb_end; ++nb, ++q) {
          const int acc = q & 1;
          const int ncols = min(kNBlock, p.NT - nb * kNBlock);
          if (!ptx::mbar_wait(acc_empty(acc), ((q >> 1) & 1) ^ 1, abort_flag)) { ok = false; break; }
          ptx::tc_fence_after();
          const uint32_t idesc = ptx::umma_idesc_bf16_f32(kBM, ncols);
          const uint32_t d = tmem_base + (uint32_t)(acc * kNBlock);
          for (int kb = 0; kb < p.KB; ++kb, e += 3) {
            const uint64_t a_hi = ptx::umma_desc_kmajor_sw128(a_base + kb * kABlockBytes);
            const uint32_t s_whi = e % kBStages, s_glo = (e + 1) % kBStages, s_wlo = (e + 2) % kBStages;
            const uint64_t w_hi = ptx::umma_desc_kmajor_sw128(b_base + s_whi * kBStageBytes);
            const uint64_t g_lo = ptx::umma_desc_kmajor_sw128(b_base + s_glo * kBStageBytes);
            const uint64_t w_lo = ptx::umma_desc_kmajor_sw128(b_base + s_wlo * kBStageBytes);
            if (!wait_entry(e)) { ok = false; break; }
            ptx::tc_fence_after();
#pragma unroll
            for (int k = 0; k < 4; ++k)
              ptx::umma_bf16(d, a_hi + (uint64_t)(2 * k), w_hi + (uint64_t)(2 * k), idesc, (kb > 0 || k > 0) ? 1u : 0u);
            if (!wait_entry(e + 1)) { ok = false; break; }
            ptx::tc_fence_after();
#pragma unroll
            for (int k = 0; k < 4; ++k)
              ptx::umma_bf16(d, g_lo + (uint64_t)(2 * k), w_hi + (uint64_t)(2 * k), idesc, 1u);
            ptx::umma_commit(b_empty(s_whi));
            ptx::umma_commit(b_empty(s_glo));
            if (!wait_entry(e + 2)) { ok = false; break; }
            ptx::tc_fence_after();
#pragma unroll
            for (int k = 0; k < 4; ++k)
              ptx::umma_bf16(d, a_hi + (uint64_t)(2 * k), w_lo + (uint64_t)(2 * k), idesc, 1u);
            ptx::umma_commit(b_empty(s_wlo));
          }
          if (ok) ptx::umma_commit(acc_full(acc));
        }
        if (ok) ptx::umma_commit(a_empty);
      }
    }
  } else if (warp == kDcolLoadWarp) {
    if (lane == 0) {
      uint32_t e = 0;
      int seg = 0;
      bool ok = true;
      auto push = [&](const uint8_t* src, uint32_t bytes) {
        const int sb = e % kBStages;
        if (!ptx::mbar_wait(b_empty(sb), ((e / kBStages) & 1) ^ 1, abort_flag)) return false;
        ptx::mbar_arrive_expect_tx(b_full(sb), bytes);
        ptx::bulk_g2s(b_base + sb * kBStageBytes, src, bytes, b_full(sb));
        ++e;
        return true;
      };
      for (long long u = u_beg; ok && u < u_end; ++seg) {
        const int tile = (int)(u / p.NB), nb_beg = (int)(u % p.NB);
        const int nb_end = (int)min((long long)p.NB, nb_beg + (u_end - u));
        u += nb_end - nb_beg;
        if (!ptx::mbar_wait(a_empty, (seg & 1) ^ 1, abort_flag)) break;
        ptx::mbar_arrive_expect_tx(a_full, (uint32_t)a_bytes);
        const uint8_t* asrc = p.gy_img + (long long)tile * p.KBT * kABlockBytes;
        for (int off = 0; off < a_bytes; off += 32768)
          ptx::bulk_g2s(a_base + off, asrc + off, (uint32_t)min(32768, a_bytes - off), a_full);
        for (int nb = nb_beg; ok && nb < nb_end; ++nb) {
          const uint32_t wbytes = (uint32_t)(min(kNBlock, p.NT - nb * kNBlock) * 128);
          for (int kb = 0; ok && kb < p.KB; ++kb) {
            const uint8_t* w_hi = p.wt_img + ((long long)nb * p.KBT + kb) * kBStageBytes;
            ok = push(w_hi, wbytes) && push(asrc + p.gy_lo_off + (long long)kb * kABlockBytes, (uint32_t)kABlockBytes) &&
                 push(w_hi + p.wt_lo_off, wbytes);
          }
        }
      }
      // drain: never exit with a bulk copy in flight
      const uint32_t issued = e;
      for (uint32_t qq = (issued > (uint32_t)kBStages ? issued - kBStages : 0); qq < issued; ++qq) {
        const long long t0 = clock64();
        while (!ptx::mbar_try_wait(b_full(qq % kBStages), (qq / kBStages) & 1))
          if (clock64() - t0 > ptx::kWaitBudgetCycles) break;
      }
      if (seg > 0) {
        const long long t0 = clock64();
        while (!ptx::mbar_try_wait(a_full, (seg - 1) & 1))
          if (clock64() - t0 > ptx::kWaitBudgetCycles) break;
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

// ---- (b) sampling gradient + scatter ---------------------------------------------------------------

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  // volatile (must not be dropped) but no memory clobber: read-only loads may move across it
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d));
}

// Block = 32 voxels of one (clip, offset group) -- blockIdx.y -- times 8 threads per voxel; thread j owns
// channels [8j, 8j+8) of each 64-channel slice.  The block walks the K taps; the record and the gradient
// columns of tap t+1 are requested before tap t is processed, so the HBM stream of dcol (slice-major:
// 8 KB contiguous per block and slice) stays in flight behind the L2 gathers and reductions.
// kF32X: the channels-last staging of x is fp32 (fp32-parity mode) instead of fp16.
// kNarrow: 32 channels per offset group.  The gradient columns keep their 64-channel
// slices, each now holding two neighbouring groups; a block still serves one (clip, group) and its threads
// own channels [4j, 4j+4) of the group's half of the slice.
template <bool FieldOut, bool kF32X, bool kNarrow = false>
__global__ void __launch_bounds__(256, kF32X ? 2 : 3)
sample_grad_taps_kernel(Geom g, ClStrides cs, int b0, int nh, const float4* __restrict__ recs,
                        const float* __restrict__ dcol, const void* __restrict__ x_cl_v, bool has_mask,
                        float* __restrict__ grad_coord, float* __restrict__ grad_mask, float* __restrict__ gx_cl,
                        int field_nch, int3 field_ch, const float* __restrict__ field_axes, HeadCfg head) {
  const int j = threadIdx.x & 7;
  const int v = blockIdx.x * 32 + (threadIdx.x >> 3);
  const int grp = blockIdx.y % g.G, bl = blockIdx.y / g.G;
  const int b = b0 + bl;
  const bool active = v < g.V;
  const int vc = active ? v : g.V - 1;                       // clamped: inactive threads load valid memory
  const long long S = kNarrow ? (long long)(g.G / 2) * g.K : (long long)g.G * g.K * nh;
  const float4* recp = recs + (((long long)b * g.G + grp) * g.K) * g.V + vc;
  // thread j owns channels [4j, 4j+4) and [32+4j, 32+4j+4) of a slice: one warp-wide 16-byte access then
  // covers whole 32-byte sectors (two lanes each), which halves the sector operations of the reductions
  const float* dp = kNarrow
      ? dcol + (((long long)bl * S + (long long)(grp >> 1) * g.K) * g.V + vc) * 64 + (grp & 1) * 32 + j * 4
      : dcol + (((long long)bl * S + (long long)grp * g.K * nh) * g.V + vc) * 64 + j * 4;
  const long long slice_stride = (long long)g.V * 64;
  using XT = typename std::conditional<kF32X, float, __half>::type;
  const XT* xb = reinterpret_cast<const XT*>(x_cl_v) + (long long)b * g.Vin * g.Cin;
  float* gxb = gx_cl + (long long)b * g.Vin * g.Cin;
  const int chbase = grp * g.cpg + j * 4;

  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  float fsum[3] = {0.f, 0.f, 0.f};
  auto ld_cols = [&](const float* q, float4& a, float4& b) {
    a = __ldg(reinterpret_cast<const float4*>(q));
    b = kNarrow ? zero4 : __ldg(reinterpret_cast<const float4*>(q + 32));
  };
  float4 rec_n = __ldg(recp);
  float4 d0_n, d1_n;
  ld_cols(dp, d0_n, d1_n);
  for (int tap = 0; tap < g.K; ++tap) {
    const float4 rec = rec_n;
    float4 d0 = d0_n, d1 = d1_n;
    if (tap + 1 < g.K) {
      rec_n = __ldg(recp + (long long)(tap + 1) * g.V);
      ld_cols(dp + (long long)(tap + 1) * nh * slice_stride, d0_n, d1_n);
    }
    const float m = rec.w;
    const Sample<float> s = make_sample(g, rec.x, rec.y, rec.z);
    // scatter weights of the reference's col2im: (1-|z-zp|)(1-|y-yp|)(1-|x-xp|), corners at distance
    // exactly 1 excluded (dconv3d_gpu.cu:626-637)
    const float wz[2] = {sub_rn(1.f, s.fz), sub_rn(1.f, s.gz)};
    const float wy[2] = {sub_rn(1.f, s.fy), sub_rn(1.f, s.gy)};
    const float wx[2] = {sub_rn(1.f, s.fx), sub_rn(1.f, s.gx)};
    const bool okz[2] = {true, s.gz < 1.f}, oky[2] = {true, s.gy < 1.f}, okx[2] = {true, s.gx < 1.f};
    const unsigned valid = active ? s.valid : 0u;
    const int off0 = ((s.z0 * g.H + s.y0) * g.W + s.x0) * g.Cin + chbase;
    float G[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) G[q] = 0.f;
    for (int h = 0; h < nh; ++h) {
      if (h > 0) {
        ld_cols(dp + ((long long)tap * nh + h) * slice_stride, d0, d1);
      }
      // corner values of this thread's 8 channels ([4j, 4j+4) and [32+4j, 32+4j+4)), as loaded.  fp16 staging:
      // the loads are unconditional -- a corner outside the volume reads the clip's first voxel instead and its
      // dot product is discarded by a select after the slice loop (a select, so a non-finite stand-in cannot
      // leak); measured 0.13 ms per step faster than predicated loads.  fp32 staging: predicated loads (twice
      // the bytes per corner; fetching the stand-ins measured 0.08 ms slower).
      uint4 c[8], chi[kF32X ? 8 : 1];
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const int off_in = off0 + h * 64 + (q >> 2) * cs.dz + ((q >> 1) & 1) * cs.dy + (q & 1) * cs.dx;
        if constexpr (kF32X) {
          if ((valid >> q) & 1u) {
            c[q] = ptx::ldg_nc_v4(xb + off_in);
            chi[q] = kNarrow ? make_uint4(0u, 0u, 0u, 0u) : ptx::ldg_nc_v4(xb + off_in + 32);
          } else {
            c[q] = chi[q] = make_uint4(0u, 0u, 0u, 0u);
          }
        } else {
          const int off = ((valid >> q) & 1u) ? off_in : chbase + h * 64;
          const uint2 lo = ptx::ldg_nc_v2(xb + off);
          const uint2 hi = kNarrow ? make_uint2(0u, 0u) : ptx::ldg_nc_v2(xb + off + 32);
          c[q] = make_uint4(lo.x, lo.y, hi.x, hi.y);
        }
      }
#pragma unroll
      for (int q = 0; q < 8; ++q) {
        const int dz = q >> 2, dy = (q >> 1) & 1, dx = q & 1;
        if constexpr (kF32X) {
          if constexpr (kNarrow)
            G[q] += d0.x * __uint_as_float(c[q].x) + d0.y * __uint_as_float(c[q].y) +
                    d0.z * __uint_as_float(c[q].z) + d0.w * __uint_as_float(c[q].w);
          else
            G[q] += d0.x * __uint_as_float(c[q].x) + d0.y * __uint_as_float(c[q].y) +
                    d0.z * __uint_as_float(c[q].z) + d0.w * __uint_as_float(c[q].w) +
                    d1.x * __uint_as_float(chi[q].x) + d1.y * __uint_as_float(chi[q].y) +
                    d1.z * __uint_as_float(chi[q].z) + d1.w * __uint_as_float(chi[q].w);
        } else {
          const float2 x0 = __half22float2(bits_h2(c[q].x)), x1 = __half22float2(bits_h2(c[q].y));
          const float2 x2 = __half22float2(bits_h2(c[q].z)), x3 = __half22float2(bits_h2(c[q].w));
          if constexpr (kNarrow)
            G[q] += d0.x * x0.x + d0.y * x0.y + d0.z * x1.x + d0.w * x1.y;
          else
            G[q] += d0.x * x0.x + d0.y * x0.y + d0.z * x1.x + d0.w * x1.y + d1.x * x2.x + d1.y * x2.y +
                    d1.z * x3.x + d1.w * x3.y;
        }
        if (((valid >> q) & 1u) && okz[dz] && oky[dy] && okx[dx]) {
          const float sw = mul_rn(mul_rn(wz[dz], wy[dy]), wx[dx]) * m;
          float* dst = gxb + (off0 + h * 64 + dz * cs.dz + dy * cs.dy + dx * cs.dx);
          red_add_v4(dst, sw * d0.x, sw * d0.y, sw * d0.z, sw * d0.w);
          if (!kNarrow) red_add_v4(dst + 32, sw * d1.x, sw * d1.y, sw * d1.z, sw * d1.w);
        }
      }
    }
    // channel reduction of the 8 corner dot-products across the voxel's 8 threads (corners outside: zero)
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      if (!kF32X) G[q] = ((valid >> q) & 1u) ? G[q] : 0.f;
      G[q] += __shfl_xor_sync(0xffffffffu, G[q], 1);
      G[q] += __shfl_xor_sync(0xffffffffu, G[q], 2);
      G[q] += __shfl_xor_sync(0xffffffffu, G[q], 4);
    }
    if (active && j == 0) {
      float wts[3];
      coord_weights(G, s, wts);    // linear in the corner values: applies to the channel-summed corners
      // head.*_bstride != 0: the gradients go into the gradient of the predictor's raw output (clip stride = all of
      // its channels), the mask's through the derivative of its activation (taken from the activated value m)
      if (has_mask && grad_mask) {
        float a[8];
        sample_weights(s, a);
        const long long ri = head.mask_bstride ? (long long)b * head.mask_bstride + ((long long)grp * g.K + tap) * g.V + v
                                               : (((long long)b * g.G + grp) * g.K + tap) * g.V + v;
        grad_mask[ri] = s.inside ? blend(G, a) * mask_act_slope(head.mask_act, m) : 0.f;
      }
      if constexpr (!FieldOut) {
        float* go = grad_coord + (head.geo_bstride ? (long long)b * head.geo_bstride + ((long long)grp * 3 * g.K + 3 * tap) * g.V + v
                                                   : (((long long)b * g.G + grp) * 3 * g.K + 3 * tap) * g.V + v);
        go[0] = m * wts[0];
        go[g.V] = m * wts[1];
        go[2 * (long long)g.V] = m * wts[2];
      } else {
        // the field's gradient sums over taps (and groups): taps are summed here, one atomic per group after
        const int k = tap % g.kw, jj = (tap / g.kw) % g.kh, i = tap / (g.kw * g.kh);
        fsum[0] += field_axes[i] * (m * wts[0]);
        fsum[1] += field_axes[kMaxFieldKernelDim + jj] * (m * wts[1]);
        fsum[2] += field_axes[2 * kMaxFieldKernelDim + k] * (m * wts[2]);
      }
    }
  }
  if constexpr (FieldOut) {
    if (active && j == 0) {
      float* gs = grad_coord + (long long)b * (head.geo_bstride ? head.geo_bstride : (long long)field_nch * g.V) + v;
      if (field_ch.x >= 0) atomicAdd(gs + (long long)field_ch.x * g.V, fsum[0]);
      if (field_ch.y >= 0) atomicAdd(gs + (long long)field_ch.y * g.V, fsum[1]);
      if (field_ch.z >= 0) atomicAdd(gs + (long long)field_ch.z * g.V, fsum[2]);
    }
  }
}

// ---- (c) channels-last fp32 -> NCDHW ----------------------------------------------------------------
__global__ void __launch_bounds__(256)
unstage_grad_input_kernel(int C, long long Vin, const float* __restrict__ gx_cl, float* __restrict__ gx) {
  __shared__ float tile[32][33];
  const int b = blockIdx.z, c0 = blockIdx.y * 32;
  const long long v0 = (long long)blockIdx.x * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int vv = ty; vv < 32; vv += 8) {
    const long long v = v0 + vv;
    tile[vv][tx] = (v < Vin && c0 + tx < C) ? __ldg(gx_cl + ((long long)b * Vin + v) * C + c0 + tx) : 0.f;
  }
  __syncthreads();
  for (int cc = ty; cc < 32; cc += 8) {
    const long long v = v0 + tx;
    if (v < Vin && c0 + cc < C) gx[((long long)b * C + c0 + cc) * Vin + v] = tile[tx][cc];
  }
}

// grad[b, c, v] *= d size_act / d raw (raw[b, c, v]) for the field's channels (both tensors with clip stride bstride)
__global__ void __launch_bounds__(256)
field_act_grad_kernel(const float* __restrict__ raw, float* __restrict__ grad, long long bstride, int nch, int V, int B, int act) {
  const long long i = (long long)blockIdx.x * 256 + threadIdx.x;
  if (i >= (long long)B * nch * V) return;
  const long long b = i / ((long long)nch * V), r = i % ((long long)nch * V);
  grad[b * bstride + r] *= size_act_slope(act, __ldg(raw + b * bstride + r));
}

template <typename Coords>
int field_nch_of(const Coords&) { return 0; }
template <>
int field_nch_of<FieldCoords<float>>(const FieldCoords<float>& c) { return c.nch; }

struct BwdPlan {
  int nh, S, NT, KB, KBT, NB, tiles_per_clip, tmem_cols, smem_bytes, clips_per_chunk;
  bool pairg;       // 32 channels per offset group: a 64-channel slice holds two neighbouring groups
  bool split;       // fp32-parity mode with Cout > 256: separate hi / lo operand images, dcol_sm100_split_kernel
  long long gy_lo_off, wt_lo_off;
  size_t x_cl_bytes, rec_bytes, gat_bytes, gy_img_bytes, wt_img_bytes, dcol_bytes, gx_cl_bytes, axes_bytes;
};

bool make_bwd_plan(const Geom& g, unsigned long long cap, bool x3, BwdPlan* pl) {
  // 32 channels per group (an even number of groups): groups are contiguous channel ranges, so slices of 64
  // channels simply span two of them
  pl->pairg = g.cpg == 32 && g.G % 2 == 0;
  if (g.groups != 1 || (g.cpg % 64 != 0 && !pl->pairg) || g.Cout % 64 != 0 || g.Cout > 512) return false;
  if (g.Vin * g.Cin > 0x7fffffffLL) return false;
  if ((long long)g.G * g.K * g.B > 65535) return false;
  if (g.K * 64 * (int)sizeof(float) > 48 * 1024 || g.Cin > 65535) return false;   // weight staging kernel
  pl->nh = pl->pairg ? 1 : g.cpg / 64;
  pl->S = pl->pairg ? (g.G / 2) * g.K : g.G * g.K * pl->nh;
  pl->NT = pl->S * 64;
  pl->split = x3 && g.Cout > 256;
  pl->KBT = g.Cout / ((x3 && !pl->split) ? 32 : 64);     // K blocks per image
  pl->KB = pl->KBT;                                      // all resident (<= 8 blocks of 16 KB)
  pl->NB = (pl->NT + kNBlock - 1) / kNBlock;
  pl->tiles_per_clip = (g.V + kBM - 1) / kBM;
  pl->tmem_cols = 512;
  pl->smem_bytes = pl->KB * kABlockBytes + kBStages * kBStageBytes + 256 + 1024;
  if (pl->smem_bytes > kSmemLimit) return false;
  pl->clips_per_chunk = bwd_slice_clips(g, cap);
  pl->x_cl_bytes = align_up((size_t)g.B * g.Vin * g.Cin * (x3 ? 4 : 2), 256);
  pl->rec_bytes = pos_records_bytes(g);
  pl->gat_bytes = gather_records_bytes(g);
  pl->gy_lo_off = (long long)pl->clips_per_chunk * pl->tiles_per_clip * pl->KBT * kABlockBytes;
  pl->wt_lo_off = (long long)pl->NB * pl->KBT * kBStageBytes;
  pl->gy_img_bytes = align_up((size_t)pl->gy_lo_off * (pl->split ? 2 : 1), 256);
  pl->wt_img_bytes = align_up((size_t)pl->wt_lo_off * (pl->split ? 2 : 1), 256);
  pl->dcol_bytes = align_up((size_t)pl->clips_per_chunk * g.V * pl->NT * 4, 256);
  pl->gx_cl_bytes = align_up((size_t)g.B * g.Vin * g.Cin * 4, 256);
  pl->axes_bytes = 256;
  return true;
}

template <typename Coords, bool FieldOut>
int run_bwd(const Geom& g, bool x3, const Coords& coords, unsigned long long cap, const float* gy, const float* x,
            const float* mask, const float* w, float* grad_x, float* grad_coord, size_t grad_coord_elems,
            float* grad_mask, float* grad_w, float* grad_bias, void* ws, cudaStream_t st, cudaEvent_t params_ready,
            const HeadCfg& head, const float* raw_field) {
  BwdPlan pl;
  if (!make_bwd_plan(g, cap, x3, &pl)) return D2C_ERR_MODE;
  uint8_t* wsp = reinterpret_cast<uint8_t*>(ws);
  void* x_cl = wsp; wsp += pl.x_cl_bytes;
  float4* recs = reinterpret_cast<float4*>(wsp); wsp += pl.rec_bytes;
  uint4* gat = reinterpret_cast<uint4*>(wsp); wsp += pl.gat_bytes;
  uint8_t* gy_img = wsp; wsp += pl.gy_img_bytes;
  uint8_t* wt_img = wsp; wsp += pl.wt_img_bytes;
  float* dcol = reinterpret_cast<float*>(wsp); wsp += pl.dcol_bytes;
  float* gx_cl = reinterpret_cast<float*>(wsp); wsp += pl.gx_cl_bytes;
  float* axes_dev = reinterpret_cast<float*>(wsp); wsp += pl.axes_bytes;
  void* dw_ws = wsp;

  int sm_count = 0, rc;
  if ((rc = device_sm_count(&sm_count))) return rc;
  ptx::bind_status_sink();
  ClStrides cs;
  cs.dz = g.H * g.W * g.Cin; cs.dy = g.W * g.Cin; cs.dx = g.Cin;
  const void* sav = nullptr;

  // dilation-field variant: tap positions per dim, read by the kernel that accumulates grad_size_map
  int field_nch = 0;
  int3 field_ch = make_int3(-1, -1, -1);
  if constexpr (FieldOut) {
    field_nch = coords.nch;
    field_ch = make_int3(coords.ch[0], coords.ch[1], coords.ch[2]);
    D2C_CUDA_TRY(cudaMemcpyAsync(axes_dev, &coords.axis[0][0], sizeof(float) * 3 * kMaxFieldKernelDim,
                                 cudaMemcpyHostToDevice, st));
  }

  prof_mark(st, "bwd_stage_operands");
  D2C_CUDA_TRY(cudaMemsetAsync(gx_cl, 0, (size_t)g.B * g.Vin * g.Cin * 4, st));
  if (FieldOut) {
    if (head.geo_bstride)      // the field's gradient channels inside the raw gradient: nch planes per clip
      D2C_CUDA_TRY(cudaMemset2DAsync(grad_coord, sizeof(float) * head.geo_bstride, 0, sizeof(float) * field_nch_of(coords) * g.V,
                                     g.B, st));
    else
      D2C_CUDA_TRY(cudaMemsetAsync(grad_coord, 0, sizeof(float) * grad_coord_elems, st));
  }
  if (grad_bias) D2C_CUDA_TRY(cudaMemsetAsync(grad_bias, 0, sizeof(float) * g.Cout, st));
  // What the forward of this call kept in this mode's format: its operand tiles (the weight gradient streams them, no
  // gather records needed), the staged input and the position records -- nothing is staged a second time.
  if (SampleCache* sc = current_sample_cache()) {
    int np = 0;
    SampleCacheLayout lay{};
    if (sc->data && sc->format == (x3 ? 2 : 1) && sm100_sample_cache_layout(g, x3, &np, &lay) && sc->bytes >= lay.total()) {
      sav = sc->data;
      x_cl = reinterpret_cast<uint8_t*>(sc->data) + lay.image_bytes;
      recs = reinterpret_cast<float4*>(reinterpret_cast<uint8_t*>(sc->data) + lay.image_bytes + lay.x_cl_bytes);
    }
  }
  if (!sav) {
    dim3 grid((unsigned)((g.Vin + 31) / 32), (unsigned)((g.Cin + 63) / 64), (unsigned)g.B);
    if (x3)
      stage_input_cl_f32_kernel<<<grid, 256, 0, st>>>(g.Cin, g.Vin, x, reinterpret_cast<float*>(x_cl));
    else
      stage_input_cl_f16_kernel<<<grid, 256, 0, st>>>(g.Cin, g.Vin, x, reinterpret_cast<__half*>(x_cl));
    D2C_LAUNCH_CHECK();
    if (!sav && (rc = launch_sample_records(g, coords, mask, head, recs, gat, st, x3))) return rc;
  }
  // The parameter gradients come first: the weight gradient (tensor-core implicit GEMM over the re-sampled tile)
  // needs only the records and the staged input, and its grad_out staging pass also sums grad_bias.  A caller that
  // reduces them across GPUs can start as soon as `params_ready` fires, under the data-side kernels below.
  if ((rc = sm100_dw(g, x3, gy, x_cl, gat, grad_w, grad_bias, dw_ws, st, sav))) return rc;
  if (params_ready) D2C_CUDA_TRY(cudaEventRecord(params_ready, st));
  prof_mark(st, "bwd_stage_weights");
  const int img_mode = pl.split ? 2 : (x3 ? 1 : 0);
  stage_wt_img_kernel<<<dim3((unsigned)pl.KBT, (unsigned)g.Cin), 64, 64 * g.K * sizeof(float), st>>>(
      g.Cout, g.Cin, g.K, pl.pairg ? 64 : g.cpg, pl.nh, img_mode, w, wt_img, pl.wt_lo_off);
  D2C_LAUNCH_CHECK();
  D2C_CUDA_TRY(cudaFuncSetAttribute(dcol_sm100_kernel<0>, cudaFuncAttributeMaxDynamicSharedMemorySize, pl.smem_bytes));
  D2C_CUDA_TRY(cudaFuncSetAttribute(dcol_sm100_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, pl.smem_bytes));
  D2C_CUDA_TRY(cudaFuncSetAttribute(dcol_sm100_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, pl.smem_bytes));

  for (int b0 = 0; b0 < g.B; b0 += pl.clips_per_chunk) {
    const int nbc = (g.B - b0 < pl.clips_per_chunk) ? g.B - b0 : pl.clips_per_chunk;
    const int n_tiles = nbc * pl.tiles_per_clip;
    prof_mark(st, "bwd_stage_grad_out");
    stage_gy_img_kernel<<<dim3((unsigned)n_tiles, (unsigned)pl.KBT), 256, 0, st>>>(g.Cout, g.V, pl.tiles_per_clip, b0,
                                                                                  img_mode, gy, gy_img, pl.gy_lo_off);
    D2C_LAUNCH_CHECK();
    DcolParams p;
    p.gy_img = gy_img; p.wt_img = wt_img; p.dcol = dcol;
    p.V = g.V; p.NT = pl.NT; p.KB = pl.KB; p.NB = pl.NB;
    p.tiles_per_clip = pl.tiles_per_clip; p.n_tiles = n_tiles; p.n_units = (long long)n_tiles * pl.NB;
    p.tmem_cols = pl.tmem_cols;
    long long grid = p.n_units / 4;
    if (grid > sm_count) grid = sm_count;
    if (grid < 1) grid = 1;
    prof_mark(st, "bwd_dcol_sm100");
    p.KBT = pl.KBT; p.kb0 = 0; p.KB = pl.KB;
    p.gy_lo_off = pl.gy_lo_off; p.wt_lo_off = pl.wt_lo_off;
    if (pl.split)
      dcol_sm100_split_kernel<<<(unsigned)grid, kDcolThreads, pl.smem_bytes, st>>>(p);
    else if (x3)
      dcol_sm100_kernel<1><<<(unsigned)grid, kDcolThreads, pl.smem_bytes, st>>>(p);
    else
      dcol_sm100_kernel<0><<<(unsigned)grid, kDcolThreads, pl.smem_bytes, st>>>(p);
    D2C_LAUNCH_CHECK();
    prof_mark(st, "bwd_sample_grad");
    dim3 sgrid((unsigned)((g.V + 31) / 32), (unsigned)(nbc * g.G));
    if (pl.pairg && x3)
      sample_grad_taps_kernel<FieldOut, true, true><<<sgrid, 256, 0, st>>>(g, cs, b0, pl.nh, recs, dcol, x_cl,
                                                                           mask != nullptr, grad_coord, grad_mask,
                                                                           gx_cl, field_nch, field_ch, axes_dev, head);
    else if (pl.pairg)
      sample_grad_taps_kernel<FieldOut, false, true><<<sgrid, 256, 0, st>>>(g, cs, b0, pl.nh, recs, dcol, x_cl,
                                                                            mask != nullptr, grad_coord, grad_mask,
                                                                            gx_cl, field_nch, field_ch, axes_dev, head);
    else if (x3)
      sample_grad_taps_kernel<FieldOut, true><<<sgrid, 256, 0, st>>>(g, cs, b0, pl.nh, recs, dcol, x_cl,
                                                                     mask != nullptr, grad_coord, grad_mask, gx_cl,
                                                                     field_nch, field_ch, axes_dev, head);
    else
      sample_grad_taps_kernel<FieldOut, false><<<sgrid, 256, 0, st>>>(g, cs, b0, pl.nh, recs, dcol, x_cl,
                                                                      mask != nullptr, grad_coord, grad_mask, gx_cl,
                                                                      field_nch, field_ch, axes_dev, head);
    D2C_LAUNCH_CHECK();
  }
  if constexpr (FieldOut) {
    if (head.size_act != 0 && raw_field) {      // chain rule through the size activation, on the summed gradient
      const long long n = (long long)g.B * field_nch * g.V;
      field_act_grad_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(
          raw_field, grad_coord, head.geo_bstride ? head.geo_bstride : (long long)field_nch * g.V, field_nch, g.V, g.B,
          head.size_act);
      D2C_LAUNCH_CHECK();
    }
  }
  prof_mark(st, "bwd_unstage_grad_input");
  {
    dim3 grid((unsigned)((g.Vin + 31) / 32), (unsigned)((g.Cin + 31) / 32), (unsigned)g.B);
    unstage_grad_input_kernel<<<grid, 256, 0, st>>>(g.Cin, g.Vin, gx_cl, grad_x);
    D2C_LAUNCH_CHECK();
  }
  prof_mark(st, nullptr);
  return D2C_OK;
}

}  // namespace

// bf16 mode runs the single-pass kernels where their plans fit (32 channels per group: the weight gradient needs
// room for a second record set, i.e. Cout <= 256) and the fp32-parity kernels otherwise.
static bool bwd_use_x3(const Geom& g, int math_mode, unsigned long long cap) {
  if (math_mode != D2C_MATH_BF16) return true;
  BwdPlan pl;
  return !(make_bwd_plan(g, cap, false, &pl) && sm100_dw_workspace(g, false) > 0);
}

bool sm100_bwd_variant(const Geom& g, int math_mode, unsigned long long cap, bool* x3) {
  *x3 = bwd_use_x3(g, math_mode, cap);
  BwdPlan pl;
  return make_bwd_plan(g, cap, *x3, &pl) && sm100_dw_workspace(g, *x3) > 0;
}

bool sm100_bwd_supported(const Geom& g, int dtype, int math_mode, unsigned long long cap) {
  if (dtype != D2C_F32 || math_mode == D2C_MATH_FP32) return false;
  const bool x3 = bwd_use_x3(g, math_mode, cap);
  BwdPlan pl;
  return make_bwd_plan(g, cap, x3, &pl) && sm100_dw_workspace(g, x3) > 0;
}

size_t sm100_bwd_workspace(const Geom& g, int dtype, int math_mode, unsigned long long cap) {
  if (!sm100_bwd_supported(g, dtype, math_mode, cap)) return 0;
  const bool x3 = bwd_use_x3(g, math_mode, cap);
  BwdPlan pl;
  make_bwd_plan(g, cap, x3, &pl);
  return pl.x_cl_bytes + pl.rec_bytes + pl.gat_bytes + pl.gy_img_bytes + pl.wt_img_bytes + pl.dcol_bytes + pl.gx_cl_bytes +
         pl.axes_bytes + sm100_dw_workspace(g, x3);
}

int sm100_bwd_offsets(const Geom& g, int math_mode, unsigned long long cap, const float* gy, const float* x, const float* offset,
                      const float* mask, const float* w, float* grad_x, float* grad_offset, float* grad_mask,
                      float* grad_w, float* grad_bias, void* ws, cudaStream_t st, cudaEvent_t params_ready,
                      const HeadCfg& head) {
  OffsetCoords<float> oc{offset, head.geo_bstride};
  return run_bwd<OffsetCoords<float>, false>(g, bwd_use_x3(g, math_mode, cap), oc, cap, gy, x, mask, w, grad_x, grad_offset, 0, grad_mask, grad_w,
                                             grad_bias, ws, st, params_ready, head, nullptr);
}

int sm100_bwd_field(const Geom& g, int math_mode, unsigned long long cap, const FieldCoords<float>& fc, const float* gy,
                    const float* x, const float* mask, const float* w, float* grad_x, float* grad_size_map,
                    size_t grad_size_elems, float* grad_mask, float* grad_w, float* grad_bias, void* ws,
                    cudaStream_t st, cudaEvent_t params_ready, const HeadCfg& head) {
  return run_bwd<FieldCoords<float>, true>(g, bwd_use_x3(g, math_mode, cap), fc, cap, gy, x, mask, w, grad_x, grad_size_map, grad_size_elems,
                                           grad_mask, grad_w, grad_bias, ws, st, params_ready, head, fc.size_map);
}

}  // namespace d2c
