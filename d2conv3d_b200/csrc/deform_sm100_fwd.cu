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
// Work decomposition: the (tile, slice) units of every clip are cut into one contiguous range per CTA
// (stream-K inside the clip), so 102 tiles per clip do not run as ragged waves on 148 SMs and all CTAs
// gather from the same clip at the same time (one clip's staged input fits in L2, the batch does not).
// A CTA whose range covers a whole tile stores it; partial tiles are combined with fp32 reductions into
// the zero-initialised output.  Where a CTA has eight or more tiles (large volumes), whole tiles are
// dealt round-robin instead: the CTAs then work on consecutive tiles, whose sampling neighbourhoods
// overlap.
//
// Per CTA, 24 warps in warpgroup-aligned roles (deform_sm100_fwd_kernel.cuh):
//   warps 0-3   epilogue: tcgen05.ld the 128 x N accumulator, add bias, store / reduce NCDHW
//   warp  4     one thread issues tcgen05.mma and the commits that free the stages
//   warp  5     one thread streams pre-swizzled weight slices with cp.async.bulk
//   warp  6     one thread bulk-copies each unit's gather records into the record ring and writes the unit
//               header (staging offset of the slice, valid rows), so the producers do no index arithmetic
//   warp  7     idle (completes the warpgroup)
//   warps 8-23  gather producers: unit header + gather record from the shared-memory record ring, 8
//               unconditional corner loads (16 B) per row, the next row's loads issued before the current row is
//               blended (setmaxnreg moves registers from warps 0-7 to these), blend with pre-modulated weights,
//               bf16 pack, swizzled st.shared of the A tile
// Stage hand-off is by mbarriers; every wait in the kernel's own code is bounded (sm100_ptx.cuh).
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
  int n_parts, part_shift;     // see cta_part_range
  int rr;                      // 1: parts are whole tiles dealt round-robin (part r = tile r * gridDim.x + blockIdx.x)
  long long units_per_part;
  int seg_cap;                 // at most this many units accumulate in tensor memory before the partial result is
                               // added to y (see run_fwd); S = no limit
  int b_stages, b_stage_bytes;
  int tmem_cols;
  // Samples kept for the weight gradient (nullable): the blended A tiles, written to global as they are produced,
  // in blocks of 8 KB = one 64-channel slice x 64 voxels (rows of 128 B, 16-byte chunks XOR-swizzled by row & 7):
  //   bf16 mode:  [tile][64-voxel block][slice s, padded to 2*sav_np]
  //   bf16x3:     [tile][64-voxel block][slice pair][hi | lo][slice of the pair]   (a unit fills half of each row)
  // exactly the operand images deform_sm100_dw.cu bulk-copies.
#ifdef D2C_UNIT_TRACE
  long long* trace;            // instrumentation buffer (deform_sm100_fwd_kernel.cuh), nullptr = off
  int trace_cta, trace_k0;
#endif
  uint8_t* sav;
  int sav_np;                  // slice pairs of the weight gradient
  int sav_pairg;               // bf16x3: 32 channels per offset group (a 64-channel slice spans two groups)
};

__device__ __forceinline__ void cta_unit_range(long long n_units, long long& beg, long long& end) {
  beg = n_units * blockIdx.x / gridDim.x;
  end = n_units * (blockIdx.x + 1) / gridDim.x;
}

// Part r of a CTA's work: the units of part r (a clip, FwdParams::units_per_part each) are cut into one contiguous
// range per CTA, and the CTA takes the range (blockIdx.x + r * part_shift) mod gridDim.x.  All CTAs therefore work
// inside the SAME clip at the same time -- the staged input they gather from is one clip, not the whole batch, which
// is what L2 can hold -- and a CTA's ranges lie at different depths of successive clips, which evens out the cost
// of ranges in the middle of the volume (more in-volume corners, more distinct lines) against those at its faces.
__device__ __forceinline__ void cta_part_range(const FwdParams& p, int part, long long& beg, long long& end) {
  const long long q = ((long long)blockIdx.x + (long long)part * p.part_shift) % gridDim.x;
  const long long base = (long long)part * p.units_per_part;
  beg = base + p.units_per_part * q / gridDim.x;
  end = base + p.units_per_part * (q + 1) / gridDim.x;
}

#include "deform_sm100_fwd_kernel.cuh"
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
  if ((long long)pl->n_tiles * pl->S > 0x7fffffffLL) return false;   // the kernel counts units in 31 bits
  pl->b_stage_bytes = g.Cout * 128;
  // 256 bytes of barriers + 272 bytes of part ranges (rounded to 512) + 1 KB of alignment slack
  int nb = (kSmemLimit - 1024 - 768 - kAStages * kAStageBytes - kRStages * pl->r_stage_bytes) / pl->b_stage_bytes;
  if (nb > 4) nb = 4;
  if (nb < 2) return false;
  pl->b_stages = nb;
  int cols = 32;
  while (cols < g.Cout) cols <<= 1;
  pl->tmem_cols = cols;
  pl->smem_bytes = kAStages * kAStageBytes + pl->b_stages * pl->b_stage_bytes + kRStages * pl->r_stage_bytes + 768 + 1024;
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
int run_fwd(const Geom& g, int math_mode, const Coords& coords, const HeadCfg& head, const float* x, const float* mask,
            const float* w, const float* bias, float* y, void* ws, cudaStream_t st) {
  bool x3 = false;
  Plan pl;
  if (!pick_variant(g, math_mode, &x3, &pl)) return D2C_ERR_MODE;
  uint8_t* wsp = reinterpret_cast<uint8_t*>(ws);
  void* x_cl = wsp; wsp += pl.x_cl_bytes;
  uint8_t* w_sw = wsp; wsp += pl.w_sw_bytes;
  uint4* recs = reinterpret_cast<uint4*>(wsp);
  // A bound sample cache that is large enough takes the operand tiles (written by the kernel), and the staged input
  // and the position records move into it, so that the backward of this call stages nothing a second time.
  SampleCache* sc = current_sample_cache();
  SampleCacheLayout lay{};
  int sav_np = 0;
  uint8_t* sav = nullptr;
  float4* pos = nullptr;
  if (sc) {
    sc->format = 0;
    if (sc->data && sm100_sample_cache_layout(g, x3, &sav_np, &lay) && sc->bytes >= lay.total()) {
      sav = reinterpret_cast<uint8_t*>(sc->data);
      x_cl = sav + lay.image_bytes;
      pos = reinterpret_cast<float4*>(sav + lay.image_bytes + lay.x_cl_bytes);
    }
  }
  int sm_count = 0, rc;
  if ((rc = device_sm_count(&sm_count))) return rc;
  ptx::bind_status_sink();

  const long long n_units = (long long)pl.n_tiles * pl.S;
  long long grid = n_units / kMinUnitsPerCta;
  if (grid > sm_count) grid = sm_count;
  if (grid < 1) grid = 1;
  // The tensor cores add into their fp32 accumulator with truncation: a chain of n accumulating MMAs loses about
  // n * 2^-26 of the result (measured: 2e-5 of scale after 2 600 steps, 8e-5 after 5 200).  The fp32-parity mode
  // therefore ends a chain after 108 units (648 MMAs, ~1e-5) and adds the partial tile to y with fp32 atomics,
  // exactly as it does where a tile is shared between two CTAs.
  const int seg_cap = x3 ? 108 : pl.S;
  // One part per clip (cta_part_range) while every CTA still gets a worthwhile range inside each clip.
  const long long units_per_clip = (long long)pl.tiles_per_clip * pl.S;
  // Many tiles per CTA: deal whole tiles round-robin (fwd_sm100_kernel, part_range) -- consecutive tiles are worked
  // on at the same time and every tile is finished by one CTA; the last round leaves at most 1/8 of a CTA's work
  // unbalanced.
  const bool rr = grid == sm_count && pl.n_tiles >= 8 * grid;
  const int n_parts = rr ? (int)((pl.n_tiles + grid - 1) / grid)
                         : ((g.B > 1 && g.B <= 16 && units_per_clip / grid >= 4 * kMinUnitsPerCta) ? g.B : 1);
  bool whole_tiles_only = seg_cap >= pl.S && (rr || ((pl.n_tiles % grid == 0) && n_parts == 1));

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

  if (pair_clusters > 0) { sav = nullptr; pos = nullptr; x_cl = ws; }       // the CTA-pair kernel keeps nothing
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
    if ((rc = launch_sample_records(g, coords, mask, head, pos, recs, st, x3))) return rc;
    if (!whole_tiles_only) D2C_CUDA_TRY(cudaMemsetAsync(y, 0, sizeof(float) * (size_t)g.B * g.Cout * g.V, st));
  }

  FwdParams p;
  p.g = g; p.x_cl = x_cl; p.w_sw = w_sw; p.recs = recs; p.bias = bias; p.y = y;
  p.cs.dz = g.H * g.W * g.Cin; p.cs.dy = g.W * g.Cin; p.cs.dx = g.Cin;
  p.N = g.Cout; p.nh = pl.nh; p.S = pl.S; p.tiles_per_clip = pl.tiles_per_clip; p.n_tiles = pl.n_tiles;
  p.n_units = n_units;
  p.n_parts = n_parts; p.rr = rr ? 1 : 0;
  p.units_per_part = rr ? 0 : n_units / n_parts; p.part_shift = rr ? 0 : (int)(grid / n_parts);
  p.seg_cap = seg_cap;
  p.b_stages = pl.b_stages; p.b_stage_bytes = pl.b_stage_bytes; p.tmem_cols = pl.tmem_cols;
  // keep the samples for the weight gradient when the caller bound a cache that is large enough
  p.sav = sav; p.sav_np = sav_np; p.sav_pairg = (g.cpg == 32) ? 1 : 0;
  if (sav) sc->format = x3 ? 2 : 1;

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
#ifdef D2C_UNIT_TRACE
  // D2C_UNIT_TRACE=<cta> [D2C_UNIT_TRACE_K0=<first unit of the window>] [D2C_UNIT_TRACE_FILE=<path>]: the call
  // synchronises and writes the buffer after the kernel (instrumented builds only)
  constexpr size_t kTraceWords = 5 * 64 * 8 + 1024 * 4;
  static long long* trace_dev = nullptr;
  p.trace = nullptr; p.trace_cta = 0; p.trace_k0 = 0;
  if (const char* tc = getenv("D2C_UNIT_TRACE")) {
    if (!trace_dev) D2C_CUDA_TRY(cudaMalloc(&trace_dev, kTraceWords * sizeof(long long)));
    D2C_CUDA_TRY(cudaMemsetAsync(trace_dev, 0, kTraceWords * sizeof(long long), st));
    p.trace = trace_dev; p.trace_cta = atoi(tc);
    p.trace_k0 = getenv("D2C_UNIT_TRACE_K0") ? atoi(getenv("D2C_UNIT_TRACE_K0")) : 200;
  }
#endif
  prof_mark(st, "fwd_sm100_fused");
  auto kern = sav ? (x3 ? fwd_sm100_kernel<1, 0, 1> : (pl.dual ? fwd_sm100_kernel<0, 1, 1> : fwd_sm100_kernel<0, 0, 1>))
                  : (x3 ? fwd_sm100_kernel<1, 0, 0> : (pl.dual ? fwd_sm100_kernel<0, 1, 0> : fwd_sm100_kernel<0, 0, 0>));
  D2C_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, pl.smem_bytes));
  kern<<<(unsigned)grid, kThreadsFwd, pl.smem_bytes, st>>>(p);
  D2C_LAUNCH_CHECK();
#ifdef D2C_UNIT_TRACE
  if (p.trace) {
    static long long host[kTraceWords];
    D2C_CUDA_TRY(cudaStreamSynchronize(st));
    D2C_CUDA_TRY(cudaMemcpy(host, trace_dev, sizeof(host), cudaMemcpyDeviceToHost));
    const char* path = getenv("D2C_UNIT_TRACE_FILE");
    FILE* f = fopen(path ? path : (x3 ? "unit_trace_x3.bin" : "unit_trace_bf16.bin"), "wb");
    if (f) {
      const long long hdr[2] = {(long long)grid, (long long)p.trace_k0};
      fwrite(hdr, sizeof(long long), 2, f);
      fwrite(host, sizeof(long long), 5 * 64 * 8 + (size_t)grid * 4, f);
      fclose(f);
    }
  }
#endif
  prof_mark(st, nullptr);
  return D2C_OK;
}

}  // namespace

bool sm100_fwd_variant(const Geom& g, int math_mode, bool* x3) {
  Plan pl;
  return pick_variant(g, math_mode, x3, &pl);
}

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
                      const float* w, const float* bias, float* y, void* ws, cudaStream_t st, const HeadCfg& head) {
  OffsetCoords<float> oc{offset, head.geo_bstride};
  return run_fwd(g, math_mode, oc, head, x, mask, w, bias, y, ws, st);
}

int sm100_fwd_field(const Geom& g, int math_mode, const FieldCoords<float>& fc, const float* x,
                    const float* mask, const float* w, const float* bias, float* y, void* ws, cudaStream_t st,
                    const HeadCfg& head) {
  return run_fwd(g, math_mode, fc, head, x, mask, w, bias, y, ws, st);
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
