// fp32 depthwise 3x3x3 kernels (stride 1, dilation 1, padding 1, channel multiplier 1, even W) built on the
// same bulk-copy pipeline as depthwise_bulk.cuh, with the arithmetic reorganised around sm_100's packed fp32
// FMA (fma.rn.f32x2, two independent fp32 FMAs per issued instruction):
//
//   * outputs are kept as x-adjacent pairs (x0, x0+1), x0 even; the pair of inputs that meets such a pair under
//     tap kx is (x0+kx-1, x0+kx), so every product of the 27-tap stencil is one packed FMA;
//   * a thread owns an R-row x 2-column patch and marches along z; per staged plane and input row it issues one
//     8-byte and two 4-byte shared-memory loads.  Consecutive lanes own consecutive pairs, so the 8-byte loads
//     and the stores of a warp are contiguous (a 4-column patch per thread was tried first: its 16-byte lane
//     stride cost 4-way bank conflicts and the shared-memory pipe became the limit);
//   * forward / input gradient (R = 4): the 27 weights live in registers as broadcast pairs, read from a small
//     shared-memory table -- a pair built in registers from one scalar is rebuilt by the compiler at every use;
//   * weight gradient (R = 2): the 27 sums are (even-x, odd-x) pairs, added when the block flushes.
//
// Staged layout as in depthwise_bulk.cuh, but every gap holds W + 4 zeros (rounded up to 16 bytes) so that
// column -1 of row -1 and column W of row H stay inside the stage.  In real rows columns -1 and W hold a
// neighbouring row's data and are replaced by zero with a select (never multiplied by zero, so non-finite
// data next to a border stays where the reference keeps it).
// Reference: ops/fast-depthwise-conv3d/csrc/grouped_conv3d.cu:22-276.
#pragma once

#include "depthwise_bulk.cuh"

namespace d2c {
namespace {

using u64 = unsigned long long;

struct DwQuadPlan {
  int nvol;               // volumes per chunk (conv); 1 for the weight gradient
  long long nchunks;
  uint32_t plane_bytes, gap_bytes, stage_x_bytes, stage_bytes;
  int nyp, nxp, items;    // row groups, column pairs, patches per volume
  int threads, blocks;
  size_t smem;
};

constexpr int kDwQuadMaxThreads = 224;
constexpr int kDwQuadWgradMaxThreads = 448;   // compute threads + the loader warp
constexpr int kDwQuadTab = 28;         // weight-pair table entries per volume: 27 taps + bias
constexpr int kDwQuadConvRows = 4;     // patch rows, forward / input gradient
constexpr int kDwQuadWgradRows = 2;    // patch rows, weight gradient

inline bool dw_quad_plan(const Geom& g, int tensors, DwQuadPlan* p) {
  if (!(g.kd == 3 && g.kh == 3 && g.kw == 3 && g.sd == 1 && g.sh == 1 && g.sw == 1 && g.dd == 1 && g.dh == 1 &&
        g.dw == 1 && g.pd == 1 && g.ph == 1 && g.pw == 1 && g.Cout == g.Cin))
    return false;
  if (g.W % 2 != 0 || g.W < 2) return false;
  const long long vols = (long long)g.B * g.Cin;
  const size_t pbytes = (size_t)g.H * g.W * 4;
  if (pbytes % 16 != 0) return false;
  const size_t gap = align_up((size_t)(g.W + 4) * 4, 16);
  const size_t vstage = (size_t)g.D * (pbytes + gap);
  const int R = tensors == 2 ? kDwQuadWgradRows : kDwQuadConvRows;
  p->nyp = (g.H + R - 1) / R;
  p->nxp = g.W / 2;
  p->items = p->nyp * p->nxp;
  int n = 1;
  if (tensors == 1)
    while ((n * vstage) < 24 * 1024 && vols % (2 * n) == 0 && vols / (2 * n) >= 148 * 4) n *= 2;
  const size_t stage_x = n * vstage + gap;
  const size_t stage = stage_x + (tensors == 2 ? (size_t)g.D * pbytes : 0);
  const size_t need = 2 * stage + 128 + (tensors == 1 ? 2 * (size_t)n * kDwQuadTab * 8 : 0);
  if (need > kDwBulkSmemMax) return false;
  p->nvol = n;
  p->nchunks = vols / n;
  p->plane_bytes = (uint32_t)pbytes;
  p->gap_bytes = (uint32_t)gap;
  p->stage_x_bytes = (uint32_t)stage_x;
  p->stage_bytes = (uint32_t)stage;
  p->smem = need;
  const int per_sm = (tensors == 1 && need <= 112 * 1024) ? 2 : 1;
  const int cap = tensors == 2 ? kDwQuadWgradMaxThreads - 32 : kDwQuadMaxThreads;
  const long long work = (long long)n * p->items;
  const long long passes = (work + cap - 1) / cap;
  int threads = (int)(((work + passes - 1) / passes + 31) / 32 * 32);
  if (threads < 64) threads = 64;
  p->threads = threads;
  long long blocks = 148LL * per_sm;
  if (blocks > p->nchunks) blocks = p->nchunks;
  p->blocks = (int)blocks;
  return true;
}

__device__ __forceinline__ u64 pk2(float a, float b) {
  u64 r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ float2 unpk2(u64 v) {
  float2 r;
  asm("mov.b64 {%0, %1}, %2;" : "=f"(r.x), "=f"(r.y) : "l"(v));
  return r;
}
// d += a * b on both halves, each rounded once (same result as two fmaf)
__device__ __forceinline__ void fma2(u64& d, u64 a, u64 b) {
  asm("fma.rn.f32x2 %0, %1, %2, %0;" : "+l"(d) : "l"(a), "l"(b));
}
__device__ __forceinline__ u64 fma2c(u64 a, u64 b, u64 c) {
  u64 d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}

// Element offsets, from the start of a staged plane, of column x0-1 of the patch's N input rows y0-1 ..
// y0+N-2 (rows -1 and >= H are the zero gaps).
template <int N>
struct DwqRows {
  int a[N];
  bool okL, okR;   // column x0-1 / column x0+2 inside the plane
};

template <int N>
__device__ __forceinline__ DwqRows<N> dwq_rows(int y0, int x0, int H, int W) {
  DwqRows<N> R;
#pragma unroll
  for (int j = 0; j < N; ++j) R.a[j] = min(y0 - 1 + j, H) * W + x0 - 1;
  R.okL = x0 > 0;
  R.okR = x0 + 2 < W;
  return R;
}

// Raw values of input row j: columns x0-1, (x0, x0+1), x0+2.
struct DwqRaw {
  float v0, v3;
  float2 a;
};

template <int N>
__device__ __forceinline__ DwqRaw dwq_row_load(const float* plane, const DwqRows<N>& R, int j) {
  const float* ra = plane + R.a[j];
  DwqRaw q;
  q.v0 = ra[0];
  q.a = *reinterpret_cast<const float2*>(ra + 1);
  q.v3 = ra[3];
  return q;
}

// The three x-adjacent input pairs (x0-1,x0), (x0,x0+1), (x0+1,x0+2) of a loaded row.
template <int N>
__device__ __forceinline__ void dwq_row_pairs(const DwqRaw& q, const DwqRows<N>& R, u64 (&P)[3]) {
  const float v0 = R.okL ? q.v0 : 0.f;
  const float v3 = R.okR ? q.v3 : 0.f;
  P[0] = pk2(v0, q.a.x);
  P[1] = pk2(q.a.x, q.a.y);
  P[2] = pk2(q.a.y, v3);
}

// One z step of the conv march: plane p feeds outputs p-1 (kz=2), p (kz=1), p+1 (kz=0); output p+1 starts
// from the bias pair bb.  acc[r]: row r of the patch.
template <int R>
__device__ __forceinline__ void dwq_conv_step(const float* plane, const DwqRows<R + 2>& rows, const u64 (&wk)[27],
                                              u64 bb, u64 (&am1)[R], u64 (&a0)[R], u64 (&ap1)[R]) {
  // the shared-memory loads of row j+1 are issued before the arithmetic of row j
  DwqRaw raw[2];
  raw[0] = dwq_row_load<R + 2>(plane, rows, 0);
#pragma unroll
  for (int j = 0; j < R + 2; ++j) {
    if (j + 1 < R + 2) raw[(j + 1) & 1] = dwq_row_load<R + 2>(plane, rows, j + 1);
    u64 P[3];
    dwq_row_pairs<R + 2>(raw[j & 1], rows, P);
    // kx outermost: successive updates of one accumulator are 3 x (rows) packed FMAs apart
#pragma unroll
    for (int kx = 0; kx < 3; ++kx)
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const int ky = j - r;
        if (ky < 0 || ky > 2) continue;
        fma2(am1[r], wk[(2 * 3 + ky) * 3 + kx], P[kx]);
        fma2(a0[r], wk[(1 * 3 + ky) * 3 + kx], P[kx]);
        if (ky == 0 && kx == 0)
          ap1[r] = fma2c(wk[0], P[0], bb);
        else
          fma2(ap1[r], wk[(0 * 3 + ky) * 3 + kx], P[kx]);
      }
  }
}

template <int R>
__device__ __forceinline__ void dwq_store(float* dst, int W, int rows_ok, const u64 (&a)[R]) {
#pragma unroll
  for (int r = 0; r < R; ++r)
    if (r < rows_ok) *reinterpret_cast<float2*>(dst + r * W) = unpk2(a[r]);
}

// Forward / input gradient.  The last warp of the block is the loader: it fills a stage's weight-pair table and
// issues the stage's bulk copies as soon as every compute warp has released that stage ("empty" mbarrier, one
// arrival per compute warp); compute warps wait on the stage's "full" mbarrier, never on each other.
// Shared memory: [stage 0][stage 1][full 0, full 1, empty 0, empty 1][abort flag at +64][weight-pair tables of
// both stages at +128].
__global__ void __launch_bounds__(kDwQuadMaxThreads + 32, 2)
dw_quad_conv_kernel(Geom g, int nyp, int nxp, int nvol, long long nchunks, uint32_t plane_bytes, uint32_t gap_bytes,
                    uint32_t stage_bytes, const float* __restrict__ in, const float* __restrict__ w,
                    const float* __restrict__ bias, float* __restrict__ out, int flip) {
  constexpr int R = kDwQuadConvRows;
  extern __shared__ __align__(128) unsigned char dwb_smem[];
  const uint32_t bar0 = ptx::smem_u32(dwb_smem + 2 * (size_t)stage_bytes);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(dwb_smem + 2 * (size_t)stage_bytes + 64);
  float2* wtab = reinterpret_cast<float2*>(dwb_smem + 2 * (size_t)stage_bytes + 128);
  const long long lo = nchunks * blockIdx.x / gridDim.x, hi = nchunks * (blockIdx.x + 1) / gridDim.x;
  const int planes = nvol * g.D, HW = g.H * g.W;
  const uint32_t pstride = plane_bytes + gap_bytes;
  const int compute_threads = (int)blockDim.x - 32;
  auto full_bar = [&](int s) { return bar0 + 8 * s; };
  auto empty_bar = [&](int s) { return bar0 + 16 + 8 * s; };
  if (threadIdx.x == 0) {
    ptx::mbar_init(full_bar(0), 1);
    ptx::mbar_init(full_bar(1), 1);
    ptx::mbar_init(empty_bar(0), (uint32_t)(compute_threads / 32));
    ptx::mbar_init(empty_bar(1), (uint32_t)(compute_threads / 32));
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  dwb_zero_gaps(dwb_smem, stage_bytes, plane_bytes, gap_bytes, planes);   // ends with a block barrier
  const int tab_n = nvol * kDwQuadTab;

  if ((int)threadIdx.x >= compute_threads) {
    // ---- loader warp ----
    const int lane = threadIdx.x & 31;
    const unsigned char* src_bytes = reinterpret_cast<const unsigned char*>(in);
    int it = 0;
    bool ok = true;
    for (long long ch = lo; ch < hi; ++ch, ++it) {
      const int s = it & 1;
      if (it >= 2 && !ptx::mbar_wait(empty_bar(s), ((it >> 1) - 1) & 1, abort_flag)) { ok = false; break; }
      // table entry e = (vol, t): (w, w) of that volume's channel, t = 27: the bias
      for (int e = lane; e < tab_n; e += 32) {
        const int vol = e / kDwQuadTab, t = e - vol * kDwQuadTab;
        const int c = (int)((ch * nvol + vol) % g.Cin);
        const float v = t < 27 ? __ldg(w + (long long)c * 27 + (flip ? 26 - t : t)) : (bias ? __ldg(bias + c) : 0.f);
        wtab[s * tab_n + e] = make_float2(v, v);
      }
      __syncwarp();
      if (lane == 0) {
        // the arrive (release) below orders the table writes of the whole warp before the stage becomes full
        ptx::mbar_arrive_expect_tx(full_bar(s), (uint32_t)planes * plane_bytes);
        const unsigned char* src = src_bytes + ch * (long long)planes * plane_bytes;
        const uint32_t dst = ptx::smem_u32(dwb_smem + (size_t)s * stage_bytes + gap_bytes);
        for (int k = 0; k < planes; ++k)
          ptx::bulk_g2s(dst + k * pstride, src + (size_t)k * plane_bytes, plane_bytes, full_bar(s));
      }
      __syncwarp();
    }
    // never leave with a bulk copy in flight: the last two stages issued must have landed
    if (lane == 0)
      for (int back = 1; back <= 2 && back <= it; ++back) {
        const int j = it - back;
        const long long t0 = clock64();
        while (!ptx::mbar_try_wait(full_bar(j & 1), (j >> 1) & 1))
          if (clock64() - t0 > ptx::kWaitBudgetCycles) break;
      }
    if (!ok && lane == 0) *abort_flag = 1;
  } else {
    // ---- compute warps ----
    const int items = nyp * nxp, work = nvol * items;
    const int pstride_e = (int)(pstride / 4);
    int it = 0;
    for (long long ch = lo; ch < hi; ++ch, ++it) {
      const int s = it & 1;
      if (!ptx::mbar_wait(full_bar(s), (it >> 1) & 1, abort_flag)) break;
      const float* stage = reinterpret_cast<const float*>(dwb_smem + (size_t)s * stage_bytes + gap_bytes);
      for (int wi = threadIdx.x; wi < work; wi += compute_threads) {
        const int vol = wi / items, rem = wi - vol * items;
        const int yp = rem / nxp, xp = rem - yp * nxp, y0 = yp * R, x0 = xp * 2;
        const long long bc = ch * nvol + vol;
        const u64* wt = reinterpret_cast<const u64*>(wtab) + (s * nvol + vol) * kDwQuadTab;
        u64 wk[27];
#pragma unroll
        for (int t = 0; t < 27; ++t) wk[t] = wt[t];
        const u64 bb = wt[27];
        const DwqRows<R + 2> rows = dwq_rows<R + 2>(y0, x0, g.H, g.W);
        const float* sm = stage + (long long)vol * g.D * pstride_e;
        float* dst = out + bc * g.Vin + (long long)y0 * g.W + x0;
        const int rows_ok = min(R, g.H - y0);
        u64 aa[R], ab[R], ac[R];
#pragma unroll
        for (int r = 0; r < R; ++r) aa[r] = ab[r] = ac[r] = bb;
        // plane p completes output plane p-1; the accumulator roles rotate with period 3
        for (int p = 0; p < g.D; p += 3) {
          dwq_conv_step<R>(sm + p * pstride_e, rows, wk, bb, aa, ab, ac);
          if (p >= 1) dwq_store<R>(dst + (long long)(p - 1) * HW, g.W, rows_ok, aa);
          if (p + 1 >= g.D) { dwq_store<R>(dst + (long long)p * HW, g.W, rows_ok, ab); break; }
          dwq_conv_step<R>(sm + (p + 1) * pstride_e, rows, wk, bb, ab, ac, aa);
          dwq_store<R>(dst + (long long)p * HW, g.W, rows_ok, ab);
          if (p + 2 >= g.D) { dwq_store<R>(dst + (long long)(p + 1) * HW, g.W, rows_ok, ac); break; }
          dwq_conv_step<R>(sm + (p + 2) * pstride_e, rows, wk, bb, ac, aa, ab);
          dwq_store<R>(dst + (long long)(p + 1) * HW, g.W, rows_ok, ac);
          if (p + 3 >= g.D) dwq_store<R>(dst + (long long)(p + 2) * HW, g.W, rows_ok, aa);
        }
      }
      __syncwarp();
      if ((threadIdx.x & 31) == 0) ptx::mbar_arrive(empty_bar(s));   // this warp is done with stage s
    }
  }
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) ptx::report_device_timeout();
}

// Weight gradient.  grad_out pairs of the patch's R rows at plane q of the contiguous staged volume; rows and
// planes outside the tensor give zero pairs, so that whatever input they meet contributes nothing.
template <int R>
__device__ __forceinline__ void dwq_load_grads(const float* gs, int W, int rows_ok, bool in_range, u64 (&G)[R]) {
#pragma unroll
  for (int r = 0; r < R; ++r) {
    float2 a = make_float2(0.f, 0.f);
    if (in_range && r < rows_ok) a = *reinterpret_cast<const float2*>(gs + r * W);
    G[r] = pk2(a.x, a.y);
  }
}

// One z step of the weight-gradient march: x plane p meets grad_out planes p+1 (kz=0), p (kz=1), p-1 (kz=2).
template <int R>
__device__ __forceinline__ void dwq_wgrad_step(const float* xplane, const DwqRows<R + 2>& rows, u64 (&acc)[27],
                                               const u64 (&gm1)[R], const u64 (&g0)[R], const u64 (&gp1)[R]) {
  DwqRaw raw[2];
  raw[0] = dwq_row_load<R + 2>(xplane, rows, 0);
#pragma unroll
  for (int j = 0; j < R + 2; ++j) {
    if (j + 1 < R + 2) raw[(j + 1) & 1] = dwq_row_load<R + 2>(xplane, rows, j + 1);
    u64 P[3];
    dwq_row_pairs<R + 2>(raw[j & 1], rows, P);
#pragma unroll
    for (int r = 0; r < R; ++r) {
      const int ky = j - r;
      if (ky < 0 || ky > 2) continue;
#pragma unroll
      for (int kx = 0; kx < 3; ++kx) {
        fma2(acc[(0 * 3 + ky) * 3 + kx], gp1[r], P[kx]);
        fma2(acc[(1 * 3 + ky) * 3 + kx], g0[r], P[kx]);
        fma2(acc[(2 * 3 + ky) * 3 + kx], gm1[r], P[kx]);
      }
    }
  }
}

// Sum of the 27 pair accumulators over the warp, one atomic per tap into partial[c][27]; clears acc.
__device__ __forceinline__ void dwq_flush_warp(u64 (&acc)[27], float* __restrict__ partial, int c) {
  const int lane = threadIdx.x & 31;
  float mine = 0.f;
#pragma unroll
  for (int t = 0; t < 27; ++t) {
    const float2 v = unpk2(acc[t]);
    float sv = v.x + v.y;
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) sv += __shfl_xor_sync(0xffffffffu, sv, o);
    if (lane == t) mine = sv;
    acc[t] = 0ull;
  }
  if (lane < 27) atomicAdd(partial + (long long)c * 27 + lane, mine);
}

// Work items are (channel, clip) pairs, channel-major; a warp flushes its 27 sums (shuffles + one atomic per
// tap) when the channel changes.  The block's last warp is the loader, as in the conv kernel; compute warps
// never meet at a block barrier.  Shared memory: [stage0: gapped x volume, grad_out volume][stage1: ...]
// [full 0, full 1, empty 0, empty 1][abort flag at +64].
__global__ void __launch_bounds__(kDwQuadWgradMaxThreads, 1)
dw_quad_wgrad_kernel(Geom g, int nyp, int nxp, uint32_t plane_bytes, uint32_t gap_bytes, uint32_t stage_x_bytes,
                     uint32_t stage_bytes, const float* __restrict__ gy, const float* __restrict__ x,
                     float* __restrict__ partial) {
  constexpr int R = kDwQuadWgradRows;
  extern __shared__ __align__(128) unsigned char dwb_smem[];
  const uint32_t bar0 = ptx::smem_u32(dwb_smem + 2 * (size_t)stage_bytes);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(dwb_smem + 2 * (size_t)stage_bytes + 64);
  const long long n_items = (long long)g.Cin * g.B;
  const long long lo = n_items * blockIdx.x / gridDim.x, hi = n_items * (blockIdx.x + 1) / gridDim.x;
  const int HW = g.H * g.W;
  const uint32_t pstride = plane_bytes + gap_bytes, vol_bytes = (uint32_t)g.D * plane_bytes;
  const int compute_threads = (int)blockDim.x - 32;
  auto full_bar = [&](int s) { return bar0 + 8 * s; };
  auto empty_bar = [&](int s) { return bar0 + 16 + 8 * s; };
  if (threadIdx.x == 0) {
    ptx::mbar_init(full_bar(0), 1);
    ptx::mbar_init(full_bar(1), 1);
    ptx::mbar_init(empty_bar(0), (uint32_t)(compute_threads / 32));
    ptx::mbar_init(empty_bar(1), (uint32_t)(compute_threads / 32));
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  dwb_zero_gaps(dwb_smem, stage_bytes, plane_bytes, gap_bytes, g.D);   // ends with a block barrier

  if ((int)threadIdx.x >= compute_threads) {
    // ---- loader warp (one lane) ----
    if ((threadIdx.x & 31) == 0) {
      const unsigned char* xb = reinterpret_cast<const unsigned char*>(x);
      const unsigned char* gb = reinterpret_cast<const unsigned char*>(gy);
      int it = 0;
      bool ok = true;
      for (long long item = lo; item < hi; ++item, ++it) {
        const int s = it & 1;
        if (it >= 2 && !ptx::mbar_wait(empty_bar(s), ((it >> 1) - 1) & 1, abort_flag)) { ok = false; break; }
        const long long c = item / g.B, b = item - c * g.B;
        const long long voff = (b * g.Cin + c) * (long long)vol_bytes;
        ptx::mbar_arrive_expect_tx(full_bar(s), 2 * vol_bytes);
        const uint32_t dst = ptx::smem_u32(dwb_smem + (size_t)s * stage_bytes);
        for (int k = 0; k < g.D; ++k)
          ptx::bulk_g2s(dst + gap_bytes + k * pstride, xb + voff + (size_t)k * plane_bytes, plane_bytes, full_bar(s));
        ptx::bulk_g2s(dst + stage_x_bytes, gb + voff, vol_bytes, full_bar(s));
      }
      // never leave with a bulk copy in flight
      for (int back = 1; back <= 2 && back <= it; ++back) {
        const int j = it - back;
        const long long t0 = clock64();
        while (!ptx::mbar_try_wait(full_bar(j & 1), (j >> 1) & 1))
          if (clock64() - t0 > ptx::kWaitBudgetCycles) break;
      }
      if (!ok) *abort_flag = 1;
    }
  } else {
    // ---- compute warps ----
    const int patches = nyp * nxp, pstride_e = (int)(pstride / 4);
    u64 acc[27];
#pragma unroll
    for (int t = 0; t < 27; ++t) acc[t] = 0ull;
    int it = 0;
    long long c_open = -1;                    // channel whose sums are in acc
    for (long long item = lo; item < hi; ++item, ++it) {
      const int s = it & 1;
      if (!ptx::mbar_wait(full_bar(s), (it >> 1) & 1, abort_flag)) break;
      const float* xs = reinterpret_cast<const float*>(dwb_smem + (size_t)s * stage_bytes + gap_bytes);
      const float* gs0 = reinterpret_cast<const float*>(dwb_smem + (size_t)s * stage_bytes + stage_x_bytes);
      c_open = item / g.B;
      for (int wi = threadIdx.x; wi < patches; wi += compute_threads) {
        const int yp = wi / nxp, xp = wi - yp * nxp, y0 = yp * R, x0 = xp * 2;
        const DwqRows<R + 2> rows = dwq_rows<R + 2>(y0, x0, g.H, g.W);
        const int rows_ok = min(R, g.H - y0);
        const float* gs = gs0 + y0 * g.W + x0;
        u64 ga[R], gbv[R], gc[R];
        auto grads = [&](int q, u64 (&G)[R]) {
          dwq_load_grads<R>(gs + (long long)q * HW, g.W, rows_ok, q >= 0 && q < g.D, G);
        };
        grads(-1, ga); grads(0, gbv); grads(1, gc);
        for (int p = 0; p < g.D; p += 3) {
          dwq_wgrad_step<R>(xs + p * pstride_e, rows, acc, ga, gbv, gc);
          if (p + 1 >= g.D) break;
          grads(p + 2, ga);
          dwq_wgrad_step<R>(xs + (p + 1) * pstride_e, rows, acc, gbv, gc, ga);
          if (p + 2 >= g.D) break;
          grads(p + 3, gbv);
          dwq_wgrad_step<R>(xs + (p + 2) * pstride_e, rows, acc, gc, ga, gbv);
          grads(p + 4, gc);
        }
      }
      __syncwarp();
      if ((threadIdx.x & 31) == 0) ptx::mbar_arrive(empty_bar(s));   // this warp is done with stage s
      if (item + 1 == hi || (item + 1) / g.B != c_open) {
        dwq_flush_warp(acc, partial, (int)c_open);
        c_open = -1;
      }
    }
    if (c_open >= 0) dwq_flush_warp(acc, partial, (int)c_open);      // left the loop early: keep what was summed
  }
  __syncthreads();
  if (threadIdx.x == 0 && *abort_flag) ptx::report_device_timeout();
}

inline int dw_quad_conv(const Geom& g, const DwQuadPlan& p, const float* in, const float* w, const float* bias,
                        float* out, int flip, cudaStream_t st) {
  D2C_CUDA_TRY(cudaFuncSetAttribute(dw_quad_conv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem));
  dw_quad_conv_kernel<<<p.blocks, p.threads + 32, p.smem, st>>>(g, p.nyp, p.nxp, p.nvol, p.nchunks, p.plane_bytes,
                                                           p.gap_bytes, p.stage_bytes, in, w, bias, out, flip);
  D2C_LAUNCH_CHECK();
  return D2C_OK;
}

inline int dw_quad_wgrad(const Geom& g, const DwQuadPlan& p, const float* gy, const float* x, float* partial,
                         cudaStream_t st) {
  const size_t smem = p.smem;
  D2C_CUDA_TRY(cudaFuncSetAttribute(dw_quad_wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dw_quad_wgrad_kernel<<<p.blocks, p.threads + 32, smem, st>>>(g, p.nyp, p.nxp, p.plane_bytes, p.gap_bytes,
                                                          p.stage_x_bytes, p.stage_bytes, gy, x, partial);
  D2C_LAUNCH_CHECK();
  return D2C_OK;
}

}  // namespace
}  // namespace d2c
