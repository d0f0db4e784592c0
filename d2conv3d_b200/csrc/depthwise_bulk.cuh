// Bulk-copy pipelined kernels for the common depthwise case (3x3x3, stride 1, dilation 1, padding 1, channel
// multiplier 1) when whole (clip, channel) volumes fit in shared memory.
//
// In the [B][C][D][H][W] layout every z-plane of a (clip, channel) volume is one contiguous byte range, so a
// persistent block streams its share of the tensor with untiled bulk async copies (cp.async.bulk global ->
// shared, completion on an mbarrier): one elected thread keeps the copies of chunk i+1 in flight while all
// threads compute chunk i from shared memory.  That puts ~100 KB per SM in flight with no global loads in the
// compute loop, which the register-window march kernels (depthwise_tile.cuh) cannot do: they stall on
// global-load latency at 25 % occupancy.
//
// Staged layout of one volume: [gap][plane 0][gap][plane 1] ... [plane D-1][gap], every gap one row of zeros
// (rounded up to 16 bytes), written once per block and never touched by the copies.  Rows -1 and H of any
// plane therefore read zeros without a predicate.  Column borders are handled by clamping the neighbour
// column to the thread's own column (so the value read is a finite member of the output's neighbourhood) and
// zeroing the matching weights (forward / input gradient) or grad_out copies (weight gradient) per thread.
//
// Compute is a z march: a thread owns R adjacent rows at one x, reads the (R+2) x 3 neighbourhood of each
// plane from shared memory once, and scatters it into the accumulators of output planes p-1, p, p+1.
// Reference: ops/fast-depthwise-conv3d/csrc/grouped_conv3d.cu:22-276.
#pragma once

#include "depthwise_tile.cuh"
#include "sm100_ptx.cuh"

namespace d2c {
namespace {


struct DwBulkPlan {
  int nvol;               // volumes per chunk (forward / input gradient); 1 for the weight gradient
  long long nchunks;
  uint32_t plane_bytes;   // H*W*esize, a multiple of 16
  uint32_t gap_bytes;     // >= one row, a multiple of 16
  uint32_t stage_x_bytes; // gapped staging of one chunk
  uint32_t stage_bytes;   // stage_x_bytes (+ contiguous grad_out volume for the weight gradient)
  int threads, blocks;
  size_t smem;            // 2 stages + barriers + abort flag (+ reduction scratch, added by the launcher)
};

constexpr size_t kDwBulkSmemMax = 220 * 1024;
constexpr int kDwBulkConvThreads = 320;    // x2 blocks per SM when two stages fit twice, no register cap
constexpr int kDwBulkWgradThreads = 832;   // one block per SM (two tensors staged)

// tensors: how many tensors are staged per chunk (1: conv, 2: weight gradient).
inline bool dw_bulk_plan(const Geom& g, size_t esize, int tensors, const DwTilePlan& tp, DwBulkPlan* p) {
  const long long vols = (long long)g.B * g.Cin;
  const size_t pbytes = (size_t)g.H * g.W * esize;
  if (pbytes % 16 != 0) return false;
  const size_t gap = align_up((size_t)g.W * esize, 16);
  const size_t vstage = (size_t)g.D * (pbytes + gap);      // + one more gap per chunk
  int n = 1;
  if (tensors == 1)
    while ((n * vstage) < 24 * 1024 && vols % (2 * n) == 0 && vols / (2 * n) >= 148 * 4) n *= 2;
  const size_t stage_x = n * vstage + gap;
  const size_t stage = stage_x + (tensors == 2 ? (size_t)g.D * pbytes : 0);
  const size_t need = 2 * stage + 128;
  if (need > kDwBulkSmemMax) return false;
  p->nvol = n;
  p->nchunks = vols / n;
  p->plane_bytes = (uint32_t)pbytes;
  p->gap_bytes = (uint32_t)gap;
  p->stage_x_bytes = (uint32_t)stage_x;
  p->stage_bytes = (uint32_t)stage;
  p->smem = need;
  const int per_sm = need <= 112 * 1024 ? 2 : 1;
  const long long cols = (long long)n * tp.ncol;
  int threads = tensors == 2 ? kDwBulkWgradThreads : (per_sm == 2 ? kDwBulkConvThreads : 512);
  // do not leave most of the last pass idle: spread the columns evenly over the passes
  const long long passes = (cols + threads - 1) / threads;
  threads = (int)(((cols + passes - 1) / passes + 31) / 32 * 32);
  if (threads < 64) threads = 64;
  p->threads = threads;
  long long blocks = 148LL * per_sm;
  if (blocks > p->nchunks) blocks = p->nchunks;
  p->blocks = (int)blocks;
  return true;
}

template <typename T, typename A> __device__ __forceinline__ A dwb_cvt(T v) { return (A)v; }
template <> __device__ __forceinline__ float dwb_cvt<__half, float>(__half v) { return __half2float(v); }

// Element offsets, relative to the start of a staged plane, of the (R+2) x 3 neighbourhood of rows
// [y0, y0+R) at column x: rows run from y0-1 (row -1 is the zero gap) to min(y0+R, H) (row H is the next
// gap); the neighbour columns are clamped to x at the plane's left/right border.
template <int R>
__device__ __forceinline__ void dwb_offsets(int y0, int x, int H, int W, int (&off)[R + 2][3]) {
  const int xl = x > 0 ? x - 1 : x, xr = x < W - 1 ? x + 1 : x;
#pragma unroll
  for (int j = 0; j < R + 2; ++j) {
    const int row = min(y0 - 1 + j, H) * W;
    off[j][0] = row + xl;
    off[j][1] = row + x;
    off[j][2] = row + xr;
  }
}

template <typename T, typename A, int R>
__device__ __forceinline__ void dwb_plane(const T* plane, const int (&off)[R + 2][3], A (&v)[R + 2][3]) {
#pragma unroll
  for (int j = 0; j < R + 2; ++j)
#pragma unroll
    for (int i = 0; i < 3; ++i) v[j][i] = dwb_cvt<T, A>(plane[off[j][i]]);
}

// Zero the gaps of both stages (block-wide; ends with a barrier).  Gaps sit at k * (plane + gap) for
// k = 0 .. planes_per_stage.
__device__ __forceinline__ void dwb_zero_gaps(unsigned char* smem, uint32_t stage_bytes, uint32_t plane_bytes,
                                              uint32_t gap_bytes, int planes_per_stage) {
  const int words = gap_bytes / 4, total = 2 * (planes_per_stage + 1) * words;
  for (int e = threadIdx.x; e < total; e += blockDim.x) {
    const int gi = e / words, wd = e - gi * words;
    const int s = gi / (planes_per_stage + 1), k = gi - s * (planes_per_stage + 1);
    reinterpret_cast<uint32_t*>(smem + (size_t)s * stage_bytes + (size_t)k * (plane_bytes + gap_bytes))[wd] = 0u;
  }
  __syncthreads();
}

// One z step of the conv march over a staged volume: plane p feeds outputs p-1 (kz=2), p (kz=1), p+1 (kz=0).
template <typename T, typename A, int R>
__device__ __forceinline__ void dwb_conv_step(const T* plane, T* __restrict__ dst, int p, int D, int HW, int W,
                                              int rows_ok, const int (&off)[R + 2][3], const A (&wk)[27], A bb,
                                              A (&am1)[R], A (&a0)[R], A (&ap1)[R]) {
  A v[R + 2][3];
  dwb_plane<T, A, R>(plane, off, v);
#pragma unroll
  for (int r = 0; r < R; ++r) ap1[r] = bb;
#pragma unroll
  for (int ky = 0; ky < 3; ++ky)
#pragma unroll
    for (int kx = 0; kx < 3; ++kx)
#pragma unroll
      for (int r = 0; r < R; ++r) {
        am1[r] += wk[(2 * 3 + ky) * 3 + kx] * v[r + ky][kx];
        a0[r] += wk[(1 * 3 + ky) * 3 + kx] * v[r + ky][kx];
        ap1[r] += wk[(0 * 3 + ky) * 3 + kx] * v[r + ky][kx];
      }
#pragma unroll
  for (int r = 0; r < R; ++r)
    if (r < rows_ok) {
      if (p >= 1) dst[(long long)(p - 1) * HW + r * W] = dwt_st<T, A>(am1[r]);
      if (p == D - 1) dst[(long long)p * HW + r * W] = dwt_st<T, A>(a0[r]);
    }
}

// Shared memory: [stage 0][stage 1][2 mbarriers][abort flag].
template <typename T, typename A, int R>
__global__ void __launch_bounds__(512)
dw_bulk_conv_kernel(Geom g, int nyp, int nvol, long long nchunks, uint32_t plane_bytes, uint32_t gap_bytes,
                    uint32_t stage_bytes, const T* __restrict__ in, const T* __restrict__ w,
                    const T* __restrict__ bias, T* __restrict__ out, int flip) {
  extern __shared__ __align__(128) unsigned char dwb_smem[];
  const uint32_t bar0 = ptx::smem_u32(dwb_smem + 2 * (size_t)stage_bytes);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(dwb_smem + 2 * (size_t)stage_bytes + 16);
  const long long lo = nchunks * blockIdx.x / gridDim.x, hi = nchunks * (blockIdx.x + 1) / gridDim.x;
  const int planes = nvol * g.D, HW = g.H * g.W;
  const uint32_t pstride = plane_bytes + gap_bytes;
  if (threadIdx.x == 0) {
    ptx::mbar_init(bar0, 1);
    ptx::mbar_init(bar0 + 8, 1);
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  dwb_zero_gaps(dwb_smem, stage_bytes, plane_bytes, gap_bytes, planes);
  const unsigned char* src_bytes = reinterpret_cast<const unsigned char*>(in);
  auto issue = [&](long long ch, int s) {
    const uint32_t bar = bar0 + 8 * s;
    ptx::mbar_arrive_expect_tx(bar, (uint32_t)planes * plane_bytes);
    const unsigned char* src = src_bytes + ch * (long long)planes * plane_bytes;
    const uint32_t dst = ptx::smem_u32(dwb_smem + (size_t)s * stage_bytes + gap_bytes);
    for (int k = 0; k < planes; ++k) ptx::bulk_g2s(dst + k * pstride, src + (size_t)k * plane_bytes, plane_bytes, bar);
  };
  if (threadIdx.x == 0 && lo < hi) issue(lo, 0);
  const int ncol = nyp * g.W, cols = nvol * ncol;
  const int pstride_e = (int)(pstride / sizeof(T));
  int it = 0;
  for (long long ch = lo; ch < hi; ++ch, ++it) {
    const int s = it & 1;
    // stage s^1 was released by the barrier that ended iteration it-1
    if (threadIdx.x == 0 && ch + 1 < hi) issue(ch + 1, s ^ 1);
    if (!ptx::mbar_wait(bar0 + 8 * s, (it >> 1) & 1, abort_flag)) break;
    const T* stage = reinterpret_cast<const T*>(dwb_smem + (size_t)s * stage_bytes + gap_bytes);
    for (int col = threadIdx.x; col < cols; col += blockDim.x) {
      const int vol = col / ncol, rem = col - vol * ncol;
      const int yp = rem / g.W, x = rem - yp * g.W, y0 = yp * R;
      const long long bc = ch * nvol + vol;
      const int c = (int)(bc % g.Cin);
      const A ml = x > 0 ? (A)1 : (A)0, mr = x < g.W - 1 ? (A)1 : (A)0;
      A wk[27];
#pragma unroll
      for (int t = 0; t < 27; ++t) {
        const A wv = dwt_ld<T, A>(w + (long long)c * 27 + (flip ? 26 - t : t));
        wk[t] = (t % 3 == 0) ? wv * ml : ((t % 3 == 2) ? wv * mr : wv);
      }
      const A bb = bias ? dwt_ld<T, A>(bias + c) : (A)0;
      int off[R + 2][3];
      dwb_offsets<R>(y0, x, g.H, g.W, off);
      const T* sm = stage + (long long)vol * g.D * pstride_e;
      T* dst = out + bc * g.Vin + (long long)y0 * g.W + x;
      const int rows_ok = min(R, g.H - y0);
      A aa[R], ab[R], ac[R];
#pragma unroll
      for (int r = 0; r < R; ++r) aa[r] = ab[r] = ac[r] = bb;
      for (int p = 0; p < g.D; p += 3) {
        dwb_conv_step<T, A, R>(sm + p * pstride_e, dst, p, g.D, HW, g.W, rows_ok, off, wk, bb, aa, ab, ac);
        if (p + 1 >= g.D) break;
        dwb_conv_step<T, A, R>(sm + (p + 1) * pstride_e, dst, p + 1, g.D, HW, g.W, rows_ok, off, wk, bb, ab, ac, aa);
        if (p + 2 >= g.D) break;
        dwb_conv_step<T, A, R>(sm + (p + 2) * pstride_e, dst, p + 2, g.D, HW, g.W, rows_ok, off, wk, bb, ac, aa, ab);
      }
    }
    __syncthreads();   // every thread is done reading stage s before it is refilled
  }
  if (threadIdx.x == 0 && *abort_flag) ptx::report_device_timeout();
}

// One z step of the weight-gradient march over staged volumes: x plane p meets grad_out planes p+1 (kz=0),
// p (kz=1) and p-1 (kz=2).  ml / mr zero the clamped border columns.
template <typename T, typename A, int R>
__device__ __forceinline__ void dwb_wgrad_step(const T* xplane, const T* gs, int p, int D, int HW, int W,
                                               int rows_ok, const int (&off)[R + 2][3], A ml, A mr, A (&acc)[27],
                                               A (&gm1)[R], const A (&g0)[R], const A (&gp1)[R]) {
  A v[R + 2][3];
  dwb_plane<T, A, R>(xplane, off, v);
#pragma unroll
  for (int j = 0; j < R + 2; ++j) {
    v[j][0] *= ml;
    v[j][2] *= mr;
  }
#pragma unroll
  for (int ky = 0; ky < 3; ++ky)
#pragma unroll
    for (int kx = 0; kx < 3; ++kx)
#pragma unroll
      for (int r = 0; r < R; ++r) {
        acc[(0 * 3 + ky) * 3 + kx] += gp1[r] * v[r + ky][kx];
        acc[(1 * 3 + ky) * 3 + kx] += g0[r] * v[r + ky][kx];
        acc[(2 * 3 + ky) * 3 + kx] += gm1[r] * v[r + ky][kx];
      }
  // gm1 is dead now: it becomes grad_out plane p+2 for the next step
#pragma unroll
  for (int r = 0; r < R; ++r)
    gm1[r] = (p + 2 < D && r < rows_ok) ? dwb_cvt<T, A>(gs[(p + 2) * HW + r * W]) : (A)0;
}

// Block-wide sum of the 27 per-thread accumulators, one atomic per tap into partial[c][27]; clears acc.
template <typename A>
__device__ __forceinline__ void dwb_flush(A (&acc)[27], A* red, A* __restrict__ partial, int c) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll
  for (int t = 0; t < 27; ++t) {
    A sv = acc[t];
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) sv += __shfl_xor_sync(0xffffffffu, sv, o);
    if (lane == 0) red[warp * 27 + t] = sv;
    acc[t] = (A)0;
  }
  __syncthreads();
  if (threadIdx.x < 27) {
    A sv = (A)0;
    for (int wp = 0; wp < nwarps; ++wp) sv += red[wp * 27 + threadIdx.x];
    atomicAdd(partial + (long long)c * 27 + threadIdx.x, sv);
  }
  __syncthreads();
}

// Work items are (channel, clip) pairs, channel-major, so a block's contiguous range changes channel rarely;
// the 27 accumulators are flushed when it does.  Shared memory: [stage0: gapped x volume, grad_out volume]
// [stage1: ...][2 mbarriers][abort flag][reduction scratch 26 x 27].
template <typename T, typename A, int R>
__global__ void __launch_bounds__(kDwBulkWgradThreads, 1)
dw_bulk_wgrad_kernel(Geom g, int nyp, uint32_t plane_bytes, uint32_t gap_bytes, uint32_t stage_x_bytes,
                     uint32_t stage_bytes, const T* __restrict__ gy, const T* __restrict__ x,
                     A* __restrict__ partial) {
  extern __shared__ __align__(128) unsigned char dwb_smem[];
  const uint32_t bar0 = ptx::smem_u32(dwb_smem + 2 * (size_t)stage_bytes);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(dwb_smem + 2 * (size_t)stage_bytes + 16);
  A* red = reinterpret_cast<A*>(dwb_smem + 2 * (size_t)stage_bytes + 32);
  const long long items = (long long)g.Cin * g.B;
  const long long lo = items * blockIdx.x / gridDim.x, hi = items * (blockIdx.x + 1) / gridDim.x;
  const int HW = g.H * g.W;
  const uint32_t pstride = plane_bytes + gap_bytes, vol_bytes = (uint32_t)g.D * plane_bytes;
  if (threadIdx.x == 0) {
    ptx::mbar_init(bar0, 1);
    ptx::mbar_init(bar0 + 8, 1);
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  dwb_zero_gaps(dwb_smem, stage_bytes, plane_bytes, gap_bytes, g.D);
  const unsigned char* xb = reinterpret_cast<const unsigned char*>(x);
  const unsigned char* gb = reinterpret_cast<const unsigned char*>(gy);
  auto issue = [&](long long item, int s) {
    const long long c = item / g.B, b = item - c * g.B;
    const long long voff = (b * g.Cin + c) * (long long)vol_bytes;
    const uint32_t bar = bar0 + 8 * s;
    ptx::mbar_arrive_expect_tx(bar, 2 * vol_bytes);
    const uint32_t dst = ptx::smem_u32(dwb_smem + (size_t)s * stage_bytes);
    for (int k = 0; k < g.D; ++k)
      ptx::bulk_g2s(dst + gap_bytes + k * pstride, xb + voff + (size_t)k * plane_bytes, plane_bytes, bar);
    ptx::bulk_g2s(dst + stage_x_bytes, gb + voff, vol_bytes, bar);
  };
  if (threadIdx.x == 0 && lo < hi) issue(lo, 0);
  const int ncol = nyp * g.W, pstride_e = (int)(pstride / sizeof(T));
  A acc[27];
#pragma unroll
  for (int t = 0; t < 27; ++t) acc[t] = (A)0;
  int it = 0;
  bool ok = true;
  for (long long item = lo; item < hi; ++item, ++it) {
    const int s = it & 1;
    if (threadIdx.x == 0 && item + 1 < hi) issue(item + 1, s ^ 1);
    if (!ptx::mbar_wait(bar0 + 8 * s, (it >> 1) & 1, abort_flag)) { ok = false; break; }
    const T* xs = reinterpret_cast<const T*>(dwb_smem + (size_t)s * stage_bytes + gap_bytes);
    const T* gs0 = reinterpret_cast<const T*>(dwb_smem + (size_t)s * stage_bytes + stage_x_bytes);
    for (int col = threadIdx.x; col < ncol; col += blockDim.x) {
      const int yp = col / g.W, xx = col - yp * g.W, y0 = yp * R;
      const A ml = xx > 0 ? (A)1 : (A)0, mr = xx < g.W - 1 ? (A)1 : (A)0;
      int off[R + 2][3];
      dwb_offsets<R>(y0, xx, g.H, g.W, off);
      const int rows_ok = min(R, g.H - y0);
      const T* gs = gs0 + y0 * g.W + xx;
      A ga[R], gbv[R], gc[R];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        ga[r] = (A)0;
        gbv[r] = r < rows_ok ? dwb_cvt<T, A>(gs[r * g.W]) : (A)0;
        gc[r] = (r < rows_ok && g.D > 1) ? dwb_cvt<T, A>(gs[HW + r * g.W]) : (A)0;
      }
      for (int p = 0; p < g.D; p += 3) {
        dwb_wgrad_step<T, A, R>(xs + p * pstride_e, gs, p, g.D, HW, g.W, rows_ok, off, ml, mr, acc, ga, gbv, gc);
        if (p + 1 >= g.D) break;
        dwb_wgrad_step<T, A, R>(xs + (p + 1) * pstride_e, gs, p + 1, g.D, HW, g.W, rows_ok, off, ml, mr, acc, gbv,
                                gc, ga);
        if (p + 2 >= g.D) break;
        dwb_wgrad_step<T, A, R>(xs + (p + 2) * pstride_e, gs, p + 2, g.D, HW, g.W, rows_ok, off, ml, mr, acc, gc,
                                ga, gbv);
      }
    }
    const long long c = item / g.B;
    if (item + 1 == hi || (item + 1) / g.B != c)
      dwb_flush<A>(acc, red, partial, (int)c);   // ends with a block barrier
    else
      __syncthreads();   // every thread is done reading stage s before it is refilled
  }
  if (threadIdx.x == 0 && (!ok || *abort_flag)) ptx::report_device_timeout();
}

template <typename T, typename A>
int dw_bulk_conv(const Geom& g, const DwTilePlan& tp, const DwBulkPlan& p, const T* in, const T* w, const T* bias,
                 T* out, int flip, cudaStream_t st) {
  D2C_CUDA_TRY(cudaFuncSetAttribute(dw_bulk_conv_kernel<T, A, kDwRows>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)p.smem));
  dw_bulk_conv_kernel<T, A, kDwRows><<<p.blocks, p.threads, p.smem, st>>>(
      g, tp.nyp, p.nvol, p.nchunks, p.plane_bytes, p.gap_bytes, p.stage_bytes, in, w, bias, out, flip);
  D2C_LAUNCH_CHECK();
  return D2C_OK;
}

template <typename T, typename A>
int dw_bulk_wgrad(const Geom& g, const DwTilePlan& tp, const DwBulkPlan& p, const T* gy, const T* x, A* partial,
                  cudaStream_t st) {
  const size_t smem = p.smem + (kDwBulkWgradThreads / 32) * 27 * sizeof(A);
  D2C_CUDA_TRY(cudaFuncSetAttribute(dw_bulk_wgrad_kernel<T, A, kDwRows>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)smem));
  dw_bulk_wgrad_kernel<T, A, kDwRows><<<p.blocks, p.threads, smem, st>>>(
      g, tp.nyp, p.plane_bytes, p.gap_bytes, p.stage_x_bytes, p.stage_bytes, gy, x, partial);
  D2C_LAUNCH_CHECK();
  return D2C_OK;
}

}  // namespace
}  // namespace d2c
