// Bulk-copy pipelined kernels for the common depthwise case (3x3x3, stride 1, dilation 1, padding 1, channel
// multiplier 1) when whole (clip, channel) volumes fit in shared memory.
//
// In the [B][C][D][H][W] layout one (clip, channel) volume -- and any run of consecutive ones -- is a single
// contiguous byte range, so a persistent block streams its share of the tensor with untiled bulk async copies
// (cp.async.bulk global -> shared, completion on an mbarrier): one elected thread keeps the copy of chunk i+1
// in flight while all threads compute chunk i from shared memory.  That puts ~100 KB per SM in flight with no
// load instructions in the compute loop beyond shared-memory reads, which the register-window march kernels
// (depthwise_tile.cuh) cannot do: they stall on global-load latency at 25 % occupancy.
//
// Compute is the same z march: a thread owns R adjacent rows at one x, reads the (R+2) x 3 neighbourhood of
// each plane from shared memory once, and scatters it into the accumulators of output planes p-1, p, p+1.
// Borders are handled by a per-thread mask, so the staged volume carries no halo.
// Reference: ops/fast-depthwise-conv3d/csrc/grouped_conv3d.cu:22-276.
#pragma once

#include "depthwise_tile.cuh"
#include "sm100_ptx.cuh"

namespace d2c {
namespace {

__device__ int g_dw_status = 0;   // sticky: 1 after a bulk copy did not complete within the wait budget

struct DwBulkPlan {
  int nvol;               // volumes per chunk (forward / input gradient); 1 for the weight gradient
  long long nchunks;
  uint32_t chunk_bytes;   // bytes of one tensor's chunk
  int threads, blocks;
  size_t smem;
};

constexpr size_t kDwBulkSmemMax = 220 * 1024;

// tensors: how many tensors are staged per chunk (1: conv, 2: weight gradient).
inline bool dw_bulk_plan(const Geom& g, size_t esize, int tensors, const DwTilePlan& tp, DwBulkPlan* p) {
  const long long vols = (long long)g.B * g.Cin;
  const size_t vbytes = (size_t)g.Vin * esize;
  int n = 1;
  while (n <= 8 && (n * vbytes) % 16 != 0) n *= 2;
  if (n > 8 || vols % n != 0) return false;
  if (tensors == 1)
    while (n * vbytes < 24 * 1024 && vols % (2 * n) == 0 && vols / (2 * n) >= 148 * 4) n *= 2;
  else if (n != 1)
    return false;
  const size_t chunk = n * vbytes;
  const size_t need = 2 * tensors * chunk + 128;
  if (need > kDwBulkSmemMax || chunk > 0x7fffffffu) return false;
  p->nvol = n;
  p->nchunks = vols / n;
  p->chunk_bytes = (uint32_t)chunk;
  p->smem = need;
  const int per_sm = need <= 110 * 1024 ? 2 : 1;
  const long long cols = (long long)n * tp.ncol;
  int threads = per_sm == 2 ? 320 : 512;
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

// (R+2) x 3 neighbourhood of one staged plane around rows [y0, y0+R) and column x; zero outside the plane.
template <typename T, typename A, int R>
__device__ __forceinline__ void dwb_plane(const T* p, int W, unsigned okmask, A (&v)[R + 2][3]) {
#pragma unroll
  for (int j = 0; j < R + 2; ++j)
#pragma unroll
    for (int i = 0; i < 3; ++i)
      v[j][i] = ((okmask >> (j * 3 + i)) & 1u) ? dwb_cvt<T, A>(p[(j - 1) * W + (i - 1)]) : (A)0;
}

// One z step of the conv march over a staged volume: plane p feeds outputs p-1 (kz=2), p (kz=1), p+1 (kz=0).
template <typename T, typename A, int R>
__device__ __forceinline__ void dwb_conv_step(const Geom& g, const T* sm, T* __restrict__ dst, int p, int y0,
                                              unsigned okmask, const A (&wk)[27], A bb, A (&am1)[R], A (&a0)[R],
                                              A (&ap1)[R]) {
  const int HW = g.H * g.W;
  A v[R + 2][3];
  dwb_plane<T, A, R>(sm + p * HW, g.W, okmask, v);
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
    if (y0 + r < g.H) {
      if (p >= 1) dst[(long long)(p - 1) * HW + r * g.W] = dwt_st<T, A>(am1[r]);
      if (p == g.D - 1) dst[(long long)p * HW + r * g.W] = dwt_st<T, A>(a0[r]);
    }
}

// Shared memory: [stage 0 chunk][stage 1 chunk][2 mbarriers][abort flag].
template <typename T, typename A, int R>
__global__ void __launch_bounds__(512)
dw_bulk_conv_kernel(Geom g, int nyp, int nvol, long long nchunks, uint32_t chunk_bytes, const T* __restrict__ in,
                    const T* __restrict__ w, const T* __restrict__ bias, T* __restrict__ out, int flip) {
  extern __shared__ __align__(128) unsigned char dwb_smem[];
  const uint32_t bar0 = ptx::smem_u32(dwb_smem + 2 * (size_t)chunk_bytes);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(dwb_smem + 2 * (size_t)chunk_bytes + 16);
  const long long lo = nchunks * blockIdx.x / gridDim.x, hi = nchunks * (blockIdx.x + 1) / gridDim.x;
  if (threadIdx.x == 0) {
    ptx::mbar_init(bar0, 1);
    ptx::mbar_init(bar0 + 8, 1);
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  __syncthreads();
  const unsigned char* src_bytes = reinterpret_cast<const unsigned char*>(in);
  if (threadIdx.x == 0 && lo < hi) {
    ptx::mbar_arrive_expect_tx(bar0, chunk_bytes);
    ptx::bulk_g2s(ptx::smem_u32(dwb_smem), src_bytes + lo * (long long)chunk_bytes, chunk_bytes, bar0);
  }
  const int ncol = nyp * g.W, cols = nvol * ncol;
  int it = 0;
  for (long long ch = lo; ch < hi; ++ch, ++it) {
    const int s = it & 1;
    if (threadIdx.x == 0 && ch + 1 < hi) {   // stage s^1 was released by the barrier that ended iteration it-1
      const uint32_t bar = bar0 + 8 * (s ^ 1);
      ptx::mbar_arrive_expect_tx(bar, chunk_bytes);
      ptx::bulk_g2s(ptx::smem_u32(dwb_smem + (size_t)(s ^ 1) * chunk_bytes),
                    src_bytes + (ch + 1) * (long long)chunk_bytes, chunk_bytes, bar);
    }
    if (!ptx::mbar_wait(bar0 + 8 * s, (it >> 1) & 1, abort_flag)) break;
    const T* stage = reinterpret_cast<const T*>(dwb_smem + (size_t)s * chunk_bytes);
    for (int col = threadIdx.x; col < cols; col += blockDim.x) {
      const int vol = col / ncol, rem = col - vol * ncol;
      const int yp = rem / g.W, x = rem - yp * g.W, y0 = yp * R;
      const long long bc = ch * nvol + vol;
      const int c = (int)(bc % g.Cin);
      A wk[27];
#pragma unroll
      for (int t = 0; t < 27; ++t) wk[t] = dwt_ld<T, A>(w + (long long)c * 27 + (flip ? 26 - t : t));
      const A bb = bias ? dwt_ld<T, A>(bias + c) : (A)0;
      const unsigned okmask = dwt_okmask<R>(y0, x, g.H, g.W);
      const T* sm = stage + (long long)vol * g.Vin + y0 * g.W + x;
      T* dst = out + bc * g.Vin + (long long)y0 * g.W + x;
      A aa[R], ab[R], ac[R];
#pragma unroll
      for (int r = 0; r < R; ++r) aa[r] = ab[r] = ac[r] = bb;
      for (int p = 0; p < g.D; p += 3) {
        dwb_conv_step<T, A, R>(g, sm, dst, p, y0, okmask, wk, bb, aa, ab, ac);
        if (p + 1 >= g.D) break;
        dwb_conv_step<T, A, R>(g, sm, dst, p + 1, y0, okmask, wk, bb, ab, ac, aa);
        if (p + 2 >= g.D) break;
        dwb_conv_step<T, A, R>(g, sm, dst, p + 2, y0, okmask, wk, bb, ac, aa, ab);
      }
    }
    __syncthreads();   // every thread is done reading stage s before it is refilled
  }
  if (threadIdx.x == 0 && *abort_flag) atomicExch(&g_dw_status, 1);
}

// One z step of the weight-gradient march over staged volumes: x plane p meets grad_out planes p+1 (kz=0),
// p (kz=1) and p-1 (kz=2).
template <typename T, typename A, int R>
__device__ __forceinline__ void dwb_wgrad_step(const Geom& g, const T* xs, const T* gs, int p, int y0,
                                               unsigned okmask, A (&acc)[27], A (&gm1)[R], const A (&g0)[R],
                                               const A (&gp1)[R]) {
  const int HW = g.H * g.W;
  A v[R + 2][3];
  dwb_plane<T, A, R>(xs + p * HW, g.W, okmask, v);
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
    gm1[r] = (p + 2 < g.D && y0 + r < g.H) ? dwb_cvt<T, A>(gs[(p + 2) * HW + r * g.W]) : (A)0;
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
// the 27 accumulators are flushed when it does.  Shared memory: [stage0: x vol, gy vol][stage1: ...]
// [2 mbarriers][abort flag][reduction scratch 16 x 27].
template <typename T, typename A, int R>
__global__ void __launch_bounds__(512)
dw_bulk_wgrad_kernel(Geom g, int nyp, uint32_t vol_bytes, const T* __restrict__ gy, const T* __restrict__ x,
                     A* __restrict__ partial) {
  extern __shared__ __align__(128) unsigned char dwb_smem[];
  const size_t stage_bytes = 2 * (size_t)vol_bytes;
  const uint32_t bar0 = ptx::smem_u32(dwb_smem + 2 * stage_bytes);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(dwb_smem + 2 * stage_bytes + 16);
  A* red = reinterpret_cast<A*>(dwb_smem + 2 * stage_bytes + 32);
  const long long items = (long long)g.Cin * g.B;
  const long long lo = items * blockIdx.x / gridDim.x, hi = items * (blockIdx.x + 1) / gridDim.x;
  if (threadIdx.x == 0) {
    ptx::mbar_init(bar0, 1);
    ptx::mbar_init(bar0 + 8, 1);
    *abort_flag = 0;
    ptx::fence_mbar_init();
  }
  __syncthreads();
  const unsigned char* xb = reinterpret_cast<const unsigned char*>(x);
  const unsigned char* gb = reinterpret_cast<const unsigned char*>(gy);
  auto issue = [&](long long item, int s) {
    const long long c = item / g.B, b = item - c * g.B;
    const long long off = (b * g.Cin + c) * (long long)vol_bytes;
    const uint32_t bar = bar0 + 8 * s;
    ptx::mbar_arrive_expect_tx(bar, 2 * vol_bytes);
    ptx::bulk_g2s(ptx::smem_u32(dwb_smem + s * stage_bytes), xb + off, vol_bytes, bar);
    ptx::bulk_g2s(ptx::smem_u32(dwb_smem + s * stage_bytes + vol_bytes), gb + off, vol_bytes, bar);
  };
  if (threadIdx.x == 0 && lo < hi) issue(lo, 0);
  const int ncol = nyp * g.W, HW = g.H * g.W;
  A acc[27];
#pragma unroll
  for (int t = 0; t < 27; ++t) acc[t] = (A)0;
  int it = 0;
  bool ok = true;
  for (long long item = lo; item < hi; ++item, ++it) {
    const int s = it & 1;
    if (threadIdx.x == 0 && item + 1 < hi) issue(item + 1, s ^ 1);
    if (!ptx::mbar_wait(bar0 + 8 * s, (it >> 1) & 1, abort_flag)) { ok = false; break; }
    const T* xs0 = reinterpret_cast<const T*>(dwb_smem + s * stage_bytes);
    const T* gs0 = reinterpret_cast<const T*>(dwb_smem + s * stage_bytes + vol_bytes);
    for (int col = threadIdx.x; col < ncol; col += blockDim.x) {
      const int yp = col / g.W, xx = col - yp * g.W, y0 = yp * R;
      const unsigned okmask = dwt_okmask<R>(y0, xx, g.H, g.W);
      const T* xs = xs0 + y0 * g.W + xx;
      const T* gs = gs0 + y0 * g.W + xx;
      A ga[R], gbv[R], gc[R];
#pragma unroll
      for (int r = 0; r < R; ++r) {
        const bool rowok = y0 + r < g.H;
        ga[r] = (A)0;
        gbv[r] = rowok ? dwb_cvt<T, A>(gs[r * g.W]) : (A)0;
        gc[r] = (rowok && g.D > 1) ? dwb_cvt<T, A>(gs[HW + r * g.W]) : (A)0;
      }
      for (int p = 0; p < g.D; p += 3) {
        dwb_wgrad_step<T, A, R>(g, xs, gs, p, y0, okmask, acc, ga, gbv, gc);
        if (p + 1 >= g.D) break;
        dwb_wgrad_step<T, A, R>(g, xs, gs, p + 1, y0, okmask, acc, gbv, gc, ga);
        if (p + 2 >= g.D) break;
        dwb_wgrad_step<T, A, R>(g, xs, gs, p + 2, y0, okmask, acc, gc, ga, gbv);
      }
    }
    const long long c = item / g.B;
    if (item + 1 == hi || (item + 1) / g.B != c)
      dwb_flush<A>(acc, red, partial, (int)c);   // ends with a block barrier
    else
      __syncthreads();   // every thread is done reading stage s before it is refilled
  }
  if (threadIdx.x == 0 && (!ok || *abort_flag)) atomicExch(&g_dw_status, 1);
}

template <typename T, typename A>
int dw_bulk_conv(const Geom& g, const DwTilePlan& tp, const DwBulkPlan& p, const T* in, const T* w, const T* bias,
                 T* out, int flip, cudaStream_t st) {
  D2C_CUDA_TRY(cudaFuncSetAttribute(dw_bulk_conv_kernel<T, A, kDwRows>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)p.smem));
  dw_bulk_conv_kernel<T, A, kDwRows><<<p.blocks, p.threads, p.smem, st>>>(g, tp.nyp, p.nvol, p.nchunks,
                                                                           p.chunk_bytes, in, w, bias, out, flip);
  D2C_LAUNCH_CHECK();
  return D2C_OK;
}

template <typename T, typename A>
int dw_bulk_wgrad(const Geom& g, const DwTilePlan& tp, const DwBulkPlan& p, const T* gy, const T* x, A* partial,
                  cudaStream_t st) {
  const size_t smem = p.smem + 16 * 27 * sizeof(A);
  D2C_CUDA_TRY(cudaFuncSetAttribute(dw_bulk_wgrad_kernel<T, A, kDwRows>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                    (int)smem));
  dw_bulk_wgrad_kernel<T, A, kDwRows><<<p.blocks, p.threads, smem, st>>>(g, tp.nyp, p.chunk_bytes, gy, x, partial);
  D2C_LAUNCH_CHECK();
  return D2C_OK;
}

}  // namespace
}  // namespace d2c
