// Register-window kernels for the common depthwise case: 3x3x3 kernel, stride 1, dilation 1, padding 1,
// channel multiplier 1 (the ir-CSN bottleneck conv).
//
// The pass moves two (forward, input gradient) or three (weight gradient) tensors through HBM for 27 MACs
// per element, so the kernel has to stay close to "one instruction per MAC" to remain memory-bound.  A thread
// owns R vertically adjacent (y) columns at one x and marches along z: per z-plane it loads the (R+2) x 3
// neighbourhood of plane z+1 (lanes run along x, so the loads are coalesced and the x/y overlap between
// threads is served by L1), keeps planes z-1, z, z+1 in registers, and produces R outputs with 27*R FMAs.
// That is 3*(R+2)/R loads per output instead of 27, no shared memory and no integer division in the loop.
//   forward:         out = conv(x, w) + bias
//   input gradient:  grad_x = conv(grad_out, w point-reflected)        (same kernel, flip = 1)
//   weight gradient: dW[c, t] = sum_{b, v} grad_out[b, c, v] * x[b, c, v + delta_t]   (27 accumulators/thread)
// Reference: ops/fast-depthwise-conv3d/csrc/grouped_conv3d.cu:22-276.
#pragma once

#include "d2c_common.cuh"

namespace d2c {
namespace {

constexpr int kDwRows = 2;   // R: output rows per thread

struct DwTilePlan {
  int nyp;        // row groups per plane = ceil(H / R)
  int ncol;       // thread columns per (clip, channel) = nyp * W
};

inline bool dw_tile_plan(const Geom& g, size_t /*esize*/, DwTilePlan* p) {
  if (!(g.kd == 3 && g.kh == 3 && g.kw == 3 && g.sd == 1 && g.sh == 1 && g.sw == 1 && g.dd == 1 && g.dh == 1 &&
        g.dw == 1 && g.pd == 1 && g.ph == 1 && g.pw == 1 && g.Cout == g.Cin))
    return false;
  p->nyp = (g.H + kDwRows - 1) / kDwRows;
  p->ncol = p->nyp * g.W;
  if ((long long)g.B * g.Cin * p->ncol > 0x7fffffffLL) return false;
  return true;
}

template <typename T, typename A>
__device__ __forceinline__ A dwt_ld(const T* p);
template <> __device__ __forceinline__ float dwt_ld<float, float>(const float* p) { return __ldg(p); }
template <> __device__ __forceinline__ double dwt_ld<double, double>(const double* p) { return __ldg(p); }
template <> __device__ __forceinline__ float dwt_ld<__half, float>(const __half* p) { return __half2float(__ldg(p)); }
template <typename T, typename A> __device__ __forceinline__ T dwt_st(A a) { return (T)a; }
template <> __device__ __forceinline__ __half dwt_st<__half, float>(float a) { return __float2half_rn(a); }

// The (R+2) x 3 neighbourhood of one z-plane around rows [y0, y0+R) and column x; zero outside the plane.
// okmask bit (j*3+i) <-> row y0-1+j, column x-1+i readable.
template <typename T, typename A, int R>
__device__ __forceinline__ void dwt_load_plane(const T* __restrict__ p, int H_W_unused, int W, unsigned okmask,
                                               A (&v)[R + 2][3]) {
#pragma unroll
  for (int j = 0; j < R + 2; ++j)
#pragma unroll
    for (int i = 0; i < 3; ++i)
      v[j][i] = ((okmask >> (j * 3 + i)) & 1u) ? dwt_ld<T, A>(p + (j - 1) * W + (i - 1)) : (A)0;
}

template <int R>
__device__ __forceinline__ unsigned dwt_okmask(int y0, int x, int H, int W) {
  unsigned m = 0;
#pragma unroll
  for (int j = 0; j < R + 2; ++j)
#pragma unroll
    for (int i = 0; i < 3; ++i) {
      const int y = y0 - 1 + j, xx = x - 1 + i;
      if (y >= 0 && y < H && xx >= 0 && xx < W) m |= 1u << (j * 3 + i);
    }
  return m;
}

// One z step of the forward / input-gradient march: fetch plane z+1 into `nxt`, emit outputs of plane z.
template <typename T, typename A, int R>
__device__ __forceinline__ void dwt_conv_step(const Geom& g, const T* __restrict__ src, T* __restrict__ dst, int z,
                                              int y0, unsigned okmask, const A (&wk)[27], A bb,
                                              const A (&prv)[R + 2][3], const A (&cur)[R + 2][3],
                                              A (&nxt)[R + 2][3]) {
  const int HW = g.H * g.W;
  dwt_load_plane<T, A, R>(src + (long long)(z + 1) * HW, HW, g.W, (z + 1 < g.D) ? okmask : 0u, nxt);
  A acc[R];
#pragma unroll
  for (int r = 0; r < R; ++r) acc[r] = bb;
#pragma unroll
  for (int ky = 0; ky < 3; ++ky)
#pragma unroll
    for (int kx = 0; kx < 3; ++kx)
#pragma unroll
      for (int r = 0; r < R; ++r) {
        acc[r] += wk[(0 * 3 + ky) * 3 + kx] * prv[r + ky][kx];
        acc[r] += wk[(1 * 3 + ky) * 3 + kx] * cur[r + ky][kx];
        acc[r] += wk[(2 * 3 + ky) * 3 + kx] * nxt[r + ky][kx];
      }
#pragma unroll
  for (int r = 0; r < R; ++r)
    if (y0 + r < g.H) dst[(long long)z * HW + r * g.W] = dwt_st<T, A>(acc[r]);
}

template <typename T, typename A, int R>
__global__ void __launch_bounds__(256)
dw_march_conv_kernel(Geom g, int nyp, long long total, const T* __restrict__ in, const T* __restrict__ w,
                     const T* __restrict__ bias, T* __restrict__ out, int flip) {
  const long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const int x = (int)(idx % g.W);
  const long long t1 = idx / g.W;
  const int yp = (int)(t1 % nyp);
  const long long bc = t1 / nyp;
  const int c = (int)(bc % g.Cin), y0 = yp * R;
  A wk[27];
#pragma unroll
  for (int t = 0; t < 27; ++t) wk[t] = dwt_ld<T, A>(w + (long long)c * 27 + (flip ? 26 - t : t));
  const A bb = bias ? dwt_ld<T, A>(bias + c) : (A)0;
  const unsigned okmask = dwt_okmask<R>(y0, x, g.H, g.W);
  const T* src = in + bc * g.Vin + (long long)y0 * g.W + x;     // (z = 0, y0, x)
  T* dst = out + bc * g.Vin + (long long)y0 * g.W + x;
  A w0[R + 2][3], w1[R + 2][3], w2[R + 2][3];
#pragma unroll
  for (int j = 0; j < R + 2; ++j)
#pragma unroll
    for (int i = 0; i < 3; ++i) w0[j][i] = (A)0;
  dwt_load_plane<T, A, R>(src, 0, g.W, okmask, w1);
  for (int z = 0; z < g.D; z += 3) {
    dwt_conv_step<T, A, R>(g, src, dst, z, y0, okmask, wk, bb, w0, w1, w2);
    if (z + 1 >= g.D) break;
    dwt_conv_step<T, A, R>(g, src, dst, z + 1, y0, okmask, wk, bb, w1, w2, w0);
    if (z + 2 >= g.D) break;
    dwt_conv_step<T, A, R>(g, src, dst, z + 2, y0, okmask, wk, bb, w2, w0, w1);
  }
}

// One z step of the weight-gradient march: fetch x plane z+1 into `nxt`, accumulate plane z.
template <typename T, typename A, int R>
__device__ __forceinline__ void dwt_wgrad_step(const Geom& g, const T* __restrict__ xsrc, const T* __restrict__ gsrc,
                                               int z, int y0, unsigned okmask, A (&acc)[27],
                                               const A (&prv)[R + 2][3], const A (&cur)[R + 2][3],
                                               A (&nxt)[R + 2][3]) {
  const int HW = g.H * g.W;
  dwt_load_plane<T, A, R>(xsrc + (long long)(z + 1) * HW, HW, g.W, (z + 1 < g.D) ? okmask : 0u, nxt);
  A go[R];
#pragma unroll
  for (int r = 0; r < R; ++r) go[r] = (y0 + r < g.H) ? dwt_ld<T, A>(gsrc + (long long)z * HW + r * g.W) : (A)0;
#pragma unroll
  for (int ky = 0; ky < 3; ++ky)
#pragma unroll
    for (int kx = 0; kx < 3; ++kx)
#pragma unroll
      for (int r = 0; r < R; ++r) {
        acc[(0 * 3 + ky) * 3 + kx] += go[r] * prv[r + ky][kx];
        acc[(1 * 3 + ky) * 3 + kx] += go[r] * cur[r + ky][kx];
        acc[(2 * 3 + ky) * 3 + kx] += go[r] * nxt[r + ky][kx];
      }
}

// One block per (channel, slice of clips): every thread keeps 27 partial sums over the columns it
// marches, the block reduces them and issues one atomic per tap into partial[Cout][27] (accumulator type,
// zeroed beforehand).
template <typename T, typename A, int R>
__global__ void __launch_bounds__(256)
dw_march_wgrad_kernel(Geom g, int nyp, int clips_per_block, const T* __restrict__ gy, const T* __restrict__ x,
                      A* __restrict__ partial) {
  __shared__ A red[8 * 27];
  const int c = blockIdx.x, ncol = nyp * g.W;
  const int bbeg = blockIdx.y * clips_per_block, bend = min(g.B, bbeg + clips_per_block);
  A acc[27];
#pragma unroll
  for (int t = 0; t < 27; ++t) acc[t] = (A)0;
  for (int b = bbeg; b < bend; ++b) {
    const long long plane = ((long long)b * g.Cin + c) * g.Vin;
    for (int col = threadIdx.x; col < ncol; col += blockDim.x) {
      const int yp = col / g.W, xx = col - yp * g.W, y0 = yp * R;
      const unsigned okmask = dwt_okmask<R>(y0, xx, g.H, g.W);
      const T* xsrc = x + plane + (long long)y0 * g.W + xx;
      const T* gsrc = gy + plane + (long long)y0 * g.W + xx;
      A w0[R + 2][3], w1[R + 2][3], w2[R + 2][3];
#pragma unroll
      for (int j = 0; j < R + 2; ++j)
#pragma unroll
        for (int i = 0; i < 3; ++i) w0[j][i] = (A)0;
      dwt_load_plane<T, A, R>(xsrc, 0, g.W, okmask, w1);
      for (int z = 0; z < g.D; z += 3) {
        dwt_wgrad_step<T, A, R>(g, xsrc, gsrc, z, y0, okmask, acc, w0, w1, w2);
        if (z + 1 >= g.D) break;
        dwt_wgrad_step<T, A, R>(g, xsrc, gsrc, z + 1, y0, okmask, acc, w1, w2, w0);
        if (z + 2 >= g.D) break;
        dwt_wgrad_step<T, A, R>(g, xsrc, gsrc, z + 2, y0, okmask, acc, w2, w0, w1);
      }
    }
  }
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int t = 0; t < 27; ++t) {
    A sv = acc[t];
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) sv += __shfl_xor_sync(0xffffffffu, sv, o);
    if (lane == 0) red[warp * 27 + t] = sv;
  }
  __syncthreads();
  if (threadIdx.x < 27) {
    A sv = (A)0;
    for (int wp = 0; wp < (int)(blockDim.x >> 5); ++wp) sv += red[wp * 27 + threadIdx.x];
    atomicAdd(partial + (long long)c * 27 + threadIdx.x, sv);
  }
}

template <typename T, typename A>
int dw_tile_conv(const Geom& g, const DwTilePlan& p, const T* in, const T* w, const T* bias, T* out, int flip,
                 cudaStream_t st) {
  const long long total = (long long)g.B * g.Cin * p.ncol;
  const unsigned blocks = (unsigned)((total + 255) / 256);
  dw_march_conv_kernel<T, A, kDwRows><<<blocks, 256, 0, st>>>(g, p.nyp, total, in, w, bias, out, flip);
  D2C_LAUNCH_CHECK();
  return D2C_OK;
}

template <typename T, typename A>
int dw_tile_wgrad(const Geom& g, const DwTilePlan& p, const T* gy, const T* x, A* partial, cudaStream_t st) {
  // enough (channel, clip-slice) blocks for a few waves
  long long slices = (148LL * 8 + g.Cin - 1) / g.Cin;
  if (slices > g.B) slices = g.B;
  if (slices < 1) slices = 1;
  if (slices > 65535) slices = 65535;
  const int cpb = (int)((g.B + slices - 1) / slices);
  // block size: the smallest multiple of 32 that covers the columns in the fewest passes of <= 256 threads
  const int passes = (p.ncol + 255) / 256;
  int threads = ((p.ncol + passes - 1) / passes + 31) / 32 * 32;
  if (threads > 256) threads = 256;
  dim3 grid((unsigned)g.Cin, (unsigned)((g.B + cpb - 1) / cpb));
  dw_march_wgrad_kernel<T, A, kDwRows><<<grid, threads, 0, st>>>(g, p.nyp, cpb, gy, x, partial);
  D2C_LAUNCH_CHECK();
  return D2C_OK;
}

}  // namespace
}  // namespace d2c
