// Channel-separated (depthwise, optional channel multiplier) conv3d: forward,
// input gradient, weight gradient, bias gradient.  HBM-bound: 2 tensors of B*C*V
// elements move per pass while each output needs only 27 MACs.
//
// Stands in for the kernels of the reference's fast_depthwise_conv3d extension
// (csrc/grouped_conv3d.cu:22-91 forward, :93-174 input gradient, :176-276 weight
// gradient, :609 bias gradient).
#include <cuda_fp16.h>

#include <mutex>

#include "d2c_common.cuh"
#include "depthwise_quad.cuh"
#include "depthwise_tile.cuh"

namespace d2c {

template <typename T> struct AccOf { using type = T; };
template <> struct AccOf<__half> { using type = float; };

template <typename T> __device__ __forceinline__ typename AccOf<T>::type ld(const T* p) { return __ldg(p); }
template <> __device__ __forceinline__ float ld<__half>(const __half* p) { return __half2float(__ldg(p)); }
template <typename T, typename A> __device__ __forceinline__ T cvt(A a) { return (T)a; }
template <> __device__ __forceinline__ __half cvt<__half, float>(float a) { return __float2half_rn(a); }

// ---- forward -----------------------------------------------------------------------------------
// Thread per output element, x fastest: neighbouring threads read neighbouring
// input addresses, so the 27 taps of a warp are served from L1 after the first
// touch and DRAM sees each input line about once.
template <typename T, int KD, int KH, int KW>
__global__ void __launch_bounds__(256)
dw_fwd_kernel(Geom g, const T* __restrict__ x, const T* __restrict__ w, const T* __restrict__ bias,
              T* __restrict__ y) {
  using A = typename AccOf<T>::type;
  const int kd = KD > 0 ? KD : g.kd, kh = KH > 0 ? KH : g.kh, kw = KW > 0 ? KW : g.kw;
  const int mult = g.Cout / g.Cin;
  const long long total = (long long)g.B * g.Cout * g.V;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int ow = (int)(idx % g.Wo);
    const int oh = (int)((idx / g.Wo) % g.Ho);
    const int ot = (int)((idx / ((long long)g.Wo * g.Ho)) % g.Do);
    const int oc = (int)((idx / g.V) % g.Cout);
    const int b = (int)(idx / ((long long)g.V * g.Cout));
    const T* in = x + ((long long)b * g.Cin + oc / mult) * g.Vin;
    const T* kp = w + (long long)oc * g.K;
    const int t0 = ot * g.sd - g.pd, h0 = oh * g.sh - g.ph, w0 = ow * g.sw - g.pw;
    A sum = 0;
#pragma unroll
    for (int kf = 0; kf < kd; ++kf) {
      const int it = t0 + kf * g.dd;
#pragma unroll
      for (int kr = 0; kr < kh; ++kr) {
        const int ih = h0 + kr * g.dh;
#pragma unroll
        for (int kc = 0; kc < kw; ++kc) {
          const int iw = w0 + kc * g.dw;
          const A op1 = ld(kp + (kf * kh + kr) * kw + kc);
          if (it >= 0 && ih >= 0 && iw >= 0 && it < g.D && ih < g.H && iw < g.W)
            sum += op1 * ld(in + ((long long)it * g.H + ih) * g.W + iw);
        }
      }
    }
    if (bias) sum += ld(bias + oc);
    y[idx] = cvt<T, A>(sum);
  }
}

// ---- input gradient (gather form; stride handled by a divisibility test) --------------------------
template <typename T, int KD, int KH, int KW>
__global__ void __launch_bounds__(256)
dw_bwd_input_kernel(Geom g, const T* __restrict__ gy, const T* __restrict__ w, T* __restrict__ gx) {
  using A = typename AccOf<T>::type;
  const int kd = KD > 0 ? KD : g.kd, kh = KH > 0 ? KH : g.kh, kw = KW > 0 ? KW : g.kw;
  const int mult = g.Cout / g.Cin;
  const long long total = (long long)g.B * g.Cin * g.Vin;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int iw = (int)(idx % g.W);
    const int ih = (int)((idx / g.W) % g.H);
    const int it = (int)((idx / ((long long)g.W * g.H)) % g.D);
    const int ic = (int)((idx / g.Vin) % g.Cin);
    const int b = (int)(idx / (g.Vin * g.Cin));
    A sum = 0;
    for (int oc = ic * mult; oc < (ic + 1) * mult; ++oc) {
      const T* go = gy + ((long long)b * g.Cout + oc) * g.V;
      const T* kp = w + (long long)oc * g.K;
#pragma unroll
      for (int kf = 0; kf < kd; ++kf) {
        const int raw_t = it + g.pd - kf * g.dd, ot = raw_t / g.sd;
#pragma unroll
        for (int kr = 0; kr < kh; ++kr) {
          const int raw_h = ih + g.ph - kr * g.dh, oh = raw_h / g.sh;
#pragma unroll
          for (int kc = 0; kc < kw; ++kc) {
            const int raw_w = iw + g.pw - kc * g.dw, ow = raw_w / g.sw;
            const A op1 = ld(kp + (kf * kh + kr) * kw + kc);
            if (raw_t >= 0 && raw_h >= 0 && raw_w >= 0 && ot < g.Do && oh < g.Ho && ow < g.Wo &&
                ot * g.sd == raw_t && oh * g.sh == raw_h && ow * g.sw == raw_w)
              sum += op1 * ld(go + ((long long)ot * g.Ho + oh) * g.Wo + ow);
          }
        }
      }
    }
    gx[idx] = cvt<T, A>(sum);
  }
}

// ---- weight gradient ------------------------------------------------------------------------------
// One block per (output channel, slice of clips): every thread keeps all K partial
// sums for the voxels it visits (grad_out is read once, the K input neighbours come
// from L1), then the block reduces K values.  Slices accumulate with fp32/fp64
// atomics into `partial` ([Cout, K] in the accumulator type, zeroed beforehand);
// a tiny second kernel converts to T.

template <typename T, int KD, int KH, int KW>
__global__ void __launch_bounds__(256)
dw_bwd_weight_kernel(Geom g, int clips_per_block, const T* __restrict__ gy, const T* __restrict__ x,
                     typename AccOf<T>::type* __restrict__ partial) {
  using A = typename AccOf<T>::type;
  constexpr int K = KD * KH * KW;
  const int mult = g.Cout / g.Cin;
  const int oc = blockIdx.x, ic = oc / mult;
  const int bbeg = blockIdx.y * clips_per_block, bend = min(g.B, bbeg + clips_per_block);
  A acc[K];
#pragma unroll
  for (int t = 0; t < K; ++t) acc[t] = 0;
  for (int b = bbeg; b < bend; ++b) {
    const T* go = gy + ((long long)b * g.Cout + oc) * g.V;
    const T* in = x + ((long long)b * g.Cin + ic) * g.Vin;
    for (int v = threadIdx.x; v < g.V; v += blockDim.x) {
      const int ow = v % g.Wo, oh = (v / g.Wo) % g.Ho, ot = v / (g.Wo * g.Ho);
      const A op1 = ld(go + v);
      const int t0 = ot * g.sd - g.pd, h0 = oh * g.sh - g.ph, w0 = ow * g.sw - g.pw;
#pragma unroll
      for (int kf = 0; kf < KD; ++kf) {
        const int it = t0 + kf * g.dd;
#pragma unroll
        for (int kr = 0; kr < KH; ++kr) {
          const int ih = h0 + kr * g.dh;
#pragma unroll
          for (int kc = 0; kc < KW; ++kc) {
            const int iw = w0 + kc * g.dw;
            if (it >= 0 && ih >= 0 && iw >= 0 && it < g.D && ih < g.H && iw < g.W)
              acc[(kf * KH + kr) * KW + kc] += op1 * ld(in + ((long long)it * g.H + ih) * g.W + iw);
          }
        }
      }
    }
  }
  __shared__ A red[8][K];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
  for (int t = 0; t < K; ++t) {
    A s = acc[t];
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if (lane == 0) red[warp][t] = s;
  }
  __syncthreads();
  if (threadIdx.x < K) {
    A s = 0;
#pragma unroll
    for (int wp = 0; wp < 8; ++wp) s += red[wp][threadIdx.x];
    atomicAdd(partial + (long long)oc * K + threadIdx.x, s);
  }
}

// Any kernel shape: one block per (output channel, tap), as the reference lays it out.
template <typename T>
__global__ void __launch_bounds__(256)
dw_bwd_weight_any_kernel(Geom g, const T* __restrict__ gy, const T* __restrict__ x,
                         typename AccOf<T>::type* __restrict__ partial) {
  using A = typename AccOf<T>::type;
  const int mult = g.Cout / g.Cin;
  const int tap = blockIdx.x % g.K, oc = blockIdx.x / g.K, ic = oc / mult;
  const int kc = tap % g.kw, kr = (tap / g.kw) % g.kh, kf = tap / (g.kw * g.kh);
  A s = 0;
  for (int b = 0; b < g.B; ++b) {
    const T* go = gy + ((long long)b * g.Cout + oc) * g.V;
    const T* in = x + ((long long)b * g.Cin + ic) * g.Vin;
    for (int v = threadIdx.x; v < g.V; v += blockDim.x) {
      const int ow = v % g.Wo, oh = (v / g.Wo) % g.Ho, ot = v / (g.Wo * g.Ho);
      const int it = ot * g.sd - g.pd + kf * g.dd, ih = oh * g.sh - g.ph + kr * g.dh,
                iw = ow * g.sw - g.pw + kc * g.dw;
      if (it >= 0 && ih >= 0 && iw >= 0 && it < g.D && ih < g.H && iw < g.W)
        s += ld(go + v) * ld(in + ((long long)it * g.H + ih) * g.W + iw);
    }
  }
  __shared__ A red[256];
  red[threadIdx.x] = s;
  __syncthreads();
  for (int i = 128; i >= 1; i >>= 1) {
    if ((int)threadIdx.x < i) red[threadIdx.x] += red[threadIdx.x + i];
    __syncthreads();
  }
  if (threadIdx.x == 0) partial[(long long)oc * g.K + tap] = red[0];
}

template <typename T>
__global__ void dw_cast_kernel(long long n, const typename AccOf<T>::type* __restrict__ src,
                               T* __restrict__ dst) {
  using A = typename AccOf<T>::type;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
       i += (long long)gridDim.x * blockDim.x)
    dst[i] = cvt<T, A>(src[i]);
}

template <typename T>
__global__ void __launch_bounds__(256)
dw_grad_bias_kernel(int B, int Cout, int V, const T* __restrict__ gy, T* __restrict__ grad_bias) {
  using A = typename AccOf<T>::type;
  __shared__ A red[256];
  const int co = blockIdx.x;
  A s = 0;
  for (int b = 0; b < B; ++b) {
    const T* p = gy + ((long long)b * Cout + co) * V;
    for (int v = threadIdx.x; v < V; v += blockDim.x) s += ld(p + v);
  }
  red[threadIdx.x] = s;
  __syncthreads();
  for (int i = 128; i >= 1; i >>= 1) {
    if ((int)threadIdx.x < i) red[threadIdx.x] += red[threadIdx.x + i];
    __syncthreads();
  }
  if (threadIdx.x == 0) grad_bias[co] = cvt<T, A>(red[0]);
}

static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static unsigned blocks_for(long long total) {
  long long n = (total + 255) / 256;
  const long long cap = 148LL * 32;
  return (unsigned)(n < 1 ? 1 : (n > cap ? cap : n));
}

// fp32, even W: the packed-FMA kernels.  Returns false when they do not apply (then *rc is untouched).
template <typename T>
static bool quad_conv(const Geom& g, const void* in, const void* w, const void* bias, void* out, int flip,
                      cudaStream_t st, int* rc) {
  if constexpr (std::is_same<T, float>::value) {
    DwQuadPlan qp;
    if (!aligned16(in) || !aligned16(out) || !dw_quad_plan(g, 1, &qp)) return false;
    *rc = dw_quad_conv(g, qp, (const float*)in, (const float*)w, (const float*)bias, (float*)out, flip, st);
    return true;
  }
  return false;
}

template <typename T>
static bool quad_wgrad(const Geom& g, const void* gy, const void* x, void* partial, cudaStream_t st, int* rc) {
  if constexpr (std::is_same<T, float>::value) {
    DwQuadPlan qp;
    if (!aligned16(gy) || !aligned16(x) || !dw_quad_plan(g, 2, &qp)) return false;
    *rc = dw_quad_wgrad(g, qp, (const float*)gy, (const float*)x, (float*)partial, st);
    return true;
  }
  return false;
}

template <typename T>
static int dw_fwd_t(const Geom& g, const void* x, const void* w, const void* bias, void* y, cudaStream_t st) {
  const long long total = (long long)g.B * g.Cout * g.V;
  ptx::bind_status_sink();
  prof_mark(st, "depthwise_fwd");
  DwTilePlan plan;
  if (dw_tile_plan(g, sizeof(typename AccOf<T>::type), &plan)) {
    using A = typename AccOf<T>::type;
    DwBulkPlan bulk;
    int rc;
    if (quad_conv<T>(g, x, w, bias, y, 0, st, &rc)) {
    } else if (aligned16(x) && dw_bulk_plan(g, sizeof(T), 1, plan, &bulk)) {
      rc = dw_bulk_conv<T, A>(g, plan, bulk, (const T*)x, (const T*)w, (const T*)bias, (T*)y, 0, st);
    } else {
      rc = dw_tile_conv<T, A>(g, plan, (const T*)x, (const T*)w, (const T*)bias, (T*)y, 0, st);
    }
    prof_mark(st, nullptr);
    return rc;
  }
  if (g.kd == 3 && g.kh == 3 && g.kw == 3)
    dw_fwd_kernel<T, 3, 3, 3><<<blocks_for(total), 256, 0, st>>>(g, (const T*)x, (const T*)w, (const T*)bias, (T*)y);
  else
    dw_fwd_kernel<T, 0, 0, 0><<<blocks_for(total), 256, 0, st>>>(g, (const T*)x, (const T*)w, (const T*)bias, (T*)y);
  D2C_LAUNCH_CHECK();
  prof_mark(st, nullptr);
  return D2C_OK;
}

template <typename T>
static int dw_bwd_t(const Geom& g, const void* gy, const void* x, const void* w, void* gx, void* gw,
                    void* gbias, void* ws, cudaStream_t st) {
  using A = typename AccOf<T>::type;
  const bool k333 = g.kd == 3 && g.kh == 3 && g.kw == 3;
  DwTilePlan plan;
  const bool tiled = dw_tile_plan(g, sizeof(A), &plan);
  ptx::bind_status_sink();
  if (gx) {
    const long long total = (long long)g.B * g.Cin * g.Vin;
    prof_mark(st, "depthwise_bwd_input");
    if (tiled) {
      // grad_x = correlation of grad_out with the point-reflected kernel
      DwBulkPlan bulk;
      int rc;
      if (quad_conv<T>(g, gy, w, nullptr, gx, 1, st, &rc)) {
      } else if (aligned16(gy) && dw_bulk_plan(g, sizeof(T), 1, plan, &bulk)) {
        rc = dw_bulk_conv<T, A>(g, plan, bulk, (const T*)gy, (const T*)w, (const T*)nullptr, (T*)gx, 1, st);
      } else {
        rc = dw_tile_conv<T, A>(g, plan, (const T*)gy, (const T*)w, (const T*)nullptr, (T*)gx, 1, st);
      }
      if (rc) return rc;
    } else if (k333)
      dw_bwd_input_kernel<T, 3, 3, 3><<<blocks_for(total), 256, 0, st>>>(g, (const T*)gy, (const T*)w, (T*)gx);
    else
      dw_bwd_input_kernel<T, 0, 0, 0><<<blocks_for(total), 256, 0, st>>>(g, (const T*)gy, (const T*)w, (T*)gx);
    D2C_LAUNCH_CHECK();
  }
  if (gw) {
    A* partial = (A*)ws;
    const long long n = (long long)g.Cout * g.K;
    prof_mark(st, "depthwise_bwd_weight");
    if (tiled) {
      D2C_CUDA_TRY(cudaMemsetAsync(partial, 0, sizeof(A) * (size_t)n, st));
      DwBulkPlan bulk;
      int rc;
      if (quad_wgrad<T>(g, gy, x, partial, st, &rc)) {
      } else if (aligned16(gy) && aligned16(x) && dw_bulk_plan(g, sizeof(T), 2, plan, &bulk)) {
        rc = dw_bulk_wgrad<T, A>(g, plan, bulk, (const T*)gy, (const T*)x, partial, st);
      } else {
        rc = dw_tile_wgrad<T, A>(g, plan, (const T*)gy, (const T*)x, partial, st);
      }
      if (rc) return rc;
    } else if (k333) {
      D2C_CUDA_TRY(cudaMemsetAsync(partial, 0, sizeof(A) * (size_t)n, st));
      // enough (channel, clip-slice) blocks to fill the GPU a few times over
      int slices = (148 * 8 + g.Cout - 1) / g.Cout;
      if (slices > g.B) slices = g.B;
      if (slices < 1) slices = 1;
      const int cpb = (g.B + slices - 1) / slices;
      dim3 grid(g.Cout, (g.B + cpb - 1) / cpb);
      dw_bwd_weight_kernel<T, 3, 3, 3><<<grid, 256, 0, st>>>(g, cpb, (const T*)gy, (const T*)x, partial);
    } else {
      dw_bwd_weight_any_kernel<T><<<(unsigned)n, 256, 0, st>>>(g, (const T*)gy, (const T*)x, partial);
    }
    D2C_LAUNCH_CHECK();
    dw_cast_kernel<T><<<blocks_for(n), 256, 0, st>>>(n, partial, (T*)gw);
    D2C_LAUNCH_CHECK();
  }
  if (gbias) {
    prof_mark(st, "depthwise_bwd_bias");
    dw_grad_bias_kernel<T><<<g.Cout, 256, 0, st>>>(g.B, g.Cout, g.V, (const T*)gy, (T*)gbias);
    D2C_LAUNCH_CHECK();
  }
  prof_mark(st, nullptr);
  return D2C_OK;
}

size_t depthwise_bwd_workspace(const Geom& g) { return align_up(sizeof(double) * (size_t)g.Cout * g.K, 256); }

int depthwise_fwd(const Geom& g, int dtype, const void* x, const void* w, const void* bias, void* y,
                  cudaStream_t st) {
  switch (dtype) {
    case D2C_F32: return dw_fwd_t<float>(g, x, w, bias, y, st);
    case D2C_F64: return dw_fwd_t<double>(g, x, w, bias, y, st);
    case D2C_F16: return dw_fwd_t<__half>(g, x, w, bias, y, st);
    default: return D2C_ERR_DTYPE;
  }
}

int depthwise_bwd(const Geom& g, int dtype, const void* gy, const void* x, const void* w, void* gx,
                  void* gw, void* gbias, void* ws, cudaStream_t st) {
  switch (dtype) {
    case D2C_F32: return dw_bwd_t<float>(g, gy, x, w, gx, gw, gbias, ws, st);
    case D2C_F64: return dw_bwd_t<double>(g, gy, x, w, gx, gw, gbias, ws, st);
    case D2C_F16: return dw_bwd_t<__half>(g, gy, x, w, gx, gw, gbias, ws, st);
    default: return D2C_ERR_DTYPE;
  }
}

// ---- depthwise backward without any device allocation -----------------------------------------------
//
// Some users of this C ABI cannot hand the library a workspace: a host program that sizes all of its
// device memory once at start-up and then runs under a fixed budget (a serving process that shares the
// GPU with other tenants, an embedded pipeline with a static memory plan) has nothing left to allocate
// from, and a latency-critical loop cannot afford cudaMalloc/cudaFree at all because they synchronise the
// whole device.  For those callers the weight-gradient accumulators of the depthwise backward live in
// the fixed array below instead of a caller-supplied workspace.
//
// The array is part of the library image: every GPU that loads libd2conv3d.so holds these 256 KB from
// load until the process exits.  All calls on a device share it and it keeps the last call's contents, so
// (a) the kernels' launch sequence clears it on the stream before accumulating and (b) two calls whose
// GPU work overlaps (different streams, or host threads racing on one device) corrupt each other.
constexpr size_t kNoAllocScratchElems = 32768;   // accumulator slots: out_channels * kd*kh*kw must fit
static __device__ __align__(256) double g_dw_noalloc_scratch[kNoAllocScratchElems];

constexpr int kMaxDevices = 64;
static void* g_dw_noalloc_ptr[kMaxDevices];      // device address of the array, per device (0 = not set up)
static std::mutex g_dw_noalloc_mu;

// In host code the array's name is only a handle; the address a kernel can use has to be asked for,
// per device, with that device current.
static int dw_noalloc_scratch(void** out) {
  int dev = -1;
  D2C_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return D2C_ERR_TOO_LARGE;
  std::lock_guard<std::mutex> lk(g_dw_noalloc_mu);
  if (!g_dw_noalloc_ptr[dev]) {
    void* ptr = nullptr;
    D2C_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_dw_noalloc_scratch));
    g_dw_noalloc_ptr[dev] = ptr;
  }
  *out = g_dw_noalloc_ptr[dev];
  return D2C_OK;
}

}  // namespace d2c

extern "C" int d2c_depthwise_conv3d_bwd_noalloc(const d2c_conv_desc* desc, const void* grad_y, const void* x,
                                                const void* w, void* grad_x, void* grad_w, void* grad_bias,
                                                d2c_stream_t stream) {
  using namespace d2c;
  if (!desc || !grad_y || !x || !w) return D2C_ERR_NULL;
  Geom g;
  int rc = make_geom(desc, &g, true);
  if (rc) return rc;
  if ((long long)g.B * g.Cin * g.Vin > 0x7fffffffLL || (long long)g.B * g.Cout * g.V > 0x7fffffffLL)
    return D2C_ERR_TOO_LARGE;
  if (grad_w && (size_t)g.Cout * g.K > kNoAllocScratchElems) return D2C_ERR_SCRATCH_LIMIT;
  void* scratch = nullptr;
  if ((rc = dw_noalloc_scratch(&scratch))) return rc;
  return depthwise_bwd(g, desc->dtype, grad_y, x, w, grad_x, grad_w, grad_bias, scratch, (cudaStream_t)stream);
}
