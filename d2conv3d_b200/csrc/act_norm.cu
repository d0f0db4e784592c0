// Fused activation + group normalisation, forward and backward: y = GroupNorm(relu(x)) for NCDHW fp32 tensors.
//
// The unit right after every convolution of the reference's refine blocks is `ActivationType(), NormType(planes)`
// with NormType = GroupNorm (network/modules/refinement.py:38-43; network/segmentation/encoder_decoder.py:116-119).
// With few groups and one clip per call a group is tens of millions of elements, which a one-block-per-group
// reduction turns into the dominant cost of decoder inference; here the moments are reduced by the whole grid
// (fp32 per thread, fp64 per block and across blocks) and the normalisation is a second streaming pass:
// x is read twice and y written once, all with 16-byte accesses.  HBM-bound: 3 * 4 bytes per element.
#include <cuda_runtime.h>

#include "d2c_common.cuh"

namespace d2c {
namespace {

// ws: [batch*groups][2] doubles = {sum, sum of squares}, zeroed before.
__global__ void __launch_bounds__(256)
act_moments_kernel(const float* __restrict__ x, long long group_elems, int apply_relu, int vec,
                   double* __restrict__ ws) {
  const long long bg = blockIdx.y;
  const float* p = x + bg * group_elems;
  const long long n4 = vec ? (group_elems >> 2) : 0;      // elements beyond 4*n4 are taken one by one below
  float s = 0.f, q = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 v = __ldg(reinterpret_cast<const float4*>(p) + i);
    if (apply_relu) { v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f); }
    s += (v.x + v.y) + (v.z + v.w);
    q += (v.x * v.x + v.y * v.y) + (v.z * v.z + v.w * v.w);
  }
  for (long long i = (n4 << 2) + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < group_elems;
       i += (long long)gridDim.x * blockDim.x) {
    float v = __ldg(p + i);
    if (apply_relu) v = fmaxf(v, 0.f);
    s += v; q += v * v;
  }
  double ds = s, dq = q;
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) {
    ds += __shfl_xor_sync(0xffffffffu, ds, o);
    dq += __shfl_xor_sync(0xffffffffu, dq, o);
  }
  __shared__ double red[2][8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { red[0][warp] = ds; red[1][warp] = dq; }
  __syncthreads();
  if (threadIdx.x == 0) {
    double a = 0, b = 0;
    for (int w = 0; w < 8; ++w) { a += red[0][w]; b += red[1][w]; }
    atomicAdd(ws + 2 * bg, a);
    atomicAdd(ws + 2 * bg + 1, b);
  }
}

// One block row per (clip, channel): y = (act(x) - mean) * rstd * gamma[c] + beta[c].
__global__ void __launch_bounds__(256)
act_normalize_kernel(const float* __restrict__ x, const float* __restrict__ gamma, const float* __restrict__ beta,
                     float* __restrict__ y, int channels, int cpg_norm, long long spatial, long long group_elems,
                     float eps, int apply_relu, int vec, const double* __restrict__ ws) {
  const long long bc = blockIdx.y;
  const int c = (int)(bc % channels);
  const long long bg = (bc / channels) * (channels / cpg_norm) + c / cpg_norm;
  const double mean = ws[2 * bg] / (double)group_elems;
  const double var = fmax(ws[2 * bg + 1] / (double)group_elems - mean * mean, 0.0);
  const float rstd = (float)(1.0 / sqrt(var + (double)eps));
  const float ga = gamma ? __ldg(gamma + c) : 1.f, be = beta ? __ldg(beta + c) : 0.f;
  const float a = rstd * ga, b = be - (float)mean * a;
  const float* px = x + bc * spatial;
  float* py = y + bc * spatial;
  if (vec) {
    const long long n4 = spatial >> 2;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
      float4 v = __ldg(reinterpret_cast<const float4*>(px) + i);
      if (apply_relu) { v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f); }
      reinterpret_cast<float4*>(py)[i] = make_float4(fmaf(v.x, a, b), fmaf(v.y, a, b), fmaf(v.z, a, b), fmaf(v.w, a, b));
    }
  } else {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < spatial; i += (long long)gridDim.x * blockDim.x) {
      float v = __ldg(px + i);
      if (apply_relu) v = fmaxf(v, 0.f);
      py[i] = fmaf(v, a, b);
    }
  }
}

}  // namespace
}  // namespace d2c

extern "C" size_t d2c_act_group_norm_workspace_bytes(int batch, int groups) {
  return d2c::align_up(sizeof(double) * 2 * (size_t)(batch > 0 ? batch : 0) * (size_t)(groups > 0 ? groups : 0), 256);
}

extern "C" int d2c_act_group_norm_fwd(const float* x, const float* gamma, const float* beta, float* y, int batch,
                                      int channels, long long spatial, int groups, float eps, int apply_relu,
                                      void* workspace, size_t workspace_bytes, d2c_stream_t stream) {
  using namespace d2c;
  if (!x || !y || !workspace) return D2C_ERR_NULL;
  if (batch < 1 || channels < 1 || spatial < 1 || groups < 1 || channels % groups != 0) return D2C_ERR_SHAPE;
  if (workspace_bytes < d2c_act_group_norm_workspace_bytes(batch, groups)) return D2C_ERR_WORKSPACE;
  const long long bg = (long long)batch * groups, bc = (long long)batch * channels;
  if (bg > 65535 || bc > 65535) return D2C_ERR_TOO_LARGE;
  const int cpg_norm = channels / groups;
  const long long group_elems = (long long)cpg_norm * spatial;
  // 16-byte accesses need every group (moments) / every channel plane (normalisation) on a 16-byte boundary
  const bool al = ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15u) == 0;
  const int vec_m = (al && (group_elems & 3) == 0) ? 1 : 0, vec_n = (al && (spatial & 3) == 0) ? 1 : 0;
  cudaStream_t st = (cudaStream_t)stream;
  double* ws = reinterpret_cast<double*>(workspace);
  D2C_CUDA_TRY(cudaMemsetAsync(ws, 0, sizeof(double) * 2 * (size_t)bg, st));
  prof_mark(st, "act_group_norm");
  long long per = (148LL * 8 + bg - 1) / bg;                      // blocks per group: a few waves in total
  const long long maxb = (group_elems / 4 + 255) / 256;
  if (per > maxb) per = maxb;
  if (per < 1) per = 1;
  act_moments_kernel<<<dim3((unsigned)per, (unsigned)bg), 256, 0, st>>>(x, group_elems, apply_relu, vec_m, ws);
  D2C_LAUNCH_CHECK();
  long long perc = (148LL * 8 + bc - 1) / bc;
  const long long maxc = (spatial / 4 + 255) / 256;
  if (perc > maxc) perc = maxc;
  if (perc < 1) perc = 1;
  act_normalize_kernel<<<dim3((unsigned)perc, (unsigned)bc), 256, 0, st>>>(x, gamma, beta, y, channels, cpg_norm, spatial,
                                                                       group_elems, eps, apply_relu, vec_n, ws);
  D2C_LAUNCH_CHECK();
  prof_mark(st, nullptr);
  return D2C_OK;
}

// ---- backward ------------------------------------------------------------------------------------------
// With a = act(x), ah = (a - mean) * rstd, y = ah * gamma + beta and N = elements of a group:
//   grad_beta[c]  = sum_{b,v} gy           grad_gamma[c] = sum_{b,v} gy * ah
//   grad_a = rstd * (gamma*gy - S1/N - ah * S2/N),  S1 = sum_group gamma*gy,  S2 = sum_group gamma*gy*ah
//   grad_x = grad_a * (x > 0)   (relu)
// Three passes: per-(clip, channel) sums t1 = sum_v gy, t2 = sum_v gy*ah (grid-wide, fp64 atomics); a tiny
// kernel that folds them into S1, S2 per (clip, group) and grad_gamma / grad_beta; the streaming grad_x pass.
namespace d2c {
namespace {

__device__ __forceinline__ void group_stats(const double* __restrict__ stats, long long bg, long long n, float eps,
                                            float& mean, float& rstd) {
  const double m = stats[2 * bg] / (double)n;
  const double var = fmax(stats[2 * bg + 1] / (double)n - m * m, 0.0);
  mean = (float)m;
  rstd = (float)(1.0 / sqrt(var + (double)eps));
}

// t: [batch*channels][2] doubles, zeroed before.
__global__ void __launch_bounds__(256)
act_norm_bwd_sums_kernel(const float* __restrict__ x, const float* __restrict__ gy, int channels, int cpg_norm,
                         long long spatial, long long group_elems, float eps, int apply_relu,
                         const double* __restrict__ stats, double* __restrict__ t) {
  const long long bc = blockIdx.y;
  const int c = (int)(bc % channels);
  const long long bg = (bc / channels) * (channels / cpg_norm) + c / cpg_norm;
  float mean, rstd;
  group_stats(stats, bg, group_elems, eps, mean, rstd);
  const float* px = x + bc * spatial;
  const float* pg = gy + bc * spatial;
  float s1 = 0.f, s2 = 0.f;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < spatial; i += (long long)gridDim.x * blockDim.x) {
    float a = __ldg(px + i);
    if (apply_relu) a = fmaxf(a, 0.f);
    const float g = __ldg(pg + i);
    s1 += g;
    s2 += g * ((a - mean) * rstd);
  }
  double d1 = s1, d2 = s2;
#pragma unroll
  for (int o = 16; o >= 1; o >>= 1) {
    d1 += __shfl_xor_sync(0xffffffffu, d1, o);
    d2 += __shfl_xor_sync(0xffffffffu, d2, o);
  }
  __shared__ double red[2][8];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (lane == 0) { red[0][warp] = d1; red[1][warp] = d2; }
  __syncthreads();
  if (threadIdx.x == 0) {
    double a = 0, b = 0;
    for (int w = 0; w < 8; ++w) { a += red[0][w]; b += red[1][w]; }
    atomicAdd(t + 2 * bc, a);
    atomicAdd(t + 2 * bc + 1, b);
  }
}

// One thread per channel: grad_gamma / grad_beta over the clips; one thread per (clip, group): S1, S2.
__global__ void __launch_bounds__(256)
act_norm_bwd_fold_kernel(int batch, int channels, int groups, const float* __restrict__ gamma,
                         const double* __restrict__ t, double* __restrict__ s, float* __restrict__ grad_gamma,
                         float* __restrict__ grad_beta) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < channels) {
    double a = 0, b = 0;
    for (int bb = 0; bb < batch; ++bb) { a += t[2 * ((long long)bb * channels + i)]; b += t[2 * ((long long)bb * channels + i) + 1]; }
    if (grad_beta) grad_beta[i] = (float)a;
    if (grad_gamma) grad_gamma[i] = (float)b;
  }
  if (i < batch * groups) {
    const int bb = i / groups, gidx = i % groups, cpg_norm = channels / groups;
    double a = 0, b = 0;
    for (int c = gidx * cpg_norm; c < (gidx + 1) * cpg_norm; ++c) {
      const double ga = gamma ? (double)gamma[c] : 1.0;
      a += ga * t[2 * ((long long)bb * channels + c)];
      b += ga * t[2 * ((long long)bb * channels + c) + 1];
    }
    s[2 * i] = a;
    s[2 * i + 1] = b;
  }
}

__global__ void __launch_bounds__(256)
act_norm_bwd_dx_kernel(const float* __restrict__ x, const float* __restrict__ gy, const float* __restrict__ gamma,
                       float* __restrict__ gx, int channels, int cpg_norm, long long spatial, long long group_elems,
                       float eps, int apply_relu, const double* __restrict__ stats, const double* __restrict__ s) {
  const long long bc = blockIdx.y;
  const int c = (int)(bc % channels);
  const long long bg = (bc / channels) * (channels / cpg_norm) + c / cpg_norm;
  float mean, rstd;
  group_stats(stats, bg, group_elems, eps, mean, rstd);
  const float ga = gamma ? __ldg(gamma + c) : 1.f;
  const float m1 = (float)(s[2 * bg] / (double)group_elems), m2 = (float)(s[2 * bg + 1] / (double)group_elems);
  const float* px = x + bc * spatial;
  const float* pg = gy + bc * spatial;
  float* po = gx + bc * spatial;
  for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < spatial; i += (long long)gridDim.x * blockDim.x) {
    const float xv = __ldg(px + i);
    const float a = apply_relu ? fmaxf(xv, 0.f) : xv;
    const float ah = (a - mean) * rstd;
    const float da = rstd * (ga * __ldg(pg + i) - m1 - ah * m2);
    po[i] = (apply_relu && !(xv > 0.f)) ? 0.f : da;
  }
}

}  // namespace
}  // namespace d2c

extern "C" size_t d2c_act_group_norm_bwd_workspace_bytes(int batch, int channels, int groups) {
  const size_t b = batch > 0 ? batch : 0;
  return d2c::align_up(sizeof(double) * 2 * b * (size_t)(channels > 0 ? channels : 0), 256) +
         d2c::align_up(sizeof(double) * 2 * b * (size_t)(groups > 0 ? groups : 0), 256);
}

extern "C" int d2c_act_group_norm_bwd(const float* x, const float* gamma, const float* grad_y, const void* fwd_stats,
                                      float* grad_x, float* grad_gamma, float* grad_beta, int batch, int channels,
                                      long long spatial, int groups, float eps, int apply_relu, void* workspace,
                                      size_t workspace_bytes, d2c_stream_t stream) {
  using namespace d2c;
  if (!x || !grad_y || !fwd_stats || !grad_x || !workspace) return D2C_ERR_NULL;
  if (batch < 1 || channels < 1 || spatial < 1 || groups < 1 || channels % groups != 0) return D2C_ERR_SHAPE;
  if (workspace_bytes < d2c_act_group_norm_bwd_workspace_bytes(batch, channels, groups)) return D2C_ERR_WORKSPACE;
  const long long bc = (long long)batch * channels;
  if (bc > 65535) return D2C_ERR_TOO_LARGE;
  const int cpg_norm = channels / groups;
  const long long group_elems = (long long)cpg_norm * spatial;
  cudaStream_t st = (cudaStream_t)stream;
  double* t = reinterpret_cast<double*>(workspace);
  double* s = reinterpret_cast<double*>(reinterpret_cast<uint8_t*>(workspace) + align_up(sizeof(double) * 2 * (size_t)bc, 256));
  const double* stats = reinterpret_cast<const double*>(fwd_stats);
  D2C_CUDA_TRY(cudaMemsetAsync(t, 0, sizeof(double) * 2 * (size_t)bc, st));
  prof_mark(st, "act_group_norm_bwd");
  long long per = (148LL * 8 + bc - 1) / bc;
  const long long maxb = (spatial + 255) / 256;
  if (per > maxb) per = maxb;
  if (per < 1) per = 1;
  act_norm_bwd_sums_kernel<<<dim3((unsigned)per, (unsigned)bc), 256, 0, st>>>(x, grad_y, channels, cpg_norm, spatial,
                                                                           group_elems, eps, apply_relu, stats, t);
  D2C_LAUNCH_CHECK();
  const int n = channels > batch * groups ? channels : batch * groups;
  act_norm_bwd_fold_kernel<<<(n + 255) / 256, 256, 0, st>>>(batch, channels, groups, gamma, t, s, grad_gamma, grad_beta);
  D2C_LAUNCH_CHECK();
  act_norm_bwd_dx_kernel<<<dim3((unsigned)per, (unsigned)bc), 256, 0, st>>>(x, grad_y, gamma, grad_x, channels, cpg_norm,
                                                                         spatial, group_elems, eps, apply_relu, stats, s);
  D2C_LAUNCH_CHECK();
  prof_mark(st, nullptr);
  return D2C_OK;
}
