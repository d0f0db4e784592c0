// Fused activation + group normalisation, forward (inference): y = GroupNorm(relu(x)) for NCDHW fp32 tensors.
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
