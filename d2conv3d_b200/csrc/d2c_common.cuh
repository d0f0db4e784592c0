// Shared host/device definitions of libd2conv3d: geometry, coordinate formation,
// trilinear corner set-up.  Everything that decides an INTEGER (floor corners,
// validity of a corner, which channel of which tensor is read) lives here so that
// the generic and the tensor-core kernels cannot disagree.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/d2conv3d.h"

namespace d2c {

constexpr int kMaxFieldKernelDim = 16;  // dilation-field path: per-dim kernel size limit

struct Geom {
  int B, Cin, Cout, D, H, W;
  int kd, kh, kw, sd, sh, sw, pd, ph, pw, dd, dh, dw;
  int groups, G;           // weight groups, offset (deformable) groups
  int Do, Ho, Wo, K, V;    // output dims, taps, output voxels per clip
  int cin_g, cout_g, cpg;  // Cin/groups, Cout/groups, Cin/G
  long long Vin;           // D*H*W
};

// get_output_size, reference csrc/ops/dconv_gpu_common.h:13-15
inline int out_size(int in, int k, int s, int p, int d) { return (in + 2 * p - (d * (k - 1) + 1)) / s + 1; }

inline int make_geom(const d2c_conv_desc* d, Geom* g, bool depthwise) {
  if (!d) return D2C_ERR_NULL;
  g->B = d->batch; g->Cin = d->in_channels; g->Cout = d->out_channels;
  g->D = d->in_d; g->H = d->in_h; g->W = d->in_w;
  g->kd = d->kd; g->kh = d->kh; g->kw = d->kw;
  g->sd = d->stride_d; g->sh = d->stride_h; g->sw = d->stride_w;
  g->pd = d->pad_d; g->ph = d->pad_h; g->pw = d->pad_w;
  g->dd = d->dil_d; g->dh = d->dil_h; g->dw = d->dil_w;
  g->groups = depthwise ? d->in_channels : d->groups;
  g->G = depthwise ? 1 : d->offset_groups;
  if (g->B <= 0 || g->Cin <= 0 || g->Cout <= 0 || g->D <= 0 || g->H <= 0 || g->W <= 0) return D2C_ERR_SHAPE;
  if (g->kd <= 0 || g->kh <= 0 || g->kw <= 0 || g->sd <= 0 || g->sh <= 0 || g->sw <= 0 ||
      g->dd <= 0 || g->dh <= 0 || g->dw <= 0 || g->pd < 0 || g->ph < 0 || g->pw < 0)
    return D2C_ERR_SHAPE;
  if (g->groups <= 0 || g->G <= 0) return D2C_ERR_GROUPS;
  if (depthwise) {
    if (g->Cout % g->Cin) return D2C_ERR_WEIGHT_SHAPE;
  } else {
    // SANITY_CHECK_DCONV_GROUPS, reference csrc/ops/dconv_gpu_common.h:19-25
    if (g->Cin % g->groups || g->Cout % g->groups || g->Cout % g->G || g->Cin % g->G) return D2C_ERR_GROUPS;
  }
  g->Do = out_size(g->D, g->kd, g->sd, g->pd, g->dd);
  g->Ho = out_size(g->H, g->kh, g->sh, g->ph, g->dh);
  g->Wo = out_size(g->W, g->kw, g->sw, g->pw, g->dw);
  if (g->Do <= 0 || g->Ho <= 0 || g->Wo <= 0) return D2C_ERR_OUT_DIMS;
  g->K = g->kd * g->kh * g->kw;
  const long long V = (long long)g->Do * g->Ho * g->Wo;
  g->Vin = (long long)g->D * g->H * g->W;
  if (V > 0x7fffffffLL || g->Vin > 0x7fffffffLL) return D2C_ERR_TOO_LARGE;
  g->V = (int)V;
  g->cin_g = g->Cin / g->groups; g->cout_g = g->Cout / g->groups; g->cpg = g->Cin / g->G;
  return D2C_OK;
}

// ---- explicitly rounded arithmetic (never contracted into FMA by the compiler) -------------
__device__ __forceinline__ float add_rn(float a, float b) { return __fadd_rn(a, b); }
__device__ __forceinline__ double add_rn(double a, double b) { return __dadd_rn(a, b); }
__device__ __forceinline__ float sub_rn(float a, float b) { return __fsub_rn(a, b); }
__device__ __forceinline__ double sub_rn(double a, double b) { return __dsub_rn(a, b); }
__device__ __forceinline__ float mul_rn(float a, float b) { return __fmul_rn(a, b); }
__device__ __forceinline__ double mul_rn(double a, double b) { return __dmul_rn(a, b); }
__device__ __forceinline__ float fma_rn(float a, float b, float c) { return __fmaf_rn(a, b, c); }
__device__ __forceinline__ double fma_rn(double a, double b, double c) { return __fma_rn(a, b, c); }
__device__ __forceinline__ int floor_int(float a) { return __float2int_rd(a); }
__device__ __forceinline__ int floor_int(double a) { return __double2int_rd(a); }

// ---- deformation head fused into the op ---------------------------------------------------------
// The layers around the op (network/layers.py:107-120, 171-181, 302-313) take ONE tensor from their predictor
// convolution, split it into [geometry | mask logits] channels and apply an activation to each part.  With a head
// configuration the kernels read that raw tensor in place (clip stride = all of its channels), apply the
// activation where they read it, and write the gradient w.r.t. the raw tensor (chain rule included).
// All-zero configuration = the plain op: dense tensors, no activation.
struct HeadCfg {
  long long geo_bstride;    // elements between clips of the offset / field tensor (0: dense)
  long long mask_bstride;   // ... of the mask tensor (0: dense)
  int mask_act;             // d2c_mask_act
  int size_act;             // d2c_size_act (dilation-field variants)
};

// mask activations of the reference's layers (network/layers.py:19-25)
template <typename T>
__host__ __device__ __forceinline__ T mask_act_value(int act, T r) {
  switch (act) {
    case D2C_MASK_SIGMOID: return (T)1 / ((T)1 + exp(-r));
    case D2C_MASK_RELU: return r > (T)0 ? r : (T)0;
    case D2C_MASK_TANH: return tanh(r);
    default: return r;
  }
}
// derivative of the activation, from the ACTIVATED value m
template <typename T>
__host__ __device__ __forceinline__ T mask_act_slope(int act, T m) {
  switch (act) {
    case D2C_MASK_SIGMOID: return m * ((T)1 - m);
    case D2C_MASK_RELU: return m > (T)0 ? (T)1 : (T)0;
    case D2C_MASK_TANH: return (T)1 - m * m;
    default: return (T)1;
  }
}
// size activations (network/layers.py:171-181): elu(x)+1, relu(x+1), relu(x+1e-3)+1, identity
template <typename T>
__host__ __device__ __forceinline__ T size_act_value(int act, T r) {
  switch (act) {
    case D2C_SIZE_ELU: return (r > (T)0 ? r : (exp(r) - (T)1)) + (T)1;
    case D2C_SIZE_RELU: { const T t = r + (T)1; return t > (T)0 ? t : (T)0; }
    case D2C_SIZE_RELU_PLUS_ONE: { const T t = r + (T)1e-3; return (t > (T)0 ? t : (T)0) + (T)1; }
    default: return r;
  }
}
// derivative w.r.t. the RAW value r (torch's conventions at the kinks: elu' (0) = 1, relu'(0) = 0)
template <typename T>
__host__ __device__ __forceinline__ T size_act_slope(int act, T r) {
  switch (act) {
    case D2C_SIZE_ELU: return r > (T)0 ? (T)1 : exp(r);
    case D2C_SIZE_RELU: return r + (T)1 > (T)0 ? (T)1 : (T)0;
    case D2C_SIZE_RELU_PLUS_ONE: return r + (T)1e-3 > (T)0 ? (T)1 : (T)0;
    default: return (T)1;
  }
}

// ---- where the sampling coordinates come from ----------------------------------------------

// Offsets given explicitly: [B, G*3K, V], channel 3*(grp*K+tap)+{0:z,1:y,2:x}
// (reference csrc/ops/dconv3d_gpu.cu:166-194).
template <typename T>
struct OffsetCoords {
  const T* offset;
  long long bstride;   // elements between clips; 0 = dense [B, G*3K, V]
  __device__ __forceinline__ void get(const Geom& g, int b, int grp, int tap, int v, int bz, int by,
                                      int bx, T& z, T& y, T& x) const {
    const long long bs = bstride ? bstride : (long long)g.G * 3 * g.K * g.V;
    const T* p = offset + (long long)b * bs + ((long long)grp * 3 * g.K + 3 * tap) * g.V + v;
    z = add_rn((T)bz, __ldg(p));
    y = add_rn((T)by, __ldg(p + g.V));
    x = add_rn((T)bx, __ldg(p + 2 * (long long)g.V));
  }
};

// deform_conv1d evaluated on a [B, C, 1, 1, L] view: one offset per (group, tap, position),
// offset [B, G*K, Lo]; depth and height coordinates are exactly 0 (reference csrc/ops/dconv1d_gpu.cu:44-46).
template <typename T>
struct Offset1dCoords {
  const T* offset;
  __device__ __forceinline__ void get(const Geom& g, int b, int grp, int tap, int v, int bz, int by,
                                      int bx, T& z, T& y, T& x) const {
    z = (T)bz;
    y = (T)by;
    x = add_rn((T)bx, __ldg(offset + (((long long)b * g.G + grp) * g.K + tap) * g.V + v));
  }
};

template <typename Coords>
struct CoordsIs1d { static constexpr bool value = false; };
template <typename T>
struct CoordsIs1d<Offset1dCoords<T>> { static constexpr bool value = true; };

// Offsets synthesised from a dilation field shared by all offset groups:
// offset_d = base_d[tap] * (s_d - 1) with the two roundings of the reference's
// PyTorch expression `base_offset * (size_map - 1)` (utils/grid.py:97), then the
// same single add as above.  ch[d] < 0 means "this dim keeps scale 1".
template <typename T>
struct FieldCoords {
  const T* size_map;  // [B, nch, V]
  int nch;
  int ch[3];
  T axis[3][kMaxFieldKernelDim];  // linspace(-dil*(k/2), dil*(k/2), k) per dim
  long long bstride;  // elements between clips; 0 = dense [B, nch, V]
  int act;            // d2c_size_act applied to the values read (0: the map holds the scales themselves)
  __device__ __forceinline__ void get(const Geom& g, int b, int /*grp*/, int tap, int v, int bz,
                                      int by, int bx, T& z, T& y, T& x) const {
    const int k = tap % g.kw, j = (tap / g.kw) % g.kh, i = tap / (g.kw * g.kh);
    const T* p = size_map + (long long)b * (bstride ? bstride : (long long)nch * g.V) + v;
    const T sz = ch[0] < 0 ? (T)1 : size_act_value(act, __ldg(p + (long long)ch[0] * g.V));
    const T sy = ch[1] < 0 ? (T)1 : size_act_value(act, __ldg(p + (long long)ch[1] * g.V));
    const T sx = ch[2] < 0 ? (T)1 : size_act_value(act, __ldg(p + (long long)ch[2] * g.V));
    z = add_rn((T)bz, mul_rn(axis[0][i], sub_rn(sz, (T)1)));
    y = add_rn((T)by, mul_rn(axis[1][j], sub_rn(sy, (T)1)));
    x = add_rn((T)bx, mul_rn(axis[2][k], sub_rn(sx, (T)1)));
  }
};

// ---- trilinear corner set-up ----------------------------------------------------------------

// One sampling position resolved to its floor corner, per-corner validity bits
// (bit = dz*4 + dy*2 + dx, the reference's point order 000..111) and the eight
// interpolation weights, multiplied exactly as reference dconv3d_gpu.cu:87-94.
template <typename T>
struct Sample {
  int z0, y0, x0;
  unsigned valid;  // corner inside the volume
  bool inside;     // forward early-out passed (dconv3d_gpu.cu:59-61)
  T fz, fy, fx;    // (z - z0) etc.
  T gz, gy, gx;    // (z1 - z) etc.
};

template <typename T>
__device__ __forceinline__ Sample<T> make_sample(const Geom& g, T z, T y, T x) {
  Sample<T> s;
  s.inside = !(z <= (T)-1 || (T)g.D <= z || y <= (T)-1 || (T)g.H <= y || x <= (T)-1 || (T)g.W <= x);
  s.z0 = floor_int(z); s.y0 = floor_int(y); s.x0 = floor_int(x);
  const int z1 = s.z0 + 1, y1 = s.y0 + 1, x1 = s.x0 + 1;
  const bool vz0 = s.z0 >= 0 && s.z0 < g.D, vz1 = z1 >= 0 && z1 < g.D;
  const bool vy0 = s.y0 >= 0 && s.y0 < g.H, vy1 = y1 >= 0 && y1 < g.H;
  const bool vx0 = s.x0 >= 0 && s.x0 < g.W, vx1 = x1 >= 0 && x1 < g.W;
  s.valid = (unsigned)(vz0 && vy0 && vx0) | ((unsigned)(vz0 && vy0 && vx1) << 1) |
            ((unsigned)(vz0 && vy1 && vx0) << 2) | ((unsigned)(vz0 && vy1 && vx1) << 3) |
            ((unsigned)(vz1 && vy0 && vx0) << 4) | ((unsigned)(vz1 && vy0 && vx1) << 5) |
            ((unsigned)(vz1 && vy1 && vx0) << 6) | ((unsigned)(vz1 && vy1 && vx1) << 7);
  s.fz = sub_rn(z, (T)s.z0); s.fy = sub_rn(y, (T)s.y0); s.fx = sub_rn(x, (T)s.x0);
  s.gz = sub_rn((T)z1, z); s.gy = sub_rn((T)y1, y); s.gx = sub_rn((T)x1, x);
  return s;
}

// interpolation weights a000..a111 ((dz?fz:gz)*(dy?fy:gy))*(dx?fx:gx), left to right
template <typename T>
__device__ __forceinline__ void sample_weights(const Sample<T>& s, T a[8]) {
  const T zy00 = mul_rn(s.gz, s.gy), zy01 = mul_rn(s.gz, s.fy);
  const T zy10 = mul_rn(s.fz, s.gy), zy11 = mul_rn(s.fz, s.fy);
  a[0] = mul_rn(zy00, s.gx); a[1] = mul_rn(zy00, s.fx);
  a[2] = mul_rn(zy01, s.gx); a[3] = mul_rn(zy01, s.fx);
  a[4] = mul_rn(zy10, s.gx); a[5] = mul_rn(zy10, s.fx);
  a[6] = mul_rn(zy11, s.gx); a[7] = mul_rn(zy11, s.fx);
}

// the eight corner values of one channel plane (0 where the corner is outside)
template <typename T>
__device__ __forceinline__ void gather_corners(const Geom& g, const T* plane, const Sample<T>& s,
                                               T c[8]) {
  const long long base = ((long long)s.z0 * g.H + s.y0) * g.W + s.x0;
  const int sy = g.W, sz = g.H * g.W;
  c[0] = (s.valid & 1u) ? __ldg(plane + base) : (T)0;
  c[1] = (s.valid & 2u) ? __ldg(plane + base + 1) : (T)0;
  c[2] = (s.valid & 4u) ? __ldg(plane + base + sy) : (T)0;
  c[3] = (s.valid & 8u) ? __ldg(plane + base + sy + 1) : (T)0;
  c[4] = (s.valid & 16u) ? __ldg(plane + base + sz) : (T)0;
  c[5] = (s.valid & 32u) ? __ldg(plane + base + sz + 1) : (T)0;
  c[6] = (s.valid & 64u) ? __ldg(plane + base + sz + sy) : (T)0;
  c[7] = (s.valid & 128u) ? __ldg(plane + base + sz + sy + 1) : (T)0;
}

// trilinear_interpolate, reference dconv3d_gpu.cu:48-109: fma chain in corner order
template <typename T>
__device__ __forceinline__ T blend(const T c[8], const T a[8]) {
  T r = (T)0;
#pragma unroll
  for (int j = 0; j < 8; ++j) r = fma_rn(c[j], a[j], r);
  return r;
}

// get_coordinate_weights, reference dconv3d_gpu.cu:708-754
template <typename T>
__device__ __forceinline__ void coord_weights(const T c[8], const Sample<T>& s, T out[3]) {
  const T dz = s.fz, dy = s.fy, dx = s.fx;
  out[0] = ((c[4] - c[0]) * (1 - dx) + (c[5] - c[1]) * dx) * (1 - dy) +
           ((c[6] - c[2]) * (1 - dx) + (c[7] - c[3]) * dx) * dy;
  out[1] = ((c[2] - c[0]) * (1 - dz) + (c[6] - c[4]) * dz) * (1 - dx) +
           ((c[3] - c[1]) * (1 - dz) + (c[7] - c[5]) * dz) * dx;
  out[2] = ((c[1] - c[0]) * (1 - dz) + (c[5] - c[4]) * dz) * (1 - dy) +
           ((c[3] - c[2]) * (1 - dz) + (c[7] - c[6]) * dz) * dy;
}

// integer base coordinate of (output voxel, tap): (o*stride - pad) + i*dil
__device__ __forceinline__ void voxel_tap_base(const Geom& g, int v, int tap, int& bz, int& by, int& bx) {
  const int ox = v % g.Wo, oy = (v / g.Wo) % g.Ho, oz = v / (g.Wo * g.Ho);
  const int k = tap % g.kw, j = (tap / g.kw) % g.kh, i = tap / (g.kw * g.kh);
  bz = (oz * g.sd - g.pd) + i * g.dd;
  by = (oy * g.sh - g.ph) + j * g.dh;
  bx = (ox * g.sw - g.pw) + k * g.dw;
}

// ---- host-side error plumbing ----------------------------------------------------------------
void set_last_cuda_error(cudaError_t e);
inline int check_cuda(cudaError_t e) {
  if (e == cudaSuccess) return D2C_OK;
  set_last_cuda_error(e);
  return D2C_ERR_CUDA;
}
#define D2C_CUDA_TRY(expr)                                \
  do {                                                    \
    int _rc = ::d2c::check_cuda((expr));                  \
    if (_rc) return _rc;                                  \
  } while (0)
// Every kernel launch of the library goes through this: counts it and checks it.
void count_launch();
#define D2C_LAUNCH_CHECK()               \
  do {                                   \
    ::d2c::count_launch();               \
    D2C_CUDA_TRY(cudaGetLastError());    \
  } while (0)

// Phase profiling (off by default): when enabled, a CUDA event is recorded on the
// caller's stream at every mark; the phase `name` lasts until the next mark.
// name == nullptr closes the current phase.
void prof_mark(cudaStream_t st, const char* name);

inline size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Multiprocessor count of the current device (cached per device).
int device_sm_count(int* out);

}  // namespace d2c
