// Generic (any geometry, fp32 / fp64) CUDA-core kernels of the deformable conv3d
// path.  This is the tier every call can fall back to: stride / dilation / kernel
// shape / group counts are unrestricted and all arithmetic is done in T on the FMA
// pipe, so fp32 results differ from a cuBLAS-based evaluation only by summation
// order and fp64 supports gradcheck.  The tensor-core tier (deform_sm100_*.cu)
// replaces these kernels for the shapes it supports.
//
// Unlike the reference (csrc/ops/dconv3d_gpu.cu) no column matrix is built in the
// forward or in the weight gradient: samples are produced tile by tile in shared
// memory and consumed by the contraction in the same kernel.  Only the backward's
// gradient columns (dcol) are materialised, in caller-supplied workspace.
#pragma once

#include "d2c_common.cuh"

namespace d2c {

constexpr int kTileV = 64;   // output voxels per block tile
constexpr int kTileN = 64;   // output channels (or column rows) per block tile
constexpr int kTileR = 16;   // reduction rows staged per step
constexpr int kGemmThreads = 256;

// One modulated sample: mask * trilinear(x[b,c], p) for reduction row r = c_local*K + tap
// of weight group wg (reference dconv3d_gpu.cu:184-199).
template <typename T, typename Coords>
__device__ __forceinline__ T sample_row(const Geom& g, const Coords& coords, const T* __restrict__ x,
                                        const T* __restrict__ mask, int b, int wg, int r, int v) {
  const int c_local = r / g.K, tap = r - c_local * g.K;
  const int c = wg * g.cin_g + c_local;
  const int grp = c / g.cpg;
  int bz, by, bx;
  voxel_tap_base(g, v, tap, bz, by, bx);
  T z, y, xx;
  coords.get(g, b, grp, tap, v, bz, by, bx, z, y, xx);
  const Sample<T> s = make_sample(g, z, y, xx);
  if (!s.inside) return (T)0;
  T a[8], cv[8];
  sample_weights(s, a);
  gather_corners(g, x + ((long long)b * g.Cin + c) * g.Vin, s, cv);
  const T m = mask ? __ldg(mask + (((long long)b * g.G + grp) * g.K + tap) * g.V + v) : (T)1;
  return mul_rn(m, blend(cv, a));
}

// ---- forward: y[b, co, v] = sum_r W[co, r] * sample(b, r, v) + bias[co] ---------------------
template <typename T, typename Coords>
__global__ void __launch_bounds__(kGemmThreads)
fwd_generic_kernel(Geom g, Coords coords, const T* __restrict__ x, const T* __restrict__ mask,
                   const T* __restrict__ w, const T* __restrict__ bias, T* __restrict__ y) {
  __shared__ T As[kTileR][kTileV];       // samples  [r][v]
  __shared__ T Bs[kTileR][kTileN + 1];   // weights  [r][co]
  const int t = threadIdx.x, tx = t % 16, ty = t / 16;
  const int v0 = blockIdx.x * kTileV, n0 = blockIdx.y * kTileN;
  const int b = blockIdx.z / g.groups, wg = blockIdx.z % g.groups;
  const int R = g.cin_g * g.K;
  T acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = (T)0;

  for (int r0 = 0; r0 < R; r0 += kTileR) {
#pragma unroll
    for (int i = 0; i < (kTileR * kTileV) / kGemmThreads; ++i) {
      const int e = t + i * kGemmThreads, rl = e / kTileV, vl = e % kTileV;
      const int r = r0 + rl, v = v0 + vl;
      As[rl][vl] = (r < R && v < g.V) ? sample_row(g, coords, x, mask, b, wg, r, v) : (T)0;
    }
#pragma unroll
    for (int i = 0; i < (kTileR * kTileN) / kGemmThreads; ++i) {
      const int e = t + i * kGemmThreads, rl = e % kTileR, nl = e / kTileR;
      const int r = r0 + rl, n = n0 + nl;
      Bs[rl][nl] = (r < R && n < g.cout_g) ? __ldg(w + ((long long)(wg * g.cout_g + n)) * R + r) : (T)0;
    }
    __syncthreads();
#pragma unroll
    for (int rl = 0; rl < kTileR; ++rl) {
      T av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[rl][tx * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = Bs[rl][ty * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fma_rn(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int n = n0 + ty * 4 + j;
    if (n >= g.cout_g) continue;
    const int co = wg * g.cout_g + n;
    const T bb = bias ? __ldg(bias + co) : (T)0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int v = v0 + tx * 4 + i;
      if (v < g.V) y[((long long)b * g.Cout + co) * g.V + v] = acc[i][j] + bb;
    }
  }
}

// ---- backward step 1: dcol[bl, c*K+tap, v] = sum_co W[co, r] * gy[b, co, v] ------------------
// (reference dconv3d_gpu.cu:981-999).  dcol is the workspace slice of clips [b0, b0+nb).
template <typename T>
__global__ void __launch_bounds__(kGemmThreads)
dcol_generic_kernel(Geom g, int b0, const T* __restrict__ gy, const T* __restrict__ w,
                    T* __restrict__ dcol) {
  __shared__ T As[kTileR][kTileV];       // gy  [co][v]
  __shared__ T Bs[kTileR][kTileN + 1];   // W   [co][r]
  const int t = threadIdx.x, tx = t % 16, ty = t / 16;
  const int v0 = blockIdx.x * kTileV, r0 = blockIdx.y * kTileN;
  const int bl = blockIdx.z / g.groups, wg = blockIdx.z % g.groups, b = b0 + bl;
  const int R = g.cin_g * g.K;
  T acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = (T)0;
  for (int c0 = 0; c0 < g.cout_g; c0 += kTileR) {
#pragma unroll
    for (int i = 0; i < (kTileR * kTileV) / kGemmThreads; ++i) {
      const int e = t + i * kGemmThreads, cl = e / kTileV, vl = e % kTileV;
      const int co = c0 + cl, v = v0 + vl;
      As[cl][vl] = (co < g.cout_g && v < g.V)
                       ? __ldg(gy + ((long long)b * g.Cout + wg * g.cout_g + co) * g.V + v) : (T)0;
    }
#pragma unroll
    for (int i = 0; i < (kTileR * kTileN) / kGemmThreads; ++i) {
      const int e = t + i * kGemmThreads, cl = e / kTileN, rl = e % kTileN;
      const int co = c0 + cl, r = r0 + rl;
      Bs[cl][rl] = (co < g.cout_g && r < R) ? __ldg(w + ((long long)(wg * g.cout_g + co)) * R + r) : (T)0;
    }
    __syncthreads();
#pragma unroll
    for (int cl = 0; cl < kTileR; ++cl) {
      T av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[cl][tx * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = Bs[cl][ty * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fma_rn(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int r = r0 + ty * 4 + j;
    if (r >= R) continue;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int v = v0 + tx * 4 + i;
      if (v < g.V) dcol[((long long)bl * g.Cin * g.K + (long long)wg * R + r) * g.V + v] = acc[i][j];
    }
  }
}

// ---- backward step 2: offset / mask gradients (reference dconv3d_gpu.cu:756-864) -------------
// One thread per (clip, offset group, tap, voxel); the corner set-up is hoisted out
// of the channel loop and the eight corner values serve both the sample (for
// grad_mask) and its three coordinate derivatives.
// FieldOut == false: writes grad_offset[b, 3(gK+tap)+d, v] = mask * val[d].
// FieldOut == true : accumulates base_d[tap] * mask * val[d] into grad_size_map (pre-zeroed).
template <typename T, typename Coords, bool FieldOut>
__global__ void __launch_bounds__(256)
coord_grad_generic_kernel(Geom g, Coords coords, int b0, int nb, const T* __restrict__ dcol,
                          const T* __restrict__ x, const T* __restrict__ mask,
                          T* __restrict__ grad_offset, T* __restrict__ grad_mask) {
  const long long total = (long long)nb * g.G * g.K * g.V;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(idx % g.V);
    const int tap = (int)((idx / g.V) % g.K);
    const int grp = (int)((idx / ((long long)g.V * g.K)) % g.G);
    const int bl = (int)(idx / ((long long)g.V * g.K * g.G));
    const int b = b0 + bl;
    int bz, by, bx;
    voxel_tap_base(g, v, tap, bz, by, bx);
    T z, y, xx;
    coords.get(g, b, grp, tap, v, bz, by, bx, z, y, xx);
    const Sample<T> s = make_sample(g, z, y, xx);
    T a[8];
    sample_weights(s, a);
    T val0 = 0, val1 = 0, val2 = 0, mval = 0;
    const T* dc = dcol + (((long long)bl * g.Cin + (long long)grp * g.cpg) * g.K + tap) * g.V + v;
    const T* plane = x + ((long long)b * g.Cin + (long long)grp * g.cpg) * g.Vin;
    for (int c = 0; c < g.cpg; ++c) {
      const T cvl = __ldg(dc);
      T cv[8], wts[3];
      gather_corners(g, plane, s, cv);
      if (mask && s.inside) mval += cvl * blend(cv, a);
      coord_weights(cv, s, wts);
      val0 += wts[0] * cvl; val1 += wts[1] * cvl; val2 += wts[2] * cvl;
      dc += (long long)g.K * g.V;
      plane += g.Vin;
    }
    const long long mi = (((long long)b * g.G + grp) * g.K + tap) * g.V + v;
    const T m = mask ? __ldg(mask + mi) : (T)1;
    if constexpr (!FieldOut) {
      T* go = grad_offset + (((long long)b * g.G + grp) * 3 * g.K + 3 * tap) * g.V + v;
      go[0] = m * val0;
      go[g.V] = m * val1;
      go[2 * (long long)g.V] = m * val2;
    } else {
      const int k = tap % g.kw, j = (tap / g.kw) % g.kh, i = tap / (g.kw * g.kh);
      T* gs = grad_offset + (long long)b * coords.nch * g.V + v;
      if (coords.ch[0] >= 0) atomicAdd(gs + (long long)coords.ch[0] * g.V, coords.axis[0][i] * (m * val0));
      if (coords.ch[1] >= 0) atomicAdd(gs + (long long)coords.ch[1] * g.V, coords.axis[1][j] * (m * val1));
      if (coords.ch[2] >= 0) atomicAdd(gs + (long long)coords.ch[2] * g.V, coords.axis[2][k] * (m * val2));
    }
    if (mask && grad_mask) grad_mask[mi] = mval;
  }
}

// ---- deform_conv1d: offset / modulation gradients (reference csrc/ops/dconv1d_gpu.cu:300-349) -----------
// The 1-D op has its own convention where linear interpolation is not differentiable: when the sampling
// position is (within 1e-8 of) an integer, the LEFT neighbour moves one further left (`x0 -= 1`, line 336) while
// the right neighbour stays x0 + 1, so grad_offset becomes the two-cell difference input[x+1] - input[x-1] and
// grad_alpha is interpolated between those two cells with parameter x - x0 (= 1 at an integer, i.e. the value
// of the RIGHT cell).  Followed literally, with the reference's lerp (line 13-15).
// One thread per (clip, offset group, tap, output position); x is [B, Cin, L], dcol [nb, Cin*K, Lo].
template <typename T>
__device__ __forceinline__ T lerp_1d(T v0, T v1, T t) { return fma_rn(t, v1, fma_rn(-t, v0, v0)); }

template <typename T>
__global__ void __launch_bounds__(256)
coord_grad_1d_kernel(Geom g, Offset1dCoords<T> coords, int b0, int nb, const T* __restrict__ dcol,
                     const T* __restrict__ x, const T* __restrict__ mask, T* __restrict__ grad_offset,
                     T* __restrict__ grad_mask) {
  const long long total = (long long)nb * g.G * g.K * g.V;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(idx % g.V);
    const int tap = (int)((idx / g.V) % g.K);
    const int grp = (int)((idx / ((long long)g.V * g.K)) % g.G);
    const int bl = (int)(idx / ((long long)g.V * g.K * g.G));
    const int b = b0 + bl;
    int bz, by, bx;
    voxel_tap_base(g, v, tap, bz, by, bx);
    T z, y, pos;
    coords.get(g, b, grp, tap, v, bz, by, bx, z, y, pos);
    int x0 = floor_int(pos);
    const int x1 = x0 + 1;
    if (sub_rn(pos, (T)x0) < (T)1e-8) x0 -= 1;
    const T t = sub_rn(pos, (T)x0);
    const long long mi = (((long long)b * g.G + grp) * g.K + tap) * g.V + v;
    const T a = mask ? __ldg(mask + mi) : (T)1;
    T val = 0, alpha_val = 0;
    const T* dc = dcol + (((long long)bl * g.Cin + (long long)grp * g.cpg) * g.K + tap) * g.V + v;
    const T* row = x + ((long long)b * g.Cin + (long long)grp * g.cpg) * g.Vin;
    for (int c = 0; c < g.cpg; ++c) {
      const T v0 = (x0 >= 0 && x0 < g.W) ? __ldg(row + x0) : (T)0;
      const T v1 = (x1 >= 0 && x1 < g.W) ? __ldg(row + x1) : (T)0;
      const T col = __ldg(dc);
      alpha_val += col * lerp_1d(v0, v1, t);
      val += (v1 - v0) * col * a;
      dc += (long long)g.K * g.V;
      row += g.Vin;
    }
    grad_offset[mi] = val;
    if (mask && grad_mask) grad_mask[mi] = alpha_val;
  }
}

// ---- backward step 3: col2im scatter (reference dconv3d_gpu.cu:562-643) ----------------------
template <typename T, typename Coords>
__global__ void __launch_bounds__(256)
col2im_generic_kernel(Geom g, Coords coords, int b0, int nb, const T* __restrict__ dcol,
                      const T* __restrict__ mask, T* __restrict__ grad_x) {
  const long long total = (long long)nb * g.Cin * g.K * g.V;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(idx % g.V);
    const int tap = (int)((idx / g.V) % g.K);
    const int c = (int)((idx / ((long long)g.V * g.K)) % g.Cin);
    const int bl = (int)(idx / ((long long)g.V * g.K * g.Cin));
    const int b = b0 + bl, grp = c / g.cpg;
    int bz, by, bx;
    voxel_tap_base(g, v, tap, bz, by, bx);
    T z, y, xx;
    coords.get(g, b, grp, tap, v, bz, by, bx, z, y, xx);
    const Sample<T> s = make_sample(g, z, y, xx);
    if (!s.valid) continue;
    const T m = mask ? __ldg(mask + (((long long)b * g.G + grp) * g.K + tap) * g.V + v) : (T)1;
    const T base_grad = m * __ldg(dcol + idx);
    // (1 - |z - zp|): zp = z0 -> 1 - fz ; zp = z0+1 -> 1 - gz.  A corner at distance
    // exactly 1 (fz == 0, zp = z0+1) fails the reference's `< 1` test and is skipped.
    const T wz[2] = {sub_rn((T)1, s.fz), sub_rn((T)1, s.gz)};
    const T wy[2] = {sub_rn((T)1, s.fy), sub_rn((T)1, s.gy)};
    const T wx[2] = {sub_rn((T)1, s.fx), sub_rn((T)1, s.gx)};
    const bool okz[2] = {true, s.gz < (T)1}, oky[2] = {true, s.gy < (T)1}, okx[2] = {true, s.gx < (T)1};
    T* gp = grad_x + ((long long)b * g.Cin + c) * g.Vin;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int dz = j >> 2, dy = (j >> 1) & 1, dx = j & 1;
      if (((s.valid >> j) & 1u) && okz[dz] && oky[dy] && okx[dx]) {
        const T wgt = mul_rn(mul_rn(wz[dz], wy[dy]), wx[dx]);
        atomicAdd(gp + ((long long)(s.z0 + dz) * g.H + (s.y0 + dy)) * g.W + (s.x0 + dx), wgt * base_grad);
      }
    }
  }
}

// ---- backward step 4: dW[co, r] += sum_{b in slice, v in split} gy[b,co,v] * sample(b,r,v) ----
// (reference dconv3d_gpu.cu:1037-1088).  grad_w must be zeroed beforehand; blocks of
// different (clip, voxel-split) accumulate with atomics.
template <typename T, typename Coords>
__global__ void __launch_bounds__(kGemmThreads)
dw_generic_kernel(Geom g, Coords coords, int v_per_split, const T* __restrict__ gy,
                  const T* __restrict__ x, const T* __restrict__ mask, T* __restrict__ grad_w) {
  __shared__ T As[kTileR][kTileV + 1];   // samples [v][r]   (kTileV rows r)
  __shared__ T Bs[kTileR][kTileN + 1];   // gy      [v][co]
  const int t = threadIdx.x, tx = t % 16, ty = t / 16;
  const int R = g.cin_g * g.K;
  const int r0 = blockIdx.x * kTileV, n0 = blockIdx.y * kTileN;
  const int nsplit = (g.V + v_per_split - 1) / v_per_split;
  int zi = blockIdx.z;
  const int split = zi % nsplit; zi /= nsplit;
  const int wg = zi % g.groups;
  const int b = zi / g.groups;
  const int vbeg = split * v_per_split, vend = min(g.V, vbeg + v_per_split);
  T acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = (T)0;
  for (int v0 = vbeg; v0 < vend; v0 += kTileR) {
#pragma unroll
    for (int i = 0; i < (kTileR * kTileV) / kGemmThreads; ++i) {
      const int e = t + i * kGemmThreads, vl = e % kTileR, rl = e / kTileR;
      const int r = r0 + rl, v = v0 + vl;
      As[vl][rl] = (r < R && v < vend) ? sample_row(g, coords, x, mask, b, wg, r, v) : (T)0;
    }
#pragma unroll
    for (int i = 0; i < (kTileR * kTileN) / kGemmThreads; ++i) {
      const int e = t + i * kGemmThreads, vl = e % kTileR, nl = e / kTileR;
      const int n = n0 + nl, v = v0 + vl;
      Bs[vl][nl] = (n < g.cout_g && v < vend)
                       ? __ldg(gy + ((long long)b * g.Cout + wg * g.cout_g + n) * g.V + v) : (T)0;
    }
    __syncthreads();
#pragma unroll
    for (int vl = 0; vl < kTileR; ++vl) {
      T av[4], bv[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) av[i] = As[vl][tx * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) bv[j] = Bs[vl][ty * 4 + j];
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fma_rn(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int n = n0 + ty * 4 + j;
    if (n >= g.cout_g) continue;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = r0 + tx * 4 + i;
      if (r < R) atomicAdd(grad_w + ((long long)(wg * g.cout_g + n)) * R + r, acc[i][j]);
    }
  }
}

// ---- grad_bias[co] = sum_{b,v} gy[b,co,v]  (reference dconv3d_gpu.cu:1329) --------------------
template <typename T>
__global__ void __launch_bounds__(256)
grad_bias_kernel(int B, int Cout, int V, const T* __restrict__ gy, T* __restrict__ grad_bias) {
  __shared__ T red[256];
  const int co = blockIdx.x;
  T s = 0;
  for (int b = 0; b < B; ++b) {
    const T* p = gy + ((long long)b * Cout + co) * V;
    for (int v = threadIdx.x; v < V; v += blockDim.x) s += __ldg(p + v);
  }
  red[threadIdx.x] = s;
  __syncthreads();
  for (int i = 128; i >= 1; i >>= 1) {
    if ((int)threadIdx.x < i) red[threadIdx.x] += red[threadIdx.x + i];
    __syncthreads();
  }
  if (threadIdx.x == 0) grad_bias[co] = red[0];
}

// ---- integer corner probe -----------------------------------------------------------------------
template <typename T, typename Coords>
__global__ void __launch_bounds__(256)
corners_kernel(Geom g, Coords coords, int32_t* __restrict__ corners) {
  const long long total = (long long)g.B * g.G * g.K * g.V;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const int v = (int)(idx % g.V);
    const int tap = (int)((idx / g.V) % g.K);
    const int grp = (int)((idx / ((long long)g.V * g.K)) % g.G);
    const int b = (int)(idx / ((long long)g.V * g.K * g.G));
    int bz, by, bx;
    voxel_tap_base(g, v, tap, bz, by, bx);
    T z, y, xx;
    coords.get(g, b, grp, tap, v, bz, by, bx, z, y, xx);
    const Sample<T> s = make_sample(g, z, y, xx);
    int32_t* o = corners + ((((long long)b * g.G + grp) * g.K + tap) * 3) * g.V + v;
    o[0] = s.z0; o[g.V] = s.y0; o[2 * (long long)g.V] = s.x0;
  }
}

// ---- launch helpers --------------------------------------------------------------------------
inline unsigned grid_1d(long long total, int block, int max_blocks = 148 * 16) {
  long long n = (total + block - 1) / block;
  if (n < 1) n = 1;
  if (n > max_blocks) n = max_blocks;
  return (unsigned)n;
}

template <typename T, typename Coords>
int launch_fwd_generic(const Geom& g, const Coords& coords, const T* x, const T* mask, const T* w,
                       const T* bias, T* y, cudaStream_t st) {
  dim3 grid((g.V + kTileV - 1) / kTileV, (g.cout_g + kTileN - 1) / kTileN, g.B * g.groups);
  if (grid.y > 65535 || grid.z > 65535) return D2C_ERR_TOO_LARGE;
  prof_mark(st, "fwd_generic");
  fwd_generic_kernel<T, Coords><<<grid, kGemmThreads, 0, st>>>(g, coords, x, mask, w, bias, y);
  D2C_LAUNCH_CHECK();
  prof_mark(st, nullptr);
  return D2C_OK;
}

// Clips per backward slice under the intermediate-element cap.
inline int bwd_slice_clips(const Geom& g, unsigned long long cap) {
  const unsigned long long per = (unsigned long long)g.Cin * g.K * g.V;
  unsigned long long nb = per ? cap / per : 1;
  if (nb < 1) nb = 1;
  if (nb > (unsigned long long)g.B) nb = g.B;
  return (int)nb;
}

template <typename T, typename Coords, bool FieldOut>
int launch_bwd_generic(const Geom& g, const Coords& coords, const T* gy, const T* x, const T* mask,
                       const T* w, T* grad_x, T* grad_coord, size_t grad_coord_elems, T* grad_mask,
                       T* grad_w, T* grad_bias, T* dcol, int slice_clips, cudaStream_t st) {
  const int R = g.cin_g * g.K;
  prof_mark(st, "bwd_zero_fill");
  D2C_CUDA_TRY(cudaMemsetAsync(grad_x, 0, sizeof(T) * (size_t)g.B * g.Cin * g.Vin, st));
  D2C_CUDA_TRY(cudaMemsetAsync(grad_w, 0, sizeof(T) * (size_t)g.Cout * R, st));
  if (FieldOut) D2C_CUDA_TRY(cudaMemsetAsync(grad_coord, 0, sizeof(T) * grad_coord_elems, st));
  for (int b0 = 0; b0 < g.B; b0 += slice_clips) {
    const int nb = (g.B - b0 < slice_clips) ? g.B - b0 : slice_clips;
    dim3 grid((g.V + kTileV - 1) / kTileV, (R + kTileN - 1) / kTileN, nb * g.groups);
    if (grid.y > 65535 || grid.z > 65535) return D2C_ERR_TOO_LARGE;
    prof_mark(st, "bwd_dcol_generic");
    dcol_generic_kernel<T><<<grid, kGemmThreads, 0, st>>>(g, b0, gy, w, dcol);
    D2C_LAUNCH_CHECK();
    prof_mark(st, "bwd_coord_grad_generic");
    if constexpr (CoordsIs1d<Coords>::value)
      coord_grad_1d_kernel<T><<<grid_1d((long long)nb * g.G * g.K * g.V, 256), 256, 0, st>>>(
          g, coords, b0, nb, dcol, x, mask, grad_coord, grad_mask);
    else
      coord_grad_generic_kernel<T, Coords, FieldOut>
          <<<grid_1d((long long)nb * g.G * g.K * g.V, 256), 256, 0, st>>>(g, coords, b0, nb, dcol, x, mask,
                                                                         grad_coord, grad_mask);
    D2C_LAUNCH_CHECK();
    prof_mark(st, "bwd_col2im_generic");
    col2im_generic_kernel<T, Coords>
        <<<grid_1d((long long)nb * g.Cin * g.K * g.V, 256), 256, 0, st>>>(g, coords, b0, nb, dcol, mask, grad_x);
    D2C_LAUNCH_CHECK();
  }
  {
    // split the voxel reduction so that the grid fills the GPU
    const int tiles = ((R + kTileV - 1) / kTileV) * ((g.cout_g + kTileN - 1) / kTileN) * g.groups * g.B;
    int nsplit = (148 * 4 + tiles - 1) / tiles;
    const int max_split = (g.V + 4 * kTileR - 1) / (4 * kTileR);
    if (nsplit > max_split) nsplit = max_split;
    if (nsplit < 1) nsplit = 1;
    int v_per_split = (g.V + nsplit - 1) / nsplit;
    v_per_split = (v_per_split + kTileR - 1) / kTileR * kTileR;
    nsplit = (g.V + v_per_split - 1) / v_per_split;
    dim3 grid((R + kTileV - 1) / kTileV, (g.cout_g + kTileN - 1) / kTileN, g.B * g.groups * nsplit);
    if (grid.y > 65535 || grid.z > 65535) return D2C_ERR_TOO_LARGE;
    prof_mark(st, "bwd_dw_generic");
    dw_generic_kernel<T, Coords><<<grid, kGemmThreads, 0, st>>>(g, coords, v_per_split, gy, x, mask, grad_w);
    D2C_LAUNCH_CHECK();
  }
  if (grad_bias) {
    prof_mark(st, "bwd_grad_bias");
    grad_bias_kernel<T><<<g.Cout, 256, 0, st>>>(g.B, g.Cout, g.V, gy, grad_bias);
    D2C_LAUNCH_CHECK();
  }
  prof_mark(st, nullptr);
  return D2C_OK;
}

}  // namespace d2c
