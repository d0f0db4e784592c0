// The C++ side of the drop-in: definitions of the four functions that the reference's extension declares in
// csrc/ops/dconv3d_gpu.h:5-30 and csrc/ops/dconv1d_gpu.h:6-33 (and implements in dconv3d_gpu.cu / dconv1d_gpu.cu),
// written on top of the C ABI of libd2conv3d.so.  Compiled together with the reference's UNMODIFIED dconv.cpp,
// dconv3d.h and dconv1d.h (baseline/build_binding.py), it yields a `_ops` module whose pybind signatures and
// autograd nodes (DeformConv3dFunction, csrc/ops/dconv3d.h:70-186; DeformConv1dFunction, dconv1d.h:69-156) are
// the reference's own while every kernel is this library's.  Test infrastructure: it shows a maintainer of the
// reference the two .cu files that this library replaces and nothing else.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/torch.h>

#include <tuple>

#include "d2conv3d.h"

namespace {

using Triple = std::tuple<int, int, int>;

d2c_conv_desc make_desc(const at::Tensor& x, const at::Tensor& w, Triple s, Triple p, Triple d, int groups,
                        int offset_groups) {
  d2c_conv_desc c{};
  TORCH_CHECK(x.scalar_type() == at::kFloat || x.scalar_type() == at::kDouble,
              "\"deform_conv3d\" not implemented for '", x.scalar_type(), "'");
  c.dtype = x.scalar_type() == at::kDouble ? D2C_F64 : D2C_F32;
  c.batch = (int32_t)x.size(0); c.in_channels = (int32_t)x.size(1); c.out_channels = (int32_t)w.size(0);
  c.in_d = (int32_t)x.size(2); c.in_h = (int32_t)x.size(3); c.in_w = (int32_t)x.size(4);
  c.kd = (int32_t)w.size(2); c.kh = (int32_t)w.size(3); c.kw = (int32_t)w.size(4);
  std::tie(c.stride_d, c.stride_h, c.stride_w) = s;
  std::tie(c.pad_d, c.pad_h, c.pad_w) = p;
  std::tie(c.dil_d, c.dil_h, c.dil_w) = d;
  c.groups = groups; c.offset_groups = offset_groups;
  return c;
}

void check(int rc, const char* what) {
  TORCH_CHECK(rc == 0, what, ": ", d2c_status_string(rc), rc > 0 ? " / " : "", rc > 0 ? d2c_last_cuda_error() : "");
}

void* ptr(const at::Tensor& t) { return t.defined() ? t.data_ptr() : nullptr; }

at::Tensor workspace(int op, const d2c_conv_desc& c, const at::Tensor& like, size_t* bytes) {
  *bytes = d2c_workspace_bytes(op, &c);
  return at::empty({(int64_t)(*bytes ? *bytes : 1)}, like.options().dtype(at::kByte));
}

// the reference's argument checks that do not depend on a kernel (csrc/ops/dconv_gpu_common.h:26-44)
void sanity(const at::Tensor& x, const at::Tensor& off, const at::Tensor& m, const at::Tensor& w, const at::Tensor& b,
            int nd) {
  TORCH_CHECK(x.ndimension() == nd && off.ndimension() == nd && w.ndimension() == nd);
  TORCH_CHECK(!m.defined() || m.ndimension() == nd);
  TORCH_CHECK(!b.defined() || b.ndimension() == 1);
  TORCH_CHECK(x.device().is_cuda() && off.device().is_cuda() && w.device().is_cuda());
  TORCH_CHECK(!m.defined() || m.device().is_cuda());
  TORCH_CHECK(!b.defined() || b.device().is_cuda());
  TORCH_CHECK(off.size(0) == x.size(0));
  TORCH_CHECK(!m.defined() || m.size(0) == x.size(0));
}

}  // namespace

size_t get_max_intermediate_elements() { return (size_t)d2c_get_max_intermediate_elements(); }
void set_max_intermediate_elements(size_t m) { d2c_set_max_intermediate_elements((uint64_t)m); }

at::Tensor deform_conv3d_forward_cuda(const at::Tensor& input, const at::Tensor& offset, const at::Tensor& alpha,
                                      const at::Tensor& weight, const at::Tensor& bias, Triple stride, Triple pad,
                                      Triple dilation, int n_weight_groups, int n_offset_groups) {
  sanity(input, offset, alpha, weight, bias, 5);
  TORCH_CHECK(weight.size(1) * n_weight_groups == input.size(1));
  c10::cuda::CUDAGuard guard(input.device());
  d2c_conv_desc c = make_desc(input, weight, stride, pad, dilation, n_weight_groups, n_offset_groups);
  int64_t od[4] = {offset.size(1), offset.size(2), offset.size(3), offset.size(4)};
  int64_t md[4] = {0, 0, 0, 0};
  if (alpha.defined()) for (int i = 0; i < 4; ++i) md[i] = alpha.size(i + 1);
  check(d2c_deform_conv3d_check(&c, od, alpha.defined() ? md : nullptr), "deform_conv3d");
  int32_t o[3];
  check(d2c_output_dims(&c, o), "deform_conv3d");
  auto y = at::empty({input.size(0), weight.size(0), o[0], o[1], o[2]}, input.options());
  size_t ws_bytes;
  auto ws = workspace(D2C_OP_DEFORM_FWD, c, input, &ws_bytes);
  check(d2c_deform_conv3d_fwd(&c, ptr(input), ptr(offset), ptr(alpha), ptr(weight), ptr(bias), ptr(y),
                              ws_bytes ? ws.data_ptr() : nullptr, ws_bytes, at::cuda::getCurrentCUDAStream().stream()),
        "deform_conv3d forward");
  return y;
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor> deform_conv3d_backward_cuda(
    const at::Tensor& grad_out, const at::Tensor& input, const at::Tensor& offset, const at::Tensor& alpha,
    const at::Tensor& weight, const at::Tensor& bias, Triple stride, Triple pad, Triple dilation, int n_weight_groups,
    int n_offset_groups) {
  c10::cuda::CUDAGuard guard(input.device());
  d2c_conv_desc c = make_desc(input, weight, stride, pad, dilation, n_weight_groups, n_offset_groups);
  // the library overwrites every gradient completely: no zero-fill; undefined tensors for a missing mask / bias
  // as csrc/ops/dconv3d_gpu.cu:1305-1331 returns them
  auto gx = at::empty_like(input), goff = at::empty_like(offset), gw = at::empty_like(weight);
  at::Tensor gm = alpha.defined() ? at::empty_like(alpha) : at::Tensor();
  at::Tensor gb = bias.defined() ? at::empty_like(bias) : at::Tensor();
  size_t ws_bytes;
  auto ws = workspace(D2C_OP_DEFORM_BWD, c, input, &ws_bytes);
  check(d2c_deform_conv3d_bwd(&c, ptr(grad_out), ptr(input), ptr(offset), ptr(alpha), ptr(weight), ptr(gx), ptr(goff),
                              ptr(gm), ptr(gw), ptr(gb), ws_bytes ? ws.data_ptr() : nullptr, ws_bytes,
                              at::cuda::getCurrentCUDAStream().stream()),
        "deform_conv3d backward");
  return std::make_tuple(gx, goff, gm, gw, gb);
}

namespace {
d2c_conv_desc make_desc_1d(const at::Tensor& x, const at::Tensor& w, int stride, int pad, int dil, int groups,
                           int offset_groups) {
  d2c_conv_desc c{};
  TORCH_CHECK(x.scalar_type() == at::kFloat || x.scalar_type() == at::kDouble);
  c.dtype = x.scalar_type() == at::kDouble ? D2C_F64 : D2C_F32;
  c.batch = (int32_t)x.size(0); c.in_channels = (int32_t)x.size(1); c.out_channels = (int32_t)w.size(0);
  c.in_d = c.in_h = 1; c.in_w = (int32_t)x.size(2);
  c.kd = c.kh = 1; c.kw = (int32_t)w.size(2);
  c.stride_d = c.stride_h = 1; c.stride_w = stride;
  c.pad_d = c.pad_h = 0; c.pad_w = pad;
  c.dil_d = c.dil_h = 1; c.dil_w = dil;
  c.groups = groups; c.offset_groups = offset_groups;
  return c;
}
}  // namespace

at::Tensor deform_conv1d_forward_cuda(const at::Tensor& input, const at::Tensor& offset, const at::Tensor& alpha,
                                      const at::Tensor& weight, const at::Tensor& bias, int stride, int padding,
                                      int dilation, int groups, int offset_groups) {
  sanity(input, offset, alpha, weight, bias, 3);
  c10::cuda::CUDAGuard guard(input.device());
  d2c_conv_desc c = make_desc_1d(input, weight, stride, padding, dilation, groups, offset_groups);
  int32_t o[3];
  check(d2c_output_dims(&c, o), "deform_conv1d");
  TORCH_CHECK(offset.size(2) == o[2], "offset output dims do not match computed dims. Got: ", offset.size(2),
              " but expected: ", o[2]);
  TORCH_CHECK(offset.size(1) == (int64_t)offset_groups * weight.size(2));
  TORCH_CHECK(!alpha.defined() || (alpha.size(2) == o[2] && alpha.size(1) == offset.size(1)),
              "mask output dims do not match computed dims.");
  auto y = at::empty({input.size(0), weight.size(0), o[2]}, input.options());
  check(d2c_deform_conv1d_fwd(&c, ptr(input), ptr(offset), ptr(alpha), ptr(weight), ptr(bias), ptr(y),
                              at::cuda::getCurrentCUDAStream().stream()),
        "deform_conv1d forward");
  return y;
}

std::tuple<at::Tensor, at::Tensor, at::Tensor, at::Tensor, at::Tensor> deform_conv1d_backward_cuda(
    const at::Tensor& grad, const at::Tensor& input, const at::Tensor& offset, const at::Tensor& alpha,
    const at::Tensor& weight, const at::Tensor& bias, int stride, int padding, int dilation, int groups,
    int offset_groups) {
  c10::cuda::CUDAGuard guard(input.device());
  d2c_conv_desc c = make_desc_1d(input, weight, stride, padding, dilation, groups, offset_groups);
  auto gx = at::empty_like(input), goff = at::empty_like(offset), gw = at::empty_like(weight);
  at::Tensor gm = alpha.defined() ? at::empty_like(alpha) : at::Tensor();
  at::Tensor gb = bias.defined() ? at::empty_like(bias) : at::Tensor();
  size_t ws_bytes;
  auto ws = workspace(D2C_OP_DEFORM_BWD, c, input, &ws_bytes);
  check(d2c_deform_conv1d_bwd(&c, ptr(grad), ptr(input), ptr(offset), ptr(alpha), ptr(weight), ptr(gx), ptr(goff),
                              ptr(gm), ptr(gw), ptr(gb), ws_bytes ? ws.data_ptr() : nullptr, ws_bytes,
                              at::cuda::getCurrentCUDAStream().stream()),
        "deform_conv1d backward");
  return std::make_tuple(gx, goff, gm, gw, gb);
}
