// Tensor-core (tcgen05 / TMEM) tier of the deformable conv3d path for sm_100a.
// The API layer asks *_supported() first; unsupported geometries use the generic
// CUDA-core kernels.
#pragma once

#include "d2c_common.cuh"

namespace d2c {

bool sm100_fwd_supported(const Geom& g, int dtype, int math_mode);
size_t sm100_fwd_workspace(const Geom& g, int dtype, int math_mode);
// head: where offsets / field (FieldCoords carries its own stride and activation) and mask are read from and how
// they are activated; HeadCfg{} = the plain op.
int sm100_fwd_offsets(const Geom& g, int math_mode, const float* x, const float* offset,
                      const float* mask, const float* w, const float* bias, float* y, void* ws,
                      cudaStream_t st, const HeadCfg& head = HeadCfg{});
int sm100_fwd_field(const Geom& g, int math_mode, const FieldCoords<float>& fc, const float* x,
                    const float* mask, const float* w, const float* bias, float* y, void* ws,
                    cudaStream_t st, const HeadCfg& head = HeadCfg{});

// Samples handed from a forward call to the backward call of the same layer invocation (same layout as the public
// d2c_sample_cache).  The forward writes its blended operand tiles into `data` and sets `format` (0 = nothing kept,
// 1 = single-pass bf16 image, 2 = bf16 hi/lo image); a backward whose weight-gradient kernel runs in the matching
// mode reads them instead of gathering and blending every sample a second time.
struct SampleCache {
  void* data;
  size_t bytes;
  int32_t format;
  int32_t reserved;
};
// The cache bound to the API call that is running on this thread, or nullptr (d2c_api.cu).
SampleCache* current_sample_cache();
// Image geometry for this shape in this mode: slice pairs of the weight gradient and total bytes; false when the
// weight-gradient kernel does not take the shape.
bool sm100_sample_image_plan(const Geom& g, bool x3, int* n_pairs, size_t* bytes);
// What else the cache carries behind the image, so that the backward stages nothing twice: the channels-last copy of
// x (fp16 / fp32 as the mode wants it) and the sampling-position records {z, y, x, mask} of every sample.
struct SampleCacheLayout {
  size_t image_bytes, x_cl_bytes, pos_bytes;
  size_t total() const { return image_bytes + x_cl_bytes + pos_bytes; }
};
bool sm100_sample_cache_layout(const Geom& g, bool x3, int* n_pairs, SampleCacheLayout* lay);
// Which kernel family (single-pass / hi-lo split) the forward and the backward of this shape run in this mode.
bool sm100_fwd_variant(const Geom& g, int math_mode, bool* x3);
bool sm100_bwd_variant(const Geom& g, int math_mode, unsigned long long cap, bool* x3);

// Weight gradient (implicit GEMM over the sampled tile).  x_cl = channels-last bf16 staging of x,
// recs = the call's sampling records (float4 {z, y, x, mask} per (clip, group, tap, voxel)).
size_t sm100_dw_workspace(const Geom& g, bool x3);
// grad_bias (nullable, zeroed by the caller) is accumulated by the staging pass over grad_out.
// sav (nullable): the forward's sample image for this mode; x_cl and recs are not read then.
int sm100_dw(const Geom& g, bool x3, const float* gy, const void* x_cl, const void* recs, float* grad_w,
             float* grad_bias, void* ws, cudaStream_t st, const void* sav = nullptr);

// `cap` = maximum number of gradient-column elements held at once (clips are processed in chunks).
bool sm100_bwd_supported(const Geom& g, int dtype, int math_mode, unsigned long long cap);
size_t sm100_bwd_workspace(const Geom& g, int dtype, int math_mode, unsigned long long cap);
// params_ready (nullable): recorded on the stream as soon as grad_w and grad_bias are final -- the weight gradient
// runs first, so a caller can start reducing the parameter gradients while the data-side backward still runs.
int sm100_bwd_offsets(const Geom& g, int math_mode, unsigned long long cap, const float* gy, const float* x, const float* offset,
                      const float* mask, const float* w, float* grad_x, float* grad_offset, float* grad_mask,
                      float* grad_w, float* grad_bias, void* ws, cudaStream_t st, cudaEvent_t params_ready,
                      const HeadCfg& head = HeadCfg{});
int sm100_bwd_field(const Geom& g, int math_mode, unsigned long long cap, const FieldCoords<float>& fc, const float* gy,
                    const float* x, const float* mask, const float* w, float* grad_x, float* grad_size_map,
                    size_t grad_size_elems, float* grad_mask, float* grad_w, float* grad_bias, void* ws,
                    cudaStream_t st, cudaEvent_t params_ready, const HeadCfg& head = HeadCfg{});

// Test-only kernel: one warp waits `budget_cycles` on an mbarrier that nobody arrives on, gives up and reports
// through the status word like every product kernel does.
int sm100_selftest_wait_expiry(long long budget_cycles, cudaStream_t st);

}  // namespace d2c
