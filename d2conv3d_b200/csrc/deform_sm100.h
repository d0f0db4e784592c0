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

// Weight gradient (implicit GEMM over the sampled tile).  x_cl = channels-last bf16 staging of x,
// recs = the call's sampling records (float4 {z, y, x, mask} per (clip, group, tap, voxel)).
size_t sm100_dw_workspace(const Geom& g, bool x3);
// grad_bias (nullable, zeroed by the caller) is accumulated by the staging pass over grad_out.
int sm100_dw(const Geom& g, bool x3, const float* gy, const void* x_cl, const void* recs, float* grad_w,
             float* grad_bias, void* ws, cudaStream_t st);

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
