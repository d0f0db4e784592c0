/*
 * d2conv3d.h -- C ABI of libd2conv3d.so
 *
 * B200 (sm_100a) implementation of the D2Conv3D hot path: modulated deformable
 * conv3d, dynamic-dilated ("size conditioned") conv3d and channel-separated
 * depthwise conv3d, forward and backward.
 *
 * Conventions shared by every entry point
 *   - All tensor pointers are DEVICE pointers owned by the caller, contiguous
 *     NCDHW, element type given by `dtype`.  Nullable pointers are marked.
 *   - Nothing here allocates device memory: scratch is a caller-supplied
 *     workspace of at least d2c_workspace_bytes() bytes (256-byte aligned).
 *   - Every launch goes to the caller-supplied stream; calls are asynchronous.
 *   - Return value: 0 = ok, negative = invalid argument (nothing launched),
 *     positive = CUDA runtime / device-side failure.  Nothing throws or aborts.
 *     d2c_status_string() turns a code into text.
 *
 * Each declaration cites the interface of the reference extension
 * (Schmiddo/d2conv3d, paths relative to that project) that it stands in for.
 */
#ifndef D2CONV3D_H_
#define D2CONV3D_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Opaque to this header so that C callers need no CUDA headers. */
typedef void* d2c_stream_t; /* a cudaStream_t */
typedef void* d2c_event_t;  /* a cudaEvent_t */

enum d2c_dtype { D2C_F32 = 0, D2C_F64 = 1, D2C_F16 = 2 /* depthwise only */ };

/* How the Cin*K x Cout contraction of the deformable ops is evaluated.
 *   D2C_MATH_FP32   fp32 (or fp64) FMA pipeline; matches a cuBLAS S/Dgemm up to
 *                   summation order.  Always used for fp64.
 *   D2C_MATH_BF16X3 tcgen05 bf16 tensor cores, each fp32 operand split into
 *                   hi+lo bf16 (3 MMA passes, fp32 accumulate): ~2^-16 relative
 *                   operand error, keeps the 1e-4 parity bound.
 *   D2C_MATH_BF16   single-pass bf16 operands, fp32 accumulate (looser bound).
 *   D2C_MATH_AUTO   BF16X3 where the tensor-core kernels apply, else FP32.
 */
enum d2c_math_mode { D2C_MATH_AUTO = 0, D2C_MATH_FP32 = 1, D2C_MATH_BF16X3 = 2, D2C_MATH_BF16 = 3 };

/* Dilation-field layouts; names follow utils/grid.py:72-98 (`mode`). */
enum d2c_field_mode {
  D2C_FIELD_X = 0,   /* 1 channel  s      -> (1, s, s)       "xx1" scripts */
  D2C_FIELD_XY = 1,  /* 2 channels (y,x)  -> (1, s_y, s_x)   "xy1" scripts */
  D2C_FIELD_XXZ = 2, /* 2 channels (z,x)  -> (s_z, s_x, s_x)               */
  D2C_FIELD_XYZ = 3  /* 3 channels (z,y,x)                                 */
};

/* Activations of the deformation head (see d2c_head_desc).  Names follow network/layers.py:19-25 and :171-181. */
enum d2c_mask_act { D2C_MASK_LINEAR = 0, D2C_MASK_SIGMOID = 1, D2C_MASK_RELU = 2, D2C_MASK_TANH = 3 };
enum d2c_size_act {
  D2C_SIZE_LINEAR = 0,       /* s = r                  */
  D2C_SIZE_ELU = 1,          /* s = elu(r) + 1         */
  D2C_SIZE_RELU = 2,         /* s = relu(r + 1)        */
  D2C_SIZE_RELU_PLUS_ONE = 3 /* s = relu(r + 1e-3) + 1 */
};

enum d2c_status {
  D2C_OK = 0,
  D2C_ERR_NULL = -1,          /* required pointer is NULL */
  D2C_ERR_DTYPE = -2,         /* dtype not supported by this op */
  D2C_ERR_SHAPE = -3,         /* non-positive size / stride / dilation, negative pad */
  D2C_ERR_GROUPS = -4,        /* channel counts not divisible by groups / offset_groups */
  D2C_ERR_OUT_DIMS = -5,      /* computed output size is not positive */
  D2C_ERR_OFFSET_SHAPE = -6,  /* offset channels != G*3*K or spatial dims != output dims */
  D2C_ERR_MASK_SHAPE = -7,    /* mask channels != G*K or spatial dims != output dims */
  D2C_ERR_WORKSPACE = -8,     /* workspace NULL, misaligned or too small */
  D2C_ERR_TOO_LARGE = -9,     /* a tensor exceeds the 2^31-1 element index range of the op */
  D2C_ERR_MODE = -10,         /* unknown math / field mode */
  D2C_ERR_WEIGHT_SHAPE = -11, /* weight.size(1)*groups != Cin, or depthwise weight rule */
  D2C_ERR_SCRATCH_LIMIT = -12,/* problem needs more scratch than the library's built-in buffer holds */
  D2C_ERR_CUDA = 1,           /* a CUDA runtime call failed (see d2c_last_cuda_error) */
  D2C_ERR_DEVICE_TIMEOUT = 2  /* a bounded device-side wait gave up */
};

/* Geometry of one convolution call.
 * Stands in for the positional int arguments of
 * dconv_native._ops.deform_conv3d (csrc/ops/dconv3d.h:188-205) plus the sizes
 * the reference reads from its tensors (csrc/ops/dconv3d_gpu.cu:477-502). */
typedef struct d2c_conv_desc {
  int32_t dtype;                /* d2c_dtype */
  int32_t batch;                /* B  (clips) */
  int32_t in_channels;          /* Cin */
  int32_t out_channels;         /* Cout */
  int32_t in_d, in_h, in_w;     /* input D,H,W */
  int32_t kd, kh, kw;           /* weight.size(2..4) */
  int32_t stride_d, stride_h, stride_w;
  int32_t pad_d, pad_h, pad_w;
  int32_t dil_d, dil_h, dil_w;
  int32_t groups;               /* weight groups  (n_weight_groups) */
  int32_t offset_groups;        /* deformable groups (n_offset_groups) */
} d2c_conv_desc;

enum d2c_op {
  D2C_OP_DEFORM_FWD = 0,
  D2C_OP_DEFORM_BWD = 1,
  D2C_OP_DYNDIL_FWD = 2,
  D2C_OP_DYNDIL_BWD = 3,
  D2C_OP_DEPTHWISE_FWD = 4,
  D2C_OP_DEPTHWISE_BWD = 5
};

/* ---- helpers ------------------------------------------------------------ */

/* get_output_size, csrc/ops/dconv_gpu_common.h:13-15, for the three dims. */
int d2c_output_dims(const d2c_conv_desc* desc, int32_t out_dhw[3]);

/* The argument checks of deform_conv3d_forward_cuda
 * (csrc/ops/dconv_gpu_common.h:17-51, csrc/ops/dconv3d_gpu.cu:472-527) on
 * sizes only.  offset_dims / mask_dims are {channels, D, H, W} of the offset
 * and mask tensors; mask_dims may be NULL when no mask is given. */
int d2c_deform_conv3d_check(const d2c_conv_desc* desc, const int64_t offset_dims[4],
                            const int64_t mask_dims[4]);

/* Scratch bytes needed by `op` (enum d2c_op) for this geometry under the
 * current math mode and intermediate-element cap. */
size_t d2c_workspace_bytes(int op, const d2c_conv_desc* desc);

const char* d2c_status_string(int status);
/* Text of the last CUDA runtime error seen by this thread ("" if none). */
const char* d2c_last_cuda_error(void);

/* Process-wide math mode (enum d2c_math_mode); returns status. */
int d2c_set_math_mode(int mode);
int d2c_get_math_mode(void);

/* Device-side failure reporting.  Every wait inside the kernels is bounded; a kernel
 * whose wait gave up returns early (its outputs are then incomplete) and raises the
 * current device's status word, which lives in page-locked host memory.
 *   - Every compute entry point first looks at that word (a host memory read, no
 *     synchronisation): if it is raised, the call launches nothing, returns
 *     D2C_ERR_DEVICE_TIMEOUT once and clears the word.  So a failure surfaces at the
 *     next library call on that device at the latest.
 *   - d2c_device_status() synchronises with the device first and then reports and
 *     clears in the same way: call it after a step whose results must be trusted.
 *   - d2c_device_status_peek() reports without synchronising or clearing;
 *     d2c_device_status_clear() clears without reporting.
 * The reference has no counterpart: its kernels have no waits (launch failures are
 * only printed, csrc/ops/dconv3d_gpu.cu:259-262). */
int d2c_device_status(void);
int d2c_device_status_peek(void);
void d2c_device_status_clear(void);

/* Self-test of the reporting path: launches a one-warp kernel that waits `budget_us`
 * microseconds (1 .. 100000) on a barrier nobody arrives on, gives up and raises the
 * status word; the kernel returns normally and the context stays usable.  Expect
 * d2c_device_status() == D2C_ERR_DEVICE_TIMEOUT afterwards, once. */
int d2c_selftest_wait_expiry(uint32_t budget_us, d2c_stream_t stream);

/* Number of kernels this library has launched in this process so far. */
uint64_t d2c_launch_count(void);

/* Phase timing, the library's counterpart of the reference's `Timer` helper
 * (utils/util.py:27-53) and benchmark loop (csrc/benchmark.cpp:13-25): while
 * enabled, every entry point brackets its phases (kernels or kernel groups) with
 * CUDA events recorded on the caller's stream.  d2c_profile_read synchronises with
 * the last event, writes up to `max_records` {name, milliseconds} pairs in launch
 * order, stores the count in *n_records and clears the log. */
typedef struct d2c_profile_record {
  const char* name; /* static string owned by the library */
  float ms;
} d2c_profile_record;
int d2c_profile_enable(int on);
int d2c_profile_read(d2c_profile_record* records, int max_records, int* n_records);

/* dconv_native._ops.config.{get,set}_max_intermediate_elements
 * (csrc/ops/dconv.cpp:9-11, csrc/ops/dconv3d_gpu.cu:12-14).  Here it caps the
 * element count of the backward's gradient-column scratch; larger problems are
 * processed in batch slices. */
uint64_t d2c_get_max_intermediate_elements(void);
void d2c_set_max_intermediate_elements(uint64_t n);

/* ---- samples handed from the forward to the backward ---------------------- */

/* The reference builds the column matrix of trilinear samples twice per training step: deformable_im2col in the
 * forward (csrc/ops/dconv3d_gpu.cu:111-203) and again for the weight gradient in the backward (:1037-1060).  On the
 * tensor-core tier the forward can instead KEEP its blended operand tiles (16-bit, the byte image its tensor-core
 * operand has in shared memory) in a caller-owned buffer, and the weight gradient of the matching backward call
 * streams them back with bulk copies: no second gather, no second blend.
 *
 *   d2c_sample_cache c = { buf, d2c_sample_cache_bytes(&desc), 0, 0 };
 *   d2c_bind_sample_cache(&c);  d2c_deform_conv3d_fwd(...);       -- fills buf, sets c.format (0 = nothing kept)
 *   ...
 *   d2c_bind_sample_cache(&c);  d2c_deform_conv3d_bwd_ev(...);    -- reads buf when c.format fits the call
 *
 * d2c_bind_sample_cache applies to the NEXT deformable / dilation-field (plain or *_head) forward or backward call
 * made by the calling thread and is consumed by it, whatever that call returns; `cache` must stay valid until that
 * call has returned and `data` until the backward's work on the stream is done.  Binding NULL unbinds.  A call that
 * cannot use the cache (CUDA-core tier, math mode changed between the two calls, buffer too small) ignores it, so
 * results never depend on it being there; x, offsets / field / raw head output and mask passed to the backward
 * must be the forward's, as for any backward call.
 * d2c_sample_cache_bytes: bytes to allocate (256-byte aligned) for this shape under the current math mode and
 * intermediate-element cap (the image holds batch*Cin*K*V elements; shapes above the cap keep nothing): 0 when the
 * call pair would not use a cache. */
typedef struct d2c_sample_cache {
  void* data;
  size_t bytes;
  int32_t format;    /* written by the forward: 0 nothing kept, otherwise the image format */
  int32_t reserved;
} d2c_sample_cache;
size_t d2c_sample_cache_bytes(const d2c_conv_desc* desc);
int d2c_bind_sample_cache(d2c_sample_cache* cache);

/* ---- modulated deformable conv3d ----------------------------------------- */

/* deform_conv3d_forward_cuda, csrc/ops/dconv3d_gpu.cu:460-560.
 *   x      [B, Cin, D, H, W]
 *   offset [B, G*3*K, Do, Ho, Wo]   channel 3*(g*K+tap)+{0:z,1:y,2:x}
 *   mask   [B, G*K,   Do, Ho, Wo]   nullable (== all ones)
 *   w      [Cout, Cin/groups, kd, kh, kw]
 *   bias   [Cout]                   nullable
 *   y      [B, Cout, Do, Ho, Wo]    fully overwritten */
int d2c_deform_conv3d_fwd(const d2c_conv_desc* desc, const void* x, const void* offset,
                          const void* mask, const void* w, const void* bias, void* y,
                          void* workspace, size_t workspace_bytes, d2c_stream_t stream);

/* deform_conv3d_backward_cuda, csrc/ops/dconv3d_gpu.cu:1261-1332.
 * All five gradients are fully overwritten (no pre-zeroing needed).
 * grad_mask is ignored when mask is NULL; grad_bias may be NULL. */
int d2c_deform_conv3d_bwd(const d2c_conv_desc* desc, const void* grad_y, const void* x,
                          const void* offset, const void* mask, const void* w, void* grad_x,
                          void* grad_offset, void* grad_mask, void* grad_w, void* grad_bias,
                          void* workspace, size_t workspace_bytes, d2c_stream_t stream);

/* Same as d2c_deform_conv3d_bwd, plus an event (nullable) that is recorded on `stream` as soon as grad_w and
 * grad_bias hold their final values.  On the tensor-core tier the weight gradient runs first, so a data-parallel
 * caller can wait for the event on a second stream and all-reduce the parameter gradients while the data-side
 * backward (grad_x, grad_offset, grad_mask) is still running -- what the reference gets from DistributedDataParallel's
 * bucketed overlap (trainer.py:111).  On the CUDA-core tier the event fires at the end of the call. */
int d2c_deform_conv3d_bwd_ev(const d2c_conv_desc* desc, const void* grad_y, const void* x,
                             const void* offset, const void* mask, const void* w, void* grad_x,
                             void* grad_offset, void* grad_mask, void* grad_w, void* grad_bias,
                             void* workspace, size_t workspace_bytes, d2c_stream_t stream,
                             d2c_event_t params_ready);

/* Parity probe: the integer corner (floor) coordinates the kernels use.
 * Same coordinate formation as csrc/ops/dconv3d_gpu.cu:192-194 followed by the
 * floor of :63-65.  corners is int32 [B, G*K, 3, Do*Ho*Wo] (z0, y0, x0). */
int d2c_deform_conv3d_corners(const d2c_conv_desc* desc, const void* offset, int32_t* corners,
                              d2c_stream_t stream);

/* ---- modulated deformable conv1d ------------------------------------------ */

/* deform_conv1d_forward_cuda / deform_conv1d_backward_cuda, csrc/ops/dconv1d_gpu.cu:101-198, :351-538
 * (dconv_native._ops.deform_conv1d).  The descriptor describes the [B, C, 1, 1, L] view of the problem:
 * in_d = in_h = 1, kd = kh = 1, stride_d = stride_h = 1, pad_d = pad_h = 0 (anything else: D2C_ERR_SHAPE);
 * in_w = L, kw = K, stride_w / pad_w / dil_w the 1-D geometry.
 *   x [B, Cin, L]   offset [B, G*K, Lo]   mask [B, G*K, Lo] nullable   w [Cout, Cin/groups, K]   bias nullable
 * Linear interpolation with out-of-range neighbours read as zero.  The backward follows the 1-D reference's own
 * rule at sampling positions within 1e-8 of an integer (:334-337): there the left neighbour is taken one cell
 * further left, so grad_offset is mask * (x[p+1] - x[p-1]) * dcol and grad_mask uses the right cell's value.
 * fp32 / fp64, CUDA-core kernels.  Workspace of the backward: d2c_workspace_bytes(D2C_OP_DEFORM_BWD, desc). */
int d2c_deform_conv1d_fwd(const d2c_conv_desc* desc, const void* x, const void* offset, const void* mask,
                          const void* w, const void* bias, void* y, d2c_stream_t stream);
int d2c_deform_conv1d_bwd(const d2c_conv_desc* desc, const void* grad_y, const void* x, const void* offset,
                          const void* mask, const void* w, void* grad_x, void* grad_offset, void* grad_mask,
                          void* grad_w, void* grad_bias, void* workspace, size_t workspace_bytes,
                          d2c_stream_t stream);

/* ---- dynamic-dilated conv3d (dilation field instead of offsets) ---------- */

/* Fuses offsets_from_size_map (utils/grid.py:72-98; older copy
 * ops/dconv-native/src/dconv_native/grid.py:62-80) into the deformable conv:
 *   offset[b, 3*tap+d, v] = base[d][tap] * (s_d[b, v] - 1)
 * with base = linspace(-dil*(k/2), dil*(k/2), k) per dim, evaluated with the
 * same two roundings, and never materialised.
 *   size_map [B, {1,2,2,3}, Do, Ho, Wo] per `field_mode`; one field shared by
 *   all offset groups; mask [B, G*K, Do,Ho,Wo] nullable. */
int d2c_dyn_dilated_conv3d_fwd(const d2c_conv_desc* desc, int field_mode, const void* x,
                               const void* size_map, const void* mask, const void* w,
                               const void* bias, void* y, void* workspace,
                               size_t workspace_bytes, d2c_stream_t stream);

/* Backward of the above; grad_size_map has the shape of size_map and equals
 * the autograd gradient through offsets_from_size_map of the reference's
 * grad_offset (sum over taps, offset groups and shared dims). */
int d2c_dyn_dilated_conv3d_bwd(const d2c_conv_desc* desc, int field_mode, const void* grad_y,
                               const void* x, const void* size_map, const void* mask,
                               const void* w, void* grad_x, void* grad_size_map,
                               void* grad_mask, void* grad_w, void* grad_bias, void* workspace,
                               size_t workspace_bytes, d2c_stream_t stream);

/* d2c_dyn_dilated_conv3d_bwd with the parameter-gradient event of d2c_deform_conv3d_bwd_ev. */
int d2c_dyn_dilated_conv3d_bwd_ev(const d2c_conv_desc* desc, int field_mode, const void* grad_y,
                                  const void* x, const void* size_map, const void* mask,
                                  const void* w, void* grad_x, void* grad_size_map, void* grad_mask,
                                  void* grad_w, void* grad_bias, void* workspace,
                                  size_t workspace_bytes, d2c_stream_t stream, d2c_event_t params_ready);

/* Corner probe for the field path (see d2c_deform_conv3d_corners). */
int d2c_dyn_dilated_conv3d_corners(const d2c_conv_desc* desc, int field_mode,
                                   const void* size_map, int32_t* corners, d2c_stream_t stream);

/* ---- deformation head fused into the op ------------------------------------ */

/* The reference's layers (network/layers.py:107-120 MDConv3d, :171-181 size activations, :302-313
 * XYZSizeConditionedMDConv3d and their siblings) run a predictor convolution, split its output `raw`
 * [B, raw_channels, Do, Ho, Wo] into geometry channels (3*G*K offsets, or the 1..3 channels of a dilation field)
 * and G*K mask logits, apply sigmoid / relu / tanh to the logits and elu+1 / ... to the field, and only then call
 * the op -- four elementwise passes over tensors as large as the offsets.  The *_head entry points take `raw` as it
 * leaves the predictor: the kernels read its channels in place, activate where they read, and the backward writes
 * grad_raw (same shape as raw, every channel, chain rule through the activations included).  On the tensor-core
 * tier nothing activated is ever written to memory; on the CUDA-core tier the library stages the activated
 * tensors in the workspace itself. */
typedef struct d2c_head_desc {
  int32_t raw_channels;   /* channels of `raw` */
  int32_t geo_channel0;   /* first geometry channel: 3*G*K offset channels, or the field's 1..3 channels */
  int32_t mask_channel0;  /* first of the G*K mask-logit channels; -1 = no mask */
  int32_t mask_act;       /* enum d2c_mask_act */
  int32_t size_act;       /* enum d2c_size_act; dilation-field entry points only */
} d2c_head_desc;

/* Workspace of the four entry points below: `op` is D2C_OP_DEFORM_FWD / _BWD / D2C_OP_DYNDIL_FWD / _BWD. */
size_t d2c_head_workspace_bytes(int op, const d2c_conv_desc* desc, const d2c_head_desc* head, int field_mode);

int d2c_deform_conv3d_head_fwd(const d2c_conv_desc* desc, const d2c_head_desc* head, const void* x, const void* raw,
                               const void* w, const void* bias, void* y, void* workspace, size_t workspace_bytes,
                               d2c_stream_t stream);
int d2c_deform_conv3d_head_bwd(const d2c_conv_desc* desc, const d2c_head_desc* head, const void* grad_y, const void* x,
                               const void* raw, const void* w, void* grad_x, void* grad_raw, void* grad_w,
                               void* grad_bias, void* workspace, size_t workspace_bytes, d2c_stream_t stream,
                               d2c_event_t params_ready);
int d2c_dyn_dilated_conv3d_head_fwd(const d2c_conv_desc* desc, const d2c_head_desc* head, int field_mode, const void* x,
                                    const void* raw, const void* w, const void* bias, void* y, void* workspace,
                                    size_t workspace_bytes, d2c_stream_t stream);
int d2c_dyn_dilated_conv3d_head_bwd(const d2c_conv_desc* desc, const d2c_head_desc* head, int field_mode,
                                    const void* grad_y, const void* x, const void* raw, const void* w, void* grad_x,
                                    void* grad_raw, void* grad_w, void* grad_bias, void* workspace,
                                    size_t workspace_bytes, d2c_stream_t stream, d2c_event_t params_ready);

/* ---- depthwise conv3d ------------------------------------------------------ */

/* For the depthwise entry points desc->groups is ignored (groups == Cin),
 * out_channels must be a multiple of in_channels (channel multiplier) and
 * w is [Cout, 1, kd, kh, kw]; dtype may be F16/F32/F64. */

/* conv_depthwise3d_cuda, csrc/grouped_conv3d.cu:385-449
 * (fast_depthwise_conv3d._ops.depthwise_separable_conv3d forward). */
int d2c_depthwise_conv3d_fwd(const d2c_conv_desc* desc, const void* x, const void* w,
                             const void* bias, void* y, d2c_stream_t stream);

/* conv_depthwise3d_backward_cuda, csrc/grouped_conv3d.cu:513-678.  Any of
 * grad_x / grad_w / grad_bias may be NULL (the reference's output_mask). */
int d2c_depthwise_conv3d_bwd(const d2c_conv_desc* desc, const void* grad_y, const void* x,
                             const void* w, void* grad_x, void* grad_w, void* grad_bias,
                             void* workspace, size_t workspace_bytes, d2c_stream_t stream);

/* y = GroupNorm(act(x)) for a contiguous fp32 NCDHW tensor, act = relu when
 * apply_relu != 0 else identity.  Replaces the `ActivationType(), NormType(planes)` tail of every conv unit of
 * the reference's refine blocks (network/modules/refinement.py:38-43 with NormType = GroupNorm,
 * network/segmentation/encoder_decoder.py:116-119) as two grid-wide streaming passes; statistics follow
 * torch.nn.GroupNorm (biased variance over the group's channels x voxels, eps inside the square root);
 * gamma / beta [channels] may be NULL (1 / 0).  x and y must not overlap.  workspace: see the size function. */
size_t d2c_act_group_norm_workspace_bytes(int batch, int groups);
/* Backward of the same unit: grad_x (and, when not NULL, grad_gamma / grad_beta [channels]) from grad_y.
 * fwd_stats = the forward call's workspace, kept unchanged since (it holds the per-(clip, group) sums). */
size_t d2c_act_group_norm_bwd_workspace_bytes(int batch, int channels, int groups);
int d2c_act_group_norm_bwd(const float* x, const float* gamma, const float* grad_y, const void* fwd_stats,
                           float* grad_x, float* grad_gamma, float* grad_beta, int batch, int channels,
                           long long spatial, int groups, float eps, int apply_relu, void* workspace,
                           size_t workspace_bytes, d2c_stream_t stream);
int d2c_act_group_norm_fwd(const float* x, const float* gamma, const float* beta, float* y, int batch, int channels,
                           long long spatial, int groups, float eps, int apply_relu, void* workspace,
                           size_t workspace_bytes, d2c_stream_t stream);

/* No counterpart in the reference.  Same results as d2c_depthwise_conv3d_bwd, for callers that
 * have no device memory to give and may not allocate any: a process that planned its whole device-memory
 * budget at start-up (e.g. a server sharing the GPU with other tenants) or a latency-critical loop in
 * which cudaMalloc/cudaFree, which synchronise the device, are not acceptable.  The weight-gradient
 * accumulators live in a 256 KB array inside the library (held by every GPU that loads the library,
 * until the process exits) instead of a workspace; the call itself allocates nothing.
 *   - Limit: out_channels * kd*kh*kw <= 32768 when grad_w is requested, else D2C_ERR_SCRATCH_LIMIT.
 *   - The first call on each device looks up the array's device address (one-time set-up); make that
 *     first call before any stream capture is started on that device.
 *   - All calls on a device share the array: calls whose GPU work can overlap (different streams, or
 *     several host threads) race on it.  Issue them on one stream, or otherwise order them.
 *   - Keep phase profiling (d2c_profile_enable) off: it creates CUDA events. */
int d2c_depthwise_conv3d_bwd_noalloc(const d2c_conv_desc* desc, const void* grad_y, const void* x,
                                     const void* w, void* grad_x, void* grad_w, void* grad_bias,
                                     d2c_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* D2CONV3D_H_ */
