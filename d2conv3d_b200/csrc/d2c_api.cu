// C ABI of libd2conv3d.so: argument validation, tier selection and launch
// sequencing.  See include/d2conv3d.h for the contract of every entry point.
#include <atomic>
#include <cstring>
#include <mutex>
#include <vector>

#include "d2c_common.cuh"
#include "deform_generic.cuh"
#include "deform_sm100.h"

namespace d2c {

static thread_local char g_last_cuda_error[256] = "";
void set_last_cuda_error(cudaError_t e) {
  std::strncpy(g_last_cuda_error, cudaGetErrorString(e), sizeof(g_last_cuda_error) - 1);
  cudaGetLastError();  // clear the sticky-free error state
}

static std::atomic<unsigned long long> g_launches{0};
void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

struct ProfMark { const char* name; cudaEvent_t ev; };
static std::atomic<bool> g_prof_on{false};
static std::mutex g_prof_mu;
static std::vector<ProfMark> g_prof;
void prof_mark(cudaStream_t st, const char* name) {
  if (!g_prof_on.load(std::memory_order_relaxed)) return;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  if (g_prof.size() >= 65536) return;
  cudaEvent_t ev;
  if (cudaEventCreate(&ev) != cudaSuccess) return;
  cudaEventRecord(ev, st);
  g_prof.push_back({name, ev});
}

static std::atomic<int> g_math_mode{D2C_MATH_AUTO};
// Default of the reference's MAX_INTERMEDIATE_ELEMENTS (csrc/ops/dconv3d_gpu.cu:12).
static std::atomic<unsigned long long> g_max_intermediate{1ull << 32};

// ---- per-device state ---------------------------------------------------------------------------
constexpr int kMaxDevices = 64;

// Status words: one int per device (64 bytes apart) in a page of the library's own image that is page-locked
// and mapped into the devices' address space on first use -- nothing is allocated.  A kernel whose bounded wait
// gave up stores 1 there (sm100_ptx.cuh: report_device_timeout); the host reads it at the start of the next
// library call on that device, reports D2C_ERR_DEVICE_TIMEOUT once and clears it.
struct alignas(4096) StatusPage { volatile int word[kMaxDevices][16]; };
static StatusPage g_status_page;
static std::mutex g_status_mu;
static bool g_status_registered = false;
static int* g_status_dev_ptr[kMaxDevices];

int status_word_device_ptr(int** dev_ptr) {
  int dev = -1;
  D2C_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return D2C_ERR_TOO_LARGE;
  std::lock_guard<std::mutex> lk(g_status_mu);
  if (!g_status_registered) {
    D2C_CUDA_TRY(cudaHostRegister((void*)&g_status_page, sizeof(g_status_page),
                                  cudaHostRegisterMapped | cudaHostRegisterPortable));
    g_status_registered = true;
  }
  if (!g_status_dev_ptr[dev]) {
    void* d = nullptr;
    D2C_CUDA_TRY(cudaHostGetDevicePointer(&d, (void*)&g_status_page.word[dev][0], 0));
    g_status_dev_ptr[dev] = reinterpret_cast<int*>(d);
  }
  *dev_ptr = g_status_dev_ptr[dev];
  return D2C_OK;
}

// Reads and clears the current device's status word.  No synchronisation: sees what finished kernels reported.
static int status_take() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return D2C_OK;
  volatile int* w = &g_status_page.word[dev][0];
  if (*w == 0) return D2C_OK;
  *w = 0;
  return D2C_ERR_DEVICE_TIMEOUT;
}
#define D2C_TAKE_STATUS()                      \
  do {                                         \
    const int _st = ::d2c::status_take();      \
    if (_st) return _st;                       \
  } while (0)

// ---- sample cache binding ------------------------------------------------------------------------
// d2c_bind_sample_cache() parks the caller's cache in a thread-local slot; the next deformable / dilation-field
// forward or backward call of the same thread takes it for its own duration (a forward first marks it empty).
static thread_local SampleCache* g_bound_cache = nullptr;
static thread_local SampleCache* g_current_cache = nullptr;

SampleCache* current_sample_cache() { return g_current_cache; }

namespace {
struct SampleCacheScope {
  explicit SampleCacheScope(bool forward) {
    g_current_cache = g_bound_cache;
    g_bound_cache = nullptr;
    if (forward && g_current_cache) g_current_cache->format = 0;
  }
  ~SampleCacheScope() { g_current_cache = nullptr; }
  SampleCacheScope(const SampleCacheScope&) = delete;
  SampleCacheScope& operator=(const SampleCacheScope&) = delete;
};
}  // namespace

int device_sm_count(int* out) {
  static std::atomic<int> cache[kMaxDevices];
  int dev = -1;
  D2C_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) return D2C_ERR_TOO_LARGE;
  int n = cache[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    D2C_CUDA_TRY(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
    cache[dev].store(n, std::memory_order_relaxed);
  }
  *out = n;
  return D2C_OK;
}

int depthwise_fwd(const Geom& g, int dtype, const void* x, const void* w, const void* bias, void* y,
                  cudaStream_t st);
int depthwise_bwd(const Geom& g, int dtype, const void* gy, const void* x, const void* w, void* gx,
                  void* gw, void* gbias, void* ws, cudaStream_t st);
size_t depthwise_bwd_workspace(const Geom& g);

static size_t dtype_size(int dtype) { return dtype == D2C_F64 ? 8 : (dtype == D2C_F16 ? 2 : 4); }

// torch.linspace(-dil*(k/2), dil*(k/2), k) as get_kernel_grid of the reference
// evaluates it (utils/grid.py:21-25): in float32 whatever the field's dtype,
// ascending from `start` in the first half, descending from `end` in the second.
template <typename T>
static void kernel_axis(int k, int dil, T* out) {
  const float start = (float)(-dil * (k / 2)), end = (float)(dil * (k / 2));
  if (k == 1) { out[0] = (T)start; return; }
  const float step = (end - start) / (float)(k - 1);
  const int half = k / 2;
  for (int i = 0; i < k; ++i)
    out[i] = (T)((i < half) ? start + step * (float)i : end - step * (float)(k - i - 1));
}

static int field_channels(int mode) {
  switch (mode) {
    case D2C_FIELD_X: return 1;
    case D2C_FIELD_XY: case D2C_FIELD_XXZ: return 2;
    case D2C_FIELD_XYZ: return 3;
    default: return -1;
  }
}

// size_map channel feeding dim d (0:z 1:y 2:x), -1 = constant one (utils/grid.py:79-92)
static int field_channel(int mode, int d) {
  switch (mode) {
    case D2C_FIELD_X: return d == 0 ? -1 : 0;
    case D2C_FIELD_XY: return d == 0 ? -1 : d - 1;
    case D2C_FIELD_XXZ: return d == 0 ? 0 : 1;
    default: return d;
  }
}

template <typename T>
static int make_field_coords(const Geom& g, int mode, const void* size_map, FieldCoords<T>* fc) {
  const int nch = field_channels(mode);
  if (nch < 0) return D2C_ERR_MODE;
  if (g.kd > kMaxFieldKernelDim || g.kh > kMaxFieldKernelDim || g.kw > kMaxFieldKernelDim) return D2C_ERR_SHAPE;
  std::memset(fc, 0, sizeof(*fc));
  fc->size_map = (const T*)size_map;
  fc->nch = nch;
  for (int d = 0; d < 3; ++d) fc->ch[d] = field_channel(mode, d);
  kernel_axis<T>(g.kd, g.dd, fc->axis[0]);
  kernel_axis<T>(g.kh, g.dh, fc->axis[1]);
  kernel_axis<T>(g.kw, g.dw, fc->axis[2]);
  return D2C_OK;
}

static bool ws_ok(const void* ws, size_t have, size_t need) {
  if (need == 0) return true;
  return ws != nullptr && (reinterpret_cast<uintptr_t>(ws) % 256) == 0 && have >= need;
}

static size_t generic_bwd_workspace(const Geom& g, int dtype, unsigned long long cap) {
  const int nb = bwd_slice_clips(g, cap);
  return align_up(dtype_size(dtype) * (size_t)nb * g.Cin * g.K * g.V, 256);
}

}  // namespace d2c

using namespace d2c;

extern "C" {

int d2c_output_dims(const d2c_conv_desc* desc, int32_t out_dhw[3]) {
  if (!desc || !out_dhw) return D2C_ERR_NULL;
  Geom g;
  // groups do not influence the output size; validate them only in the op calls
  d2c_conv_desc d = *desc;
  d.groups = 1; d.offset_groups = 1;
  int rc = make_geom(&d, &g, false);
  if (rc) return rc;
  out_dhw[0] = g.Do; out_dhw[1] = g.Ho; out_dhw[2] = g.Wo;
  return D2C_OK;
}

int d2c_deform_conv3d_check(const d2c_conv_desc* desc, const int64_t offset_dims[4],
                            const int64_t mask_dims[4]) {
  if (!desc || !offset_dims) return D2C_ERR_NULL;
  if (desc->dtype != D2C_F32 && desc->dtype != D2C_F64) return D2C_ERR_DTYPE;
  Geom g;
  int rc = make_geom(desc, &g, false);
  if (rc) return rc;
  if (offset_dims[0] != (int64_t)g.G * 3 * g.K || offset_dims[1] != g.Do || offset_dims[2] != g.Ho ||
      offset_dims[3] != g.Wo)
    return D2C_ERR_OFFSET_SHAPE;
  if (mask_dims && (mask_dims[0] != (int64_t)g.G * g.K || mask_dims[1] != g.Do || mask_dims[2] != g.Ho ||
                    mask_dims[3] != g.Wo))
    return D2C_ERR_MASK_SHAPE;
  return D2C_OK;
}

size_t d2c_workspace_bytes(int op, const d2c_conv_desc* desc) {
  Geom g;
  const bool dw = (op == D2C_OP_DEPTHWISE_FWD || op == D2C_OP_DEPTHWISE_BWD);
  if (make_geom(desc, &g, dw)) return 0;
  // the mode and the cap are read once per call: a concurrent setter cannot make one call see two plans
  const int mode = g_math_mode.load();
  const unsigned long long cap = g_max_intermediate.load();
  switch (op) {
    case D2C_OP_DEFORM_FWD:
    case D2C_OP_DYNDIL_FWD:
      return sm100_fwd_workspace(g, desc->dtype, mode);
    case D2C_OP_DEFORM_BWD:
    case D2C_OP_DYNDIL_BWD: {
      const size_t fast = sm100_bwd_workspace(g, desc->dtype, mode, cap);
      const size_t gen = generic_bwd_workspace(g, desc->dtype, cap);
      return fast > gen ? fast : gen;
    }
    case D2C_OP_DEPTHWISE_BWD:
      return depthwise_bwd_workspace(g);
    default:
      return 0;
  }
}

const char* d2c_status_string(int status) {
  switch (status) {
    case D2C_OK: return "ok";
    case D2C_ERR_NULL: return "a required pointer is NULL";
    case D2C_ERR_DTYPE: return "dtype not supported by this op";
    case D2C_ERR_SHAPE: return "sizes, strides and dilations must be positive and padding non-negative";
    case D2C_ERR_GROUPS: return "channel counts must be divisible by groups and offset_groups";
    case D2C_ERR_OUT_DIMS: return "computed output size is not positive";
    case D2C_ERR_OFFSET_SHAPE: return "offset must have offset_groups*3*K channels and the output's spatial dims";
    case D2C_ERR_MASK_SHAPE: return "mask must have offset_groups*K channels and the output's spatial dims";
    case D2C_ERR_WORKSPACE: return "workspace is NULL, not 256-byte aligned or too small";
    case D2C_ERR_TOO_LARGE: return "tensor too large for this op";
    case D2C_ERR_MODE: return "unknown math or field mode";
    case D2C_ERR_WEIGHT_SHAPE: return "weight shape does not match the channel counts";
    case D2C_ERR_SCRATCH_LIMIT:
      return "out_channels * kernel taps exceeds the 32768 accumulator slots of the built-in scratch buffer";
    case D2C_ERR_CUDA: return "CUDA runtime error";
    case D2C_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
    default: return "unknown status";
  }
}

const char* d2c_last_cuda_error(void) { return g_last_cuda_error; }

int d2c_device_status(void) {
  int rc = check_cuda(cudaDeviceSynchronize());
  if (rc) return rc;
  return status_take();
}

int d2c_device_status_peek(void) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return D2C_ERR_CUDA;
  return g_status_page.word[dev][0] ? D2C_ERR_DEVICE_TIMEOUT : D2C_OK;
}

void d2c_device_status_clear(void) { (void)status_take(); }

int d2c_selftest_wait_expiry(uint32_t budget_us, d2c_stream_t stream) {
  if (budget_us == 0 || budget_us > 100000u) return D2C_ERR_SHAPE;     // at most 0.1 s
  int dev = 0, khz = 0;
  D2C_CUDA_TRY(cudaGetDevice(&dev));
  D2C_CUDA_TRY(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev));
  return sm100_selftest_wait_expiry((long long)budget_us * (long long)(khz / 1000), (cudaStream_t)stream);
}

uint64_t d2c_launch_count(void) { return g_launches.load(); }

int d2c_profile_enable(int on) {
  g_prof_on.store(on != 0);
  return D2C_OK;
}

int d2c_profile_read(d2c_profile_record* records, int max_records, int* n_records) {
  if (!n_records || (max_records > 0 && !records)) return D2C_ERR_NULL;
  std::lock_guard<std::mutex> lk(g_prof_mu);
  int n = 0, rc = D2C_OK;
  if (!g_prof.empty()) rc = check_cuda(cudaEventSynchronize(g_prof.back().ev));
  for (size_t i = 0; i + 1 < g_prof.size() && rc == D2C_OK; ++i) {
    if (!g_prof[i].name) continue;
    float ms = 0.f;
    rc = check_cuda(cudaEventElapsedTime(&ms, g_prof[i].ev, g_prof[i + 1].ev));
    if (n < max_records) records[n++] = {g_prof[i].name, ms};
  }
  for (auto& m : g_prof) cudaEventDestroy(m.ev);
  g_prof.clear();
  *n_records = n;
  return rc;
}

int d2c_set_math_mode(int mode) {
  if (mode < D2C_MATH_AUTO || mode > D2C_MATH_BF16) return D2C_ERR_MODE;
  g_math_mode.store(mode);
  return D2C_OK;
}
int d2c_get_math_mode(void) { return g_math_mode.load(); }

uint64_t d2c_get_max_intermediate_elements(void) { return g_max_intermediate.load(); }
void d2c_set_max_intermediate_elements(uint64_t n) { g_max_intermediate.store(n ? n : 1); }

// ---- sample cache ----------------------------------------------------------------------------------

size_t d2c_sample_cache_bytes(const d2c_conv_desc* desc) {
  Geom g;
  if (!desc || make_geom(desc, &g, false) || desc->dtype != D2C_F32) return 0;
  const int mode = g_math_mode.load();
  const unsigned long long cap = g_max_intermediate.load();
  // the image is a column matrix in 16 bits: the cap on intermediate elements applies to it
  if ((unsigned long long)g.B * g.Cin * g.K * g.V > cap) return 0;
  bool fx3 = false, bx3 = false;
  if (!sm100_fwd_variant(g, mode, &fx3) || !sm100_bwd_variant(g, mode, cap, &bx3) || fx3 != bx3) return 0;
  int np = 0;
  SampleCacheLayout lay{};
  return sm100_sample_cache_layout(g, fx3, &np, &lay) ? lay.total() : 0;
}

int d2c_bind_sample_cache(d2c_sample_cache* cache) {
  static_assert(sizeof(d2c_sample_cache) == sizeof(SampleCache), "public and internal cache structs differ");
  g_bound_cache = reinterpret_cast<SampleCache*>(cache);
  return D2C_OK;
}

// ---- deformable conv ---------------------------------------------------------------------------

int d2c_deform_conv3d_fwd(const d2c_conv_desc* desc, const void* x, const void* offset,
                          const void* mask, const void* w, const void* bias, void* y,
                          void* workspace, size_t workspace_bytes, d2c_stream_t stream) {
  SampleCacheScope cache_scope(true);
  if (!desc || !x || !offset || !w || !y) return D2C_ERR_NULL;
  Geom g;
  int rc = make_geom(desc, &g, false);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  D2C_TAKE_STATUS();
  if (desc->dtype == D2C_F32) {
    OffsetCoords<float> oc{(const float*)offset};
    const int mode = g_math_mode.load();
    if (sm100_fwd_supported(g, desc->dtype, mode)) {
      if (!ws_ok(workspace, workspace_bytes, sm100_fwd_workspace(g, desc->dtype, mode))) return D2C_ERR_WORKSPACE;
      return sm100_fwd_offsets(g, mode, (const float*)x, (const float*)offset, (const float*)mask,
                               (const float*)w, (const float*)bias, (float*)y, workspace, st);
    }
    return launch_fwd_generic<float>(g, oc, (const float*)x, (const float*)mask, (const float*)w,
                                     (const float*)bias, (float*)y, st);
  } else if (desc->dtype == D2C_F64) {
    OffsetCoords<double> oc{(const double*)offset};
    return launch_fwd_generic<double>(g, oc, (const double*)x, (const double*)mask, (const double*)w,
                                      (const double*)bias, (double*)y, st);
  }
  return D2C_ERR_DTYPE;
}

int d2c_deform_conv3d_bwd(const d2c_conv_desc* desc, const void* grad_y, const void* x,
                          const void* offset, const void* mask, const void* w, void* grad_x,
                          void* grad_offset, void* grad_mask, void* grad_w, void* grad_bias,
                          void* workspace, size_t workspace_bytes, d2c_stream_t stream) {
  return d2c_deform_conv3d_bwd_ev(desc, grad_y, x, offset, mask, w, grad_x, grad_offset, grad_mask, grad_w, grad_bias,
                                  workspace, workspace_bytes, stream, nullptr);
}

int d2c_deform_conv3d_bwd_ev(const d2c_conv_desc* desc, const void* grad_y, const void* x,
                             const void* offset, const void* mask, const void* w, void* grad_x,
                             void* grad_offset, void* grad_mask, void* grad_w, void* grad_bias,
                             void* workspace, size_t workspace_bytes, d2c_stream_t stream,
                             d2c_event_t params_ready) {
  SampleCacheScope cache_scope(false);
  if (!desc || !grad_y || !x || !offset || !w || !grad_x || !grad_offset || !grad_w) return D2C_ERR_NULL;
  if (mask && !grad_mask) return D2C_ERR_NULL;
  Geom g;
  int rc = make_geom(desc, &g, false);
  if (rc) return rc;
  if (desc->dtype != D2C_F32 && desc->dtype != D2C_F64) return D2C_ERR_DTYPE;
  cudaStream_t st = (cudaStream_t)stream;
  D2C_TAKE_STATUS();
  const unsigned long long cap = g_max_intermediate.load();
  const int mode = g_math_mode.load();
  if (sm100_bwd_supported(g, desc->dtype, mode, cap)) {
    if (!ws_ok(workspace, workspace_bytes, sm100_bwd_workspace(g, desc->dtype, mode, cap)))
      return D2C_ERR_WORKSPACE;
    return sm100_bwd_offsets(g, mode, cap, (const float*)grad_y, (const float*)x, (const float*)offset,
                             (const float*)mask, (const float*)w, (float*)grad_x, (float*)grad_offset,
                             (float*)grad_mask, (float*)grad_w, (float*)grad_bias, workspace, st,
                             (cudaEvent_t)params_ready);
  }
  const size_t need = generic_bwd_workspace(g, desc->dtype, cap);
  if (!ws_ok(workspace, workspace_bytes, need)) return D2C_ERR_WORKSPACE;
  const int nb = bwd_slice_clips(g, cap);
  if (desc->dtype == D2C_F32) {
    OffsetCoords<float> oc{(const float*)offset};
    rc = launch_bwd_generic<float, OffsetCoords<float>, false>(
        g, oc, (const float*)grad_y, (const float*)x, (const float*)mask, (const float*)w,
        (float*)grad_x, (float*)grad_offset, 0, (float*)grad_mask, (float*)grad_w, (float*)grad_bias,
        (float*)workspace, nb, st);
  } else {
    OffsetCoords<double> oc{(const double*)offset};
    rc = launch_bwd_generic<double, OffsetCoords<double>, false>(
        g, oc, (const double*)grad_y, (const double*)x, (const double*)mask, (const double*)w,
        (double*)grad_x, (double*)grad_offset, 0, (double*)grad_mask, (double*)grad_w,
        (double*)grad_bias, (double*)workspace, nb, st);
  }
  // the CUDA-core kernels produce the parameter gradients last
  if (rc == D2C_OK && params_ready) D2C_CUDA_TRY(cudaEventRecord((cudaEvent_t)params_ready, st));
  return rc;
}

int d2c_deform_conv3d_corners(const d2c_conv_desc* desc, const void* offset, int32_t* corners,
                              d2c_stream_t stream) {
  if (!desc || !offset || !corners) return D2C_ERR_NULL;
  Geom g;
  int rc = make_geom(desc, &g, false);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const long long total = (long long)g.B * g.G * g.K * g.V;
  if (desc->dtype == D2C_F32) {
    OffsetCoords<float> oc{(const float*)offset};
    corners_kernel<float><<<grid_1d(total, 256), 256, 0, st>>>(g, oc, corners);
  } else if (desc->dtype == D2C_F64) {
    OffsetCoords<double> oc{(const double*)offset};
    corners_kernel<double><<<grid_1d(total, 256), 256, 0, st>>>(g, oc, corners);
  } else {
    return D2C_ERR_DTYPE;
  }
  D2C_LAUNCH_CHECK();
  return D2C_OK;
}

// ---- deform_conv1d --------------------------------------------------------------------------------

static int make_geom_1d(const d2c_conv_desc* desc, Geom* g) {
  int rc = make_geom(desc, g, false);
  if (rc) return rc;
  if (g->D != 1 || g->H != 1 || g->kd != 1 || g->kh != 1 || g->sd != 1 || g->sh != 1 || g->pd != 0 || g->ph != 0)
    return D2C_ERR_SHAPE;
  return D2C_OK;
}

int d2c_deform_conv1d_fwd(const d2c_conv_desc* desc, const void* x, const void* offset, const void* mask,
                          const void* w, const void* bias, void* y, d2c_stream_t stream) {
  if (!desc || !x || !offset || !w || !y) return D2C_ERR_NULL;
  Geom g;
  int rc = make_geom_1d(desc, &g);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  D2C_TAKE_STATUS();
  if (desc->dtype == D2C_F32) {
    Offset1dCoords<float> oc{(const float*)offset};
    return launch_fwd_generic<float>(g, oc, (const float*)x, (const float*)mask, (const float*)w, (const float*)bias,
                                     (float*)y, st);
  } else if (desc->dtype == D2C_F64) {
    Offset1dCoords<double> oc{(const double*)offset};
    return launch_fwd_generic<double>(g, oc, (const double*)x, (const double*)mask, (const double*)w,
                                      (const double*)bias, (double*)y, st);
  }
  return D2C_ERR_DTYPE;
}

int d2c_deform_conv1d_bwd(const d2c_conv_desc* desc, const void* grad_y, const void* x, const void* offset,
                          const void* mask, const void* w, void* grad_x, void* grad_offset, void* grad_mask,
                          void* grad_w, void* grad_bias, void* workspace, size_t workspace_bytes,
                          d2c_stream_t stream) {
  if (!desc || !grad_y || !x || !offset || !w || !grad_x || !grad_offset || !grad_w) return D2C_ERR_NULL;
  if (mask && !grad_mask) return D2C_ERR_NULL;
  Geom g;
  int rc = make_geom_1d(desc, &g);
  if (rc) return rc;
  if (desc->dtype != D2C_F32 && desc->dtype != D2C_F64) return D2C_ERR_DTYPE;
  cudaStream_t st = (cudaStream_t)stream;
  D2C_TAKE_STATUS();
  const unsigned long long cap = g_max_intermediate.load();
  if (!ws_ok(workspace, workspace_bytes, generic_bwd_workspace(g, desc->dtype, cap))) return D2C_ERR_WORKSPACE;
  const int nb = bwd_slice_clips(g, cap);
  if (desc->dtype == D2C_F32) {
    Offset1dCoords<float> oc{(const float*)offset};
    return launch_bwd_generic<float, Offset1dCoords<float>, false>(
        g, oc, (const float*)grad_y, (const float*)x, (const float*)mask, (const float*)w, (float*)grad_x,
        (float*)grad_offset, 0, (float*)grad_mask, (float*)grad_w, (float*)grad_bias, (float*)workspace, nb, st);
  }
  Offset1dCoords<double> oc{(const double*)offset};
  return launch_bwd_generic<double, Offset1dCoords<double>, false>(
      g, oc, (const double*)grad_y, (const double*)x, (const double*)mask, (const double*)w, (double*)grad_x,
      (double*)grad_offset, 0, (double*)grad_mask, (double*)grad_w, (double*)grad_bias, (double*)workspace, nb, st);
}

// ---- dynamic-dilated conv ------------------------------------------------------------------------

int d2c_dyn_dilated_conv3d_fwd(const d2c_conv_desc* desc, int field_mode, const void* x,
                               const void* size_map, const void* mask, const void* w,
                               const void* bias, void* y, void* workspace, size_t workspace_bytes,
                               d2c_stream_t stream) {
  SampleCacheScope cache_scope(true);
  if (!desc || !x || !size_map || !w || !y) return D2C_ERR_NULL;
  Geom g;
  int rc = make_geom(desc, &g, false);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  D2C_TAKE_STATUS();
  if (desc->dtype == D2C_F32) {
    FieldCoords<float> fc;
    if ((rc = make_field_coords<float>(g, field_mode, size_map, &fc))) return rc;
    const int mode = g_math_mode.load();
    if (sm100_fwd_supported(g, desc->dtype, mode)) {
      if (!ws_ok(workspace, workspace_bytes, sm100_fwd_workspace(g, desc->dtype, mode))) return D2C_ERR_WORKSPACE;
      return sm100_fwd_field(g, mode, fc, (const float*)x, (const float*)mask, (const float*)w,
                             (const float*)bias, (float*)y, workspace, st);
    }
    return launch_fwd_generic<float>(g, fc, (const float*)x, (const float*)mask, (const float*)w,
                                     (const float*)bias, (float*)y, st);
  } else if (desc->dtype == D2C_F64) {
    FieldCoords<double> fc;
    if ((rc = make_field_coords<double>(g, field_mode, size_map, &fc))) return rc;
    return launch_fwd_generic<double>(g, fc, (const double*)x, (const double*)mask, (const double*)w,
                                      (const double*)bias, (double*)y, st);
  }
  return D2C_ERR_DTYPE;
}

int d2c_dyn_dilated_conv3d_bwd(const d2c_conv_desc* desc, int field_mode, const void* grad_y,
                               const void* x, const void* size_map, const void* mask,
                               const void* w, void* grad_x, void* grad_size_map, void* grad_mask,
                               void* grad_w, void* grad_bias, void* workspace,
                               size_t workspace_bytes, d2c_stream_t stream) {
  return d2c_dyn_dilated_conv3d_bwd_ev(desc, field_mode, grad_y, x, size_map, mask, w, grad_x, grad_size_map, grad_mask,
                                       grad_w, grad_bias, workspace, workspace_bytes, stream, nullptr);
}

int d2c_dyn_dilated_conv3d_bwd_ev(const d2c_conv_desc* desc, int field_mode, const void* grad_y,
                                  const void* x, const void* size_map, const void* mask,
                                  const void* w, void* grad_x, void* grad_size_map, void* grad_mask,
                                  void* grad_w, void* grad_bias, void* workspace,
                                  size_t workspace_bytes, d2c_stream_t stream, d2c_event_t params_ready) {
  SampleCacheScope cache_scope(false);
  if (!desc || !grad_y || !x || !size_map || !w || !grad_x || !grad_size_map || !grad_w) return D2C_ERR_NULL;
  if (mask && !grad_mask) return D2C_ERR_NULL;
  Geom g;
  int rc = make_geom(desc, &g, false);
  if (rc) return rc;
  if (desc->dtype != D2C_F32 && desc->dtype != D2C_F64) return D2C_ERR_DTYPE;
  cudaStream_t st = (cudaStream_t)stream;
  D2C_TAKE_STATUS();
  const unsigned long long cap = g_max_intermediate.load();
  const int mode = g_math_mode.load();
  const size_t need = generic_bwd_workspace(g, desc->dtype, cap);
  if (!ws_ok(workspace, workspace_bytes, need)) return D2C_ERR_WORKSPACE;
  const int nb = bwd_slice_clips(g, cap);
  const int nch = field_channels(field_mode);
  if (nch < 0) return D2C_ERR_MODE;
  const size_t gs_elems = (size_t)g.B * nch * g.V;
  if (desc->dtype == D2C_F32) {
    FieldCoords<float> fc;
    if ((rc = make_field_coords<float>(g, field_mode, size_map, &fc))) return rc;
    if (sm100_bwd_supported(g, desc->dtype, mode, cap)) {
      if (!ws_ok(workspace, workspace_bytes, sm100_bwd_workspace(g, desc->dtype, mode, cap)))
        return D2C_ERR_WORKSPACE;
      return sm100_bwd_field(g, mode, cap, fc, (const float*)grad_y, (const float*)x, (const float*)mask,
                             (const float*)w, (float*)grad_x, (float*)grad_size_map, gs_elems,
                             (float*)grad_mask, (float*)grad_w, (float*)grad_bias, workspace, st,
                             (cudaEvent_t)params_ready);
    }
    rc = launch_bwd_generic<float, FieldCoords<float>, true>(
        g, fc, (const float*)grad_y, (const float*)x, (const float*)mask, (const float*)w,
        (float*)grad_x, (float*)grad_size_map, gs_elems, (float*)grad_mask, (float*)grad_w,
        (float*)grad_bias, (float*)workspace, nb, st);
  } else {
    FieldCoords<double> fc;
    if ((rc = make_field_coords<double>(g, field_mode, size_map, &fc))) return rc;
    rc = launch_bwd_generic<double, FieldCoords<double>, true>(
        g, fc, (const double*)grad_y, (const double*)x, (const double*)mask, (const double*)w,
        (double*)grad_x, (double*)grad_size_map, gs_elems, (double*)grad_mask, (double*)grad_w,
        (double*)grad_bias, (double*)workspace, nb, st);
  }
  if (rc == D2C_OK && params_ready) D2C_CUDA_TRY(cudaEventRecord((cudaEvent_t)params_ready, st));
  return rc;
}

int d2c_dyn_dilated_conv3d_corners(const d2c_conv_desc* desc, int field_mode, const void* size_map,
                                   int32_t* corners, d2c_stream_t stream) {
  if (!desc || !size_map || !corners) return D2C_ERR_NULL;
  Geom g;
  int rc = make_geom(desc, &g, false);
  if (rc) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  const long long total = (long long)g.B * g.G * g.K * g.V;
  if (desc->dtype == D2C_F32) {
    FieldCoords<float> fc;
    if ((rc = make_field_coords<float>(g, field_mode, size_map, &fc))) return rc;
    corners_kernel<float><<<grid_1d(total, 256), 256, 0, st>>>(g, fc, corners);
  } else if (desc->dtype == D2C_F64) {
    FieldCoords<double> fc;
    if ((rc = make_field_coords<double>(g, field_mode, size_map, &fc))) return rc;
    corners_kernel<double><<<grid_1d(total, 256), 256, 0, st>>>(g, fc, corners);
  } else {
    return D2C_ERR_DTYPE;
  }
  D2C_LAUNCH_CHECK();
  return D2C_OK;
}

// ---- deformation head fused into the op ------------------------------------------------------------

}  // extern "C"

namespace d2c {
namespace {

struct HeadPlan {
  int geo_n, mask_n;          // geometry / mask channels
  long long rstride;          // raw_channels * V
  size_t geo_bytes, mask_bytes;   // dense staging tensors of the CUDA-core route (element size applied)
};

int make_head_plan(const Geom& g, const d2c_head_desc* h, int field_nch, int dtype, HeadPlan* hp) {
  if (!h) return D2C_ERR_NULL;
  hp->geo_n = field_nch > 0 ? field_nch : g.G * 3 * g.K;
  hp->mask_n = h->mask_channel0 >= 0 ? g.G * g.K : 0;
  if (h->raw_channels <= 0 || h->geo_channel0 < 0 || h->geo_channel0 + hp->geo_n > h->raw_channels)
    return D2C_ERR_OFFSET_SHAPE;
  if (hp->mask_n) {
    if (h->mask_channel0 + hp->mask_n > h->raw_channels) return D2C_ERR_MASK_SHAPE;
    const bool disjoint = h->mask_channel0 >= h->geo_channel0 + hp->geo_n || h->geo_channel0 >= h->mask_channel0 + hp->mask_n;
    if (!disjoint) return D2C_ERR_MASK_SHAPE;
  }
  if (h->mask_act < D2C_MASK_LINEAR || h->mask_act > D2C_MASK_TANH) return D2C_ERR_MODE;
  if (h->size_act < D2C_SIZE_LINEAR || h->size_act > D2C_SIZE_RELU_PLUS_ONE) return D2C_ERR_MODE;
  hp->rstride = (long long)h->raw_channels * g.V;
  const size_t es = dtype == D2C_F64 ? 8 : 4;
  hp->geo_bytes = align_up(es * (size_t)g.B * hp->geo_n * g.V, 256);
  hp->mask_bytes = align_up(es * (size_t)g.B * hp->mask_n * g.V, 256);
  return D2C_OK;
}

// CUDA-core route: activated dense copies of the geometry and mask channels
template <typename T>
__global__ void __launch_bounds__(256)
head_apply_kernel(const T* __restrict__ raw, long long rstride, int V, int B, int geo_c0, int geo_n, int mask_c0, int mask_n,
                  int size_act, int mask_act, T* __restrict__ geo, T* __restrict__ mask) {
  const long long per = (long long)(geo_n + mask_n) * V;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < (long long)B * per; i += (long long)gridDim.x * 256) {
    const long long b = i / per, r = i % per;
    const int c = (int)(r / V), v = (int)(r % V);
    if (c < geo_n)
      geo[((long long)b * geo_n + c) * V + v] = size_act_value(size_act, raw[b * rstride + (long long)(geo_c0 + c) * V + v]);
    else
      mask[((long long)b * mask_n + (c - geo_n)) * V + v] =
          mask_act_value(mask_act, raw[b * rstride + (long long)(mask_c0 + c - geo_n) * V + v]);
  }
}

// CUDA-core route: dense gradients -> gradient of the raw tensor (every channel written)
template <typename T>
__global__ void __launch_bounds__(256)
head_grad_kernel(const T* __restrict__ raw, long long rstride, int C, int V, int B, int geo_c0, int geo_n, int mask_c0, int mask_n,
                 int size_act, int mask_act, const T* __restrict__ ggeo, const T* __restrict__ gmask,
                 const T* __restrict__ mask_activated, T* __restrict__ graw) {
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < (long long)B * C * V; i += (long long)gridDim.x * 256) {
    const long long b = i / ((long long)C * V), r = i % ((long long)C * V);
    const int c = (int)(r / V), v = (int)(r % V);
    T out = (T)0;
    if (c >= geo_c0 && c < geo_c0 + geo_n) {
      out = ggeo[((long long)b * geo_n + (c - geo_c0)) * V + v] * size_act_slope(size_act, raw[b * rstride + r]);
    } else if (mask_n && c >= mask_c0 && c < mask_c0 + mask_n) {
      const long long mi = ((long long)b * mask_n + (c - mask_c0)) * V + v;
      out = gmask[mi] * mask_act_slope(mask_act, mask_activated[mi]);
    }
    graw[b * rstride + r] = out;
  }
}

bool head_fused_fwd(const Geom& g, int dtype, int mode) { return sm100_fwd_supported(g, dtype, mode); }
bool head_fused_bwd(const Geom& g, int dtype, int mode, unsigned long long cap) { return sm100_bwd_supported(g, dtype, mode, cap); }

template <typename T>
int head_fwd_t(const Geom& g, const d2c_head_desc* h, const HeadPlan& hp, int field_mode, bool is_field, const T* x, const T* raw,
               const T* w, const T* bias, T* y, void* workspace, size_t workspace_bytes, cudaStream_t st) {
  // the CUDA-core route: stage activated dense tensors, then the ordinary kernels
  uint8_t* wsp = reinterpret_cast<uint8_t*>(workspace);
  if (!ws_ok(workspace, workspace_bytes, hp.geo_bytes + hp.mask_bytes)) return D2C_ERR_WORKSPACE;
  T* geo = reinterpret_cast<T*>(wsp);
  T* mask = hp.mask_n ? reinterpret_cast<T*>(wsp + hp.geo_bytes) : nullptr;
  head_apply_kernel<T><<<grid_1d((long long)g.B * (hp.geo_n + hp.mask_n) * g.V, 256), 256, 0, st>>>(
      raw, hp.rstride, g.V, g.B, h->geo_channel0, hp.geo_n, h->mask_channel0, hp.mask_n, is_field ? h->size_act : 0,
      h->mask_act, geo, mask);
  D2C_LAUNCH_CHECK();
  if (is_field) {
    FieldCoords<T> fc;
    int rc = make_field_coords<T>(g, field_mode, geo, &fc);
    if (rc) return rc;
    return launch_fwd_generic<T>(g, fc, x, mask, w, bias, y, st);
  }
  OffsetCoords<T> oc{geo, 0};
  return launch_fwd_generic<T>(g, oc, x, mask, w, bias, y, st);
}

template <typename T>
int head_bwd_t(const Geom& g, const d2c_head_desc* h, const HeadPlan& hp, int field_mode, bool is_field, unsigned long long cap,
               const T* gy, const T* x, const T* raw, const T* w, T* gx, T* graw, T* gw, T* gbias, void* workspace,
               size_t workspace_bytes, cudaStream_t st) {
  const size_t stage = 2 * (hp.geo_bytes + hp.mask_bytes);
  const size_t need = stage + generic_bwd_workspace(g, sizeof(T) == 8 ? D2C_F64 : D2C_F32, cap);
  if (!ws_ok(workspace, workspace_bytes, need)) return D2C_ERR_WORKSPACE;
  uint8_t* wsp = reinterpret_cast<uint8_t*>(workspace);
  T* geo = reinterpret_cast<T*>(wsp);
  T* mask = hp.mask_n ? reinterpret_cast<T*>(wsp + hp.geo_bytes) : nullptr;
  T* ggeo = reinterpret_cast<T*>(wsp + hp.geo_bytes + hp.mask_bytes);
  T* gmask = hp.mask_n ? reinterpret_cast<T*>(wsp + 2 * hp.geo_bytes + hp.mask_bytes) : nullptr;
  T* dcol = reinterpret_cast<T*>(wsp + stage);
  head_apply_kernel<T><<<grid_1d((long long)g.B * (hp.geo_n + hp.mask_n) * g.V, 256), 256, 0, st>>>(
      raw, hp.rstride, g.V, g.B, h->geo_channel0, hp.geo_n, h->mask_channel0, hp.mask_n, is_field ? h->size_act : 0,
      h->mask_act, geo, mask);
  D2C_LAUNCH_CHECK();
  const int nb = bwd_slice_clips(g, cap);
  int rc;
  if (is_field) {
    FieldCoords<T> fc;
    if ((rc = make_field_coords<T>(g, field_mode, geo, &fc))) return rc;
    rc = launch_bwd_generic<T, FieldCoords<T>, true>(g, fc, gy, x, mask, w, gx, ggeo, (size_t)g.B * hp.geo_n * g.V, gmask, gw,
                                                     gbias, dcol, nb, st);
  } else {
    OffsetCoords<T> oc{geo, 0};
    rc = launch_bwd_generic<T, OffsetCoords<T>, false>(g, oc, gy, x, mask, w, gx, ggeo, 0, gmask, gw, gbias, dcol, nb, st);
  }
  if (rc) return rc;
  head_grad_kernel<T><<<grid_1d((long long)g.B * h->raw_channels * g.V, 256), 256, 0, st>>>(
      raw, hp.rstride, h->raw_channels, g.V, g.B, h->geo_channel0, hp.geo_n, h->mask_channel0, hp.mask_n,
      is_field ? h->size_act : 0, h->mask_act, ggeo, gmask, mask, graw);
  D2C_LAUNCH_CHECK();
  return D2C_OK;
}

int head_fwd(const d2c_conv_desc* desc, const d2c_head_desc* head, int field_mode, bool is_field, const void* x, const void* raw,
             const void* w, const void* bias, void* y, void* workspace, size_t workspace_bytes, cudaStream_t st) {
  SampleCacheScope cache_scope(true);
  if (!desc || !head || !x || !raw || !w || !y) return D2C_ERR_NULL;
  Geom g;
  int rc = make_geom(desc, &g, false);
  if (rc) return rc;
  if (desc->dtype != D2C_F32 && desc->dtype != D2C_F64) return D2C_ERR_DTYPE;
  const int nch = is_field ? field_channels(field_mode) : 0;
  if (is_field && nch < 0) return D2C_ERR_MODE;
  HeadPlan hp;
  if ((rc = make_head_plan(g, head, nch, desc->dtype, &hp))) return rc;
  D2C_TAKE_STATUS();
  const int mode = g_math_mode.load();
  if (head_fused_fwd(g, desc->dtype, mode)) {
    if (!ws_ok(workspace, workspace_bytes, sm100_fwd_workspace(g, desc->dtype, mode))) return D2C_ERR_WORKSPACE;
    const float* r = (const float*)raw;
    HeadCfg cfg{hp.rstride, hp.mask_n ? hp.rstride : 0, head->mask_act, head->size_act};
    const float* mask = hp.mask_n ? r + (long long)head->mask_channel0 * g.V : nullptr;
    if (is_field) {
      FieldCoords<float> fc;
      if ((rc = make_field_coords<float>(g, field_mode, r + (long long)head->geo_channel0 * g.V, &fc))) return rc;
      fc.bstride = hp.rstride;
      fc.act = head->size_act;
      return sm100_fwd_field(g, mode, fc, (const float*)x, mask, (const float*)w, (const float*)bias, (float*)y, workspace, st, cfg);
    }
    return sm100_fwd_offsets(g, mode, (const float*)x, r + (long long)head->geo_channel0 * g.V, mask, (const float*)w,
                             (const float*)bias, (float*)y, workspace, st, cfg);
  }
  if (desc->dtype == D2C_F32)
    return head_fwd_t<float>(g, head, hp, field_mode, is_field, (const float*)x, (const float*)raw, (const float*)w,
                             (const float*)bias, (float*)y, workspace, workspace_bytes, st);
  return head_fwd_t<double>(g, head, hp, field_mode, is_field, (const double*)x, (const double*)raw, (const double*)w,
                            (const double*)bias, (double*)y, workspace, workspace_bytes, st);
}

int head_bwd(const d2c_conv_desc* desc, const d2c_head_desc* head, int field_mode, bool is_field, const void* gy, const void* x,
             const void* raw, const void* w, void* gx, void* graw, void* gw, void* gbias, void* workspace,
             size_t workspace_bytes, cudaStream_t st, cudaEvent_t params_ready) {
  SampleCacheScope cache_scope(false);
  if (!desc || !head || !gy || !x || !raw || !w || !gx || !graw || !gw) return D2C_ERR_NULL;
  Geom g;
  int rc = make_geom(desc, &g, false);
  if (rc) return rc;
  if (desc->dtype != D2C_F32 && desc->dtype != D2C_F64) return D2C_ERR_DTYPE;
  const int nch = is_field ? field_channels(field_mode) : 0;
  if (is_field && nch < 0) return D2C_ERR_MODE;
  HeadPlan hp;
  if ((rc = make_head_plan(g, head, nch, desc->dtype, &hp))) return rc;
  D2C_TAKE_STATUS();
  const int mode = g_math_mode.load();
  const unsigned long long cap = g_max_intermediate.load();
  if (head_fused_bwd(g, desc->dtype, mode, cap)) {
    if (!ws_ok(workspace, workspace_bytes, sm100_bwd_workspace(g, desc->dtype, mode, cap))) return D2C_ERR_WORKSPACE;
    const float* r = (const float*)raw;
    float* gr = (float*)graw;
    // channels of raw that feed neither part get a zero gradient
    if (hp.geo_n + hp.mask_n < head->raw_channels)
      D2C_CUDA_TRY(cudaMemsetAsync(gr, 0, sizeof(float) * (size_t)g.B * hp.rstride, st));
    HeadCfg cfg{hp.rstride, hp.mask_n ? hp.rstride : 0, head->mask_act, head->size_act};
    const float* mask = hp.mask_n ? r + (long long)head->mask_channel0 * g.V : nullptr;
    float* gmask = hp.mask_n ? gr + (long long)head->mask_channel0 * g.V : nullptr;
    float* ggeo = gr + (long long)head->geo_channel0 * g.V;
    if (is_field) {
      FieldCoords<float> fc;
      if ((rc = make_field_coords<float>(g, field_mode, r + (long long)head->geo_channel0 * g.V, &fc))) return rc;
      fc.bstride = hp.rstride;
      fc.act = head->size_act;
      return sm100_bwd_field(g, mode, cap, fc, (const float*)gy, (const float*)x, mask, (const float*)w, (float*)gx, ggeo,
                             (size_t)g.B * nch * g.V, gmask, (float*)gw, (float*)gbias, workspace, st, params_ready, cfg);
    }
    return sm100_bwd_offsets(g, mode, cap, (const float*)gy, (const float*)x, r + (long long)head->geo_channel0 * g.V, mask,
                             (const float*)w, (float*)gx, ggeo, gmask, (float*)gw, (float*)gbias, workspace, st, params_ready,
                             cfg);
  }
  if (desc->dtype == D2C_F32)
    rc = head_bwd_t<float>(g, head, hp, field_mode, is_field, cap, (const float*)gy, (const float*)x, (const float*)raw,
                           (const float*)w, (float*)gx, (float*)graw, (float*)gw, (float*)gbias, workspace, workspace_bytes, st);
  else
    rc = head_bwd_t<double>(g, head, hp, field_mode, is_field, cap, (const double*)gy, (const double*)x, (const double*)raw,
                            (const double*)w, (double*)gx, (double*)graw, (double*)gw, (double*)gbias, workspace,
                            workspace_bytes, st);
  if (rc == D2C_OK && params_ready) D2C_CUDA_TRY(cudaEventRecord(params_ready, st));
  return rc;
}

}  // namespace
}  // namespace d2c

extern "C" {

size_t d2c_head_workspace_bytes(int op, const d2c_conv_desc* desc, const d2c_head_desc* head, int field_mode) {
  Geom g;
  if (!desc || !head || make_geom(desc, &g, false)) return 0;
  const bool is_field = op == D2C_OP_DYNDIL_FWD || op == D2C_OP_DYNDIL_BWD;
  const bool bwd = op == D2C_OP_DEFORM_BWD || op == D2C_OP_DYNDIL_BWD;
  const int nch = is_field ? field_channels(field_mode) : 0;
  HeadPlan hp;
  if ((is_field && nch < 0) || make_head_plan(g, head, nch, desc->dtype, &hp)) return 0;
  const int mode = g_math_mode.load();
  const unsigned long long cap = g_max_intermediate.load();
  // whichever route the call takes under the current settings, and never less than the plain op's workspace
  const size_t plain = d2c_workspace_bytes(op, desc);
  const size_t staged = (bwd ? 2 : 1) * (hp.geo_bytes + hp.mask_bytes) + (bwd ? generic_bwd_workspace(g, desc->dtype, cap) : 0);
  const bool fused = bwd ? head_fused_bwd(g, desc->dtype, mode, cap) : head_fused_fwd(g, desc->dtype, mode);
  return fused ? plain : (staged > plain ? staged : plain);
}

int d2c_deform_conv3d_head_fwd(const d2c_conv_desc* desc, const d2c_head_desc* head, const void* x, const void* raw,
                               const void* w, const void* bias, void* y, void* workspace, size_t workspace_bytes,
                               d2c_stream_t stream) {
  return head_fwd(desc, head, 0, false, x, raw, w, bias, y, workspace, workspace_bytes, (cudaStream_t)stream);
}

int d2c_deform_conv3d_head_bwd(const d2c_conv_desc* desc, const d2c_head_desc* head, const void* grad_y, const void* x,
                               const void* raw, const void* w, void* grad_x, void* grad_raw, void* grad_w,
                               void* grad_bias, void* workspace, size_t workspace_bytes, d2c_stream_t stream,
                               d2c_event_t params_ready) {
  return head_bwd(desc, head, 0, false, grad_y, x, raw, w, grad_x, grad_raw, grad_w, grad_bias, workspace, workspace_bytes,
                  (cudaStream_t)stream, (cudaEvent_t)params_ready);
}

int d2c_dyn_dilated_conv3d_head_fwd(const d2c_conv_desc* desc, const d2c_head_desc* head, int field_mode, const void* x,
                                    const void* raw, const void* w, const void* bias, void* y, void* workspace,
                                    size_t workspace_bytes, d2c_stream_t stream) {
  return head_fwd(desc, head, field_mode, true, x, raw, w, bias, y, workspace, workspace_bytes, (cudaStream_t)stream);
}

int d2c_dyn_dilated_conv3d_head_bwd(const d2c_conv_desc* desc, const d2c_head_desc* head, int field_mode,
                                    const void* grad_y, const void* x, const void* raw, const void* w, void* grad_x,
                                    void* grad_raw, void* grad_w, void* grad_bias, void* workspace,
                                    size_t workspace_bytes, d2c_stream_t stream, d2c_event_t params_ready) {
  return head_bwd(desc, head, field_mode, true, grad_y, x, raw, w, grad_x, grad_raw, grad_w, grad_bias, workspace,
                  workspace_bytes, (cudaStream_t)stream, (cudaEvent_t)params_ready);
}

// ---- depthwise -----------------------------------------------------------------------------------

int d2c_depthwise_conv3d_fwd(const d2c_conv_desc* desc, const void* x, const void* w,
                             const void* bias, void* y, d2c_stream_t stream) {
  if (!desc || !x || !w || !y) return D2C_ERR_NULL;
  Geom g;
  int rc = make_geom(desc, &g, true);
  if (rc) return rc;
  // int32 range rule of the reference (csrc/grouped_conv3d.cu:431-440)
  if ((long long)g.B * g.Cin * g.Vin > 0x7fffffffLL || (long long)g.B * g.Cout * g.V > 0x7fffffffLL)
    return D2C_ERR_TOO_LARGE;
  D2C_TAKE_STATUS();
  return depthwise_fwd(g, desc->dtype, x, w, bias, y, (cudaStream_t)stream);
}

int d2c_depthwise_conv3d_bwd(const d2c_conv_desc* desc, const void* grad_y, const void* x,
                             const void* w, void* grad_x, void* grad_w, void* grad_bias,
                             void* workspace, size_t workspace_bytes, d2c_stream_t stream) {
  if (!desc || !grad_y || !x || !w) return D2C_ERR_NULL;
  Geom g;
  int rc = make_geom(desc, &g, true);
  if (rc) return rc;
  if ((long long)g.B * g.Cin * g.Vin > 0x7fffffffLL || (long long)g.B * g.Cout * g.V > 0x7fffffffLL)
    return D2C_ERR_TOO_LARGE;
  if (grad_w && !ws_ok(workspace, workspace_bytes, depthwise_bwd_workspace(g))) return D2C_ERR_WORKSPACE;
  D2C_TAKE_STATUS();
  return depthwise_bwd(g, desc->dtype, grad_y, x, w, grad_x, grad_w, grad_bias, workspace,
                       (cudaStream_t)stream);
}

}  // extern "C"
