// Microbenchmark of the two L2 rates that bound the sampling kernels of this library on one GPU:
//
//   scatter  how fast fp32 scatter-add payload reaches an L2-resident accumulator with the access pattern of the
//            sampling-gradient kernel: per (clip, group, tap, voxel) sample 8 corner cells of 64 channels
//            (256 B each) around a position ~ N(0, 2 voxels) from the output voxel, 8 threads per sample, two
//            red.global.add.v4.f32 per thread and corner -- and, for comparison, the same payload sent as bulk
//            reductions (cp.reduce.async.bulk ... add.f32) of 256 B from shared memory.
//   gather   how fast the forward / weight-gradient producers' corner loads come back: per sample 8 lines of
//            128 B (8 threads x 16 B), 16 loads in flight per thread, fp16 (26 MB) and fp32 (53 MB) staging.
//
// Shapes are those of the headline layer (B = 2, 512 channels in 8 groups, 8 x 30 x 54, 27 taps): 5.6 M samples,
// 11.5 GB of scatter payload, 5.8 / 11.5 GB gathered.  Build and run:
//     python -m d2conv3d_b200.build --microbench && d2conv3d_b200/build/l2_rates
// Prints one line per variant: milliseconds (best of 3), bytes, GB/s.  Every wait in here is a hardware
// bulk-group wait; there is no spin loop.
#include <cstdint>
#include <cstdio>
#include <cstdlib>

#include <cuda_runtime.h>

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("CUDA error %s at line %d\n", cudaGetErrorString(e_), __LINE__); exit(1); } } while (0)

constexpr int B = 2, G = 8, K = 27, D = 8, H = 30, W = 54, V = D * H * W, CPG = 64, CIN = G * CPG;

__device__ __forceinline__ uint32_t hash32(uint32_t x) {
  x ^= x >> 16; x *= 0x7feb352dU; x ^= x >> 15; x *= 0x846ca68bU; x ^= x >> 16;
  return x;
}

// integer offset ~ N(0, sigma = 2 voxels): sum of three uniforms
__device__ __forceinline__ int rand_offset(uint32_t bits) {
  const int a = (int)(bits & 0xff), c = (int)((bits >> 8) & 0xff), d = (int)((bits >> 16) & 0xff);
  return (int)floorf(((a + c + d) / 255.f - 1.5f) * 4.f * 0.866f);
}

// corner 000 of sample (b, g, tap, v), clamped so that all 8 corners are inside the volume
__device__ __forceinline__ void sample_cell(int b, int g, int tap, int v, int& z, int& y, int& x) {
  const uint32_t h = hash32((uint32_t)(((b * G + g) * K + tap) * V + v) * 2654435761u + 12345u);
  z = v / (H * W) + (tap / 9 - 1) + rand_offset(h);
  y = (v / W) % H + ((tap / 3) % 3 - 1) + rand_offset(hash32(h));
  x = v % W + (tap % 3 - 1) + rand_offset(hash32(h + 77u));
  z = min(max(z, 0), D - 2); y = min(max(y, 0), H - 2); x = min(max(x, 0), W - 2);
}

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d));
}

__device__ __forceinline__ long long cell_off(int b, int g, int z, int y, int x) {      // channels-last [B][V][CIN]
  return ((long long)b * V + ((long long)z * H + y) * W + x) * CIN + g * CPG;
}

// ---- scatter: vector reductions -----------------------------------------------------------------------------
__global__ void __launch_bounds__(256) scatter_red_kernel(float* gx, long long nsamples, int corner_mask) {
  const int j = threadIdx.x & 7;
  const long long s = (long long)blockIdx.x * 32 + (threadIdx.x >> 3);
  if (s >= nsamples) return;
  const int v = (int)(s % V), tap = (int)((s / V) % K), g = (int)((s / ((long long)V * K)) % G), b = (int)(s / ((long long)V * K * G));
  int z, y, x;
  sample_cell(b, g, tap, v, z, y, x);
  const float val = 1e-3f * (float)(j + 1);
#pragma unroll
  for (int q = 0; q < 8; ++q) {
    if (!((corner_mask >> q) & 1)) continue;
    float* dst = gx + cell_off(b, g, z + (q >> 2), y + ((q >> 1) & 1), x + (q & 1)) + j * 4;
    red_add_v4(dst, val, val, val, val);
    red_add_v4(dst + 32, val, val, val, val);
  }
}

// ---- scatter: bulk reductions of 256 B staged in shared memory ----------------------------------------------
__global__ void __launch_bounds__(128) scatter_bulk_kernel(float* gx, long long nsamples) {
  extern __shared__ __align__(128) uint8_t smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, j = lane & 7, sl = lane >> 3;
  uint8_t* wbuf = smem + warp * 2 * 8192;      // two buffers of 4 samples x 8 corners x 256 B
  const long long nwarps = (long long)gridDim.x * 4, gw = (long long)blockIdx.x * 4 + warp;
  int it = 0;
  for (long long s0 = gw * 4; s0 < nsamples; s0 += nwarps * 4, ++it) {
    uint8_t* buf = wbuf + (it & 1) * 8192;
    asm volatile("cp.async.bulk.wait_group.read 1;" ::: "memory");     // the buffer's previous bulk reads are done
    __syncwarp();
    const float val = 1e-3f * (float)(j + 1);
    const float4 v4 = make_float4(val, val, val, val);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      float4* d = reinterpret_cast<float4*>(buf + (sl * 8 + q) * 256) + j;
      d[0] = v4; d[8] = v4;
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncwarp();
    const long long s = s0 + (lane >> 3);                    // lane = (sample, corner)
    if (s < nsamples) {
      const int v = (int)(s % V), tap = (int)((s / V) % K), g = (int)((s / ((long long)V * K)) % G), b = (int)(s / ((long long)V * K * G));
      int z, y, x;
      sample_cell(b, g, tap, v, z, y, x);
      const int q = lane & 7;
      float* dst = gx + cell_off(b, g, z + (q >> 2), y + ((q >> 1) & 1), x + (q & 1));
      const uint32_t src = (uint32_t)__cvta_generic_to_shared(buf + lane * 256);
      asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;" ::"l"(dst), "r"(src), "r"(256u) : "memory");
    }
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
  }
  asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

// ---- gather ---------------------------------------------------------------------------------------------------
__device__ __forceinline__ uint4 ldg_nc_v4(const void* p) {
  uint4 r;
  asm("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
  return r;
}

// units in the forward's order: tile of 128 voxels, then slices (group, tap, half); 512 threads = 64 rows x 8
// chunks of 16 B, two passes per unit; every thread has its 16 loads in flight before it consumes them.
// cin_bytes = bytes of one voxel's channels-last row; a unit row is 128 B of it.
__global__ void __launch_bounds__(512) gather_kernel(const uint8_t* x, int cin_bytes, int nh, long long n_units, unsigned* sink) {
  const int j = threadIdx.x & 7, r0 = threadIdx.x >> 3;
  const int S = G * K * nh, tiles_per_clip = (V + 127) / 128;
  const long long u_beg = n_units * blockIdx.x / gridDim.x, u_end = n_units * (blockIdx.x + 1) / gridDim.x;
  unsigned acc = 0;
  for (long long u = u_beg; u < u_end; ++u) {
    const int tile = (int)(u / S), s = (int)(u % S);
    const int b = tile / tiles_per_clip, v0 = (tile % tiles_per_clip) * 128;
    const int h = s % nh, gt = s / nh, tap = gt % K, g = gt / K;
    uint4 c[2][8];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      int v = v0 + r0 + 64 * i;
      if (v >= V) v = V - 1;
      int z, y, xx;
      sample_cell(b, g, tap, v, z, y, xx);
      const uint8_t* p0 = x + ((long long)b * V + ((long long)z * H + y) * W + xx) * cin_bytes + (g * nh + h) * 128 + j * 16;
#pragma unroll
      for (int q = 0; q < 8; ++q)
        c[i][q] = ldg_nc_v4(p0 + ((long long)(q >> 2) * H * W + ((q >> 1) & 1) * W + (q & 1)) * cin_bytes);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
      for (int q = 0; q < 8; ++q) acc ^= c[i][q].x ^ c[i][q].y ^ c[i][q].z ^ c[i][q].w;
  }
  if (acc == 0x12345678u) sink[0] = acc;
}

template <typename F>
static float best_of(F launch, cudaEvent_t e0, cudaEvent_t e1) {
  launch();
  CK(cudaDeviceSynchronize());
  float best = 1e9f;
  for (int r = 0; r < 3; ++r) {
    CK(cudaEventRecord(e0));
    launch();
    CK(cudaEventRecord(e1));
    CK(cudaEventSynchronize(e1));
    float ms;
    CK(cudaEventElapsedTime(&ms, e0, e1));
    if (ms < best) best = ms;
  }
  CK(cudaGetLastError());
  return best;
}

int main() {
  cudaEvent_t e0, e1;
  CK(cudaEventCreate(&e0));
  CK(cudaEventCreate(&e1));
  const long long nsamples = (long long)B * G * K * V;
  {
    const size_t bytes = (size_t)B * V * CIN * 4;
    float* gx;
    CK(cudaMalloc(&gx, bytes));
    CK(cudaMemset(gx, 0, bytes));
    const double payload = (double)nsamples * 8 * 256;
    const unsigned grid = (unsigned)((nsamples + 31) / 32);
    const struct { const char* name; int mask; double frac; } red_cases[] = {
        {"scatter red.v4, 8 corners per sample", 0xff, 1.0}, {"scatter red.v4, 4 corners per sample", 0x0f, 0.5},
        {"scatter red.v4, 1 corner per sample", 0x01, 0.125}};
    for (const auto& c : red_cases) {
      const float ms = best_of([&] { scatter_red_kernel<<<grid, 256>>>(gx, nsamples, c.mask); }, e0, e1);
      printf("%-46s %8.3f ms  %6.2f GB  %7.1f GB/s\n", c.name, ms, payload * c.frac / 1e9, payload * c.frac / ms / 1e6);
    }
    const int smem = 4 * 2 * 8192;
    CK(cudaFuncSetAttribute(scatter_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    for (int per_sm = 1; per_sm <= 3; ++per_sm) {
      const float ms = best_of([&] { scatter_bulk_kernel<<<148 * per_sm, 128, smem>>>(gx, nsamples); }, e0, e1);
      char nm[80];
      snprintf(nm, sizeof nm, "scatter bulk reduce 256 B, %d blocks per SM", per_sm);
      printf("%-46s %8.3f ms  %6.2f GB  %7.1f GB/s\n", nm, ms, payload / 1e9, payload / ms / 1e6);
    }
    CK(cudaFree(gx));
  }
  unsigned* sink;
  CK(cudaMalloc(&sink, 4));
  for (int fp32 = 0; fp32 <= 1; ++fp32) {
    const int cin_bytes = CIN * (fp32 ? 4 : 2), nh = fp32 ? 2 : 1;      // fp32: a 64-channel group = two 128-byte units
    const size_t bytes = (size_t)B * V * cin_bytes;
    uint8_t* x;
    CK(cudaMalloc(&x, bytes));
    CK(cudaMemset(x, 1, bytes));
    const long long n_units = (long long)B * ((V + 127) / 128) * G * K * nh;
    const double gathered = (double)n_units * 128 * 8 * 128;
    const float ms = best_of([&] { gather_kernel<<<148, 512>>>(x, cin_bytes, nh, n_units, sink); }, e0, e1);
    printf("%-46s %8.3f ms  %6.2f GB  %7.1f GB/s\n", fp32 ? "gather 8 corners x 128 B, fp32 staging" : "gather 8 corners x 128 B, fp16 staging", ms,
           gathered / 1e9, gathered / ms / 1e6);
    CK(cudaFree(x));
  }
  return 0;
}
