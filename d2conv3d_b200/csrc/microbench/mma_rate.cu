// Microbenchmark: how many clocks does one tcgen05.mma.cta_group::1.kind::f16 of shape M128 x N256 x K16 take when
// one thread issues them back to back from fixed shared-memory tiles -- (a) always into the SAME accumulator columns
// (N = 256: a dependent accumulation chain) and (b) alternating between two accumulators (N = 512 as 2 x 256, what
// the forward kernel does for 512 output channels) -- with and without a tcgen05.commit between groups of MMAs.
// Build and run:  python -m d2conv3d_b200.build --microbench && d2conv3d_b200/build/mma_rate
// The only wait is the library's bounded mbarrier wait.
#include <cstdio>
#include <cstdlib>
#include <cuda_runtime.h>
#include "../sm100_ptx.cuh"
namespace d2c { int status_word_device_ptr(int** p) { *p = nullptr; return 0; } }
using namespace d2c;
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e), __LINE__); exit(1); } } while (0)

// per_commit: MMA steps between intermediate commits (0 = none); the final commit is the one that is waited for
__global__ void __launch_bounds__(128, 1) k(int n_mma, int N, int per_commit, long long* out) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t base = (raw + 1023u) & ~1023u;
  uint8_t* bp = smem_raw + (base - raw);
  const uint32_t a_base = base, b_base = base + 16384, bar = base + 16384 + 65536;
  volatile uint32_t* slot = reinterpret_cast<volatile uint32_t*>(bp + 16384 + 65536 + 64);
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    ptx::mbar_init(bar, 1);
    ptx::mbar_init(bar + 8, 1 << 20);      // collects the intermediate commits; nobody waits on it
    abort_flag = 0;
    ptx::fence_mbar_init();
  }
  for (int i = threadIdx.x; i < (16384 + 65536) / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(bp)[i] = 0x3c003c00u;
  ptx::fence_proxy_async_smem();
  if (threadIdx.x < 32) { ptx::tmem_alloc(ptx::smem_u32((const void*)slot), 512); ptx::tmem_relinquish(); }
  ptx::tc_fence_before(); __syncthreads(); ptx::tc_fence_after();
  const uint32_t tmem = *slot;
  if (threadIdx.x == 0) {
    const long long t0 = clock64();
    const uint32_t idesc = ptx::umma_idesc_bf16_f32(128, 256);
    for (int i = 0; i < n_mma; ++i) {
      const int kk = i & 3;
      const uint64_t ad = ptx::umma_desc_kmajor_sw128(a_base) + (uint64_t)(2 * kk);
      for (int n0 = 0; n0 < N; n0 += 256) {
        const uint64_t bd = ptx::umma_desc_kmajor_sw128(b_base + n0 * 128) + (uint64_t)(2 * kk);
        ptx::umma_bf16(tmem + n0, ad, bd, idesc, i > 0 ? 1u : 0u);
      }
      if (per_commit && (i % per_commit) == per_commit - 1 && i + 1 < n_mma) {
        // a commit that nobody waits for (arrives on a second barrier word)
        ptx::umma_commit(bar + 8);
      }
    }
    ptx::umma_commit(bar);
    ptx::mbar_wait(bar, 0, &abort_flag);
    out[blockIdx.x] = clock64() - t0;
  }
  ptx::tc_fence_before(); __syncthreads();
  if (threadIdx.x < 32) { ptx::tc_fence_after(); ptx::tmem_dealloc(tmem, 512); }
}

int main() {
  long long* out; CK(cudaMalloc(&out, 148 * 8));
  const int smem = 16384 + 65536 + 1024 + 256;
  CK(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  for (int N : {256, 512}) for (int pc : {0, 1, 6, 12, 24, 48, 96, 512}) for (int grid : {148}) {
    const int n = 4096;
    k<<<grid, 128, smem>>>(n, N, pc, out);
    CK(cudaDeviceSynchronize());
    long long h[148]; CK(cudaMemcpy(h, out, grid * 8, cudaMemcpyDeviceToHost));
    long long mx = 0; for (int i = 0; i < grid; ++i) mx = h[i] > mx ? h[i] : mx;
    printf("N=%d commits every %d, %3d CTAs: %.1f clk per (M128 x N%d x K16) step, %.1f per 256-wide MMA\n", N, pc, grid,
           (double)mx / n, N, (double)mx / n / (N / 256));
  }
  return 0;
}
