// Issue cost (cycles per op, one thread) of the synchronisation ops in the MMA/producer loops.
#include <cstdio>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>
#include "../tc_common.cuh"
using namespace tc;

__global__ void __launch_bounds__(128) cost_kernel(long long* out, int iters) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ uint64_t bar[4];
  __shared__ uint32_t tmem_base;
  uint32_t sbase = (smem_u32(smem) + 1023) & ~1023u;
  for (int i = threadIdx.x; i < (64 * 1024) / 4; i += blockDim.x) ((float*)smem)[i] = 0.f;
  if (threadIdx.x == 0) { for (int i = 0; i < 4; ++i) mbar_init(smem_u32(&bar[i]), 1); fence_barrier_init(); }
  __syncthreads();
  if (threadIdx.x < 32) { tmem_alloc(smem_u32(&tmem_base), 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  fence_proxy_async();
  if (threadIdx.x == 0) {
    volatile int abort_flag = 0;
    long long t0, t1;
    uint32_t acc = 0;
    // (0) try_wait on a phase that is already complete (parity 1 of a fresh barrier)
    t0 = clock64();
    for (int i = 0; i < iters; ++i) acc += mbar_try_wait(smem_u32(&bar[0]), 1u);
    t1 = clock64(); out[0] = t1 - t0;
    // (1) arrive.expect_tx with 0 bytes (completes a phase each time)
    t0 = clock64();
    for (int i = 0; i < iters; ++i) mbar_expect_tx(smem_u32(&bar[1]), 0);
    t1 = clock64(); out[1] = t1 - t0;
    // (2) tcgen05.fence::after_thread_sync
    t0 = clock64();
    for (int i = 0; i < iters; ++i) tc_fence_after();
    t1 = clock64(); out[2] = t1 - t0;
    // (3) tcgen05.commit with nothing outstanding
    t0 = clock64();
    for (int i = 0; i < iters; ++i) mma_commit(smem_u32(&bar[2]));
    t1 = clock64(); out[3] = t1 - t0;
    // (4) issue of 4 MMAs (N=64) + commit, no waiting: issue cost while the pipe is busy
    {
      const uint32_t idesc = idesc_tf32(128, 64, 0, 0);
      const uint32_t a_lo = desc_lo_kmajor(sbase), b_lo = desc_lo_kmajor(sbase + 32768), hi = desc_hi_kmajor();
      t0 = clock64();
      for (int i = 0; i < iters; ++i) {
#pragma unroll
        for (int k = 0; k < 4; ++k) mma_tf32_words(tmem_base, a_lo + 2 * k, hi, b_lo + 2 * k, hi, idesc, 1);
        mma_commit(smem_u32(&bar[3]));
      }
      t1 = clock64(); out[4] = t1 - t0;
      // wait for everything: bar[3] has completed `iters` phases; wait on the last one
      mbar_wait(smem_u32(&bar[3]), (uint32_t)((iters - 1) & 1), &abort_flag, 1);
      out[5] = clock64() - t0;
      // (6) the same with a try_wait + fence per group (as in the kernels)
      t0 = clock64();
      for (int i = 0; i < iters; ++i) {
        acc += mbar_try_wait(smem_u32(&bar[0]), 1u);
        tc_fence_after();
#pragma unroll
        for (int k = 0; k < 4; ++k) mma_tf32_words(tmem_base, a_lo + 2 * k, hi, b_lo + 2 * k, hi, idesc, 1);
        mma_commit(smem_u32(&bar[3]));
      }
      t1 = clock64(); out[6] = t1 - t0;
      // bar[3] now completed 2*iters phases
      mbar_wait(smem_u32(&bar[3]), (uint32_t)((2 * iters - 1) & 1), &abort_flag, 1);
      out[7] = clock64() - t0;
    }
    out[15] = acc;
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) tmem_dealloc(tmem_base, 512);
}

int main() {
  long long* d;
  cudaMalloc(&d, 128);
  const int iters = 1000;
  cudaFuncSetAttribute(cost_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024);
  cost_kernel<<<1, 128, 80 * 1024>>>(d, iters);
  cost_kernel<<<1, 128, 80 * 1024>>>(d, iters);
  cudaError_t e = cudaDeviceSynchronize();
  long long h[16];
  cudaMemcpy(h, d, 128, cudaMemcpyDeviceToHost);
  printf("status: %s\n", cudaGetErrorString(e));
  const char* names[8] = {"try_wait (ready)", "arrive.expect_tx(0)", "tcgen05.fence::after", "tcgen05.commit (idle)", "4 MMA(N=64)+commit issue", "  ... until complete",
                          "try_wait+fence+4 MMA+commit issue", "  ... until complete"};
  for (int i = 0; i < 8; ++i) printf("%-36s %8.1f cycles/iter\n", names[i], (double)h[i] / iters);
  return 0;
}
