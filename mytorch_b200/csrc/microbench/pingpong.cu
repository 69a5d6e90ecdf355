// Producer/consumer ring of mbarriers between two single threads (as in the tcgen05 kernels),
// nothing else: cycles per iteration against ring depth, with the consumer releasing a slot
// through tcgen05.commit or through a plain arrive.
#include <cstdio>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>
#include "../tc_common.cuh"
using namespace tc;

template <int MODE, int NM, int BN>  // 0: commit, 1: plain arrive, 2: commit + NM MMAs of width BN
__global__ void __launch_bounds__(192) pp_kernel(long long* out, int iters, int depth) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ uint64_t full[8], empty[8];
  __shared__ uint32_t tmem_base;
  __shared__ int abort_flag;
  uint32_t sbase = (smem_u32(smem) + 1023) & ~1023u;
  for (int i = threadIdx.x; i < (64 * 1024) / 4; i += blockDim.x) ((float*)smem)[i] = 0.f;
  if (threadIdx.x == 0) {
    for (int i = 0; i < 8; ++i) { mbar_init(smem_u32(&full[i]), 1); mbar_init(smem_u32(&empty[i]), 1); }
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x >= 32 && threadIdx.x < 64) { tmem_alloc(smem_u32(&tmem_base), 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  fence_proxy_async();
  volatile int* ab = &abort_flag;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (warp == 0 && lane == 0) {
    int s = 0; uint32_t ph = 0;
    long long t0 = clock64();
    for (int i = 0; i < iters; ++i) {
      if (!mbar_wait(smem_u32(&empty[s]), ph ^ 1u, ab, 1)) break;
      mbar_expect_tx(smem_u32(&full[s]), 0);
      if (++s == depth) { s = 0; ph ^= 1u; }
    }
    out[0] = clock64() - t0;
  } else if (warp == 1 && lane == 0) {
    const uint32_t idesc = idesc_tf32(128, BN, 0, 0);
    const uint32_t a_lo = desc_lo_kmajor(sbase), b_lo = desc_lo_kmajor(sbase + 32768), hi = desc_hi_kmajor();
    int s = 0; uint32_t ph = 0;
    long long t0 = clock64();
    for (int i = 0; i < iters; ++i) {
      if (!mbar_wait(smem_u32(&full[s]), ph, ab, 2)) break;
      tc_fence_after();
      if (MODE == 2) {
#pragma unroll
        for (int k = 0; k < NM; ++k) mma_tf32_words(tmem_base, a_lo + 2 * (k & 3), hi, b_lo + 2 * (k & 3), hi, idesc, 1);
      }
      if (MODE == 1) mbar_arrive(smem_u32(&empty[s])); else mma_commit(smem_u32(&empty[s]));
      if (++s == depth) { s = 0; ph ^= 1u; }
    }
    out[1] = clock64() - t0;
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x >= 32 && threadIdx.x < 64) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

template <int MODE, int NM, int BN>
void run(long long* d, int depth) {
  const int iters = 4000;
  cudaFuncSetAttribute(pp_kernel<MODE, NM, BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024);
  pp_kernel<MODE, NM, BN><<<1, 192, 80 * 1024>>>(d, iters, depth);
  pp_kernel<MODE, NM, BN><<<1, 192, 80 * 1024>>>(d, iters, depth);
  cudaError_t e = cudaDeviceSynchronize();
  long long h[2];
  cudaMemcpy(h, d, 16, cudaMemcpyDeviceToHost);
  printf("mode %d NM %2d BN %3d depth %d: producer %7.1f  consumer %7.1f cycles/iter (%s)\n", MODE, NM, BN, depth, (double)h[0] / iters, (double)h[1] / iters, cudaGetErrorString(e));
}

int main() {
  long long* d;
  cudaMalloc(&d, 64);
  run<1, 0, 64>(d, 4);
  run<0, 0, 64>(d, 4);
  run<2, 4, 64>(d, 4);
  run<2, 8, 64>(d, 4);
  run<2, 12, 64>(d, 4);
  run<2, 16, 64>(d, 4);
  run<2, 36, 64>(d, 4);
  run<2, 4, 128>(d, 4);
  run<2, 8, 128>(d, 4);
  run<2, 12, 128>(d, 4);
  run<2, 4, 256>(d, 4);
  run<2, 8, 256>(d, 4);
  return 0;
}
