// Cycles per tcgen05.mma (kind::tf32, K=8) for several (M,N); operands in smem (contents irrelevant).
#include <cstdio>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>
#include "../tc_common.cuh"
using namespace tc;

template <int M, int N>
__global__ void __launch_bounds__(128) rate_kernel(long long* out, int iters, int shift_rows) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base;
  uint32_t sbase = (smem_u32(smem) + 1023) & ~1023u;
  // zero the operands so that the accumulators stay finite
  for (int i = threadIdx.x; i < (64 * 1024) / 4; i += blockDim.x) ((float*)smem)[i] = 0.f;
  if (threadIdx.x == 0) { mbar_init(smem_u32(&bar), 1); fence_barrier_init(); }
  __syncthreads();
  if (threadIdx.x < 32) { tmem_alloc(smem_u32(&tmem_base), 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  fence_proxy_async();
  long long t0 = 0, t1 = 0;
  if (threadIdx.x == 0) {
    const uint32_t idesc = idesc_tf32(M, N, 0, 0);
    const uint32_t a_lo = desc_lo_kmajor(sbase + shift_rows * 128), b_lo = desc_lo_kmajor(sbase + 32768);
    const uint32_t hi = desc_hi_kmajor();
    t0 = clock64();
    for (int it = 0; it < iters; ++it) {
#pragma unroll
      for (int k = 0; k < 4; ++k) mma_tf32_words(tmem_base, a_lo + 2 * k, hi, b_lo + 2 * k, hi, idesc, 1);
    }
    mma_commit(smem_u32(&bar));
    volatile int abort_flag = 0;
    mbar_wait(smem_u32(&bar), 0, &abort_flag, 1);
    t1 = clock64();
    out[0] = t1 - t0;
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) tmem_dealloc(tmem_base, 512);
}

template <int M, int N>
void run(long long* d, int iters, int shift_rows = 0) {
  cudaFuncSetAttribute(rate_kernel<M, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024);
  rate_kernel<M, N><<<1, 128, 80 * 1024>>>(d, iters, shift_rows);
  rate_kernel<M, N><<<1, 128, 80 * 1024>>>(d, iters, shift_rows);
  cudaError_t e = cudaDeviceSynchronize();
  long long h = 0;
  cudaMemcpy(&h, d, 8, cudaMemcpyDeviceToHost);
  double per = (double)h / (iters * 4.0);
  printf("shift %2d M=%3d N=%3d: %7.1f cycles/MMA  -> %6.1f flop/cycle/SM  (%s)\n", shift_rows, M, N, per, 2.0 * M * N * 8 / per, cudaGetErrorString(e));
}

int main() {
  long long* d;
  cudaMalloc(&d, 64);
  const int iters = 2000;
  run<128, 64>(d, iters);
  run<128, 128>(d, iters);
  run<128, 256>(d, iters);
  run<64, 64>(d, iters);
  run<64, 128>(d, iters);
  run<64, 256>(d, iters);
  for (int sh : {1, 3, 4, 8, 35}) { run<128, 64>(d, iters, sh); run<128, 128>(d, iters, sh); run<128, 256>(d, iters, sh); }
  return 0;
}
