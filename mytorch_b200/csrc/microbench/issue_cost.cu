// (Operand regions: A at +1 KB, nine weight taps of N*128 B from +64 KB; N <= 64 keeps them inside the
// 160 KB that are zeroed and the 200 KB that are allocated.)
// Issue cost of tcgen05.mma from (a) a lane-0 branch and (b) a converged warp with elect.sync,
// with descriptors that change per MMA (runtime strides), on a cheap shape so that the tensor
// pipe is not the limit.
#include <cstdio>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>
#include "../tc_common.cuh"
using namespace tc;

template <int MODE, int M, int N>
__global__ void __launch_bounds__(128) issue_kernel(long long* out, int iters, int row_step, int tap_step, int kw_n) {
  extern __shared__ __align__(1024) unsigned char smem[];
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base;
  __shared__ int abort_flag;
  uint32_t sbase = (smem_u32(smem) + 1023) & ~1023u;
  for (int i = threadIdx.x; i < (160 * 1024) / 4; i += blockDim.x) ((float*)smem)[i] = 0.f;
  if (threadIdx.x == 0) { mbar_init(smem_u32(&bar), 1); abort_flag = 0; fence_barrier_init(); }
  __syncthreads();
  if (threadIdx.x < 32) { tmem_alloc(smem_u32(&tmem_base), 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  fence_proxy_async();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t idesc = idesc_tf32(M, N, 0, 0);
  const uint32_t hi = desc_hi_kmajor();
  const uint32_t a0 = desc_lo_kmajor(sbase + 1024), b0 = desc_lo_kmajor(sbase + 65536);
  const uint32_t d = tmem_base;
  if (warp == 1) {
    long long t0 = clock64();
    if (MODE == 0) {
      if (lane == 0) {
        for (int it = 0; it < iters; ++it) {
          uint32_t a_row = a0, a_lo = a0, b_lo = b0;
          int kw = 0;
          for (int tap = 0; tap < 9; ++tap, b_lo += tap_step) {
            mma_tf32_words(d, a_lo, hi, b_lo, hi, idesc, 1u);
            mma_tf32_words(d, a_lo + 2u, hi, b_lo + 2u, hi, idesc, 1u);
            mma_tf32_words(d, a_lo + 4u, hi, b_lo + 4u, hi, idesc, 1u);
            mma_tf32_words(d, a_lo + 6u, hi, b_lo + 6u, hi, idesc, 1u);
            a_lo += 8u;
            if (++kw == kw_n) { kw = 0; a_row += row_step; a_lo = a_row; }
          }
        }
        mma_commit(smem_u32(&bar));
      }
    } else {
      for (int it = 0; it < iters; ++it) {
        if (elect_one()) {
#pragma unroll
          for (int kh = 0; kh < 3; ++kh)
#pragma unroll
            for (int kw = 0; kw < 3; ++kw)
#pragma unroll
              for (int k = 0; k < 4; ++k)
                mma_tf32_words(d, a0 + kh * row_step + kw * 8 + 2 * k, hi, b0 + (kh * 3 + kw) * tap_step + 2 * k, hi, idesc, 1u);
        }
        __syncwarp();
      }
      if (elect_one()) mma_commit(smem_u32(&bar));
    }
    long long t1 = clock64();
    volatile int* ab = &abort_flag;
    mbar_wait(smem_u32(&bar), 0, ab, 1);
    long long t2 = clock64();
    if (lane == 0) { out[0] = t1 - t0; out[1] = t2 - t0; }
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

template <int MODE, int M, int N>
void run(long long* d) {
  const int iters = 200;
  auto k = issue_kernel<MODE, M, N>;
  cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
  k<<<1, 128, 200 * 1024>>>(d, iters, 34 * 8, (N * 128) >> 4, 3);
  k<<<1, 128, 200 * 1024>>>(d, iters, 34 * 8, (N * 128) >> 4, 3);
  cudaError_t e = cudaDeviceSynchronize();
  long long h[2];
  cudaMemcpy(h, d, 16, cudaMemcpyDeviceToHost);
  printf("%s M=%3d N=%3d: issue %6.1f cycles/MMA, until complete %6.1f cycles/MMA (%s)\n", MODE ? "elect+unrolled" : "lane0+loops   ", M, N,
         (double)h[0] / (iters * 36.0), (double)h[1] / (iters * 36.0), cudaGetErrorString(e));
}

int main() {
  long long* d;
  cudaMalloc(&d, 64);
  run<0, 64, 8>(d);
  run<1, 64, 8>(d);
  run<0, 128, 16>(d);
  run<1, 128, 16>(d);
  run<0, 128, 64>(d);
  run<1, 128, 64>(d);
  return 0;
}
