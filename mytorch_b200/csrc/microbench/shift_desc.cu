// Does a K-major SWIZZLE_128B A descriptor whose start address is a multiple of 128 B (a whole
// row) but not of 1024 B read the rows one expects?  With and without the base-offset field.
#include <cstdio>
#include <cstdint>
#include <cstdlib>
#include <vector>
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>
#include "../tc_common.cuh"
using namespace tc;

constexpr int kRowsPerLoad = 34, kLoads = 7, kARows = kRowsPerLoad * kLoads;  // 238
constexpr int kNumShift = 6, kVariants = kNumShift * 2;
__constant__ int c_shift[kNumShift] = {0, 1, 3, 8, 35, 69};

__global__ void __launch_bounds__(128) shift_kernel(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB, float* out) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ uint64_t bar_load, bar_mma;
  __shared__ uint32_t tmem_base;
  uint32_t sbase = (smem_u32(smem_raw) + 1023) & ~1023u;
  const uint32_t sA = sbase, sB = sbase + 32768;
  volatile int abort_flag = 0;
  if (threadIdx.x == 0) { mbar_init(smem_u32(&bar_load), 1); mbar_init(smem_u32(&bar_mma), 1); fence_barrier_init(); }
  __syncthreads();
  if (threadIdx.x < 32) { tmem_alloc(smem_u32(&tmem_base), 64); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (threadIdx.x == 0) {
    mbar_expect_tx(smem_u32(&bar_load), kARows * 128 + 64 * 128);
    for (int i = 0; i < kLoads; ++i) tma_load_2d(sA + i * kRowsPerLoad * 128, &mapA, smem_u32(&bar_load), 0, i * kRowsPerLoad);
    tma_load_2d(sB, &mapB, smem_u32(&bar_load), 0, 0);
  }
  bool ok = mbar_wait(smem_u32(&bar_load), 0, &abort_flag, 1);
  __syncthreads();
  tc_fence_after();
  for (int v = 0; v < kVariants && ok; ++v) {
    const int shift = c_shift[v % kNumShift];
    const int use_bo = v / kNumShift;
    if (threadIdx.x == 0) {
      const uint32_t a_addr = sA + shift * 128;
      const uint32_t bo = use_bo ? ((a_addr >> 7) & 7u) : 0u;
      const uint32_t a_hi = desc_hi_kmajor() | (bo << 17);
      const uint32_t a_lo = desc_lo_kmajor(a_addr), b_lo = desc_lo_kmajor(sB);
      const uint32_t idesc = idesc_tf32(128, 64, 0, 0);
      for (int k = 0; k < 4; ++k) mma_tf32_words(tmem_base, a_lo + 2 * k, a_hi, b_lo + 2 * k, desc_hi_kmajor(), idesc, k > 0);
      mma_commit(smem_u32(&bar_mma));
    }
    ok = mbar_wait(smem_u32(&bar_mma), v & 1, &abort_flag, 2);
    tc_fence_after();
    if (ok) {
      const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
      uint32_t r[32];
      for (int c0 = 0; c0 < 64; c0 += 32) {
        tmem_ld_32x32(tmem_base + ((uint32_t)(warp * 32) << 16) + c0, r);
        tmem_ld_wait();
        for (int j = 0; j < 32; ++j) out[((long long)v * 128 + warp * 32 + lane) * 64 + c0 + j] = __uint_as_float(r[j]);
      }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }
  tc_fence_before();
  __syncthreads();
  if (threadIdx.x < 32) tmem_dealloc(tmem_base, 64);
}

static PFN_cuTensorMapEncodeTiled_v12000 enc;
static void make_map(CUtensorMap* m, const float* base, int rows, int box_rows) {
  cuuint64_t dims[2] = {32, (cuuint64_t)rows};
  cuuint64_t strides[1] = {128};
  cuuint32_t box[2] = {32, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { printf("encode failed %d\n", (int)r); exit(1); }
}

int main() {
  cudaDriverEntryPointQueryResult q;
  void* fn = nullptr;
  cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
  enc = (PFN_cuTensorMapEncodeTiled_v12000)fn;
  const int R = 320;
  std::vector<float> A(R * 32), B(64 * 32);
  for (int r = 0; r < R; ++r) for (int k = 0; k < 32; ++k) A[r * 32 + k] = (float)(((r * 7 + k * 3) % 17) - 8);
  for (int n = 0; n < 64; ++n) for (int k = 0; k < 32; ++k) B[n * 32 + k] = (float)(((n * 5 + k) % 13) - 6);
  float *dA, *dB, *dO;
  cudaMalloc(&dA, A.size() * 4); cudaMalloc(&dB, B.size() * 4); cudaMalloc(&dO, kVariants * 128 * 64 * 4);
  cudaMemcpy(dA, A.data(), A.size() * 4, cudaMemcpyHostToDevice);
  cudaMemcpy(dB, B.data(), B.size() * 4, cudaMemcpyHostToDevice);
  cudaMemset(dO, 0, kVariants * 128 * 64 * 4);
  CUtensorMap mA, mB;
  make_map(&mA, dA, R, kRowsPerLoad);
  make_map(&mB, dB, 64, 64);
  cudaFuncSetAttribute(shift_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 48 * 1024);
  shift_kernel<<<1, 128, 48 * 1024>>>(mA, mB, dO);
  cudaError_t e = cudaDeviceSynchronize();
  printf("kernel: %s\n", cudaGetErrorString(e));
  if (e != cudaSuccess) return 1;
  std::vector<float> O(kVariants * 128 * 64);
  cudaMemcpy(O.data(), dO, O.size() * 4, cudaMemcpyDeviceToHost);
  const int shifts[kNumShift] = {0, 1, 3, 8, 35, 69};
  for (int v = 0; v < kVariants; ++v) {
    int s = shifts[v % kNumShift];
    double worst = 0; int bad = 0;
    for (int m = 0; m < 128; ++m) for (int n = 0; n < 64; ++n) {
      double ref = 0;
      for (int k = 0; k < 32; ++k) ref += (double)A[(m + s) * 32 + k] * B[n * 32 + k];
      double d = fabs(ref - O[((long long)v * 128 + m) * 64 + n]);
      if (d > worst) worst = d;
      if (d > 1e-3) ++bad;
    }
    printf("shift %3d base_offset %s: max abs err %.3f, wrong elements %d / 8192\n", s, v / kNumShift ? "set" : "0  ", worst, bad);
  }
  return 0;
}
