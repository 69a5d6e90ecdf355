// MN-major (32-byte-atom 128B swizzle) operands read through descriptors whose start is shifted
// by whole 128-byte rows (= K index), and an A operand whose four 32-wide M blocks are the SAME
// panel shifted by one row each (LBO = 128 B).
#include <cstdio>
#include <cstdint>
#include <cstdlib>
#include <cmath>
#include <vector>
#include <cuda.h>
#include <cudaTypedefs.h>
#include <cuda_runtime.h>
#include "../tc_common.cuh"
using namespace tc;

constexpr int kRowsPerLoad = 34, kLoads = 5, kRows = kRowsPerLoad * kLoads;  // 170 positions staged
constexpr uint32_t kPanel = kRows * 128;                                       // 21760 B
constexpr int kCases = 6;
__constant__ int c_s0[kCases] = {0, 1, 2, 5, 35, 69};
__constant__ int c_s1[kCases] = {0, 0, 3, 35, 1, 70};

__global__ void __launch_bounds__(128) mn_kernel(const __grid_constant__ CUtensorMap mapX, const __grid_constant__ CUtensorMap mapY, float* out) {
  extern __shared__ unsigned char smem_raw[];
  __shared__ uint64_t bar_load, bar_mma;
  __shared__ uint32_t tmem_base;
  uint32_t sbase = (smem_u32(smem_raw) + 1023) & ~1023u;
  const uint32_t sX = sbase, sY = sbase + 22528;  // X panel, then two Y panels kPanel apart
  volatile int abort_flag = 0;
  if (threadIdx.x == 0) { mbar_init(smem_u32(&bar_load), 1); mbar_init(smem_u32(&bar_mma), 1); fence_barrier_init(); }
  __syncthreads();
  if (threadIdx.x < 32) { tmem_alloc(smem_u32(&tmem_base), 64); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  if (threadIdx.x == 0) {
    mbar_expect_tx(smem_u32(&bar_load), 3 * kPanel);
    for (int i = 0; i < kLoads; ++i) {
      tma_load_2d(sX + i * kRowsPerLoad * 128, &mapX, smem_u32(&bar_load), 0, i * kRowsPerLoad);
      tma_load_2d(sY + i * kRowsPerLoad * 128, &mapY, smem_u32(&bar_load), 0, i * kRowsPerLoad);
      tma_load_2d(sY + kPanel + i * kRowsPerLoad * 128, &mapY, smem_u32(&bar_load), 32, i * kRowsPerLoad);
    }
  }
  bool ok = mbar_wait(smem_u32(&bar_load), 0, &abort_flag, 1);
  __syncthreads();
  tc_fence_after();
  for (int v = 0; v < kCases && ok; ++v) {
    if (threadIdx.x == 0) {
      const uint32_t a_lo = desc_lo_mnmajor(sX + c_s0[v] * 128, 128u);      // four M blocks one row apart
      const uint32_t b_lo = desc_lo_mnmajor(sY + c_s1[v] * 128, kPanel);    // two N blocks one panel apart
      const uint32_t idesc = idesc_tf32(128, 64, 1, 1);
      for (int k = 0; k < 4; ++k) mma_tf32_words(tmem_base, a_lo + k * 64, desc_hi_mnmajor(), b_lo + k * 64, desc_hi_mnmajor(), idesc, k > 0);
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
static void make_map(CUtensorMap* m, const float* base, int rows, int cols, int box_rows) {
  cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)cols * 4};
  cuuint32_t box[2] = {32, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, (void*)base, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { printf("encode failed %d\n", (int)r); exit(1); }
}

int main() {
  cudaDriverEntryPointQueryResult q;
  void* fn = nullptr;
  cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
  enc = (PFN_cuTensorMapEncodeTiled_v12000)fn;
  const int R = 256;
  std::vector<float> X(R * 32), Y(R * 64);
  for (int r = 0; r < R; ++r) for (int c = 0; c < 32; ++c) X[r * 32 + c] = (float)(((r * 7 + c * 3) % 17) - 8);
  for (int r = 0; r < R; ++r) for (int c = 0; c < 64; ++c) Y[r * 64 + c] = (float)(((r * 5 + c * 11) % 13) - 6);
  float *dX, *dY, *dO;
  cudaMalloc(&dX, X.size() * 4); cudaMalloc(&dY, Y.size() * 4); cudaMalloc(&dO, kCases * 128 * 64 * 4);
  cudaMemcpy(dX, X.data(), X.size() * 4, cudaMemcpyHostToDevice);
  cudaMemcpy(dY, Y.data(), Y.size() * 4, cudaMemcpyHostToDevice);
  cudaMemset(dO, 0, kCases * 128 * 64 * 4);
  CUtensorMap mX, mY;
  make_map(&mX, dX, R, 32, kRowsPerLoad);
  make_map(&mY, dY, R, 64, kRowsPerLoad);
  // 1024 slack + X panel (22528) + 2 Y panels (43520) = 67072
  cudaFuncSetAttribute(mn_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 72 * 1024);
  mn_kernel<<<1, 128, 72 * 1024>>>(mX, mY, dO);
  cudaError_t e = cudaDeviceSynchronize();
  printf("kernel: %s\n", cudaGetErrorString(e));
  if (e != cudaSuccess) return 1;
  std::vector<float> O(kCases * 128 * 64);
  cudaMemcpy(O.data(), dO, O.size() * 4, cudaMemcpyDeviceToHost);
  const int s0[kCases] = {0, 1, 2, 5, 35, 69}, s1[kCases] = {0, 0, 3, 35, 1, 70};
  for (int v = 0; v < kCases; ++v) {
    double worst = 0; int bad = 0;
    for (int m = 0; m < 128; ++m) for (int n = 0; n < 64; ++n) {
      const int j = m / 32, c = m % 32;
      double ref = 0;
      for (int k = 0; k < 32; ++k) ref += (double)X[(s0[v] + j + k) * 32 + c] * Y[(s1[v] + k) * 64 + n];
      double d = fabs(ref - O[((long long)v * 128 + m) * 64 + n]);
      if (d > worst) worst = d;
      if (d > 1e-3) ++bad;
    }
    printf("A shift %3d, B shift %3d: max abs err %.3f, wrong elements %d / 8192\n", s0[v], s1[v], worst, bad);
  }
  return 0;
}
