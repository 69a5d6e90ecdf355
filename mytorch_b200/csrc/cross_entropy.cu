// Softmax cross-entropy (mean over the batch) forward and backward: one warp per sample,
// shuffle reductions over the class dimension, per-sample losses combined in a fixed order.
#include "common.cuh"

namespace {

__device__ __forceinline__ float warp_max(float v) {
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__global__ void __launch_bounds__(128) ce_rows_kernel(const float* __restrict__ z, const long long* __restrict__ target, int B, int C,
                                                       float* __restrict__ row_loss, float* __restrict__ dz, const float* __restrict__ dy) {
  int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  int lane = threadIdx.x & 31;
  if (row >= B) return;
  const float* p = z + (long long)row * C;
  float mx = -3.402823466e38f;
  for (int c = lane; c < C; c += 32) mx = fmaxf(mx, p[c]);
  mx = warp_max(mx);
  float s = 0.f;
  for (int c = lane; c < C; c += 32) s += expf(p[c] - mx);
  s = warp_sum(s);
  long long t = target[row];
  if (row_loss) {
    // -log(softmax[t]) = log(sum) - (z_t - max)
    if (lane == 0) row_loss[row] = (t >= 0 && t < C) ? logf(s) - (p[t] - mx) : 0.f;
  }
  if (dz) {
    float g = dy[0] / (float)B;
    float inv = 1.f / s;
    for (int c = lane; c < C; c += 32) {
      float sm = expf(p[c] - mx) * inv;
      dz[(long long)row * C + c] = (sm - (c == t ? 1.f : 0.f)) * g;
    }
  }
}

__global__ void __launch_bounds__(256) ce_mean_kernel(const float* __restrict__ row_loss, int B, float* __restrict__ loss) {
  __shared__ double sm[256];
  double s = 0;
  for (int i = threadIdx.x; i < B; i += 256) s += row_loss[i];
  sm[threadIdx.x] = s;
  __syncthreads();
  for (int w = 128; w > 0; w >>= 1) {
    if (threadIdx.x < w) sm[threadIdx.x] += sm[threadIdx.x + w];
    __syncthreads();
  }
  if (threadIdx.x == 0) loss[0] = (float)(sm[0] / B);
}

}  // namespace

MTB_API long long mtb_cross_entropy_workspace_bytes(int batch) { return (long long)batch * 4 + 256; }

// loss[0] = mean_b(-log softmax(logits[b])[target[b]]); logits row-major [B, C], target int64.
MTB_API int mtb_cross_entropy_forward_f32(int batch, int classes, const float* logits, const long long* target, float* loss, void* workspace,
                                          long long workspace_bytes, void* stream) {
  MTB_REQUIRE(batch > 0 && classes > 0 && logits && target && loss && workspace, "cross_entropy_forward: bad arguments");
  MTB_REQUIRE(workspace_bytes >= mtb_cross_entropy_workspace_bytes(batch), "cross_entropy_forward: workspace too small");
  cudaStream_t st = (cudaStream_t)stream;
  ce_rows_kernel<<<mtb_div_up(batch, 4), 128, 0, st>>>(logits, target, batch, classes, (float*)workspace, nullptr, nullptr);
  MTB_LAUNCH_CHECK("ce_rows_kernel");
  ce_mean_kernel<<<1, 256, 0, st>>>((const float*)workspace, batch, loss);
  MTB_LAUNCH_CHECK("ce_mean_kernel");
  return MTB_OK;
}

// dlogits = (softmax - onehot) * dy[0] / B, dy a one-element device tensor.
MTB_API int mtb_cross_entropy_backward_f32(int batch, int classes, const float* logits, const long long* target, const float* dy,
                                           float* dlogits, void* stream) {
  MTB_REQUIRE(batch > 0 && classes > 0 && logits && target && dy && dlogits, "cross_entropy_backward: bad arguments");
  ce_rows_kernel<<<mtb_div_up(batch, 4), 128, 0, (cudaStream_t)stream>>>(logits, target, batch, classes, nullptr, dlogits, dy);
  MTB_LAUNCH_CHECK("ce_rows_kernel");
  return MTB_OK;
}
