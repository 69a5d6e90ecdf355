// SGD with momentum / dampening / Nesterov / weight decay / maximize, per tensor and as a
// multi-tensor launch (pointer table passed by value in kernel parameters, so a whole model
// updates in a few launches and the launch can be captured in a CUDA graph).
#include "common.cuh"

namespace {

struct SgdHyper {
  float lr, weight_decay, momentum, one_minus_dampening, grad_scale;
  int nesterov, maximize, first;
};

__device__ __forceinline__ void sgd_update(float& p, float g, float& buf, const SgdHyper& h) {
  g = (h.maximize ? -g : g) * h.grad_scale + h.weight_decay * p;
  buf = h.first ? g : (h.momentum * buf + h.one_minus_dampening * g);
  g = h.nesterov ? (g + h.momentum * buf) : buf;
  p -= g * h.lr;
}

__device__ __forceinline__ void sgd_span(float* p, const float* g, float* buf, long long n, const SgdHyper& h, long long tid, long long nthreads) {
  bool vec = ((reinterpret_cast<uintptr_t>(p) | reinterpret_cast<uintptr_t>(g) | reinterpret_cast<uintptr_t>(buf)) & 15u) == 0;
  long long n4 = vec ? n / 4 : 0;
  for (long long v = tid; v < n4; v += nthreads) {
    float4 pp = ld4(p + 4 * v), gg = ld4(g + 4 * v), bb = h.first ? make_float4(0, 0, 0, 0) : ld4(buf + 4 * v);
    sgd_update(pp.x, gg.x, bb.x, h);
    sgd_update(pp.y, gg.y, bb.y, h);
    sgd_update(pp.z, gg.z, bb.z, h);
    sgd_update(pp.w, gg.w, bb.w, h);
    st4(p + 4 * v, pp);
    st4(buf + 4 * v, bb);
  }
  for (long long t = 4 * n4 + tid; t < n; t += nthreads) {
    float pp = p[t], bb = h.first ? 0.f : buf[t];
    sgd_update(pp, g[t], bb, h);
    p[t] = pp;
    buf[t] = bb;
  }
}

__global__ void __launch_bounds__(256) sgd_kernel(float* p, const float* g, float* buf, long long n, SgdHyper h) {
  sgd_span(p, g, buf, n, h, blockIdx.x * (long long)blockDim.x + threadIdx.x, (long long)gridDim.x * blockDim.x);
}

constexpr int kMaxTensors = 96;
constexpr int kSgdChunk = 4096;  // elements per CTA: four float4 per thread and array in flight
struct SgdTable {
  float* p[kMaxTensors];
  const float* g[kMaxTensors];
  float* buf[kMaxTensors];
  long long n[kMaxTensors];
  int first[kMaxTensors];
  int chunk_start[kMaxTensors + 1];  // CTA b works on tensor k with chunk_start[k] <= b < chunk_start[k + 1]
  int count;
};

// One CTA per chunk of kSgdChunk elements of one tensor (a model has a few large tensors and dozens of
// tiny ones: a grid of tensors x the largest tensor's chunks would be mostly empty CTAs).
__global__ void __launch_bounds__(256) sgd_multi_kernel(const __grid_constant__ SgdTable t, SgdHyper h) {
  int lo = 0, hi = t.count - 1;
  while (lo < hi) {  // last k with chunk_start[k] <= blockIdx.x
    const int mid = (lo + hi + 1) >> 1;
    if (t.chunk_start[mid] <= (int)blockIdx.x) lo = mid; else hi = mid - 1;
  }
  const int k = lo;
  const long long e0 = (long long)((int)blockIdx.x - t.chunk_start[k]) * kSgdChunk;
  const long long left = t.n[k] - e0;
  h.first = t.first[k];
  sgd_span(t.p[k] + e0, t.g[k] + e0, t.buf[k] + e0, left < kSgdChunk ? left : kSgdChunk, h, threadIdx.x, blockDim.x);
}

// Gather `count` gradient tensors into one flat buffer, scaling on the way.
struct PackTable {
  const float* src[kMaxTensors];
  long long off[kMaxTensors];
  long long n[kMaxTensors];
  int count;
};
__global__ void __launch_bounds__(256) pack_kernel(const __grid_constant__ PackTable t, float* dst, float scale) {
  int k = blockIdx.y;
  if (k >= t.count) return;
  long long n = t.n[k];
  const float* s = t.src[k];
  float* d = dst + t.off[k];
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += stride) d[i] = s[i] * scale;
}

}  // namespace

// One parameter tensor. grad_scale multiplies the gradient first (1/world_size under data
// parallelism, 1 otherwise). is_first != 0: the momentum buffer is initialised to g.
MTB_API int mtb_sgd_f32(float* param, const float* grad, float* momentum_buffer, long long n, int is_first, double lr, double weight_decay,
                        double momentum, double dampening, int nesterov, int maximize, double grad_scale, void* stream) {
  MTB_REQUIRE(n >= 0 && ((param && grad && momentum_buffer) || n == 0), "sgd: bad arguments");
  if (n == 0) return MTB_OK;
  SgdHyper h{(float)lr, (float)weight_decay, (float)momentum, (float)(1.0 - dampening), (float)grad_scale, nesterov, maximize, is_first};
  sgd_kernel<<<mtb_stream_grid((n + 3) / 4, 256), 256, 0, (cudaStream_t)stream>>>(param, grad, momentum_buffer, n, h);
  MTB_LAUNCH_CHECK("sgd_kernel");
  return MTB_OK;
}

// `count` parameter tensors with shared hyper-parameters. Host arrays of device pointers.
MTB_API int mtb_sgd_multi_f32(int count, float* const* params, const float* const* grads, float* const* momentum_buffers, const long long* sizes,
                              const int* is_first, double lr, double weight_decay, double momentum, double dampening, int nesterov,
                              int maximize, double grad_scale, void* stream) {
  MTB_REQUIRE(count >= 0 && (count == 0 || (params && grads && momentum_buffers && sizes && is_first)), "sgd_multi: bad arguments");
  SgdHyper h{(float)lr, (float)weight_decay, (float)momentum, (float)(1.0 - dampening), (float)grad_scale, nesterov, maximize, 0};
  for (int base = 0; base < count; base += kMaxTensors) {
    SgdTable t;
    t.count = count - base < kMaxTensors ? count - base : kMaxTensors;
    long long chunks = 0;
    for (int k = 0; k < t.count; ++k) {
      MTB_REQUIRE(sizes[base + k] >= 0 && params[base + k] && grads[base + k] && momentum_buffers[base + k], "sgd_multi: null tensor %d", base + k);
      t.p[k] = params[base + k];
      t.g[k] = grads[base + k];
      t.buf[k] = momentum_buffers[base + k];
      t.n[k] = sizes[base + k];
      t.first[k] = is_first[base + k];
      t.chunk_start[k] = (int)chunks;
      chunks += (t.n[k] + kSgdChunk - 1) / kSgdChunk;
      MTB_REQUIRE(chunks < (1LL << 30), "sgd_multi: too many elements in one call");
    }
    t.chunk_start[t.count] = (int)chunks;
    if (chunks == 0) continue;
    dim3 grid((unsigned int)chunks);
    sgd_multi_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(t, h);
    MTB_LAUNCH_CHECK("sgd_multi_kernel");
  }
  return MTB_OK;
}

// dst[offsets[k] : offsets[k] + sizes[k]] = scale * srcs[k][:] for k < count.
MTB_API int mtb_pack_scale_f32(int count, const float* const* srcs, const long long* offsets, const long long* sizes, float* dst, double scale,
                               void* stream) {
  MTB_REQUIRE(count >= 0 && (count == 0 || (srcs && offsets && sizes && dst)), "pack_scale: bad arguments");
  for (int base = 0; base < count; base += kMaxTensors) {
    PackTable t;
    t.count = count - base < kMaxTensors ? count - base : kMaxTensors;
    long long maxn = 1;
    for (int k = 0; k < t.count; ++k) {
      t.src[k] = srcs[base + k];
      t.off[k] = offsets[base + k];
      t.n[k] = sizes[base + k];
      if (t.n[k] > maxn) maxn = t.n[k];
    }
    int gx = mtb_div_up(maxn, 256 * 4);
    int cap = mtb_sm_count() * 4;
    if (gx > cap) gx = cap;
    if (gx < 1) gx = 1;
    pack_kernel<<<dim3(gx, t.count), 256, 0, (cudaStream_t)stream>>>(t, dst, (float)scale);
    MTB_LAUNCH_CHECK("pack_kernel");
  }
  return MTB_OK;
}
