// Reductions: per-channel column sums (bias gradients), global average pooling over
// channels-last activations, and a generic strided sum for the remaining `sum_scale` cases.
// All are deterministic: per-CTA partials in scratch, combined in a fixed order.
#include "colreduce.cuh"

namespace {

template <int V>
__global__ void __launch_bounds__(256) colsum_partial_kernel(const float* __restrict__ a, long long rows, int C, int L, long long rows_per_block,
                                                              float* __restrict__ partial) {
  const int lane = threadIdx.x & (L - 1);
  const int rsub = threadIdx.x / L;
  const int R = 256 / L;
  const int cg = blockIdx.x * L + lane;
  const bool active = cg * V < C;
  float acc[V];
#pragma unroll
  for (int i = 0; i < V; ++i) acc[i] = 0.f;
  long long r0 = blockIdx.y * rows_per_block;
  long long r1 = r0 + rows_per_block < rows ? r0 + rows_per_block : rows;
  if (active) {
#pragma unroll 4
    for (long long r = r0 + rsub; r < r1; r += R) {
      VecF<V> f = vload<V>(a + r * C + (long long)cg * V);
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] += f.v[i];
    }
  }
  __shared__ float sm[V][256];
#pragma unroll
  for (int i = 0; i < V; ++i) sm[i][threadIdx.x] = acc[i];
  __syncthreads();
  if (rsub == 0 && active) {
    for (int k = 1; k < R; ++k) {
#pragma unroll
      for (int i = 0; i < V; ++i) acc[i] += sm[i][k * L + lane];
    }
    float* p = partial + (long long)blockIdx.y * C + (long long)cg * V;
#pragma unroll
    for (int i = 0; i < V; ++i) p[i] = acc[i];
  }
}

// Thirty-two threads per channel (consecutive threads read consecutive channels), fixed order.
__global__ void __launch_bounds__(1024) colsum_final_kernel(const float* __restrict__ partial, int P, int C, float scale, float* __restrict__ out) {
  const int cx = threadIdx.x & 31, py = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float s = 0.f;
  if (c < C) {
#pragma unroll 4
    for (int p = py; p < P; p += 32) s += partial[(long long)p * C + c];
  }
  __shared__ float t[32][33];
  t[py][cx] = s;
  __syncthreads();
  if (py != 0 || c >= C) return;
  for (int k = 1; k < 32; ++k) s += t[k][cx];
  out[c] = s * scale;
}

// y[n, c] = scale * sum_{hw} x[n, hw, c]; one thread per (n, c) with c fastest (coalesced).
__global__ void __launch_bounds__(256) nhwc_spatial_sum_kernel(const float* __restrict__ x, float* __restrict__ y, long long nc, int C, int HW, float scale) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= nc) return;
  long long n = i / C;
  int c = (int)(i % C);
  const float* p = x + n * HW * C + c;
  float s = 0.f;
  for (int k = 0; k < HW; ++k) s += p[(long long)k * C];
  y[i] = s * scale;
}

__global__ void __launch_bounds__(256) nhwc_spatial_bcast_kernel(const float* __restrict__ dy, float* __restrict__ dx, long long total, int C, int HW, float scale) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    int c = (int)(i % C);
    long long n = i / ((long long)C * HW);
    dx[i] = dy[n * C + c] * scale;
  }
}

struct RedDims {
  int nk, nr;
  long long kshape[6], kstride[6];  // kept dims: extent and input stride
  long long rshape[6], rstride[6];  // reduced dims
};

// One CTA per output element; threads stride over the reduced index space; fixed-order tree.
__global__ void __launch_bounds__(256) strided_sum_kernel(const float* __restrict__ x, float* __restrict__ y, RedDims d, long long rcount, float scale) {
  long long o = blockIdx.x;
  long long base = 0;
  for (int k = d.nk - 1; k >= 0; --k) {
    base += (o % d.kshape[k]) * d.kstride[k];
    o /= d.kshape[k];
  }
  float s = 0.f;
  for (long long t = threadIdx.x; t < rcount; t += 256) {
    long long r = t, off = base;
    for (int k = d.nr - 1; k >= 0; --k) {
      off += (r % d.rshape[k]) * d.rstride[k];
      r /= d.rshape[k];
    }
    s += x[off];
  }
  __shared__ float sm[256];
  sm[threadIdx.x] = s;
  __syncthreads();
  for (int w = 128; w > 0; w >>= 1) {
    if (threadIdx.x < w) sm[threadIdx.x] += sm[threadIdx.x + w];
    __syncthreads();
  }
  if (threadIdx.x == 0) y[blockIdx.x] = sm[0] * scale;
}

}  // namespace

MTB_API long long mtb_colsum_workspace_bytes(int c) { return (long long)mtb_col_max_partials() * c * 4 + 256; }

// out[c] = scale * sum_r a[r, c] for a row-major [rows, C] matrix (bias gradients; sums over
// N,H,W of a channels-last activation).
MTB_API int mtb_colsum_f32(const float* a, long long rows, int c, float scale, float* out, void* workspace, long long workspace_bytes,
                           void* stream) {
  MTB_REQUIRE(a && out && workspace && rows > 0 && c > 0, "colsum: bad arguments");
  MTB_REQUIRE(workspace_bytes >= mtb_colsum_workspace_bytes(c), "colsum: workspace too small");
  cudaStream_t st = (cudaStream_t)stream;
  ColCfg cfg = mtb_col_cfg(rows, c, mtb_aligned16(a));
  dim3 grid(cfg.col_blocks, cfg.row_blocks);
  float* partial = (float*)workspace;
  if (cfg.vec == 4) colsum_partial_kernel<4><<<grid, 256, 0, st>>>(a, rows, c, cfg.lanes, cfg.rows_per_block, partial);
  else colsum_partial_kernel<1><<<grid, 256, 0, st>>>(a, rows, c, cfg.lanes, cfg.rows_per_block, partial);
  MTB_LAUNCH_CHECK("colsum_partial_kernel");
  colsum_final_kernel<<<mtb_div_up(c, 32), 1024, 0, st>>>(partial, cfg.row_blocks, c, scale, out);
  MTB_LAUNCH_CHECK("colsum_final_kernel");
  return MTB_OK;
}

// Global pooling over H,W of a channels-last [N,H,W,C] tensor: y[N,C] = scale * sum_hw x.
MTB_API int mtb_nhwc_spatial_sum_f32(const float* x, float* y, int n, int c, int hw, float scale, void* stream) {
  MTB_REQUIRE(x && y && n > 0 && c > 0 && hw > 0, "nhwc_spatial_sum: bad arguments");
  long long nc = (long long)n * c;
  nhwc_spatial_sum_kernel<<<mtb_div_up(nc, 256), 256, 0, (cudaStream_t)stream>>>(x, y, nc, c, hw, scale);
  MTB_LAUNCH_CHECK("nhwc_spatial_sum_kernel");
  return MTB_OK;
}

// Backward of the above: dx[n,hw,c] = scale * dy[n,c].
MTB_API int mtb_nhwc_spatial_bcast_f32(const float* dy, float* dx, int n, int c, int hw, float scale, void* stream) {
  MTB_REQUIRE(dy && dx && n > 0 && c > 0 && hw > 0, "nhwc_spatial_bcast: bad arguments");
  long long total = (long long)n * c * hw;
  nhwc_spatial_bcast_kernel<<<mtb_stream_grid(total, 256), 256, 0, (cudaStream_t)stream>>>(dy, dx, total, c, hw, scale);
  MTB_LAUNCH_CHECK("nhwc_spatial_bcast_kernel");
  return MTB_OK;
}

// Generic sum over a set of logical dimensions. kept_* describe the output index space (extent,
// input stride in elements), red_* the reduced one. Output is dense in kept-dimension order.
MTB_API int mtb_sum_strided_f32(const float* x, float* y, int nkept, const long long* kept_shape, const long long* kept_strides, int nred,
                                const long long* red_shape, const long long* red_strides, float scale, void* stream) {
  MTB_REQUIRE(x && y && nkept >= 0 && nkept <= 6 && nred >= 0 && nred <= 6, "sum_strided: bad arguments");
  RedDims d;
  d.nk = nkept;
  d.nr = nred;
  long long outs = 1, rc = 1;
  for (int i = 0; i < nkept; ++i) { d.kshape[i] = kept_shape[i]; d.kstride[i] = kept_strides[i]; outs *= kept_shape[i]; }
  for (int i = 0; i < nred; ++i) { d.rshape[i] = red_shape[i]; d.rstride[i] = red_strides[i]; rc *= red_shape[i]; }
  MTB_REQUIRE(outs > 0 && outs < (1LL << 31), "sum_strided: output too large");
  strided_sum_kernel<<<(unsigned)outs, 256, 0, (cudaStream_t)stream>>>(x, y, d, rc, scale);
  MTB_LAUNCH_CHECK("strided_sum_kernel");
  return MTB_OK;
}

// ------------------------------------------------------------------ allocation-free variant
//
// Some callers cannot hand this library a scratch buffer and may not allocate one either: an
// embedding runtime that gave all device memory to its own arena at start-up, or a step loop
// in which any driver allocation is forbidden because it would synchronise the device.  For
// them the column sum is also offered with its scratch inside the library image: a file-scope
// device array of fixed size that every GPU loading the library carries until the process ends.
namespace {

constexpr int kNoAllocMaxChannels = 1024;
constexpr int kNoAllocMaxPartials = 256;
constexpr int kNoAllocMaxDevices = 64;
// 256 partial rows x 1024 channels x 4 bytes = 1 MiB per GPU.
static __device__ __align__(256) float g_colsum_scratch[kNoAllocMaxPartials * kNoAllocMaxChannels];

// In host code the name of a __device__ array is only a host-side stand-in; the device address
// has to be asked for, once per device, with that device current.
float* noalloc_scratch_for_current_device(int* status) {
  // one slot per device ordinal; host threads racing on a first call store the same address
  static float* cached[kNoAllocMaxDevices] = {nullptr};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) {
    *status = mtb_fail(MTB_ERR_CUDA, "colsum_noalloc: cudaGetDevice failed: %s", cudaGetErrorString(e));
    return nullptr;
  }
  if (dev < 0 || dev >= kNoAllocMaxDevices) {
    *status = mtb_fail(MTB_ERR_UNSUPPORTED, "colsum_noalloc: device ordinal %d is outside the %d ordinals this entry point keeps an address for",
                       dev, kNoAllocMaxDevices);
    return nullptr;
  }
  float* ptr = __atomic_load_n(&cached[dev], __ATOMIC_ACQUIRE);
  if (!ptr) {
    e = cudaGetSymbolAddress((void**)&ptr, g_colsum_scratch);
    if (e != cudaSuccess || !ptr) {
      *status = mtb_fail(MTB_ERR_CUDA, "colsum_noalloc: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
      return nullptr;
    }
    __atomic_store_n(&cached[dev], ptr, __ATOMIC_RELEASE);
  }
  *status = MTB_OK;
  return ptr;
}

}  // namespace

// out[c] = scale * sum_r a[r, c], like mtb_colsum_f32, but with no workspace argument and no
// allocation of any kind: the per-CTA partial sums go to a 1 MiB array that is part of the
// library.  Limits: c <= 1024 (more is rejected with MTB_ERR_UNSUPPORTED); at most 256 partial
// rows are used, so very tall matrices run with fewer CTAs than mtb_colsum_f32 would use.
// The first call on a device looks up the array's device address (cudaGetSymbolAddress), and with
// lazy module loading that lookup is also the moment the driver loads this module and backs the
// array: make one warm-up call per device before the region in which nothing may allocate and
// before any stream capture begins.  All calls on a device share the one array
// (it keeps the previous call's partials, every element that is read is rewritten first), so two
// calls that may overlap on the GPU - different streams, no dependency - race with each other.
MTB_API int mtb_colsum_noalloc_f32(const float* a, long long rows, int c, float scale, float* out, void* stream) {
  MTB_REQUIRE(a && out && rows > 0 && c > 0, "colsum_noalloc: bad arguments");
  if (c > kNoAllocMaxChannels)
    return mtb_fail(MTB_ERR_UNSUPPORTED, "colsum_noalloc: %d channels exceed the built-in scratch (max %d); use mtb_colsum_f32 with a workspace",
                    c, kNoAllocMaxChannels);
  int status = MTB_OK;
  float* partial = noalloc_scratch_for_current_device(&status);
  if (!partial) return status;
  cudaStream_t st = (cudaStream_t)stream;
  ColCfg cfg = mtb_col_cfg(rows, c, mtb_aligned16(a), kNoAllocMaxPartials);
  if (cfg.row_blocks > kNoAllocMaxPartials) return mtb_fail(MTB_ERR_UNSUPPORTED, "colsum_noalloc: internal partition exceeds the scratch");
  dim3 grid(cfg.col_blocks, cfg.row_blocks);
  if (cfg.vec == 4) colsum_partial_kernel<4><<<grid, 256, 0, st>>>(a, rows, c, cfg.lanes, cfg.rows_per_block, partial);
  else colsum_partial_kernel<1><<<grid, 256, 0, st>>>(a, rows, c, cfg.lanes, cfg.rows_per_block, partial);
  MTB_LAUNCH_CHECK("colsum_partial_kernel");
  colsum_final_kernel<<<mtb_div_up(c, 32), 1024, 0, st>>>(partial, cfg.row_blocks, c, scale, out);
  MTB_LAUNCH_CHECK("colsum_final_kernel");
  return MTB_OK;
}
