// Bandwidth kernels with no cross-element dependency: fill, copy, cast, ReLU, add, bias add,
// generic strided copy / broadcast binary ops, NCHW<->NHWC layout changes.
// All are grid-stride loops over float4 where alignment allows; grids are capped at a
// multiple of the SM count.
#include "common.cuh"

namespace {

constexpr int kThreads = 256;

template <class F>
__global__ void __launch_bounds__(kThreads) map1_kernel(float* out, const float* a, long long n4, long long n, F f) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long v = i; v < n4; v += stride) {
    float4 x = ld4(a + 4 * v);
    float4 r = make_float4(f(x.x), f(x.y), f(x.z), f(x.w));
    st4(out + 4 * v, r);
  }
  for (long long t = 4 * n4 + i; t < n; t += stride) out[t] = f(a[t]);
}

template <class F>
__global__ void __launch_bounds__(kThreads) map2_kernel(float* out, const float* a, const float* b,
                                                         long long n4, long long n, F f) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long v = i; v < n4; v += stride) {
    float4 x = ld4(a + 4 * v), y = ld4(b + 4 * v);
    st4(out + 4 * v, make_float4(f(x.x, y.x), f(x.y, y.y), f(x.z, y.z), f(x.w, y.w)));
  }
  for (long long t = 4 * n4 + i; t < n; t += stride) out[t] = f(a[t], b[t]);
}

struct ReluF { __device__ float operator()(float x) const { return fmaxf(x, 0.f); } };
// Gradient is blocked only for x < 0 (the CPU reference passes it at x == 0).
struct ReluBwdF { __device__ float operator()(float dy, float x) const { return x < 0.f ? 0.f : dy; } };
struct AxpyF { float alpha; __device__ float operator()(float x, float y) const { return x + y * alpha; } };
struct AddReluF { __device__ float operator()(float x, float y) const { return fmaxf(x + y, 0.f); } };
struct MulF { __device__ float operator()(float x, float y) const { return x * y; } };
struct ScaleF { float s; __device__ float operator()(float x) const { return x * s; } };
struct CopyF { __device__ float operator()(float x) const { return x; } };

// g = (x + y < 0) ? 0 : dy — backward of max(0, x + y); the sum is recomputed from the two
// forward inputs (bit-identical to the forward's), and a sum of exactly 0 passes the gradient.
__global__ void __launch_bounds__(kThreads) add_relu_bwd_kernel(float* g, const float* dy, const float* x, const float* y, long long n4, long long n) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long v = i; v < n4; v += stride) {
    float4 d = ld4(dy + 4 * v), a = ld4(x + 4 * v), b = ld4(y + 4 * v);
    d.x = (a.x + b.x < 0.f) ? 0.f : d.x;
    d.y = (a.y + b.y < 0.f) ? 0.f : d.y;
    d.z = (a.z + b.z < 0.f) ? 0.f : d.z;
    d.w = (a.w + b.w < 0.f) ? 0.f : d.w;
    st4(g + 4 * v, d);
  }
  for (long long t = 4 * n4 + i; t < n; t += stride) g[t] = (x[t] + y[t] < 0.f) ? 0.f : dy[t];
}

template <class F>
int launch_map1(float* out, const float* a, long long n, F f, cudaStream_t s, const char* name) {
  if (n == 0) return MTB_OK;
  bool vec = mtb_aligned16(out) && mtb_aligned16(a);
  long long n4 = vec ? n / 4 : 0;
  int grid = mtb_stream_grid(vec ? (n4 > 0 ? n4 : 1) : n, kThreads);
  map1_kernel<<<grid, kThreads, 0, s>>>(out, a, n4, n, f);
  MTB_LAUNCH_CHECK(name);
  return MTB_OK;
}

template <class F>
int launch_map2(float* out, const float* a, const float* b, long long n, F f, cudaStream_t s, const char* name) {
  if (n == 0) return MTB_OK;
  bool vec = mtb_aligned16(out) && mtb_aligned16(a) && mtb_aligned16(b);
  long long n4 = vec ? n / 4 : 0;
  int grid = mtb_stream_grid(vec ? (n4 > 0 ? n4 : 1) : n, kThreads);
  map2_kernel<<<grid, kThreads, 0, s>>>(out, a, b, n4, n, f);
  MTB_LAUNCH_CHECK(name);
  return MTB_OK;
}

// y[r, c] = x[r, c] + alpha * bias[c]; cols % 4 == 0 fast path.
__global__ void __launch_bounds__(kThreads) bias_rows_kernel(float* __restrict__ y, const float* __restrict__ x, const float* __restrict__ bias,
                                                              long long n, int cols, float alpha) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = i; t < n; t += stride) y[t] = x[t] + alpha * bias[t % cols];
}

__global__ void __launch_bounds__(kThreads) fill_kernel(float* out, long long n4, long long n, float v) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long stride = (long long)gridDim.x * blockDim.x;
  float4 v4 = make_float4(v, v, v, v);
  for (long long k = i; k < n4; k += stride) st4(out + 4 * k, v4);
  for (long long t = 4 * n4 + i; t < n; t += stride) out[t] = v;
}

struct Strides6 {
  int ndim;
  long long shape[6];
  long long a[6];
  long long b[6];
  long long o[6];
};

template <int OP>
__global__ void __launch_bounds__(kThreads) strided_binary_kernel(float* __restrict__ out, const float* __restrict__ a, const float* __restrict__ b,
                                                                   long long n, Strides6 s, float alpha) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (long long t = i; t < n; t += stride) {
    long long r = t, oa = 0, ob = 0, oo = 0;
    for (int d = s.ndim - 1; d >= 0; --d) {
      long long c = r % s.shape[d];
      r /= s.shape[d];
      oa += c * s.a[d];
      ob += c * s.b[d];
      oo += c * s.o[d];
    }
    float x = a[oa];
    float y = (OP == 5) ? 0.f : b[ob];
    float v;
    if (OP == 0) v = x + alpha * y;
    else if (OP == 1) v = x - alpha * y;
    else if (OP == 2) v = x * y;
    else if (OP == 3) v = x / y;
    else if (OP == 4) v = powf(x, y);
    else if (OP == 6) v = y * powf(x, y - 1.f);   // d(x^y)/dx
    else if (OP == 7) v = powf(x, y) * logf(x);   // d(x^y)/dy
    else v = x * alpha;  // OP == 5: strided copy (alpha 1) / scaled broadcast
    out[oo] = v;
  }
}

// NCHW -> NHWC through a shared-memory tile transpose of the [C, HW] plane of each image.
__global__ void __launch_bounds__(256) transpose_planes_kernel(float* __restrict__ dst, const float* __restrict__ src, int rows, int cols) {
  // src: [batch][rows][cols] -> dst: [batch][cols][rows]
  __shared__ float tile[32][33];
  const float* s = src + (long long)blockIdx.z * rows * cols;
  float* d = dst + (long long)blockIdx.z * rows * cols;
  int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  for (int j = threadIdx.y; j < 32; j += 8) {
    int r = r0 + j, c = c0 + threadIdx.x;
    if (r < rows && c < cols) tile[j][threadIdx.x] = s[(long long)r * cols + c];
  }
  __syncthreads();
  for (int j = threadIdx.y; j < 32; j += 8) {
    int c = c0 + j, r = r0 + threadIdx.x;
    if (r < rows && c < cols) d[(long long)c * rows + r] = tile[threadIdx.x][j];
  }
}

__global__ void cast_i32_i64_kernel(long long* out, const int* in, long long n) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) out[i] = in[i];
}
__global__ void cast_i64_f32_kernel(float* out, const long long* in, long long n) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) out[i] = (float)in[i];
}
__global__ void cast_f32_i64_kernel(long long* out, const float* in, long long n) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) out[i] = (long long)in[i];
}

__global__ void cast_i8_f32_kernel(float* out, const signed char* in, long long n) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) out[i] = (float)in[i];
}

int transpose_planes(float* dst, const float* src, int batch, int rows, int cols, cudaStream_t s) {
  if ((long long)batch * rows * cols == 0) return MTB_OK;
  MTB_REQUIRE(batch <= 65535 * 1, "layout change: batch %d exceeds grid.z", batch);
  dim3 grid(mtb_div_up(cols, 32), mtb_div_up(rows, 32), batch), block(32, 8);
  MTB_REQUIRE(grid.y <= 65535, "layout change: too many rows");
  transpose_planes_kernel<<<grid, block, 0, s>>>(dst, src, rows, cols);
  MTB_LAUNCH_CHECK("transpose_planes_kernel");
  return MTB_OK;
}

// dst[r][c] = c < c_src ? src[r][c] : 0 for c < c_dst: widen a [rows, c_src] matrix with zero
// columns (c_dst > c_src) or keep its first c_dst columns (c_dst < c_src), in one pass.
__global__ void __launch_bounds__(256) resize_channels_kernel(const float* __restrict__ src, float* __restrict__ dst, long long rows, int c_src, int c_dst) {
  const long long total = rows * c_dst;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / c_dst;
    const int c = (int)(i - r * c_dst);
    dst[i] = c < c_src ? src[r * c_src + c] : 0.f;
  }
}

}  // namespace

// Copy a row-major [rows, c_src] matrix into [rows, c_dst]: extra columns are zero, surplus columns are
// dropped.  Pads the 1- or 3-channel image stem (and its filter) to one 32-channel block for the
// tensor-core convolution and cuts the weight gradient back; no counterpart in the reference.
MTB_API int mtb_resize_channels_f32(const float* src, float* dst, long long rows, int c_src, int c_dst, void* stream) {
  MTB_REQUIRE(src && dst && rows > 0 && c_src > 0 && c_dst > 0, "resize_channels: bad arguments");
  resize_channels_kernel<<<mtb_stream_grid(rows * c_dst, kThreads), kThreads, 0, (cudaStream_t)stream>>>(src, dst, rows, c_src, c_dst);
  MTB_LAUNCH_CHECK("resize_channels_kernel");
  return MTB_OK;
}

MTB_API int mtb_fill_f32(float* x, long long n, float value, void* stream) {
  MTB_REQUIRE(n >= 0 && (x || n == 0), "fill: bad arguments");
  if (n == 0) return MTB_OK;
  long long n4 = mtb_aligned16(x) ? n / 4 : 0;
  fill_kernel<<<mtb_stream_grid(n4 > 0 ? n4 : n, kThreads), kThreads, 0, (cudaStream_t)stream>>>(x, n4, n, value);
  MTB_LAUNCH_CHECK("fill_kernel");
  return MTB_OK;
}

MTB_API int mtb_copy_f32(float* dst, const float* src, long long n, void* stream) {
  MTB_REQUIRE(n >= 0 && ((dst && src) || n == 0), "copy: bad arguments");
  return launch_map1(dst, src, n, CopyF{}, (cudaStream_t)stream, "copy");
}

MTB_API int mtb_scale_f32(float* dst, const float* src, long long n, float scale, void* stream) {
  MTB_REQUIRE(n >= 0 && ((dst && src) || n == 0), "scale: bad arguments");
  return launch_map1(dst, src, n, ScaleF{scale}, (cudaStream_t)stream, "scale");
}

MTB_API int mtb_relu_forward_f32(const float* x, float* y, long long n, void* stream) {
  MTB_REQUIRE(n >= 0 && ((x && y) || n == 0), "relu: bad arguments");
  return launch_map1(y, x, n, ReluF{}, (cudaStream_t)stream, "relu_forward");
}

MTB_API int mtb_relu_backward_f32(const float* dy, const float* x, float* dx, long long n, void* stream) {
  MTB_REQUIRE(n >= 0 && ((x && dy && dx) || n == 0), "relu_backward: bad arguments");
  return launch_map2(dx, dy, x, n, ReluBwdF{}, (cudaStream_t)stream, "relu_backward");
}

// z = x + alpha * y, same number of elements and same physical layout. z may alias x.
MTB_API int mtb_add_f32(const float* x, const float* y, float* z, long long n, float alpha, void* stream) {
  MTB_REQUIRE(n >= 0 && ((x && y && z) || n == 0), "add: bad arguments");
  return launch_map2(z, x, y, n, AxpyF{alpha}, (cudaStream_t)stream, "add");
}

// z = max(0, x + y): residual add and ReLU in one pass.
MTB_API int mtb_add_relu_f32(const float* x, const float* y, float* z, long long n, void* stream) {
  MTB_REQUIRE(n >= 0 && ((x && y && z) || n == 0), "add_relu: bad arguments");
  return launch_map2(z, x, y, n, AddReluF{}, (cudaStream_t)stream, "add_relu");
}

// g = (x + y < 0) ? 0 : dy: the gradient of max(0, x + y) with respect to x and to y.
MTB_API int mtb_add_relu_backward_f32(const float* dy, const float* x, const float* y, float* g, long long n, void* stream) {
  MTB_REQUIRE(n >= 0 && ((dy && x && y && g) || n == 0), "add_relu_backward: bad arguments");
  if (n == 0) return MTB_OK;
  bool vec = mtb_aligned16(dy) && mtb_aligned16(x) && mtb_aligned16(y) && mtb_aligned16(g);
  long long n4 = vec ? n / 4 : 0;
  add_relu_bwd_kernel<<<mtb_stream_grid(vec ? (n4 > 0 ? n4 : 1) : n, kThreads), kThreads, 0, (cudaStream_t)stream>>>(g, dy, x, y, n4, n);
  MTB_LAUNCH_CHECK("add_relu_bwd_kernel");
  return MTB_OK;
}

MTB_API int mtb_mul_f32(const float* x, const float* y, float* z, long long n, void* stream) {
  MTB_REQUIRE(n >= 0 && ((x && y && z) || n == 0), "mul: bad arguments");
  return launch_map2(z, x, y, n, MulF{}, (cudaStream_t)stream, "mul");
}

// y[r, :] = x[r, :] + alpha * bias[:] for a row-major [rows, cols] matrix.
MTB_API int mtb_add_bias_rows_f32(const float* x, const float* bias, float* y, long long rows, int cols, float alpha, void* stream) {
  MTB_REQUIRE(rows >= 0 && cols > 0 && x && bias && y, "add_bias_rows: bad arguments");
  long long n = rows * cols;
  if (n == 0) return MTB_OK;
  bias_rows_kernel<<<mtb_stream_grid(n, kThreads), kThreads, 0, (cudaStream_t)stream>>>(y, x, bias, n, cols, alpha);
  MTB_LAUNCH_CHECK("bias_rows_kernel");
  return MTB_OK;
}

// Generic broadcast binary op over up to 6 logical dimensions. Strides are in elements; a stride
// of 0 broadcasts. op: 0 add (x + alpha*y), 1 sub (x - alpha*y), 2 mul, 3 div, 4 pow, 5 alpha*x (y unused),
// 6 y*x^(y-1) and 7 x^y*ln(x) (the two partial derivatives of pow).
MTB_API int mtb_binary_strided_f32(int op, int ndim, const long long* shape, const long long* x_strides, const long long* y_strides,
                                   const long long* z_strides, const float* x, const float* y, float* z, float alpha, void* stream) {
  MTB_REQUIRE(ndim >= 0 && ndim <= 6 && op >= 0 && op <= 7 && x && z && (y || op == 5), "binary_strided: bad arguments");
  Strides6 s;
  s.ndim = ndim;
  long long n = 1;
  for (int d = 0; d < ndim; ++d) {
    s.shape[d] = shape[d];
    s.a[d] = x_strides[d];
    s.b[d] = (op == 5) ? 0 : y_strides[d];
    s.o[d] = z_strides[d];
    n *= shape[d];
  }
  if (n == 0) return MTB_OK;
  int grid = mtb_stream_grid(n, kThreads);
  cudaStream_t st = (cudaStream_t)stream;
  switch (op) {
    case 0: strided_binary_kernel<0><<<grid, kThreads, 0, st>>>(z, x, y, n, s, alpha); break;
    case 1: strided_binary_kernel<1><<<grid, kThreads, 0, st>>>(z, x, y, n, s, alpha); break;
    case 2: strided_binary_kernel<2><<<grid, kThreads, 0, st>>>(z, x, y, n, s, alpha); break;
    case 3: strided_binary_kernel<3><<<grid, kThreads, 0, st>>>(z, x, y, n, s, alpha); break;
    case 4: strided_binary_kernel<4><<<grid, kThreads, 0, st>>>(z, x, y, n, s, alpha); break;
    case 6: strided_binary_kernel<6><<<grid, kThreads, 0, st>>>(z, x, y, n, s, alpha); break;
    case 7: strided_binary_kernel<7><<<grid, kThreads, 0, st>>>(z, x, y, n, s, alpha); break;
    default: strided_binary_kernel<5><<<grid, kThreads, 0, st>>>(z, x, y, n, s, alpha); break;
  }
  MTB_LAUNCH_CHECK("strided_binary_kernel");
  return MTB_OK;
}

// Logical NCHW buffer -> channels-last (NHWC) buffer and back.
MTB_API int mtb_nchw_to_nhwc_f32(const float* src, float* dst, int n, int c, int h, int w, void* stream) {
  MTB_REQUIRE(src && dst && n >= 0 && c > 0 && h > 0 && w > 0, "nchw_to_nhwc: bad arguments");
  return transpose_planes(dst, src, n, c, h * w, (cudaStream_t)stream);
}

MTB_API int mtb_nhwc_to_nchw_f32(const float* src, float* dst, int n, int c, int h, int w, void* stream) {
  MTB_REQUIRE(src && dst && n >= 0 && c > 0 && h > 0 && w > 0, "nhwc_to_nchw: bad arguments");
  return transpose_planes(dst, src, n, h * w, c, (cudaStream_t)stream);
}

// kind: 0 int32->int64, 1 int64->float32, 2 float32->int64.
MTB_API int mtb_cast(int kind, const void* src, void* dst, long long n, void* stream) {
  MTB_REQUIRE(n >= 0 && ((src && dst) || n == 0), "cast: bad arguments");
  if (n == 0) return MTB_OK;
  int grid = mtb_stream_grid(n, kThreads);
  cudaStream_t st = (cudaStream_t)stream;
  if (kind == 0) cast_i32_i64_kernel<<<grid, kThreads, 0, st>>>((long long*)dst, (const int*)src, n);
  else if (kind == 1) cast_i64_f32_kernel<<<grid, kThreads, 0, st>>>((float*)dst, (const long long*)src, n);
  else if (kind == 2) cast_f32_i64_kernel<<<grid, kThreads, 0, st>>>((long long*)dst, (const float*)src, n);
  else if (kind == 3) cast_i8_f32_kernel<<<grid, kThreads, 0, st>>>((float*)dst, (const signed char*)src, n);
  else return mtb_fail(MTB_ERR_UNSUPPORTED, "cast kind %d", kind);
  MTB_LAUNCH_CHECK("cast kernel");
  return MTB_OK;
}
