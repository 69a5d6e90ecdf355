// Operators outside the training step's hot path that the reference's API offers on the GPU: max with
// indices along one dimension (or over everything) and its backward, and element-wise equality.
// Tensors are addressed through logical-dimension strides, so channels-last activations need no copy.
#include "common.cuh"

namespace {

struct MaxDims {
  int nk;
  long long kshape[6], kstride[6];
};

// One CTA per output element.  Ties go to the lowest index (numpy.argmax).
__global__ void __launch_bounds__(256) max_strided_kernel(const float* __restrict__ x, float* __restrict__ y, long long* __restrict__ idx, MaxDims d,
                                                          long long red_len, long long red_stride) {
  long long o = blockIdx.x, base = 0;
  for (int k = d.nk - 1; k >= 0; --k) {
    base += (o % d.kshape[k]) * d.kstride[k];
    o /= d.kshape[k];
  }
  float best = -INFINITY;
  long long at = red_len;  // "nothing yet": any real index is lower
  for (long long t = threadIdx.x; t < red_len; t += 256) {
    const float v = x[base + t * red_stride];
    if (v > best || at == red_len) { best = v; at = t; }
  }
  __shared__ float sv[256];
  __shared__ long long si[256];
  sv[threadIdx.x] = best;
  si[threadIdx.x] = at;
  __syncthreads();
  for (int w = 128; w > 0; w >>= 1) {
    if (threadIdx.x < w) {
      const float v = sv[threadIdx.x + w];
      const long long i = si[threadIdx.x + w];
      if (i < red_len && (si[threadIdx.x] == red_len || v > sv[threadIdx.x] || (v == sv[threadIdx.x] && i < si[threadIdx.x]))) {
        sv[threadIdx.x] = v;
        si[threadIdx.x] = i;
      }
    }
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    y[blockIdx.x] = sv[0];
    idx[blockIdx.x] = si[0];
  }
}

// dx (zero-filled beforehand) receives dy at the recorded index of every output element.
__global__ void max_scatter_kernel(const float* __restrict__ dy, const long long* __restrict__ idx, float* __restrict__ dx, MaxDims d, long long outs,
                                   long long red_stride) {
  for (long long o = blockIdx.x * (long long)blockDim.x + threadIdx.x; o < outs; o += (long long)gridDim.x * blockDim.x) {
    long long r = o, base = 0;
    for (int k = d.nk - 1; k >= 0; --k) {
      base += (r % d.kshape[k]) * d.kstride[k];
      r /= d.kshape[k];
    }
    dx[base + idx[o] * red_stride] = dy[o];
  }
}

struct EqDims {
  int nd;
  long long shape[6], a[6], b[6];
};

template <class T>
__global__ void eq_strided_kernel(const T* __restrict__ x, const T* __restrict__ y, signed char* __restrict__ out, EqDims d, long long n) {
  for (long long t = blockIdx.x * (long long)blockDim.x + threadIdx.x; t < n; t += (long long)gridDim.x * blockDim.x) {
    long long r = t, oa = 0, ob = 0;
    for (int k = d.nd - 1; k >= 0; --k) {
      const long long c = r % d.shape[k];
      r /= d.shape[k];
      oa += c * d.a[k];
      ob += c * d.b[k];
    }
    out[t] = x[oa] == y[ob] ? 1 : 0;
  }
}

int fill_dims(MaxDims& d, int nkept, const long long* shape, const long long* strides, long long* outs) {
  MTB_REQUIRE(nkept >= 0 && nkept <= 6, "max: at most 6 kept dimensions");
  d.nk = nkept;
  *outs = 1;
  for (int i = 0; i < nkept; ++i) { d.kshape[i] = shape[i]; d.kstride[i] = strides[i]; *outs *= shape[i]; }
  MTB_REQUIRE(*outs > 0 && *outs < (1LL << 31), "max: output size out of range");
  return MTB_OK;
}

}  // namespace

// y[kept...] = max over one strided dimension of x, idx = position of the first maximum along it (int64).
// kept_shape / kept_strides (HOST arrays, strides in elements) describe the output index space inside x.
MTB_API int mtb_max_strided_f32(const float* x, float* y, long long* idx, int nkept, const long long* kept_shape, const long long* kept_strides,
                                long long red_len, long long red_stride, void* stream) {
  MTB_REQUIRE(x && y && idx && red_len > 0, "max: bad arguments");
  MaxDims d;
  long long outs;
  if (int rc = fill_dims(d, nkept, kept_shape, kept_strides, &outs)) return rc;
  max_strided_kernel<<<(unsigned)outs, 256, 0, (cudaStream_t)stream>>>(x, y, idx, d, red_len, red_stride);
  MTB_LAUNCH_CHECK("max_strided_kernel");
  return MTB_OK;
}

// dx[...] = dy where the maximum was taken, 0 elsewhere; dx holds dx_elems floats and is addressed with the
// same kept strides / reduced stride as x was.
MTB_API int mtb_max_backward_f32(const float* dy, const long long* idx, float* dx, long long dx_elems, int nkept, const long long* kept_shape,
                                 const long long* kept_strides, long long red_stride, void* stream) {
  MTB_REQUIRE(dy && idx && dx && dx_elems > 0, "max_backward: bad arguments");
  MaxDims d;
  long long outs;
  if (int rc = fill_dims(d, nkept, kept_shape, kept_strides, &outs)) return rc;
  cudaStream_t st = (cudaStream_t)stream;
  MTB_CUDA(cudaMemsetAsync(dx, 0, (size_t)dx_elems * 4, st));
  max_scatter_kernel<<<mtb_stream_grid(outs, 256), 256, 0, st>>>(dy, idx, dx, d, outs, red_stride);
  MTB_LAUNCH_CHECK("max_scatter_kernel");
  return MTB_OK;
}

// out[i] = (x[i] == y[i]) as int8, dense in logical order; kind 0: float32, 1: int64.
MTB_API int mtb_eq_strided(int kind, int ndim, const long long* shape, const long long* x_strides, const long long* y_strides, const void* x,
                           const void* y, signed char* out, void* stream) {
  MTB_REQUIRE(x && y && out && ndim >= 0 && ndim <= 6 && (kind == 0 || kind == 1), "eq: bad arguments");
  EqDims d;
  d.nd = ndim;
  long long n = 1;
  for (int i = 0; i < ndim; ++i) { d.shape[i] = shape[i]; d.a[i] = x_strides[i]; d.b[i] = y_strides[i]; n *= shape[i]; }
  if (n == 0) return MTB_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (kind == 0) eq_strided_kernel<float><<<mtb_stream_grid(n, 256), 256, 0, st>>>((const float*)x, (const float*)y, out, d, n);
  else eq_strided_kernel<long long><<<mtb_stream_grid(n, 256), 256, 0, st>>>((const long long*)x, (const long long*)y, out, d, n);
  MTB_LAUNCH_CHECK("eq_strided_kernel");
  return MTB_OK;
}
