// MaxPool2d over channels-last activations.  Forward writes the window maximum and, per output
// element, a 16-bit tie mask: bit kh*KW+kw is set where that window element equals the
// maximum (padding cells take part with value 0, as in the reference).  The lowest set bit is
// the argmax (first maximum in row-major window order); the whole mask lets backward send the
// gradient to every tied element without re-reading the input.  Backward is a gather over the
// windows that cover each input element: no atomics, deterministic.
#include "colreduce.cuh"
#include <cstdlib>

namespace {

struct PoolDims {
  int N, C, H, W, KH, KW, SH, SW, PH, PW, OH, OW;
};

// IdxT = unsigned when the element count fits 32 bits (cheap div/mod), long long otherwise.
template <int V, typename IdxT>
__global__ void __launch_bounds__(256) maxpool_fwd_kernel(const float* __restrict__ x, float* __restrict__ y, unsigned short* __restrict__ mask,
                                                           PoolDims d, long long total_ll) {
  const IdxT cv = (IdxT)(d.C / V), total = (IdxT)total_ll;
  IdxT i = (IdxT)blockIdx.x * blockDim.x + threadIdx.x;
  const IdxT stride = (IdxT)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    int cg = (int)(i % cv);
    IdxT t = i / cv;
    int ow = (int)(t % (IdxT)d.OW); t /= (IdxT)d.OW;
    int oh = (int)(t % (IdxT)d.OH);
    int n = (int)(t / (IdxT)d.OH);
    float best[V];
    unsigned m[V];
#pragma unroll
    for (int k = 0; k < V; ++k) { best[k] = -3.402823466e38f; m[k] = 0u; }
    for (int kh = 0; kh < d.KH; ++kh) {
      int ih = oh * d.SH - d.PH + kh;
      for (int kw = 0; kw < d.KW; ++kw) {
        int iw = ow * d.SW - d.PW + kw;
        VecF<V> f;
        if (ih >= 0 && ih < d.H && iw >= 0 && iw < d.W) {
          f = vload<V>(x + (((long long)n * d.H + ih) * d.W + iw) * d.C + (long long)cg * V);
        } else {
#pragma unroll
          for (int k = 0; k < V; ++k) f.v[k] = 0.f;
        }
        unsigned bit = 1u << ((kh * d.KW + kw) & 15);
#pragma unroll
        for (int k = 0; k < V; ++k) {
          if (f.v[k] > best[k]) { best[k] = f.v[k]; m[k] = bit; }
          else if (f.v[k] == best[k]) m[k] |= bit;
        }
      }
    }
    long long o = (long long)i * V;
    VecF<V> r;
#pragma unroll
    for (int k = 0; k < V; ++k) r.v[k] = best[k];
    vstore<V>(y + o, r);
    if (mask) {
      if (V == 4) {
        *reinterpret_cast<uint2*>(mask + o) = make_uint2(m[0] | (m[1 % V] << 16), m[2 % V] | (m[3 % V] << 16));
      } else {
#pragma unroll
        for (int k = 0; k < V; ++k) mask[o + k] = (unsigned short)m[k];
      }
    }
  }
}

// 2x2 windows with stride 2 that tile the input exactly (no padding, even extents), 4 channels per
// thread: the four loads of a window are issued back to back with nothing between them but address
// arithmetic (no bounds tests, 32-bit indices), and every thread works on two windows at once, so eight
// 16-byte loads are in flight per thread.  Same results as the general kernel above.
__device__ __forceinline__ void pool2x2_one(float a, float b, float c, float e, float& best, unsigned& m) {
  best = fmaxf(fmaxf(a, b), fmaxf(c, e));
  m = (a == best ? 1u : 0u) | (b == best ? 2u : 0u) | (c == best ? 4u : 0u) | (e == best ? 8u : 0u);
}

__global__ void __launch_bounds__(256) maxpool2x2_fwd_kernel(const float4* __restrict__ x, float4* __restrict__ y, uint2* __restrict__ mask,
                                                              unsigned C4, unsigned OW, unsigned OH, unsigned total) {
  const unsigned W_C4 = 2u * OW * C4;  // one input row, in float4 units
  const unsigned stride = gridDim.x * blockDim.x;
  for (unsigned i0 = blockIdx.x * blockDim.x + threadIdx.x; i0 < total; i0 += 2u * stride) {
    unsigned idx[2] = {i0, i0 + stride};
    float4 v[2][4];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (idx[u] < total) {
        const unsigned cg = idx[u] % C4;
        unsigned t = idx[u] / C4;
        const unsigned ow = t % OW;
        t /= OW;  // t = n * OH + oh; the input row is 2 t
        const unsigned base = (2u * t) * W_C4 + 2u * ow * C4 + cg;
        v[u][0] = x[base];
        v[u][1] = x[base + C4];
        v[u][2] = x[base + W_C4];
        v[u][3] = x[base + W_C4 + C4];
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (idx[u] < total) {
        float4 r;
        unsigned m0, m1, m2, m3;
        pool2x2_one(v[u][0].x, v[u][1].x, v[u][2].x, v[u][3].x, r.x, m0);
        pool2x2_one(v[u][0].y, v[u][1].y, v[u][2].y, v[u][3].y, r.y, m1);
        pool2x2_one(v[u][0].z, v[u][1].z, v[u][2].z, v[u][3].z, r.z, m2);
        pool2x2_one(v[u][0].w, v[u][1].w, v[u][2].w, v[u][3].w, r.w, m3);
        y[idx[u]] = r;
        if (mask) mask[idx[u]] = make_uint2(m0 | (m1 << 16), m2 | (m3 << 16));
      }
    }
  }
}

// MODE 0: tie mask from forward; MODE 1: recompute x == out (any window size).
template <int V, int MODE>
__global__ void __launch_bounds__(256) maxpool_bwd_kernel(const float* __restrict__ dy, const unsigned short* __restrict__ mask,
                                                           const float* __restrict__ out, const float* __restrict__ x, float* __restrict__ dx,
                                                           PoolDims d, long long total) {
  const int cv = d.C / V;
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    int cg = (int)(i % cv);
    long long t = i / cv;
    int w = (int)(t % d.W); t /= d.W;
    int h = (int)(t % d.H);
    int n = (int)(t / d.H);
    float acc[V];
#pragma unroll
    for (int k = 0; k < V; ++k) acc[k] = 0.f;
    VecF<V> xv;
    if (MODE == 1) xv = vload<V>(x + i * V);
    // windows oh with oh*SH - PH <= h <= oh*SH - PH + KH - 1
    int hp = h + d.PH, wp = w + d.PW;
    int oh0 = hp - d.KH + 1; oh0 = oh0 > 0 ? (oh0 + d.SH - 1) / d.SH : 0;
    int oh1 = hp / d.SH; if (oh1 > d.OH - 1) oh1 = d.OH - 1;
    int ow0 = wp - d.KW + 1; ow0 = ow0 > 0 ? (ow0 + d.SW - 1) / d.SW : 0;
    int ow1 = wp / d.SW; if (ow1 > d.OW - 1) ow1 = d.OW - 1;
    for (int oh = oh0; oh <= oh1; ++oh) {
      for (int ow = ow0; ow <= ow1; ++ow) {
        long long o = ((((long long)n * d.OH + oh) * d.OW + ow) * d.C) + (long long)cg * V;
        VecF<V> g = vload<V>(dy + o);
        if (MODE == 0) {
          unsigned bit = 1u << (((hp - oh * d.SH) * d.KW + (wp - ow * d.SW)) & 15);
#pragma unroll
          for (int k = 0; k < V; ++k) if (mask[o + k] & bit) acc[k] += g.v[k];
        } else {
          VecF<V> ov = vload<V>(out + o);
#pragma unroll
          for (int k = 0; k < V; ++k) if (xv.v[k] == ov.v[k]) acc[k] += g.v[k];
        }
      }
    }
    VecF<V> r;
#pragma unroll
    for (int k = 0; k < V; ++k) r.v[k] = acc[k];
    vstore<V>(dx + i * V, r);
  }
}

// Non-overlapping windows that tile the input exactly (kernel == stride, no padding, extents
// divisible): one thread per output window and 4 channels reads dy and the tie mask once and
// writes the KH*KW input gradients of its window, so nothing is read twice.
__global__ void __launch_bounds__(256) maxpool_bwd_window_kernel(const float* __restrict__ dy, const unsigned short* __restrict__ mask,
                                                                  float* __restrict__ dx, PoolDims d, unsigned total) {
  const unsigned cv = d.C / 4;
  unsigned i = blockIdx.x * blockDim.x + threadIdx.x;
  const unsigned stride = gridDim.x * blockDim.x;
  for (; i < total; i += stride) {
    unsigned cg = i % cv, t = i / cv;
    unsigned ow = t % d.OW; t /= d.OW;
    unsigned oh = t % d.OH, n = t / d.OH;
    const long long o = (long long)i * 4;
    const float4 g = ld4(dy + o);
    const uint2 mm = *reinterpret_cast<const uint2*>(mask + o);
    const unsigned m0 = mm.x & 0xffffu, m1 = mm.x >> 16, m2 = mm.y & 0xffffu, m3 = mm.y >> 16;
    for (int kh = 0; kh < d.KH; ++kh) {
      float* row = dx + ((((long long)n * d.H + oh * d.KH + kh) * d.W + (long long)ow * d.KW) * d.C) + cg * 4;
      for (int kw = 0; kw < d.KW; ++kw) {
        const unsigned bit = 1u << (kh * d.KW + kw);
        st4(row + (long long)kw * d.C, make_float4((m0 & bit) ? g.x : 0.f, (m1 & bit) ? g.y : 0.f, (m2 & bit) ? g.z : 0.f, (m3 & bit) ? g.w : 0.f));
      }
    }
  }
}

__global__ void mask_to_argmax_kernel(const unsigned short* __restrict__ mask, unsigned char* __restrict__ argmax, long long n) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) argmax[i] = (unsigned char)(__ffs((int)mask[i]) - 1);
}

int pool_dims(PoolDims& d, int n, int c, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw) {
  MTB_REQUIRE(n > 0 && c > 0 && h > 0 && w > 0 && kh > 0 && kw > 0 && sh > 0 && sw > 0 && ph >= 0 && pw >= 0, "max_pool2d: bad shape");
  d = PoolDims{n, c, h, w, kh, kw, sh, sw, ph, pw, (2 * ph + h - kh) / sh + 1, (2 * pw + w - kw) / sw + 1};
  MTB_REQUIRE(d.OH > 0 && d.OW > 0, "max_pool2d: empty output");
  return MTB_OK;
}

}  // namespace

// x [N,H,W,C] -> y [N,OH,OW,C]; tiemask (uint16 per output element, may be NULL) requires
// KH*KW <= 16.
MTB_API int mtb_max_pool2d_forward_f32(int n, int c, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, const float* x, float* y,
                                       unsigned short* tiemask, void* stream) {
  PoolDims d;
  int rc = pool_dims(d, n, c, h, w, kh, kw, sh, sw, ph, pw);
  if (rc) return rc;
  MTB_REQUIRE(x && y, "max_pool2d_forward: null pointer");
  MTB_REQUIRE(!tiemask || kh * kw <= 16, "max_pool2d_forward: tie mask needs KH*KW <= 16");
  bool vec = c % 4 == 0 && mtb_aligned16(x) && mtb_aligned16(y) && (reinterpret_cast<uintptr_t>(tiemask) & 7u) == 0;
  long long total = (long long)n * d.OH * d.OW * (c / (vec ? 4 : 1));
  int grid = mtb_stream_grid(total, 256);
  cudaStream_t st = (cudaStream_t)stream;
  const bool small = total < (1LL << 31) - (1LL << 26);  // room for the grid-stride overshoot
  const bool tiles2x2 = kh == 2 && kw == 2 && sh == 2 && sw == 2 && ph == 0 && pw == 0 && h % 2 == 0 && w % 2 == 0;
  if (vec && tiles2x2 && (long long)n * h * w * (c / 4) < (1LL << 32) - (1LL << 27) && !getenv("MTB_POOL_GENERIC")) {
    const int g2 = mtb_stream_grid((total + 1) / 2, 256);
    maxpool2x2_fwd_kernel<<<g2, 256, 0, st>>>((const float4*)x, (float4*)y, (uint2*)tiemask, (unsigned)(c / 4), (unsigned)d.OW, (unsigned)d.OH,
                                              (unsigned)total);
    MTB_LAUNCH_CHECK("maxpool2x2_fwd_kernel");
    return MTB_OK;
  }
  if (vec && small) maxpool_fwd_kernel<4, unsigned><<<grid, 256, 0, st>>>(x, y, tiemask, d, total);
  else if (vec) maxpool_fwd_kernel<4, long long><<<grid, 256, 0, st>>>(x, y, tiemask, d, total);
  else if (small) maxpool_fwd_kernel<1, unsigned><<<grid, 256, 0, st>>>(x, y, tiemask, d, total);
  else maxpool_fwd_kernel<1, long long><<<grid, 256, 0, st>>>(x, y, tiemask, d, total);
  MTB_LAUNCH_CHECK("maxpool_fwd_kernel");
  return MTB_OK;
}

// dx[i] = sum over windows covering i of (i is a maximum of the window ? dy[window] : 0).
// Pass tiemask from forward, or (out, x) to recompute the equality (needed when KH*KW > 16).
MTB_API int mtb_max_pool2d_backward_f32(int n, int c, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, const float* dy,
                                        const unsigned short* tiemask, const float* out, const float* x, float* dx, void* stream) {
  PoolDims d;
  int rc = pool_dims(d, n, c, h, w, kh, kw, sh, sw, ph, pw);
  if (rc) return rc;
  MTB_REQUIRE(dy && dx && (tiemask || (out && x)), "max_pool2d_backward: need a tie mask or (out, x)");
  MTB_REQUIRE(!tiemask || kh * kw <= 16, "max_pool2d_backward: tie mask needs KH*KW <= 16");
  bool vec = c % 4 == 0 && mtb_aligned16(dy) && mtb_aligned16(dx) && (tiemask || (mtb_aligned16(out) && mtb_aligned16(x)));
  long long total = (long long)n * h * w * (c / (vec ? 4 : 1));
  int grid = mtb_stream_grid(total, 256);
  cudaStream_t st = (cudaStream_t)stream;
  const bool tiles_exactly = kh == sh && kw == sw && ph == 0 && pw == 0 && h % kh == 0 && w % kw == 0;
  if (tiemask && vec && tiles_exactly && (long long)n * d.OH * d.OW * (c / 4) < (1LL << 31) &&
      (reinterpret_cast<uintptr_t>(tiemask) & 7u) == 0) {
    const unsigned windows = (unsigned)((long long)n * d.OH * d.OW * (c / 4));
    maxpool_bwd_window_kernel<<<mtb_stream_grid(windows, 256), 256, 0, st>>>(dy, tiemask, dx, d, windows);
  } else if (tiemask) {
    if (vec) maxpool_bwd_kernel<4, 0><<<grid, 256, 0, st>>>(dy, tiemask, out, x, dx, d, total);
    else maxpool_bwd_kernel<1, 0><<<grid, 256, 0, st>>>(dy, tiemask, out, x, dx, d, total);
  } else {
    if (vec) maxpool_bwd_kernel<4, 1><<<grid, 256, 0, st>>>(dy, tiemask, out, x, dx, d, total);
    else maxpool_bwd_kernel<1, 1><<<grid, 256, 0, st>>>(dy, tiemask, out, x, dx, d, total);
  }
  MTB_LAUNCH_CHECK("maxpool_bwd_kernel");
  return MTB_OK;
}

// argmax[i] = index (kh*KW+kw) of the first maximum of window i, from the tie mask.
MTB_API int mtb_max_pool2d_argmax_u8(const unsigned short* tiemask, unsigned char* argmax, long long n, void* stream) {
  MTB_REQUIRE(tiemask && argmax && n >= 0, "max_pool2d_argmax: bad arguments");
  if (n == 0) return MTB_OK;
  mask_to_argmax_kernel<<<mtb_stream_grid(n, 256), 256, 0, (cudaStream_t)stream>>>(tiemask, argmax, n);
  MTB_LAUNCH_CHECK("mask_to_argmax_kernel");
  return MTB_OK;
}
