// CUDA-core (FFMA) tiled GEMM with functor-addressed operands.  This is the general path for
// shapes the tensor-core kernels do not take (channel counts that are not a multiple of the
// TMA alignment, e.g. 1- or 3-channel stems; odd sizes; tiny matrices) and for the plain `mm`
// operator.  64x64x16 tiles, 256 threads, 4x4 outputs per thread, optional split-K into
// scratch with a fixed-order second pass (deterministic, no atomics).
#include "common.cuh"

namespace {

struct ConvDims {
  int N, Cin, H, W, KH, KW, SH, SW, PH, PW, Cout, OH, OW;
};

// Dense operand: element (i, k) at p[i*si + k*sk].
struct Dense {
  const float* p;
  long long si, sk;
  __device__ __forceinline__ float operator()(int i, long long k) const { return p[i * si + k * sk]; }
};

// Patch matrix of a channels-last input: row m = (n, oh, ow), column k = (kh, kw, ci).
struct PatchRows {
  const float* x;
  ConvDims d;
  __device__ __forceinline__ float at(long long m, int k) const {
    int ci = k % d.Cin;
    int t = k / d.Cin;
    int kw = t % d.KW, kh = t / d.KW;
    int ow = (int)(m % d.OW);
    long long t2 = m / d.OW;
    int oh = (int)(t2 % d.OH);
    int n = (int)(t2 / d.OH);
    int ih = oh * d.SH - d.PH + kh, iw = ow * d.SW - d.PW + kw;
    if (ih < 0 || ih >= d.H || iw < 0 || iw >= d.W) return 0.f;
    return x[(((long long)n * d.H + ih) * d.W + iw) * d.Cin + ci];
  }
};
struct PatchA {  // A(i = m, k)
  PatchRows r;
  __device__ __forceinline__ float operator()(int i, long long k) const { return r.at(i, (int)k); }
};
struct PatchB {  // B(k = m, j = patch column)
  PatchRows r;
  __device__ __forceinline__ float operator()(int j, long long k) const { return r.at(k, j); }
};

// dgrad operand: row m = input pixel (n, h, w), column k = (kh, kw, co); value dY at the output
// pixel that tap (kh, kw) connects to this input pixel, or 0 when there is none.
struct DgradA {
  const float* dy;
  ConvDims d;
  __device__ __forceinline__ float operator()(int i, long long kk) const {
    int k = (int)kk;
    int co = k % d.Cout;
    int t = k / d.Cout;
    int kw = t % d.KW, kh = t / d.KW;
    int w = i % d.W;
    int t2 = i / d.W;
    int h = t2 % d.H;
    int n = t2 / d.H;
    int hh = h + d.PH - kh, ww = w + d.PW - kw;
    if (hh < 0 || ww < 0 || hh % d.SH || ww % d.SW) return 0.f;
    int oh = hh / d.SH, ow = ww / d.SW;
    if (oh >= d.OH || ow >= d.OW) return 0.f;
    return dy[(((long long)n * d.OH + oh) * d.OW + ow) * d.Cout + co];
  }
};
// dgrad weights: B(k = (kh,kw,co), j = ci) = W[co][kh][kw][ci].
struct DgradB {
  const float* w;
  ConvDims d;
  __device__ __forceinline__ float operator()(int j, long long kk) const {
    int k = (int)kk;
    int co = k % d.Cout;
    int tap = k / d.Cout;
    return w[((long long)co * d.KH * d.KW + tap) * d.Cin + j];
  }
};

struct StoreBias {  // out[i*ld + j] = acc (+ bias[j]) (relu)
  float* out;
  long long ld;
  const float* bias;
  int relu;
  __device__ __forceinline__ void operator()(int i, int j, float v, int) const {
    if (bias) v += bias[j];
    if (relu) v = fmaxf(v, 0.f);
    out[i * ld + j] = v;
  }
};
struct StoreSplit {  // out[(z*M + i)*ld + j]
  float* out;
  long long ld;
  long long plane;
  __device__ __forceinline__ void operator()(int i, int j, float v, int z) const { out[z * plane + i * ld + j] = v; }
};

constexpr int BM = 64, BN = 64, BK = 16;

// C[i, j] = sum_k A(i, k) * B(j, k).  A_KFAST / B_KFAST: consecutive k are consecutive in
// memory for that operand (choose the load mapping that coalesces).
template <class LA, class LB, class ST, bool A_KFAST, bool B_KFAST>
__global__ void __launch_bounds__(256) gemm_simt_kernel(LA la, LB lb, ST st, int M, int N, long long K, long long k_per_split) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Bs[BK][BN + 4];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int m0 = blockIdx.x * BM, n0 = blockIdx.y * BN;
  long long k0 = blockIdx.z * k_per_split;
  long long k1 = k0 + k_per_split < K ? k0 + k_per_split : K;
  float acc[4][4];
#pragma unroll
  for (int a = 0; a < 4; ++a)
#pragma unroll
    for (int b = 0; b < 4; ++b) acc[a][b] = 0.f;
  for (long long kb = k0; kb < k1; kb += BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int r, kk;
      if (A_KFAST) { kk = tid & 15; r = (tid >> 4) + 16 * i; }
      else { r = tid & 63; kk = (tid >> 6) + 4 * i; }
      float v = 0.f;
      if (m0 + r < M && kb + kk < k1) v = la(m0 + r, kb + kk);
      As[kk][r] = v;
      if (B_KFAST) { kk = tid & 15; r = (tid >> 4) + 16 * i; }
      else { r = tid & 63; kk = (tid >> 6) + 4 * i; }
      v = 0.f;
      if (n0 + r < N && kb + kk < k1) v = lb(n0 + r, kb + kk);
      Bs[kk][r] = v;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float4 a4 = *reinterpret_cast<const float4*>(&As[kk][ty * 4]);
      float4 b4 = *reinterpret_cast<const float4*>(&Bs[kk][tx * 4]);
      float a[4] = {a4.x, a4.y, a4.z, a4.w}, b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
      for (int p = 0; p < 4; ++p)
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[p][q] += a[p] * b[q];
    }
    __syncthreads();
  }
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    int i = m0 + ty * 4 + p;
    if (i >= M) continue;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      int j = n0 + tx * 4 + q;
      if (j < N) st(i, j, acc[p][q], blockIdx.z);
    }
  }
}

__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ ws, float* __restrict__ out, long long n, int splits) {
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  long long stride = (long long)gridDim.x * blockDim.x;
  for (; i < n; i += stride) {
    float s = 0.f;
    for (int z = 0; z < splits; ++z) s += ws[z * n + i];
    out[i] = s;
  }
}

template <class LA, class LB, class ST, bool AK, bool BK_>
int launch_gemm(LA la, LB lb, ST st, long long M, long long N, long long K, int splits, cudaStream_t s, const char* name) {
  MTB_REQUIRE(M > 0 && N > 0 && K > 0 && M < (1LL << 31) && N < (1LL << 31), "%s: bad GEMM extents", name);
  long long kps = (K + splits - 1) / splits;
  kps = (kps + BK - 1) / BK * BK;
  dim3 grid(mtb_div_up(M, BM), mtb_div_up(N, BN), splits);
  MTB_REQUIRE(grid.y <= 65535 && grid.z <= 65535, "%s: grid too large", name);
  gemm_simt_kernel<LA, LB, ST, AK, BK_><<<grid, 256, 0, s>>>(la, lb, st, (int)M, (int)N, K, kps);
  MTB_LAUNCH_CHECK(name);
  return MTB_OK;
}

int conv_dims(ConvDims& d, int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout) {
  MTB_REQUIRE(n > 0 && cin > 0 && h > 0 && w > 0 && kh > 0 && kw > 0 && sh > 0 && sw > 0 && ph >= 0 && pw >= 0 && cout > 0, "conv2d: bad shape");
  d = ConvDims{n, cin, h, w, kh, kw, sh, sw, ph, pw, cout, (h + 2 * ph - kh) / sh + 1, (w + 2 * pw - kw) / sw + 1};
  MTB_REQUIRE(d.OH > 0 && d.OW > 0, "conv2d: empty output");
  MTB_REQUIRE((long long)n * d.OH * d.OW < (1LL << 31) && (long long)n * h * w < (1LL << 31), "conv2d: too many pixels for this kernel");
  return MTB_OK;
}

int wgrad_splits(const ConvDims& d) {
  long long K = (long long)d.KH * d.KW * d.Cin, M = (long long)d.N * d.OH * d.OW;
  long long tiles = (long long)mtb_div_up(d.Cout, BM) * mtb_div_up(K, BN);
  long long s = (2LL * mtb_sm_count() + tiles - 1) / tiles;
  long long maxs = (M + 255) / 256;
  if (s > maxs) s = maxs;
  if (s < 1) s = 1;
  return (int)s;
}

}  // namespace

// ------------------------------------------------------------------ convolution (general path)

MTB_API int mtb_conv2d_forward_simt_f32(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* x,
                                        const float* wt, const float* bias, float* y, int relu, void* stream) {
  ConvDims d;
  int rc = conv_dims(d, n, cin, h, w, kh, kw, sh, sw, ph, pw, cout);
  if (rc) return rc;
  MTB_REQUIRE(x && wt && y, "conv2d_forward: null pointer");
  long long K = (long long)kh * kw * cin, M = (long long)n * d.OH * d.OW;
  return launch_gemm<PatchA, Dense, StoreBias, true, true>(PatchA{{x, d}}, Dense{wt, K, 1}, StoreBias{y, cout, bias, relu}, M, cout, K, 1,
                                                           (cudaStream_t)stream, "conv2d_forward_simt");
}

MTB_API int mtb_conv2d_dgrad_simt_f32(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* dy,
                                      const float* wt, float* dx, void* stream) {
  ConvDims d;
  int rc = conv_dims(d, n, cin, h, w, kh, kw, sh, sw, ph, pw, cout);
  if (rc) return rc;
  MTB_REQUIRE(dy && wt && dx, "conv2d_dgrad: null pointer");
  long long K = (long long)kh * kw * cout, M = (long long)n * h * w;
  return launch_gemm<DgradA, DgradB, StoreBias, true, false>(DgradA{dy, d}, DgradB{wt, d}, StoreBias{dx, cin, nullptr, 0}, M, cin, K, 1,
                                                             (cudaStream_t)stream, "conv2d_dgrad_simt");
}

MTB_API long long mtb_conv2d_wgrad_simt_workspace_bytes(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout) {
  ConvDims d;
  if (conv_dims(d, n, cin, h, w, kh, kw, sh, sw, ph, pw, cout)) return -1;
  return (long long)wgrad_splits(d) * cout * kh * kw * cin * 4 + 256;
}

MTB_API int mtb_conv2d_wgrad_simt_f32(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* x,
                                      const float* dy, float* dw, void* workspace, long long workspace_bytes, void* stream) {
  ConvDims d;
  int rc = conv_dims(d, n, cin, h, w, kh, kw, sh, sw, ph, pw, cout);
  if (rc) return rc;
  MTB_REQUIRE(x && dy && dw, "conv2d_wgrad: null pointer");
  long long K = (long long)kh * kw * cin, M = (long long)n * d.OH * d.OW;
  int splits = wgrad_splits(d);
  cudaStream_t st = (cudaStream_t)stream;
  if (splits == 1) {
    return launch_gemm<Dense, PatchB, StoreBias, false, false>(Dense{dy, 1, cout}, PatchB{{x, d}}, StoreBias{dw, K, nullptr, 0}, cout, K, M, 1, st,
                                                               "conv2d_wgrad_simt");
  }
  MTB_REQUIRE(workspace && workspace_bytes >= (long long)splits * cout * K * 4, "conv2d_wgrad: workspace too small");
  rc = launch_gemm<Dense, PatchB, StoreSplit, false, false>(Dense{dy, 1, cout}, PatchB{{x, d}}, StoreSplit{(float*)workspace, K, (long long)cout * K},
                                                            cout, K, M, splits, st, "conv2d_wgrad_simt");
  if (rc) return rc;
  long long total = (long long)cout * K;
  splitk_reduce_kernel<<<mtb_stream_grid(total, 256), 256, 0, st>>>((const float*)workspace, dw, total, splits);
  MTB_LAUNCH_CHECK("splitk_reduce_kernel");
  return MTB_OK;
}

// ------------------------------------------------------------------ few-row products (classifier weight gradient)

namespace {

// C[M,N] = A^T B for A stored [K][M] with M <= 16 and B [K][N]: the weight gradient of a Linear layer
// with few outputs (dW[10][512] = dY^T X).  The 64x64-tile kernel above would run a handful of CTAs
// that each walk all of K; here a CTA owns 32 columns, its 8 warps split K, every lane keeps M
// accumulators for its column, and the 8 partial results are added in warp order through shared memory.
__global__ void __launch_bounds__(256) gemm_few_rows_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ c,
                                                             int M, int N, int K) {
  __shared__ float part[8][16][33];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int col = blockIdx.x * 32 + lane;
  float acc[16];
#pragma unroll
  for (int m = 0; m < 16; ++m) acc[m] = 0.f;
  if (col < N) {
#pragma unroll 8
    for (int k = warp; k < K; k += 8) {  // unrolled: eight rows' loads are in flight before the first FMA
      const float bv = b[(long long)k * N + col];
      const float* ar = a + (long long)k * M;
#pragma unroll
      for (int m = 0; m < 16; ++m)
        if (m < M) acc[m] = fmaf(__ldg(ar + m), bv, acc[m]);
    }
  }
#pragma unroll
  for (int m = 0; m < 16; ++m) part[warp][m][lane] = acc[m];
  __syncthreads();
  for (int m = warp; m < M; m += 8) {
    float t = part[0][m][lane];
#pragma unroll
    for (int w = 1; w < 8; ++w) t += part[w][m][lane];
    if (col < N) c[(long long)m * N + col] = t;
  }
}

}  // namespace

// ------------------------------------------------------------------ dense GEMM (general path)

// C[M,N] = op(A) * op(B) (+ bias[N]) (relu). A is [M,K] (trans_a == 0) or [K,M]; B is [K,N]
// (trans_b == 0) or [N,K]; all row-major and dense.
MTB_API int mtb_gemm_simt_f32(int m, int n, int k, const float* a, int trans_a, const float* b, int trans_b, const float* bias, int relu,
                              float* c, void* stream) {
  MTB_REQUIRE(a && b && c && m > 0 && n > 0 && k > 0, "gemm: bad arguments");
  if (trans_a && !trans_b && m <= 16 && !bias && !relu) {
    gemm_few_rows_kernel<<<mtb_div_up(n, 32), 256, 0, (cudaStream_t)stream>>>(a, b, c, m, n, k);
    MTB_LAUNCH_CHECK("gemm_few_rows_kernel");
    return MTB_OK;
  }
  Dense la = trans_a ? Dense{a, 1, m} : Dense{a, k, 1};
  Dense lb = trans_b ? Dense{b, k, 1} : Dense{b, 1, n};  // B(j, kk)
  StoreBias st{c, n, bias, relu};
  cudaStream_t s = (cudaStream_t)stream;
  if (!trans_a && trans_b) return launch_gemm<Dense, Dense, StoreBias, true, true>(la, lb, st, m, n, k, 1, s, "gemm_simt");
  if (!trans_a && !trans_b) return launch_gemm<Dense, Dense, StoreBias, true, false>(la, lb, st, m, n, k, 1, s, "gemm_simt");
  if (trans_a && trans_b) return launch_gemm<Dense, Dense, StoreBias, false, true>(la, lb, st, m, n, k, 1, s, "gemm_simt");
  return launch_gemm<Dense, Dense, StoreBias, false, false>(la, lb, st, m, n, k, 1, s, "gemm_simt");
}
