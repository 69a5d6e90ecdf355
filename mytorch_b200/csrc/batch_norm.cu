// BatchNorm2d forward / backward over channels-last activations viewed as a [rows = N*H*W, C]
// matrix.  HBM-bound: forward reads x twice and writes y once (3S), backward reads x and dy
// twice and writes dx once (5S).  Per-channel statistics come from per-CTA Welford-style
// partials (shifted sums, Chan merge) combined in a fixed order by a one-CTA-per-256-channels
// finalise kernel, so results are bit-reproducible.
#include "colreduce.cuh"

MTB_API long long mtb_batch_norm2d_workspace_bytes(int n, int c, int h, int w);

namespace {

// ---------------------------------------------------------------- forward: statistics

template <int V>
__global__ void __launch_bounds__(256) bn_stats_partial_kernel(const float* __restrict__ x, long long rows, int C, int L, long long rows_per_block,
                                                                float* __restrict__ partial) {
  const int lane = threadIdx.x & (L - 1);
  const int rsub = threadIdx.x / L;
  const int R = 256 / L;
  const int cg = blockIdx.x * L + lane;  // column group
  const bool active = cg * V < C;
  long long r0 = blockIdx.y * rows_per_block;
  long long r1 = r0 + rows_per_block < rows ? r0 + rows_per_block : rows;

  float pivot[V], s1[V], s2[V];
  int cnt = 0;
#pragma unroll
  for (int i = 0; i < V; ++i) { pivot[i] = 0.f; s1[i] = 0.f; s2[i] = 0.f; }
  if (active) {
    long long r = r0 + rsub;
    if (r < r1) {
      VecF<V> f = vload<V>(x + r * C + (long long)cg * V);
#pragma unroll
      for (int i = 0; i < V; ++i) pivot[i] = f.v[i];
      cnt = 1;
      r += R;
    }
#pragma unroll 4
    for (; r < r1; r += R) {
      VecF<V> f = vload<V>(x + r * C + (long long)cg * V);
#pragma unroll
      for (int i = 0; i < V; ++i) {
        float d = f.v[i] - pivot[i];
        s1[i] += d;
        s2[i] += d * d;
      }
      ++cnt;
    }
  }
  __shared__ float sm_mean[V][256];
  __shared__ float sm_m2[V][256];
  __shared__ int sm_cnt[256];
  float inv = cnt > 0 ? 1.f / (float)cnt : 0.f;
#pragma unroll
  for (int i = 0; i < V; ++i) {
    sm_mean[i][threadIdx.x] = pivot[i] + s1[i] * inv;
    sm_m2[i][threadIdx.x] = s2[i] - s1[i] * s1[i] * inv;
  }
  sm_cnt[threadIdx.x] = cnt;
  __syncthreads();
  if (rsub == 0 && active) {
    float n = (float)cnt;
    float mean[V], m2[V];
#pragma unroll
    for (int i = 0; i < V; ++i) { mean[i] = sm_mean[i][lane]; m2[i] = sm_m2[i][lane]; }
    for (int k = 1; k < R; ++k) {
      float nb = (float)sm_cnt[k * L + lane];
      if (nb == 0.f) continue;
      float nt = n + nb;
      float wb = nb / nt;
#pragma unroll
      for (int i = 0; i < V; ++i) {
        float d = sm_mean[i][k * L + lane] - mean[i];
        mean[i] += d * wb;
        m2[i] += sm_m2[i][k * L + lane] + d * d * n * wb;
      }
      n = nt;
    }
    float* p = partial + (long long)blockIdx.y * 3 * C + (long long)cg * V;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      p[i] = n;
      p[C + i] = mean[i];
      p[2 * C + i] = m2[i];
    }
  }
}

// Chan's parallel update of (count, mean, M2).  The finalise kernel below combines the per-CTA
// partials with it and writes the batch mean / biased variance, the per-channel scale
// gamma/sqrt(var+eps) used by the normalise pass, and the blended running statistics.
__device__ __forceinline__ void chan_merge(float& n, float& mean, float& m2, float nb, float mb, float qb) {
  if (nb == 0.f) return;
  float nt = n + nb;
  float d = mb - mean;
  float wb = nb / nt;
  mean += d * wb;
  m2 += qb + d * d * n * wb;
  n = nt;
}

__global__ void __launch_bounds__(1024) bn_stats_final_kernel(const float* __restrict__ partial, int P, int C, const float* __restrict__ gamma, float eps,
                                                               float one_minus_m, float m, float* running_mean, float* running_var,
                                                               float* __restrict__ mean_out, float* __restrict__ var_out, float* __restrict__ scale_out) {
  // 8 channels x 128 partial-groups per CTA.  Group g merges partials g, g+128, ... (all loads are
  // issued before the first merge), then the 128 results are merged pairwise in a fixed tree, so the
  // kernel is a couple of memory round trips long and the result does not depend on scheduling.
  constexpr int G = 128, B = 5;
  const int cx = threadIdx.x & 7, g = threadIdx.x >> 3;
  const int c = blockIdx.x * 8 + cx;
  float n = 0.f, mean = 0.f, m2 = 0.f;
  if (c < C) {
    for (int p0 = g; p0 < P; p0 += G * B) {
      float v[B][3];
#pragma unroll
      for (int u = 0; u < B; ++u) {
        const int p = p0 + G * u;
        const float* q = partial + (long long)p * 3 * C + c;
        const bool in = p < P;
        v[u][0] = in ? q[0] : 0.f;
        v[u][1] = in ? q[C] : 0.f;
        v[u][2] = in ? q[2 * C] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < B; ++u) chan_merge(n, mean, m2, v[u][0], v[u][1], v[u][2]);
    }
  }
  __shared__ float sn[G][9], smean[G][9], sm2[G][9];
  sn[g][cx] = n; smean[g][cx] = mean; sm2[g][cx] = m2;
#pragma unroll
  for (int s = G / 2; s >= 1; s >>= 1) {
    __syncthreads();
    if (g < s) {
      chan_merge(n, mean, m2, sn[g + s][cx], smean[g + s][cx], sm2[g + s][cx]);
      sn[g][cx] = n; smean[g][cx] = mean; sm2[g][cx] = m2;
    }
  }
  if (g != 0 || c >= C) return;
  float mu = mean;
  float var = n > 0.f ? m2 / n : 0.f;
  mean_out[c] = mu;
  var_out[c] = var;
  float rstd = 1.0f / sqrtf(var + eps);
  scale_out[c] = gamma ? gamma[c] * rstd : rstd;
  if (running_mean) running_mean[c] = __fadd_rn(__fmul_rn(one_minus_m, running_mean[c]), __fmul_rn(m, mu));
  if (running_var) running_var[c] = __fadd_rn(__fmul_rn(one_minus_m, running_var[c]), __fmul_rn(m, var));
}

// Inference mode: statistics are the running ones.
__global__ void bn_eval_prep_kernel(int C, const float* __restrict__ gamma, float eps, const float* __restrict__ rm, const float* __restrict__ rv,
                                    float* __restrict__ mean_out, float* __restrict__ var_out, float* __restrict__ scale_out) {
  int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C) return;
  mean_out[c] = rm[c];
  var_out[c] = rv[c];
  float rstd = 1.0f / sqrtf(rv[c] + eps);
  scale_out[c] = gamma ? gamma[c] * rstd : rstd;
}

// ---------------------------------------------------------------- forward: normalise

// MODE 0: y = bn(x); 1: y = max(0, bn(x)); 2: y = max(0, bn(x) + res) (res has the shape of x)
template <int V, int MODE>
__global__ void __launch_bounds__(256) bn_normalize_kernel(const float* __restrict__ x, float* __restrict__ y, long long rows, int C, int L,
                                                            long long rows_per_block, const float* __restrict__ mean,
                                                            const float* __restrict__ scale, const float* __restrict__ beta,
                                                            const float* __restrict__ res) {
  const int lane = threadIdx.x & (L - 1);
  const int rsub = threadIdx.x / L;
  const int R = 256 / L;
  const int cg = blockIdx.x * L + lane;
  if (cg * V >= C) return;
  float mu[V], g[V], b[V];
#pragma unroll
  for (int i = 0; i < V; ++i) {
    mu[i] = mean[cg * V + i];
    g[i] = scale[cg * V + i];
    b[i] = beta ? beta[cg * V + i] : 0.f;
  }
  long long r0 = blockIdx.y * rows_per_block;
  long long r1 = r0 + rows_per_block < rows ? r0 + rows_per_block : rows;
#pragma unroll 4
  for (long long r = r0 + rsub; r < r1; r += R) {
    long long off = r * C + (long long)cg * V;
    VecF<V> f = vload<V>(x + off);
    VecF<V> a;
    if (MODE == 2) a = vload<V>(res + off);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      float t = (f.v[i] - mu[i]) * g[i] + b[i];
      if (MODE == 2) t = t + a.v[i];
      f.v[i] = MODE ? fmaxf(t, 0.f) : t;
    }
    vstore<V>(y + off, f);
  }
}

// ---------------------------------------------------------------- backward

// partial[p][0][c] = sum dy, partial[p][1][c] = sum dy * xhat over the CTA's rows.
// MODE 1 / 2: the forward output went through max(0, .) (MODE 2: after adding `res`) in the same pass;
// the upstream gradient is first masked where the (recomputed, bit-identical) value was negative.
template <int V, int MODE>
__global__ void __launch_bounds__(256) bn_bwd_partial_kernel(const float* __restrict__ dy, const float* __restrict__ x, long long rows, int C, int L,
                                                              long long rows_per_block, const float* __restrict__ mean,
                                                              const float* __restrict__ var, float eps, const float* __restrict__ gamma,
                                                              const float* __restrict__ beta, float* __restrict__ partial,
                                                              const float* __restrict__ res) {
  const int lane = threadIdx.x & (L - 1);
  const int rsub = threadIdx.x / L;
  const int R = 256 / L;
  const int cg = blockIdx.x * L + lane;
  const bool active = cg * V < C;
  float mu[V], rstd[V], a0[V], a1[V], gs[V], bt[V];
#pragma unroll
  for (int i = 0; i < V; ++i) {
    a0[i] = 0.f; a1[i] = 0.f;
    mu[i] = active ? mean[cg * V + i] : 0.f;
    rstd[i] = active ? 1.0f / sqrtf(var[cg * V + i] + eps) : 0.f;
    gs[i] = (active && gamma) ? gamma[cg * V + i] * rstd[i] : rstd[i];
    bt[i] = (active && beta) ? beta[cg * V + i] : 0.f;
  }
  long long r0 = blockIdx.y * rows_per_block;
  long long r1 = r0 + rows_per_block < rows ? r0 + rows_per_block : rows;
  if (active) {
#pragma unroll 4
    for (long long r = r0 + rsub; r < r1; r += R) {
      long long off = r * C + (long long)cg * V;
      VecF<V> g = vload<V>(dy + off);
      VecF<V> f = vload<V>(x + off);
      VecF<V> a;
      if (MODE == 2) a = vload<V>(res + off);
#pragma unroll
      for (int i = 0; i < V; ++i) {
        float gi = g.v[i];
        if (MODE) {
          float t = (f.v[i] - mu[i]) * gs[i] + bt[i];
          if (MODE == 2) t = t + a.v[i];
          if (t < 0.f) gi = 0.f;
        }
        a0[i] += gi;
        a1[i] += gi * ((f.v[i] - mu[i]) * rstd[i]);
      }
    }
  }
  __shared__ float sm0[V][256];
  __shared__ float sm1[V][256];
#pragma unroll
  for (int i = 0; i < V; ++i) { sm0[i][threadIdx.x] = a0[i]; sm1[i][threadIdx.x] = a1[i]; }
  __syncthreads();
  if (rsub == 0 && active) {
    for (int k = 1; k < R; ++k) {
#pragma unroll
      for (int i = 0; i < V; ++i) { a0[i] += sm0[i][k * L + lane]; a1[i] += sm1[i][k * L + lane]; }
    }
    float* p = partial + (long long)blockIdx.y * 2 * C + (long long)cg * V;
#pragma unroll
    for (int i = 0; i < V; ++i) { p[i] = a0[i]; p[C + i] = a1[i]; }
  }
}

// dbeta = sum dy, dgamma = sum dy*xhat; coefficients for dx = k1 * (dy - k2 - (x - mean) * k3).
// Thirty-two threads per channel, fixed summation order.
__global__ void __launch_bounds__(1024) bn_bwd_final_kernel(const float* __restrict__ partial, int P, int C, const float* __restrict__ gamma,
                                                             const float* __restrict__ var, float eps, float inv_m, float* __restrict__ dgamma,
                                                             float* __restrict__ dbeta, float* __restrict__ coef) {
  // 8 channels x 128 partial-groups per CTA, loads first, then a fixed pairwise tree (see above).
  constexpr int G = 128, B = 5;
  const int cx = threadIdx.x & 7, g = threadIdx.x >> 3;
  const int c = blockIdx.x * 8 + cx;
  float s0 = 0.f, s1 = 0.f;
  if (c < C) {
    for (int p0 = g; p0 < P; p0 += G * B) {
      float v[B][2];
#pragma unroll
      for (int u = 0; u < B; ++u) {
        const int p = p0 + G * u;
        const bool in = p < P;
        v[u][0] = in ? partial[(long long)p * 2 * C + c] : 0.f;
        v[u][1] = in ? partial[(long long)p * 2 * C + C + c] : 0.f;
      }
#pragma unroll
      for (int u = 0; u < B; ++u) { s0 += v[u][0]; s1 += v[u][1]; }
    }
  }
  __shared__ float t0[G][9], t1[G][9];
  t0[g][cx] = s0; t1[g][cx] = s1;
#pragma unroll
  for (int s = G / 2; s >= 1; s >>= 1) {
    __syncthreads();
    if (g < s) {
      s0 += t0[g + s][cx]; s1 += t1[g + s][cx];
      t0[g][cx] = s0; t1[g][cx] = s1;
    }
  }
  if (g != 0 || c >= C) return;
  float db = s0, dg = s1;
  if (dbeta) dbeta[c] = db;
  if (dgamma) dgamma[c] = dg;
  float rstd = 1.0f / sqrtf(var[c] + eps);
  float gm = gamma ? gamma[c] : 1.f;
  coef[c] = gm * rstd;               // k1
  coef[C + c] = db * inv_m;          // k2
  coef[2 * C + c] = rstd * dg * inv_m;  // k3: (x - mean) * k3 = xhat * dgamma / m
}

// MODE 2 also writes the masked upstream gradient, which is the gradient of the added tensor, to dres.
template <int V, int MODE>
__global__ void __launch_bounds__(256) bn_bwd_dx_kernel(const float* __restrict__ dy, const float* __restrict__ x, float* __restrict__ dx,
                                                         long long rows, int C, int L, long long rows_per_block,
                                                         const float* __restrict__ mean, const float* __restrict__ coef,
                                                         const float* __restrict__ beta, const float* __restrict__ res, float* __restrict__ dres) {
  const int lane = threadIdx.x & (L - 1);
  const int rsub = threadIdx.x / L;
  const int R = 256 / L;
  const int cg = blockIdx.x * L + lane;
  if (cg * V >= C) return;
  float mu[V], k1[V], k2[V], k3[V], bt[V];
#pragma unroll
  for (int i = 0; i < V; ++i) {
    mu[i] = mean[cg * V + i];
    k1[i] = coef[cg * V + i];
    k2[i] = coef[C + cg * V + i];
    k3[i] = coef[2 * C + cg * V + i];
    bt[i] = beta ? beta[cg * V + i] : 0.f;
  }
  long long r0 = blockIdx.y * rows_per_block;
  long long r1 = r0 + rows_per_block < rows ? r0 + rows_per_block : rows;
#pragma unroll 4
  for (long long r = r0 + rsub; r < r1; r += R) {
    long long off = r * C + (long long)cg * V;
    VecF<V> g = vload<V>(dy + off);
    VecF<V> f = vload<V>(x + off);
    VecF<V> a, m;
    if (MODE == 2) a = vload<V>(res + off);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      float gi = g.v[i];
      if (MODE) {
        float t = (f.v[i] - mu[i]) * k1[i] + bt[i];  // k1 = gamma / sigma, the forward's scale
        if (MODE == 2) t = t + a.v[i];
        if (t < 0.f) gi = 0.f;
      }
      m.v[i] = gi;
      g.v[i] = k1[i] * (gi - k2[i] - (f.v[i] - mu[i]) * k3[i]);
    }
    vstore<V>(dx + off, g);
    if (MODE == 2) vstore<V>(dres + off, m);
  }
}

// A streaming pass wants more CTAs than a reduction (no partial rows to combine afterwards).
ColCfg stream_cfg(long long rows, int C, bool aligned) {
  ColCfg c = mtb_col_cfg(rows, C, aligned);
  long long target = (long long)mtb_sm_count() * 8 / c.col_blocks;
  if (target < 1) target = 1;
  long long min_rows = (long long)c.rows_per_iter * 4;
  long long want = (rows + min_rows - 1) / min_rows;
  if (want < 1) want = 1;
  long long rb = want < target ? want : target;
  long long rpb = (rows + rb - 1) / rb;
  rpb = (rpb + c.rows_per_iter - 1) / c.rows_per_iter * c.rows_per_iter;
  c.rows_per_block = rpb;
  c.row_blocks = (int)((rows + rpb - 1) / rpb);
  return c;
}

int launch_normalize(const float* x, float* y, long long rows, int c, bool aligned, const float* mean, const float* scale, const float* beta,
                     int mode, const float* res, cudaStream_t st) {
  ColCfg s = stream_cfg(rows, c, aligned);
  dim3 grid(s.col_blocks, s.row_blocks);
#define MTB_BN_NORM(V_, M_) bn_normalize_kernel<V_, M_><<<grid, 256, 0, st>>>(x, y, rows, c, s.lanes, s.rows_per_block, mean, scale, beta, res)
  if (s.vec == 4) { if (mode == 2) MTB_BN_NORM(4, 2); else if (mode == 1) MTB_BN_NORM(4, 1); else MTB_BN_NORM(4, 0); }
  else { if (mode == 2) MTB_BN_NORM(1, 2); else if (mode == 1) MTB_BN_NORM(1, 1); else MTB_BN_NORM(1, 0); }
#undef MTB_BN_NORM
  MTB_LAUNCH_CHECK("bn_normalize_kernel");
  return MTB_OK;
}

// mode 0: y = bn(x); 1: y = max(0, bn(x)); 2: y = max(0, bn(x) + res).  stats / stats_rows: batch statistics
// prepared by the producer of x as partial rows (see mtb_conv2d_forward_stats_f32); 0 rows = compute them here.
int bn_forward(int n, int c, int h, int w, const float* x, const float* gamma, const float* beta, double eps, int training, double momentum,
               float* running_mean, float* running_var, float* y, float* mean, float* var, int mode, const float* res, const float* stats,
               int stats_rows, void* workspace, long long workspace_bytes, cudaStream_t st) {
  MTB_REQUIRE(n > 0 && c > 0 && h > 0 && w > 0 && x && y && mean && var && workspace, "batch_norm2d_forward: bad arguments");
  MTB_REQUIRE(workspace_bytes >= mtb_batch_norm2d_workspace_bytes(n, c, h, w), "batch_norm2d_forward: workspace too small");
  MTB_REQUIRE(training || (running_mean && running_var), "batch_norm2d_forward: inference needs running statistics");
  MTB_REQUIRE(mode != 2 || res, "batch_norm2d_add_relu_forward: the tensor to add is missing");
  long long rows = (long long)n * h * w;
  bool aligned = mtb_aligned16(x) && mtb_aligned16(y) && (mode != 2 || mtb_aligned16(res));
  float* partial = (float*)workspace;
  float* scale = partial + (long long)mtb_col_max_partials() * 3 * c;
  if (training) {
    int P = stats_rows;
    if (!(stats && stats_rows > 0)) {
      ColCfg cfg = mtb_col_cfg(rows, c, mtb_aligned16(x));
      dim3 grid(cfg.col_blocks, cfg.row_blocks);
      if (cfg.vec == 4) bn_stats_partial_kernel<4><<<grid, 256, 0, st>>>(x, rows, c, cfg.lanes, cfg.rows_per_block, partial);
      else bn_stats_partial_kernel<1><<<grid, 256, 0, st>>>(x, rows, c, cfg.lanes, cfg.rows_per_block, partial);
      MTB_LAUNCH_CHECK("bn_stats_partial_kernel");
      stats = partial;
      P = cfg.row_blocks;
    }
    bn_stats_final_kernel<<<mtb_div_up(c, 8), 1024, 0, st>>>(stats, P, c, gamma, (float)eps, (float)(1.0 - momentum), (float)momentum,
                                                              running_mean, running_var, mean, var, scale);
    MTB_LAUNCH_CHECK("bn_stats_final_kernel");
  } else {
    bn_eval_prep_kernel<<<mtb_div_up(c, 128), 128, 0, st>>>(c, gamma, (float)eps, running_mean, running_var, mean, var, scale);
    MTB_LAUNCH_CHECK("bn_eval_prep_kernel");
  }
  return launch_normalize(x, y, rows, c, aligned, mean, scale, beta, mode, res, st);
}

// dx = gamma/sigma * (g - dbeta/m - xhat * dgamma/m) with g = dy masked by the forward's ReLU (modes 1, 2);
// mode 2 also writes g to dres (the gradient of the added tensor).
int bn_backward(int n, int c, int h, int w, const float* dy, const float* mean, const float* var, const float* x, const float* gamma,
                const float* beta, double eps, int mode, const float* res, float* dx, float* dres, float* dgamma, float* dbeta, void* workspace,
                long long workspace_bytes, cudaStream_t st) {
  MTB_REQUIRE(n > 0 && c > 0 && h > 0 && w > 0 && dy && mean && var && x && dx && workspace, "batch_norm2d_backward: bad arguments");
  MTB_REQUIRE(workspace_bytes >= mtb_batch_norm2d_workspace_bytes(n, c, h, w), "batch_norm2d_backward: workspace too small");
  MTB_REQUIRE(mode != 2 || (res && dres), "batch_norm2d_add_relu_backward: the added tensor and its gradient buffer are required");
  long long rows = (long long)n * h * w;
  bool aligned = mtb_aligned16(x) && mtb_aligned16(dy) && mtb_aligned16(dx) && (mode != 2 || (mtb_aligned16(res) && mtb_aligned16(dres)));
  float* partial = (float*)workspace;
  float* coef = partial + (long long)mtb_col_max_partials() * 3 * c;  // 3*C floats fit in the 4*C tail
  ColCfg cfg = mtb_col_cfg(rows, c, aligned);
  dim3 grid(cfg.col_blocks, cfg.row_blocks);
#define MTB_BN_PARTIAL(V_, M_) \
  bn_bwd_partial_kernel<V_, M_><<<grid, 256, 0, st>>>(dy, x, rows, c, cfg.lanes, cfg.rows_per_block, mean, var, (float)eps, gamma, beta, partial, res)
  if (cfg.vec == 4) { if (mode == 2) MTB_BN_PARTIAL(4, 2); else if (mode == 1) MTB_BN_PARTIAL(4, 1); else MTB_BN_PARTIAL(4, 0); }
  else { if (mode == 2) MTB_BN_PARTIAL(1, 2); else if (mode == 1) MTB_BN_PARTIAL(1, 1); else MTB_BN_PARTIAL(1, 0); }
#undef MTB_BN_PARTIAL
  MTB_LAUNCH_CHECK("bn_bwd_partial_kernel");
  bn_bwd_final_kernel<<<mtb_div_up(c, 8), 1024, 0, st>>>(partial, cfg.row_blocks, c, gamma, var, (float)eps, (float)(1.0 / (double)rows),
                                                          dgamma, dbeta, coef);
  MTB_LAUNCH_CHECK("bn_bwd_final_kernel");
  ColCfg s = stream_cfg(rows, c, aligned);
  dim3 g2(s.col_blocks, s.row_blocks);
#define MTB_BN_DX(V_, M_) bn_bwd_dx_kernel<V_, M_><<<g2, 256, 0, st>>>(dy, x, dx, rows, c, s.lanes, s.rows_per_block, mean, coef, beta, res, dres)
  if (s.vec == 4) { if (mode == 2) MTB_BN_DX(4, 2); else if (mode == 1) MTB_BN_DX(4, 1); else MTB_BN_DX(4, 0); }
  else { if (mode == 2) MTB_BN_DX(1, 2); else if (mode == 1) MTB_BN_DX(1, 1); else MTB_BN_DX(1, 0); }
#undef MTB_BN_DX
  MTB_LAUNCH_CHECK("bn_bwd_dx_kernel");
  return MTB_OK;
}

}  // namespace

// Scratch the forward and backward entry points need, in bytes (an upper bound for the shape).
MTB_API long long mtb_batch_norm2d_workspace_bytes(int n, int c, int h, int w) {
  (void)n; (void)h; (void)w;
  long long floats = (long long)mtb_col_max_partials() * 3 * c + 4LL * c;
  return floats * 4 + 256;
}

// Training: batch statistics (biased variance also goes into running_var). Inference: running
// statistics. x, y are channels-last [N,H,W,C]; mean/var outputs are [C]. gamma/beta/running_*
// may be NULL. relu != 0 applies max(0, .) to y in the same pass.
MTB_API int mtb_batch_norm2d_forward_f32(int n, int c, int h, int w, const float* x, const float* gamma, const float* beta, double eps,
                                         int training, double momentum, float* running_mean, float* running_var, float* y,
                                         float* mean, float* var, int relu, void* workspace, long long workspace_bytes, void* stream) {
  return bn_forward(n, c, h, w, x, gamma, beta, eps, training, momentum, running_mean, running_var, y, mean, var, relu ? 1 : 0, nullptr, nullptr, 0,
                    workspace, workspace_bytes, (cudaStream_t)stream);
}

// Training-mode forward whose batch statistics were prepared by the producer of x: `stats` holds
// stats_rows partial rows [row][3][C] of per-channel (count, mean, M2) that together cover every element
// of x exactly once (mtb_conv2d_forward_stats_f32 writes them from the convolution's epilogue).  The
// statistics pass over x is skipped: the partials are merged (fixed order), then x is normalised.
MTB_API int mtb_batch_norm2d_forward_prestats_f32(int n, int c, int h, int w, const float* x, const float* gamma, const float* beta, double eps,
                                                  double momentum, float* running_mean, float* running_var, float* y, float* mean, float* var,
                                                  int relu, const float* stats, int stats_rows, void* workspace, long long workspace_bytes,
                                                  void* stream) {
  MTB_REQUIRE(stats && stats_rows > 0, "batch_norm2d_forward_prestats: no statistics rows");
  return bn_forward(n, c, h, w, x, gamma, beta, eps, 1, momentum, running_mean, running_var, y, mean, var, relu ? 1 : 0, nullptr, stats, stats_rows,
                    workspace, workspace_bytes, (cudaStream_t)stream);
}

// y = max(0, batch_norm(x) + residual): the tail of a residual block (BatchNorm, shortcut addition, ReLU) in
// one normalise pass; the BatchNorm output is never stored.  stats / stats_rows as above (NULL / 0: the
// statistics are computed here).  residual has the shape of x.
MTB_API int mtb_batch_norm2d_add_relu_forward_f32(int n, int c, int h, int w, const float* x, const float* residual, const float* gamma,
                                                  const float* beta, double eps, int training, double momentum, float* running_mean,
                                                  float* running_var, float* y, float* mean, float* var, const float* stats, int stats_rows,
                                                  void* workspace, long long workspace_bytes, void* stream) {
  return bn_forward(n, c, h, w, x, gamma, beta, eps, training, momentum, running_mean, running_var, y, mean, var, 2, residual, stats, stats_rows,
                    workspace, workspace_bytes, (cudaStream_t)stream);
}

// dx = gamma/sigma * (dy - dbeta/m - xhat * dgamma/m); dgamma, dbeta may be NULL (not affine).
// relu != 0: backward of the fused forward (relu flag set there); dy is masked where the
// normalised value gamma*xhat+beta is negative, which needs beta (NULL = 0).
MTB_API int mtb_batch_norm2d_backward_f32(int n, int c, int h, int w, const float* dy, const float* mean, const float* var, const float* x,
                                          const float* gamma, const float* beta, double eps, int relu, float* dx, float* dgamma,
                                          float* dbeta, void* workspace, long long workspace_bytes, void* stream) {
  return bn_backward(n, c, h, w, dy, mean, var, x, gamma, beta, eps, relu ? 1 : 0, nullptr, dx, nullptr, dgamma, dbeta, workspace, workspace_bytes,
                     (cudaStream_t)stream);
}

// Backward of mtb_batch_norm2d_add_relu_forward_f32: the ReLU mask is recomputed from x, the statistics and
// residual with the forward's own expression; dresidual receives the masked upstream gradient (the
// gradient of the added tensor), dx the BatchNorm input gradient.
MTB_API int mtb_batch_norm2d_add_relu_backward_f32(int n, int c, int h, int w, const float* dy, const float* mean, const float* var,
                                                   const float* x, const float* residual, const float* gamma, const float* beta, double eps,
                                                   float* dx, float* dresidual, float* dgamma, float* dbeta, void* workspace,
                                                   long long workspace_bytes, void* stream) {
  return bn_backward(n, c, h, w, dy, mean, var, x, gamma, beta, eps, 2, residual, dx, dresidual, dgamma, dbeta, workspace, workspace_bytes,
                     (cudaStream_t)stream);
}
