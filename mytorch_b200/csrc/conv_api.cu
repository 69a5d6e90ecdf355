// Public convolution / GEMM entry points.  Each picks the kernel family for the shape: the
// tcgen05 tensor-core kernels when the shape meets their alignment rules, otherwise the
// general CUDA-core kernels.  Both families run on the GPU; there is no host fallback.
#include "common.cuh"
#include "kernels.h"

MTB_API long long mtb_conv2d_workspace_bytes(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout) {
  long long a = mtb_conv2d_wgrad_simt_workspace_bytes(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout);
  long long b = mtb_tc_conv2d_workspace_bytes(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout);
  return a > b ? a : b;
}

// workspace (may be NULL): scratch of mtb_conv2d_workspace_bytes(); with it, layers whose output has too few
// tiles to fill the GPU split their reduction across CTAs (partials in the workspace, added in a fixed order).
MTB_API int mtb_conv2d_forward_f32(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* x,
                                   const float* wt, const float* bias, float* y, int relu, void* workspace, long long workspace_bytes,
                                   void* stream) {
  if (mtb_tc_conv2d_forward_supported(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout, x, wt, y))
    return mtb_tc_conv2d_forward_f32(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout, x, wt, bias, y, relu, workspace, workspace_bytes, stream);
  return mtb_conv2d_forward_simt_f32(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout, x, wt, bias, y, relu, stream);
}

// Forward convolution that also prepares the batch statistics of its output for a BatchNorm layer
// that follows (the statistics pass of BatchNorm re-reads the whole activation otherwise).  stats:
// room for mtb_conv2d_stats_max_rows() x 3 x cout floats; *stats_rows (HOST) receives the number of
// partial rows [row][3][cout] = (count, mean, M2) written, to be passed to
// mtb_batch_norm2d_forward_prestats_f32, or 0 when this shape's kernel does not produce them (the
// caller then runs the ordinary BatchNorm forward).
MTB_API int mtb_conv2d_stats_max_rows() { return 4 * mtb_sm_count(); }

MTB_API int mtb_conv2d_forward_stats_f32(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* x,
                                         const float* wt, const float* bias, float* y, int relu, float* stats, int* stats_rows, void* workspace,
                                         long long workspace_bytes, void* stream) {
  MTB_REQUIRE(stats && stats_rows, "conv2d_forward_stats: stats buffer and row counter are required");
  *stats_rows = 0;
  if (mtb_tc_conv2d_forward_supported(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout, x, wt, y))
    return mtb_tc_conv2d_forward_f32(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout, x, wt, bias, y, relu, workspace, workspace_bytes, stream, stats,
                                     stats_rows);
  return mtb_conv2d_forward_simt_f32(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout, x, wt, bias, y, relu, stream);
}

MTB_API int mtb_conv2d_dgrad_f32(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* dy,
                                 const float* wt, float* dx, void* workspace, long long workspace_bytes, void* stream) {
  if (mtb_tc_conv2d_dgrad_supported(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout, dy, wt, dx))
    return mtb_tc_conv2d_dgrad_f32(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout, dy, wt, nullptr, dx, workspace, workspace_bytes, stream);
  return mtb_conv2d_dgrad_simt_f32(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout, dy, wt, dx, stream);
}

// dx = dgrad(dy, wt) + addend: the data gradient added to a gradient the same tensor already received
// from another consumer (residual connections).  On the row-staged tensor-core path the sum happens
// in the epilogue, which saves one pass over dx and one launch; elsewhere it is dgrad followed by an
// add.  addend has the shape of dx and must not alias it, except where
// mtb_conv2d_dgrad_accumulates_in_place answers 1: there addend == dx means dx += data gradient.
MTB_API int mtb_conv2d_dgrad_add_f32(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* dy,
                                     const float* wt, const float* addend, float* dx, void* workspace, long long workspace_bytes, void* stream) {
  MTB_REQUIRE(addend, "conv2d_dgrad_add: addend must be given");
  if (addend == dx) {  // accumulate in place: only where mtb_conv2d_dgrad_accumulates_in_place says so
    MTB_REQUIRE(mtb_tc_conv2d_dgrad_in_place(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout, dy, wt, dx),
                "conv2d_dgrad_add: this shape cannot accumulate in place (addend must not alias dx)");
    return mtb_tc_conv2d_dgrad_f32(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout, dy, wt, addend, dx, workspace, workspace_bytes, stream);
  }
  if (mtb_tc_conv2d_dgrad_supported(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout, dy, wt, dx))
    return mtb_tc_conv2d_dgrad_f32(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout, dy, wt, addend, dx, workspace, workspace_bytes, stream);
  int rc = mtb_conv2d_dgrad_simt_f32(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout, dy, wt, dx, stream);
  if (rc) return rc;
  return mtb_add_f32(dx, addend, dx, (long long)n * h * w * cin, 1.0f, stream);
}

// 1 when mtb_conv2d_dgrad_add_f32 may be called with addend == dx for this convolution (dx += data gradient,
// nothing else touched) and that is its cheaper form; 0 otherwise.  Host code only.
MTB_API int mtb_conv2d_dgrad_accumulates_in_place(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout,
                                                  const float* dy, const float* wt, const float* dx) {
  return mtb_tc_conv2d_dgrad_in_place(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout, dy, wt, dx) ? 1 : 0;
}

MTB_API int mtb_conv2d_wgrad_f32(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* x,
                                 const float* dy, float* dw, void* workspace, long long workspace_bytes, void* stream) {
  if (mtb_tc_conv2d_wgrad_supported(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout, x, dy, dw))
    return mtb_tc_conv2d_wgrad_f32(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout, x, dy, dw, workspace, workspace_bytes, stream);
  return mtb_conv2d_wgrad_simt_f32(n, cin, h, w, kh, kw, sh, sw, ph, pw, cout, x, dy, dw, workspace, workspace_bytes, stream);
}

MTB_API int mtb_gemm_f32(int m, int n, int k, const float* a, int trans_a, const float* b, int trans_b, const float* bias, int relu, float* c,
                         void* stream) {
  if (mtb_tc_gemm_supported(m, n, k, a, trans_a, b, trans_b, c))
    return mtb_tc_gemm_f32(m, n, k, a, trans_a, b, trans_b, bias, relu, c, stream);
  return mtb_gemm_simt_f32(m, n, k, a, trans_a, b, trans_b, bias, relu, c, stream);
}
