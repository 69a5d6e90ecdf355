// Internal declarations shared between the entry-point file and the kernel families.
#pragma once
#include "common.cuh"

// general CUDA-core family (gemm_simt.cu)
MTB_API int mtb_conv2d_forward_simt_f32(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* x,
                                        const float* wt, const float* bias, float* y, int relu, void* stream);
MTB_API int mtb_conv2d_dgrad_simt_f32(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* dy,
                                      const float* wt, float* dx, void* stream);
MTB_API long long mtb_conv2d_wgrad_simt_workspace_bytes(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout);
MTB_API int mtb_conv2d_wgrad_simt_f32(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* x,
                                      const float* dy, float* dw, void* workspace, long long workspace_bytes, void* stream);
MTB_API int mtb_gemm_simt_f32(int m, int n, int k, const float* a, int trans_a, const float* b, int trans_b, const float* bias, int relu,
                              float* c, void* stream);

// tcgen05 tensor-core family (tc_*.cu)
long long mtb_tc_conv2d_workspace_bytes(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout);
bool mtb_tc_conv2d_forward_supported(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* x,
                                     const float* wt, const float* y);
int mtb_tc_conv2d_forward_f32(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* x,
                              const float* wt, const float* bias, float* y, int relu, void* workspace, long long workspace_bytes, void* stream,
                              float* stats = nullptr, int* stats_rows = nullptr);
bool mtb_tc_conv2d_dgrad_supported(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* dy,
                                   const float* wt, const float* dx);
bool mtb_tc_conv2d_dgrad_in_place(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* dy,
                                  const float* wt, const float* dx);
int mtb_tc_conv2d_dgrad_f32(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* dy,
                            const float* wt, const float* addend, float* dx, void* workspace, long long workspace_bytes, void* stream);
MTB_API int mtb_add_f32(const float* x, const float* y, float* z, long long n, float alpha, void* stream);
bool mtb_tc_conv2d_wgrad_supported(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* x,
                                   const float* dy, const float* dw);
int mtb_tc_conv2d_wgrad_f32(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* x,
                            const float* dy, float* dw, void* workspace, long long workspace_bytes, void* stream);
bool mtb_tc_gemm_supported(int m, int n, int k, const float* a, int trans_a, const float* b, int trans_b, const float* c);
int mtb_tc_gemm_f32(int m, int n, int k, const float* a, int trans_a, const float* b, int trans_b, const float* bias, int relu, float* c,
                    void* stream);

