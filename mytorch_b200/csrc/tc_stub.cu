// Placeholder for the tcgen05 family while it is being brought up: nothing is supported yet,
// so every shape takes the general CUDA-core kernels.
#include "kernels.h"

long long mtb_tc_conv2d_workspace_bytes(int, int, int, int, int, int, int, int, int, int, int) { return 0; }
bool mtb_tc_conv2d_forward_supported(int, int, int, int, int, int, int, int, int, int, int, const float*, const float*, const float*) { return false; }
int mtb_tc_conv2d_forward_f32(int, int, int, int, int, int, int, int, int, int, int, const float*, const float*, const float*, float*, int, void*) {
  return mtb_fail(MTB_ERR_UNSUPPORTED, "tensor-core conv forward not built");
}
bool mtb_tc_conv2d_dgrad_supported(int, int, int, int, int, int, int, int, int, int, int, const float*, const float*, const float*) { return false; }
int mtb_tc_conv2d_dgrad_f32(int, int, int, int, int, int, int, int, int, int, int, const float*, const float*, float*, void*, long long, void*) {
  return mtb_fail(MTB_ERR_UNSUPPORTED, "tensor-core conv dgrad not built");
}
bool mtb_tc_conv2d_wgrad_supported(int, int, int, int, int, int, int, int, int, int, int, const float*, const float*, const float*) { return false; }
int mtb_tc_conv2d_wgrad_f32(int, int, int, int, int, int, int, int, int, int, int, const float*, const float*, float*, void*, long long, void*) {
  return mtb_fail(MTB_ERR_UNSUPPORTED, "tensor-core conv wgrad not built");
}
bool mtb_tc_gemm_supported(int, int, int, const float*, int, const float*, int, const float*) { return false; }
int mtb_tc_gemm_f32(int, int, int, const float*, int, const float*, int, const float*, int, float*, void*) {
  return mtb_fail(MTB_ERR_UNSUPPORTED, "tensor-core gemm not built");
}
