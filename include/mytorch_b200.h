/* C ABI of libmytorch_b200.so — hand-written sm_100a kernels for the CNN training step of
 * tigert1998/mytorch.
 *
 * Conventions
 *  - Every pointer is a raw device pointer unless a comment says "host".  The caller owns all
 *    buffers, including scratch ("workspace"); the kernels allocate nothing and keep no
 *    reference after a call returns.  Memory comes from the pool in the runtime section below
 *    (or from any other allocator: the kernels only see pointers).
 *  - 4-D activations and convolution weights are channels-last: x[N][H][W][C],
 *    w[Cout][KH][KW][Cin].  Everything else is dense row-major.
 *  - `stream` is a cudaStream_t; work is enqueued on it and the call returns without
 *    synchronising, so calls may be captured in a CUDA graph.
 *  - Functions returning int return 0 on success or an MtbStatus code; mtb_last_error() then
 *    holds a message for the calling thread.  Nothing aborts or traps.
 *
 * Each declaration names the reference interface it replaces (file:line inside the
 * tigert1998/mytorch tree).  The reference's own native entry points return void and take NCHW
 * tensors; its generated symbol names are <Func>_<dtype> (mytorch/backends/cuda/env.py:201-221).
 */
#ifndef MYTORCH_B200_H
#define MYTORCH_B200_H

#ifdef __cplusplus
extern "C" {
#endif

enum MtbStatus { MTB_OK = 0, MTB_ERR_INVALID = 1, MTB_ERR_CUDA = 2, MTB_ERR_UNSUPPORTED = 3, MTB_ERR_WORKSPACE = 4, MTB_ERR_DEVICE = 5 };

/* ---- runtime (replaces check_cuda_errors, mytorch/backends/cuda/env.py:26-38) ---- */
const char* mtb_last_error(void);
int mtb_version(void);
int mtb_device_check(void); /* MTB_OK iff the current device is compute capability 10.x */
/* Synchronises the device and reports (then clears) the status word of the tensor-core kernels:
 * 0 = fine, otherwise a bounded in-kernel wait ran out and that kernel exited without finishing.
 * No counterpart in the reference (its kernels have no waits). status_out is a HOST pointer. */
int mtb_tc_status(int* status_out);
/* Self-test of that give-up path (no counterpart in the reference): one CTA allocates tensor memory and
 * waits at most limit_cycles (1..2e8 SM cycles, i.e. at most ~0.1 s) on an mbarrier that nothing completes;
 * the wait runs out, `code` (non-zero) lands in the status word, tensor memory is freed and the kernel
 * returns.  Nothing traps; the context stays usable. */
int mtb_tc_wait_selftest(long long limit_cycles, int code, void* stream);

/* ---- device memory, copies, streams, events, graphs (replace the reference's runtime layer:
 *      CudaMemory / allocate_memory / transfer_memory, mytorch/backends/cuda/env.py:524-580; the size-keyed
 *      caching allocator, mytorch/backends/cuda/memory_allocator.py:16-51; stream handling, env.py:61-94) ----
 * mtb_malloc serves the current device from a pool of freed blocks keyed by size (a step that repeats its
 * allocation pattern gets the same addresses again and never reaches the driver); it returns NULL on failure.
 * The pool does no stream tracking: memory used on another stream than the one its owner computes on must be
 * kept alive until that stream is done.  Between mtb_graph_begin_capture and mtb_graph_end_capture work
 * enqueued on `stream` is recorded instead of run, and every block handed out belongs to the graph until
 * mtb_graph_destroy: it can be reused inside the capture but never by anything outside it. */
void* mtb_malloc(long long nbytes);
int mtb_free(void* ptr);
long long mtb_pool_reserved_bytes(void);
long long mtb_pool_in_use_bytes(void);
int mtb_pool_trim(void);
int mtb_set_device(int device);
int mtb_get_device(int* device);              /* HOST out */
int mtb_device_count(int* count);             /* HOST out */
int mtb_device_synchronize(void);
int mtb_mem_get_info(long long* free_bytes, long long* total_bytes); /* HOST out */
int mtb_memcpy_h2d_async(void* dst, const void* src_host, long long nbytes, void* stream);
int mtb_memcpy_d2h_async(void* dst_host, const void* src, long long nbytes, void* stream);
int mtb_memcpy_d2d_async(void* dst, const void* src, long long nbytes, void* stream);
int mtb_memset_async(void* dst, int value, long long nbytes, void* stream);
void* mtb_host_alloc_pinned(long long nbytes);
int mtb_host_free_pinned(void* ptr);
void* mtb_stream_create(void);
int mtb_stream_destroy(void* stream);
int mtb_stream_synchronize(void* stream);
int mtb_stream_wait_event(void* stream, void* event);
void* mtb_event_create(int timing);
int mtb_event_destroy(void* event);
int mtb_event_record(void* event, void* stream);
int mtb_event_synchronize(void* event);
int mtb_event_elapsed_ms(void* start, void* end, float* ms); /* HOST out */
int mtb_graph_begin_capture(void* stream);
int mtb_graph_end_capture(void* stream, void** graph_exec_out); /* HOST out */
int mtb_graph_launch(void* graph_exec, void* stream);
int mtb_graph_destroy(void* graph_exec);

/* ---- convolution (replaces ConvForwardImplicitGEMM_float32 / ConvBackwardImplicitGEMM_float32,
 *      mytorch/native/cuda/conv.cu/source.cu:419-443 and :445-483, called from
 *      mytorch/backends/cuda/ops/conv.py:9-90) ---- */
long long mtb_conv2d_workspace_bytes(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout);
/* y[N,OH,OW,Cout] = conv(x[N,H,W,Cin], wt[Cout,KH,KW,Cin]) + bias (bias may be NULL); relu != 0 clamps at 0.
 * workspace (mtb_conv2d_workspace_bytes(); may be NULL): lets a layer with too few output tiles to fill the
 * GPU split its reduction across CTAs; the partials are added in a fixed order, results are reproducible. */
int mtb_conv2d_forward_f32(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* x,
                           const float* wt, const float* bias, float* y, int relu, void* workspace, long long workspace_bytes, void* stream);
/* The same forward pass for a convolution whose output feeds a BatchNorm layer: where the kernel family
 * allows, the epilogue also reduces per-channel batch statistics of y from the accumulator rows it
 * already holds, so BatchNorm's own statistics pass (a full re-read of y) can be skipped.  stats: room
 * for mtb_conv2d_stats_max_rows() * 3 * cout floats.  *stats_rows (HOST pointer) receives the number of
 * partial rows [row][3][cout] = (count, mean, M2) written, or 0 when this shape produced none (run the
 * ordinary BatchNorm forward then).  Fuses the seam between mytorch/nn/conv.py:71 and
 * mytorch/nn/batch_norm.py:123-135; no counterpart in the reference. */
int mtb_conv2d_stats_max_rows(void);
int mtb_conv2d_forward_stats_f32(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* x,
                                 const float* wt, const float* bias, float* y, int relu, float* stats, int* stats_rows, void* workspace,
                                 long long workspace_bytes, void* stream);
/* dx[N,H,W,Cin]: every element is written (zeros where no window reaches); no atomics */
int mtb_conv2d_dgrad_f32(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* dy,
                         const float* wt, float* dx, void* workspace, long long workspace_bytes, void* stream);
/* dx = data gradient + addend (addend: same shape as dx, not aliasing it): gradient accumulation for
 * a tensor with a second consumer, fused into the convolution's epilogue where the kernel allows.
 * Where mtb_conv2d_dgrad_accumulates_in_place answers 1 (strided convolutions whose filter is smaller than
 * the stride, e.g. the 1x1 / stride-2 shortcut of a residual stage), addend == dx is allowed and means
 * dx += data gradient: only the pixels a filter tap reaches are touched.
 * No counterpart in the reference, whose tape adds the two gradients with a separate `add`
 * (mytorch/autograd.py:160-170). */
int mtb_conv2d_dgrad_add_f32(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* dy,
                             const float* wt, const float* addend, float* dx, void* workspace, long long workspace_bytes, void* stream);
int mtb_conv2d_dgrad_accumulates_in_place(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout,
                                          const float* dy, const float* wt, const float* dx);
/* Introspection, host code only (works without a GPU): which kernel family forward / dgrad / wgrad
 * would take for this shape and how the row-staged kernels lay out shared and tensor memory.
 * out: 25 ints, see the definition in csrc/tc_kernels.cu.  No counterpart in the reference. */
int mtb_conv2d_plan_f32(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, int* out);
/* dw[Cout,KH,KW,Cin]; split-K partials go to workspace and are summed in a fixed order */
int mtb_conv2d_wgrad_f32(int n, int cin, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, int cout, const float* x,
                         const float* dy, float* dw, void* workspace, long long workspace_bytes, void* stream);

/* ---- dense GEMM for Linear / mm (replaces the cublasLtMatmul call site,
 *      mytorch/backends/cuda/ops/mm.py:10-128, and the permute that materialises W^T,
 *      mytorch/nn/linear.py:62) ----
 * C[M,N] = op(A) op(B) (+ bias[N]) (relu). A is [M,K] (trans_a 0) or [K,M]; B is [K,N] (trans_b 0) or [N,K]. */
int mtb_gemm_f32(int m, int n, int k, const float* a, int trans_a, const float* b, int trans_b, const float* bias, int relu, float* c,
                 void* stream);

/* ---- BatchNorm2d (replaces batch_norm2d_reference_<dt> and its backward,
 *      mytorch/native/cuda/batch_norm.cu/source.cu:134-166 and :269-289) ---- */
long long mtb_batch_norm2d_workspace_bytes(int n, int c, int h, int w);
int mtb_batch_norm2d_forward_f32(int n, int c, int h, int w, const float* x, const float* gamma, const float* beta, double eps, int training,
                                 double momentum, float* running_mean, float* running_var, float* y, float* mean, float* var, int relu,
                                 void* workspace, long long workspace_bytes, void* stream);
/* training-mode forward from statistics partials prepared by mtb_conv2d_forward_stats_f32 (stats_rows > 0) */
int mtb_batch_norm2d_forward_prestats_f32(int n, int c, int h, int w, const float* x, const float* gamma, const float* beta, double eps,
                                          double momentum, float* running_mean, float* running_var, float* y, float* mean, float* var,
                                          int relu, const float* stats, int stats_rows, void* workspace, long long workspace_bytes, void* stream);
/* y = max(0, batch_norm(x) + residual): BatchNorm, shortcut addition and ReLU of a residual block's tail in
 * one normalise pass (the reference runs batch_norm2d, add_reference and relu_reference:
 * mytorch/nn/batch_norm.py:123-135, mytorch/tensor.py:292-300, mytorch/nn/relu.py:5-10).  stats / stats_rows as
 * in the prestats variant, or NULL / 0.  Backward recomputes the ReLU mask from x, the statistics and
 * residual; dresidual receives the masked upstream gradient (the gradient of the added tensor). */
int mtb_batch_norm2d_add_relu_forward_f32(int n, int c, int h, int w, const float* x, const float* residual, const float* gamma,
                                          const float* beta, double eps, int training, double momentum, float* running_mean,
                                          float* running_var, float* y, float* mean, float* var, const float* stats, int stats_rows,
                                          void* workspace, long long workspace_bytes, void* stream);
int mtb_batch_norm2d_add_relu_backward_f32(int n, int c, int h, int w, const float* dy, const float* mean, const float* var, const float* x,
                                           const float* residual, const float* gamma, const float* beta, double eps, float* dx,
                                           float* dresidual, float* dgamma, float* dbeta, void* workspace, long long workspace_bytes,
                                           void* stream);
/* relu != 0 in forward fuses max(0, .) into the normalise pass; the same flag in backward masks dy where
 * gamma*xhat + beta < 0 (recomputed, so the ReLU output need not be kept).  beta may be NULL (= 0). */
int mtb_batch_norm2d_backward_f32(int n, int c, int h, int w, const float* dy, const float* mean, const float* var, const float* x,
                                  const float* gamma, const float* beta, double eps, int relu, float* dx, float* dgamma, float* dbeta,
                                  void* workspace, long long workspace_bytes, void* stream);

/* ---- MaxPool2d (replaces max_pool2d_reference / max_pool2d_backward_reference,
 *      mytorch/native/cuda/pool_ops.cu/1.template:5-52 and 2.template:5-50) ----
 * tiemask: uint16 per output element, bit kh*KW+kw set where the window element equals the
 * maximum (padding counts as 0); lowest set bit = argmax. Needs KH*KW <= 16, may be NULL. */
int mtb_max_pool2d_forward_f32(int n, int c, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, const float* x, float* y,
                               unsigned short* tiemask, void* stream);
/* pass tiemask, or out and x (the equality is then recomputed, as the reference does) */
int mtb_max_pool2d_backward_f32(int n, int c, int h, int w, int kh, int kw, int sh, int sw, int ph, int pw, const float* dy,
                                const unsigned short* tiemask, const float* out, const float* x, float* dx, void* stream);
int mtb_max_pool2d_argmax_u8(const unsigned short* tiemask, unsigned char* argmax, long long n, void* stream);

/* ---- elementwise (replaces relu_reference / relu_backward_reference / fill_reference,
 *      mytorch/native/cuda/elementwise_ops.cu/vars.json:2-21, and the same-shape and bias cases of
 *      add_reference, mytorch/native/cuda/broadcast_binary_ops.cu/1.template) ---- */
int mtb_fill_f32(float* x, long long n, float value, void* stream);
int mtb_copy_f32(float* dst, const float* src, long long n, void* stream);
int mtb_scale_f32(float* dst, const float* src, long long n, float scale, void* stream);
int mtb_relu_forward_f32(const float* x, float* y, long long n, void* stream);
int mtb_relu_backward_f32(const float* dy, const float* x, float* dx, long long n, void* stream); /* blocks only x < 0 */
int mtb_add_f32(const float* x, const float* y, float* z, long long n, float alpha, void* stream); /* z = x + alpha*y */
int mtb_mul_f32(const float* x, const float* y, float* z, long long n, void* stream);
/* residual add + ReLU in one pass (the reference runs add_reference then relu_reference), and its gradient
 * g = (x + y < 0) ? 0 : dy, which is the gradient for both operands */
int mtb_add_relu_f32(const float* x, const float* y, float* z, long long n, void* stream);
int mtb_add_relu_backward_f32(const float* dy, const float* x, const float* y, float* g, long long n, void* stream);
int mtb_add_bias_rows_f32(const float* x, const float* bias, float* y, long long rows, int cols, float alpha, void* stream);
/* general broadcast op over <= 6 logical dims; shape/strides are HOST arrays (strides in elements, 0 broadcasts);
 * op: 0 add, 1 sub, 2 mul, 3 div, 4 pow, 5 alpha*x (replaces broadcast(), broadcast_utils.cuh:4-37, and
 * permute_reference, mytorch/native/cuda/basic_ops.cu/source.cu:5-41) */
int mtb_binary_strided_f32(int op, int ndim, const long long* shape, const long long* x_strides, const long long* y_strides,
                           const long long* z_strides, const float* x, const float* y, float* z, float alpha, void* stream);
/* dst[rows][c_dst] from src[rows][c_src]: extra channels are zero, surplus channels are dropped (channel
 * padding of the image stem for the tensor-core convolution; no counterpart in the reference) */
int mtb_resize_channels_f32(const float* src, float* dst, long long rows, int c_src, int c_dst, void* stream);
int mtb_nchw_to_nhwc_f32(const float* src, float* dst, int n, int c, int h, int w, void* stream);
int mtb_nhwc_to_nchw_f32(const float* src, float* dst, int n, int c, int h, int w, void* stream);
/* kind: 0 int32->int64, 1 int64->float32, 2 float32->int64, 3 int8->float32 (replaces cast_reference, cast.cu/source.cu:5-14) */
int mtb_cast(int kind, const void* src, void* dst, long long n, void* stream);

/* ---- reductions (replace sum_scale_reference / _backward, mytorch/native/cuda/reduce_ops.cu/1.template, 2.template,
 *      and ReduceTemplate, reduce_utils.cuh:24-62) ---- */
long long mtb_colsum_workspace_bytes(int c);
int mtb_colsum_f32(const float* a, long long rows, int c, float scale, float* out, void* workspace, long long workspace_bytes, void* stream);
/* The same column sum for callers that can neither pass nor allocate scratch (an embedder whose arena
 * owns all device memory, a step loop where driver allocations are off limits).  It has no counterpart
 * in the reference.  Partials live in a 1 MiB device array inside the library; c <= 1024, otherwise
 * MTB_ERR_UNSUPPORTED.  The call itself allocates nothing.  The first call on each device resolves the
 * array's address; with lazy module loading the driver may load the library's device code and back
 * the array at that moment, so make one warm-up call per device before the stretch of code in which
 * nothing may allocate, and before any stream capture.  Calls share the array: do not let two of
 * them overlap on one GPU. */
int mtb_colsum_noalloc_f32(const float* a, long long rows, int c, float scale, float* out, void* stream);
int mtb_nhwc_spatial_sum_f32(const float* x, float* y, int n, int c, int hw, float scale, void* stream);
int mtb_nhwc_spatial_bcast_f32(const float* dy, float* dx, int n, int c, int hw, float scale, void* stream);
int mtb_sum_strided_f32(const float* x, float* y, int nkept, const long long* kept_shape, const long long* kept_strides, int nred,
                        const long long* red_shape, const long long* red_strides, float scale, void* stream);

/* ---- max with indices, equality (replace MaxReference_<dt> / max_backward_reference_<dt>, mytorch/backends/cuda/ops/max.py:10-120,
 *      and the eq kernel, mytorch/backends/cuda/ops/eq.py:9).  Shapes and strides are HOST arrays, strides in elements. ---- */
int mtb_max_strided_f32(const float* x, float* y, long long* idx, int nkept, const long long* kept_shape, const long long* kept_strides,
                        long long red_len, long long red_stride, void* stream);
int mtb_max_backward_f32(const float* dy, const long long* idx, float* dx, long long dx_elems, int nkept, const long long* kept_shape,
                         const long long* kept_strides, long long red_stride, void* stream);
/* out: int8, dense in logical order; kind 0 float32, 1 int64 */
int mtb_eq_strided(int kind, int ndim, const long long* shape, const long long* x_strides, const long long* y_strides, const void* x,
                   const void* y, signed char* out, void* stream);

/* ---- softmax cross-entropy (replaces cross_entropy_reference / _backward_reference,
 *      mytorch/native/cuda/cross_entropy.cu/source.cu:6-99); target is int64 ---- */
long long mtb_cross_entropy_workspace_bytes(int batch);
int mtb_cross_entropy_forward_f32(int batch, int classes, const float* logits, const long long* target, float* loss, void* workspace,
                                  long long workspace_bytes, void* stream);
int mtb_cross_entropy_backward_f32(int batch, int classes, const float* logits, const long long* target, const float* dy, float* dlogits,
                                   void* stream);

/* ---- SGD (replaces sgd_reference, mytorch/native/cuda/optim.cu/source.cu:3-19, launched per parameter from
 *      mytorch/backends/cuda/ops/sgd.py:8-35) ---- */
int mtb_sgd_f32(float* param, const float* grad, float* momentum_buffer, long long n, int is_first, double lr, double weight_decay,
                double momentum, double dampening, int nesterov, int maximize, double grad_scale, void* stream);
/* params/grads/momentum_buffers/sizes/is_first are HOST arrays of length count */
int mtb_sgd_multi_f32(int count, float* const* params, const float* const* grads, float* const* momentum_buffers, const long long* sizes,
                      const int* is_first, double lr, double weight_decay, double momentum, double dampening, int nesterov, int maximize,
                      double grad_scale, void* stream);
/* gather gradient tensors into one flat all-reduce buffer (no counterpart: the reference has no
 * distributed code); srcs/offsets/sizes are HOST arrays */
int mtb_pack_scale_f32(int count, const float* const* srcs, const long long* offsets, const long long* sizes, float* dst, double scale,
                       void* stream);

#ifdef __cplusplus
}
#endif
#endif
