/*
 * cnet_b200 — C ABI of the B200 (sm_100a) device path of CNet's batched complex
 * training step.
 *
 * Every entry point is `extern "C"`, takes raw device pointers to fp32 planes
 * (the reference's split real_/imag_ storage, impl/vars.h:16-46), explicit
 * dimensions and the CUDA stream to launch on (passed as void*; NULL = legacy
 * default stream), and returns an int status: 0 = ok, negative = error class
 * below; the message is available from cnb_last_error().  Nothing here calls
 * exit(), abort() or traps; nothing blocks except cnb_sync and cnb_d2h.
 *
 * Layout conventions (row-major, sample-major):
 *   activations / activation gradients : two planes [B, N]   (re, im)
 *   Linear weights                     : two planes [out, in] exactly as inside the
 *                                        reference's Linear block (impl/linear.h:58)
 *   broadcast vectors (Hadamard h)     : two planes [N]
 *   embedding table                    : two planes [V, D]
 * Only the dL/dz* gradient chain is stored; dL/dz is its conjugate for the
 * real-valued losses of this path (impl/crossent.h:95-101).
 *
 * Each declaration cites the reference interface it replaces (file:line within
 * the reference project).
 */
#ifndef CNET_B200_H_
#define CNET_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------ status */
#define CNB_OK            0
#define CNB_ERR_ARG      -1   /* bad dimension / null pointer / misalignment      */
#define CNB_ERR_ARENA    -2   /* device arena exhausted                           */
#define CNB_ERR_CUDA     -3   /* a CUDA runtime / driver call failed              */
#define CNB_ERR_DEVICE   -4   /* a kernel reported an error word (bounded wait)   */
#define CNB_ERR_UNSUPPORTED -5

typedef struct cnb_ctx cnb_ctx;

/* Replaces gpuErrchk's print-and-exit (gpu/kernels.h:18-28) and the allocator's
 * CHECK macros (gpu/allocator.h:19-28): last error message of the calling thread. */
const char* cnb_last_error(void);

/* ----------------------------------------------------------- context, arena
 * Replaces GpuHelper (gpu/allocator.h:97-408) and the per-call cudaMalloc /
 * cudaFree of scratch in gpu/reduce.cpp:382-393, 581-604 and
 * gpu/reducegrad.cpp:309-322: ONE device block, bump sub-allocation (256-byte
 * aligned), no allocation on the step path. */
int cnb_create(int device, size_t arena_bytes, cnb_ctx** out);
/* Same, over memory the caller owns (e.g. a framework tensor); never freed here. */
int cnb_create_external(int device, void* arena, size_t arena_bytes, cnb_ctx** out);
int cnb_destroy(cnb_ctx* ctx);
int cnb_alloc(cnb_ctx* ctx, size_t bytes, void** out);        /* GpuHelper::allocate, gpu/allocator.h:121-137 */
int cnb_reset(cnb_ctx* ctx);                                  /* GpuHelper::deallocate, gpu/allocator.h:330-346 */
size_t cnb_arena_used(const cnb_ctx* ctx);
size_t cnb_arena_size(const cnb_ctx* ctx);
int cnb_device_info(int device, int* sm_count, int* cc_major, int* cc_minor,
                    size_t* total_mem);                       /* PrintInfo, gpu/gpu_func.cpp:52-77 */

/* float_copy_to_gpu / float_copy_from_gpu / int_copy_to_gpu (gpu/allocator.h:308-322, 375-388).
 * Asynchronous on `stream` when the host buffer is pinned; cnb_d2h synchronises the stream. */
int cnb_h2d(cnb_ctx* ctx, void* dst_dev, const void* src_host, size_t bytes, void* stream);
int cnb_d2h(cnb_ctx* ctx, void* dst_host, const void* src_dev, size_t bytes, void* stream);
int cnb_memset0(cnb_ctx* ctx, void* dst_dev, size_t bytes, void* stream);  /* gpu_zero_gradients, gpu/kernels.cpp:444-469 */
int cnb_sync(cnb_ctx* ctx, void* stream);                     /* cudaDeviceSynchronize after every launch, gpu/kernels.cpp:45-46 */
/* Reads and clears the device error word kernels with bounded waits may set. */
int cnb_check_device_status(cnb_ctx* ctx, void* stream);

/* ------------------------------------------------------------ complex Linear
 * Y[b,o] = sum_i X[b,i] * W[o,i] (+ R[b,o] if res_* != NULL: the Residual add fused).
 * Replaces LinearGpu::gpu_linear_forward (gpu/reduce.h:57, gpu/reduce.cpp:581-604:
 * reducing_kernel + new_l_kernel_end) and, with res_*, gpu_residual_forward
 * (gpu/kernels.cpp:145-166).  CPU semantics: impl/linear.h:51-71. */
int cnb_linear_fwd(cnb_ctx* ctx, const float* x_re, const float* x_im,
                   const float* w_re, const float* w_im,
                   const float* res_re, const float* res_im,
                   float* y_re, float* y_im, int B, int in, int out, void* stream);
/* dX*[b,i] (+)= sum_o G*[b,o] * conj(W[o,i]).  Replaces the activation half of
 * LinearGpu::gpu_linear_backward (gpu/reduce.h:59, gpu/reducegrad.cpp:309-322,
 * 77-155, 216-245).  CPU semantics: impl/linear.h:73-93. */
int cnb_linear_bwd_x(cnb_ctx* ctx, const float* g_re, const float* g_im,
                     const float* w_re, const float* w_im,
                     float* dx_re, float* dx_im, int B, int in, int out,
                     int accumulate, void* stream);
/* dW*[o,i] (+)= sum_b G*[b,o] * conj(X[b,i]).  Replaces the atomicAdd side effect of
 * Fdz (gpu/reducegrad.cpp:20-44) and gpu_grad_from_clones (gpu/kernels.cpp:566-598).
 * CPU semantics: impl/linear.h:95-106 summed over samples by impl/cinput.h:54-65. */
int cnb_linear_bwd_w(cnb_ctx* ctx, const float* g_re, const float* g_im,
                     const float* x_re, const float* x_im,
                     float* dw_re, float* dw_im, int B, int in, int out,
                     int accumulate, void* stream);
/* Scratch bytes the three products of a Linear(B, in, out) may take from the arena (operand
 * split buffers of the tensor-core GEMM), and a way to reserve the step's maximum up front
 * so that no call on the step path grows the scratch region.  Replace the per-call cudaMalloc of
 * gpu/reduce.cpp:594-598 and gpu/reducegrad.cpp:309-322. */
size_t cnb_linear_workspace(int B, int in, int out);
int cnb_reserve_scratch(cnb_ctx* ctx, size_t bytes);
/* The same three products on operands the caller has split once: a tensor
 * used by several products (X by forward and dW*, G by dX* and dW*, W by forward and dX*) is then
 * read by the tensor-core GEMM in place, row-major for one product and as the transposed operand
 * for the other.  The split of x: hi = x cut to TF32, lo = x - hi; the product takes hi.hi on the TF32
 * pipe and the cross terms hi.lo + lo.hi on the BF16 pipe from bf16 roundings of hi and lo.  A `split`
 * buffer holds cnb_split_floats(n) = 4 np floats, np = n rounded up to 64: [0, np) hi of the real plane,
 * [np, 2 np) hi of the imaginary plane (fp32), then as bf16: np values bf16(hi_re), np of bf16(hi_im),
 * np of bf16(lo_re), np of bf16(lo_im).
 * Eligible when cnb_linear_split_ok (all dims >= 64, in and out multiples of 64).  Same reference
 * call sites as cnb_linear_fwd / _bwd_x / _bwd_w above. */
/* The schedule cnb_linear_*_split / the tensor-core products would choose for an M x N x K product on a device
 * of sm_count SMs of which the launch may fill sm_limit (0: all): host arithmetic only, no device needed (no
 * reference counterpart; for tests and tuning).  out8 = {CTA pairs (cta_group::2) or not, CTAs of the launch,
 * CTAs per cluster, k-blocks per run, whole tiles per CTA before the shared remainder, k-segments per tile
 * (capped chains), tiles summed with atomics or not, first row of the output that atomics touch}. */
int cnb_gemm_schedule(int M, int N, int K, int accumulate, int sm_count, int sm_limit, int* out8);
size_t cnb_split_floats(size_t n);
int cnb_split_planes(cnb_ctx* ctx, const float* re, const float* im, size_t n, float* split, void* stream);
int cnb_linear_split_ok(int B, int in, int out);
int cnb_linear_fwd_split(cnb_ctx* ctx, const float* x_split, const float* w_split,
                         const float* res_re, const float* res_im,
                         float* y_re, float* y_im, int B, int in, int out, void* stream);
int cnb_linear_bwd_x_split(cnb_ctx* ctx, const float* g_split, const float* w_split,
                           float* dx_re, float* dx_im, int B, int in, int out, int accumulate, void* stream);
int cnb_linear_bwd_w_split(cnb_ctx* ctx, const float* g_split, const float* x_split,
                           float* dw_re, float* dw_im, int B, int in, int out, int accumulate, void* stream);
/* The tensor-core GEMM is persistent (one CTA per SM, all shared memory).  max_ctas > 0 caps its
 * grid so that the remaining SMs stay free for kernels that must run beside it (the gradient
 * all-reduce of a data-parallel job); 0 restores the full grid.  No reference counterpart. */
int cnb_set_gemm_sm_limit(cnb_ctx* ctx, int max_ctas);
/* Which GEMM engine the last cnb_linear_* call on this thread used:
 * 1 = tcgen05 tensor-core tiles (split operands: TF32 hi.hi + BF16 cross terms), 2 = fp32 SIMT tiles (ragged shapes),
 * 4 = skinny fp32 kernels (out <= 16, HBM-bound). */
int cnb_last_gemm_engine(void);

/* ---------------------------------------------------------------- FourierTrans
 * Y[b,p] = N^-1/2 sum_q X[b,q] e^{-2 pi i pq/N}.  Replaces FourierGpu::gpu_fft_forward
 * (gpu/reduce.h:79, gpu/reduce.cpp:382-393: dense one-thread-per-term DFT) and
 * u_roots_allocate_and_copy_on_gpu (gpu/allocator.h:389-407).  CPU: impl/ft.h:37-55. */
int cnb_dft_fwd(cnb_ctx* ctx, const float* x_re, const float* x_im,
                float* y_re, float* y_im, int B, int N, void* stream);
/* dX*[b,q] (+)= N^-1/2 sum_p G*[b,p] e^{+2 pi i pq/N}.  Replaces
 * FourierGpu::gpu_fft_backward (gpu/reduce.h:85, gpu/reducegrad.cpp:324-336).
 * CPU: impl/ft.h:57-80. */
int cnb_dft_bwd(cnb_ctx* ctx, const float* g_re, const float* g_im,
                float* dx_re, float* dx_im, int B, int N, int accumulate, void* stream);
/* FourierTrans -> Hadamard(shared h) -> CGelu in one pass over the row (N = 256, 1024, 4096, see
 * cnb_dft_fused_ok): u = DFT(x) is kept for the backward, y = gelu(u o h), optionally with the
 * operand split of y for the Linear that follows; y_re = y_im = NULL is allowed when y_split
 * is given (hi + l16 of the split is y to 2^-19, all the product sees of it, so a caller that only feeds the
 * Linear need not store y twice).
 * The Hadamard product a = u o h is not stored: cnb_hadamard_gelu_bwd recomputes it when a_re == NULL.  Same reference kernels as
 * cnb_dft_fwd + cnb_hadamard_gelu_fwd. */
int cnb_dft_fused_ok(int N);
int cnb_dft_hadamard_gelu_fwd(cnb_ctx* ctx, const float* x_re, const float* x_im,
                              const float* h_re, const float* h_im,
                              float* u_re, float* u_im, float* y_re, float* y_im,
                              float* y_split, int B, int N, void* stream);
/* TriangFourier: Y[b,p] = N^-1/2 sum_{q <= p} X[b,q] e^{-2 pi i pq/N} and its backward
 * dX*[b,q] (+)= N^-1/2 sum_{p >= q} G*[b,p] e^{+2 pi i pq/N}: the complex GEMM against the
 * lower-triangular twiddle matrix.  Replaces TrianFourierGpu::gpu_T_fft_forward / _backward
 * (gpu/reduce.h:101-107, gpu/reduce.cpp:37-46, gpu/reducegrad.cpp:49-56).  CPU: impl/ft.h:139-188. */
int cnb_tdft_fwd(cnb_ctx* ctx, const float* x_re, const float* x_im,
                 float* y_re, float* y_im, int B, int N, void* stream);
int cnb_tdft_bwd(cnb_ctx* ctx, const float* g_re, const float* g_im,
                 float* dx_re, float* dx_im, int B, int N, int accumulate, void* stream);
/* N = 256, 1024, 4096 run as a shared-memory FFT (one read + one write of the tensor); any other
 * N, or every N after cnb_set_dft_engine(ctx, 1), as a complex GEMM against the twiddle matrix.
 * cnb_last_gemm_engine() reports 3 after an FFT-kernel call. */
int cnb_set_dft_engine(cnb_ctx* ctx, int force_gemm);

/* --------------------------------------------------------- element-wise layers
 * Hadamard y = u o v; v is one vector [N] shared by the batch (v_batched = 0) or [B,N].
 * Replaces HadamardGpu::gpu_hadamard_forward (gpu/kernels.h:217, gpu/kernels.cpp:204-241).
 * CPU: impl/hadamard.h:34-44. */
int cnb_hadamard_fwd(cnb_ctx* ctx, const float* u_re, const float* u_im,
                     const float* v_re, const float* v_im, int v_batched,
                     float* y_re, float* y_im, int B, int N, void* stream);
/* du* (+)= g* o conj(v); dv* (+)= g* o conj(u), summed over the batch when v is shared
 * (deterministic two-stage column reduction; scratch from the arena).  du_* or dv_* may
 * be NULL to skip that operand.  Replaces gpu_hadamard_backward (gpu/kernels.cpp:243-274)
 * + gpu_input_backward / gpu_grad_from_clones for the shared vector.  CPU: impl/hadamard.h:46-68. */
int cnb_hadamard_bwd(cnb_ctx* ctx, const float* g_re, const float* g_im,
                     const float* u_re, const float* u_im,
                     const float* v_re, const float* v_im, int v_batched,
                     float* du_re, float* du_im, int accumulate_u,
                     float* dv_re, float* dv_im, int accumulate_v,
                     int B, int N, void* stream);
/* Allocation-free form of cnb_hadamard_bwd for a shared v (no counterpart in the reference,
 * which allocates scratch per call).  For callers that must not allocate device memory when
 * they call in — a host whose own pool already owns the whole device, or a loop that cannot
 * take the device-wide stall of cudaMalloc/cudaFree: no context, no arena; the column-reduction
 * partials live in a 2 MiB array built into the library (per GPU that loads it, until exit).
 * Limit: N <= CNB_STATIC_MAX_N, else CNB_ERR_ARG with a message.  The first call on a device
 * looks up the array's device address (make that call before any stream capture starts).
 * With CUDA's lazy module loading that first call is also when the driver materialises the
 * module's data segment on that device (the 2 MiB array included): "allocates nothing" holds
 * from the second call on a device onwards.  The buffers must live on the current device
 * (checked; CNB_ERR_ARG otherwise).
 * All calls share the one array, so two calls that overlap on the GPU (different streams)
 * race; contents from the previous call are never read. */
#define CNB_STATIC_MAX_N 4096
int cnb_hadamard_bwd_static(const float* g_re, const float* g_im,
                            const float* u_re, const float* u_im,
                            const float* v_re, const float* v_im,
                            float* du_re, float* du_im, int accumulate_u,
                            float* dv_re, float* dv_im, int accumulate_v,
                            int B, int N, void* stream);
/* CGelu: y = gelu(re) + i gelu(im) (tanh form).  Replaces GeluGpu::gpu_gelu_forward /
 * gpu_gelu_backward (gpu/kernels.h:262-268, gpu/kernels.cpp:276-360).  CPU: impl/relu.h:119-168.
 * Backward: dz* (+)= conj(g*) (dx-dy) + g* (dx+dy), dx = gelu'(re)/2, dy = gelu'(im)/2. */
int cnb_gelu_fwd(cnb_ctx* ctx, const float* z_re, const float* z_im,
                 float* y_re, float* y_im, size_t n, void* stream);
int cnb_gelu_bwd(cnb_ctx* ctx, const float* g_re, const float* g_im,
                 const float* z_re, const float* z_im,
                 float* dz_re, float* dz_im, size_t n, int accumulate, void* stream);
/* CRelu: y = z where re > 0 and im > 0, else 0; backward dz* (+)= g* through the same gate.
 * Replaces ReluGpu::gpu_relu_forward / _backward (gpu/kernels.h:284-289, gpu/kernels.cpp:18-87).
 * CPU: impl/relu.h:31-62. */
int cnb_crelu_fwd(cnb_ctx* ctx, const float* z_re, const float* z_im,
                  float* y_re, float* y_im, size_t n, void* stream);
int cnb_crelu_bwd(cnb_ctx* ctx, const float* g_re, const float* g_im,
                  const float* z_re, const float* z_im,
                  float* dz_re, float* dz_im, size_t n, int accumulate, void* stream);
/* Fused Hadamard(shared h) -> CGelu: a = u o h (kept for the backward), y = gelu(a).
 * Same reference kernels as the two above, one pass over HBM. */
int cnb_hadamard_gelu_fwd(cnb_ctx* ctx, const float* u_re, const float* u_im,
                          const float* h_re, const float* h_im,
                          float* a_re, float* a_im, float* y_re, float* y_im,
                          int B, int N, void* stream);
/* Same, and when y_split != NULL also writes the operand split of y
 * (cnb_split_floats(B*N) floats) that cnb_linear_fwd_split / _bwd_w_split consume. */
int cnb_hadamard_gelu_fwd_split(cnb_ctx* ctx, const float* u_re, const float* u_im,
                                const float* h_re, const float* h_im,
                                float* a_re, float* a_im, float* y_re, float* y_im,
                                float* y_split, int B, int N, void* stream);
/* Fused backward of the pair: t = gelu_bwd(g*, a); du* (+)= t o conj(h); dh* (+)= sum_b t o conj(u).
 * a_re == a_im == NULL: a = u o h is recomputed. */
int cnb_hadamard_gelu_bwd(cnb_ctx* ctx, const float* g_re, const float* g_im,
                          const float* a_re, const float* a_im,
                          const float* u_re, const float* u_im,
                          const float* h_re, const float* h_im,
                          float* du_re, float* du_im, int accumulate_u,
                          float* dh_re, float* dh_im, int accumulate_h,
                          int B, int N, void* stream);
/* Residual y = u + v (gpu_residual_forward, gpu/kernels.cpp:145-166; CPU impl/residual.h:40-50);
 * its backward is a pass-through to both operands = cnb_axpy below. */
int cnb_residual_fwd(cnb_ctx* ctx, const float* u_re, const float* u_im,
                     const float* v_re, const float* v_im,
                     float* y_re, float* y_im, size_t n, void* stream);
/* dst = (accumulate ? dst : 0) + src on both planes: gradient pass-through
 * (gpu_residual_backward gpu/kernels.cpp:168-202, gpu_input_backward :120-143). */
int cnb_axpy(cnb_ctx* ctx, const float* src_re, const float* src_im,
             float* dst_re, float* dst_im, size_t n, int accumulate, void* stream);

/* ------------------------------------------------------------ row reductions
 * Reference "SoftMax" = L2 normalisation y = z / max(||z||, 1e-15); inv_norm[b] is kept
 * for the backward.  Replaces SoftMaxGpu::gpu_soft_max_forward (gpu/reduce.h:123,
 * gpu/reduce.cpp:189-230).  CPU: impl/softmax.h:33-59. */
int cnb_softmax_fwd(cnb_ctx* ctx, const float* z_re, const float* z_im,
                    float* y_re, float* y_im, float* inv_norm, int B, int N, void* stream);
/* dz*_i (+)= g*_i / n - z_i / n^3 * Re sum_j g*_j conj(z_j): closed form of the generic
 * Jacobian loop.  Replaces gpu_soft_max_backward (gpu/reduce.h:129,
 * gpu/reducegrad.cpp:10-19, 60-66, 268-286).  CPU: impl/softmax.h:61-73 via impl/cfunc.h:290-325. */
int cnb_softmax_bwd(cnb_ctx* ctx, const float* g_re, const float* g_im,
                    const float* z_re, const float* z_im, const float* inv_norm,
                    float* dz_re, float* dz_im, int B, int N, int accumulate, void* stream);
/* CrossEntropy forward + backward seed in one pass: loss[b] = -log(max(|z_l|^2/S, 1e-15)),
 * S = max(sum|z|^2, 1e-15); dz*_k = z_k/S (k != l), dz*_l = -z_l (S-m)/(m S), m = max(|z_l|^2, 1e-15).
 * dz_* may be NULL (forward only).  Replaces CrossEntropyGpu::gpu_cross_ent_forward / _backward
 * (gpu/reduce.h:150-156, gpu/reduce.cpp:469-530, 609-655).  CPU: impl/crossent.h:50-104. */
int cnb_crossent_fwd_bwd(cnb_ctx* ctx, const float* z_re, const float* z_im,
                         const int32_t* labels, float* loss,
                         float* dz_re, float* dz_im, int B, int M, void* stream);

/* L2Out: loss[b] = sum_k |z_k|^2 and the backward seed dz* = z (dz_* may be NULL).  Replaces
 * L2Gpu::gpu_norm_forward / gpu_norm_backward (gpu/reduce.h:175-181, gpu/reduce.cpp:232-251,
 * 424-467).  CPU: impl/l2out.h:31-57 through CFunc::out_backward (impl/cfunc.h:327-339). */
int cnb_l2out_fwd_bwd(cnb_ctx* ctx, const float* z_re, const float* z_im, float* loss,
                      float* dz_re, float* dz_im, int B, int N, void* stream);

/* ------------------------------------------------------------------ embedding
 * out[b, t*D + d] = table[tok[b,t], d]; tok < 0 (NO_TOKEN, impl/batch.h:11) gives zeros.
 * Replaces EmbeddingGpu::gpu_embedding_forward (gpu/kernels.h:183, gpu/kernels.cpp:362-403).
 * CPU: impl/embed.h:109-131. */
int cnb_embed_fwd(cnb_ctx* ctx, const float* tab_re, const float* tab_im,
                  const int32_t* tokens, float* out_re, float* out_im,
                  int B, int T, int D, int V, void* stream);
/* dtable[tok[b,t], d] += g*[b, t*D + d] (fp32 atomics: order of equal-token sums is not
 * fixed).  Replaces gpu_embedding_backward (gpu/kernels.h:200, gpu/kernels.cpp:405-442).
 * CPU: impl/embed.h:133-148. */
int cnb_embed_bwd(cnb_ctx* ctx, const float* g_re, const float* g_im,
                  const int32_t* tokens, float* dtab_re, float* dtab_im,
                  int B, int T, int D, int V, void* stream);

/* --------------------------------------------------------------------- update
 * w -= lr * g over n floats (re and im planes are just floats here); g is zeroed when
 * zero_grad != 0.  Replaces gpu_update_input (gpu/kernels.h:75, gpu/kernels.cpp:471-492).
 * CPU: impl/cfunc.h:147-152 + impl/cnet.h:413-421. */
int cnb_sgd_update(cnb_ctx* ctx, float* w, float* g, size_t n, float lr, int zero_grad,
                   void* stream);
/* The same update; the floats of [begin, begin + count) of every span (the planes of Linear weights)
 * also leave their operand split (see cnb_split_floats) in hi[i - begin] (fp32), h16[i - begin] and
 * l16[i - begin] (bf16), so the products of the next step need no split pass over the weights.  n, begins and counts are multiples of 4; at most
 * CNB_MAX_SPLIT_SPANS spans.  Same reference call site as cnb_sgd_update. */
#define CNB_MAX_SPLIT_SPANS 48
typedef struct cnb_split_span { size_t begin; size_t count; float* hi; void* h16; void* l16; } cnb_split_span;
int cnb_sgd_update_split(cnb_ctx* ctx, float* w, float* g, size_t n, float lr, int zero_grad,
                         const cnb_split_span* spans, int nspans, void* stream);

/* The reference's momentum-only "Adam": m = beta m + (1 - beta) g; w -= lr m / (1 - beta^(t+1));
 * g = 0.  Replaces gpu_update_adam_input (gpu/kernels.h:77, gpu/kernels.cpp:494-525).
 * CPU: impl/cfunc.h:273-287 + impl/cnet.h:423-431. */
int cnb_adam_update(cnb_ctx* ctx, float* w, float* m, float* g, size_t n, float lr, float beta, int t,
                    void* stream);

/* ------------------------------------------------------------- data parallelism
 * Sum of `count` floats at `local` over the ranks of one NVSwitch domain, in place, by this library's own kernel
 * on symmetric memory (no counterpart in the reference, which is single-GPU; the intra-GPU analogue is
 * gpu_grad_from_clones, gpu/kernels.cpp:566-598).  The caller maps every rank's arena into this process (peer
 * pointers, e.g. torch.distributed symmetric memory or cuMem handles) and, where the platform supports it, binds
 * them to one multicast address; `flags` are CNB_DP_MAX_RANKS zeroed 32-bit words per rank in symmetric memory,
 * `state` is cnb_dp_state_bytes() of zeroed local device memory.  Rank r sums its 1/world slice of the range over
 * all ranks (in the switch with multimem.ld_reduce, else by loads from every peer) and writes it to all ranks.
 * `local` must lie inside the arena, 16-byte aligned, count a multiple of 4 x world.  Every rank must make the
 * same sequence of calls.  Waits on peers are bounded: a missing peer sets the error word read by
 * cnb_check_device_status.  ctas = 0: one CTA per SM (256 threads, no shared memory: they run beside the GEMM's). */
#define CNB_DP_MAX_RANKS 8
typedef struct cnb_dp_peers {
    int rank, world;
    void* multicast_base;                    /* the arena at its multicast address, or NULL */
    void* arena_base[CNB_DP_MAX_RANKS];      /* every rank's arena as mapped in this process; [rank] is the local one */
    size_t arena_bytes;
    void* flags[CNB_DP_MAX_RANKS];           /* every rank's flag block as mapped in this process */
    void* state;                             /* local */
    int ctas;
} cnb_dp_peers;
size_t cnb_dp_state_bytes(void);
int cnb_dp_allreduce(cnb_ctx* ctx, const cnb_dp_peers* peers, float* local, size_t count, void* stream);

/* Number of kernels this library has launched in this process (diagnostics / benches). */
unsigned long long cnb_launch_count(void);

#ifdef __cplusplus
}
#endif
#endif /* CNET_B200_H_ */
