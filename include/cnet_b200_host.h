/*
 * Flat C binding of the host facade (cnet_b200/host/cnet.h) for callers that cannot
 * include C++ — the Python package binds these with ctypes.  One handle = one CNet
 * (gpu/gpu_func.h:41-1113 in the reference).  Every function returns 0 / a positive uid on
 * success and a negative cnb status on failure; cnh_error() gives the message.
 * Host pointers unless said otherwise.
 */
#ifndef CNET_B200_HOST_H_
#define CNET_B200_HOST_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct cnh_net cnh_net;
typedef int (*cnh_bucket_hook)(void* user, float* dev_grads, size_t count, int bucket, int n_buckets);

cnh_net* cnh_create(int device, size_t arena_bytes, void* ext_arena_dev);   /* CNet() + device choice */
void cnh_destroy(cnh_net* net);
/* Device and arena to use (ext_arena_dev != NULL: caller-owned device memory); before cnh_allocate. */
int cnh_set_device(cnh_net* net, int device, size_t arena_bytes, void* ext_arena_dev);
const char* cnh_error(cnh_net* net);
void cnh_clear_error(cnh_net* net);

/* CNet::add(CFunc*, {uids}) (gpu/gpu_func.h:1013-1019).  type = the reference's type id
 * (impl/cnet.h:31-44); (a,b,c): CInput(a) | CEmbedding(dim a, tokens b, vocab c) |
 * FourierTrans(a) | Hadamard(a,a) | CGelu(a) | Linear(in1 a, in2 b) | Residual(a) |
 * SoftMax(a) | CrossEntropy(a) | CRelu(a) | L2Out(a) | TriangFourier(a). */
int cnh_add(cnh_net* net, int type, int a, int b, int c, const int* prev, int nprev);
int cnh_out_size(cnh_net* net, int uid);
int cnh_init_inputs(cnh_net* net, uint64_t seed);                            /* CNet::init_inputs(seed) */
int cnh_set_values(cnh_net* net, int uid, const float* re, const float* im, int len);
int cnh_get_values(cnh_net* net, int uid, float* re, float* im, int len);   /* getInputsFromGpu, one input */
int cnh_get_wgrad(cnh_net* net, int uid, float* re, float* im, int len);
int cnh_set_stream(cnh_net* net, void* stream);
int cnh_set_fusion(cnh_net* net, int on);
int cnh_set_bucket_hook(cnh_net* net, cnh_bucket_hook hook, void* user);
size_t cnh_required_arena(cnh_net* net, int batch);
int cnh_allocate(cnh_net* net, int batch);                                   /* CNet::allocateOnGpu */
/* batchToGpu (gpu/gpu_func.h:368-427): planes [B, n] or tokens [B, T]; labels [B] */
int cnh_upload(cnh_net* net, const float* re, const float* im, const int32_t* tokens,
               const int32_t* labels, int batch);
/* Double-buffered input pipeline (replaces the synchronous per-sample copies of batchToGpu): start the
 * H2D copy of the NEXT batch from pinned host memory on a copy stream; commit = compute stream waits
 * for it and moves it into the input tensors; losses come back asynchronously. */
int cnh_prefetch(cnh_net* net, const float* re, const float* im, const int32_t* tokens,
                 const int32_t* labels, int batch);
int cnh_commit(cnh_net* net);
int cnh_read_losses_async(cnh_net* net, float* pinned_host_out, int n);
int cnh_wait_losses(cnh_net* net);
int cnh_forward(cnh_net* net);                                               /* GpuForward, :645-657 */
int cnh_backward(cnh_net* net);                                              /* gpuBackward, :1096-1101 */
int cnh_backward_label(cnh_net* net, int label);                             /* CNet::backward(label) */
int cnh_update(cnh_net* net, float lr);                                      /* gpuUpdateInputs, :491-495 */
int cnh_adam_update(cnh_net* net, float lr, float beta, int t);              /* CNet::adamUpdate, gpu/gpu_func.h:503-510 */
int cnh_infer(cnh_net* net);                                                 /* ComplexNet::infer, impl/cnet.h:379-389 */
int cnh_get_losses(cnh_net* net, float* out, int n);                         /* getLoss, :906-926 */
int cnh_sync(cnh_net* net);
int cnh_read_output(cnh_net* net, int uid, int what, float* re, float* im); /* testDataFromGpu, :840-862 */
int cnh_grad_arena(cnh_net* net, void** dev_ptr, size_t* count, int* n_buckets);
int cnh_weight_arena(cnh_net* net, void** dev_ptr, size_t* count);
/* CNet::save / CNet::restore (gpu/gpu_func.h:1103-1111) in the reference's ModelSaver byte format
 * (impl/model_saver.h:27, 530-795): files written here load in the reference and vice versa.
 * cnh_restore needs an empty net; the graph can then be inspected and allocated. */
int cnh_save(cnh_net* net, const char* path);
int cnh_restore(cnh_net* net, const char* path);
int cnh_num_funcs(cnh_net* net);
int cnh_uid_at(cnh_net* net, int index);
int cnh_type_of(cnh_net* net, int uid);
int cnh_in_size(cnh_net* net, int uid);
void* cnh_context(cnh_net* net);                                             /* the cnb_ctx* of the net */

/* Data parallelism (no counterpart in the reference, which is single-GPU: gpu/gpu_func.h:38-40; the
 * intra-GPU analogue is gpu_grad_from_clones, gpu/kernels.cpp:566-598).  One rank makes a 128-byte
 * NCCL id, every rank (one per GPU) passes it in after cnh_allocate; cnh_backward then sums every
 * finished gradient bucket over the ranks on a communication stream and cnh_update waits for them.
 * The caller gives cnh_update lr / global_batch. */
int cnh_dp_unique_id(char* out128);
int cnh_dp_init(cnh_net* net, const char* id128, int rank, int nranks);
int cnh_dp_async_error(cnh_net* net);                                        /* 0 = communicator healthy */
/* Sums the whole weight-gradient arena over the ranks now, on the communication stream, and makes the net's
 * stream wait for it: what cnh_backward does bucket by bucket, as one call. */
int cnh_dp_allreduce_grads(cnh_net* net);
/* Data parallelism with this library's own all-reduce kernel on symmetric memory (cnb_dp_allreduce) instead of
 * NCCL: after cnh_allocate on a caller-owned arena that is symmetric memory, pass every rank's arena base as
 * mapped in this process, the multicast address of the arena (or NULL) and one zeroed flag block per rank. */
int cnh_dp_set_symmetric(cnh_net* net, int rank, int world, void* multicast_base, void* const* arena_bases,
                         void* const* flag_blocks, int ctas);
/* Before cnh_allocate (no external arena): take the arena from NCCL's allocator so that cnh_dp_init can
 * register the weights and their gradients as a symmetric window (NCCL then runs its symmetric-memory
 * kernels on the buffers themselves).  cnh_dp_symmetric: 1 once such a window is registered. */
int cnh_dp_use_nccl_arena(cnh_net* net, int on);
int cnh_dp_symmetric(cnh_net* net);
/* CUDA graph of a step: begin; cnh_forward; cnh_backward; cnh_update; end; then cnh_graph_launch
 * replays it on the net's stream (replaces the per-launch cudaDeviceSynchronize cadence of
 * gpu/gpu_func.h:645-681).  Needs a non-default stream (cnh_set_stream). */
int cnh_capture_begin(cnh_net* net);
int cnh_capture_end(cnh_net* net);
int cnh_graph_launch(cnh_net* net);
unsigned long long cnh_graph_kernel_count(cnh_net* net);

/* MnistDataReader (data/data.h:82-165): `count` images / labels of the idx3 / idx1 files read into host memory the
 * way the reference reads them (headers skipped unread, a pixel as a signed char, real = imaginary = that value);
 * cnh_mnist_next_batch fills split planes [batch, 784] and labels [batch], wrapping around at the end like
 * BatchedDataReader::nextBatch (data/data.h:58-68).  NULL / negative on failure. */
void* cnh_mnist_open(const char* image_file, const char* label_file, int count);
void cnh_mnist_close(void* reader);
int cnh_mnist_size(void* reader);
int cnh_mnist_shuffle(void* reader, unsigned seed);
int cnh_mnist_has_next(void* reader, int batch);
int cnh_mnist_next_batch(void* reader, int batch, float* re, float* im, int* labels);

#ifdef __cplusplus
}
#endif
#endif /* CNET_B200_HOST_H_ */
