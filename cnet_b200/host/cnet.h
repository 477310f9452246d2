// Host side of the B200 device path: the reference's plugin contract (CFunc
// forward()/backward(), impl/cfunc.h:47-350) and net API (CNet::add / init_exec_graph /
// forward / backward / updateInputs / allocateOnGpu / gpuForward / gpuBackward /
// gpuUpdateInputs / getLoss, gpu/gpu_func.h:491-501, 906-926, 1013-1101) re-done around a
// real batch dimension instead of one net clone per sample (impl/cnet.h:486-583).
//
// Differences a user of the reference will notice:
//  * a function owns its OUTPUT tensor ([batch, outSize] re/im planes in device memory, or
//    [outSize] for weight CInputs), not a concatenated input block; consumers read their
//    producers' outputs in place, so CInput::forward copies nothing;
//  * only dL/dz* is stored (dL/dz is its conjugate for the real losses of this path);
//  * forward()/backward() launch CUDA kernels through the C ABI (include/cnet_b200.h) on the
//    net's stream; there is no CPU implementation and no fallback;
//  * weights exist once; their dL/dz* accumulates over the batch (and over successive
//    backward passes) until updateInputs, as CInput::backward does (impl/cinput.h:54-65).
#ifndef CNET_B200_HOST_CNET_H_
#define CNET_B200_HOST_CNET_H_

#include <complex>
#include <cstdint>
#include <initializer_list>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "../../include/cnet_b200.h"
#include "dp_nccl.h"

namespace cnet_b200 {

// type ids: the reference's own (impl/cnet.h:31-44)
const int isHadamard = 1, isEmbedding = 2, isLinear = 3, isFourier = 4, isCrossEntropy = 5,
          isResidual = 6, isSoftMax = 7, isInput = 8, isCrelu = 9, isGelu = 10, isL2Out = 11,
          isTrianFourier = 12;
const int NO_TOKEN = -1;   // impl/batch.h:11

// strong ints of the kept constructor signatures (impl/sizes.h:8-56)
class InSize { unsigned v_; public: InSize(int v) : v_(v) {} unsigned value() const { return v_; } };
class OutSize { unsigned v_; public: OutSize(int v) : v_(v) {} unsigned value() const { return v_; } };
class Uid { int v_; public: Uid(int v) : v_(v) {} int value() const { return v_; } };

// Device-resident split planes (impl/vars.h:16-46 without the unused dz planes):
// rows_ x length_ floats per plane, row-major.  Pointers are DEVICE pointers.
struct Vars {
	int length_ = 0;
	int rows_ = 0;
	float* real_ = nullptr;
	float* imag_ = nullptr;
	float* dz_star_real_ = nullptr;
	float* dz_star_imag_ = nullptr;
	size_t count() const { return (size_t) rows_ * length_; }
};

class CNet;

// Host staging of one batch (impl/batch.h:13-209): split re/im sample planes or token ids,
// labels, per-sample losses filled by CNet::getLoss.
class Batch {
	friend class CNet;
protected:
	std::vector<float> losses_;
	std::vector<int> labels_;
	int current_pos_ = 0, batch_size_ = 0, sample_dim_ = 0;
public:
	Batch() {}
	Batch(int batch_size, int sample_dim) : batch_size_(batch_size), sample_dim_(sample_dim) {}
	virtual ~Batch() {}
	int size() const { return batch_size_; }
	int sampleDim() const { return sample_dim_; }
	float loss(int i) const { return losses_.at(i); }
	int label(int i) const { return labels_.at(i); }
	const int* labelsPtr() const { return labels_.data(); }
	int noOfLabels() const { return (int) labels_.size(); }
};

class InputBatch : public Batch {
	std::vector<float> real_data_, imag_data_;
public:
	InputBatch() {}
	InputBatch(int batch_size, int sample_dim) : Batch(batch_size, sample_dim) {}
	void add(const std::vector<std::complex<float> >& sample, int label);   // zero-padded to sampleDim
	void assign(const float* re, const float* im, const int* labels, int batch);  // bulk fill
	const float* realDataPtr() const { return real_data_.data(); }
	const float* imagDataPtr() const { return imag_data_.data(); }
};

class EmbeddingBatch : public Batch {
	std::vector<int> token_;
public:
	EmbeddingBatch() {}
	EmbeddingBatch(int batch_size, int sample_dim) : Batch(batch_size, sample_dim) {}
	void add(const std::vector<int>& sample, int label);                    // padded with NO_TOKEN
	void assign(const int* tokens, const int* labels, int batch);
	const int* tokensPtr() const { return token_.data(); }
	int noOfTokens() const { return (int) token_.size(); }
};

class OutputFunc {                       // impl/cfunc.h:13-30
	bool isMainOutput_ = false;
public:
	virtual ~OutputFunc() {}
	virtual int outputLength() = 0;
	virtual float loss(int sample) = 0;  // loss of sample `sample` of the last forward (device read-back)
	bool isMainOutput() { return isMainOutput_; }
	void setIsMainOutput(bool v) { isMainOutput_ = v; }
};

class InputFunc {                        // impl/cfunc.h:32-45
	bool isMainInput_ = false;
public:
	virtual ~InputFunc() {}
	bool isMainInput() { return isMainInput_; }
	void setIsMainInput(bool v) { isMainInput_ = v; }
};

// The layer contract (impl/cfunc.h:47-350).  forward()/backward() enqueue the layer's
// kernels for the whole batch; errors are recorded on the owning net (CNet::ok()).
class CFunc {
	friend class CNet;
protected:
	int uid_, in_size_, out_size_;
	std::vector<CFunc*> prev_func_, next_func_;   // not owned
	std::vector<int> offset_;
	int depth_ = 0;
	bool is_input_ = false, is_output_ = false;
	int type_ = 0;
	CNet* net_ = nullptr;
	std::vector<float> host_re_, host_im_;        // values of inputs before allocateOnGpu

	cnb_ctx* ctx() const;
	void* stream() const;
	int batch() const;
	void check(int status);
	int accumulate_into(CFunc* producer);          // 0 for the first writer of this backward, then 1
	const Vars& in(int k) const { return prev_func_.at(k)->out_; }
	virtual size_t extraBytes(int batch) const { (void) batch; return 0; }
	virtual void bindExtra(char* mem, int batch) { (void) mem; (void) batch; }
public:
	// device state, set by CNet::allocateOnGpu (public like the reference's gpu_var_, impl/cfunc.h:71)
	Vars out_;
	bool batched_ = true;        // false: one row shared by the batch (weights)
	bool grad_written_ = false;  // has a consumer already written dL/dz* of out_ in this backward?
	const float* value_split_ = nullptr; // value planes are not stored: out = hi + l16 of this split buffer (the value to 2^-19)
	bool grad_transient_ = false; // dL/dz* planes are shared with a Residual operand and accumulated over in place
	bool fused_away_ = false;    // a neighbour's fused kernel does this layer's work

	CFunc(Uid uid, InSize in, OutSize out) : uid_(uid.value()), in_size_(in.value()), out_size_(out.value()) {}
	CFunc(InSize in, OutSize out) : uid_(0), in_size_(in.value()), out_size_(out.value()) {}
	virtual ~CFunc() {}

	virtual CFunc* clone(Uid uid) = 0;
	virtual std::string getName() = 0;
	virtual void forward() = 0;
	// Entries of the layer's Jacobians (impl/cfunc.h:144-145).  The reference's default backward() loops over
	// them per sample on the CPU (impl/cfunc.h:290-325); nothing on the device path calls them: every layer
	// here has a closed-form batched backward() kernel.  They are kept so that a layer written against the
	// reference header still compiles; the built-in layers return NaN ("not used on the device path").
	// A user layer that only supplies these two (and a CPU forward()) is refused by CNet::add unless it
	// says it launches its own kernels (runsOnDevice).
	virtual std::complex<float> dz(int out_indx, int in_indx);
	virtual std::complex<float> dz_star(int out_indx, int in_indx);
	// A layer outside the built-in set returns true once its forward()/backward() enqueue device work on
	// stream() through the C ABI; the default (false) makes CNet::add refuse it.
	virtual bool runsOnDevice() const { return false; }
	virtual void backward() {}
	virtual void backward(int label) { (void) label; backward(); }
	virtual void updateInput(float learningRate);   // w -= lr dz*_w ; dz*_w = 0 (impl/cfunc.h:147-152 + impl/cnet.h:418)
	virtual void init_inputs(uint64_t seed);        // impl/cfunc.h:190-196 distribution, own generator

	int uid() const { return uid_; }
	int outSize() const { return out_size_; }
	int inSize() const { return in_size_; }
	int depth() const { return depth_; }
	int getType() const { return type_; }
	bool isInput() const { return is_input_; }
	bool isOutput() const { return is_output_; }
	const Vars& output() const { return out_; }     // device planes of this function's output
	int no_outputs() const { return (int) next_func_.size(); }
	int no_previous_func() const { return (int) prev_func_.size(); }
	CFunc* next(int i) const { return next_func_.at(i); }
	CFunc* previous(int i) const { return prev_func_.at(i); }
	int offset(int i) const { return offset_.at(i); }
	void addOutput(CFunc* next, int offset);        // impl/cfunc.h:211-224
	virtual int sizeInBytes() const { return 4 * (int) sizeof(float) * out_size_; }
};

class CInput : public CFunc, public InputFunc {     // impl/cinput.h:10-118
public:
	CInput(Uid uid, OutSize n) : CFunc(uid, InSize(n.value()), n) { is_input_ = true; }
	explicit CInput(OutSize n) : CFunc(InSize(n.value()), n) { is_input_ = true; }
	CFunc* clone(Uid uid) override { return new CInput(uid, OutSize(out_size_)); }
	std::string getName() override { return "Input_" + std::to_string(uid_); }
	void forward() override {}          // consumers read the planes in place
	void backward() override {}         // consumers accumulate straight into dz*
};

class CEmbedding : public CFunc, public InputFunc { // impl/embed.h:12-223
	friend class CNet;
	int embedding_dim_, no_embeddings_, no_out_tokens_;
	Vars table_;                        // [V, D] + gradient planes
	int32_t* tokens_ = nullptr;         // device [batch, T]
	size_t extraBytes(int batch) const override;
	void bindExtra(char* mem, int batch) override;
public:
	CEmbedding(Uid uid, int dim, int max_out_tokens, int no_embeddings)
		: CFunc(uid, InSize(no_embeddings * dim), OutSize(max_out_tokens * dim)), embedding_dim_(dim),
		  no_embeddings_(no_embeddings), no_out_tokens_(max_out_tokens) { is_input_ = true; }
	CEmbedding(int dim, int max_out_tokens, int no_embeddings)
		: CFunc(InSize(no_embeddings * dim), OutSize(max_out_tokens * dim)), embedding_dim_(dim),
		  no_embeddings_(no_embeddings), no_out_tokens_(max_out_tokens) { is_input_ = true; }
	int embeddingDim() const { return embedding_dim_; }
	int noEmbeddings() const { return no_embeddings_; }
	int noOutTokens() const { return no_out_tokens_; }
	const Vars& table() const { return table_; }
	int32_t* deviceTokens() const { return tokens_; }
	CFunc* clone(Uid uid) override { return new CEmbedding(uid, embedding_dim_, no_out_tokens_, no_embeddings_); }
	std::string getName() override { return "Embedding " + std::to_string(uid_); }
	void forward() override;
	void backward() override;
	void updateInput(float learningRate) override;
	void init_inputs(uint64_t seed) override;       // impl/embed.h:101-107 distribution
};

class Hadamard;
class FourierTrans : public CFunc {                 // impl/ft.h:11-113
	friend class CNet;
	Hadamard* fused_hg_ = nullptr;                  // FFT epilogue does Hadamard(shared h) -> CGelu
public:
	FourierTrans(Uid uid, InSize n) : CFunc(uid, n, OutSize(n.value())) {}
	explicit FourierTrans(InSize n) : CFunc(n, OutSize(n.value())) {}
	CFunc* clone(Uid uid) override { return new FourierTrans(uid, InSize(in_size_)); }
	std::string getName() override { return "FourierTrans_" + std::to_string(uid_); }
	void forward() override;
	void backward() override;
};

class Hadamard : public CFunc {                     // impl/hadamard.h:11-107
	friend class CNet;
	friend class CGelu;
	friend class FourierTrans;
	CFunc* fused_gelu_ = nullptr;                   // Hadamard(shared h) -> CGelu run as one kernel pair
	bool in_fft_epilogue_ = false;                  // the producing FourierTrans computes this layer's forward
	float* consumerSplit();                         // split planes of the Linear fed by the fused GELU, or NULL
public:
	Hadamard(Uid uid, InSize a, InSize b) : CFunc(uid, InSize(a.value() + b.value()), OutSize(a.value())) {}
	Hadamard(InSize a, InSize b) : CFunc(InSize(a.value() + b.value()), OutSize(a.value())) {}
	CFunc* clone(Uid uid) override { return new Hadamard(uid, InSize(out_size_), InSize(out_size_)); }
	std::string getName() override { return "Hadamard_" + std::to_string(uid_); }
	void forward() override;
	void backward() override;
};

class CGelu : public CFunc {                        // impl/relu.h:99-201
public:
	CGelu(Uid uid, InSize n) : CFunc(uid, n, OutSize(n.value())) {}
	explicit CGelu(InSize n) : CFunc(n, OutSize(n.value())) {}
	CFunc* clone(Uid uid) override { return new CGelu(uid, InSize(in_size_)); }
	std::string getName() override { return "CGelu_" + std::to_string(uid_); }
	void forward() override;
	void backward() override;
};

class Linear : public CFunc {                       // impl/linear.h:11-156
	friend class CNet;
	friend class Hadamard;
	int in1_len, in2_len;
	CFunc* fused_residual_ = nullptr;               // Residual add done in the GEMM epilogue
	int residual_operand_ = 0;                      // which Residual input is the other addend
	// operand split buffers kept by the layer: x is split in forward() and reused by dW*, W is
	// split when the weights change and reused by forward and dX*
	float* x_split_ = nullptr;
	float* w_split_ = nullptr;
	bool use_split_ = false;
	bool x_presplit_ = false;                       // the producer of x writes x_split_ itself
	unsigned long long w_split_version_ = ~0ull;
	size_t extraBytes(int batch) const override;
	void bindExtra(char* mem, int batch) override;
	void splitWeights();
public:
	Linear(Uid uid, InSize in1, InSize in2);
	Linear(InSize in1, InSize in2);
	int firstInputLength() const { return in1_len; }
	int secondInputLength() const { return in2_len; }
	CFunc* clone(Uid uid) override { return new Linear(uid, InSize(in1_len), InSize(in2_len)); }
	std::string getName() override { return "Linear_" + std::to_string(uid_); }
	void forward() override;
	void backward() override;
};

class Residual : public CFunc {                     // impl/residual.h:12-120
public:
	Residual(Uid uid, InSize n) : CFunc(uid, InSize(2 * n.value()), OutSize(n.value())) {}
	explicit Residual(InSize n) : CFunc(InSize(2 * n.value()), OutSize(n.value())) {}
	CFunc* clone(Uid uid) override { return new Residual(uid, InSize(out_size_)); }
	std::string getName() override { return "Res_" + std::to_string(uid_); }
	void forward() override;
	void backward() override;
};

class SoftMax : public CFunc {                      // impl/softmax.h:9-96 (an L2 normalisation)
	float* inv_norm_ = nullptr;                     // device [batch]
	size_t extraBytes(int batch) const override { return (size_t) batch * sizeof(float); }
	void bindExtra(char* mem, int) override { inv_norm_ = reinterpret_cast<float*>(mem); }
public:
	SoftMax(Uid uid, InSize n) : CFunc(uid, n, OutSize(n.value())) {}
	explicit SoftMax(InSize n) : CFunc(n, OutSize(n.value())) {}
	CFunc* clone(Uid uid) override { return new SoftMax(uid, InSize(in_size_)); }
	std::string getName() override { return "SoftMax_" + std::to_string(uid_); }
	void forward() override;
	void backward() override;
};

// A loss layer: device buffers for the labels and the per-sample losses of the batch.  forward()
// computes the loss AND seeds dL/dz* of its input in the same pass.
class LossFunc : public CFunc, public OutputFunc {
	friend class CNet;
protected:
	float* loss_ = nullptr;                         // device [batch]
	int32_t* labels_ = nullptr;                     // device [batch]
	size_t extraBytes(int batch) const override { return 2 * (((size_t) batch * 4 + 255) & ~size_t(255)); }
	void bindExtra(char* mem, int batch) override;
public:
	LossFunc(Uid uid, InSize n) : CFunc(uid, n, OutSize(1)) { is_output_ = true; }
	explicit LossFunc(InSize n) : CFunc(n, OutSize(1)) { is_output_ = true; }
	float loss(int sample) override;
	float* deviceLosses() const { return loss_; }
	int32_t* deviceLabels() const { return labels_; }
	void backward() override {}
	void backward(int label) override;  // batch of one sample: reseeds with `label`
};

class CrossEntropy : public LossFunc {              // impl/crossent.h:9-185
public:
	CrossEntropy(Uid uid, InSize n) : LossFunc(uid, n) {}
	explicit CrossEntropy(InSize n) : LossFunc(n) {}
	CFunc* clone(Uid uid) override { return new CrossEntropy(uid, InSize(in_size_)); }
	std::string getName() override { return "CrossEntropy_" + std::to_string(uid_); }
	int outputLength() override { return in_size_; }
	void forward() override;
};

class L2Out : public LossFunc {                     // impl/l2out.h:10-79: loss = sum |z|^2, dz* = z
public:
	L2Out(Uid uid, InSize n) : LossFunc(uid, n) {}
	explicit L2Out(InSize n) : LossFunc(n) {}
	CFunc* clone(Uid uid) override { return new L2Out(uid, InSize(in_size_)); }
	std::string getName() override { return "L2Out_" + std::to_string(uid_); }
	int outputLength() override { return 1; }
	void forward() override;
};

class CRelu : public CFunc {                        // impl/relu.h:12-96
public:
	CRelu(Uid uid, InSize n) : CFunc(uid, n, OutSize(n.value())) {}
	explicit CRelu(InSize n) : CFunc(n, OutSize(n.value())) {}
	CFunc* clone(Uid uid) override { return new CRelu(uid, InSize(in_size_)); }
	std::string getName() override { return "CRelu_" + std::to_string(uid_); }
	void forward() override;
	void backward() override;
};

class TriangFourier : public CFunc {                // impl/ft.h:115-222: lower-triangular DFT
public:
	TriangFourier(Uid uid, InSize n) : CFunc(uid, n, OutSize(n.value())) {}
	explicit TriangFourier(InSize n) : CFunc(n, OutSize(n.value())) {}
	CFunc* clone(Uid uid) override { return new TriangFourier(uid, InSize(in_size_)); }
	std::string getName() override { return "TriangFourier_" + std::to_string(uid_); }
	void forward() override;
	void backward() override;
};

// Called after every gradient bucket (a contiguous range of the weight-gradient arena, in
// backward order) is complete on the net's stream; data-parallel trainers all-reduce it.
typedef int (*BucketHook)(void* user, float* grads, size_t count, int bucket, int n_buckets);

class CNet {
	friend class CFunc;
	friend class Linear;
	friend class CrossEntropy;
	friend class L2Out;
	std::vector<CFunc*> func_list_;                 // owned, insertion order
	std::map<int, CFunc*> map_;
	std::vector<CFunc*> inputs_, outputs_;
	int next_uid_ = 0;
	std::vector<std::vector<CFunc*> > func_at_depth_;
	cnb_ctx* ctx_ = nullptr;
	void* stream_ = nullptr;
	int device_ = 0;
	size_t arena_bytes_ = 0;
	void* ext_arena_ = nullptr;
	bool nccl_arena_ = false;                       // the arena comes from NCCL's allocator (registrable as a symmetric window)
	void* own_nccl_arena_ = nullptr;
	int batch_ = 0;                                 // allocated batch
	int cur_batch_ = 0;                             // rows of the batch in flight
	bool fuse_ = true;
	bool ok_ = true;
	std::string error_;
	CFunc* main_in_ = nullptr;
	LossFunc* main_out_ = nullptr;
	float* wgrad_base_ = nullptr;                   // contiguous dz* planes of every weight, backward order
	size_t wgrad_count_ = 0;
	float* weight_base_ = nullptr;                  // contiguous value planes, same order
	float* momentum_base_ = nullptr;                // Adam momentum, same layout (allocated on first adamUpdate)
	bool infer_only_ = false;
	struct Bucket { size_t begin, count; CFunc* last_writer; };
	std::vector<Bucket> buckets_;
	BucketHook hook_ = nullptr;
	void* hook_user_ = nullptr;
	int dp_gemm_ctas_ = 0;                          // GEMM grid cap while all-reduces are in flight
	unsigned long long weights_version_ = 0;        // bumped whenever weight values change
	float* g_split_ = nullptr;                      // shared split planes of a Linear's output gradient
	void* side_stream_ = nullptr;                   // second compute stream: dW* runs beside dX* at small batches
	void* ev_side_fork_ = nullptr;
	void* ev_side_join_ = nullptr;
	int sm_count_ = 0;
	NcclGroup nccl_;                                // native data parallelism (setDataParallel)
	// data parallelism over symmetric memory with the library's own all-reduce kernel (setSymmetricPeers)
	cnb_dp_peers sym_ = {};
	bool sym_active_ = false, sym_pending_ = false;
	void* sym_stream_ = nullptr;
	void* ev_sym_fork_ = nullptr;
	void* ev_sym_join_ = nullptr;
	bool joinCollectives();                         // the compute stream waits for every collective in flight
	void* graph_exec_ = nullptr;                    // cudaGraphExec_t of a captured step
	bool capturing_ = false;
	unsigned long long graph_launches_ = 0;         // kernels inside the captured step
	int graph_batch_ = 0;                           // rows of the batch the captured launches were sized for
	std::string graph_stale_;                       // why the captured step may no longer be replayed ("" = it may)
	bool reduced_since_update_ = false;             // the gradient arena holds a sum over the ranks already
	bool reduceBucket(size_t index);
	// double-buffered input pipeline (prefetchBatch / commitBatch / readLossesAsync)
	void* copy_stream_ = nullptr;                   // cudaStream_t for host <-> device copies
	void* ev_h2d_ = nullptr;                        // staged batch has arrived
	void* ev_commit_ = nullptr;                     // staging buffer has been consumed
	void* ev_step_ = nullptr;                       // losses of the step are final
	void* ev_d2h_ = nullptr;                        // losses have reached the host
	char* stage_in_ = nullptr;                      // device staging: [re | im] planes or token ids
	int32_t* stage_labels_ = nullptr;
	int staged_batch_ = 0;
	bool d2h_pending_ = false;
	bool pipelineInit();

	void fail(int status, const std::string& where);
	bool planFusion();
public:
	CNet();
	// device / arena to use; call before allocateOnGpu.  ext_arena != NULL: caller-owned memory.
	void setDevice(int device, size_t arena_bytes, void* ext_arena = nullptr);
	// Take the arena from NCCL's allocator (ncclMemAlloc) instead of cudaMalloc, so that setDataParallel can
	// register the weight / gradient region with the communicator as a symmetric window.  Call before allocateOnGpu.
	void setNcclArena(bool on) { nccl_arena_ = on; }
	bool symmetricWindow() const { return nccl_.hasWindow(); }
	void setStream(void* stream) { stream_ = stream; }
	void setFusion(bool on) { fuse_ = on; }
	void setBucketHook(BucketHook hook, void* user) { hook_ = hook; hook_user_ = user; }
	// Native NCCL data parallelism: every rank calls this with the id made by ncclUniqueId() on one
	// rank.  backward() then all-reduces each finished gradient bucket on a communication stream and
	// updateInputs() waits for them; the caller passes lr / global_batch.
	static bool ncclUniqueId(char out[kNcclUniqueIdBytes], std::string* err) { return NcclGroup::uniqueId(out, err); }
	bool setDataParallel(const char id[kNcclUniqueIdBytes], int rank, int nranks);
	// Data parallelism without NCCL in the data path: the arena of every rank is symmetric memory mapped into
	// every process (base pointers, optional multicast address, a zeroed flag block per rank; see cnb_dp_allreduce).
	// backward() then sums every finished gradient bucket with the library's own kernel on a communication
	// stream; its CTAs run beside the GEMM's on the same SMs, so no SMs are set aside.  Call after allocateOnGpu.
	bool setSymmetricPeers(int rank, int world, void* multicast_base, void* const* arena_bases, void* const* flag_blocks, int ctas);
	int dataParallelError() { return nccl_.asyncError(); }
	// Sums the whole weight-gradient arena over the ranks now (every bucket, then joins the compute stream):
	// what backward() does bucket by bucket, as one call, for callers that drive the layers themselves.
	bool allReduceGradients();
	// CUDA graph of a step: beginCapture(); forward(); backward(); updateInputs(lr); endCapture();
	// then launchGraph() replays it (same batch buffers, labels and learning rate).
	bool beginCapture();
	bool endCapture();
	bool launchGraph();
	unsigned long long graphKernelCount() const { return graph_launches_; }
	virtual ~CNet();

	int add(CFunc* func);
	int add(CFunc* func, std::initializer_list<int> in_uids);
	int add(CFunc* func, const std::vector<int>& in_uids);
	CFunc*& operator[](int uid) { return map_[uid]; }
	const std::vector<CFunc*>& inputs() const { return inputs_; }
	const std::vector<CFunc*>& functionList() const { return func_list_; }
	CFunc* findFirstOfType(int typeId);
	CFunc* findFirstInput();
	CFunc* findFirstOutput();
	static int getType(CFunc* func);                // impl/cnet.h:110-151
	void init_inputs();
	void init_inputs(uint64_t seed);
	void init_exec_graph(bool print_status = false);
	int maxDepth() const { return (int) func_at_depth_.size(); }

	// device lifecycle (gpu/gpu_func.h:1071-1086): builds batched tensors, uploads weights
	bool allocateOnGpu(int batch_size);
	size_t requiredArenaBytes(int batch_size) const;
	size_t scratchBytes(int batch_size) const;
	bool setInputValues(int uid, const float* re, const float* im, int len);     // host -> weights
	bool getInputValues(int uid, float* re, float* im, int len);
	bool getInputGradients(int uid, float* re, float* im, int len);
	bool getInputsFromGpu();                        // gpu/gpu_func.h:512-527 (weights to the host copies)

	// batch upload (batchToGpu, gpu/gpu_func.h:368-427): ONE copy per plane
	bool batchToGpu(const float* re, const float* im, const int* tokens, const int* labels, int batch);
	// Input pipeline (the reference uploads 2*B small copies synchronously before every forward,
	// gpu/gpu_func.h:368-427).  prefetchBatch() starts the host-to-device copy of the NEXT batch into a
	// staging buffer on a copy stream while the current step runs; commitBatch() makes the compute
	// stream wait for it and moves it into the input tensors (device-to-device); readLossesAsync()
	// brings the per-sample losses back on the copy stream and waitLosses() blocks until they arrived.
	// Host buffers should be pinned, or the copies are not asynchronous.
	bool prefetchBatch(const float* re, const float* im, const int* tokens, const int* labels, int batch);
	bool commitBatch();
	bool readLossesAsync(float* host_out, int n);
	bool waitLosses();
	// the step
	void forward();                                 // all layers, insertion order (impl/cnet.h:366-377)
	void backward();                                // reverse order with the uploaded labels
	void backward(int label);                       // one-sample form (impl/cnet.h:400-411)
	void updateInputs(float l_rate);                // impl/cnet.h:413-421 via gpu/gpu_func.h:497-501
	bool gpuForward(InputFunc* inp, OutputFunc* outp, InputBatch& batch);
	bool gpuForward(InputFunc* inp, OutputFunc* outp, EmbeddingBatch& batch);
	bool gpuBackward();
	void gpuUpdateInputs(float l_rate) { updateInputs(l_rate); }
	// The reference's momentum-only Adam (CNet::adamUpdate, gpu/gpu_func.h:503-510): t counts updates
	// from 0; the caller passes l_rate / batch.  The momentum planes are allocated on first use.
	void adamUpdate(float l_rate, float beta, int t);
	void infer();                                   // forward without seeding gradients (impl/cnet.h:379-389)
	float getLoss(OutputFunc* outp, Batch* batch);  // mean loss, per-sample losses into the batch
	bool getLosses(float* out, int n);
	bool sync();

	// Checkpoints in the reference's ModelSaver byte format (impl/model_saver.h; CNet::save / restore,
	// gpu/gpu_func.h:1103-1111).  restore() needs an empty net; allocateOnGpu afterwards.
	bool save(const std::string& file);
	bool restore(const std::string& file);
	std::string saveToString();
	bool restoreFromString(const std::string& data);
	int noFunctions() const { return (int) func_list_.size(); }
	int uidAt(int i) const { return func_list_.at(i)->uid(); }

	bool readOutput(int uid, int what, float* re, float* im);   // 0 values, 1 dL/dz*: for tests
	bool ok() const { return ok_; }
	const std::string& error() const { return error_; }
	void clearError() { ok_ = true; error_.clear(); }
	cnb_ctx* context() const { return ctx_; }
	void* stream() const { return stream_; }
	int batchSize() const { return cur_batch_; }
	float* gradArena(size_t* count) const { if (count) *count = wgrad_count_; return wgrad_base_; }
	float* weightArena(size_t* count) const { if (count) *count = wgrad_count_; return weight_base_; }
	int noBuckets() const { return (int) buckets_.size(); }
};

}  // namespace cnet_b200

#endif  // CNET_B200_HOST_CNET_H_
