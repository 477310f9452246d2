// Host orchestration of the batched complex training step: graph bookkeeping, device
// tensor planning in the arena, layer -> C-ABI kernel calls, fusion planning, gradient
// buckets for data parallelism.  See cnet.h for the contract and its reference citations.
#include "cnet.h"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>

#include <cuda_runtime.h>

namespace cnet_b200 {

namespace {

inline size_t pad64(size_t n) { return (n + 63) & ~size_t(63); }   // floats -> 256-byte multiples

// splitmix64: deterministic host generator for init_inputs
struct SplitMix {
	uint64_t s;
	explicit SplitMix(uint64_t seed) : s(seed) {}
	uint64_t next() {
		uint64_t z = (s += 0x9E3779B97F4A7C15ull);
		z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
		z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
		return z ^ (z >> 31);
	}
	double uniform() { return (next() >> 11) * (1.0 / 9007199254740992.0); }
};

}  // namespace

// ------------------------------------------------------------------ batches
void InputBatch::add(const std::vector<std::complex<float> >& sample, int label) {
	for (auto c : sample) { real_data_.push_back(c.real()); imag_data_.push_back(c.imag()); }
	while (real_data_.size() < (size_t) (1 + current_pos_) * sample_dim_) {
		real_data_.push_back(0.f); imag_data_.push_back(0.f);
	}
	labels_.push_back(label);
	current_pos_++;
}

void InputBatch::assign(const float* re, const float* im, const int* labels, int batch) {
	batch_size_ = batch;
	size_t n = (size_t) batch * sample_dim_;
	real_data_.assign(re, re + n);
	imag_data_.assign(im, im + n);
	labels_.assign(labels, labels + batch);
	current_pos_ = batch;
}

void EmbeddingBatch::add(const std::vector<int>& sample, int label) {
	token_.insert(token_.end(), sample.begin(), sample.end());
	while (token_.size() < (size_t) (1 + current_pos_) * sample_dim_) token_.push_back(NO_TOKEN);
	labels_.push_back(label);
	current_pos_++;
}

void EmbeddingBatch::assign(const int* tokens, const int* labels, int batch) {
	batch_size_ = batch;
	token_.assign(tokens, tokens + (size_t) batch * sample_dim_);
	labels_.assign(labels, labels + batch);
	current_pos_ = batch;
}

// -------------------------------------------------------------------- CFunc
cnb_ctx* CFunc::ctx() const { return net_ ? net_->ctx_ : nullptr; }
void* CFunc::stream() const { return net_ ? net_->stream_ : nullptr; }
int CFunc::batch() const { return net_ ? net_->cur_batch_ : 0; }

void CFunc::check(int status) {
	if (status != CNB_OK && net_) net_->fail(status, getName());
}

int CFunc::accumulate_into(CFunc* p) {
	if (!p->batched_) return 1;                 // weight gradients accumulate until updateInputs
	int acc = p->grad_written_ ? 1 : 0;
	p->grad_written_ = true;
	return acc;
}

void CFunc::addOutput(CFunc* next, int offset) {
	next_func_.push_back(next);
	offset_.push_back(offset);
	if (next->depth_ <= depth_) next->depth_ = depth_ + 1;
}

std::complex<float> CFunc::dz(int, int) { return std::complex<float>(NAN, NAN); }
std::complex<float> CFunc::dz_star(int, int) { return std::complex<float>(NAN, NAN); }

void CFunc::updateInput(float lr) {
	if (!is_input_ || !out_.dz_star_real_ || batched_) return;
	check(cnb_sgd_update(ctx(), out_.real_, out_.dz_star_real_, out_.count(), lr, 1, stream()));
	check(cnb_sgd_update(ctx(), out_.imag_, out_.dz_star_imag_, out_.count(), lr, 1, stream()));
}

void CFunc::init_inputs(uint64_t seed) {
	SplitMix r(seed);
	host_re_.resize(out_size_);
	host_im_.resize(out_size_);
	for (int i = 0; i < out_size_; ++i) {
		float re = (float) r.uniform() - 0.5f;
		host_re_[i] = re / out_size_;
		host_im_[i] = std::sqrt(1 - re * re) / out_size_;
	}
}

// --------------------------------------------------------------- CEmbedding
size_t CEmbedding::extraBytes(int batch) const {
	return (((size_t) batch * no_out_tokens_ * sizeof(int32_t)) + 255) & ~size_t(255);
}

void CEmbedding::bindExtra(char* mem, int) { tokens_ = reinterpret_cast<int32_t*>(mem); }

void CEmbedding::forward() {
	check(cnb_embed_fwd(ctx(), table_.real_, table_.imag_, tokens_, out_.real_, out_.imag_, batch(),
			no_out_tokens_, embedding_dim_, no_embeddings_, stream()));
}

void CEmbedding::backward() {
	if (!grad_written_) return;                 // no consumer produced a gradient
	check(cnb_embed_bwd(ctx(), out_.dz_star_real_, out_.dz_star_imag_, tokens_, table_.dz_star_real_,
			table_.dz_star_imag_, batch(), no_out_tokens_, embedding_dim_, no_embeddings_, stream()));
}

void CEmbedding::updateInput(float lr) {
	check(cnb_sgd_update(ctx(), table_.real_, table_.dz_star_real_, table_.count(), lr, 1, stream()));
	check(cnb_sgd_update(ctx(), table_.imag_, table_.dz_star_imag_, table_.count(), lr, 1, stream()));
}

void CEmbedding::init_inputs(uint64_t seed) {
	SplitMix r(seed);
	host_re_.resize(in_size_);
	host_im_.resize(in_size_);
	float s = std::sqrt((float) embedding_dim_);
	for (int i = 0; i < in_size_; ++i) {
		float re = (float) r.uniform() - 0.5f;
		host_re_[i] = re / s;
		host_im_[i] = std::sqrt(1 - re * re) / s;
	}
}

// ------------------------------------------------------------- FourierTrans
void FourierTrans::forward() {
	const Vars& x = in(0);
	if (fused_hg_) {
		const Vars& h = fused_hg_->previous(1)->output();
		Vars& y = fused_hg_->fused_gelu_->out_;
		// the only reader of y is the Linear that takes the split planes: y itself is not stored a second time
		float* ysplit = fused_hg_->consumerSplit();
		fused_hg_->fused_gelu_->value_split_ = ysplit;
		check(cnb_dft_hadamard_gelu_fwd(ctx(), x.real_, x.imag_, h.real_, h.imag_, out_.real_, out_.imag_,
				ysplit ? nullptr : y.real_, ysplit ? nullptr : y.imag_, ysplit, batch(), in_size_, stream()));
		return;
	}
	check(cnb_dft_fwd(ctx(), x.real_, x.imag_, out_.real_, out_.imag_, batch(), in_size_, stream()));
}

void FourierTrans::backward() {
	CFunc* p = prev_func_[0];
	int acc = accumulate_into(p);
	check(cnb_dft_bwd(ctx(), out_.dz_star_real_, out_.dz_star_imag_, p->out_.dz_star_real_, p->out_.dz_star_imag_,
			batch(), in_size_, acc, stream()));
}

// ----------------------------------------------------------------- Hadamard
float* Hadamard::consumerSplit() {
	// a Linear that is the only consumer of the GELU output gets its operand split planes from the producer
	if (!fused_gelu_ || fused_gelu_->no_outputs() != 1) return nullptr;
	Linear* l = dynamic_cast<Linear*>(fused_gelu_->next(0));
	if (l && l->use_split_ && l->previous(0) == fused_gelu_ &&
			cnb_linear_split_ok(batch(), l->firstInputLength(), l->outSize())) {
		l->x_presplit_ = true;
		return l->x_split_;
	}
	return nullptr;
}

void Hadamard::forward() {
	if (in_fft_epilogue_) return;
	const Vars& u = in(0);
	const Vars& v = in(1);
	if (fused_gelu_) {
		Vars& y = fused_gelu_->out_;
		float* ysplit = consumerSplit();
		check(cnb_hadamard_gelu_fwd_split(ctx(), u.real_, u.imag_, v.real_, v.imag_, out_.real_, out_.imag_, y.real_,
				y.imag_, ysplit, batch(), out_size_, stream()));
		return;
	}
	check(cnb_hadamard_fwd(ctx(), u.real_, u.imag_, v.real_, v.imag_, prev_func_[1]->batched_ ? 1 : 0, out_.real_,
			out_.imag_, batch(), out_size_, stream()));
}

void Hadamard::backward() {
	CFunc* pu = prev_func_[0];
	CFunc* pv = prev_func_[1];
	int acc_u = accumulate_into(pu), acc_v = accumulate_into(pv);
	if (fused_gelu_) {
		const Vars& g = fused_gelu_->out_;
		check(cnb_hadamard_gelu_bwd(ctx(), g.dz_star_real_, g.dz_star_imag_, out_.real_, out_.imag_, pu->out_.real_,
				pu->out_.imag_, pv->out_.real_, pv->out_.imag_, pu->out_.dz_star_real_, pu->out_.dz_star_imag_, acc_u,
				pv->out_.dz_star_real_, pv->out_.dz_star_imag_, acc_v, batch(), out_size_, stream()));
		return;
	}
	check(cnb_hadamard_bwd(ctx(), out_.dz_star_real_, out_.dz_star_imag_, pu->out_.real_, pu->out_.imag_,
			pv->out_.real_, pv->out_.imag_, pv->batched_ ? 1 : 0, pu->out_.dz_star_real_, pu->out_.dz_star_imag_, acc_u,
			pv->out_.dz_star_real_, pv->out_.dz_star_imag_, acc_v, batch(), out_size_, stream()));
}

// -------------------------------------------------------------------- CGelu
void CGelu::forward() {
	const Vars& z = in(0);
	check(cnb_gelu_fwd(ctx(), z.real_, z.imag_, out_.real_, out_.imag_, (size_t) batch() * out_size_, stream()));
}

void CGelu::backward() {
	CFunc* p = prev_func_[0];
	int acc = accumulate_into(p);
	check(cnb_gelu_bwd(ctx(), out_.dz_star_real_, out_.dz_star_imag_, p->out_.real_, p->out_.imag_,
			p->out_.dz_star_real_, p->out_.dz_star_imag_, (size_t) batch() * out_size_, acc, stream()));
}

// ------------------------------------------------------------------- Linear
Linear::Linear(Uid uid, InSize in1, InSize in2)
	: CFunc(uid, InSize(in1.value() + in2.value()), OutSize(in2.value() / in1.value())), in1_len(in1.value()),
	  in2_len(in2.value()) {}

Linear::Linear(InSize in1, InSize in2)
	: CFunc(InSize(in1.value() + in2.value()), OutSize(in2.value() / in1.value())), in1_len(in1.value()),
	  in2_len(in2.value()) {}

size_t Linear::extraBytes(int batch) const {
	if (!cnb_linear_split_ok(batch, in1_len, out_size_)) return 0;
	return (cnb_split_floats((size_t) batch * in1_len) + cnb_split_floats((size_t) in2_len)) * sizeof(float);
}

void Linear::bindExtra(char* mem, int batch) {
	use_split_ = true;
	x_split_ = reinterpret_cast<float*>(mem);
	w_split_ = x_split_ + cnb_split_floats((size_t) batch * in1_len);
}

void Linear::splitWeights() {
	if (!use_split_) return;
	const Vars& w = in(1);
	check(cnb_split_planes(ctx(), w.real_, w.imag_, (size_t) in2_len, w_split_, stream()));
	w_split_version_ = net_->weights_version_;
}

void Linear::forward() {
	const Vars& x = in(0);
	const Vars& w = in(1);
	const float *rr = nullptr, *ri = nullptr;
	if (fused_residual_) {
		const Vars& r = fused_residual_->previous(residual_operand_)->output();
		rr = r.real_; ri = r.imag_;
	}
	if (use_split_ && cnb_linear_split_ok(batch(), in1_len, out_size_)) {
		if (w_split_version_ != net_->weights_version_) splitWeights();
		if (!x_presplit_)
			check(cnb_split_planes(ctx(), x.real_, x.imag_, (size_t) batch() * in1_len, x_split_, stream()));
		x_presplit_ = false;
		check(cnb_linear_fwd_split(ctx(), x_split_, w_split_, rr, ri, out_.real_, out_.imag_, batch(), in1_len,
				out_size_, stream()));
		return;
	}
	check(cnb_linear_fwd(ctx(), x.real_, x.imag_, w.real_, w.imag_, rr, ri, out_.real_, out_.imag_, batch(), in1_len,
			out_size_, stream()));
}

void Linear::backward() {
	CFunc* px = prev_func_[0];
	CFunc* pw = prev_func_[1];
	int acc_x = accumulate_into(px), acc_w = accumulate_into(pw);
	if (use_split_ && cnb_linear_split_ok(batch(), in1_len, out_size_)) {
		float* gs = net_->g_split_;
		check(cnb_split_planes(ctx(), out_.dz_star_real_, out_.dz_star_imag_, (size_t) batch() * out_size_, gs, stream()));
		// Small problems give each of the 148 persistent CTAs only a few k-blocks, so prologue and
		// epilogue dominate: run the two independent products side by side on half the SMs each.
		const bool side_by_side = net_->side_stream_ != nullptr &&
				(size_t) batch() * in1_len * out_size_ <= (size_t) 1536 * 1024 * 1024;
		if (side_by_side) {
			cudaStream_t ms = (cudaStream_t) stream(), ss = (cudaStream_t) net_->side_stream_;
			int limit = net_->dp_gemm_ctas_ > 0 ? net_->dp_gemm_ctas_ : net_->sm_count_;
			cudaEventRecord((cudaEvent_t) net_->ev_side_fork_, ms);
			cudaStreamWaitEvent(ss, (cudaEvent_t) net_->ev_side_fork_, 0);
			cnb_set_gemm_sm_limit(ctx(), limit / 2);
			check(cnb_linear_bwd_w_split(ctx(), gs, x_split_, pw->out_.dz_star_real_, pw->out_.dz_star_imag_, batch(),
					in1_len, out_size_, acc_w, ss));
			check(cnb_linear_bwd_x_split(ctx(), gs, w_split_, px->out_.dz_star_real_, px->out_.dz_star_imag_, batch(),
					in1_len, out_size_, acc_x, ms));
			cnb_set_gemm_sm_limit(ctx(), net_->dp_gemm_ctas_ > 0 ? net_->dp_gemm_ctas_ : 0);
			cudaEventRecord((cudaEvent_t) net_->ev_side_join_, ss);
			cudaStreamWaitEvent(ms, (cudaEvent_t) net_->ev_side_join_, 0);
			return;
		}
		check(cnb_linear_bwd_w_split(ctx(), gs, x_split_, pw->out_.dz_star_real_, pw->out_.dz_star_imag_, batch(),
				in1_len, out_size_, acc_w, stream()));
		check(cnb_linear_bwd_x_split(ctx(), gs, w_split_, px->out_.dz_star_real_, px->out_.dz_star_imag_, batch(),
				in1_len, out_size_, acc_x, stream()));
		return;
	}
	check(cnb_linear_bwd_w(ctx(), out_.dz_star_real_, out_.dz_star_imag_, px->out_.real_, px->out_.imag_,
			pw->out_.dz_star_real_, pw->out_.dz_star_imag_, batch(), in1_len, out_size_, acc_w, stream()));
	check(cnb_linear_bwd_x(ctx(), out_.dz_star_real_, out_.dz_star_imag_, pw->out_.real_, pw->out_.imag_,
			px->out_.dz_star_real_, px->out_.dz_star_imag_, batch(), in1_len, out_size_, acc_x, stream()));
}

// ----------------------------------------------------------------- Residual
void Residual::forward() {
	const Vars& u = in(0);
	const Vars& v = in(1);
	check(cnb_residual_fwd(ctx(), u.real_, u.imag_, v.real_, v.imag_, out_.real_, out_.imag_,
			(size_t) batch() * out_size_, stream()));
}

void Residual::backward() {
	for (int k = 0; k < 2; ++k) {
		CFunc* p = prev_func_[k];
		if (p->out_.dz_star_real_ == out_.dz_star_real_) {   // fused Linear shares this gradient tensor
			p->grad_written_ = true;
			continue;
		}
		int acc = accumulate_into(p);
		check(cnb_axpy(ctx(), out_.dz_star_real_, out_.dz_star_imag_, p->out_.dz_star_real_, p->out_.dz_star_imag_,
				(size_t) batch() * out_size_, acc, stream()));
	}
}

// ------------------------------------------------------------------ SoftMax
void SoftMax::forward() {
	const Vars& z = in(0);
	check(cnb_softmax_fwd(ctx(), z.real_, z.imag_, out_.real_, out_.imag_, inv_norm_, batch(), in_size_, stream()));
}

void SoftMax::backward() {
	CFunc* p = prev_func_[0];
	int acc = accumulate_into(p);
	check(cnb_softmax_bwd(ctx(), out_.dz_star_real_, out_.dz_star_imag_, p->out_.real_, p->out_.imag_, inv_norm_,
			p->out_.dz_star_real_, p->out_.dz_star_imag_, batch(), in_size_, acc, stream()));
}

// ------------------------------------------------------------------- losses
void LossFunc::bindExtra(char* mem, int batch) {
	loss_ = reinterpret_cast<float*>(mem);
	labels_ = reinterpret_cast<int32_t*>(mem + (((size_t) batch * 4 + 255) & ~size_t(255)));
}

void LossFunc::backward(int label) {
	std::vector<int32_t> l(batch(), label);
	check(cnb_h2d(ctx(), labels_, l.data(), l.size() * sizeof(int32_t), stream()));
	check(cnb_sync(ctx(), stream()));
	forward();
}

float LossFunc::loss(int sample) {
	float v = 0.f;
	if (sample < 0 || sample >= batch()) return NAN;
	check(cnb_d2h(ctx(), &v, loss_ + sample, sizeof(float), stream()));
	return v;
}

void CrossEntropy::forward() {
	CFunc* p = prev_func_[0];
	bool seed = !net_->infer_only_;
	check(cnb_crossent_fwd_bwd(ctx(), p->out_.real_, p->out_.imag_, labels_, loss_, seed ? p->out_.dz_star_real_ : nullptr,
			seed ? p->out_.dz_star_imag_ : nullptr, batch(), in_size_, stream()));
}

void L2Out::forward() {
	CFunc* p = prev_func_[0];
	bool seed = !net_->infer_only_;
	check(cnb_l2out_fwd_bwd(ctx(), p->out_.real_, p->out_.imag_, loss_, seed ? p->out_.dz_star_real_ : nullptr,
			seed ? p->out_.dz_star_imag_ : nullptr, batch(), in_size_, stream()));
}

// -------------------------------------------------------- CRelu, TriangFourier
void CRelu::forward() {
	const Vars& z = in(0);
	check(cnb_crelu_fwd(ctx(), z.real_, z.imag_, out_.real_, out_.imag_, (size_t) batch() * out_size_, stream()));
}

void CRelu::backward() {
	CFunc* p = prev_func_[0];
	int acc = accumulate_into(p);
	check(cnb_crelu_bwd(ctx(), out_.dz_star_real_, out_.dz_star_imag_, p->out_.real_, p->out_.imag_,
			p->out_.dz_star_real_, p->out_.dz_star_imag_, (size_t) batch() * out_size_, acc, stream()));
}

void TriangFourier::forward() {
	const Vars& x = in(0);
	check(cnb_tdft_fwd(ctx(), x.real_, x.imag_, out_.real_, out_.imag_, batch(), in_size_, stream()));
}

void TriangFourier::backward() {
	CFunc* p = prev_func_[0];
	int acc = accumulate_into(p);
	check(cnb_tdft_bwd(ctx(), out_.dz_star_real_, out_.dz_star_imag_, p->out_.dz_star_real_, p->out_.dz_star_imag_,
			batch(), in_size_, acc, stream()));
}

// --------------------------------------------------------------------- CNet
CNet::CNet() {}

CNet::~CNet() {
	if (graph_exec_) cudaGraphExecDestroy((cudaGraphExec_t) graph_exec_);
	if (side_stream_) {
		cudaStreamSynchronize((cudaStream_t) side_stream_);
		cudaEventDestroy((cudaEvent_t) ev_side_fork_); cudaEventDestroy((cudaEvent_t) ev_side_join_);
		cudaStreamDestroy((cudaStream_t) side_stream_);
	}
	if (sym_stream_) {
		cudaStreamSynchronize((cudaStream_t) sym_stream_);
		cudaEventDestroy((cudaEvent_t) ev_sym_fork_); cudaEventDestroy((cudaEvent_t) ev_sym_join_);
		cudaStreamDestroy((cudaStream_t) sym_stream_);
	}
	if (copy_stream_) {
		cudaStreamSynchronize((cudaStream_t) copy_stream_);
		cudaEventDestroy((cudaEvent_t) ev_h2d_); cudaEventDestroy((cudaEvent_t) ev_commit_);
		cudaEventDestroy((cudaEvent_t) ev_step_); cudaEventDestroy((cudaEvent_t) ev_d2h_);
		cudaStreamDestroy((cudaStream_t) copy_stream_);
	}
	for (auto f : func_list_) delete f;
	if (ctx_) cnb_destroy(ctx_);
	nccl_.shutdown();                               // the window is deregistered before its memory goes
	if (own_nccl_arena_) NcclGroup::memFree(own_nccl_arena_);
}

void CNet::setDevice(int device, size_t arena_bytes, void* ext_arena) {
	device_ = device;
	arena_bytes_ = arena_bytes;
	ext_arena_ = ext_arena;
}

void CNet::fail(int status, const std::string& where) {
	if (!ok_) return;                           // keep the first error
	ok_ = false;
	error_ = where + ": status " + std::to_string(status) + ": " + cnb_last_error();
}

int CNet::getType(CFunc* f) {
	if (dynamic_cast<CInput*>(f)) return isInput;
	if (dynamic_cast<Hadamard*>(f)) return isHadamard;
	if (dynamic_cast<Linear*>(f)) return isLinear;
	if (dynamic_cast<CEmbedding*>(f)) return isEmbedding;
	if (dynamic_cast<FourierTrans*>(f)) return isFourier;
	if (dynamic_cast<Residual*>(f)) return isResidual;
	if (dynamic_cast<SoftMax*>(f)) return isSoftMax;
	if (dynamic_cast<CrossEntropy*>(f)) return isCrossEntropy;
	if (dynamic_cast<L2Out*>(f)) return isL2Out;
	if (dynamic_cast<CRelu*>(f)) return isCrelu;
	if (dynamic_cast<TriangFourier*>(f)) return isTrianFourier;
	if (dynamic_cast<CGelu*>(f)) return isGelu;
	return 0x7fffffff;
}

int CNet::add(CFunc* f) {
	if (!f) return -1;
	if (f->uid_ == 0) f->uid_ = ++next_uid_;
	else next_uid_ = std::max(next_uid_, f->uid_);
	if (map_.count(f->uid_)) { fail(CNB_ERR_ARG, "add: duplicate uid " + std::to_string(f->uid_)); return -1; }
	f->type_ = getType(f);
	if (f->type_ == 0x7fffffff && !f->runsOnDevice()) {
		fail(CNB_ERR_UNSUPPORTED, f->getName() + ": not a built-in layer and it does not run on the device: the generic "
				"dz / dz_star Jacobian loop of the reference (impl/cfunc.h:290-325) has no device form; give the layer "
				"forward() / backward() that launch kernels on stream() and return true from runsOnDevice()");
		return -1;
	}
	f->net_ = this;
	func_list_.push_back(f);
	map_[f->uid_] = f;
	if (f->is_input_) inputs_.push_back(f);
	if (f->is_output_) outputs_.push_back(f);
	return f->uid_;
}

int CNet::add(CFunc* f, const std::vector<int>& in_uids) {
	if (!f) return -1;
	// validate before registering, so a rejected function is still the caller's to delete
	int total = 0;
	for (int in_uid : in_uids) {
		auto it = map_.find(in_uid);
		if (it == map_.end()) { fail(CNB_ERR_ARG, "add: unknown producer uid " + std::to_string(in_uid)); return -1; }
		total += it->second->out_size_;
	}
	if (total > f->in_size_) {
		fail(CNB_ERR_ARG, f->getName() + ": producers give " + std::to_string(total) + " > input length " +
				std::to_string(f->in_size_));
		return -1;
	}
	int uid = add(f);
	if (uid < 0) return uid;
	int offset = 0;
	for (int in_uid : in_uids) {
		CFunc* p = map_[in_uid];
		p->addOutput(f, offset);
		offset += p->out_size_;
		f->prev_func_.push_back(p);
	}
	return uid;
}

int CNet::add(CFunc* f, std::initializer_list<int> in_uids) { return add(f, std::vector<int>(in_uids)); }

CFunc* CNet::findFirstOfType(int t) {
	for (auto f : func_list_) if (f->type_ == t) return f;
	return nullptr;
}

CFunc* CNet::findFirstInput() {
	for (auto f : func_list_) if (dynamic_cast<InputFunc*>(f)) return f;
	return nullptr;
}

CFunc* CNet::findFirstOutput() {
	for (auto f : func_list_) if (dynamic_cast<OutputFunc*>(f)) return f;
	return nullptr;
}

void CNet::init_inputs() { init_inputs(0x243F6A8885A308D3ull); }

void CNet::init_inputs(uint64_t seed) {
	uint64_t k = 0;
	for (auto f : inputs_) {
		f->init_inputs(seed + k++);
		if (ctx_ && f != main_in_) setInputValues(f->uid_, f->host_re_.data(), f->host_im_.data(), (int) f->host_re_.size());
	}
}

void CNet::init_exec_graph(bool print_status) {
	if (!func_at_depth_.empty()) return;
	int max_depth = 0;
	for (auto f : func_list_) max_depth = std::max(max_depth, f->depth_);
	func_at_depth_.assign(max_depth + 1, std::vector<CFunc*>());
	for (auto f : func_list_) func_at_depth_[f->depth_].push_back(f);
	if (print_status) {
		for (size_t d = 0; d < func_at_depth_.size(); ++d) {
			std::cout << "Depth " << d << ": ";
			for (auto f : func_at_depth_[d]) std::cout << f->getName() << " " << f->sizeInBytes() << ", ";
			std::cout << std::endl;
		}
	}
}

bool CNet::planFusion() {
	for (auto f : func_list_) {
		if (Hadamard* h = dynamic_cast<Hadamard*>(f)) {
			if (h->prev_func_.size() == 2 && !h->prev_func_[1]->batched_ && h->prev_func_[0]->batched_ &&
					h->next_func_.size() == 1) {
				CGelu* g = dynamic_cast<CGelu*>(h->next_func_[0]);
				if (g && g->prev_func_.size() == 1) { h->fused_gelu_ = g; g->fused_away_ = true; }
			}
			// ... and the whole pair moves into the epilogue of the FFT that feeds it
			FourierTrans* ft = dynamic_cast<FourierTrans*>(h->prev_func_[0]);
			if (h->fused_gelu_ && ft && ft->next_func_.size() == 1 && cnb_dft_fused_ok(ft->in_size_)) {
				ft->fused_hg_ = h;
				h->in_fft_epilogue_ = true;
			}
		}
		if (Linear* l = dynamic_cast<Linear*>(f)) {
			if (l->next_func_.size() == 1) {
				Residual* r = dynamic_cast<Residual*>(l->next_func_[0]);
				if (r && r->prev_func_.size() == 2 && r->prev_func_[0] != r->prev_func_[1]) {
					int mine = r->prev_func_[0] == l ? 0 : 1;
					CFunc* other = r->prev_func_[1 - mine];
					if (other->batched_ && !dynamic_cast<Linear*>(other)) {
						l->fused_residual_ = r;
						l->residual_operand_ = 1 - mine;
						r->fused_away_ = true;
					}
				}
			}
		}
	}
	return true;
}

size_t CNet::scratchBytes(int B) const {
	size_t scratch = 8u << 20;
	for (auto f : func_list_) {
		if (Linear* l = dynamic_cast<Linear*>(f))
			scratch = std::max(scratch, cnb_linear_workspace(B, l->firstInputLength(), l->outSize()));
		if (dynamic_cast<FourierTrans*>(f) || dynamic_cast<TriangFourier*>(f))
			scratch = std::max(scratch, cnb_linear_workspace(B, f->in_size_, f->in_size_));
		if (f->type_ == isHadamard) scratch = std::max(scratch, (size_t) 128 * f->out_size_ * 2 * sizeof(float));
	}
	return scratch + 4096;
}

size_t CNet::requiredArenaBytes(int B) const {
	size_t floats = 0, extra = 0, dft = 0;
	for (auto f : func_list_) {
		bool weight = dynamic_cast<CInput*>(f) && f != func_list_.front();
		if (weight) floats += 4 * pad64(f->out_size_);
		else floats += 4 * pad64((size_t) B * f->out_size_);
		if (CEmbedding* e = dynamic_cast<CEmbedding*>(f)) floats += 4 * pad64((size_t) e->inSize());
		if ((dynamic_cast<FourierTrans*>(f) && !cnb_dft_fused_ok((int) f->in_size_)) || dynamic_cast<TriangFourier*>(f))     // twiddle planes + their split
			dft += (size_t) 2 * f->in_size_ * f->in_size_ * 4 + cnb_split_floats((size_t) f->in_size_ * f->in_size_) * 4 + 1024;
		extra += f->extraBytes(B) + 256;
	}
	size_t gs = 0;
	for (auto f : func_list_)
		if (Linear* l = dynamic_cast<Linear*>(f))
			if (cnb_linear_split_ok(B, l->firstInputLength(), l->outSize()))
				gs = std::max(gs, cnb_split_floats((size_t) B * l->outSize()) * sizeof(float));
	size_t staging = 0;                                // input pipeline: one staged batch + labels
	if (!func_list_.empty()) {
		CFunc* f0 = func_list_.front();
		if (CEmbedding* em = dynamic_cast<CEmbedding*>(f0)) staging = (size_t) B * em->noOutTokens() * 4;
		else staging = 2 * (size_t) B * f0->out_size_ * 4;
		staging += (size_t) B * 4 + 1024;
	}
	size_t momentum = 0;                               // Adam momentum planes (allocated on first adamUpdate)
	for (auto f : func_list_) {
		bool weight = dynamic_cast<CInput*>(f) && f != func_list_.front();
		if (weight) momentum += 2 * pad64(f->out_size_) * sizeof(float);
		if (CEmbedding* e = dynamic_cast<CEmbedding*>(f)) momentum += 2 * pad64((size_t) e->inSize()) * sizeof(float);
	}
	return floats * sizeof(float) + extra + dft + gs + staging + momentum + scratchBytes(B) + (16u << 20);
}

bool CNet::allocateOnGpu(int B) {
	if (ctx_) { fail(CNB_ERR_ARG, "allocateOnGpu: already allocated"); return false; }
	if (B <= 0 || func_list_.empty()) { fail(CNB_ERR_ARG, "allocateOnGpu: empty net or batch"); return false; }
	main_in_ = findFirstInput();
	main_out_ = dynamic_cast<LossFunc*>(findFirstOutput());
	if (!main_in_ || !main_out_) { fail(CNB_ERR_ARG, "allocateOnGpu: net needs an InputFunc and a loss output (CrossEntropy or L2Out)"); return false; }
	dynamic_cast<InputFunc*>(main_in_)->setIsMainInput(true);
	main_out_->setIsMainOutput(true);
	init_exec_graph();
	// topology checks: what the batched kernels support
	for (auto f : func_list_) {
		f->batched_ = !(dynamic_cast<CInput*>(f) && f != main_in_);
		size_t want = (f->type_ == isHadamard || f->type_ == isLinear || f->type_ == isResidual) ? 2
				: (f->is_input_ ? 0 : 1);
		if (f->prev_func_.size() != want) {
			fail(CNB_ERR_UNSUPPORTED, f->getName() + ": expected " + std::to_string(want) + " producers");
			return false;
		}
		if (!f->is_output_ && f->next_func_.empty()) {
			fail(CNB_ERR_ARG, f->getName() + ": has no consumer and is not an output"); return false;
		}
	}
	for (auto f : func_list_) {
		if (Linear* l = dynamic_cast<Linear*>(f)) {
			if (!l->prev_func_[0]->batched_ || l->prev_func_[1]->batched_ ||
					l->prev_func_[0]->out_size_ != l->in1_len || l->prev_func_[1]->out_size_ != l->in2_len) {
				fail(CNB_ERR_UNSUPPORTED, l->getName() + ": needs (batched x of in1, weight CInput of in2)"); return false;
			}
		} else if (f->type_ == isHadamard || f->type_ == isResidual) {
			if (f->prev_func_[0]->out_size_ != f->out_size_ || f->prev_func_[1]->out_size_ != f->out_size_ ||
					!f->prev_func_[0]->batched_ || (f->type_ == isResidual && !f->prev_func_[1]->batched_)) {
				fail(CNB_ERR_UNSUPPORTED, f->getName() + ": operand shapes"); return false;
			}
		} else if (!f->is_input_) {
			if (!f->prev_func_[0]->batched_ || f->prev_func_[0]->out_size_ != f->in_size_) {
				fail(CNB_ERR_UNSUPPORTED, f->getName() + ": needs one batched producer of its input length"); return false;
			}
		}
	}
	if (fuse_) planFusion();
	if (arena_bytes_ == 0) arena_bytes_ = requiredArenaBytes(B);
	if (nccl_arena_ && !ext_arena_) {
		cudaSetDevice(device_);
		std::string err;
		arena_bytes_ = (arena_bytes_ + ((size_t) 2 << 20) - 1) & ~(((size_t) 2 << 20) - 1);
		own_nccl_arena_ = NcclGroup::memAlloc(arena_bytes_, &err);
		if (!own_nccl_arena_) { fail(CNB_ERR_CUDA, "allocateOnGpu: " + err); return false; }
		ext_arena_ = own_nccl_arena_;
	}
	int rc = ext_arena_ ? cnb_create_external(device_, ext_arena_, arena_bytes_, &ctx_)
			: cnb_create(device_, arena_bytes_, &ctx_);
	if (rc != CNB_OK) { fail(rc, "allocateOnGpu"); ctx_ = nullptr; return false; }
	batch_ = cur_batch_ = B;
	cnb_device_info(device_, &sm_count_, nullptr, nullptr, nullptr);
	if (stream_ && !side_stream_) {             // a second stream only makes sense beside a real (non-default) stream
		cudaStream_t st;
		cudaEvent_t e0, e1;
		if (cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) == cudaSuccess &&
				cudaEventCreateWithFlags(&e0, cudaEventDisableTiming) == cudaSuccess &&
				cudaEventCreateWithFlags(&e1, cudaEventDisableTiming) == cudaSuccess) {
			side_stream_ = st; ev_side_fork_ = e0; ev_side_join_ = e1;
		}
	}
	if ((rc = cnb_reserve_scratch(ctx_, scratchBytes(B))) != CNB_OK) { fail(rc, "scratch"); return false; }

	// 1. weights: one block of value planes and one block of dz* planes with the same layout,
	//    in backward order (reverse insertion), so gradient buckets complete front to back.
	std::vector<CFunc*> weights;
	for (auto it = func_list_.rbegin(); it != func_list_.rend(); ++it) {
		CFunc* f = *it;
		if (!f->batched_ || dynamic_cast<CEmbedding*>(f)) weights.push_back(f);
	}
	size_t total = 0;
	for (auto f : weights) total += 2 * pad64(f->is_input_ && f->batched_ ? f->in_size_ : f->out_size_);
	void* p = nullptr;
	if (total) {
		if ((rc = cnb_alloc(ctx_, total * sizeof(float), &p)) != CNB_OK) { fail(rc, "weights"); return false; }
		weight_base_ = static_cast<float*>(p);
		if ((rc = cnb_alloc(ctx_, total * sizeof(float), &p)) != CNB_OK) { fail(rc, "weight gradients"); return false; }
		wgrad_base_ = static_cast<float*>(p);
		wgrad_count_ = total;
		cnb_memset0(ctx_, weight_base_, total * sizeof(float), stream_);
		cnb_memset0(ctx_, wgrad_base_, total * sizeof(float), stream_);
	}
	size_t off = 0;
	// Fewer, larger buckets amortise the per-collective latency; the last one is exposed after backward.  Four
	// buckets of two blocks each at the benchmark net: 1.36 ms per step at 4 GPUs against 1.42 with eight, 1.46 with two.
	size_t bucket_floats = 4500000;
	if (const char* e = getenv("CNB_BUCKET_FLOATS")) bucket_floats = (size_t) atoll(e);
	size_t bucket_begin = 0, bucket_first = 0;
	for (size_t k = 0; k < weights.size(); ++k) {
		CFunc* f = weights[k];
		CEmbedding* e = dynamic_cast<CEmbedding*>(f);
		size_t len = e ? (size_t) f->in_size_ : (size_t) f->out_size_;
		Vars v;
		v.length_ = e ? e->embeddingDim() : (int) len;
		v.rows_ = e ? e->noEmbeddings() : 1;
		v.real_ = weight_base_ + off;            v.dz_star_real_ = wgrad_base_ + off;
		v.imag_ = weight_base_ + off + pad64(len); v.dz_star_imag_ = wgrad_base_ + off + pad64(len);
		off += 2 * pad64(len);
		if (e) e->table_ = v; else f->out_ = v;
		if (off - bucket_begin >= bucket_floats || k + 1 == weights.size()) {
			// complete once the earliest-inserted consumer of any of its weights has run backward
			CFunc* last = nullptr;
			size_t best = func_list_.size();
			for (size_t j = bucket_first; j <= k; ++j) {
				CFunc* w = weights[j];
				std::vector<CFunc*> users = w->next_func_;
				if (dynamic_cast<CEmbedding*>(w)) users.assign(1, w);
				for (auto u : users) {
					size_t pos = std::find(func_list_.begin(), func_list_.end(), u) - func_list_.begin();
					if (pos < best) { best = pos; last = u; }
				}
			}
			buckets_.push_back(Bucket{bucket_begin, off - bucket_begin, last});
			bucket_begin = off;
			bucket_first = k + 1;
		}
	}
	// 2. activations and their dL/dz* planes
	for (auto f : func_list_) {
		if (!f->batched_) continue;
		size_t n = pad64((size_t) B * f->out_size_);
		f->out_.length_ = f->out_size_;
		f->out_.rows_ = B;
		if (f->is_output_) continue;            // the loss has no output tensor
		bool alias = false;
		if (Linear* l = dynamic_cast<Linear*>(f)) alias = l->fused_residual_ != nullptr;
		if (alias) continue;                    // bound to the Residual's tensors below
		if (Hadamard* hd = dynamic_cast<Hadamard*>(f))
			if (hd->in_fft_epilogue_) continue;         // a = u o h is never stored (recomputed in the backward)
		bool need_grad = !(dynamic_cast<Hadamard*>(f) && static_cast<Hadamard*>(f)->fused_gelu_);
		size_t planes = need_grad ? 4 : 2;
		if ((rc = cnb_alloc(ctx_, planes * n * sizeof(float), &p)) != CNB_OK) { fail(rc, f->getName()); return false; }
		float* base = static_cast<float*>(p);
		f->out_.real_ = base; f->out_.imag_ = base + n;
		if (need_grad) { f->out_.dz_star_real_ = base + 2 * n; f->out_.dz_star_imag_ = base + 3 * n; }
	}
	// A Residual hands its dL/dz* to both operands unchanged.  Where the skip operand p gets every other
	// contribution later in the backward pass than the last reader of the Residual's gradient, p's gradient
	// planes ARE the Residual's planes: the pass-through copy disappears and the later contributions
	// accumulate in place.  Walked from the output side so that a chain of blocks shares one tensor.
	{
		std::map<CFunc*, size_t> pos;
		for (size_t k = 0; k < func_list_.size(); ++k) pos[func_list_[k]] = k;
		for (auto it = func_list_.rbegin(); it != func_list_.rend(); ++it) {
			Residual* r = dynamic_cast<Residual*>(*it);
			if (!r || !r->out_.dz_star_real_ || r->prev_func_[0] == r->prev_func_[1]) continue;
			for (int k = 0; k < 2; ++k) {
				CFunc* sp = r->prev_func_[k];
				CFunc* q = r->prev_func_[1 - k];
				Linear* ql = dynamic_cast<Linear*>(q);
				Linear* pl = dynamic_cast<Linear*>(sp);
				if (!sp->batched_ || !sp->out_.dz_star_real_ || (pl && pl->fused_residual_ == r)) continue;
				// the Residual itself reads the gradient; a Linear fused with it reads it again in its own backward
				size_t reader = (ql && ql->fused_residual_ == r) ? pos[q] : pos[r];
				bool later = true;
				for (auto c : sp->next_func_) if (c != r && pos[c] >= reader) later = false;
				if (!later) continue;
				sp->out_.dz_star_real_ = r->out_.dz_star_real_;
				sp->out_.dz_star_imag_ = r->out_.dz_star_imag_;
				r->grad_transient_ = true;
				break;
			}
		}
	}
	for (auto f : func_list_) {
		if (Linear* l = dynamic_cast<Linear*>(f)) {
			if (l->fused_residual_) {
				Vars v = l->fused_residual_->out_;
				l->out_ = v;
				l->grad_transient_ = l->fused_residual_->grad_transient_;
			}
		}
		size_t eb = f->extraBytes(B);
		if (eb) {
			if ((rc = cnb_alloc(ctx_, eb, &p)) != CNB_OK) { fail(rc, f->getName()); return false; }
			f->bindExtra(static_cast<char*>(p), B);
		}
	}
	{
		size_t gs = 0;
		for (auto f : func_list_)
			if (Linear* l = dynamic_cast<Linear*>(f))
				if (l->use_split_) gs = std::max(gs, cnb_split_floats((size_t) B * l->outSize()) * sizeof(float));
		if (gs) {
			if ((rc = cnb_alloc(ctx_, gs, &p)) != CNB_OK) { fail(rc, "gradient split planes"); return false; }
			g_split_ = static_cast<float*>(p);
		}
	}
	// 3. upload the host copies of the weights
	for (auto f : inputs_) {
		if (f == main_in_ && !dynamic_cast<CEmbedding*>(f)) continue;
		if (!f->host_re_.empty())
			setInputValues(f->uid_, f->host_re_.data(), f->host_im_.data(), (int) f->host_re_.size());
	}
	cnb_sync(ctx_, stream_);
	return ok_;
}

bool CNet::setInputValues(int uid, const float* re, const float* im, int len) {
	auto it = map_.find(uid);
	if (it == map_.end() || !it->second->is_input_) { fail(CNB_ERR_ARG, "setInputValues: uid is not an input"); return false; }
	CFunc* f = it->second;
	CEmbedding* e = dynamic_cast<CEmbedding*>(f);
	int want = e ? f->in_size_ : f->out_size_;
	if (len != want) { fail(CNB_ERR_ARG, f->getName() + ": setInputValues length"); return false; }
	f->host_re_.assign(re, re + len);
	f->host_im_.assign(im, im + len);
	if (!ctx_) return true;
	const Vars& v = e ? e->table_ : f->out_;
	if (f->batched_ && !e) return true;         // data input: filled per batch
	int rc = cnb_h2d(ctx_, v.real_, re, (size_t) len * sizeof(float), stream_);
	if (rc == CNB_OK) rc = cnb_h2d(ctx_, v.imag_, im, (size_t) len * sizeof(float), stream_);
	if (rc == CNB_OK) rc = cnb_sync(ctx_, stream_);
	if (rc != CNB_OK) { fail(rc, "setInputValues"); return false; }
	++weights_version_;
	// a captured step holds no launch that re-splits the Linear weights: it would multiply by the old ones
	if (graph_exec_) graph_stale_ = "weights were set from the host after the step was captured";
	return true;
}

bool CNet::getInputValues(int uid, float* re, float* im, int len) {
	auto it = map_.find(uid);
	if (it == map_.end() || !it->second->is_input_) { fail(CNB_ERR_ARG, "getInputValues: uid is not an input"); return false; }
	CFunc* f = it->second;
	if (!ctx_) {                                 // not on the device yet: the host copies
		if ((size_t) len != f->host_re_.size()) { fail(CNB_ERR_ARG, "getInputValues: length / no values set"); return false; }
		std::copy(f->host_re_.begin(), f->host_re_.end(), re);
		std::copy(f->host_im_.begin(), f->host_im_.end(), im);
		return true;
	}
	CEmbedding* e = dynamic_cast<CEmbedding*>(f);
	const Vars& v = e ? e->table_ : f->out_;
	if ((size_t) len != v.count()) { fail(CNB_ERR_ARG, "getInputValues: length"); return false; }
	int rc = cnb_d2h(ctx_, re, v.real_, (size_t) len * sizeof(float), stream_);
	if (rc == CNB_OK) rc = cnb_d2h(ctx_, im, v.imag_, (size_t) len * sizeof(float), stream_);
	if (rc != CNB_OK) { fail(rc, "getInputValues"); return false; }
	return true;
}

bool CNet::getInputGradients(int uid, float* re, float* im, int len) {
	auto it = map_.find(uid);
	if (it == map_.end() || !it->second->is_input_ || !ctx_) { fail(CNB_ERR_ARG, "getInputGradients: bad uid / not allocated"); return false; }
	CFunc* f = it->second;
	CEmbedding* e = dynamic_cast<CEmbedding*>(f);
	const Vars& v = e ? e->table_ : f->out_;
	if ((size_t) len != v.count() || !v.dz_star_real_) { fail(CNB_ERR_ARG, "getInputGradients: length"); return false; }
	int rc = cnb_d2h(ctx_, re, v.dz_star_real_, (size_t) len * sizeof(float), stream_);
	if (rc == CNB_OK) rc = cnb_d2h(ctx_, im, v.dz_star_imag_, (size_t) len * sizeof(float), stream_);
	if (rc != CNB_OK) { fail(rc, "getInputGradients"); return false; }
	return true;
}

bool CNet::getInputsFromGpu() {
	for (auto f : inputs_) {
		CEmbedding* e = dynamic_cast<CEmbedding*>(f);
		if (f->batched_ && !e) continue;
		size_t n = e ? e->table_.count() : f->out_.count();
		f->host_re_.resize(n);
		f->host_im_.resize(n);
		if (!getInputValues(f->uid_, f->host_re_.data(), f->host_im_.data(), (int) n)) return false;
	}
	return true;
}

bool CNet::batchToGpu(const float* re, const float* im, const int* tokens, const int* labels, int B) {
	if (!ctx_) { fail(CNB_ERR_ARG, "batchToGpu: allocateOnGpu first"); return false; }
	if (B <= 0 || B > batch_) { fail(CNB_ERR_ARG, "batchToGpu: batch " + std::to_string(B) + " exceeds the allocated " + std::to_string(batch_)); return false; }
	cur_batch_ = B;
	int rc = CNB_OK;
	if (CEmbedding* e = dynamic_cast<CEmbedding*>(main_in_)) {
		if (!tokens) { fail(CNB_ERR_ARG, "batchToGpu: token ids expected"); return false; }
		rc = cnb_h2d(ctx_, e->tokens_, tokens, (size_t) B * e->noOutTokens() * sizeof(int32_t), stream_);
	} else {
		if (!re || !im) { fail(CNB_ERR_ARG, "batchToGpu: re/im planes expected"); return false; }
		size_t bytes = (size_t) B * main_in_->out_size_ * sizeof(float);
		rc = cnb_h2d(ctx_, main_in_->out_.real_, re, bytes, stream_);
		if (rc == CNB_OK) rc = cnb_h2d(ctx_, main_in_->out_.imag_, im, bytes, stream_);
	}
	if (rc == CNB_OK && labels) rc = cnb_h2d(ctx_, main_out_->labels_, labels, (size_t) B * sizeof(int32_t), stream_);
	if (rc != CNB_OK) { fail(rc, "batchToGpu"); return false; }
	return true;
}

bool CNet::pipelineInit() {
	if (copy_stream_) return true;
	cudaStream_t st;
	cudaEvent_t e[4];
	if (cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) != cudaSuccess) { fail(CNB_ERR_CUDA, "pipeline: stream"); return false; }
	for (int i = 0; i < 4; ++i)
		if (cudaEventCreateWithFlags(&e[i], cudaEventDisableTiming) != cudaSuccess) { fail(CNB_ERR_CUDA, "pipeline: event"); return false; }
	copy_stream_ = st; ev_h2d_ = e[0]; ev_commit_ = e[1]; ev_step_ = e[2]; ev_d2h_ = e[3];
	size_t in_bytes = 0;
	if (CEmbedding* em = dynamic_cast<CEmbedding*>(main_in_)) in_bytes = (size_t) batch_ * em->noOutTokens() * sizeof(int32_t);
	else in_bytes = 2 * (size_t) batch_ * main_in_->out_size_ * sizeof(float);
	void* p = nullptr;
	int rc = cnb_alloc(ctx_, in_bytes, &p);
	if (rc != CNB_OK) { fail(rc, "pipeline staging"); return false; }
	stage_in_ = static_cast<char*>(p);
	if ((rc = cnb_alloc(ctx_, (size_t) batch_ * sizeof(int32_t), &p)) != CNB_OK) { fail(rc, "pipeline staging"); return false; }
	stage_labels_ = static_cast<int32_t*>(p);
	return true;
}

bool CNet::prefetchBatch(const float* re, const float* im, const int* tokens, const int* labels, int B) {
	if (!ctx_) { fail(CNB_ERR_ARG, "prefetchBatch: allocateOnGpu first"); return false; }
	if (B <= 0 || B > batch_) { fail(CNB_ERR_ARG, "prefetchBatch: batch " + std::to_string(B) + " exceeds the allocated " + std::to_string(batch_)); return false; }
	if (!pipelineInit()) return false;
	cudaStream_t cs = (cudaStream_t) copy_stream_;
	cudaError_t e = cudaStreamWaitEvent(cs, (cudaEvent_t) ev_commit_, 0);      // staging of the previous batch consumed
	if (CEmbedding* em = dynamic_cast<CEmbedding*>(main_in_)) {
		if (!tokens) { fail(CNB_ERR_ARG, "prefetchBatch: token ids expected"); return false; }
		if (e == cudaSuccess) e = cudaMemcpyAsync(stage_in_, tokens, (size_t) B * em->noOutTokens() * sizeof(int32_t), cudaMemcpyHostToDevice, cs);
	} else {
		if (!re || !im) { fail(CNB_ERR_ARG, "prefetchBatch: re/im planes expected"); return false; }
		size_t bytes = (size_t) B * main_in_->out_size_ * sizeof(float);
		if (e == cudaSuccess) e = cudaMemcpyAsync(stage_in_, re, bytes, cudaMemcpyHostToDevice, cs);
		if (e == cudaSuccess) e = cudaMemcpyAsync(stage_in_ + bytes, im, bytes, cudaMemcpyHostToDevice, cs);
	}
	if (e == cudaSuccess && labels) e = cudaMemcpyAsync(stage_labels_, labels, (size_t) B * sizeof(int32_t), cudaMemcpyHostToDevice, cs);
	if (e == cudaSuccess) e = cudaEventRecord((cudaEvent_t) ev_h2d_, cs);
	if (e != cudaSuccess) { fail(CNB_ERR_CUDA, std::string("prefetchBatch: ") + cudaGetErrorString(e)); return false; }
	staged_batch_ = B;
	return true;
}

bool CNet::commitBatch() {
	if (!copy_stream_ || staged_batch_ <= 0) { fail(CNB_ERR_ARG, "commitBatch: no staged batch"); return false; }
	cudaStream_t ms = (cudaStream_t) stream_;
	int B = staged_batch_;
	cudaError_t e = cudaStreamWaitEvent(ms, (cudaEvent_t) ev_h2d_, 0);
	if (e == cudaSuccess && d2h_pending_) e = cudaStreamWaitEvent(ms, (cudaEvent_t) ev_d2h_, 0);   // losses of the last step are out
	if (CEmbedding* em = dynamic_cast<CEmbedding*>(main_in_)) {
		if (e == cudaSuccess) e = cudaMemcpyAsync(em->tokens_, stage_in_, (size_t) B * em->noOutTokens() * sizeof(int32_t), cudaMemcpyDeviceToDevice, ms);
	} else {
		size_t bytes = (size_t) B * main_in_->out_size_ * sizeof(float);
		if (e == cudaSuccess) e = cudaMemcpyAsync(main_in_->out_.real_, stage_in_, bytes, cudaMemcpyDeviceToDevice, ms);
		if (e == cudaSuccess) e = cudaMemcpyAsync(main_in_->out_.imag_, stage_in_ + bytes, bytes, cudaMemcpyDeviceToDevice, ms);
	}
	if (e == cudaSuccess) e = cudaMemcpyAsync(main_out_->labels_, stage_labels_, (size_t) B * sizeof(int32_t), cudaMemcpyDeviceToDevice, ms);
	if (e == cudaSuccess) e = cudaEventRecord((cudaEvent_t) ev_commit_, ms);
	if (e != cudaSuccess) { fail(CNB_ERR_CUDA, std::string("commitBatch: ") + cudaGetErrorString(e)); return false; }
	cur_batch_ = B;
	staged_batch_ = 0;
	return true;
}

bool CNet::readLossesAsync(float* host_out, int n) {
	if (!ctx_ || n <= 0 || n > cur_batch_) { fail(CNB_ERR_ARG, "readLossesAsync: bad count"); return false; }
	if (!pipelineInit()) return false;
	cudaStream_t cs = (cudaStream_t) copy_stream_;
	cudaError_t e = cudaEventRecord((cudaEvent_t) ev_step_, (cudaStream_t) stream_);
	if (e == cudaSuccess) e = cudaStreamWaitEvent(cs, (cudaEvent_t) ev_step_, 0);
	if (e == cudaSuccess) e = cudaMemcpyAsync(host_out, main_out_->loss_, (size_t) n * sizeof(float), cudaMemcpyDeviceToHost, cs);
	if (e == cudaSuccess) e = cudaEventRecord((cudaEvent_t) ev_d2h_, cs);
	if (e != cudaSuccess) { fail(CNB_ERR_CUDA, std::string("readLossesAsync: ") + cudaGetErrorString(e)); return false; }
	d2h_pending_ = true;
	return true;
}

bool CNet::waitLosses() {
	if (!d2h_pending_) return true;
	cudaError_t e = cudaEventSynchronize((cudaEvent_t) ev_d2h_);
	if (e != cudaSuccess) { fail(CNB_ERR_CUDA, std::string("waitLosses: ") + cudaGetErrorString(e)); return false; }
	return true;
}

void CNet::forward() {
	if (!ctx_) { fail(CNB_ERR_ARG, "forward: allocateOnGpu first (there is no CPU path)"); return; }
	for (auto f : func_list_) {
		if (f->fused_away_) continue;
		f->forward();
		if (!ok_) return;
	}
}

void CNet::backward() {
	if (!ctx_) { fail(CNB_ERR_ARG, "backward: allocateOnGpu first (there is no CPU path)"); return; }
	for (auto f : func_list_) f->grad_written_ = false;
	main_out_->prev_func_[0]->grad_written_ = true;        // seeded by CrossEntropy::forward
	if (dp_gemm_ctas_ > 0) cnb_set_gemm_sm_limit(ctx_, dp_gemm_ctas_);
	size_t next_bucket = 0;
	for (auto it = func_list_.rbegin(); it != func_list_.rend(); ++it) {
		CFunc* f = *it;
		if (!f->fused_away_ || dynamic_cast<Residual*>(f)) f->backward();
		if (!ok_) return;
		while (next_bucket < buckets_.size() && buckets_[next_bucket].last_writer == f) {
			if (!reduceBucket(next_bucket)) return;
			++next_bucket;
		}
	}
	while (next_bucket < buckets_.size()) {
		if (!reduceBucket(next_bucket)) return;
		++next_bucket;
	}
}

bool CNet::reduceBucket(size_t k) {
	const Bucket& b = buckets_[k];
	if ((nccl_.active() || sym_active_ || hook_) && k == 0) {
		// The arena accumulates until the update and is summed over the ranks in place: a second backward()
		// before the update would reduce the already reduced part again (earlier micro-batches x ranks).
		if (reduced_since_update_) {
			fail(CNB_ERR_UNSUPPORTED, "backward: a second backward pass before updateInputs while gradients are reduced over the "
					"ranks in place; gradient accumulation over micro-batches is not available with data parallelism");
			return false;
		}
		reduced_since_update_ = true;
	}
	if (sym_active_) {
		cudaStream_t cs = (cudaStream_t) sym_stream_;
		if (cudaEventRecord((cudaEvent_t) ev_sym_fork_, (cudaStream_t) stream_) != cudaSuccess ||
				cudaStreamWaitEvent(cs, (cudaEvent_t) ev_sym_fork_, 0) != cudaSuccess) {
			fail(CNB_ERR_CUDA, "all-reduce: fork to the communication stream failed"); return false;
		}
		int rc = cnb_dp_allreduce(ctx_, &sym_, wgrad_base_ + b.begin, b.count, sym_stream_);
		if (rc != CNB_OK) { fail(rc, "all-reduce"); return false; }
		sym_pending_ = true;
	} else if (nccl_.active()) {
		if (!nccl_.allReduce(wgrad_base_ + b.begin, b.count, stream_)) { fail(CNB_ERR_CUDA, "all-reduce: " + nccl_.error()); return false; }
	}
	if (hook_) {
		int rc = hook_(hook_user_, wgrad_base_ + b.begin, b.count, (int) k, (int) buckets_.size());
		if (rc != 0) { fail(CNB_ERR_DEVICE, "gradient bucket hook returned " + std::to_string(rc)); return false; }
	}
	return true;
}

bool CNet::joinCollectives() {
	if (!nccl_.join(stream_)) { fail(CNB_ERR_CUDA, "all-reduce join: " + nccl_.error()); return false; }
	if (sym_pending_) {
		if (cudaEventRecord((cudaEvent_t) ev_sym_join_, (cudaStream_t) sym_stream_) != cudaSuccess ||
				cudaStreamWaitEvent((cudaStream_t) stream_, (cudaEvent_t) ev_sym_join_, 0) != cudaSuccess) {
			fail(CNB_ERR_CUDA, "all-reduce join: from the communication stream failed"); return false;
		}
		sym_pending_ = false;
	}
	return true;
}

bool CNet::allReduceGradients() {
	if (!ctx_) { fail(CNB_ERR_ARG, "allReduceGradients: allocateOnGpu first"); return false; }
	const bool hook_was = hook_ != nullptr;
	BucketHook h = hook_;
	hook_ = nullptr;                                // only the device collectives
	bool flag = reduced_since_update_;
	reduced_since_update_ = false;
	bool ok = true;
	for (size_t k = 0; k < buckets_.size() && ok; ++k) ok = reduceBucket(k);
	reduced_since_update_ = flag;
	if (hook_was) hook_ = h;
	return ok && joinCollectives();
}

bool CNet::setSymmetricPeers(int rank, int world, void* multicast_base, void* const* arena_bases, void* const* flag_blocks, int ctas) {
	if (!ctx_ || !ext_arena_) { fail(CNB_ERR_ARG, "setSymmetricPeers: allocateOnGpu on a caller-owned (symmetric) arena first"); return false; }
	if (world < 1 || world > CNB_DP_MAX_RANKS || rank < 0 || rank >= world) { fail(CNB_ERR_ARG, "setSymmetricPeers: rank / world"); return false; }
	if (world == 1) return true;
	if (arena_bases[rank] != ext_arena_) { fail(CNB_ERR_ARG, "setSymmetricPeers: arena_bases[rank] is not this net's arena"); return false; }
	for (const Bucket& b : buckets_)
		if (b.begin % 4 || b.count % (4 * (size_t) world)) { fail(CNB_ERR_UNSUPPORTED, "setSymmetricPeers: a gradient bucket is not a multiple of 4 x world floats"); return false; }
	cudaSetDevice(device_);
	sym_ = cnb_dp_peers{};
	sym_.rank = rank; sym_.world = world; sym_.multicast_base = multicast_base; sym_.arena_bytes = arena_bytes_; sym_.ctas = ctas;
	for (int r = 0; r < world; ++r) { sym_.arena_base[r] = arena_bases[r]; sym_.flags[r] = flag_blocks[r]; }
	void* p = nullptr;
	int rc = cnb_alloc(ctx_, cnb_dp_state_bytes(), &p);
	if (rc != CNB_OK) { fail(rc, "setSymmetricPeers: state"); return false; }
	cnb_memset0(ctx_, p, cnb_dp_state_bytes(), stream_);
	cnb_sync(ctx_, stream_);
	sym_.state = p;
	cudaStream_t st;
	cudaEvent_t e0, e1;
	if (cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking) != cudaSuccess ||
			cudaEventCreateWithFlags(&e0, cudaEventDisableTiming) != cudaSuccess ||
			cudaEventCreateWithFlags(&e1, cudaEventDisableTiming) != cudaSuccess) {
		fail(CNB_ERR_CUDA, "setSymmetricPeers: stream / events"); return false;
	}
	sym_stream_ = st; ev_sym_fork_ = e0; ev_sym_join_ = e1;
	sym_active_ = true;
	{   // SMs left to the reduction's CTAs during backward(), as for NCCL's
		int reserve = ctas > 0 ? ctas : 6;
		if (const char* e = getenv("CNB_DP_RESERVED_SMS")) reserve = atoi(e);
		int sms = 0;
		cnb_device_info(device_, &sms, nullptr, nullptr, nullptr);
		if (reserve > 0 && sms > reserve) dp_gemm_ctas_ = sms - reserve;
	}
	return true;
}

bool CNet::setDataParallel(const char id[kNcclUniqueIdBytes], int rank, int nranks) {
	if (!ctx_) { fail(CNB_ERR_ARG, "setDataParallel: allocateOnGpu first"); return false; }
	cudaSetDevice(device_);
	if (!nccl_.init(id, rank, nranks)) { fail(CNB_ERR_CUDA, "setDataParallel: " + nccl_.error()); return false; }
	if (nccl_.active() && own_nccl_arena_) {
		// weights and their gradients (allocated back to back, first in the arena) as one symmetric window:
		// NCCL then reduces them with its symmetric-memory kernels (peer / in-switch access on the buffers
		// themselves, no staging copies, fewer CTAs).  CNB_DP_SYMM=0 leaves the buffers unregistered.
		const char* e = getenv("CNB_DP_SYMM");
		if (!(e && e[0] == '0') && weight_base_ && wgrad_base_) {
			uintptr_t lo = reinterpret_cast<uintptr_t>(weight_base_) & ~uintptr_t(4095);
			uintptr_t hi = (reinterpret_cast<uintptr_t>(wgrad_base_ + wgrad_count_) + 4095) & ~uintptr_t(4095);
			uintptr_t end = reinterpret_cast<uintptr_t>(own_nccl_arena_) + arena_bytes_;
			if (hi > end) hi = end;
			if (!nccl_.registerWindow(reinterpret_cast<void*>(lo), hi - lo)) {
				// not fatal: the all-reduce then runs NCCL's copy-based kernels on the unregistered arena
				std::cerr << "cnet_b200: gradients not registered as a symmetric window (" << nccl_.error() << ")" << std::endl;
			}
		}
	}
	if (nccl_.active()) {
		// the GEMM is one CTA per SM and fills shared memory; keep a few SMs for NCCL's kernels so the
		// bucket all-reduces really overlap the backward pass (CNB_DP_RESERVED_SMS overrides, 0 = none)
		// On a registered symmetric window NCCL reduces in the switch with a handful of CTAs (5 at 4 ranks); its
		// copy-based kernels on unregistered buffers want more.  Measured at 4 GPUs, 1024 rows each: 6 reserved
		// SMs 1.36 ms per step, 12: 1.45, none: 1.54.
		int reserve = nccl_.hasWindow() ? (nranks >= 8 ? 8 : 6) : 12;     // 8 ranks: not measured here, one SM per peer
		if (const char* e = getenv("CNB_DP_RESERVED_SMS")) reserve = atoi(e);
		int sms = 0;
		cnb_device_info(device_, &sms, nullptr, nullptr, nullptr);
		if (reserve > 0 && sms > reserve) dp_gemm_ctas_ = sms - reserve;   // applied during backward()
	}
	return true;
}

bool CNet::beginCapture() {
	if (!ctx_ || capturing_) { fail(CNB_ERR_ARG, "beginCapture: not allocated / already capturing"); return false; }
	if (!stream_) { fail(CNB_ERR_ARG, "beginCapture: the legacy default stream cannot be captured; setStream first"); return false; }
	cudaError_t e = cudaStreamBeginCapture((cudaStream_t) stream_, cudaStreamCaptureModeThreadLocal);
	if (e != cudaSuccess) { fail(CNB_ERR_CUDA, std::string("cudaStreamBeginCapture: ") + cudaGetErrorString(e)); return false; }
	capturing_ = true;
	graph_launches_ = cnb_launch_count();
	graph_batch_ = cur_batch_;
	return true;
}

bool CNet::endCapture() {
	if (!capturing_) { fail(CNB_ERR_ARG, "endCapture: no capture in progress"); return false; }
	// a backward() captured without an update leaves collectives on the communication stream: bring it back
	// into the capturing stream, or the capture cannot end
	joinCollectives();
	capturing_ = false;
	graph_launches_ = cnb_launch_count() - graph_launches_;
	cudaGraph_t g = nullptr;
	cudaError_t e = cudaStreamEndCapture((cudaStream_t) stream_, &g);
	if (e != cudaSuccess || !g) { fail(CNB_ERR_CUDA, std::string("cudaStreamEndCapture: ") + cudaGetErrorString(e)); return false; }
	if (!ok_) { cudaGraphDestroy(g); return false; }       // a layer failed while capturing
	if (graph_exec_) { cudaGraphExecDestroy((cudaGraphExec_t) graph_exec_); graph_exec_ = nullptr; }
	cudaGraphExec_t x = nullptr;
	e = cudaGraphInstantiate(&x, g, 0);
	cudaGraphDestroy(g);
	if (e != cudaSuccess) { fail(CNB_ERR_CUDA, std::string("cudaGraphInstantiate: ") + cudaGetErrorString(e)); return false; }
	graph_exec_ = x;
	graph_stale_.clear();
	return true;
}

bool CNet::launchGraph() {
	if (!graph_exec_) { fail(CNB_ERR_ARG, "launchGraph: capture a step first"); return false; }
	// grids, row counts and the "weights are already split" decision were frozen at capture time
	if (cur_batch_ != graph_batch_) {
		fail(CNB_ERR_ARG, "launchGraph: the batch in flight has " + std::to_string(cur_batch_) + " rows, the captured step was sized for " +
				std::to_string(graph_batch_) + "; capture again");
		return false;
	}
	if (!graph_stale_.empty()) { fail(CNB_ERR_ARG, "launchGraph: " + graph_stale_ + "; capture again"); return false; }
	cudaError_t e = cudaGraphLaunch((cudaGraphExec_t) graph_exec_, (cudaStream_t) stream_);
	if (e != cudaSuccess) { fail(CNB_ERR_CUDA, std::string("cudaGraphLaunch: ") + cudaGetErrorString(e)); return false; }
	return true;
}

void CNet::backward(int label) {
	if (!ctx_) { fail(CNB_ERR_ARG, "backward: allocateOnGpu first (there is no CPU path)"); return; }
	main_out_->backward(label);
	backward();
}

void CNet::updateInputs(float lr) {
	if (!ctx_ || !wgrad_count_) return;
	if (dp_gemm_ctas_ > 0) cnb_set_gemm_sm_limit(ctx_, 0);
	if (!joinCollectives()) return;
	// the new Linear weights leave the update already split, once, for the next forward and dX* products
	std::vector<cnb_split_span> spans;
	std::vector<Linear*> fused;
	for (auto f : func_list_) {
		Linear* l = dynamic_cast<Linear*>(f);
		if (!l || !l->use_split_ || spans.size() + 2 > CNB_MAX_SPLIT_SPANS || wgrad_count_ % 4) continue;
		const Vars& w = l->prev_func_[1]->out_;
		const size_t np = cnb_split_floats((size_t) l->in2_len) / 4;
		if (l->in2_len % 4 || w.real_ < weight_base_ || w.imag_ + l->in2_len > weight_base_ + wgrad_count_) continue;
		// slots of the split buffer: hi_re, hi_im (fp32), then [h16_re ; h16_im] and [l16_re ; l16_im] as bf16
		uint16_t* h16 = reinterpret_cast<uint16_t*>(l->w_split_ + 2 * np);
		uint16_t* l16 = reinterpret_cast<uint16_t*>(l->w_split_ + 3 * np);
		spans.push_back({(size_t) (w.real_ - weight_base_), (size_t) l->in2_len, l->w_split_, h16, l16});
		spans.push_back({(size_t) (w.imag_ - weight_base_), (size_t) l->in2_len, l->w_split_ + np, h16 + np, l16 + np});
		fused.push_back(l);
	}
	int rc = spans.empty()
		? cnb_sgd_update(ctx_, weight_base_, wgrad_base_, wgrad_count_, lr, 1, stream_)
		: cnb_sgd_update_split(ctx_, weight_base_, wgrad_base_, wgrad_count_, lr, 1, spans.data(), (int) spans.size(), stream_);
	if (rc != CNB_OK) { fail(rc, "updateInputs"); return; }
	reduced_since_update_ = false;
	++weights_version_;
	for (auto l : fused) l->w_split_version_ = weights_version_;
	for (auto f : func_list_)
		if (Linear* l = dynamic_cast<Linear*>(f))
			if (l->w_split_version_ != weights_version_) l->splitWeights();
}

void CNet::adamUpdate(float lr, float beta, int t) {
	if (!ctx_ || !wgrad_count_) return;
	if (capturing_) {       // the bias correction 1 - beta^(t+1) is a launch parameter: a replay would reuse step t's
		fail(CNB_ERR_UNSUPPORTED, "adamUpdate: cannot be captured in a CUDA graph (its step count is a launch parameter); "
				"capture forward + backward and call adamUpdate outside the graph");
		return;
	}
	if (dp_gemm_ctas_ > 0) cnb_set_gemm_sm_limit(ctx_, 0);
	if (!joinCollectives()) return;
	if (!momentum_base_) {
		void* p = nullptr;
		int rc = cnb_alloc(ctx_, wgrad_count_ * sizeof(float), &p);
		if (rc != CNB_OK) { fail(rc, "adamUpdate: momentum planes (size the arena for them)"); return; }
		momentum_base_ = static_cast<float*>(p);
		cnb_memset0(ctx_, momentum_base_, wgrad_count_ * sizeof(float), stream_);
	}
	int rc = cnb_adam_update(ctx_, weight_base_, momentum_base_, wgrad_base_, wgrad_count_, lr, beta, t, stream_);
	if (rc != CNB_OK) { fail(rc, "adamUpdate"); return; }
	reduced_since_update_ = false;
	++weights_version_;
	for (auto f : func_list_)
		if (Linear* l = dynamic_cast<Linear*>(f)) l->splitWeights();
}

void CNet::infer() {
	infer_only_ = true;
	forward();
	infer_only_ = false;
}

bool CNet::gpuForward(InputFunc* inp, OutputFunc* outp, InputBatch& b) {
	if (dynamic_cast<CFunc*>(inp) != main_in_ || dynamic_cast<CFunc*>(outp) != main_out_) {
		fail(CNB_ERR_ARG, "gpuForward: not the main input / output"); return false;
	}
	if (!batchToGpu(b.realDataPtr(), b.imagDataPtr(), nullptr, b.labelsPtr(), b.size())) return false;
	forward();
	return ok_;
}

bool CNet::gpuForward(InputFunc* inp, OutputFunc* outp, EmbeddingBatch& b) {
	if (dynamic_cast<CFunc*>(inp) != main_in_ || dynamic_cast<CFunc*>(outp) != main_out_) {
		fail(CNB_ERR_ARG, "gpuForward: not the main input / output"); return false;
	}
	if (!batchToGpu(nullptr, nullptr, b.tokensPtr(), b.labelsPtr(), b.size())) return false;
	forward();
	return ok_;
}

bool CNet::gpuBackward() { backward(); return ok_; }

bool CNet::getLosses(float* out, int n) {
	if (!ctx_ || n > cur_batch_) { fail(CNB_ERR_ARG, "getLosses: bad count"); return false; }
	int rc = cnb_d2h(ctx_, out, main_out_->loss_, (size_t) n * sizeof(float), stream_);
	if (rc != CNB_OK) { fail(rc, "getLosses"); return false; }
	return true;
}

float CNet::getLoss(OutputFunc* outp, Batch* batch) {
	if (dynamic_cast<CFunc*>(outp) != main_out_) { fail(CNB_ERR_ARG, "getLoss: not the main output"); return NAN; }
	std::vector<float> l(cur_batch_);
	if (!getLosses(l.data(), cur_batch_)) return NAN;
	double s = 0;
	for (float v : l) s += v;
	if (batch) batch->losses_ = l;
	return (float) (s / cur_batch_);
}

bool CNet::sync() {
	int rc = cnb_sync(ctx_, stream_);
	if (rc != CNB_OK) { fail(rc, "sync"); return false; }
	rc = cnb_check_device_status(ctx_, stream_);
	if (rc != CNB_OK) { fail(rc, "device status"); return false; }
	return ok_;
}

bool CNet::readOutput(int uid, int what, float* re, float* im) {
	auto it = map_.find(uid);
	if (it == map_.end() || !ctx_) { fail(CNB_ERR_ARG, "readOutput: bad uid / not allocated"); return false; }
	CFunc* f = it->second;
	const Vars& v = f->out_;
	const float* sr = what == 0 ? v.real_ : v.dz_star_real_;
	const float* si = what == 0 ? v.imag_ : v.dz_star_imag_;
	if (Linear* l = dynamic_cast<Linear*>(f)) {
		if (l->fused_residual_ && what == 0) sr = nullptr;   // only the post-Residual sum exists
	}
	if (what != 0 && f->grad_transient_) sr = nullptr;       // overwritten by the gradient of the Residual's operand
	if (!sr) { fail(CNB_ERR_ARG, f->getName() + ": tensor not materialised (fused)"); return false; }
	size_t n = (size_t) (f->batched_ ? cur_batch_ : 1) * f->out_size_;
	if (what == 0 && f->value_split_) {
		// Only the operand split of the value was stored: hi (the value cut to TF32) plus the bf16 rounding of
		// the remainder gives it back to 2^-19 relative, which is what the consuming product saw of it.
		const size_t np = cnb_split_floats((size_t) cur_batch_ * f->out_size_) / 4;   // plane pitch of the batch in flight
		std::vector<uint16_t> lo(n);
		const uint16_t* l16 = reinterpret_cast<const uint16_t*>(f->value_split_ + 3 * np);
		for (int q = 0; q < 2; ++q) {
			float* dst = q ? im : re;
			int rc = cnb_d2h(ctx_, dst, f->value_split_ + q * np, n * sizeof(float), stream_);
			if (rc == CNB_OK) rc = cnb_d2h(ctx_, lo.data(), l16 + q * np, n * sizeof(uint16_t), stream_);
			if (rc == CNB_OK) rc = cnb_sync(ctx_, stream_);
			if (rc != CNB_OK) { fail(rc, "readOutput"); return false; }
			for (size_t k = 0; k < n; ++k) {
				const uint32_t bits = (uint32_t) lo[k] << 16;
				float v;
				std::memcpy(&v, &bits, sizeof v);
				dst[k] += v;
			}
		}
		return true;
	}
	int rc = cnb_d2h(ctx_, re, sr, n * sizeof(float), stream_);
	if (rc == CNB_OK) rc = cnb_d2h(ctx_, im, si, n * sizeof(float), stream_);
	if (rc != CNB_OK) { fail(rc, "readOutput"); return false; }
	return true;
}

}  // namespace cnet_b200
