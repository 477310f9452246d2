// TEST INFRASTRUCTURE ONLY.  Flat C driver around the *unmodified* reference
// CPU path (ComplexNet, impl/cnet.h) so that Python tests and the bench's CPU
// baseline can build a net, run the reference's own per-sample
// forward / loss / backward(label) loop and read back what it computed.
//
// Nothing of the reference is copied here: the reference headers are included
// from where they lie (-I<reference root>) and this file only calls their
// public API:
//   ComplexNet::add / forward / backward(label) / update   impl/cnet.h:228-289, 366-421
//   CInput::setInput-equivalent plane copies               impl/cinput.h:82-88
//   CEmbedding::setInput(std::vector<int>)                 impl/embed.h:91-99
//   CrossEntropy::loss(label)                              impl/crossent.h:50-55
//
// The step it runs is the reference trainer's loop (cnet.cpp:58-102):
//   for b in batch: setInput; forward; loss; backward(label_b)
//   update(lr, batch)          -> w -= (lr/batch) * sum_b dz*_w
#include "impl/cnet.h"
#include "impl/model_saver.h"

#include <chrono>
#include <map>
#include <vector>

namespace {

struct Record {
	int out_size = 0;
	std::vector<float> act_re, act_im;     // [B, out_size] output of the function
	std::vector<float> gs_re, gs_im;       // [B, out_size] dL/dz* of that output
	std::vector<float> g_re, g_im;         // [B, out_size] dL/dz  of that output
};

struct RefNet {
	ComplexNet net;
	std::vector<int> uids;                 // insertion order
	std::map<int, Record> rec;
	int batch = 0;
};

inline CFunc* fn(RefNet* r, int uid) { return r->net[uid]; }

}  // namespace

extern "C" {

void* ref_create() {
	FILELog::ReportingLevel() = lError;   // the reference logs every forward() at DEBUG by default
	return new RefNet();
}

void ref_destroy(void* h) { delete static_cast<RefNet*>(h); }

void ref_set_threads(int n) { omp_set_num_threads(n); }

int ref_max_threads() { return omp_get_max_threads(); }

// type ids are the reference's own (impl/cnet.h:31-44).
int ref_add(void* h, int type, int a, int b, int c, const int* prev, int nprev) {
	RefNet* r = static_cast<RefNet*>(h);
	CFunc* f = NULL;
	switch (type) {
	case isInput:        f = new CInput(OutSize(a)); break;
	case isEmbedding:    f = new CEmbedding(a, b, c); break;       // dim, max tokens, vocab
	case isFourier:      f = new FourierTrans(InSize(a)); break;
	case isHadamard:     f = new Hadamard(InSize(a), InSize(a)); break;
	case isGelu:         f = new CGelu(InSize(a)); break;
	case isLinear:       f = new Linear(InSize(a), InSize(b)); break;  // in1, in2 = in1*out
	case isResidual:     f = new Residual(InSize(a)); break;
	case isSoftMax:      f = new SoftMax(InSize(a)); break;
	case isCrossEntropy: f = new CrossEntropy(InSize(a)); break;
	case isL2Out:        f = new L2Out(InSize(a)); break;
	case isCrelu:        f = new CRelu(InSize(a)); break;
	case isTrianFourier: f = new TriangFourier(InSize(a)); break;
	default: return -1;
	}
	std::vector<int> p(prev, prev + nprev);
	int uid = nprev ? r->net.add(f, p) : r->net.add(f);
	r->uids.push_back(uid);
	return uid;
}

int ref_set_values(void* h, int uid, const float* re, const float* im, int len) {
	CFunc* f = fn(static_cast<RefNet*>(h), uid);
	if (!f || f->input().length_ != len) return -1;
	std::copy(re, re + len, f->mutable_input()->real_);
	std::copy(im, im + len, f->mutable_input()->imag_);
	return 0;
}

int ref_get_values(void* h, int uid, float* re, float* im, int len) {
	CFunc* f = fn(static_cast<RefNet*>(h), uid);
	if (!f || f->input().length_ != len) return -1;
	std::copy(f->input().real_, f->input().real_ + len, re);
	std::copy(f->input().imag_, f->input().imag_ + len, im);
	return 0;
}

// accumulated dL/dz* of an input function (weights / embedding table)
int ref_get_wgrad(void* h, int uid, float* re, float* im, int len) {
	CFunc* f = fn(static_cast<RefNet*>(h), uid);
	if (!f || f->input().length_ != len) return -1;
	std::copy(f->input().dz_star_real_, f->input().dz_star_real_ + len, re);
	std::copy(f->input().dz_star_imag_, f->input().dz_star_imag_ + len, im);
	return 0;
}

int ref_zero_wgrads(void* h) {
	RefNet* r = static_cast<RefNet*>(h);
	for (int uid : r->uids) {
		if (fn(r, uid)->isInput()) fn(r, uid)->mutable_input()->zero_gradients();
	}
	return 0;
}

// One batch of the reference's per-sample loop.  main_uid is the data CInput
// (x planes [B, n]) or the CEmbedding (tokens [B, tok_per_sample], <0 = pad).
// record != 0 keeps every function's output and the gradients of that output
// for each sample; record == 2 leaves out the weight inputs (their "output" is the
// weight itself, B copies of which are gigabytes at the benchmark widths).
int ref_run_batch(void* h, int main_uid, const float* xre, const float* xim,
		const int* tokens, int tok_per_sample, const int* labels, int B,
		float* losses, int record) {
	RefNet* r = static_cast<RefNet*>(h);
	CFunc* in = fn(r, main_uid);
	if (!in) return -1;
	CEmbedding* emb = dynamic_cast<CEmbedding*>(in);
	OutputFunc* ce = NULL;                 // the loss layer: CrossEntropy or L2Out
	for (int uid : r->uids) {
		if (OutputFunc* c = dynamic_cast<OutputFunc*>(fn(r, uid))) ce = c;
	}
	if (!ce) return -2;
	r->batch = B;
	if (record) {
		r->rec.clear();
		for (int uid : r->uids) {
			CFunc* f = fn(r, uid);
			if (!f->no_outputs()) continue;
			if (record == 2 && f->isInput() && f != in) continue;
			Record& rc = r->rec[uid];
			rc.out_size = f->outSize();
			size_t n = (size_t) B * rc.out_size;
			rc.act_re.assign(n, 0.f); rc.act_im.assign(n, 0.f);
			rc.gs_re.assign(n, 0.f);  rc.gs_im.assign(n, 0.f);
			rc.g_re.assign(n, 0.f);   rc.g_im.assign(n, 0.f);
		}
	}
	int n = in->input().length_;
	for (int b = 0; b < B; ++b) {
		if (emb) {
			std::vector<int> toks;
			for (int t = 0; t < tok_per_sample; ++t) {
				int tk = tokens[(size_t) b * tok_per_sample + t];
				if (tk >= 0) toks.push_back(tk);
			}
			emb->setInput(toks);
		} else {
			std::copy(xre + (size_t) b * n, xre + (size_t) (b + 1) * n, in->mutable_input()->real_);
			std::copy(xim + (size_t) b * n, xim + (size_t) (b + 1) * n, in->mutable_input()->imag_);
		}
		r->net.forward();
		if (losses) losses[b] = ce->loss(labels[b]);
		r->net.backward(labels[b]);
		if (!record) continue;
		for (auto& kv : r->rec) {
			CFunc* f = fn(r, kv.first);
			Record& rc = kv.second;
			size_t base = (size_t) b * rc.out_size;
			for (int c = 0; c < f->no_outputs(); ++c) {
				const Vars& v = f->output(c);
				int off = f->offset(c);
				for (int i = 0; i < rc.out_size; ++i) {
					if (c == 0) {
						rc.act_re[base + i] = v.real_[off + i];
						rc.act_im[base + i] = v.imag_[off + i];
					}
					rc.gs_re[base + i] += v.dz_star_real_[off + i];
					rc.gs_im[base + i] += v.dz_star_imag_[off + i];
					rc.g_re[base + i] += v.dz_real_[off + i];
					rc.g_im[base + i] += v.dz_imag_[off + i];
				}
			}
		}
	}
	return 0;
}

// what: 0 = output activations, 1 = dL/dz* of the output, 2 = dL/dz of the output
int ref_get_record(void* h, int uid, int what, float* re, float* im) {
	RefNet* r = static_cast<RefNet*>(h);
	auto it = r->rec.find(uid);
	if (it == r->rec.end()) return -1;
	Record& rc = it->second;
	const std::vector<float>& sr = what == 0 ? rc.act_re : what == 1 ? rc.gs_re : rc.g_re;
	const std::vector<float>& si = what == 0 ? rc.act_im : what == 1 ? rc.gs_im : rc.g_im;
	std::copy(sr.begin(), sr.end(), re);
	std::copy(si.begin(), si.end(), im);
	return 0;
}

int ref_out_size(void* h, int uid) {
	CFunc* f = fn(static_cast<RefNet*>(h), uid);
	return f ? f->outSize() : -1;
}

// Checkpoints through the reference's own ModelSaver (impl/model_saver.h:799-821, 908-967).
int ref_save(void* h, const char* path) {
	ModelSaver saver;
	return saver.Save(static_cast<RefNet*>(h)->net, path) ? 0 : -1;
}

void* ref_restore(const char* path) {
	FILELog::ReportingLevel() = lError;
	RefNet* r = new RefNet();
	ModelSaver saver;
	if (!saver.Restore(r->net, path)) { delete r; return NULL; }
	for (auto f : r->net.functionList()) r->uids.push_back(f->uid());
	return r;
}

int ref_num_funcs(void* h) { return (int) static_cast<RefNet*>(h)->uids.size(); }
int ref_uid_at(void* h, int i) { return static_cast<RefNet*>(h)->uids[i]; }
int ref_type_of(void* h, int uid) { return ComplexNet::getType(fn(static_cast<RefNet*>(h), uid)); }
int ref_in_len(void* h, int uid) { return fn(static_cast<RefNet*>(h), uid)->input().length_; }

int ref_adam_update(void* h, float lr, int batch_size, float beta, int t) {
	static_cast<RefNet*>(h)->net.adamUpdate(lr, batch_size, beta, t);
	return 0;
}

int ref_update(void* h, float lr, int batch_size) {
	static_cast<RefNet*>(h)->net.update(lr, batch_size);
	return 0;
}

}  // extern "C"
