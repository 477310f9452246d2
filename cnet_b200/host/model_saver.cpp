// Checkpoints in the reference's byte format (ModelSaver, impl/model_saver.h:27, 530-795,
// 799-821, 908-967), so reference binaries and this library exchange models:
//   int32 magic 0xABCDE0EE, then per layer in insertion order
//   int32 type id | uid | input length | out size | #producers | producer uids...
//   CInput     : + re[len], im[len]
//   CEmbedding : + dim, max tokens, vocab, re[len], im[len]
//   Linear     : + in1_len, in2_len
// every int32 / float32 big-endian.  Weights are read back from the device before saving.
#include <climits>
#include <cstdio>
#include <cstring>
#include <fstream>

#include "cnet.h"

namespace cnet_b200 {

namespace {

const uint32_t kMagic = 0xABCDE0EEu;

void put32(std::string& out, uint32_t v) {
	char b[4] = {(char) (v >> 24), (char) (v >> 16), (char) (v >> 8), (char) v};
	out.append(b, 4);
}

void putFloats(std::string& out, const float* p, size_t n, size_t have) {
	size_t at = out.size();
	out.resize(at + 4 * n);
	for (size_t i = 0; i < n; ++i) {
		uint32_t v = 0;
		if (i < have) std::memcpy(&v, p + i, 4);
		out[at + 4 * i] = (char) (v >> 24); out[at + 4 * i + 1] = (char) (v >> 16);
		out[at + 4 * i + 2] = (char) (v >> 8); out[at + 4 * i + 3] = (char) v;
	}
}

struct Reader {
	const std::string& s;
	size_t at = 0;
	explicit Reader(const std::string& str) : s(str) {}
	bool get32(int32_t* v) {
		if (at + 4 > s.size()) return false;
		const unsigned char* b = reinterpret_cast<const unsigned char*>(s.data() + at);
		*v = (int32_t) (((uint32_t) b[0] << 24) | ((uint32_t) b[1] << 16) | ((uint32_t) b[2] << 8) | b[3]);
		at += 4;
		return true;
	}
	bool getFloats(std::vector<float>* out, size_t n) {
		if (n > (s.size() - at) / 4) return false;       // also when 4 * n would wrap
		out->resize(n);
		for (size_t i = 0; i < n; ++i) {
			int32_t v;
			get32(&v);
			std::memcpy(&(*out)[i], &v, 4);
		}
		return true;
	}
};

}  // namespace

std::string CNet::saveToString() {
	if (ctx_ && !getInputsFromGpu()) return "";
	std::string out;
	put32(out, kMagic);
	for (CFunc* f : func_list_) {
		put32(out, (uint32_t) f->type_);
		put32(out, (uint32_t) f->uid_);
		put32(out, (uint32_t) f->in_size_);
		put32(out, (uint32_t) f->out_size_);
		put32(out, (uint32_t) f->prev_func_.size());
		for (CFunc* p : f->prev_func_) put32(out, (uint32_t) p->uid_);
		if (CEmbedding* e = dynamic_cast<CEmbedding*>(f)) {
			put32(out, (uint32_t) e->embeddingDim());
			put32(out, (uint32_t) e->noOutTokens());
			put32(out, (uint32_t) e->noEmbeddings());
		}
		if (f->is_input_) {       // planes the device does not hold (a data input before its first batch) are zeros
			putFloats(out, f->host_re_.data(), (size_t) f->in_size_, f->host_re_.size());
			putFloats(out, f->host_im_.data(), (size_t) f->in_size_, f->host_im_.size());
		}
		if (Linear* l = dynamic_cast<Linear*>(f)) {
			put32(out, (uint32_t) l->firstInputLength());
			put32(out, (uint32_t) l->secondInputLength());
		}
	}
	return out;
}

bool CNet::restoreFromString(const std::string& data) {
	if (!func_list_.empty() || ctx_) { fail(CNB_ERR_ARG, "restore: the net must be empty"); return false; }
	Reader r(data);
	int32_t v = 0;
	if (!r.get32(&v) || (uint32_t) v != kMagic) { fail(CNB_ERR_ARG, "restore: bad magic number"); return false; }
	int32_t type;
	while (r.get32(&type)) {
		int32_t uid, in_len, out_len, nprev;
		if (!r.get32(&uid) || !r.get32(&in_len) || !r.get32(&out_len) || !r.get32(&nprev) || nprev < 0 || nprev > 64) {
			fail(CNB_ERR_ARG, "restore: truncated layer header"); return false;
		}
		// lengths come from the file: nothing below may size a buffer or a layer from a bad one
		if (uid <= 0 || in_len <= 0 || out_len <= 0) {
			fail(CNB_ERR_ARG, "restore: corrupt record (uid " + std::to_string(uid) + ", lengths " + std::to_string(in_len) +
					" / " + std::to_string(out_len) + ")");
			return false;
		}
		std::vector<int> prev(nprev);
		for (int i = 0; i < nprev; ++i) if (!r.get32(&prev[i])) { fail(CNB_ERR_ARG, "restore: truncated producer list"); return false; }
		CFunc* f = nullptr;
		std::vector<float> re, im;
		switch (type) {
		case isInput:
			f = new CInput(Uid(uid), OutSize(in_len));
			if (!r.getFloats(&re, in_len) || !r.getFloats(&im, in_len)) { delete f; fail(CNB_ERR_ARG, "restore: truncated planes"); return false; }
			break;
		case isEmbedding: {
			int32_t dim, toks, vocab;
			if (!r.get32(&dim) || !r.get32(&toks) || !r.get32(&vocab)) { fail(CNB_ERR_ARG, "restore: truncated embedding"); return false; }
			if (dim <= 0 || toks <= 0 || vocab <= 0 || (int64_t) dim * vocab != (int64_t) in_len || (int64_t) dim * toks > INT_MAX) {
				fail(CNB_ERR_ARG, "restore: corrupt record (embedding dims)"); return false;
			}
			f = new CEmbedding(Uid(uid), dim, toks, vocab);
			if (!r.getFloats(&re, (size_t) dim * vocab) || !r.getFloats(&im, (size_t) dim * vocab)) { delete f; fail(CNB_ERR_ARG, "restore: truncated planes"); return false; }
			break;
		}
		case isLinear: {
			int32_t in1, in2;
			if (!r.get32(&in1) || !r.get32(&in2) || in1 <= 0 || in2 <= 0 || in2 % in1) { fail(CNB_ERR_ARG, "restore: bad Linear record"); return false; }
			f = new Linear(Uid(uid), InSize(in1), InSize(in2));
			break;
		}
		case isHadamard:     f = new Hadamard(Uid(uid), InSize(out_len), InSize(out_len)); break;
		case isFourier:      f = new FourierTrans(Uid(uid), InSize(in_len)); break;
		case isResidual:     f = new Residual(Uid(uid), InSize(out_len)); break;
		case isSoftMax:      f = new SoftMax(Uid(uid), InSize(in_len)); break;
		case isCrossEntropy: f = new CrossEntropy(Uid(uid), InSize(in_len)); break;
		case isL2Out:        f = new L2Out(Uid(uid), InSize(in_len)); break;
		case isCrelu:        f = new CRelu(Uid(uid), InSize(out_len)); break;
		case isTrianFourier: f = new TriangFourier(Uid(uid), InSize(in_len)); break;
		case isGelu:         f = new CGelu(Uid(uid), InSize(out_len)); break;
		default:
			fail(CNB_ERR_UNSUPPORTED, "restore: layer type " + std::to_string(type) + " is outside this library's path");
			return false;
		}
		if (add(f, prev) < 0) { delete f; return false; }
		if (!re.empty()) { f->host_re_ = re; f->host_im_ = im; }
	}
	return true;
}

bool CNet::save(const std::string& file) {
	std::string s = saveToString();
	if (s.empty()) return false;
	std::ofstream out(file, std::ios::binary);
	if (!out) { fail(CNB_ERR_ARG, "save: cannot open " + file); return false; }
	out.write(s.data(), (std::streamsize) s.size());
	return (bool) out;
}

bool CNet::restore(const std::string& file) {
	std::ifstream in(file, std::ios::binary);
	if (!in) { fail(CNB_ERR_ARG, "restore: cannot open " + file); return false; }
	std::string s((std::istreambuf_iterator<char>(in)), std::istreambuf_iterator<char>());
	return restoreFromString(s);
}

}  // namespace cnet_b200
