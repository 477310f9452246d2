// Flat C binding of the host facade (declared in include/cnet_b200_host.h).
#include "../../include/cnet_b200_host.h"
#include "cnet.h"
#include "data_reader.h"

using namespace cnet_b200;

struct cnh_net {
	CNet net;
	std::string err;
};

namespace {
int status(cnh_net* n) {
	if (n->net.ok()) return 0;
	n->err = n->net.error();
	return CNB_ERR_ARG;
}
}  // namespace

extern "C" {

cnh_net* cnh_create(int device, size_t arena_bytes, void* ext_arena) {
	cnh_net* n = new cnh_net();
	n->net.setDevice(device, arena_bytes, ext_arena);
	return n;
}

void cnh_destroy(cnh_net* n) { delete n; }

int cnh_set_device(cnh_net* n, int device, size_t arena_bytes, void* ext_arena) {
	n->net.setDevice(device, arena_bytes, ext_arena);
	return 0;
}

const char* cnh_error(cnh_net* n) { return n ? n->net.error().c_str() : "null net"; }

void cnh_clear_error(cnh_net* n) { n->net.clearError(); }

int cnh_add(cnh_net* n, int type, int a, int b, int c, const int* prev, int nprev) {
	CFunc* f = nullptr;
	switch (type) {
	case isInput:        f = new CInput(OutSize(a)); break;
	case isEmbedding:    f = new CEmbedding(a, b, c); break;
	case isFourier:      f = new FourierTrans(InSize(a)); break;
	case isHadamard:     f = new Hadamard(InSize(a), InSize(a)); break;
	case isGelu:         f = new CGelu(InSize(a)); break;
	case isLinear:
		if (a <= 0 || b % a != 0) return CNB_ERR_ARG;
		f = new Linear(InSize(a), InSize(b));
		break;
	case isResidual:     f = new Residual(InSize(a)); break;
	case isSoftMax:      f = new SoftMax(InSize(a)); break;
	case isCrossEntropy: f = new CrossEntropy(InSize(a)); break;
	case isL2Out:        f = new L2Out(InSize(a)); break;
	case isCrelu:        f = new CRelu(InSize(a)); break;
	case isTrianFourier: f = new TriangFourier(InSize(a)); break;
	default: return CNB_ERR_UNSUPPORTED;
	}
	int uid = n->net.add(f, std::vector<int>(prev, prev + nprev));
	if (uid < 0) { delete f; return CNB_ERR_ARG; }
	return uid;
}

int cnh_out_size(cnh_net* n, int uid) { CFunc* f = n->net[uid]; return f ? f->outSize() : CNB_ERR_ARG; }
int cnh_init_inputs(cnh_net* n, uint64_t seed) { n->net.init_inputs(seed); return status(n); }
int cnh_set_values(cnh_net* n, int uid, const float* re, const float* im, int len) {
	n->net.setInputValues(uid, re, im, len); return status(n);
}
int cnh_get_values(cnh_net* n, int uid, float* re, float* im, int len) {
	n->net.getInputValues(uid, re, im, len); return status(n);
}
int cnh_get_wgrad(cnh_net* n, int uid, float* re, float* im, int len) {
	n->net.getInputGradients(uid, re, im, len); return status(n);
}
int cnh_set_stream(cnh_net* n, void* s) { n->net.setStream(s); return 0; }
int cnh_set_fusion(cnh_net* n, int on) { n->net.setFusion(on != 0); return 0; }
int cnh_set_bucket_hook(cnh_net* n, cnh_bucket_hook h, void* user) { n->net.setBucketHook(h, user); return 0; }
size_t cnh_required_arena(cnh_net* n, int batch) { return n->net.requiredArenaBytes(batch); }
int cnh_allocate(cnh_net* n, int batch) { n->net.allocateOnGpu(batch); return status(n); }
int cnh_upload(cnh_net* n, const float* re, const float* im, const int32_t* tokens, const int32_t* labels, int batch) {
	n->net.batchToGpu(re, im, tokens, labels, batch); return status(n);
}
int cnh_prefetch(cnh_net* n, const float* re, const float* im, const int32_t* tokens, const int32_t* labels, int batch) {
	n->net.prefetchBatch(re, im, tokens, labels, batch); return status(n);
}
int cnh_commit(cnh_net* n) { n->net.commitBatch(); return status(n); }
int cnh_read_losses_async(cnh_net* n, float* host_out, int cnt) { n->net.readLossesAsync(host_out, cnt); return status(n); }
int cnh_wait_losses(cnh_net* n) { n->net.waitLosses(); return status(n); }
int cnh_forward(cnh_net* n) { n->net.forward(); return status(n); }
int cnh_backward(cnh_net* n) { n->net.backward(); return status(n); }
int cnh_backward_label(cnh_net* n, int label) { n->net.backward(label); return status(n); }
int cnh_update(cnh_net* n, float lr) { n->net.updateInputs(lr); return status(n); }
int cnh_adam_update(cnh_net* n, float lr, float beta, int t) { n->net.adamUpdate(lr, beta, t); return status(n); }
int cnh_infer(cnh_net* n) { n->net.infer(); return status(n); }
int cnh_get_losses(cnh_net* n, float* out, int cnt) { n->net.getLosses(out, cnt); return status(n); }
int cnh_sync(cnh_net* n) { n->net.sync(); return status(n); }
int cnh_read_output(cnh_net* n, int uid, int what, float* re, float* im) {
	n->net.readOutput(uid, what, re, im); return status(n);
}
int cnh_grad_arena(cnh_net* n, void** p, size_t* count, int* nb) {
	*p = n->net.gradArena(count);
	if (nb) *nb = n->net.noBuckets();
	return 0;
}
int cnh_weight_arena(cnh_net* n, void** p, size_t* count) { *p = n->net.weightArena(count); return 0; }
void* cnh_context(cnh_net* n) { return n->net.context(); }
int cnh_save(cnh_net* n, const char* path) { n->net.save(path); return status(n); }
int cnh_restore(cnh_net* n, const char* path) { n->net.restore(path); return status(n); }
int cnh_num_funcs(cnh_net* n) { return n->net.noFunctions(); }
int cnh_uid_at(cnh_net* n, int i) { return (i >= 0 && i < n->net.noFunctions()) ? n->net.uidAt(i) : CNB_ERR_ARG; }
int cnh_type_of(cnh_net* n, int uid) { CFunc* f = n->net[uid]; return f ? f->getType() : CNB_ERR_ARG; }
int cnh_in_size(cnh_net* n, int uid) { CFunc* f = n->net[uid]; return f ? f->inSize() : CNB_ERR_ARG; }

int cnh_dp_unique_id(char* out128) {
	std::string err;
	return CNet::ncclUniqueId(out128, &err) ? 0 : CNB_ERR_CUDA;
}
int cnh_dp_init(cnh_net* n, const char* id128, int rank, int nranks) {
	n->net.setDataParallel(id128, rank, nranks); return status(n);
}
int cnh_dp_async_error(cnh_net* n) { return n->net.dataParallelError(); }
int cnh_dp_allreduce_grads(cnh_net* n) { n->net.allReduceGradients(); return status(n); }
int cnh_dp_set_symmetric(cnh_net* n, int rank, int world, void* multicast_base, void* const* arena_bases,
                         void* const* flag_blocks, int ctas) {
	n->net.setSymmetricPeers(rank, world, multicast_base, arena_bases, flag_blocks, ctas); return status(n);
}
int cnh_dp_use_nccl_arena(cnh_net* n, int on) { n->net.setNcclArena(on != 0); return 0; }
int cnh_dp_symmetric(cnh_net* n) { return n->net.symmetricWindow() ? 1 : 0; }
int cnh_capture_begin(cnh_net* n) { n->net.beginCapture(); return status(n); }
int cnh_capture_end(cnh_net* n) { n->net.endCapture(); return status(n); }
int cnh_graph_launch(cnh_net* n) { n->net.launchGraph(); return status(n); }
unsigned long long cnh_graph_kernel_count(cnh_net* n) { return n->net.graphKernelCount(); }

// MnistDataReader (data/data.h:82-165) behind a handle
void* cnh_mnist_open(const char* image_file, const char* label_file, int count) {
	MnistDataReader* r = new MnistDataReader();
	if (!r->Open(image_file, label_file, count) || !r->readData()) { delete r; return nullptr; }
	return r;
}
void cnh_mnist_close(void* h) { delete static_cast<MnistDataReader*>(h); }
int cnh_mnist_size(void* h) { return h ? static_cast<MnistDataReader*>(h)->size() : CNB_ERR_ARG; }
int cnh_mnist_shuffle(void* h, unsigned seed) { if (!h) return CNB_ERR_ARG; static_cast<MnistDataReader*>(h)->shuffle(seed); return 0; }
int cnh_mnist_has_next(void* h, int batch) { return h && static_cast<MnistDataReader*>(h)->hasNextBatch(batch) ? 1 : 0; }
int cnh_mnist_next_batch(void* h, int batch, float* re, float* im, int* labels) {
	return h && static_cast<MnistDataReader*>(h)->nextBatchInto(batch, re, im, labels) ? 0 : CNB_ERR_ARG;
}

}  // extern "C"
