#include "dp_nccl.h"

#include <cuda_runtime.h>
#include <dlfcn.h>

namespace cnet_b200 {

namespace {

// The subset of NCCL's C API used here (nccl.h: ncclGetUniqueId, ncclCommInitRank, ncclAllReduce,
// ncclCommDestroy, ncclCommAbort, ncclCommGetAsyncError, ncclGetErrorString).
struct UniqueId { char internal[kNcclUniqueIdBytes]; };
typedef int (*GetUniqueIdFn)(UniqueId*);
typedef int (*CommInitRankFn)(void**, int, UniqueId, int);
typedef int (*AllReduceFn)(const void*, void*, size_t, int, int, void*, cudaStream_t);
typedef int (*CommFn)(void*);
typedef int (*AsyncErrFn)(void*, int*);
typedef const char* (*ErrStrFn)(int);
const int kNcclFloat32 = 7, kNcclSum = 0;

struct Api {
	GetUniqueIdFn getUniqueId = nullptr;
	CommInitRankFn commInitRank = nullptr;
	AllReduceFn allReduce = nullptr;
	CommFn commDestroy = nullptr, commAbort = nullptr;
	AsyncErrFn asyncError = nullptr;
	ErrStrFn errStr = nullptr;
	bool ok = false;
	std::string why;
};

Api& api() {
	static Api a;
	static bool tried = false;
	if (tried) return a;
	tried = true;
	void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
	if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
	if (!h) { a.why = std::string("cannot load libnccl: ") + dlerror(); return a; }
	a.getUniqueId = (GetUniqueIdFn) dlsym(h, "ncclGetUniqueId");
	a.commInitRank = (CommInitRankFn) dlsym(h, "ncclCommInitRank");
	a.allReduce = (AllReduceFn) dlsym(h, "ncclAllReduce");
	a.commDestroy = (CommFn) dlsym(h, "ncclCommDestroy");
	a.commAbort = (CommFn) dlsym(h, "ncclCommAbort");
	a.asyncError = (AsyncErrFn) dlsym(h, "ncclCommGetAsyncError");
	a.errStr = (ErrStrFn) dlsym(h, "ncclGetErrorString");
	a.ok = a.getUniqueId && a.commInitRank && a.allReduce && a.commDestroy && a.commAbort && a.asyncError && a.errStr;
	if (!a.ok) a.why = "libnccl lacks an expected symbol";
	return a;
}

}  // namespace

NcclGroup::~NcclGroup() {
	if (comm_) api().commDestroy(comm_);
	if (ev_fork_) cudaEventDestroy((cudaEvent_t) ev_fork_);
	if (ev_join_) cudaEventDestroy((cudaEvent_t) ev_join_);
	if (comm_stream_) cudaStreamDestroy((cudaStream_t) comm_stream_);
}

bool NcclGroup::uniqueId(char out[kNcclUniqueIdBytes], std::string* err) {
	Api& a = api();
	if (!a.ok) { if (err) *err = a.why; return false; }
	UniqueId id;
	int rc = a.getUniqueId(&id);
	if (rc != 0) { if (err) *err = a.errStr(rc); return false; }
	for (int i = 0; i < kNcclUniqueIdBytes; ++i) out[i] = id.internal[i];
	return true;
}

bool NcclGroup::init(const char idb[kNcclUniqueIdBytes], int rank, int nranks) {
	Api& a = api();
	if (!a.ok) { error_ = a.why; return false; }
	if (nranks < 1 || rank < 0 || rank >= nranks) { error_ = "bad rank / world size"; return false; }
	rank_ = rank;
	nranks_ = nranks;
	if (nranks == 1) return true;
	UniqueId id;
	for (int i = 0; i < kNcclUniqueIdBytes; ++i) id.internal[i] = idb[i];
	int rc = a.commInitRank(&comm_, nranks, id, rank);
	if (rc != 0) { error_ = std::string("ncclCommInitRank: ") + a.errStr(rc); comm_ = nullptr; return false; }
	cudaStream_t s;
	cudaEvent_t e0, e1;
	if (cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking) != cudaSuccess ||
			cudaEventCreateWithFlags(&e0, cudaEventDisableTiming) != cudaSuccess ||
			cudaEventCreateWithFlags(&e1, cudaEventDisableTiming) != cudaSuccess) {
		error_ = "cannot create the communication stream / events";
		return false;
	}
	comm_stream_ = s; ev_fork_ = e0; ev_join_ = e1;
	return true;
}

bool NcclGroup::allReduce(float* dev, size_t count, void* compute) {
	if (!active()) return true;
	cudaStream_t cs = (cudaStream_t) comm_stream_;
	if (cudaEventRecord((cudaEvent_t) ev_fork_, (cudaStream_t) compute) != cudaSuccess ||
			cudaStreamWaitEvent(cs, (cudaEvent_t) ev_fork_, 0) != cudaSuccess) {
		error_ = "fork to the communication stream failed"; return false;
	}
	int rc = api().allReduce(dev, dev, count, kNcclFloat32, kNcclSum, comm_, cs);
	if (rc != 0) { error_ = std::string("ncclAllReduce: ") + api().errStr(rc); return false; }
	pending_ = true;
	return true;
}

bool NcclGroup::join(void* compute) {
	if (!active() || !pending_) return true;
	if (cudaEventRecord((cudaEvent_t) ev_join_, (cudaStream_t) comm_stream_) != cudaSuccess ||
			cudaStreamWaitEvent((cudaStream_t) compute, (cudaEvent_t) ev_join_, 0) != cudaSuccess) {
		error_ = "join from the communication stream failed"; return false;
	}
	pending_ = false;
	return true;
}

int NcclGroup::asyncError() {
	if (!comm_) return 0;
	int e = 0;
	int rc = api().asyncError(comm_, &e);
	return rc != 0 ? rc : e;
}

void NcclGroup::abort() {
	if (comm_) { api().commAbort(comm_); comm_ = nullptr; }
}

}  // namespace cnet_b200
