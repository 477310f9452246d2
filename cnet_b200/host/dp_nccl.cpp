#include "dp_nccl.h"

#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cstdlib>

namespace cnet_b200 {

namespace {

// The subset of NCCL's C API used here (nccl.h: ncclGetUniqueId, ncclCommInitRank, ncclAllReduce,
// ncclCommDestroy, ncclCommAbort, ncclCommGetAsyncError, ncclGetErrorString).
struct UniqueId { char internal[kNcclUniqueIdBytes]; };
typedef int (*GetUniqueIdFn)(UniqueId*);
typedef int (*CommInitRankFn)(void**, int, UniqueId, int);
typedef int (*AllReduceFn)(const void*, void*, size_t, int, int, void*, cudaStream_t);
typedef int (*AllGatherFn)(const void*, void*, size_t, int, void*, cudaStream_t);
typedef int (*MemAllocFn)(void**, size_t);
typedef int (*MemFreeFn)(void*);
typedef int (*WindowRegisterFn)(void*, void*, size_t, void**, int);
typedef int (*WindowDeregisterFn)(void*, void*);
typedef int (*GetVersionFn)(int*);
// ncclConfig_t of NCCL 2.28 (nccl.h, ncclConfig_v22800); fields left at "undefined" keep NCCL's defaults
struct Config {
	size_t size; unsigned magic; unsigned version;
	int blocking, cgaClusterSize, minCTAs, maxCTAs;
	const char* netName;
	int splitShare, trafficClass;
	const char* commName;
	int collnetEnable, CTAPolicy, shrinkShare, nvlsCTAs, nChannelsPerNetPeer, nvlinkCentricSched;
};
typedef int (*CommInitRankConfigFn)(void**, int, UniqueId, int, Config*);
const int kUndefInt = -2147483647 - 1;
const int kWinCollSymmetric = 1;
typedef int (*CommFn)(void*);
typedef int (*AsyncErrFn)(void*, int*);
typedef const char* (*ErrStrFn)(int);
const int kNcclFloat32 = 7, kNcclSum = 0;

struct Api {
	GetUniqueIdFn getUniqueId = nullptr;
	CommInitRankFn commInitRank = nullptr;
	AllReduceFn allReduce = nullptr;
	AllReduceFn reduceScatter = nullptr;        // same signature as ncclAllReduce (recvcount in place of count)
	AllGatherFn allGather = nullptr;
	MemAllocFn memAlloc = nullptr;
	MemFreeFn memFree = nullptr;
	WindowRegisterFn windowRegister = nullptr;
	WindowDeregisterFn windowDeregister = nullptr;
	CommInitRankConfigFn commInitRankConfig = nullptr;
	GetVersionFn getVersion = nullptr;
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
	a.reduceScatter = (AllReduceFn) dlsym(h, "ncclReduceScatter");
	a.allGather = (AllGatherFn) dlsym(h, "ncclAllGather");
	a.memAlloc = (MemAllocFn) dlsym(h, "ncclMemAlloc");              // optional (NCCL >= 2.19)
	a.memFree = (MemFreeFn) dlsym(h, "ncclMemFree");
	a.windowRegister = (WindowRegisterFn) dlsym(h, "ncclCommWindowRegister");   // optional (NCCL >= 2.27)
	a.windowDeregister = (WindowDeregisterFn) dlsym(h, "ncclCommWindowDeregister");
	a.commInitRankConfig = (CommInitRankConfigFn) dlsym(h, "ncclCommInitRankConfig");
	a.getVersion = (GetVersionFn) dlsym(h, "ncclGetVersion");
	a.commDestroy = (CommFn) dlsym(h, "ncclCommDestroy");
	a.commAbort = (CommFn) dlsym(h, "ncclCommAbort");
	a.asyncError = (AsyncErrFn) dlsym(h, "ncclCommGetAsyncError");
	a.errStr = (ErrStrFn) dlsym(h, "ncclGetErrorString");
	a.ok = a.getUniqueId && a.commInitRank && a.allReduce && a.reduceScatter && a.allGather && a.commDestroy && a.commAbort && a.asyncError && a.errStr;
	if (!a.ok) a.why = "libnccl lacks an expected symbol";
	return a;
}

}  // namespace

NcclGroup::~NcclGroup() { shutdown(); }

void NcclGroup::shutdown() {
	if (comm_ && window_ && api().windowDeregister) api().windowDeregister(comm_, window_);
	window_ = nullptr;
	if (comm_) api().commDestroy(comm_);
	comm_ = nullptr;
	if (ev_fork_) cudaEventDestroy((cudaEvent_t) ev_fork_);
	if (ev_join_) cudaEventDestroy((cudaEvent_t) ev_join_);
	if (comm_stream_) cudaStreamDestroy((cudaStream_t) comm_stream_);
	ev_fork_ = ev_join_ = comm_stream_ = nullptr;
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
	// CNB_NCCL_MAX_CTAS / CNB_NCCL_CTA_POLICY: upper bound of CTAs per collective and NCCL's CTA policy
	// (1 = efficiency, 2 = zero-CTA where a copy engine can do the collective), for libraries of the 2.28 layout
	const char* e_cta = getenv("CNB_NCCL_MAX_CTAS");
	const char* e_pol = getenv("CNB_NCCL_CTA_POLICY");
	int version = 0;
	if (a.getVersion) a.getVersion(&version);
	int rc;
	if ((e_cta || e_pol) && a.commInitRankConfig && version >= 22800) {
		Config c;
		c.size = sizeof(Config); c.magic = 0xcafebeef; c.version = (unsigned) version;
		c.blocking = c.cgaClusterSize = c.minCTAs = c.maxCTAs = kUndefInt;
		c.netName = nullptr; c.splitShare = c.trafficClass = kUndefInt; c.commName = nullptr;
		c.collnetEnable = c.CTAPolicy = c.shrinkShare = c.nvlsCTAs = c.nChannelsPerNetPeer = c.nvlinkCentricSched = kUndefInt;
		if (e_cta) c.maxCTAs = atoi(e_cta);
		if (e_pol) c.CTAPolicy = atoi(e_pol);
		rc = a.commInitRankConfig(&comm_, nranks, id, rank, &c);
	} else {
		rc = a.commInitRank(&comm_, nranks, id, rank);
	}
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

void* NcclGroup::memAlloc(size_t bytes, std::string* err) {
	Api& a = api();
	if (!a.ok || !a.memAlloc || !a.memFree) { if (err) *err = a.ok ? "libnccl has no ncclMemAlloc" : a.why; return nullptr; }
	void* p = nullptr;
	int rc = a.memAlloc(&p, bytes);
	if (rc != 0) { if (err) *err = std::string("ncclMemAlloc: ") + a.errStr(rc); return nullptr; }
	return p;
}

void NcclGroup::memFree(void* p) {
	if (p && api().memFree) api().memFree(p);
}

bool NcclGroup::registerWindow(void* buf, size_t bytes) {
	if (!active()) return true;
	Api& a = api();
	if (!a.windowRegister || !a.windowDeregister) { error_ = "libnccl has no ncclCommWindowRegister"; return false; }
	int rc = a.windowRegister(comm_, buf, bytes, &window_, kWinCollSymmetric);
	if (rc != 0) { error_ = std::string("ncclCommWindowRegister: ") + a.errStr(rc); window_ = nullptr; return false; }
	return true;
}

bool NcclGroup::reduceScatter(float* dev, size_t per_rank, void* compute) {
	if (!active()) return true;
	cudaStream_t cs = (cudaStream_t) comm_stream_;
	if (cudaEventRecord((cudaEvent_t) ev_fork_, (cudaStream_t) compute) != cudaSuccess ||
			cudaStreamWaitEvent(cs, (cudaEvent_t) ev_fork_, 0) != cudaSuccess) {
		error_ = "fork to the communication stream failed"; return false;
	}
	int rc = api().reduceScatter(dev, dev + (size_t) rank_ * per_rank, per_rank, kNcclFloat32, kNcclSum, comm_, cs);
	if (rc != 0) { error_ = std::string("ncclReduceScatter: ") + api().errStr(rc); return false; }
	pending_ = true;
	return true;
}

bool NcclGroup::allGather(float* dev, size_t per_rank, void* compute) {
	if (!active()) return true;
	cudaStream_t cs = (cudaStream_t) comm_stream_;
	if (cudaEventRecord((cudaEvent_t) ev_fork_, (cudaStream_t) compute) != cudaSuccess ||
			cudaStreamWaitEvent(cs, (cudaEvent_t) ev_fork_, 0) != cudaSuccess) {
		error_ = "fork to the communication stream failed"; return false;
	}
	int rc = api().allGather(dev + (size_t) rank_ * per_rank, dev, per_rank, kNcclFloat32, comm_, cs);
	if (rc != 0) { error_ = std::string("ncclAllGather: ") + api().errStr(rc); return false; }
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
