// NCCL data parallelism of the host facade: a communicator per net, bucket all-reduces issued
// from C++ on a communication stream that forks from / joins the compute stream with events,
// so the whole step (kernels and collectives) can be captured in one CUDA graph.
// NCCL is bound at run time (dlopen of libnccl.so.2, the library PyTorch ships), so the build
// needs no NCCL headers; the few declarations below follow NCCL's public C API.
#ifndef CNET_B200_HOST_DP_NCCL_H_
#define CNET_B200_HOST_DP_NCCL_H_

#include <cstddef>
#include <string>

namespace cnet_b200 {

const int kNcclUniqueIdBytes = 128;

class NcclGroup {
	void* comm_ = nullptr;          // ncclComm_t
	void* comm_stream_ = nullptr;   // cudaStream_t
	void* ev_fork_ = nullptr;       // cudaEvent_t: compute -> comm
	void* ev_join_ = nullptr;       // cudaEvent_t: comm -> compute
	int rank_ = 0, nranks_ = 1;
	bool pending_ = false;
	void* window_ = nullptr;        // ncclWindow_t of the registered weight / gradient region
	std::string error_;
public:
	~NcclGroup();
	void shutdown();                // deregisters the window and destroys the communicator (idempotent)
	// Device memory from NCCL's own allocator (ncclMemAlloc): the kind of allocation that can be registered
	// with a communicator as a symmetric window.  NULL (and *err set) when the library lacks it.
	static void* memAlloc(size_t bytes, std::string* err);
	static void memFree(void* p);
	// Collective over the ranks: registers [buf, buf + bytes) (same offsets on every rank, memAlloc'ed memory,
	// 4096-byte aligned) as a symmetric window, so that collectives on it run NCCL's symmetric-memory kernels
	// (direct peer / in-switch access, fewer CTAs).  False when the library lacks window registration.
	bool registerWindow(void* buf, size_t bytes);
	bool hasWindow() const { return window_ != nullptr; }
	static bool uniqueId(char out[kNcclUniqueIdBytes], std::string* err);
	bool init(const char id[kNcclUniqueIdBytes], int rank, int nranks);
	bool active() const { return comm_ != nullptr && nranks_ > 1; }
	int nranks() const { return nranks_; }
	// sum `count` floats in place over the ranks, after everything enqueued so far on `compute`
	bool allReduce(float* dev, size_t count, void* compute);
	// sum over the ranks, rank r keeping floats [r * count_per_rank, (r + 1) * count_per_rank) of `dev` (in place)
	bool reduceScatter(float* dev, size_t count_per_rank, void* compute);
	// every rank's slice [r * count_per_rank, ...) of `dev` to all ranks (in place)
	bool allGather(float* dev, size_t count_per_rank, void* compute);
	int rank() const { return rank_; }
	// make `compute` wait for every all-reduce issued since the last join
	bool join(void* compute);
	// 0 = healthy; otherwise the communicator reported an asynchronous error
	int asyncError();
	void abort();
	const std::string& error() const { return error_; }
};

}  // namespace cnet_b200
#endif
