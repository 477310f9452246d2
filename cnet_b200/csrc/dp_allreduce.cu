// All-reduce (sum) of a range of the weight-gradient arena over the GPUs of one NVSwitch domain, done by this
// library's own kernel on symmetric memory instead of by NCCL: the arena of every rank is mapped into every other
// rank's address space (peer pointers) and, where the platform has it, bound to one NVLink multicast address.
//
// Rank r owns the r-th slice of the range.  It reads the slice of ALL ranks and sums it
//   * in the switch, with one `multimem.ld_reduce.add.v4.f32` per 16 bytes of the multicast address, or
//   * with plain 16-byte loads from each peer's memory (no multicast support),
// and writes the sum back to all ranks (`multimem.st`, or plain 16-byte stores to each peer).  Per GPU that is the
// range once out and once in over NVLink, like a ring, but with no staging copies and no shared memory.
//
// A few CTAs of 1024 threads on SMs that the step's persistent kernels leave free.  (CTAs thin enough to share an
// SM with the GEMM's were measured first, one per SM: they fit beside the GEMM, but the FFT and the column
// reduction fill an SM's register file, so those kernels waited for the whole reduction: 2.43 ms per step at 2
// GPUs against 2.35.)
//
// Ranks meet twice per call, through flag words in symmetric memory (rank a writes slot a of rank b's flag block):
//   enter: nobody reads a peer's slice before that peer's gradients of the range are final (its kernel has started);
//   exit : nobody's kernel completes before every peer has finished writing into its memory.
// The flags carry a call counter kept in device memory, so a captured CUDA graph can replay the launch.  Every wait
// is bounded (WAIT_LIMIT_NS by %globaltimer); on expiry the error word of the context is set and the kernel runs on
// to its end, so that a missing peer costs a wrong result and an error status, never a hung GPU.
#include "common.cuh"

namespace {

constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;
constexpr int THREADS = 1024;

struct DpParams {
    float* local;                          // this rank's copy of the range (count floats)
    float* mc;                             // the same range at the multicast address, or NULL
    float* peer[CNB_DP_MAX_RANKS];         // the range in every rank's memory as mapped here ([rank] == local)
    unsigned* flags[CNB_DP_MAX_RANKS];     // every rank's flag block as mapped here: CNB_DP_MAX_RANKS words each
    unsigned* state;                       // local: [0] calls completed, [1] "peers have arrived" of the current call, [2] CTAs done
    int* status;
    size_t count;                          // floats in the range (multiple of 4 * world)
    int rank, world;
};

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ unsigned ld_acquire_gpu(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// true when *p reached `want` (counters only grow) within the limit
template <typename Load>
__device__ __forceinline__ bool wait_reach(const unsigned* p, unsigned want, Load load) {
    if ((int) (load(p) - want) >= 0) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
        for (int i = 0; i < 32; ++i)
            if ((int) (load(p) - want) >= 0) return true;
        if (global_ns() - t0 > WAIT_LIMIT_NS) return false;
        __nanosleep(64);
    }
}

// one thread: tell every peer that this rank reached `epoch`, then wait until every peer has told us the same
__device__ void meet_peers(const DpParams& p, unsigned epoch, int code) {
    __threadfence_system();
    for (int r = 0; r < p.world; ++r)
        if (r != p.rank) st_release_sys(p.flags[r] + p.rank, epoch);
    for (int r = 0; r < p.world; ++r) {
        if (r == p.rank) continue;
        if (!wait_reach(p.flags[p.rank] + r, epoch, ld_acquire_sys)) {
            atomicCAS(p.status, 0, code);
            atomicExch(p.status + 1, r);
            break;                          // report once and run on
        }
    }
}

// 16 bytes of a peer's memory, not through this SM's L1 (the peer rewrites it every step)
__device__ __forceinline__ float4 ld_peer(const float* a) {
    float4 v;
    asm volatile("ld.volatile.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(a) : "memory");
    return v;
}

__device__ __forceinline__ float4 mc_ld_reduce(const float* a) {
    float4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(a) : "memory");
    return v;
}

__device__ __forceinline__ void mc_st(float* a, float4 v) {
    asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(a), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w) : "memory");
}

__global__ void __launch_bounds__(THREADS)
dp_allreduce_k(const DpParams p) {
    // No cnb_pdl_enter(): this kernel is launched the ordinary way on the communication stream.
    __shared__ unsigned s_call;
    if (threadIdx.x == 0) s_call = ld_acquire_gpu(p.state);          // stable until the last CTA of this launch ends
    __syncthreads();
    const unsigned enter = 2u * s_call + 1u, leave = 2u * s_call + 2u;
    if (threadIdx.x == 0) {
        if (blockIdx.x == 0) {
            meet_peers(p, enter, 31);
            atomicExch(p.state + 1, enter);                          // the other CTAs of this rank may go
        } else if (!wait_reach(p.state + 1, enter, ld_acquire_gpu)) {
            atomicCAS(p.status, 0, 32);
        }
    }
    __syncthreads();

    const size_t slice = p.count / p.world;                          // floats per rank, multiple of 4
    const size_t lo = (size_t) p.rank * slice;
    const size_t step = (size_t) gridDim.x * THREADS * 4;
    if (p.mc) {
        // in-switch sum of the slice over all ranks, then the switch copies the result to all ranks
        size_t i = lo + ((size_t) blockIdx.x * THREADS + threadIdx.x) * 4;
        for (; i + 3 * step < lo + slice; i += 4 * step) {           // four 16-byte reductions in flight per thread
            const float4 a = mc_ld_reduce(p.mc + i), b = mc_ld_reduce(p.mc + i + step);
            const float4 c = mc_ld_reduce(p.mc + i + 2 * step), d = mc_ld_reduce(p.mc + i + 3 * step);
            mc_st(p.mc + i, a); mc_st(p.mc + i + step, b); mc_st(p.mc + i + 2 * step, c); mc_st(p.mc + i + 3 * step, d);
        }
        for (; i < lo + slice; i += step) mc_st(p.mc + i, mc_ld_reduce(p.mc + i));
    } else {
        for (size_t i = lo + ((size_t) blockIdx.x * THREADS + threadIdx.x) * 4; i < lo + slice; i += step) {
            float4 v[CNB_DP_MAX_RANKS];
#pragma unroll
            for (int r = 0; r < CNB_DP_MAX_RANKS; ++r)               // every peer's loads are issued before the first sum
                if (r < p.world) v[r] = ld_peer(p.peer[r] + i);
            float4 s = v[0];                                         // fixed order: the same bits on every rank
#pragma unroll
            for (int r = 1; r < CNB_DP_MAX_RANKS; ++r)
                if (r < p.world) { s.x += v[r].x; s.y += v[r].y; s.z += v[r].z; s.w += v[r].w; }
#pragma unroll
            for (int r = 0; r < CNB_DP_MAX_RANKS; ++r)
                if (r < p.world) *reinterpret_cast<float4*>(p.peer[r] + i) = s;
        }
    }

    // the last CTA of this rank to finish meets the peers again and closes the call
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned done = atomicAdd(p.state + 2, 1u);
        if (done == gridDim.x - 1) {
            meet_peers(p, leave, 33);
            atomicExch(p.state + 2, 0u);
            __threadfence();
            atomicExch(p.state, s_call + 1u);
        }
    }
}

}  // namespace

extern "C" {

size_t cnb_dp_state_bytes(void) { return 256; }

int cnb_dp_allreduce(cnb_ctx* ctx, const cnb_dp_peers* peers, float* local, size_t count, void* stream) {
    CNB_CHECK_ARG(ctx && peers && local, "cnb_dp_allreduce: null pointer");
    CNB_CHECK_ARG(peers->world >= 1 && peers->world <= CNB_DP_MAX_RANKS && peers->rank >= 0 && peers->rank < peers->world,
                  "cnb_dp_allreduce: rank %d of %d (at most %d ranks)", peers->rank, peers->world, CNB_DP_MAX_RANKS);
    if (peers->world == 1 || count == 0) return CNB_OK;
    CNB_CHECK_ARG(count % (4 * (size_t) peers->world) == 0 && (reinterpret_cast<uintptr_t>(local) & 15) == 0,
                  "cnb_dp_allreduce: the range must be 16-byte aligned and a multiple of 4 x %d floats", peers->world);
    CNB_CHECK_ARG(peers->state && peers->arena_base[peers->rank], "cnb_dp_allreduce: symmetric memory is not set up");
    const char* base = static_cast<const char*>(peers->arena_base[peers->rank]);
    const ptrdiff_t off = reinterpret_cast<const char*>(local) - base;
    CNB_CHECK_ARG(off >= 0 && (size_t) off + count * sizeof(float) <= peers->arena_bytes,
                  "cnb_dp_allreduce: the range lies outside the symmetric arena");
    DpParams p;
    p.local = local;
    p.mc = peers->multicast_base ? reinterpret_cast<float*>(static_cast<char*>(peers->multicast_base) + off) : nullptr;
    for (int r = 0; r < CNB_DP_MAX_RANKS; ++r) {
        p.peer[r] = r < peers->world ? reinterpret_cast<float*>(static_cast<char*>(peers->arena_base[r]) + off) : nullptr;
        p.flags[r] = r < peers->world ? static_cast<unsigned*>(peers->flags[r]) : nullptr;
        if (r < peers->world) CNB_CHECK_ARG(peers->arena_base[r] && peers->flags[r], "cnb_dp_allreduce: rank %d is not mapped", r);
    }
    p.state = static_cast<unsigned*>(peers->state);
    p.status = ctx->d_status;
    p.count = count;
    p.rank = peers->rank;
    p.world = peers->world;
    // ctas = 0: as many as there are SMs set aside for the collective (cnb_set_gemm_sm_limit), at least 4
    const size_t slice16 = count / peers->world / 4;
    int ctas = peers->ctas > 0 ? peers->ctas : std::max(4, ctx->sm_count - cnb::usable_sms(ctx));
    ctas = (int) std::min<size_t>((size_t) std::min(ctas, ctx->sm_count), std::max<size_t>(1, slice16 / THREADS));
    dp_allreduce_k<<<ctas, THREADS, 0, cnb::S(stream)>>>(p);
    CNB_LAUNCH_CHECK("dp_allreduce");
    return CNB_OK;
}

}  // extern "C"
