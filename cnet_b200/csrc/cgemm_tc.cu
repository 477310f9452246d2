// tcgen05 complex GEMM with an error-compensated operand split, for sm_100a.
//
//   D[m,n] (+)= sum_k A[m,k] * (conjB ? conj(B[n,k]) : B[n,k]) (+ R[m,n])
//   A [M,K], B [N,K] complex, K-major (row-major) or MN-major ([K, rows]) split planes.
//
// Numerics.  Every fp32 operand x is split once, before the GEMM, into hi = x with the 13 low
// mantissa bits cleared (exactly a TF32 value) and lo = x - hi (exact in fp32).  Each real
// product is three tensor-core MMAs with fp32 accumulation in tensor memory:
//     hi*hi                on the TF32 pipe (exact products), and
//     hi*lo + lo*hi        on the BF16 pipe, from hi and lo rounded to bf16 (h16, l16).
// The cross terms are 2^-10 of the product, so their bf16 rounding (2^-9 each factor) costs 2^-18 of the
// product per cross term at worst (2^-19.5 rms for both), next to the 2^-20 of the dropped lo*lo term; fp32's
// exponent range is kept (no scaling).
// A BF16 MMA of depth 16 takes the time of a TF32 MMA of depth 8, so a real product costs two TF32-equivalents
// instead of the three of the all-TF32 form, for the same operand bytes (8 per real element).
//
// Tiling.  One CTA computes a 128 x 128 complex tile.  The B tile is staged as ONE 256-row
// operand [B_re rows ; B_im rows], so every MMA is 128 x 256 and the complex structure
// costs two accumulators instead of four MMA shapes:
//     acc1 = A_re * [B_re ; B_im]^T      (TMEM columns   0..255)
//     acc2 = A_im * [B_re ; B_im]^T      (TMEM columns 256..511)
//     D_re = acc1[:, :128] -/+ acc2[:, 128:],   D_im = acc1[:, 128:] +/- acc2[:, :128]   (epilogue)
// Per 16-deep k-block a stage holds 8 operand slots of 8 KB = 64 KB; 3 stages:
//     A hi_re, A hi_im (fp32, 64-byte swizzle),  A h16 [re ; im], A l16 [re ; im] (bf16, 32-byte swizzle),
//     B hi_re, B hi_im,                          B h16 [re ; im], B l16 [re ; im];
// per k-block and accumulator: 2 TF32 MMAs (k-steps of 8) + 2 BF16 MMAs (one k-step of 16).
// Each CTA issues its own plain TMA tile loads; their zero fill handles every M/N/K edge.
//
// CTA pairs.  The large launches (cgemm_tc_k<true>) give a 256 x 128 tile to a cluster of two CTAs that work as
// one tensor core (cta_group::2): each CTA stages its own 128 rows of A and one half of the stacked B operand
// (B_re rows in the first CTA, B_im rows in the second), i.e. 48 KB per k-block instead of 64 KB, four stages
// instead of three.  The first CTA issues every MMA (M = 256); both CTAs load, drain their own accumulator rows
// and write them out.  Completion bytes of both CTAs' loads go to the first CTA's full barrier; its
// tcgen05.commit arrives on the stage's empty barrier (and on the "accumulators ready" barrier) of both.
//
// Scheduling.  Stream-K: the (tile, k-block) work units are cut into equal consecutive runs, one
// per CTA and one CTA per SM, so every SM finishes together whatever the tile count; a tile whose
// k-range is shared by several CTAs is summed with fp32 atomics into a pre-zeroed output.
//
// Roles.  warp 0: TMA producer; warp 1: TMEM allocation + MMA issue (one elected thread);
// warps 2..5: epilogue (tcgen05.ld, combine, stage through shared memory, coalesced 16-byte
// stores / atomics with residual or accumulate); tensor memory is handed back to the MMA warp as
// soon as it has been read, so the write-out overlaps the next run of MMAs.
// Every mbarrier wait is bounded (2 s); on expiry the kernel records an error word, skips to
// the common exit, frees its tensor memory and returns.
#include <cuda.h>

#include <algorithm>
#include <cstdlib>

#include "common.cuh"

namespace {

constexpr int BM = 128, BN = 128, BK = 16;
constexpr int PLANE_BYTES = BM * BK * 4;             // 8 KB: one operand slot of one stage
// One CTA per tile: 8 slots (A: 4, B: 4) = 64 KB per stage, 3 stages.  A pair of CTAs per 256-row tile
// (cta_group::2): each CTA stages its own 128 rows of A (4 slots) and one of the two halves of the stacked B
// operand (B_re rows in the first CTA, B_im rows in the second: 2 slots) = 48 KB per stage, 4 stages.
template <bool PAIR> struct Cfg {
    static constexpr int STAGES = PAIR ? 4 : 3;
    static constexpr int STAGE_BYTES = (PAIR ? 6 : 8) * PLANE_BYTES;
    static constexpr int TILE_M = PAIR ? 2 * BM : BM;
};
constexpr int OPERAND_BYTES = 3 * 8 * PLANE_BYTES;   // 192 KB of operand stages in both forms
constexpr int EPI_BYTES = 2 * 128 * 32 * 4;           // 32 KB: one epilogue round, re and im staging
constexpr int SMEM_BYTES = OPERAND_BYTES + EPI_BYTES + 1024 /*alignment slack*/ + 256 /*barriers*/;
static_assert(Cfg<false>::STAGES * Cfg<false>::STAGE_BYTES == OPERAND_BYTES && Cfg<true>::STAGES * Cfg<true>::STAGE_BYTES == OPERAND_BYTES, "stages");
constexpr int NUM_THREADS = 192;
constexpr uint32_t TMEM_COLS = 512;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;

struct TcParams {
    float* d_re; float* d_im;
    const float* r_re; const float* r_im;
    int M, N, K, conjB, accumulate;
    int units_per_cta;        // consecutive (tile, k-block) work units per CTA (stream-K)
    int a_mn, b_mn;           // operand stored [K, rows] (MN-major) instead of [rows, K] (K-major)
    int cluster;              // > 1: that many CTAs of one cluster share a tile, each a slice of K
    int whole_per_cta;        // > 0: every CTA first takes that many whole tiles, then its run of the remaining units
    int segments;             // > 0: CTA r takes k-segment r / tiles of tile r % tiles (units_per_cta k-blocks each)
    int* status;
    // The pair form (cgemm_tc_k<true>): cluster = K slices per tile, each slice a CTA pair (cluster of 2 * cluster CTAs).
};

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t) __cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait: false (and the error word set) if the phase did not complete in WAIT_LIMIT_NS
// or another role already gave up.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status,
                                          int code) {
    if (mbar_try_wait(bar, parity)) return true;
    unsigned long long t0 = global_ns();
    for (;;) {
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (global_ns() - t0 > WAIT_LIMIT_NS) {
            *abort_flag = 1;
            atomicCAS(status, 0, code);
            atomicExch(status + 1, (int) blockIdx.x);
            return false;
        }
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}

__device__ __forceinline__ void tma_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

// The pair form's loads: the data goes to this CTA's shared memory, the completion bytes to the barrier `bar`,
// a shared::cluster address that may lie in the peer CTA (the pair's first CTA collects both halves).
__device__ __forceinline__ void tma2_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma2_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma2_load_4d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}

// shared::cluster address of `local_addr` (a shared::cta address of this CTA's layout) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    return remote;
}

__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}

// MN-major operand tile (source stored [K, rows]): slabs of 32 rows-of-the-operand, each slab
// 16 k-lines of 128 B.  The only layout the tensor core accepts for MN-major TF32 is the 128-byte
// swizzle with 32-byte atomicity: atoms of 4 k-lines (512 B).  Leading byte offset = distance
// between slabs (2 KB), stride byte offset = distance between 4-line k atoms (512 B).
__device__ __forceinline__ uint64_t smem_desc_mn128(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t) ((addr >> 4) & 0x3FFF);
    d |= (uint64_t) (2048 >> 4) << 16;
    d |= (uint64_t) (512 >> 4) << 32;
    d |= (uint64_t) 1 << 46;
    d |= (uint64_t) 1 << 61;                          // layout type: 128-byte swizzle, 32-byte base
    return d;
}

// K-major operand tile, 64-byte swizzle: rows of 64 B, 8-row groups 512 B apart.
__device__ __forceinline__ uint64_t smem_desc_sw64(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t) ((addr >> 4) & 0x3FFF);           // start address, 16-byte units
    d |= (uint64_t) 1 << 16;                          // leading byte offset (unused with swizzle): 1
    d |= (uint64_t) (512 >> 4) << 32;                 // stride byte offset between 8-row groups
    d |= (uint64_t) 1 << 46;                          // descriptor version of sm_100
    d |= (uint64_t) 4 << 61;                          // layout type: 64-byte swizzle
    return d;
}

// bf16 K-major operand tile, 32-byte swizzle: rows of 32 B (16 bf16 = one MMA's depth), 8-row groups 256 B apart.
__device__ __forceinline__ uint64_t smem_desc_sw32(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t) ((addr >> 4) & 0x3FFF);
    d |= (uint64_t) 1 << 16;
    d |= (uint64_t) (256 >> 4) << 32;
    d |= (uint64_t) 1 << 46;
    d |= (uint64_t) 6 << 61;                          // layout type: 32-byte swizzle
    return d;
}

// bf16 MN-major operand tile (source stored [K, rows]): slabs of 64 rows-of-the-operand (128 B), each slab 16
// k-lines; plain 128-byte swizzle, atoms of 8 k-lines (1 KB).  Leading byte offset = slab to slab (2 KB),
// stride byte offset = k atom to k atom (1 KB).
__device__ __forceinline__ uint64_t smem_desc_mn128_b16(uint32_t addr) {
    uint64_t d = 0;
    d |= (uint64_t) ((addr >> 4) & 0x3FFF);
    d |= (uint64_t) (2048 >> 4) << 16;
    d |= (uint64_t) (1024 >> 4) << 32;
    d |= (uint64_t) 1 << 46;
    d |= (uint64_t) 2 << 61;                          // layout type: 128-byte swizzle
    return d;
}

// kind::f16 with bf16 operands, fp32 accumulate, M = 128, N = 256
constexpr uint32_t kInstrDesc16 = (1u << 4) | (1u << 7) | (1u << 10) | ((256u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void umma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

// kind::tf32, fp32 accumulate, A and B K-major, M = 128, N = 256
constexpr uint32_t kInstrDesc = (1u << 4) | (2u << 7) | (2u << 10) | ((256u >> 3) << 17) | ((128u >> 4) << 24);

__device__ __forceinline__ void umma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

// The pair form: one MMA of the pair's first CTA multiplies the 256 rows of A held by both CTAs (128 each, at the
// same shared-memory offsets) with the B operand whose two 128-row halves the two CTAs hold; each CTA's tensor
// memory receives the accumulator rows of its own A.
__device__ __forceinline__ void umma2_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

__device__ __forceinline__ void umma2_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}

// arrives on the barrier at this shared-memory offset in both CTAs of the pair once the MMAs issued so far are done
// (the pair = cluster ranks first_rank and first_rank + 1)
__device__ __forceinline__ void umma2_commit_both(uint32_t bar, uint32_t first_rank) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((unsigned short) (3u << first_rank)) : "memory");
}

__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* v) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

__device__ __forceinline__ void epi_bar_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// Staging tile of one epilogue round: 128 rows x 32 floats per plane, 16-byte chunks XOR-swizzled
// by the row so that both the row-per-thread writes and the row-segment reads are conflict-free.
__device__ __forceinline__ int stage_off(int row, int chunk) { return row * 32 + ((chunk ^ (row & 7)) << 2); }

// Partial tile of one CTA in cluster mode: 128 rows x 128 floats per plane over the (then idle) operand
// stages, 16-byte chunks XOR-swizzled by the row like the staging tile.
__device__ __forceinline__ int part_off(int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 2); }
constexpr int PART_PLANE_BYTES = 128 * 128 * 4;

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

// Brings `bytes` (a multiple of 16, 16-byte aligned) of global memory into L2 through the bulk-copy engine.
// The epilogue reads residual / old-D tiles 128 bytes per row and round; fetched like that from DRAM each
// row segment costs four scattered accesses, fetched here as one 512-byte piece per row, while the tile's
// MMAs run, the later reads hit L2.
__device__ __forceinline__ void l2_prefetch(const float* p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

__device__ __forceinline__ void prefetch_tile_rows(const TcParams& p, const float* re, const float* im, int row,
                                                  int n0) {
    if (row >= p.M || (p.N & 3)) return;
    const uint32_t bytes = (uint32_t) min(BN, p.N - n0) * 4u;
    const size_t o = (size_t) row * p.N + n0;
    if (((reinterpret_cast<uintptr_t>(re + o) | reinterpret_cast<uintptr_t>(im + o)) & 15) != 0) return;
    l2_prefetch(re + o, bytes);
    l2_prefetch(im + o, bytes);
}

// A 16-byte global load that stays where it is written (volatile asm keeps its place among the other
// volatile asms: the tensor-memory loads and barriers), so a batch of them is in flight together.
__device__ __forceinline__ float4 ld_global_now(const float* p) {
    float4 v;
    asm volatile("ld.global.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p));
    return v;
}

// all threads of all CTAs of the cluster; orders shared-memory writes before the peers' reads
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ float4 ld_peer(uint32_t local_addr, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    float4 v;   // volatile keeps it between the two cluster barriers; no memory clobber, so loads can be in flight together
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(remote));
    return v;
}

// Cluster mode, after the first cluster barrier: this CTA sums its band of rows of the tile over the CL
// partial tiles (its own and its peers', through distributed shared memory), adds residual / old D and
// stores.  Two 16-byte chunks per thread and round: every load of both (2 * CL peer loads per plane pair,
// residual, old D) is issued before the first sum, so a round costs one round trip.  Fixed summation order.
// The CL partial tiles sit in the CTAs of cluster rank peer0 + c * peer_step (one CTA per tile: 0 and 1; CTA pairs:
// this CTA's rank in its pair and 2: the peers are the CTAs that hold the same 128 rows).
template <int CL>
__device__ __forceinline__ void cluster_reduce(const TcParams& p, uint32_t smem_base, uint32_t crank, int m0, int n0,
                                               int et, bool vec_ok, uint32_t peer0, uint32_t peer_step) {
    constexpr int ROWS = BM / CL;
    constexpr int U = CL <= 4 ? 2 : 1;                   // chunks per thread and round
    for (int base = et; base < ROWS * 32; base += 128 * U) {
        float4 xr[U][CL], xi[U][CL], vr[U], vi[U];
        size_t o[U];
        bool live[U];
        int gn[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int idx = base + 128 * u;
            const int r = (int) crank * ROWS + (idx >> 5), ch = idx & 31;
            const int gm = m0 + r;
            gn[u] = n0 + ch * 4;
            live[u] = idx < ROWS * 32 && gm < p.M && gn[u] < p.N;
            o[u] = (size_t) gm * p.N + gn[u];
            vr[u] = make_float4(0.f, 0.f, 0.f, 0.f); vi[u] = vr[u];
            if (!live[u]) continue;
            const uint32_t local = smem_base + 4u * (uint32_t) part_off(r, ch);
#pragma unroll
            for (int c = 0; c < CL; ++c) {
                const uint32_t peer = peer0 + (uint32_t) c * peer_step;
                xr[u][c] = ld_peer(local, peer); xi[u][c] = ld_peer(local + PART_PLANE_BYTES, peer);
            }
            if (vec_ok) {
                if (p.r_re) { vr[u] = ld_global_now(p.r_re + o[u]); vi[u] = ld_global_now(p.r_im + o[u]); }
                if (p.accumulate) {
                    const float4 dr = ld_global_now(p.d_re + o[u]), di = ld_global_now(p.d_im + o[u]);
                    vr[u].x += dr.x; vr[u].y += dr.y; vr[u].z += dr.z; vr[u].w += dr.w;
                    vi[u].x += di.x; vi[u].y += di.y; vi[u].z += di.z; vi[u].w += di.w;
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (!live[u]) continue;
            float4 sr = make_float4(0.f, 0.f, 0.f, 0.f), si = sr;
#pragma unroll
            for (int c = 0; c < CL; ++c) {
                sr.x += xr[u][c].x; sr.y += xr[u][c].y; sr.z += xr[u][c].z; sr.w += xr[u][c].w;
                si.x += xi[u][c].x; si.y += xi[u][c].y; si.z += xi[u][c].z; si.w += xi[u][c].w;
            }
            if (vec_ok) {
                vr[u].x += sr.x; vr[u].y += sr.y; vr[u].z += sr.z; vr[u].w += sr.w;
                vi[u].x += si.x; vi[u].y += si.y; vi[u].z += si.z; vi[u].w += si.w;
                *reinterpret_cast<float4*>(p.d_re + o[u]) = vr[u];
                *reinterpret_cast<float4*>(p.d_im + o[u]) = vi[u];
            } else {
                const float wr[4] = {sr.x, sr.y, sr.z, sr.w}, wi[4] = {si.x, si.y, si.z, si.w};
                for (int k = 0; k < 4 && gn[u] + k < p.N; ++k) {
                    float ar = wr[k], ai = wi[k];
                    if (p.r_re) { ar += p.r_re[o[u] + k]; ai += p.r_im[o[u] + k]; }
                    if (p.accumulate) { ar += p.d_re[o[u] + k]; ai += p.d_im[o[u] + k]; }
                    p.d_re[o[u] + k] = ar; p.d_im[o[u] + k] = ai;
                }
            }
        }
    }
}

// Phase stamps of CTA 0 (a build with -DCNB_GEMM_TIMING only; read back from the status block): %globaltimer ns.
#ifdef CNB_GEMM_TIMING
#define CNB_GSTAMP(k, cond)                                                                        \
    do { if (blockIdx.x == 0 && (cond)) p.status[900 + (k)] = (int) global_ns(); } while (0)
#else
#define CNB_GSTAMP(k, cond) do { } while (0)
#endif

template <bool PAIR>
__global__ void __launch_bounds__(NUM_THREADS, 1)
cgemm_tc_k(const __grid_constant__ CUtensorMap a_hi_re, const __grid_constant__ CUtensorMap a_hi_im,
           const __grid_constant__ CUtensorMap a_h16, const __grid_constant__ CUtensorMap a_l16,
           const __grid_constant__ CUtensorMap b_hi_re, const __grid_constant__ CUtensorMap b_hi_im,
           const __grid_constant__ CUtensorMap b_h16, const __grid_constant__ CUtensorMap b_l16,
           const TcParams p) {
    extern __shared__ uint8_t smem_raw[];
    CNB_GSTAMP(0, threadIdx.x == 0);
    // operand stages need the alignment of their swizzle pattern; 1024 B covers every mode
    constexpr int STAGES = Cfg<PAIR>::STAGES, STAGE_BYTES = Cfg<PAIR>::STAGE_BYTES, TILE_M = Cfg<PAIR>::TILE_M;
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    float* stage_re = reinterpret_cast<float*>(smem + OPERAND_BYTES);
    float* stage_im = stage_re + 128 * 32;
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + OPERAND_BYTES + EPI_BYTES);
    // bars[0..S) full, bars[S..2S) empty, bars[2S] accumulators ready, bars[2S+1] accumulators drained
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_n = (p.N + BN - 1) / BN;
    const int tiles_m = (p.M + TILE_M - 1) / TILE_M;
    const int k_blocks = (p.K + BK - 1) / BK;
    const long total_units = (long) tiles_m * tiles_n * k_blocks;
    // In the pair form the two CTAs of a cluster work through the same units (each on its own 128 rows of the
    // 256-row tile): "CTA" below is the pair.
    // Cluster ranks: one CTA per tile: rank = K slice (cluster split-K) or none; pairs: rank = 2 * K slice + place in
    // the pair.
    const uint32_t rank_all = (PAIR || p.cluster > 1) ? cluster_rank() : 0u;
    const uint32_t prank = PAIR ? (rank_all & 1u) : 0u;
    const uint32_t lead_rank = rank_all & ~1u;           // pairs: the pair's first CTA
    const long cta_idx = PAIR ? (long) (blockIdx.x >> 1) : (long) blockIdx.x;
    const long cta_cnt = PAIR ? (long) (gridDim.x >> 1) : (long) gridDim.x;
    const int row_off = PAIR ? (int) prank * BM : 0;
    // up to two consecutive runs of (tile, k-block) units per CTA
    long u_begin = cta_idx * p.units_per_cta;
    long u_end = min(total_units, u_begin + p.units_per_cta);
    long u2_begin = 0, u2_end = 0;
    if (p.whole_per_cta > 0) {
        const long lead = (long) p.whole_per_cta * k_blocks;             // whole tiles first ...
        const long rest0 = lead * cta_cnt;                                // ... then a share of what is left
        u2_begin = min(total_units, rest0 + cta_idx * p.units_per_cta);
        u2_end = min(total_units, u2_begin + p.units_per_cta);
        u_begin = lead * cta_idx;
        u_end = u_begin + lead;
    }
    if (p.segments > 0) {
        // Capped chains (K > 4096): consecutive CTAs take the SAME k-segment of consecutive tiles, so the CTAs that
        // run together read the same columns of A and B and share them through L2 (tile-major runs had every CTA
        // of a wave on its own k-range: 5.0 GB of DRAM reads for 0.8 GB of operands at 1024 x 2048 x 16384).
        const long tiles = (long) tiles_m * tiles_n;
        const long seg = cta_idx / tiles, tile = cta_idx % tiles;
        u_begin = tile * k_blocks + seg * p.units_per_cta;
        u_end = min(u_begin + p.units_per_cta, (tile + 1) * k_blocks);
        if (u_begin > u_end) u_begin = u_end;
    }
    const bool split_cluster = p.cluster > 1;
    const uint32_t crank = split_cluster ? (PAIR ? rank_all >> 1 : rank_all) : 0;     // the K slice
    const int cluster_ctas = p.cluster * (PAIR ? 2 : 1);
    if (split_cluster) {                                 // one tile per cluster, an even slice of its k-blocks per CTA (pair)
        const long tile = blockIdx.x / cluster_ctas;
        u_begin = tile * k_blocks + (long) k_blocks * crank / p.cluster;
        u_end = tile * k_blocks + (long) k_blocks * (crank + 1) / p.cluster;
    }
    const uint32_t smem_base = smem_u32(smem);
    const uint32_t bar_base = smem_u32(bars);
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
    const uint32_t acc_full = bar_base + 8u * (2 * STAGES);
    const uint32_t acc_empty = bar_base + 8u * (2 * STAGES + 1);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, PAIR ? 2 : 1);              // pair: the epilogues of both CTAs hand the accumulators back
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {   // whole warp: allocate all 512 tensor-memory columns (1 CTA per SM by shared-memory size)
        if constexpr (PAIR) {                            // the same warp of both CTAs of the pair
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                         "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                         "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    if (warp == 0 && lane < 8) {   // descriptor fetch of the 8 operand maps, off the first TMA's critical path
        const CUtensorMap* maps[8] = {&a_hi_re, &a_hi_im, &a_h16, &a_l16, &b_hi_re, &b_hi_im, &b_h16, &b_l16};
        asm volatile("prefetch.tensormap [%0];" ::"l"(maps[lane]) : "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if constexpr (PAIR) cluster_sync();                  // the peer's barriers exist before anything signals them
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    // Everything above touched no memory another kernel writes: under programmatic dependent launch it ran
    // while the kernel before this one in the stream was finishing.  Operands, residual and old D are read
    // (and D written) only after that kernel has completed.
    cnb_pdl_trigger();
    cnb_pdl_wait();
    CNB_GSTAMP(1, threadIdx.x == 0);

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            const CUtensorMap* maps[8] = {&a_hi_re, &a_hi_im, &a_h16, &a_l16, &b_hi_re, &b_hi_im, &b_h16, &b_l16};
            long it = 0;
            bool live = true;
            for (int pass = 0; pass < 2 && live; ++pass)
            for (long u = pass ? u2_begin : u_begin, ue = pass ? u2_end : u_end; u < ue; ++u, ++it) {
                int tile = (int) (u / k_blocks), kb = (int) (u % k_blocks);
                int m0 = (tile / tiles_n) * TILE_M + row_off, n0 = (tile % tiles_n) * BN;
                int s = (int) (it % STAGES);
                uint32_t phase = (uint32_t) (it / STAGES) & 1;
                if (!mbar_wait(empty_bar(s), phase ^ 1, abort_flag, p.status, 1)) { live = false; break; }
                uint32_t dst = smem_base + s * STAGE_BYTES;
                if constexpr (PAIR) {
                    // Both CTAs fill their own stage; all completion bytes go to the full barrier of the pair's
                    // first CTA, which expects the bytes of both.
                    const uint32_t bar = map_to_rank(full_bar(s), lead_rank);
                    if (prank == 0) mbar_expect_tx(full_bar(s), 2 * STAGE_BYTES);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {        // this CTA's 128 rows of A: hi_re, hi_im, h16 pair, l16 pair
                        if (q < 2) {
                            if (p.a_mn) tma2_load_3d(dst + q * PLANE_BYTES, maps[q], bar, 0, kb * BK, m0 / 32);
                            else tma2_load_2d(dst + q * PLANE_BYTES, maps[q], bar, kb * BK, m0);
                        } else {
                            if (p.a_mn) tma2_load_4d(dst + q * PLANE_BYTES, maps[q], bar, 0, kb * BK, m0 / 64, 0);
                            else tma2_load_3d(dst + q * PLANE_BYTES, maps[q], bar, kb * BK, m0, 0);
                        }
                    }
                    // this CTA's half of the stacked B operand: the real planes (first CTA) or the imaginary ones
                    const int c = (int) prank;
                    uint32_t db = dst + 4 * PLANE_BYTES;
                    if (p.b_mn) tma2_load_3d(db, maps[4 + c], bar, 0, kb * BK, n0 / 32);
                    else tma2_load_2d(db, maps[4 + c], bar, kb * BK, n0);
                    db += PLANE_BYTES;
                    for (int q = 6; q < 8; ++q, db += PLANE_BYTES / 2) {      // h16, l16: boxes of one plane
                        if (p.b_mn) tma2_load_4d(db, maps[q], bar, 0, kb * BK, n0 / 64, c);
                        else tma2_load_3d(db, maps[q], bar, kb * BK, n0, c);
                    }
                    continue;
                }
                mbar_expect_tx(full_bar(s), STAGE_BYTES);
#pragma unroll
                for (int q = 0; q < 8; ++q) {
                    const int r0 = q < 4 ? m0 : n0;
                    const bool mn = q < 4 ? p.a_mn : p.b_mn;
                    if ((q & 3) < 2) {                   // an fp32 hi plane
                        if (mn) tma_load_3d(dst + q * PLANE_BYTES, maps[q], full_bar(s), 0, kb * BK, r0 / 32);
                        else tma_load_2d(dst + q * PLANE_BYTES, maps[q], full_bar(s), kb * BK, r0);
                    } else {                             // a pair of bf16 planes [re ; im]
                        if (mn) tma_load_4d(dst + q * PLANE_BYTES, maps[q], full_bar(s), 0, kb * BK, r0 / 64, 0);
                        else tma_load_3d(dst + q * PLANE_BYTES, maps[q], full_bar(s), kb * BK, r0, 0);
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer (pair: its first CTA only)
        if (lane == 0 && prank == 0) {
            bool ok = true;
            long it = 0;
            int seg = 0;
            // bits 15 / 16 of the instruction descriptor: operand A / B is MN-major
            const uint32_t mn_bits = (p.a_mn ? (1u << 15) : 0u) | (p.b_mn ? (1u << 16) : 0u);
            // pair: M = 256 over the two CTAs
            const uint32_t m_bits = PAIR ? ((256u >> 4) << 24) - ((128u >> 4) << 24) : 0u;
            const uint32_t idesc = (kInstrDesc | mn_bits) + m_bits, idesc16 = (kInstrDesc16 | mn_bits) + m_bits;
            for (int pass = 0; pass < 2; ++pass)
            for (long u = pass ? u2_begin : u_begin, ue = pass ? u2_end : u_end; u < ue && ok; ++seg) {
                int kb0 = (int) (u % k_blocks);
                int kb1 = (int) min((long) k_blocks, kb0 + (ue - u));
                // the epilogue must have drained the previous segment's accumulators
                ok = mbar_wait(acc_empty, (uint32_t) (seg & 1) ^ 1, abort_flag, p.status, 4);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int kb = kb0; kb < kb1 && ok; ++kb, ++it) {
                    int s = (int) (it % STAGES);
                    uint32_t phase = (uint32_t) (it / STAGES) & 1;
                    ok = mbar_wait(full_bar(s), phase, abort_flag, p.status, 2);
                    if (!ok) break;
                    CNB_GSTAMP(2, it == 0);
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    uint32_t st = smem_base + s * STAGE_BYTES;
                    const uint32_t first = kb == kb0 ? 0u : 1u;
                    if constexpr (PAIR) {
                        // slots: 0 / 1 A hi_re / hi_im, 2 / 3 A h16 / l16 [re ; im], 4 B hi, 5 B h16 then l16
                        auto a16 = [&](int slot, int im) {
                            const uint32_t a = st + slot * PLANE_BYTES + im * (PLANE_BYTES / 2);
                            return p.a_mn ? smem_desc_mn128_b16(a) : smem_desc_sw32(a);
                        };
                        auto b16 = [&](int half) {
                            const uint32_t a = st + 5 * PLANE_BYTES + half * (PLANE_BYTES / 2);
                            return p.b_mn ? smem_desc_mn128_b16(a) : smem_desc_sw32(a);
                        };
                        const uint64_t b_h16 = b16(0), b_l16 = b16(1);
                        umma2_bf16(tmem_base, a16(3, 0), b_h16, idesc16, first);
                        umma2_bf16(tmem_base, a16(2, 0), b_l16, idesc16, 1u);
                        umma2_bf16(tmem_base + 256, a16(3, 1), b_h16, idesc16, first);
                        umma2_bf16(tmem_base + 256, a16(2, 1), b_l16, idesc16, 1u);
#pragma unroll
                        for (int j = 0; j < BK / 8; ++j) {
                            const uint32_t ka = p.a_mn ? j * 1024 : j * 32, kbo = p.b_mn ? j * 1024 : j * 32;
                            auto adesc = [&](int plane) {
                                uint32_t a = st + plane * PLANE_BYTES + ka;
                                return p.a_mn ? smem_desc_mn128(a) : smem_desc_sw64(a);
                            };
                            const uint32_t bb = st + 4 * PLANE_BYTES + kbo;
                            const uint64_t b_h = p.b_mn ? smem_desc_mn128(bb) : smem_desc_sw64(bb);
                            umma2_tf32(tmem_base, adesc(0), b_h, idesc, 1u);
                            umma2_tf32(tmem_base + 256, adesc(1), b_h, idesc, 1u);
                        }
                        umma2_commit_both(empty_bar(s), lead_rank);  // the stage is free in both CTAs once these MMAs have read it
                        continue;
                    }
                    {
                        // the cross terms first (small terms first): one BF16 k-step covers the whole 16-deep block.
                        // A slots 2 / 3 hold [re ; im] of h16 / l16 (4 KB each), B slots 6 / 7 the 256-row operands.
                        auto a16 = [&](int slot, int im) {
                            const uint32_t a = st + slot * PLANE_BYTES + im * (PLANE_BYTES / 2);
                            return p.a_mn ? smem_desc_mn128_b16(a) : smem_desc_sw32(a);
                        };
                        auto b16 = [&](int slot) {
                            const uint32_t a = st + slot * PLANE_BYTES;
                            return p.b_mn ? smem_desc_mn128_b16(a) : smem_desc_sw32(a);
                        };
                        const uint64_t b_h16 = b16(6), b_l16 = b16(7);
                        umma_bf16(tmem_base, a16(3, 0), b_h16, idesc16, first);          // lo(A_re) . hi(B)
                        umma_bf16(tmem_base, a16(2, 0), b_l16, idesc16, 1u);             // hi(A_re) . lo(B)
                        umma_bf16(tmem_base + 256, a16(3, 1), b_h16, idesc16, first);    // lo(A_im) . hi(B)
                        umma_bf16(tmem_base + 256, a16(2, 1), b_l16, idesc16, 1u);       // hi(A_im) . lo(B)
                    }
#pragma unroll
                    for (int j = 0; j < BK / 8; ++j) {
                        // one k-step = 8 TF32: 32 bytes along a K-major swizzled row, or one 1 KB atom of k-lines
                        const uint32_t ka = p.a_mn ? j * 1024 : j * 32, kbo = p.b_mn ? j * 1024 : j * 32;
                        auto adesc = [&](int plane) {
                            uint32_t a = st + plane * PLANE_BYTES + ka;
                            return p.a_mn ? smem_desc_mn128(a) : smem_desc_sw64(a);
                        };
                        const uint32_t bb = st + 4 * PLANE_BYTES + kbo;             // [B_re ; B_im] hi, 256 rows
                        const uint64_t b_h = p.b_mn ? smem_desc_mn128(bb) : smem_desc_sw64(bb);
                        umma_tf32(tmem_base, adesc(0), b_h, idesc, 1u);              // hi(A_re) . hi(B)
                        umma_tf32(tmem_base + 256, adesc(1), b_h, idesc, 1u);        // hi(A_im) . hi(B)
                    }
                    umma_commit(empty_bar(s));       // the stage is free once these MMAs have read it
                }
                if (ok) { if constexpr (PAIR) umma2_commit_both(acc_full, lead_rank); else umma_commit(acc_full); }
                CNB_GSTAMP(3, true);
                u += kb1 - kb0;
            }
        }
    } else {
        // -------------------------------------------------------------------- epilogue
        const int q = warp & 3;                      // TMEM lane quarter this warp may read
        const int row = q * 32 + lane;
        const int et = (warp - 2) * 32 + lane;       // 0..127 within the epilogue group
        const uint32_t tl = tmem_base + ((uint32_t) (q * 32) << 16);
        const float sgn = p.conjB ? 1.f : -1.f;
        const bool vec_ok = (p.N % 4 == 0) &&
            ((reinterpret_cast<uintptr_t>(p.d_re) | reinterpret_cast<uintptr_t>(p.d_im) |
              reinterpret_cast<uintptr_t>(p.r_re) | reinterpret_cast<uintptr_t>(p.r_im)) & 15) == 0;
        int seg = 0;
        if (split_cluster) {
            // the whole k-slice is one segment; its partial sums go to shared memory for the cluster reduction
            {
                const int tile = blockIdx.x / cluster_ctas, rows_per = BM / p.cluster;
                const int row = (tile / tiles_n) * TILE_M + row_off + (int) crank * rows_per + et, n0 = (tile % tiles_n) * BN;
                if (et < rows_per) {                     // the band of rows this CTA will write out
                    if (p.r_re) prefetch_tile_rows(p, p.r_re, p.r_im, row, n0);
                    if (p.accumulate) prefetch_tile_rows(p, p.d_re, p.d_im, row, n0);
                }
            }
            mbar_wait(acc_full, 0u, abort_flag, p.status, 3);
            CNB_GSTAMP(4, et == 0);
            epi_bar_sync();
            if (!*abort_flag) {
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                float* part_re = reinterpret_cast<float*>(smem);
                float* part_im = part_re + 128 * 128;
#pragma unroll 1
                for (int c0 = 0; c0 < BN; c0 += 16) {
                    float a[16], f[16], b[16], e[16];
                    tmem_ld16(tl + c0, a);                   // A_re.B_re
                    tmem_ld16(tl + 384 + c0, f);             // A_im.B_im
                    tmem_ld16(tl + 128 + c0, b);             // A_re.B_im
                    tmem_ld16(tl + 256 + c0, e);             // A_im.B_re
                    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                    for (int i = 0; i < 16; i += 4) {
                        const int o = part_off(row, (c0 + i) >> 2);
                        *reinterpret_cast<float4*>(part_re + o) =
                            make_float4(a[i] + sgn * f[i], a[i + 1] + sgn * f[i + 1], a[i + 2] + sgn * f[i + 2],
                                        a[i + 3] + sgn * f[i + 3]);
                        *reinterpret_cast<float4*>(part_im + o) =
                            make_float4(e[i] - sgn * b[i], e[i + 1] - sgn * b[i + 1], e[i + 2] - sgn * b[i + 2],
                                        e[i + 3] - sgn * b[i + 3]);
                    }
                }
            }
            CNB_GSTAMP(5, et == 0);
            u_end = u_begin;                             // nothing left for the loop below
        }
        bool live = true;
        for (int pass = 0; pass < 2 && live; ++pass)
        for (long u = pass ? u2_begin : u_begin, ue = pass ? u2_end : u_end; u < ue; ++seg) {
            int tile = (int) (u / k_blocks), kb0 = (int) (u % k_blocks);
            int kb1 = (int) min((long) k_blocks, kb0 + (ue - u));
            int m0 = (tile / tiles_n) * TILE_M + row_off, n0 = (tile % tiles_n) * BN;
            const bool partial = !(kb0 == 0 && kb1 == k_blocks);   // split tiles are summed with atomics
            const bool add_res = p.r_re != nullptr && kb0 == 0;
            // one row of the tile per epilogue thread, requested before the wait for the MMAs
            if (add_res) prefetch_tile_rows(p, p.r_re, p.r_im, m0 + et, n0);
            if (!partial && p.accumulate) prefetch_tile_rows(p, p.d_re, p.d_im, m0 + et, n0);
            mbar_wait(acc_full, (uint32_t) seg & 1, abort_flag, p.status, 3);
            epi_bar_sync();                          // everyone arrives, then agree on the outcome
            if (*abort_flag) { live = false; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const bool need_old = !partial && p.accumulate;
            const bool pre = vec_ok && (add_res || need_old);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                // What the write-out of this round adds from global memory (residual, old D) is requested
                // now, so that it arrives while the accumulators are drained; asked for between the
                // stores below, each load would wait for the store before it.
                float4 gr[8], gi[8];
                if (pre) {
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int idx = et + 128 * j;
                        const int gm = m0 + (idx >> 3), gn = n0 + c0 + (idx & 7) * 4;
                        gr[j] = make_float4(0.f, 0.f, 0.f, 0.f); gi[j] = gr[j];
                        if (gm >= p.M || gn >= p.N) continue;
                        const size_t o = (size_t) gm * p.N + gn;
                        // the residual if there is one, else old D (both at once: old D is read at the store)
                        if (add_res) {
                            gr[j] = ld_global_now(p.r_re + o);
                            gi[j] = ld_global_now(p.r_im + o);
                        } else {
                            gr[j] = ld_global_now(p.d_re + o);
                            gi[j] = ld_global_now(p.d_im + o);
                        }
                    }
                }
                {
                    float a[16], f[16];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        tmem_ld16(tl + c0 + 16 * h, a);            // A_re.B_re
                        tmem_ld16(tl + 384 + c0 + 16 * h, f);      // A_im.B_im
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int i = 0; i < 16; i += 4)
                            *reinterpret_cast<float4*>(stage_re + stage_off(row, 4 * h + i / 4)) =
                                make_float4(a[i] + sgn * f[i], a[i + 1] + sgn * f[i + 1], a[i + 2] + sgn * f[i + 2],
                                            a[i + 3] + sgn * f[i + 3]);
                    }
                }
                {
                    float b[16], e[16];
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        tmem_ld16(tl + 128 + c0 + 16 * h, b);      // A_re.B_im
                        tmem_ld16(tl + 256 + c0 + 16 * h, e);      // A_im.B_re
                        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                        for (int i = 0; i < 16; i += 4)
                            *reinterpret_cast<float4*>(stage_im + stage_off(row, 4 * h + i / 4)) =
                                make_float4(e[i] - sgn * b[i], e[i + 1] - sgn * b[i + 1], e[i + 2] - sgn * b[i + 2],
                                            e[i + 3] - sgn * b[i + 3]);
                    }
                }
                if (c0 + 32 == BN) {
                    // last TMEM read of this segment done: hand the accumulators back to the MMA warp
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                }
                epi_bar_sync();
                if (c0 + 32 == BN && et == 0) {
                    if constexpr (PAIR) mbar_arrive_cluster(map_to_rank(acc_empty, lead_rank));   // the first CTA's MMA thread waits for both
                    else mbar_arrive(acc_empty);
                }
                // coalesced write-out: each warp instruction covers 4 rows x 128 contiguous bytes
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    int idx = et + 128 * j;
                    int r = idx >> 3, ch = idx & 7;
                    int gm = m0 + r, gn = n0 + c0 + ch * 4;
                    if (gm >= p.M || gn >= p.N) continue;
                    float4 vr = *reinterpret_cast<const float4*>(stage_re + stage_off(r, ch));
                    float4 vi = *reinterpret_cast<const float4*>(stage_im + stage_off(r, ch));
                    size_t o = (size_t) gm * p.N + gn;
                    if (vec_ok) {
                        if (pre) {
                            vr.x += gr[j].x; vr.y += gr[j].y; vr.z += gr[j].z; vr.w += gr[j].w;
                            vi.x += gi[j].x; vi.y += gi[j].y; vi.z += gi[j].z; vi.w += gi[j].w;
                        }
                        if (add_res && need_old) {       // both at once: old D is read here
                            const float4 xr = *reinterpret_cast<const float4*>(p.d_re + o), xi = *reinterpret_cast<const float4*>(p.d_im + o);
                            vr.x += xr.x; vr.y += xr.y; vr.z += xr.z; vr.w += xr.w;
                            vi.x += xi.x; vi.y += xi.y; vi.z += xi.z; vi.w += xi.w;
                        }
                        if (partial) {
                            atomicAdd(reinterpret_cast<float4*>(p.d_re + o), vr);
                            atomicAdd(reinterpret_cast<float4*>(p.d_im + o), vi);
                        } else {
                            *reinterpret_cast<float4*>(p.d_re + o) = vr;
                            *reinterpret_cast<float4*>(p.d_im + o) = vi;
                        }
                    } else {
                        float wr[4] = {vr.x, vr.y, vr.z, vr.w}, wi[4] = {vi.x, vi.y, vi.z, vi.w};
                        for (int k = 0; k < 4 && gn + k < p.N; ++k) {
                            float xr = wr[k], xi = wi[k];
                            if (add_res) { xr += p.r_re[o + k]; xi += p.r_im[o + k]; }
                            if (partial) { atomicAdd(p.d_re + o + k, xr); atomicAdd(p.d_im + o + k, xi); }
                            else {
                                if (p.accumulate) { xr += p.d_re[o + k]; xi += p.d_im[o + k]; }
                                p.d_re[o + k] = xr; p.d_im[o + k] = xi;
                            }
                        }
                    }
                }
                epi_bar_sync();                      // staging is reused by the next round
            }
            u += kb1 - kb0;
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    }
    __syncthreads();
    if (PAIR && !split_cluster) {
        // No CTA of the pair leaves (or frees tensor memory) while the other may still signal its barriers, read its
        // shared memory (the first CTA's MMAs read the peer's operand stages) or write its tensor memory.  Every thread
        // reaches this barrier, also after a bounded wait gave up.  (With a K split the two barriers below do that.)
        cluster_sync();
    }
    if (split_cluster) {
        // Every thread of every CTA of the cluster reaches both barriers, also after a bounded wait gave up.
        cluster_sync();                                  // all partial tiles are in shared memory
        CNB_GSTAMP(6, threadIdx.x == 64);
        if (warp >= 2 && !*abort_flag) {
            const int tile = blockIdx.x / cluster_ctas;
            const int m0 = (tile / tiles_n) * TILE_M + row_off, n0 = (tile % tiles_n) * BN;
            const int et = (warp - 2) * 32 + lane;
            const uint32_t peer0 = PAIR ? prank : 0u, peer_step = PAIR ? 2u : 1u;
            const bool vec_ok = (p.N % 4 == 0) &&
                ((reinterpret_cast<uintptr_t>(p.d_re) | reinterpret_cast<uintptr_t>(p.d_im) |
                  reinterpret_cast<uintptr_t>(p.r_re) | reinterpret_cast<uintptr_t>(p.r_im)) & 15) == 0;
            switch (p.cluster) {
                case 2: cluster_reduce<2>(p, smem_base, crank, m0, n0, et, vec_ok, peer0, peer_step); break;
                case 4: cluster_reduce<4>(p, smem_base, crank, m0, n0, et, vec_ok, peer0, peer_step); break;
                default: cluster_reduce<8>(p, smem_base, crank, m0, n0, et, vec_ok, peer0, peer_step); break;
            }
        }
        CNB_GSTAMP(7, threadIdx.x == 64);
        cluster_sync();                                  // no CTA leaves while a peer still reads its shared memory
        CNB_GSTAMP(8, threadIdx.x == 64);
    }
    if (warp == 1) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if constexpr (PAIR) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// The operand split (cnb_split_store*, common.cuh) of a pair of planes into a split buffer with plane pitch np.
__global__ void split_k(const float* __restrict__ s0, const float* __restrict__ s1, float* __restrict__ sp, size_t np,
                        size_t n) {
    cnb_pdl_enter();
    const cnb_split_dst d0 = cnb_split_component(sp, np, 0), d1 = cnb_split_component(sp, np, 1);
    size_t stride = (size_t) gridDim.x * blockDim.x * 4;
    for (size_t i = ((size_t) blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += stride) {
        if (i + 3 < n) {
            const float4 x = *reinterpret_cast<const float4*>(s0 + i), y = *reinterpret_cast<const float4*>(s1 + i);
            cnb_split_store4(d0, i, x.x, x.y, x.z, x.w);
            cnb_split_store4(d1, i, y.x, y.y, y.z, y.w);
        } else {
            for (size_t j = i; j < n; ++j) { cnb_split_store1(d0, j, s0[j]); cnb_split_store1(d1, j, s1[j]); }
        }
    }
}

// the same, transposed while it is split ([R,C] -> [C,R])
__global__ void split_transpose_k(const float* __restrict__ s0, const float* __restrict__ s1,
                                  float* __restrict__ sp, size_t np, int R, int C) {
    cnb_pdl_enter();
    __shared__ float t0[32][33], t1[32][33];
    const cnb_split_dst d0 = cnb_split_component(sp, np, 0), d1 = cnb_split_component(sp, np, 1);
    int c = blockIdx.x * 32 + threadIdx.x;
    for (int k = threadIdx.y; k < 32; k += 8) {
        int r = blockIdx.y * 32 + k;
        if (r < R && c < C) { t0[k][threadIdx.x] = s0[(size_t) r * C + c]; t1[k][threadIdx.x] = s1[(size_t) r * C + c]; }
    }
    __syncthreads();
    int r = blockIdx.y * 32 + threadIdx.x;
    for (int k = threadIdx.y; k < 32; k += 8) {
        int cc = blockIdx.x * 32 + k;
        if (r < R && cc < C) {
            size_t o = (size_t) cc * R + r;
            cnb_split_store1(d0, o, t0[threadIdx.x][k]);
            cnb_split_store1(d1, o, t1[threadIdx.x][k]);
        }
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// [rows, K] fp32 row-major plane; box = BK x 128 rows; 64-byte swizzle; zero fill outside.
int make_map(CUtensorMap* m, const float* base, int rows, int K) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return cnb::set_error(CNB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t) K, (cuuint64_t) rows};
    cuuint64_t strides[1] = {(cuuint64_t) K * sizeof(float)};
    cuuint32_t box[2] = {(cuuint32_t) BK, 128u};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cnb::set_error(CNB_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for a [%d,%d] plane", (int) r, rows, K);
    return CNB_OK;
}

// MN-major plane stored [K, rows] (rows contiguous, rows % 32 == 0), seen as [rows/32][K][32]:
// one box {32, BK, 4} brings four 32-row slabs of 16 k-lines, slab after slab (128-byte swizzle,
// 32-byte atomicity).
int make_map_mn(CUtensorMap* m, const float* base, int rows, int K) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return cnb::set_error(CNB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[3] = {32u, (cuuint64_t) K, (cuuint64_t) (rows / 32)};
    cuuint64_t strides[2] = {(cuuint64_t) rows * sizeof(float), 32u * sizeof(float)};
    cuuint32_t box[3] = {32u, (cuuint32_t) BK, 4u};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cnb::set_error(CNB_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for an MN-major [%d,%d] plane", (int) r, K, rows);
    return CNB_OK;
}

// A pair of bf16 planes (real, imaginary; np elements apart), each [rows, K] row-major, seen as [2][rows][K]: one
// box {BK, 128, 2} brings the 128 rows of both planes, real then imaginary (planes_per_box = 1: of one plane);
// 32-byte swizzle.
int make_map16(CUtensorMap* m, const void* base, int rows, int K, size_t np, unsigned planes_per_box) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return cnb::set_error(CNB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[3] = {(cuuint64_t) K, (cuuint64_t) rows, 2u};
    cuuint64_t strides[2] = {(cuuint64_t) K * 2u, (cuuint64_t) np * 2u};
    cuuint32_t box[3] = {(cuuint32_t) BK, 128u, planes_per_box};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_32B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cnb::set_error(CNB_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for a bf16 [%d,%d] plane pair", (int) r, rows, K);
    return CNB_OK;
}

// The same pair stored [K, rows] (rows contiguous, rows % 64 == 0), seen as [2][rows/64][K][64]: one box
// {64, BK, 2, 2} brings two 64-row slabs of 16 k-lines of both planes, slab after slab (128-byte swizzle).
int make_map16_mn(CUtensorMap* m, const void* base, int rows, int K, size_t np, unsigned planes_per_box) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return cnb::set_error(CNB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[4] = {64u, (cuuint64_t) K, (cuuint64_t) (rows / 64), 2u};
    cuuint64_t strides[3] = {(cuuint64_t) rows * 2u, 128u, (cuuint64_t) np * 2u};
    cuuint32_t box[4] = {64u, (cuuint32_t) BK, 2u, planes_per_box};
    cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cnb::set_error(CNB_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for an MN-major bf16 [%d,%d] plane pair", (int) r, K, rows);
    return CNB_OK;
}

// Clears the two output planes of a product whose tiles are summed with atomics.
__global__ void zero_pair_k(float* __restrict__ a, float* __restrict__ b, size_t n) {
    cnb_pdl_enter();
    const size_t n4 = n / 4;
    const bool vec = ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) == 0;
    const size_t tid = (size_t) blockIdx.x * blockDim.x + threadIdx.x, step = (size_t) gridDim.x * blockDim.x;
    if (vec) {
        const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
        for (size_t i = tid; i < n4; i += step) {
            reinterpret_cast<float4*>(a)[i] = z;
            reinterpret_cast<float4*>(b)[i] = z;
        }
        for (size_t i = 4 * n4 + tid; i < n; i += step) { a[i] = 0.f; b[i] = 0.f; }
    } else {
        for (size_t i = tid; i < n; i += step) { a[i] = 0.f; b[i] = 0.f; }
    }
}

// The schedule of one product: which form (one CTA per tile or CTA pairs), how many CTAs, how the (tile, k-block)
// units are dealt.  Host arithmetic only (also reachable as cnb_gemm_schedule, for tests that need no GPU).
struct Schedule { bool pair; long ctas, upc; int whole_per_cta, clear_from_row, cluster, segments; bool splits_tiles; };

Schedule choose_schedule(int M, int N, int K, int accumulate, int sm_count, int sm_limit) {
    // Schedule, by tile count ("CTA" = one CTA, or the CTA pair of a 256-row tile; sms = how many of them this launch
    // may fill: leaving a few SMs free (gemm_cta_limit) lets a concurrent collective's kernels run beside the GEMM):
    //  * tiles >= 4 x SMs, or one nearly full wave of one-tile CTAs when D is not read: whole tiles, grid =
    //    tiles, plain stores, fixed summation order;
    //  * more tiles than SMs: persistent CTAs, one per SM; each takes tiles / SMs whole tiles and then an
    //    equal run of the remaining tiles' k-blocks (summed with atomics), so every SM finishes together
    //    and only the remainder needs atomics and a cleared output;
    //  * few tiles and short runs: a cluster per tile (below); otherwise plain stream-K.
    // K > 4096 keeps to stream-K runs: one fp32 accumulation chain in tensor memory that long costs accuracy.
    struct Plan { long ctas, upc; int whole_per_cta, clear_from_row, cluster, segments; bool splits_tiles; };
    const int k_blocks = (K + BK - 1) / BK;
    auto plan = [&](bool pair) {
        Plan q = {};
        const int tile_m = pair ? 2 * BM : BM;
        const int tiles = ((M + tile_m - 1) / tile_m) * ((N + BN - 1) / BN);
        const long total = (long) tiles * k_blocks;
        const long min_units = 8;                            // do not split below 8 k-blocks per CTA
        const int all = pair ? sm_count / 2 : sm_count;
        // Pairs under an SM limit (a few SMs set aside for a collective's kernel): a pair needs both SMs of a TPC and
        // each SM set aside may cost a pair its partner, so they are counted twice (6 set aside: 68 pairs).
        // A limit of exactly half the device (two products side by side, no collective) leaves half the pairs, less
        // a margin of 4.
        const int set_aside = sm_count - sm_limit;
        const bool halved = sm_limit * 2 == sm_count;
        const int pairs_left = halved ? sm_limit / 2 - 4 : (sm_limit - set_aside) / 2;
        const int sms = sm_limit > 0
            ? std::min(pair ? std::max(1, pairs_left) : sm_limit, all) : all;
        const bool full_wave = !accumulate && tiles <= sms && (long) tiles * 100 >= (long) sms * 85 && k_blocks <= 256;
        const bool whole_tiles = (tiles >= all * 4 && sm_limit <= 0 && k_blocks <= 256) || full_wave;
        const bool lead_whole = !whole_tiles && tiles > sms && k_blocks <= 256;
        long ctas = std::min<long>(sms, std::max<long>(1, total / min_units));
        if (whole_tiles) ctas = tiles;                        // many tiles: whole tiles, no atomics
        long upc = (total + ctas - 1) / ctas;
        if (whole_tiles) upc = k_blocks;
        // The tensor core adds into its fp32 accumulator with truncation, so the error of one accumulation chain
        // in tensor memory grows with its length: measured ~2e-6 of the accumulator's magnitude per k-block, which
        // reached 1e-3 on a 443-k-block chain whose accumulator one large term dominated (the gradient of a loss
        // through a K = 8192 product).  Runs are therefore capped at kMaxChain k-blocks (the partial tiles are summed
        // outside, in fp32 round-to-nearest): several equal waves of CTAs instead of one persistent wave.
        // Only K > 4096 gets here with longer runs; a whole tile of K <= 4096 is at most 256 k-blocks.  Each tile is
        // cut into equal segments and the CTAs are numbered segment-major (see the kernel).
        constexpr long kMaxChain = 64;
        if (!whole_tiles && upc > kMaxChain && k_blocks > 256) {
            q.segments = (int) ((k_blocks + kMaxChain - 1) / kMaxChain);     // per tile, each at most kMaxChain k-blocks
            upc = (k_blocks + q.segments - 1) / q.segments;
            ctas = (long) tiles * q.segments;
        } else {
            ctas = (total + upc - 1) / upc;
        }
        if (lead_whole) {
            ctas = sms;
            q.whole_per_cta = tiles / sms;
            const long rest = (long) (tiles - q.whole_per_cta * sms) * k_blocks;
            upc = (rest + ctas - 1) / ctas;
            q.clear_from_row = (q.whole_per_cta * sms / ((N + BN - 1) / BN)) * tile_m;   // rows below are only ever stored whole
        }
        // Few tiles (small batches): a cluster of 2, 4 or 8 CTAs takes one tile, every CTA a slice of K, and
        // the partial tiles are summed through distributed shared memory: no atomics, no cleared output,
        // a fixed summation order.
        // Worth it while a stream-K run would be short (<= 48 k-blocks): with long runs the atomics are
        // amortised and using every SM wins over the clusters' rounded-down CTA count.
        q.cluster = 1;
        if (!whole_tiles && !lead_whole && upc <= 48) {
            // pairs: two slices at most (clusters of 8 CTAs do not all fit a GPC side by side: measured 0.043 ms
            // against 0.025 at 512 x 1024 x 1024)
            for (int c = pair ? 2 : 8; c >= 2; c >>= 1)
                if ((long) tiles * c <= sms && k_blocks / c >= 4) { q.cluster = c; break; }
        }
        if (q.cluster > 1) { ctas = (long) tiles * q.cluster; upc = 0; }
        q.splits_tiles = q.cluster == 1 && (lead_whole ? upc > 0 : (q.segments > 0 || (upc % k_blocks) != 0));
        q.ctas = ctas; q.upc = upc;
        return q;
    };
    // The pair form (two CTAs, cta_group::2, per 256-row tile: each CTA stages half of the B operand, so a k-block
    // costs 48 KB of shared-memory fill per CTA instead of 64 KB): at least one whole pair tile of rows; with few
    // tiles, a cluster of two pairs per tile, each pair a slice of K.
    static const bool pair_allowed = [] { const char* e = getenv("CNB_GEMM_PAIR"); return !(e && e[0] == '0'); }();
    // beside a collective (SMs set aside): measured 2.145 -> 2.115 ms per step at 2 GPUs; CNB_GEMM_PAIR_DP=0 turns it off
    static const bool pair_beside_collective = [] { const char* e = getenv("CNB_GEMM_PAIR_DP"); return !(e && e[0] == '0'); }();
    // not under a limit that halves the device (two products side by side at small batches: measured 1.25 -> 1.31 ms
    // per step at 4 GPUs with pairs there)
    const bool small_reserve = sm_limit > 0 &&
        (sm_count - sm_limit <= 16 || sm_limit * 2 == sm_count);   // or exactly half, no collective
    bool pair = pair_allowed && (sm_limit <= 0 || (pair_beside_collective && small_reserve)) && M >= 2 * BM;
    Plan q = plan(pair);
    if (pair && q.cluster > 1) {                         // K-split clusters: pairs only if they fill as many SMs
        const Plan single = plan(false);
        if (single.ctas > 2 * q.ctas) { pair = false; q = single; }
    }
    Schedule r;
    r.pair = pair; r.ctas = q.ctas; r.upc = q.upc; r.whole_per_cta = q.whole_per_cta; r.clear_from_row = q.clear_from_row;
    r.cluster = q.cluster; r.segments = q.segments; r.splits_tiles = q.splits_tiles;
    return r;
}

}  // namespace

namespace cnb {

bool cgemm_tc_shape_ok(int M, int N, int K) {
    // TMA needs a 16-byte row pitch (8 bf16); small or skinny problems are faster on the SIMT tiles
    return (K % 8 == 0) && K >= 32 && M >= 64 && N >= 64;
}

size_t cgemm_tc_workspace_bytes(int M, int N, int K) {
    return 4 * ((size_t) M * K + (size_t) N * K) * sizeof(float) + 4096;
}

void split_launch(cnb_ctx* ctx, const float* s0, const float* s1, float* sp, size_t np, size_t n, cudaStream_t st) {
    size_t blocks = (n / 4 + 255) / 256 + 1, cap = (size_t) ctx->sm_count * 16;
    cnb::launch(split_k, dim3((unsigned) (blocks < cap ? blocks : cap)), dim3(256), 0, st, 1, s0, s1, sp, np, n);
}

// The GEMM proper on operands that are already split: a[4] / b[4] = the four slots of a split buffer (hi_re,
// hi_im, [h16_re ; h16_im], [l16_re ; l16_im]; slot q+1 follows slot q at the plane pitch), elements stored
// [rows, K] (major = 0) or [K, rows] (major = 1, needs rows % 64 == 0).
int cgemm_tc_presplit(cnb_ctx* ctx, const float* const a[4], int a_mn, const float* const b[4], int b_mn, int conjB,
                      const float* r_re, const float* r_im, float* d_re, float* d_im, int M, int N, int K,
                      int accumulate, cudaStream_t st) {
    static bool attr_set[64] = {};                       // the attribute is per device
    if (!attr_set[ctx->device & 63]) {
        CNB_CUDA(cudaFuncSetAttribute(cgemm_tc_k<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        CNB_CUDA(cudaFuncSetAttribute(cgemm_tc_k<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        attr_set[ctx->device & 63] = true;
    }
    if ((reinterpret_cast<uintptr_t>(d_re) | reinterpret_cast<uintptr_t>(d_im)) & 3)
        return set_error(CNB_ERR_ARG, "cgemm_tc: misaligned output");
    if ((a_mn && M % 64) || (b_mn && N % 64))
        return set_error(CNB_ERR_ARG, "cgemm_tc: an MN-major operand needs a multiple of 64 rows");
    if ((!a_mn && K % 8) || (!b_mn && K % 8))
        return set_error(CNB_ERR_ARG, "cgemm_tc: a K-major operand needs K %% 8 == 0");
    const Schedule q = choose_schedule(M, N, K, accumulate, ctx->sm_count, ctx->gemm_cta_limit);
    const bool pair = q.pair;
    const long ctas = q.ctas, upc = q.upc;
    const int whole_per_cta = q.whole_per_cta, clear_from_row = q.clear_from_row, cluster = q.cluster, segments = q.segments;

    int rc;
    alignas(64) CUtensorMap maps[8];
    const size_t npa = (size_t) (a[3] - a[2]), npb = (size_t) (b[3] - b[2]);     // plane pitch, elements
    const unsigned b_planes = pair ? 1u : 2u;            // pair: a CTA loads the real or the imaginary plane of B
    for (int k = 0; k < 4; ++k) {
        if (k < 2) {
            rc = a_mn ? make_map_mn(&maps[k], a[k], M, K) : make_map(&maps[k], a[k], M, K);
            if (rc != CNB_OK) return rc;
            rc = b_mn ? make_map_mn(&maps[4 + k], b[k], N, K) : make_map(&maps[4 + k], b[k], N, K);
            if (rc != CNB_OK) return rc;
        } else {
            rc = a_mn ? make_map16_mn(&maps[k], a[k], M, K, npa, 2u) : make_map16(&maps[k], a[k], M, K, npa, 2u);
            if (rc != CNB_OK) return rc;
            rc = b_mn ? make_map16_mn(&maps[4 + k], b[k], N, K, npb, b_planes) : make_map16(&maps[4 + k], b[k], N, K, npb, b_planes);
            if (rc != CNB_OK) return rc;
        }
    }
    if (q.splits_tiles && !accumulate) {
        // one launch clears both planes (they need not be adjacent or in one allocation)
        const size_t first = (size_t) clear_from_row * N;
        const size_t plane = (size_t) M * N - first;
        const size_t vec = plane / 4 + 1;
        const int blocks = (int) std::min<size_t>((vec + 255) / 256, (size_t) ctx->sm_count * 8);
        cnb::launch(zero_pair_k, dim3(blocks), dim3(256), 0, st, 1, d_re + first, d_im + first, plane);
        CNB_LAUNCH_CHECK("zero_pair");
    }
    TcParams p;
    p.d_re = d_re; p.d_im = d_im; p.r_re = r_re; p.r_im = r_im;
    p.M = M; p.N = N; p.K = K; p.conjB = conjB; p.accumulate = accumulate;
    p.units_per_cta = (int) upc;
    p.a_mn = a_mn; p.b_mn = b_mn;
    p.cluster = cluster;
    p.whole_per_cta = whole_per_cta;
    p.segments = segments;
    p.status = ctx->d_status;
    if (pair)
        CNB_CUDA(cnb::launch(cgemm_tc_k<true>, dim3((unsigned) (2 * ctas)), dim3(NUM_THREADS), SMEM_BYTES, st, 2 * cluster, maps[0], maps[1],
                             maps[2], maps[3], maps[4], maps[5], maps[6], maps[7], p));
    else
        CNB_CUDA(cnb::launch(cgemm_tc_k<false>, dim3((unsigned) ctas), dim3(NUM_THREADS), SMEM_BYTES, st, cluster, maps[0], maps[1],
                             maps[2], maps[3], maps[4], maps[5], maps[6], maps[7], p));
    CNB_LAUNCH_CHECK("cgemm_tc");
    return CNB_OK;
}

// fp32 operands: split them into scratch first.  a_trans / b_trans say the source is stored
// [K, rows]; it is then consumed MN-major in place (rows % 64 == 0) or transposed while it is split.
int cgemm_tc_run(cnb_ctx* ctx, const float* a_re, const float* a_im, int a_trans, const float* b_re,
                 const float* b_im, int b_trans, int conjB, const float* r_re, const float* r_im, float* d_re,
                 float* d_im, int M, int N, int K, int accumulate, cudaStream_t st, const float* b_split) {
    float* ws = nullptr;
    int rc = ensure_scratch(ctx, cgemm_tc_workspace_bytes(M, N, K), &ws);
    if (rc != CNB_OK) return rc;
    size_t na = ((size_t) M * K + 63) & ~size_t(63), nb = ((size_t) N * K + 63) & ~size_t(63);
    float* ap[4] = {ws, ws + na, ws + 2 * na, ws + 3 * na};          // the four slots of a split buffer
    float* bp[4] = {ws + 4 * na, ws + 4 * na + nb, ws + 4 * na + 2 * nb, ws + 4 * na + 3 * nb};
    int a_mn = 0, b_mn = 0;
    auto split = [&](const float* s0, const float* s1, float** dst, int rows, int trans, int* mn) -> int {
        bool al = ((reinterpret_cast<uintptr_t>(s0) | reinterpret_cast<uintptr_t>(s1)) & 15) == 0;
        const size_t np = (size_t) (dst[1] - dst[0]);
        if (trans && !(rows % 64 == 0 && al)) {   // source is [K, rows] with ragged rows: transpose while splitting
            dim3 grid((rows + 31) / 32, (K + 31) / 32), block(32, 8);
            cnb::launch(split_transpose_k, grid, block, 0, st, 1, s0, s1, dst[0], np, K, rows);
        } else {
            if (!al) return set_error(CNB_ERR_ARG, "cgemm_tc: operand planes must be 16-byte aligned");
            *mn = trans;
            split_launch(ctx, s0, s1, dst[0], np, (size_t) rows * K, st);
        }
        CNB_LAUNCH_CHECK("split");
        return CNB_OK;
    };
    if ((rc = split(a_re, a_im, ap, M, a_trans, &a_mn)) != CNB_OK) return rc;
    if (b_split) {                                 // a constant B operand split once by its owner, [N, K]
        for (int q = 0; q < 4; ++q) bp[q] = const_cast<float*>(b_split) + q * nb;
    } else if ((rc = split(b_re, b_im, bp, N, b_trans, &b_mn)) != CNB_OK) {
        return rc;
    }
    return cgemm_tc_presplit(ctx, ap, a_mn, bp, b_mn, conjB, r_re, r_im, d_re, d_im, M, N, K, accumulate, st);
}

int split_planes(cnb_ctx* ctx, const float* re, const float* im, size_t n, float* split, cudaStream_t st) {
    if (((reinterpret_cast<uintptr_t>(re) | reinterpret_cast<uintptr_t>(im) | reinterpret_cast<uintptr_t>(split)) & 15) != 0)
        return set_error(CNB_ERR_ARG, "split: planes must be 16-byte aligned");
    size_t np = (n + 63) & ~size_t(63);
    split_launch(ctx, re, im, split, np, n, st);
    CNB_LAUNCH_CHECK("split");
    return CNB_OK;
}

int cgemm_tc_nt(cnb_ctx* ctx, const float* a_re, const float* a_im, const float* b_re, const float* b_im, int conjB,
                const float* r_re, const float* r_im, float* d_re, float* d_im, int M, int N, int K, int accumulate,
                cudaStream_t st) {
    return cgemm_tc_run(ctx, a_re, a_im, 0, b_re, b_im, 0, conjB, r_re, r_im, d_re, d_im, M, N, K, accumulate, st);
}

}  // namespace cnb

extern "C" int cnb_gemm_schedule(int M, int N, int K, int accumulate, int sm_count, int sm_limit, int* out8) {
    if (!out8 || M <= 0 || N <= 0 || K <= 0 || sm_count <= 0)
        return cnb::set_error(CNB_ERR_ARG, "cnb_gemm_schedule: M=%d N=%d K=%d sm_count=%d", M, N, K, sm_count);
    const Schedule q = choose_schedule(M, N, K, accumulate, sm_count, sm_limit);
    out8[0] = q.pair ? 1 : 0;
    out8[1] = (int) (q.pair ? 2 * q.ctas : q.ctas);      // CTAs of the launch
    out8[2] = q.cluster * (q.pair ? 2 : 1);              // CTAs per cluster (1: no cluster)
    out8[3] = (int) q.upc;
    out8[4] = q.whole_per_cta;
    out8[5] = q.segments;
    out8[6] = q.splits_tiles ? 1 : 0;
    out8[7] = q.clear_from_row;
    return CNB_OK;
}
