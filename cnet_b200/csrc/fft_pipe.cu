// FourierTrans at N = 1024 as a persistent, bulk-copy pipelined kernel.
//
// One warp owns one row at a time (four-step factorisation 1024 = 32 x 32, both 32-point
// transforms in registers).  The rows move by the bulk-copy engine, not by the warps' own
// loads and stores:
//   in : the next row of the warp (4 KB per plane) is fetched into a staging buffer with
//        cp.async.bulk + an mbarrier while the current row is being transformed;
//   out: the transformed row is written in natural order into the (then free) work tile and
//        leaves with cp.async.bulk (plain) or cp.reduce.async.bulk .add.f32 (accumulate), so
//        the backward transform's "+=" costs no load in the warp.
// The inter-pass twiddle table sits in shared memory.  Rows are dealt round-robin over the
// CTAs first and over a CTA's warps second, so a partial last round is spread over all SMs.
// Every mbarrier wait is bounded; on expiry the kernel records an error word and returns.
#include "common.cuh"
#include "fft_regs.cuh"

namespace {

using namespace cnb_fft;

constexpr int R = 32, N = 1024;
constexpr int WARPS = 12;                            // rows in flight per CTA
constexpr int THREADS = WARPS * 32;
constexpr int TW_BYTES = N * 8;                      // float2 table
constexpr int BAR_BYTES = 128;
constexpr int IN_BYTES = 2 * N * 4;                  // staged row: re plane, im plane
constexpr int WORK_BYTES = 2 * R * (R + 1) * 4;      // padded tile; also the output staging (2 * N * 4 <= this)
constexpr int WARP_BYTES = IN_BYTES + WORK_BYTES;
constexpr int SMEM_BYTES = TW_BYTES + BAR_BYTES + WARPS * WARP_BYTES;
constexpr unsigned long long WAIT_LIMIT_NS = 2000000000ull;
static_assert(WORK_BYTES % 16 == 0 && WARP_BYTES % 16 == 0 && SMEM_BYTES <= 227 * 1024, "shared-memory plan");

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t) __cvta_generic_to_shared(p); }

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

// false (and the error word set) when the row did not arrive within the limit
__device__ __forceinline__ bool row_wait(uint32_t bar, uint32_t parity, int* status) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_ns();
    for (;;) {
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (global_ns() - t0 > WAIT_LIMIT_NS) {
            atomicCAS(status, 0, 21);
            atomicExch(status + 1, (int) blockIdx.x);
            return false;
        }
    }
}

__device__ __forceinline__ void row_fetch(uint32_t dst, const float* re, const float* im, uint32_t bar) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(IN_BYTES) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst), "l"(re), "r"(N * 4), "r"(bar) : "memory");
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst + N * 4), "l"(im), "r"(N * 4), "r"(bar) : "memory");
}

__device__ __forceinline__ void row_store(float* dst, uint32_t src, int accumulate) {
    if (accumulate)
        asm volatile("cp.reduce.async.bulk.global.shared::cta.bulk_group.add.f32 [%0], [%1], %2;"
                     ::"l"(dst), "r"(src), "r"(N * 4) : "memory");
    else
        asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
                     ::"l"(dst), "r"(src), "r"(N * 4) : "memory");
}

// Phase stamps of the first rows of one warp (a build with -DCNB_FFT_TIMING only; read back from the status block).
#ifdef CNB_FFT_TIMING
#define CNB_STAMP(k)                                                                              \
    do {                                                                                          \
        if (blockIdx.x == 0 && w == 0 && t == 0 && stamp_row < 3) {                               \
            long long c_;                                                                         \
            asm volatile("mov.u64 %0, %%clock64;" : "=l"(c_)::"memory");                          \
            status[800 + stamp_row * 12 + (k)] = (int) c_;                                        \
        }                                                                                         \
    } while (0)
#else
#define CNB_STAMP(k) do { } while (0)
#endif

template <int SIGN>
__global__ void __launch_bounds__(THREADS, 1)
fft1024_pipe_k(const float* __restrict__ xr, const float* __restrict__ xi, float* __restrict__ yr,
               float* __restrict__ yi, const float2* __restrict__ tw, int B, int accumulate, const FftEpilogue ep,
               int* status) {
    extern __shared__ __align__(128) unsigned char smem[];
    float2* tws = reinterpret_cast<float2*>(smem);
    const int w = threadIdx.x >> 5, t = threadIdx.x & 31;
    const uint32_t bar = smem_u32(smem + TW_BYTES) + 8 * w;
    float* in_r = reinterpret_cast<float*>(smem + TW_BYTES + BAR_BYTES + (size_t) w * WARP_BYTES);
    float* in_i = in_r + N;
    float* sr = in_r + 2 * N;                            // padded work tile [32][33] per plane
    float* si = sr + R * (R + 1);
    float* out_r = sr;                                   // the finished row, natural order, over the same memory
    float* out_i = sr + N;
    const long stride = (long) gridDim.x * WARPS;
    long row = blockIdx.x + (long) gridDim.x * w;
    // The warp's barrier is set up and its first row requested by the same thread, before the twiddle table is
    // staged: the first fetch runs under the staging.  Rows are fetched only after the kernel before this one
    // in the stream has completed (a CTA of this size never shares an SM with the GEMM's or its own
    // predecessor's, so there is nothing to gain from staging the table ahead of the wait).
    cnb_pdl_trigger();
    cnb_pdl_wait();
    if (t == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar));
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        if (row < B) row_fetch(smem_u32(in_r), xr + row * N, xi + row * N, bar);
    }
    // The table carries the transform's N^-1/2 = 1/32 (a power of two: the products are the same bits as
    // scaling the result).
    for (int i = threadIdx.x; i < N; i += THREADS) { const float2 f = tw[i]; tws[i] = make_float2(f.x * 0.03125f, f.y * 0.03125f); }
    __syncthreads();

    uint32_t phase = 0;
    bool stored = false;
#ifdef CNB_FFT_TIMING
    int stamp_row = 0;
#endif
    for (; row < B; row += stride) {
        CNB_STAMP(0);
        const bool ok = row_wait(bar, phase, status);
        if (!__all_sync(0xffffffffu, ok)) break;
        phase ^= 1;
        float re[R], im[R];
#pragma unroll
        CNB_STAMP(1);
        for (int n1 = 0; n1 < R; ++n1) { re[n1] = in_r[n1 * R + t]; im[n1] = in_i[n1 * R + t]; }
        __syncwarp();
        CNB_STAMP(2);
        const long next = row + stride;
        if (t == 0 && next < B) {                        // the staging buffer is free: fetch the next row now
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            row_fetch(smem_u32(in_r), xr + next * N, xi + next * N, bar);
        }
        CNB_STAMP(3);
        fft_regs<R, SIGN>(re, im);
        CNB_STAMP(4);
        if (stored) {                                    // the previous row must have left the work tile
            if (t == 0) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
            __syncwarp();
        }
        // Eight table entries are read before the eight products that use them are stored: the compiler cannot
        // move a shared-memory load above an earlier shared-memory store, so read one at a time every entry
        // cost a full load latency between two stores (1500 of a row's 3700 clocks).
#pragma unroll
        for (int p0 = 0; p0 < R; p0 += 8) {
            float2 f[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = tws[bitrev<R>(p0 + j) * R + t];   // e^{-2 pi i t k1/N} / 32
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int p = p0 + j, k1 = bitrev<R>(p);                         // position p holds frequency k1
                const float c = f[j].x, s = SIGN < 0 ? f[j].y : -f[j].y;
                sr[k1 * (R + 1) + t] = re[p] * c - im[p] * s;
                si[k1 * (R + 1) + t] = re[p] * s + im[p] * c;
            }
        }
        __syncwarp();
        CNB_STAMP(5);
#pragma unroll
        for (int n2 = 0; n2 < R; ++n2) { re[n2] = sr[t * (R + 1) + n2]; im[n2] = si[t * (R + 1) + n2]; }
        CNB_STAMP(6);
        fft_regs<R, SIGN>(re, im);
        __syncwarp();                                    // the tile has been read by every lane
        CNB_STAMP(7);
#pragma unroll
        for (int p = 0; p < R; ++p) {
            const int k2 = bitrev<R>(p);                 // lane t holds X[t + R*k2]
            out_r[k2 * R + t] = re[p];
            out_i[k2 * R + t] = im[p];
        }
        CNB_STAMP(8);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        __syncwarp();
        CNB_STAMP(9);
        if (t == 0) {
            row_store(yr + row * N, smem_u32(out_r), accumulate);
            row_store(yi + row * N, smem_u32(out_i), accumulate);
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
        }
        stored = true;
        CNB_STAMP(10);
        if (ep.hr) {
            // fused tail: y = gelu(u o h) and its operand split, straight from the registers; a warp's
            // store covers 128 contiguous bytes of an fp32 plane, 64 of a bf16 plane
            const size_t o = (size_t) row * N + t;
            // h of the next position is requested before this position's stores (a load placed after them
            // would have to be issued after them: the compiler cannot tell that they do not alias)
            float hr_next = __ldg(ep.hr + t), hi_next = __ldg(ep.hi + t);      // bitrev(0) = 0
            const cnb_split_dst sp_re = cnb_split_component(ep.sp, ep.np, 0), sp_im = cnb_split_component(ep.sp, ep.np, 1);
#pragma unroll
            for (int p = 0; p < R; ++p) {
                const int e = bitrev<R>(p) * R;
                const float hr = hr_next, hi = hi_next;
                if (p + 1 < R) {
                    hr_next = __ldg(ep.hr + bitrev<R>(p + 1) * R + t);
                    hi_next = __ldg(ep.hi + bitrev<R>(p + 1) * R + t);
                }
                const float gr = cnb_gelu(re[p] * hr - im[p] * hi);
                const float gi = cnb_gelu(re[p] * hi + im[p] * hr);
                if (ep.gr) { ep.gr[o + e] = gr; ep.gi[o + e] = gi; }
                if (ep.sp) {
                    cnb_split_store1(sp_re, o + e, gr);
                    cnb_split_store1(sp_im, o + e, gi);
                }
            }
        }
        CNB_STAMP(11);
#ifdef CNB_FFT_TIMING
        ++stamp_row;
#endif
    }
    // shared memory stays allocated until the engine has read the last row out of it
    if (t == 0) asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
}

}  // namespace

namespace cnb {

int fft1024_pipe(cnb_ctx* ctx, const float* xr, const float* xi, float* yr, float* yi, const float2* tw, int B,
                 int inverse, int accumulate, const cnb_fft::FftEpilogue& ep, cudaStream_t st, bool /*fresh_table*/) {
    static bool attr_done[64] = {};                      // the attribute is per device
    if (!attr_done[ctx->device & 63]) {
        CNB_CUDA(cudaFuncSetAttribute(fft1024_pipe_k<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        CNB_CUDA(cudaFuncSetAttribute(fft1024_pipe_k<-1>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        attr_done[ctx->device & 63] = true;
    }
    const uintptr_t bits = reinterpret_cast<uintptr_t>(xr) | reinterpret_cast<uintptr_t>(xi) |
                           reinterpret_cast<uintptr_t>(yr) | reinterpret_cast<uintptr_t>(yi);
    if (bits & 15) return set_error(CNB_ERR_ARG, "fft: planes must be 16-byte aligned");
    // persistent: one CTA per SM; like the GEMM it fills an SM's shared memory, so while a collective's
    // kernels need SMs (cnb_set_gemm_sm_limit) it leaves the same SMs free instead of waiting for them
    const int sms = ctx->gemm_cta_limit > 0 && ctx->gemm_cta_limit < ctx->sm_count ? ctx->gemm_cta_limit : ctx->sm_count;
    int blocks = B < sms ? B : sms;
    if (inverse) CNB_CUDA(cnb::launch_ex(fft1024_pipe_k<1>, dim3(blocks), dim3(THREADS), SMEM_BYTES, st, 1, true, xr, xi, yr, yi, tw, B, accumulate, ep, ctx->d_status));
    else CNB_CUDA(cnb::launch_ex(fft1024_pipe_k<-1>, dim3(blocks), dim3(THREADS), SMEM_BYTES, st, 1, true, xr, xi, yr, yi, tw, B, accumulate, ep, ctx->d_status));
    CNB_LAUNCH_CHECK("fft1024_pipe");
    return CNB_OK;
}

}  // namespace cnb
