// Shared-memory FFT for FourierTrans at N = R*R (R = 16, 32, 64: N = 256, 1024, 4096).
//
// One group of R threads transforms one row with the four-step factorisation N = R x R:
//   pass 1: thread n2 loads x[R*n1 + n2] (coalesced over n2), does an R-point FFT over n1 in
//           registers, multiplies by the twiddle w_N^(n2*k1) and stores to shared memory;
//   pass 2: thread k1 reads its R values (padded rows, conflict-free), does the second R-point
//           FFT in registers and writes X[k1 + R*k2] (coalesced over k1), scaled by N^-1/2.
// HBM traffic is one read and one write of the tensor; a dense DFT GEMM of the same size is
// 8*N flops per element instead.  Twiddles: register FFTs use literal constants; the N-point
// table is generated once per N in double precision.  direction = +1 gives the conjugate
// (backward) transform dX*[q] = N^-1/2 sum_p G*[p] e^{+2 pi i pq/N}.
#include "common.cuh"
#include "fft_regs.cuh"

namespace {

using namespace cnb_fft;

// Barrier among the R threads that share a row: they sit in one warp when R <= 32, so warps run
// their load / transform / store phases independently and overlap each other's memory latency.
template <int R> __device__ __forceinline__ void row_sync() {
    if constexpr (R <= 32) __syncwarp(); else __syncthreads();
}

template <int R, int SIGN>
__global__ void __launch_bounds__(256, (R <= 32 ? 2 : 1))
fft_rr_k(const float* __restrict__ xr, const float* __restrict__ xi, float* __restrict__ yr, float* __restrict__ yi,
         const float2* __restrict__ tw, int B, int accumulate, const FftEpilogue ep) {
    cnb_pdl_enter();
    constexpr int N = R * R;
    constexpr int ROWS = 256 / R;                        // rows per block
    extern __shared__ float smem_f[];
    const int g = threadIdx.x / R, t = threadIdx.x % R;  // row group, thread within the row
    float* sr = smem_f + (size_t) g * 2 * R * (R + 1);
    float* si = sr + R * (R + 1);
    const float scale = rsqrtf((float) N);
    for (long base = (long) blockIdx.x * ROWS; base < B; base += (long) gridDim.x * ROWS) {
        // every thread of the block takes part in the barriers; rows past the end only skip the memory traffic
        const long row = base + g;
        const bool live = row < B;
        float re[R], im[R];
        if (live) {
            // the row comes in with 16-byte loads (R/4 per thread and plane) and is parked in shared memory in
            // natural order; each thread then picks its stride-R elements from there (conflict-free)
            constexpr int V = R / 4;
            const float* pr = xr + row * N;
            const float* pi = xi + row * N;
            float4 a[V], b[V];
#pragma unroll
            for (int v = 0; v < V; ++v) {
                a[v] = *reinterpret_cast<const float4*>(pr + 4 * (t + v * R));
                b[v] = *reinterpret_cast<const float4*>(pi + 4 * (t + v * R));
            }
#pragma unroll
            for (int v = 0; v < V; ++v) {
                *reinterpret_cast<float4*>(sr + 4 * (t + v * R)) = a[v];
                *reinterpret_cast<float4*>(si + 4 * (t + v * R)) = b[v];
            }
        }
        row_sync<R>();
        if (live) {
#pragma unroll
            for (int n1 = 0; n1 < R; ++n1) { re[n1] = sr[n1 * R + t]; im[n1] = si[n1 * R + t]; }
        }
        row_sync<R>();                                   // the parked row is consumed before it is overwritten
        if (live) {
            fft_regs<R, SIGN>(re, im);
#pragma unroll
            for (int p = 0; p < R; ++p) {
                const int k1 = bitrev<R>(p);             // position p holds frequency k1
                float2 w = tw[k1 * R + t];               // e^{-2 pi i t k1/N}: consecutive threads, consecutive entries
                float c = w.x, s = SIGN < 0 ? w.y : -w.y;
                float vr = re[p] * c - im[p] * s, vi = re[p] * s + im[p] * c;
                sr[k1 * (R + 1) + t] = vr;
                si[k1 * (R + 1) + t] = vi;
            }
        }
        row_sync<R>();
        if (live) {
#pragma unroll
            for (int n2 = 0; n2 < R; ++n2) { re[n2] = sr[t * (R + 1) + n2]; im[n2] = si[t * (R + 1) + n2]; }
            fft_regs<R, SIGN>(re, im);
        }
        row_sync<R>();                                   // every row of the tile has been read
        if (live) {
            // back through shared memory in natural order X[k1 + R*k2] so that the row leaves (and, when
            // accumulating, is first read) with contiguous 16-byte accesses
#pragma unroll
            for (int p = 0; p < R; ++p) {
                const int k2 = bitrev<R>(p);
                sr[k2 * (R + 1) + t] = re[p] * scale;
                si[k2 * (R + 1) + t] = im[p] * scale;
            }
        }
        row_sync<R>();
        if (live) {
            float* qr = yr + row * N;
            float* qi = yi + row * N;
            constexpr int V = N / (4 * R);               // float4 per thread and plane
            float4 o_r[V], o_i[V];
            if (accumulate) {
#pragma unroll
                for (int v = 0; v < V; ++v) {
                    o_r[v] = *reinterpret_cast<const float4*>(qr + 4 * (t + v * R));
                    o_i[v] = *reinterpret_cast<const float4*>(qi + 4 * (t + v * R));
                }
            }
#pragma unroll
            for (int v = 0; v < V; ++v) {
                const int e = 4 * (t + v * R);           // element index in the row; e = k1 + R*k2
                float a[4], c[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int idx = e + k;
                    a[k] = sr[(idx / R) * (R + 1) + (idx % R)];
                    c[k] = si[(idx / R) * (R + 1) + (idx % R)];
                }
                float4 vr = make_float4(a[0], a[1], a[2], a[3]), vi = make_float4(c[0], c[1], c[2], c[3]);
                if (accumulate) {
                    vr.x += o_r[v].x; vr.y += o_r[v].y; vr.z += o_r[v].z; vr.w += o_r[v].w;
                    vi.x += o_i[v].x; vi.y += o_i[v].y; vi.z += o_i[v].z; vi.w += o_i[v].w;
                }
                *reinterpret_cast<float4*>(qr + e) = vr;
                *reinterpret_cast<float4*>(qi + e) = vi;
                if (ep.hr) {
                    const float4 h0 = *reinterpret_cast<const float4*>(ep.hr + e), h1 = *reinterpret_cast<const float4*>(ep.hi + e);
                    const float ur[4] = {vr.x, vr.y, vr.z, vr.w}, ui[4] = {vi.x, vi.y, vi.z, vi.w};
                    const float pr[4] = {h0.x, h0.y, h0.z, h0.w}, pi[4] = {h1.x, h1.y, h1.z, h1.w};
                    float gr[4], gi[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        gr[k] = cnb_gelu(ur[k] * pr[k] - ui[k] * pi[k]);
                        gi[k] = cnb_gelu(ur[k] * pi[k] + ui[k] * pr[k]);
                    }
                    const size_t o = (size_t) row * N + e;
                    if (ep.gr) {
                        *reinterpret_cast<float4*>(ep.gr + o) = make_float4(gr[0], gr[1], gr[2], gr[3]);
                        *reinterpret_cast<float4*>(ep.gi + o) = make_float4(gi[0], gi[1], gi[2], gi[3]);
                    }
                    if (ep.sp) {
                        cnb_split_store4(cnb_split_component(ep.sp, ep.np, 0), o, gr[0], gr[1], gr[2], gr[3]);
                        cnb_split_store4(cnb_split_component(ep.sp, ep.np, 1), o, gi[0], gi[1], gi[2], gi[3]);
                    }
                }
            }
        }
        row_sync<R>();
    }
}

// tw[k1 * R + t] = e^{-2 pi i t k1 / N}: laid out so that the R threads of a row read one contiguous line
// per frequency k1 (a table indexed by the product t*k1 costs one cache line per thread).
__global__ void fft_twiddle_k(float2* __restrict__ tw, int R) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= R * R) return;
    int k1 = i / R, t = i % R;
    double s, c;
    sincospi(-2.0 * (double) (t * k1) / (double) (R * R), &s, &c);
    tw[i] = make_float2((float) c, (float) s);
}

template <int R>
int launch_rr(cnb_ctx* ctx, const float* xr, const float* xi, float* yr, float* yi, const float2* tw, int B, int inverse,
           int accumulate, const FftEpilogue& ep, cudaStream_t st) {
    constexpr int ROWS = 256 / R;
    size_t smem = (size_t) ROWS * 2 * R * (R + 1) * sizeof(float);
    static bool attr_done[64][2] = {};                   // the attribute is per device
    bool& done = attr_done[ctx->device & 63][inverse];
    if (!done) {
        if (inverse) CNB_CUDA(cudaFuncSetAttribute(fft_rr_k<R, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
        else CNB_CUDA(cudaFuncSetAttribute(fft_rr_k<R, -1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
        done = true;
    }
    int blocks = (B + ROWS - 1) / ROWS;
    int cap = ctx->sm_count * 8;
    if (blocks > cap) blocks = cap;
    if (inverse) cnb::launch(fft_rr_k<R, 1>, dim3(blocks), dim3(256), smem, st, 1, xr, xi, yr, yi, tw, B, accumulate, ep);
    else cnb::launch(fft_rr_k<R, -1>, dim3(blocks), dim3(256), smem, st, 1, xr, xi, yr, yi, tw, B, accumulate, ep);
    CNB_LAUNCH_CHECK("fft_rr");
    return CNB_OK;
}

}  // namespace

namespace cnb {

bool fft_supported(int N) { return N == 256 || N == 1024 || N == 4096; }

static int fft_dispatch(cnb_ctx* ctx, const float* xr, const float* xi, float* yr, float* yi, int B, int N, int inverse,
                        int accumulate, const FftEpilogue& ep, cudaStream_t st) {
    // the inter-pass twiddle table lives in the arena; the map key -N keeps it apart from DFT matrices
    cnb_twiddle t;
    bool fresh = false;            // the table is being made by the launch just before this one
    auto it = ctx->twiddles.find(-N);
    if (it == ctx->twiddles.end()) {
        fresh = true;
        void* p = nullptr;
        int rc = cnb_alloc(ctx, (size_t) N * sizeof(float2), &p);
        if (rc != CNB_OK) return rc;
        t.re = static_cast<float*>(p);
        fft_twiddle_k<<<(N + 255) / 256, 256, 0, st>>>(reinterpret_cast<float2*>(p), N == 256 ? 16 : N == 1024 ? 32 : 64);
        CNB_LAUNCH_CHECK("fft_twiddle");
        ctx->twiddles[-N] = t;
    } else {
        t = it->second;
    }
    const float2* tw = reinterpret_cast<const float2*>(t.re);
    if (N == 256) return launch_rr<16>(ctx, xr, xi, yr, yi, tw, B, inverse, accumulate, ep, st);
    if (N == 1024) return fft1024_pipe(ctx, xr, xi, yr, yi, tw, B, inverse, accumulate, ep, st, fresh);
    if (N == 4096) return launch_rr<64>(ctx, xr, xi, yr, yi, tw, B, inverse, accumulate, ep, st);
    return set_error(CNB_ERR_UNSUPPORTED, "fft: N=%d", N);
}

int fft_run(cnb_ctx* ctx, const float* xr, const float* xi, float* yr, float* yi, int B, int N, int inverse,
            int accumulate, cudaStream_t st) {
    return fft_dispatch(ctx, xr, xi, yr, yi, B, N, inverse, accumulate, FftEpilogue(), st);
}

int fft_hadamard_gelu(cnb_ctx* ctx, const float* xr, const float* xi, const float* hr, const float* hi, float* ur,
                      float* ui, float* yr, float* yi, float* sp, int B, int N, cudaStream_t st) {
    FftEpilogue ep;
    ep.hr = hr; ep.hi = hi; ep.gr = yr; ep.gi = yi; ep.sp = sp;
    ep.np = ((size_t) B * N + 63) & ~size_t(63);
    return fft_dispatch(ctx, xr, xi, ur, ui, B, N, 0, 0, ep, st);
}

}  // namespace cnb
