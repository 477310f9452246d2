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

namespace {

__device__ constexpr float kCos64[32] = {1.000000000e+00f, 9.951847267e-01f, 9.807852804e-01f, 9.569403357e-01f, 9.238795325e-01f, 8.819212643e-01f, 8.314696123e-01f, 7.730104534e-01f, 7.071067812e-01f, 6.343932842e-01f, 5.555702330e-01f, 4.713967368e-01f, 3.826834324e-01f, 2.902846773e-01f, 1.950903220e-01f, 9.801714033e-02f, 6.123233996e-17f, -9.801714033e-02f, -1.950903220e-01f, -2.902846773e-01f, -3.826834324e-01f, -4.713967368e-01f, -5.555702330e-01f, -6.343932842e-01f, -7.071067812e-01f, -7.730104534e-01f, -8.314696123e-01f, -8.819212643e-01f, -9.238795325e-01f, -9.569403357e-01f, -9.807852804e-01f, -9.951847267e-01f};
__device__ constexpr float kSin64[32] = {0.000000000e+00f, 9.801714033e-02f, 1.950903220e-01f, 2.902846773e-01f, 3.826834324e-01f, 4.713967368e-01f, 5.555702330e-01f, 6.343932842e-01f, 7.071067812e-01f, 7.730104534e-01f, 8.314696123e-01f, 8.819212643e-01f, 9.238795325e-01f, 9.569403357e-01f, 9.807852804e-01f, 9.951847267e-01f, 1.000000000e+00f, 9.951847267e-01f, 9.807852804e-01f, 9.569403357e-01f, 9.238795325e-01f, 8.819212643e-01f, 8.314696123e-01f, 7.730104534e-01f, 7.071067812e-01f, 6.343932842e-01f, 5.555702330e-01f, 4.713967368e-01f, 3.826834324e-01f, 2.902846773e-01f, 1.950903220e-01f, 9.801714033e-02f};

template <int R> __device__ __forceinline__ constexpr int bitrev(int v) {
    int r = 0;
    for (int b = 1; b < R; b <<= 1) { r = (r << 1) | (v & 1); v >>= 1; }
    return r;
}

// In-register radix-2 decimation-in-frequency FFT of R points; output index k is found at
// position bitrev(k).  SIGN = -1: e^{-2 pi i jk/R}; +1: conjugate.
template <int R, int SIGN>
__device__ __forceinline__ void fft_regs(float (&re)[R], float (&im)[R]) {
#pragma unroll
    for (int len = R; len >= 2; len >>= 1) {
        const int half = len >> 1;
#pragma unroll
        for (int base = 0; base < R; base += len) {
#pragma unroll
            for (int j = 0; j < half; ++j) {
                const int i0 = base + j, i1 = base + j + half;
                float ar = re[i0], ai = im[i0], br = re[i1], bi = im[i1];
                re[i0] = ar + br; im[i0] = ai + bi;
                float dr = ar - br, di = ai - bi;
                const int t = j * (64 / len);            // w_len^j = w_64^(j*64/len)
                if (t == 0) { re[i1] = dr; im[i1] = di; }
                else {
                    const float c = kCos64[t], s = SIGN * kSin64[t];   // e^{SIGN * 2 pi i t/64}
                    re[i1] = dr * c - di * s;
                    im[i1] = dr * s + di * c;
                }
            }
        }
    }
}

// Barrier among the R threads that share a row: they sit in one warp when R <= 32, so warps run
// their load / transform / store phases independently and overlap each other's memory latency.
template <int R> __device__ __forceinline__ void row_sync() {
    if constexpr (R <= 32) __syncwarp(); else __syncthreads();
}

template <int R, int SIGN>
__global__ void __launch_bounds__(256, (R <= 32 ? 2 : 1))
fft_rr_k(const float* __restrict__ xr, const float* __restrict__ xi, float* __restrict__ yr, float* __restrict__ yi,
         const float2* __restrict__ tw, int B, int accumulate) {
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
            const float* pr = xr + row * N + t;
            const float* pi = xi + row * N + t;
#pragma unroll
            for (int n1 = 0; n1 < R; ++n1) { re[n1] = pr[n1 * R]; im[n1] = pi[n1 * R]; }
            fft_regs<R, SIGN>(re, im);
#pragma unroll
            for (int p = 0; p < R; ++p) {
                const int k1 = bitrev<R>(p);             // position p holds frequency k1
                float2 w = tw[(t * k1) & (N - 1)];       // e^{-2 pi i t k1/N}
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
            }
        }
        row_sync<R>();
    }
}

__global__ void fft_twiddle_k(float2* __restrict__ tw, int N) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= N) return;
    double s, c;
    sincospi(-2.0 * (double) i / (double) N, &s, &c);
    tw[i] = make_float2((float) c, (float) s);
}

template <int R>
int launch(cnb_ctx* ctx, const float* xr, const float* xi, float* yr, float* yi, const float2* tw, int B, int inverse,
           int accumulate, cudaStream_t st) {
    constexpr int ROWS = 256 / R;
    size_t smem = (size_t) ROWS * 2 * R * (R + 1) * sizeof(float);
    static bool attr_done[2] = {false, false};
    if (!attr_done[inverse]) {
        if (inverse) CNB_CUDA(cudaFuncSetAttribute(fft_rr_k<R, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
        else CNB_CUDA(cudaFuncSetAttribute(fft_rr_k<R, -1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
        attr_done[inverse] = true;
    }
    int blocks = (B + ROWS - 1) / ROWS;
    int cap = ctx->sm_count * 8;
    if (blocks > cap) blocks = cap;
    if (inverse) fft_rr_k<R, 1><<<blocks, 256, smem, st>>>(xr, xi, yr, yi, tw, B, accumulate);
    else fft_rr_k<R, -1><<<blocks, 256, smem, st>>>(xr, xi, yr, yi, tw, B, accumulate);
    CNB_LAUNCH_CHECK("fft_rr");
    return CNB_OK;
}

}  // namespace

namespace cnb {

bool fft_supported(int N) { return N == 256 || N == 1024 || N == 4096; }

int fft_run(cnb_ctx* ctx, const float* xr, const float* xi, float* yr, float* yi, int B, int N, int inverse,
            int accumulate, cudaStream_t st) {
    // the N-point twiddle table lives in the arena; the map key -N keeps it apart from DFT matrices
    cnb_twiddle t;
    auto it = ctx->twiddles.find(-N);
    if (it == ctx->twiddles.end()) {
        void* p = nullptr;
        int rc = cnb_alloc(ctx, (size_t) N * sizeof(float2), &p);
        if (rc != CNB_OK) return rc;
        t.re = static_cast<float*>(p);
        fft_twiddle_k<<<(N + 255) / 256, 256, 0, st>>>(reinterpret_cast<float2*>(p), N);
        CNB_LAUNCH_CHECK("fft_twiddle");
        ctx->twiddles[-N] = t;
    } else {
        t = it->second;
    }
    const float2* tw = reinterpret_cast<const float2*>(t.re);
    if (N == 256) return launch<16>(ctx, xr, xi, yr, yi, tw, B, inverse, accumulate, st);
    if (N == 1024) return launch<32>(ctx, xr, xi, yr, yi, tw, B, inverse, accumulate, st);
    if (N == 4096) return launch<64>(ctx, xr, xi, yr, yi, tw, B, inverse, accumulate, st);
    return set_error(CNB_ERR_UNSUPPORTED, "fft: N=%d", N);
}

}  // namespace cnb
