// Skinny complex Linear (out <= 16, e.g. the 1024 -> 10 classifier head): HBM-bound fp32 kernels.
//   forward : Y[b,o]   = sum_i X[b,i] W[o,i]              one warp per pair of batch rows, shuffle reduce
//   dX*     : dX[b,i] (+)= sum_o G[b,o] conj(W[o,i])       element-wise over [B, in], W stays in L1/L2
//   dW*     : dW[o,i] (+)= sum_b G[b,o] conj(X[b,i])       two-stage deterministic reduction over the batch
// Each streams X (or dX) exactly once; W (out x in) is small and cache-resident.
#include "common.cuh"

namespace {

constexpr int MAXO = 16;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ void ldv(const float* p, float (&v)[4]) {
    const float4 t = __ldg(reinterpret_cast<const float4*>(p));
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
}
__device__ __forceinline__ void ldv(const float* p, float (&v)[1]) { v[0] = __ldg(p); }

// OT is a compile-time bound of `out` (4, 8, 10 or 16): the accumulators of the unused outputs cost
// no registers.  W = 4: every lane works on 4 consecutive inputs with 16-byte accesses (in % 4 == 0).

// Forward: W (out x in, both planes) is staged once per CTA in shared memory (one fat CTA per SM, so the
// staging is paid once per SM); every warp then walks batch rows two at a time: each lane owns a strided
// set of input groups, accumulates the `out` products against W, and the warp reduces them with
// shuffles.  X is read once.
template <int OT, int W>
__global__ void __launch_bounds__(512)
skinny_fwd_k(const float* __restrict__ xr, const float* __restrict__ xi, const float* __restrict__ wr,
             const float* __restrict__ wi, float* __restrict__ yr, float* __restrict__ yi, int B, int in, int out,
             int row_warps) {
    cnb_pdl_enter();
    extern __shared__ __align__(16) float sw[];          // [out][in] re, then [out][in] im
    float* swr = sw;
    float* swi = sw + (size_t) out * in;
    const int total = out * in;
    if constexpr (W == 4) {
        for (int e = threadIdx.x * 4; e < total; e += blockDim.x * 4) {
            *reinterpret_cast<float4*>(swr + e) = __ldg(reinterpret_cast<const float4*>(wr + e));
            *reinterpret_cast<float4*>(swi + e) = __ldg(reinterpret_cast<const float4*>(wi + e));
        }
    } else {
        for (int e = threadIdx.x; e < total; e += blockDim.x) { swr[e] = wr[e]; swi[e] = wi[e]; }
    }
    __syncthreads();
    // All warps of the CTA stage W; the first row_warps of them walk rows (small batches: few rows per SM, but the
    // staging still wants the whole CTA: with 4 warps it was 20 of a 64-row launch's 21 us).
    const int lane = threadIdx.x & 31, warp_in_cta = threadIdx.x >> 5;
    if (warp_in_cta >= row_warps) return;
    const long warp = (long) blockIdx.x * row_warps + warp_in_cta;
    const long nwarps = (long) gridDim.x * row_warps;
    const int groups = in / W;
    for (long b0 = warp * 2; b0 < B; b0 += nwarps * 2) {
        const bool two = b0 + 1 < B;
        float ar[2][OT], ai[2][OT];
#pragma unroll
        for (int o = 0; o < OT; ++o) { ar[0][o] = ai[0][o] = ar[1][o] = ai[1][o] = 0.f; }
        const float* x0r = xr + b0 * in; const float* x0i = xi + b0 * in;
        const float* x1r = x0r + (two ? in : 0); const float* x1i = x0i + (two ? in : 0);
#pragma unroll 2
        for (int c = lane; c < groups; c += 32) {
            const int i = c * W;
            float p0r[W], p0i[W], p1r[W], p1i[W];
            ldv(x0r + i, p0r); ldv(x0i + i, p0i); ldv(x1r + i, p1r); ldv(x1i + i, p1i);
#pragma unroll
            for (int o = 0; o < OT; ++o) {
                if (o < out) {
                    float cr[W], ci[W];
                    if constexpr (W == 4) {
                        const float4 t = *reinterpret_cast<const float4*>(swr + o * in + i);
                        const float4 u = *reinterpret_cast<const float4*>(swi + o * in + i);
                        cr[0] = t.x; cr[1] = t.y; cr[2] = t.z; cr[3] = t.w; ci[0] = u.x; ci[1] = u.y; ci[2] = u.z; ci[3] = u.w;
                    } else { cr[0] = swr[o * in + i]; ci[0] = swi[o * in + i]; }
#pragma unroll
                    for (int k = 0; k < W; ++k) {
                        ar[0][o] += p0r[k] * cr[k] - p0i[k] * ci[k]; ai[0][o] += p0r[k] * ci[k] + p0i[k] * cr[k];
                        ar[1][o] += p1r[k] * cr[k] - p1i[k] * ci[k]; ai[1][o] += p1r[k] * ci[k] + p1i[k] * cr[k];
                    }
                }
            }
        }
#pragma unroll
        for (int o = 0; o < OT; ++o) {
            if (o < out) {
                float s0r = warp_sum(ar[0][o]), s0i = warp_sum(ai[0][o]);
                float s1r = warp_sum(ar[1][o]), s1i = warp_sum(ai[1][o]);
                if (lane == 0) {
                    yr[b0 * out + o] = s0r; yi[b0 * out + o] = s0i;
                    if (two) { yr[(b0 + 1) * out + o] = s1r; yi[(b0 + 1) * out + o] = s1i; }
                }
            }
        }
    }
}

// dX*: a thread keeps the W columns of its W consecutive inputs in registers and walks a chunk of batch
// rows; G[b, :] is a broadcast read.  W is fetched once per (column group, row chunk).
template <int OT, int W>
__global__ void __launch_bounds__(256, (OT * W > 40 ? 1 : 2))
skinny_bwd_x_k(const float* __restrict__ gr, const float* __restrict__ gi, const float* __restrict__ wr,
               const float* __restrict__ wi, float* __restrict__ dr, float* __restrict__ di, int B, int in, int out,
               int accumulate, int rows_per_chunk) {
    cnb_pdl_enter();
    const int i = (blockIdx.x * 256 + threadIdx.x) * W;
    if (i >= in) return;
    float wre[OT][W], wim[OT][W];
#pragma unroll
    for (int o = 0; o < OT; ++o) {
        if (o < out) { ldv(wr + (size_t) o * in + i, wre[o]); ldv(wi + (size_t) o * in + i, wim[o]); }
        else {
#pragma unroll
            for (int k = 0; k < W; ++k) wre[o][k] = wim[o][k] = 0.f;
        }
    }
    const int r0 = blockIdx.y * rows_per_chunk, r1 = min(B, r0 + rows_per_chunk);
    // G of the next row is requested before this row's stores (one row of look-ahead in registers)
    float ga[OT], gc[OT];
#pragma unroll
    for (int o = 0; o < OT; ++o) {
        const bool on = o < out && r0 < r1;
        ga[o] = on ? __ldg(gr + (size_t) r0 * out + o) : 0.f;
        gc[o] = on ? __ldg(gi + (size_t) r0 * out + o) : 0.f;
    }
    for (int b = r0; b < r1; ++b) {
        float a_[OT], c_[OT];
#pragma unroll
        for (int o = 0; o < OT; ++o) { a_[o] = ga[o]; c_[o] = gc[o]; }
        if (b + 1 < r1) {
#pragma unroll
            for (int o = 0; o < OT; ++o)
                if (o < out) { ga[o] = __ldg(gr + (size_t) (b + 1) * out + o); gc[o] = __ldg(gi + (size_t) (b + 1) * out + o); }
        }
        float sr[W], si[W];
#pragma unroll
        for (int k = 0; k < W; ++k) sr[k] = si[k] = 0.f;
#pragma unroll
        for (int o = 0; o < OT; ++o) {
            if (o < out) {
                const float a = a_[o], c = c_[o];
#pragma unroll
                for (int k = 0; k < W; ++k) {
                    sr[k] += a * wre[o][k] + c * wim[o][k];      // (a + ic)(wre - i wim)
                    si[k] += c * wre[o][k] - a * wim[o][k];
                }
            }
        }
        const size_t off = (size_t) b * in + i;
        if constexpr (W == 4) {
            float4 vr = make_float4(sr[0], sr[1], sr[2], sr[3]), vi = make_float4(si[0], si[1], si[2], si[3]);
            if (accumulate) {
                const float4 pr = *reinterpret_cast<const float4*>(dr + off), pi = *reinterpret_cast<const float4*>(di + off);
                vr.x += pr.x; vr.y += pr.y; vr.z += pr.z; vr.w += pr.w;
                vi.x += pi.x; vi.y += pi.y; vi.z += pi.z; vi.w += pi.w;
            }
            *reinterpret_cast<float4*>(dr + off) = vr;
            *reinterpret_cast<float4*>(di + off) = vi;
        } else {
            if (accumulate) { sr[0] += dr[off]; si[0] += di[off]; }
            dr[off] = sr[0]; di[off] = si[0];
        }
    }
}

// stage 1: partial[c][o][i] = sum over the rows of chunk c of G[b,o] conj(X[b,i]);
// block = 32 column groups of W columns x 8 row lanes (W = 4: 16-byte reads of X)
template <int OT, int W>
__global__ void __launch_bounds__(256, (OT * W > 40 ? 1 : 2))
skinny_bwd_w_stage1_k(const float* __restrict__ gr, const float* __restrict__ gi, const float* __restrict__ xr,
                      const float* __restrict__ xi, float* __restrict__ pr, float* __restrict__ pi, int B, int in,
                      int out, int rows_per_chunk) {
    cnb_pdl_enter();
    __shared__ float sr[8][32 * W + 1], si[8][32 * W + 1];
    const int col = (blockIdx.x * 32 + threadIdx.x) * W;
    const int r0 = blockIdx.y * rows_per_chunk, r1 = min(B, r0 + rows_per_chunk);
    float ar[OT][W], ai[OT][W];
#pragma unroll
    for (int o = 0; o < OT; ++o)
#pragma unroll
        for (int k = 0; k < W; ++k) ar[o][k] = ai[o][k] = 0.f;
    if (col < in) {
#pragma unroll 2
        for (int b = r0 + threadIdx.y; b < r1; b += 8) {
            float x[W], y[W];
            ldv(xr + (size_t) b * in + col, x); ldv(xi + (size_t) b * in + col, y);
#pragma unroll
            for (int o = 0; o < OT; ++o) {
                if (o < out) {
                    const float a = __ldg(gr + (size_t) b * out + o), c = __ldg(gi + (size_t) b * out + o);
#pragma unroll
                    for (int k = 0; k < W; ++k) {
                        ar[o][k] += a * x[k] + c * y[k];       // (a + ic)(x - iy)
                        ai[o][k] += c * x[k] - a * y[k];
                    }
                }
            }
        }
    }
    const int t = threadIdx.y * 32 + threadIdx.x;
#pragma unroll
    for (int o = 0; o < OT; ++o) {
        if (o < out) {
            __syncthreads();
#pragma unroll
            for (int k = 0; k < W; ++k) {
                sr[threadIdx.y][threadIdx.x * W + k] = ar[o][k];
                si[threadIdx.y][threadIdx.x * W + k] = ai[o][k];
            }
            __syncthreads();
            if (t < 32 * W) {
                int c = blockIdx.x * 32 * W + t;
                if (c < in) {
                    float a = 0.f, d = 0.f;
#pragma unroll
                    for (int k = 0; k < 8; ++k) { a += sr[k][t]; d += si[k][t]; }
                    size_t off = ((size_t) blockIdx.y * out + o) * in + c;
                    pr[off] = a; pi[off] = d;
                }
            }
        }
    }
}

// stage 2: 32 outputs x 8 chunk lanes per block, fixed summation order
__global__ void skinny_bwd_w_stage2_k(const float* __restrict__ pr, const float* __restrict__ pi, float* __restrict__ dr,
                                      float* __restrict__ di, int chunks, size_t n, int accumulate) {
    cnb_pdl_enter();
    __shared__ float sr[8][33], si[8][33];
    size_t e = (size_t) blockIdx.x * 32 + threadIdx.x;
    float a = 0.f, c = 0.f;
    if (e < n)
        for (int k = threadIdx.y; k < chunks; k += 8) { a += pr[(size_t) k * n + e]; c += pi[(size_t) k * n + e]; }
    sr[threadIdx.y][threadIdx.x] = a;
    si[threadIdx.y][threadIdx.x] = c;
    __syncthreads();
    if (threadIdx.y == 0 && e < n) {
#pragma unroll
        for (int k = 1; k < 8; ++k) { a += sr[k][threadIdx.x]; c += si[k][threadIdx.x]; }
        if (accumulate) { a += dr[e]; c += di[e]; }
        dr[e] = a; di[e] = c;
    }
}

}  // namespace

namespace cnb {

bool skinny_ok(int B, int in, int out) {
    // the forward stages W in shared memory: out * in complex values must fit
    return out <= MAXO && in >= 32 && B >= 1 && (size_t) out * in * 8 <= 200 * 1024;
}

size_t skinny_workspace_bytes(int B, int in, int out, int sm_count) {
    (void) sm_count;
    int chunks = std::max(1, std::min((B + 7) / 8, 128));      // upper bound of the launch's choice
    return (size_t) chunks * out * in * 2 * sizeof(float);
}

// picks the instantiation whose output bound is the smallest one that covers `out`
#define CNB_SKINNY_DISPATCH(KERNEL, W, ...)                                   \
    do {                                                                      \
        if (out <= 4) cnb::launch(KERNEL<4, W>, __VA_ARGS__);                 \
        else if (out <= 8) cnb::launch(KERNEL<8, W>, __VA_ARGS__);            \
        else if (out <= 10) cnb::launch(KERNEL<10, W>, __VA_ARGS__);          \
        else cnb::launch(KERNEL<16, W>, __VA_ARGS__);                         \
    } while (0)

static bool aligned16(const void* a, const void* b, const void* c = nullptr, const void* d = nullptr) {
    return ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) | reinterpret_cast<uintptr_t>(c) |
             reinterpret_cast<uintptr_t>(d)) & 15) == 0;
}

int skinny_fwd(cnb_ctx* ctx, const float* xr, const float* xi, const float* wr, const float* wi, float* yr, float* yi,
               int B, int in, int out, cudaStream_t st) {
    const bool vec = (in % 4 == 0) && aligned16(xr, xi, wr, wi);
    const size_t smem = (size_t) out * in * 2 * sizeof(float);
    static size_t smem_set_dev[64] = {};                 // the attribute is per device
    size_t& smem_set = smem_set_dev[ctx->device & 63];
    if (smem > smem_set) {
#define CNB_SKINNY_ATTR(OT, W) CNB_CUDA(cudaFuncSetAttribute(skinny_fwd_k<OT, W>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem))
        CNB_SKINNY_ATTR(4, 4); CNB_SKINNY_ATTR(8, 4); CNB_SKINNY_ATTR(10, 4); CNB_SKINNY_ATTR(16, 4);
        CNB_SKINNY_ATTR(4, 1); CNB_SKINNY_ATTR(8, 1); CNB_SKINNY_ATTR(10, 1); CNB_SKINNY_ATTR(16, 1);
#undef CNB_SKINNY_ATTR
        smem_set = smem;
    }
    // 2 rows per warp and pass; small batches take thinner CTAs so that the rows still spread over the SMs
    const long pairs = (B + 1) / 2;
    int warps = 16;
    while (warps > 4 && pairs < (long) usable_sms(ctx) * warps / 2) warps /= 2;
    const long blocks = (pairs + warps - 1) / warps;
    const int grid = (int) std::max<long>(1, std::min<long>(blocks, usable_sms(ctx)));
    const int threads = 512;                             // every CTA stages W with 16 warps; `warps` of them take rows
    if (vec) CNB_SKINNY_DISPATCH(skinny_fwd_k, 4, dim3(grid), dim3(threads), smem, st, 1, xr, xi, wr, wi, yr, yi, B, in, out, warps);
    else CNB_SKINNY_DISPATCH(skinny_fwd_k, 1, dim3(grid), dim3(threads), smem, st, 1, xr, xi, wr, wi, yr, yi, B, in, out, warps);
    CNB_LAUNCH_CHECK("skinny_fwd");
    return CNB_OK;
}

int skinny_bwd_x(cnb_ctx* ctx, const float* gr, const float* gi, const float* wr, const float* wi, float* dr, float* di,
                 int B, int in, int out, int accumulate, cudaStream_t st) {
    const bool vec = (in % 4 == 0) && aligned16(wr, wi, dr, di);
    const int w = vec ? 4 : 1;
    const int col_blocks = (in + 256 * w - 1) / (256 * w);
    int chunks = std::max(1, usable_sms(ctx) * 2 / col_blocks);            // two CTAs per SM are resident
    chunks = std::min(chunks, B);
    const int rows = (B + chunks - 1) / chunks;
    chunks = (B + rows - 1) / rows;
    const dim3 grid(col_blocks, chunks);
    if (vec) CNB_SKINNY_DISPATCH(skinny_bwd_x_k, 4, dim3(grid), dim3(256), 0, st, 1, gr, gi, wr, wi, dr, di, B, in, out, accumulate, rows);
    else CNB_SKINNY_DISPATCH(skinny_bwd_x_k, 1, dim3(grid), dim3(256), 0, st, 1, gr, gi, wr, wi, dr, di, B, in, out, accumulate, rows);
    CNB_LAUNCH_CHECK("skinny_bwd_x");
    return CNB_OK;
}

int skinny_bwd_w(cnb_ctx* ctx, const float* gr, const float* gi, const float* xr, const float* xi, float* dr, float* di,
                 int B, int in, int out, int accumulate, cudaStream_t st) {
    const bool vec = (in % 4 == 0) && aligned16(xr, xi);
    int w = vec ? 4 : 1;
    int col_blocks = (in + 32 * w - 1) / (32 * w);
    int chunks = (usable_sms(ctx) * 2 + col_blocks - 1) / col_blocks;      // two CTAs per SM are resident
    chunks = std::max(1, std::min(chunks, std::min((B + 7) / 8, 128)));
    int rows = (B + chunks - 1) / chunks;
    chunks = (B + rows - 1) / rows;
    float* ws = nullptr;
    size_t n = (size_t) out * in;
    int rc = ensure_scratch(ctx, (size_t) chunks * n * 2 * sizeof(float), &ws);
    if (rc != CNB_OK) return rc;
    float* pr = ws;
    float* pi = ws + (size_t) chunks * n;
    const dim3 grid(col_blocks, chunks), block(32, 8);
    if (vec) CNB_SKINNY_DISPATCH(skinny_bwd_w_stage1_k, 4, grid, block, 0, st, 1, gr, gi, xr, xi, pr, pi, B, in, out, rows);
    else CNB_SKINNY_DISPATCH(skinny_bwd_w_stage1_k, 1, grid, block, 0, st, 1, gr, gi, xr, xi, pr, pi, B, in, out, rows);
    CNB_LAUNCH_CHECK("skinny_bwd_w_stage1");
    cnb::launch(skinny_bwd_w_stage2_k, dim3((unsigned) ((n + 31) / 32)), dim3(32, 8), 0, st, 1, pr, pi, dr, di, chunks, n, accumulate);
    CNB_LAUNCH_CHECK("skinny_bwd_w_stage2");
    return CNB_OK;
}

}  // namespace cnb
