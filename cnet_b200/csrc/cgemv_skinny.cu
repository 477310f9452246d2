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

// One CTA per pair of batch rows; each of the 8 warps takes one eighth of the input length, so a
// row pair is in flight on 256 threads (B/2 CTAs keep every SM busy even at a batch of a few hundred).
__global__ void __launch_bounds__(256)
skinny_fwd_k(const float* __restrict__ xr, const float* __restrict__ xi, const float* __restrict__ wr,
             const float* __restrict__ wi, float* __restrict__ yr, float* __restrict__ yi, int B, int in, int out) {
    __shared__ float red[8][2][2][MAXO];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (long b0 = (long) blockIdx.x * 2; b0 < B; b0 += (long) gridDim.x * 2) {
        const bool two = b0 + 1 < B;
        float ar[2][MAXO], ai[2][MAXO];
#pragma unroll
        for (int o = 0; o < MAXO; ++o) { ar[0][o] = ai[0][o] = ar[1][o] = ai[1][o] = 0.f; }
        const float* x0r = xr + b0 * in; const float* x0i = xi + b0 * in;
        const float* x1r = x0r + (two ? in : 0); const float* x1i = x0i + (two ? in : 0);
        for (int i = threadIdx.x; i < in; i += 256) {
            float p0r = x0r[i], p0i = x0i[i], p1r = x1r[i], p1i = x1i[i];
#pragma unroll
            for (int o = 0; o < MAXO; ++o) {
                if (o < out) {
                    float cr = wr[(size_t) o * in + i], ci = wi[(size_t) o * in + i];
                    ar[0][o] += p0r * cr - p0i * ci; ai[0][o] += p0r * ci + p0i * cr;
                    ar[1][o] += p1r * cr - p1i * ci; ai[1][o] += p1r * ci + p1i * cr;
                }
            }
        }
        __syncthreads();                                 // `red` of the previous pair has been consumed
#pragma unroll
        for (int o = 0; o < MAXO; ++o) {
            if (o < out) {
                float s0r = warp_sum(ar[0][o]), s0i = warp_sum(ai[0][o]);
                float s1r = warp_sum(ar[1][o]), s1i = warp_sum(ai[1][o]);
                if (lane == 0) { red[warp][0][0][o] = s0r; red[warp][0][1][o] = s0i; red[warp][1][0][o] = s1r; red[warp][1][1][o] = s1i; }
            }
        }
        __syncthreads();
        if (threadIdx.x < 4 * out) {
            int o = threadIdx.x % out, part = (threadIdx.x / out) & 1, r = threadIdx.x / (2 * out);
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < 8; ++w) s += red[w][r][part][o];
            if (r == 0 || two) (part ? yi : yr)[(b0 + r) * out + o] = s;
        }
    }
}

__global__ void __launch_bounds__(256)
skinny_bwd_x_k(const float* __restrict__ gr, const float* __restrict__ gi, const float* __restrict__ wr,
               const float* __restrict__ wi, float* __restrict__ dr, float* __restrict__ di, int B, int in, int out,
               int accumulate) {
    size_t total = (size_t) B * in;
    for (size_t e = (size_t) blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t) gridDim.x * blockDim.x) {
        size_t b = e / in;
        int i = (int) (e % in);
        float sr = 0.f, si = 0.f;
#pragma unroll
        for (int o = 0; o < MAXO; ++o) {
            if (o < out) {
                float a = gr[b * out + o], c = gi[b * out + o];
                float wre = wr[(size_t) o * in + i], wim = wi[(size_t) o * in + i];
                sr += a * wre + c * wim;          // (a + ic)(wre - i wim)
                si += c * wre - a * wim;
            }
        }
        if (accumulate) { sr += dr[e]; si += di[e]; }
        dr[e] = sr; di[e] = si;
    }
}

// stage 1: partial[c][o][i] = sum over the rows of chunk c of G[b,o] conj(X[b,i]); block = 32 columns x 8 row lanes
__global__ void __launch_bounds__(256)
skinny_bwd_w_stage1_k(const float* __restrict__ gr, const float* __restrict__ gi, const float* __restrict__ xr,
                      const float* __restrict__ xi, float* __restrict__ pr, float* __restrict__ pi, int B, int in,
                      int out, int rows_per_chunk) {
    __shared__ float sr[8][33], si[8][33];
    const int col = blockIdx.x * 32 + threadIdx.x;
    const int r0 = blockIdx.y * rows_per_chunk, r1 = min(B, r0 + rows_per_chunk);
    float ar[MAXO], ai[MAXO];
#pragma unroll
    for (int o = 0; o < MAXO; ++o) ar[o] = ai[o] = 0.f;
    if (col < in) {
        for (int b = r0 + threadIdx.y; b < r1; b += 8) {
            float x = xr[(size_t) b * in + col], y = xi[(size_t) b * in + col];
#pragma unroll
            for (int o = 0; o < MAXO; ++o) {
                if (o < out) {
                    float a = gr[(size_t) b * out + o], c = gi[(size_t) b * out + o];
                    ar[o] += a * x + c * y;       // (a + ic)(x - iy)
                    ai[o] += c * x - a * y;
                }
            }
        }
    }
    for (int o = 0; o < out; ++o) {
        __syncthreads();
        sr[threadIdx.y][threadIdx.x] = ar[o];
        si[threadIdx.y][threadIdx.x] = ai[o];
        __syncthreads();
        if (threadIdx.y == 0 && col < in) {
            float a = 0.f, c = 0.f;
#pragma unroll
            for (int k = 0; k < 8; ++k) { a += sr[k][threadIdx.x]; c += si[k][threadIdx.x]; }
            size_t off = ((size_t) blockIdx.y * out + o) * in + col;
            pr[off] = a; pi[off] = c;
        }
    }
}

__global__ void skinny_bwd_w_stage2_k(const float* __restrict__ pr, const float* __restrict__ pi, float* __restrict__ dr,
                                      float* __restrict__ di, int chunks, size_t n, int accumulate) {
    size_t e = (size_t) blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n) return;
    float a = 0.f, c = 0.f;
    for (int k = 0; k < chunks; ++k) { a += pr[(size_t) k * n + e]; c += pi[(size_t) k * n + e]; }
    if (accumulate) { a += dr[e]; c += di[e]; }
    dr[e] = a; di[e] = c;
}

}  // namespace

namespace cnb {

bool skinny_ok(int B, int in, int out) { return out <= MAXO && in >= 32 && B >= 1; }

size_t skinny_workspace_bytes(int B, int in, int out, int sm_count) {
    int col_blocks = (in + 31) / 32;
    int chunks = (sm_count * 4 + col_blocks - 1) / col_blocks;
    chunks = std::max(1, std::min(chunks, std::min((B + 7) / 8, 128)));
    return (size_t) chunks * out * in * 2 * sizeof(float);
}

int skinny_fwd(cnb_ctx* ctx, const float* xr, const float* xi, const float* wr, const float* wi, float* yr, float* yi,
               int B, int in, int out, cudaStream_t st) {
    long blocks = (B + 1) / 2;
    long cap = (long) ctx->sm_count * 8;
    skinny_fwd_k<<<(int) std::min(blocks, cap), 256, 0, st>>>(xr, xi, wr, wi, yr, yi, B, in, out);
    CNB_LAUNCH_CHECK("skinny_fwd");
    return CNB_OK;
}

int skinny_bwd_x(cnb_ctx* ctx, const float* gr, const float* gi, const float* wr, const float* wi, float* dr, float* di,
                 int B, int in, int out, int accumulate, cudaStream_t st) {
    size_t total = (size_t) B * in;
    size_t blocks = (total + 255) / 256, cap = (size_t) ctx->sm_count * 16;
    skinny_bwd_x_k<<<(int) std::min(blocks, cap), 256, 0, st>>>(gr, gi, wr, wi, dr, di, B, in, out, accumulate);
    CNB_LAUNCH_CHECK("skinny_bwd_x");
    return CNB_OK;
}

int skinny_bwd_w(cnb_ctx* ctx, const float* gr, const float* gi, const float* xr, const float* xi, float* dr, float* di,
                 int B, int in, int out, int accumulate, cudaStream_t st) {
    int col_blocks = (in + 31) / 32;
    int chunks = (ctx->sm_count * 4 + col_blocks - 1) / col_blocks;
    chunks = std::max(1, std::min(chunks, std::min((B + 7) / 8, 128)));
    int rows = (B + chunks - 1) / chunks;
    chunks = (B + rows - 1) / rows;
    float* ws = nullptr;
    size_t n = (size_t) out * in;
    int rc = ensure_scratch(ctx, (size_t) chunks * n * 2 * sizeof(float), &ws);
    if (rc != CNB_OK) return rc;
    float* pr = ws;
    float* pi = ws + (size_t) chunks * n;
    skinny_bwd_w_stage1_k<<<dim3(col_blocks, chunks), dim3(32, 8), 0, st>>>(gr, gi, xr, xi, pr, pi, B, in, out, rows);
    CNB_LAUNCH_CHECK("skinny_bwd_w_stage1");
    skinny_bwd_w_stage2_k<<<(int) ((n + 255) / 256), 256, 0, st>>>(pr, pi, dr, di, chunks, n, accumulate);
    CNB_LAUNCH_CHECK("skinny_bwd_w_stage2");
    return CNB_OK;
}

}  // namespace cnb
