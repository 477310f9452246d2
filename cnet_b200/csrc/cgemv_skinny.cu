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

// Forward: W (out x in, both planes) is staged once per CTA in shared memory; every warp then walks
// batch rows two at a time: each lane owns a strided slice of the input, accumulates the `out`
// products against shared-memory W, and the warp reduces them with shuffles.  X is read once.
__global__ void __launch_bounds__(256)
skinny_fwd_k(const float* __restrict__ xr, const float* __restrict__ xi, const float* __restrict__ wr,
             const float* __restrict__ wi, float* __restrict__ yr, float* __restrict__ yi, int B, int in, int out) {
    extern __shared__ float sw[];                        // [out][in] re, then [out][in] im
    float* swr = sw;
    float* swi = sw + (size_t) out * in;
    for (int e = threadIdx.x; e < out * in; e += blockDim.x) { swr[e] = wr[e]; swi[e] = wi[e]; }
    __syncthreads();
    const int lane = threadIdx.x & 31;
    const long warp = ((long) blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const long nwarps = ((long) gridDim.x * blockDim.x) >> 5;
    for (long b0 = warp * 2; b0 < B; b0 += nwarps * 2) {
        const bool two = b0 + 1 < B;
        float ar[2][MAXO], ai[2][MAXO];
#pragma unroll
        for (int o = 0; o < MAXO; ++o) { ar[0][o] = ai[0][o] = ar[1][o] = ai[1][o] = 0.f; }
        const float* x0r = xr + b0 * in; const float* x0i = xi + b0 * in;
        const float* x1r = x0r + (two ? in : 0); const float* x1i = x0i + (two ? in : 0);
        for (int i = lane; i < in; i += 32) {
            float p0r = x0r[i], p0i = x0i[i], p1r = x1r[i], p1i = x1i[i];
#pragma unroll
            for (int o = 0; o < MAXO; ++o) {
                if (o < out) {
                    float cr = swr[o * in + i], ci = swi[o * in + i];
                    ar[0][o] += p0r * cr - p0i * ci; ai[0][o] += p0r * ci + p0i * cr;
                    ar[1][o] += p1r * cr - p1i * ci; ai[1][o] += p1r * ci + p1i * cr;
                }
            }
        }
#pragma unroll
        for (int o = 0; o < MAXO; ++o) {
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

// dX*: W columns for 4 consecutive inputs are read as float4; G[b, :] is broadcast.
template <int W>
__global__ void __launch_bounds__(256)
skinny_bwd_x_k(const float* __restrict__ gr, const float* __restrict__ gi, const float* __restrict__ wr,
               const float* __restrict__ wi, float* __restrict__ dr, float* __restrict__ di, int B, int in, int out,
               int accumulate) {
    const int per_row = in / W;
    size_t total = (size_t) B * per_row;
    for (size_t e = (size_t) blockIdx.x * blockDim.x + threadIdx.x; e < total; e += (size_t) gridDim.x * blockDim.x) {
        size_t b = e / per_row;
        int i = (int) (e % per_row) * W;
        float sr[W], si[W];
#pragma unroll
        for (int k = 0; k < W; ++k) sr[k] = si[k] = 0.f;
#pragma unroll
        for (int o = 0; o < MAXO; ++o) {
            if (o < out) {
                float a = gr[b * out + o], c = gi[b * out + o];
                float wre[W], wim[W];
                if constexpr (W == 4) {
                    float4 t = *reinterpret_cast<const float4*>(wr + (size_t) o * in + i);
                    float4 u = *reinterpret_cast<const float4*>(wi + (size_t) o * in + i);
                    wre[0] = t.x; wre[1] = t.y; wre[2] = t.z; wre[3] = t.w;
                    wim[0] = u.x; wim[1] = u.y; wim[2] = u.z; wim[3] = u.w;
                } else { wre[0] = wr[(size_t) o * in + i]; wim[0] = wi[(size_t) o * in + i]; }
#pragma unroll
                for (int k = 0; k < W; ++k) {
                    sr[k] += a * wre[k] + c * wim[k];      // (a + ic)(wre - i wim)
                    si[k] += c * wre[k] - a * wim[k];
                }
            }
        }
        size_t off = b * in + i;
        if constexpr (W == 4) {
            float4 vr = make_float4(sr[0], sr[1], sr[2], sr[3]), vi = make_float4(si[0], si[1], si[2], si[3]);
            if (accumulate) {
                float4 pr = *reinterpret_cast<const float4*>(dr + off), pi = *reinterpret_cast<const float4*>(di + off);
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
template <int W>
__global__ void __launch_bounds__(256)
skinny_bwd_w_stage1_k(const float* __restrict__ gr, const float* __restrict__ gi, const float* __restrict__ xr,
                      const float* __restrict__ xi, float* __restrict__ pr, float* __restrict__ pi, int B, int in,
                      int out, int rows_per_chunk) {
    __shared__ float sr[8][32 * W + 1], si[8][32 * W + 1];
    const int col = (blockIdx.x * 32 + threadIdx.x) * W;
    const int r0 = blockIdx.y * rows_per_chunk, r1 = min(B, r0 + rows_per_chunk);
    float ar[MAXO][W], ai[MAXO][W];
#pragma unroll
    for (int o = 0; o < MAXO; ++o)
#pragma unroll
        for (int k = 0; k < W; ++k) ar[o][k] = ai[o][k] = 0.f;
    if (col < in) {
        for (int b = r0 + threadIdx.y; b < r1; b += 8) {
            float x[W], y[W];
            if constexpr (W == 4) {
                float4 t = *reinterpret_cast<const float4*>(xr + (size_t) b * in + col);
                float4 u = *reinterpret_cast<const float4*>(xi + (size_t) b * in + col);
                x[0] = t.x; x[1] = t.y; x[2] = t.z; x[3] = t.w; y[0] = u.x; y[1] = u.y; y[2] = u.z; y[3] = u.w;
            } else { x[0] = xr[(size_t) b * in + col]; y[0] = xi[(size_t) b * in + col]; }
#pragma unroll
            for (int o = 0; o < MAXO; ++o) {
                if (o < out) {
                    float a = gr[(size_t) b * out + o], c = gi[(size_t) b * out + o];
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
    for (int o = 0; o < MAXO; ++o) {
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

int skinny_fwd(cnb_ctx* ctx, const float* xr, const float* xi, const float* wr, const float* wi, float* yr, float* yi,
               int B, int in, int out, cudaStream_t st) {
    size_t smem = (size_t) out * in * 2 * sizeof(float);
    static size_t smem_set_dev[64] = {};                 // the attribute is per device
    size_t& smem_set = smem_set_dev[ctx->device & 63];
    if (smem > smem_set) {
        CNB_CUDA(cudaFuncSetAttribute(skinny_fwd_k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int) smem));
        smem_set = smem;
    }
    long blocks = ((B + 1) / 2 + 7) / 8;                 // 8 warps per CTA, 2 rows per warp and pass
    long cap = (long) ctx->sm_count * (smem > 100 * 1024 ? 1 : 2);
    skinny_fwd_k<<<(int) std::max<long>(1, std::min(blocks, cap)), 256, smem, st>>>(xr, xi, wr, wi, yr, yi, B, in, out);
    CNB_LAUNCH_CHECK("skinny_fwd");
    return CNB_OK;
}

int skinny_bwd_x(cnb_ctx* ctx, const float* gr, const float* gi, const float* wr, const float* wi, float* dr, float* di,
                 int B, int in, int out, int accumulate, cudaStream_t st) {
    bool vec = (in % 4 == 0) && ((reinterpret_cast<uintptr_t>(wr) | reinterpret_cast<uintptr_t>(wi) |
                                  reinterpret_cast<uintptr_t>(dr) | reinterpret_cast<uintptr_t>(di)) & 15) == 0;
    size_t total = (size_t) B * (vec ? in / 4 : in);
    size_t blocks = (total + 255) / 256, cap = (size_t) ctx->sm_count * 16;
    if (vec) skinny_bwd_x_k<4><<<(int) std::min(blocks, cap), 256, 0, st>>>(gr, gi, wr, wi, dr, di, B, in, out, accumulate);
    else skinny_bwd_x_k<1><<<(int) std::min(blocks, cap), 256, 0, st>>>(gr, gi, wr, wi, dr, di, B, in, out, accumulate);
    CNB_LAUNCH_CHECK("skinny_bwd_x");
    return CNB_OK;
}

int skinny_bwd_w(cnb_ctx* ctx, const float* gr, const float* gi, const float* xr, const float* xi, float* dr, float* di,
                 int B, int in, int out, int accumulate, cudaStream_t st) {
    bool vec = (in % 4 == 0) && ((reinterpret_cast<uintptr_t>(xr) | reinterpret_cast<uintptr_t>(xi)) & 15) == 0;
    int w = vec ? 4 : 1;
    int col_blocks = (in + 32 * w - 1) / (32 * w);
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
    if (vec) skinny_bwd_w_stage1_k<4><<<dim3(col_blocks, chunks), dim3(32, 8), 0, st>>>(gr, gi, xr, xi, pr, pi, B, in, out, rows);
    else skinny_bwd_w_stage1_k<1><<<dim3(col_blocks, chunks), dim3(32, 8), 0, st>>>(gr, gi, xr, xi, pr, pi, B, in, out, rows);
    CNB_LAUNCH_CHECK("skinny_bwd_w_stage1");
    skinny_bwd_w_stage2_k<<<(int) ((n + 31) / 32), dim3(32, 8), 0, st>>>(pr, pi, dr, di, chunks, n, accumulate);
    CNB_LAUNCH_CHECK("skinny_bwd_w_stage2");
    return CNB_OK;
}

}  // namespace cnb
