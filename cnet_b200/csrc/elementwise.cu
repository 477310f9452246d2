// HBM-bound element-wise layers of the complex training step: Hadamard, CGelu (and the
// fused pair), CRelu, Residual, gradient pass-through, SGD and Adam updates.
// All kernels stream each plane once with 16-byte accesses where the row length allows
// it (W = 4), else scalar (W = 1); grids are sized in multiples of the SM count.
#include <algorithm>
#include <cmath>
#include <mutex>

#include "common.cuh"

namespace {


template <int W> struct Pack { float v[W]; };

template <int W> __device__ __forceinline__ Pack<W> ld(const float* p, size_t i) {
    Pack<W> r;
    if constexpr (W == 4) {
        float4 t = *reinterpret_cast<const float4*>(p + i);
        r.v[0] = t.x; r.v[1] = t.y; r.v[2] = t.z; r.v[3] = t.w;
    } else {
        r.v[0] = p[i];
    }
    return r;
}

template <int W> __device__ __forceinline__ void st(float* p, size_t i, const Pack<W>& r) {
    if constexpr (W == 4) {
        *reinterpret_cast<float4*>(p + i) = make_float4(r.v[0], r.v[1], r.v[2], r.v[3]);
    } else {
        p[i] = r.v[0];
    }
}

__device__ __forceinline__ float gelu_f(float x) { return cnb_gelu(x); }
__device__ __forceinline__ float dgelu_f(float x) { return cnb_dgelu(x); }

inline int grid_for(size_t work_items, int threads, int sm_count) {
    size_t blocks = (work_items + threads - 1) / threads;
    size_t cap = (size_t) sm_count * 16;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int) blocks;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ------------------------------------------------------------------ Hadamard
template <int W>
__global__ void hadamard_fwd_k(const float* __restrict__ ur, const float* __restrict__ ui,
                               const float* __restrict__ vr, const float* __restrict__ vi, int v_batched,
                               float* __restrict__ yr, float* __restrict__ yi, size_t total, int N) {
    cnb_pdl_enter();
    size_t stride = (size_t) gridDim.x * blockDim.x * W;
    for (size_t i = ((size_t) blockIdx.x * blockDim.x + threadIdx.x) * W; i < total; i += stride) {
        size_t j = v_batched ? i : i % N;
        Pack<W> a = ld<W>(ur, i), b = ld<W>(ui, i), c = ld<W>(vr, j), d = ld<W>(vi, j), r, s;
#pragma unroll
        for (int k = 0; k < W; ++k) {
            r.v[k] = a.v[k] * c.v[k] - b.v[k] * d.v[k];
            s.v[k] = a.v[k] * d.v[k] + b.v[k] * c.v[k];
        }
        st<W>(yr, i, r); st<W>(yi, i, s);
    }
}

// dst (+)= g o conj(o): the element-wise half of the Hadamard backward
template <int W>
__global__ void hadamard_bwd_elem_k(const float* __restrict__ gr, const float* __restrict__ gi,
                                    const float* __restrict__ orr, const float* __restrict__ oi, int o_batched,
                                    float* __restrict__ dr, float* __restrict__ di, int accumulate,
                                    size_t total, int N) {
    cnb_pdl_enter();
    size_t stride = (size_t) gridDim.x * blockDim.x * W;
    for (size_t i = ((size_t) blockIdx.x * blockDim.x + threadIdx.x) * W; i < total; i += stride) {
        size_t j = o_batched ? i : i % N;
        Pack<W> a = ld<W>(gr, i), b = ld<W>(gi, i), c = ld<W>(orr, j), d = ld<W>(oi, j), r, s;
        if (accumulate) { r = ld<W>(dr, i); s = ld<W>(di, i); }
#pragma unroll
        for (int k = 0; k < W; ++k) {
            float pr = a.v[k] * c.v[k] + b.v[k] * d.v[k];     // (a+ib)(c-id)
            float pi = b.v[k] * c.v[k] - a.v[k] * d.v[k];
            r.v[k] = accumulate ? r.v[k] + pr : pr;
            s.v[k] = accumulate ? s.v[k] + pi : pi;
        }
        st<W>(dr, i, r); st<W>(di, i, s);
    }
}

// Column reduction stage 1: partial[c][n] = sum over the rows of chunk c of t[b,n] o conj(u[b,n]).
// MODE 0: t = g (plain Hadamard).  MODE 1: t = CGelu backward of g at a (fused pair); then
// du (+)= t o conj(h) is written in the same pass.
// Block = 32 column groups of W columns x 8 row lanes; with W = 4 every access is 16 bytes and a
// warp touches 512 contiguous bytes of each plane per row.
template <int MODE, int W>
__global__ void __launch_bounds__(256, 4)       // 4 CTAs per SM: the grid below is one full wave
colreduce_stage1_k(const float* __restrict__ gr, const float* __restrict__ gi,
                   const float* __restrict__ ar, const float* __restrict__ ai,
                   const float* __restrict__ ur, const float* __restrict__ ui,
                   const float* __restrict__ hr, const float* __restrict__ hi,
                   float* __restrict__ dur, float* __restrict__ dui, int accumulate_u,
                   float* __restrict__ pr, float* __restrict__ pi,
                   int B, int N, int rows_per_chunk,
                   int* __restrict__ done, float* __restrict__ dvr, float* __restrict__ dvi, int accumulate_v) {
    cnb_pdl_enter();
    __shared__ float sr[8][32 * W + 1], si[8][32 * W + 1];
    __shared__ int s_last;
    const int col = (blockIdx.x * 32 + threadIdx.x) * W;
    const int r0 = blockIdx.y * rows_per_chunk;
    const int r1 = min(B, r0 + rows_per_chunk);
    float accr[W], acci[W];
#pragma unroll
    for (int k = 0; k < W; ++k) accr[k] = acci[k] = 0.f;
    if (col < N) {
        Pack<W> hre, him;
        if (MODE == 1) { hre = ld<W>(hr, col); him = ld<W>(hi, col); }
        for (int b = r0 + threadIdx.y; b < r1; b += 8) {
            size_t i = (size_t) b * N + col;
            Pack<W> tr = ld<W>(gr, i), ti = ld<W>(gi, i), xr = ld<W>(ur, i), xi = ld<W>(ui, i);
            if (MODE == 1) {
                Pack<W> zr, zi, vr, vi;
                if (ar) { zr = ld<W>(ar, i); zi = ld<W>(ai, i); }
                else {                                   // the Hadamard output was not kept: a = u o h again
#pragma unroll
                    for (int k = 0; k < W; ++k) {
                        zr.v[k] = xr.v[k] * hre.v[k] - xi.v[k] * him.v[k];
                        zi.v[k] = xr.v[k] * him.v[k] + xi.v[k] * hre.v[k];
                    }
                }
                if (dur && accumulate_u) { vr = ld<W>(dur, i); vi = ld<W>(dui, i); }
#pragma unroll
                for (int k = 0; k < W; ++k) {
                    // dz* = conj(g*) (dx-dy) + g* (dx+dy) with dx, dy = gelu'(Re a) / 2, gelu'(Im a) / 2:
                    // the real part is Re g* . gelu'(Re a), the imaginary part Im g* . gelu'(Im a)
                    float nr = tr.v[k] * dgelu_f(zr.v[k]), ni = ti.v[k] * dgelu_f(zi.v[k]);
                    tr.v[k] = nr; ti.v[k] = ni;
                    float wr = nr * hre.v[k] + ni * him.v[k], wi = ni * hre.v[k] - nr * him.v[k];   // t o conj(h)
                    if (dur && accumulate_u) { vr.v[k] += wr; vi.v[k] += wi; } else { vr.v[k] = wr; vi.v[k] = wi; }
                }
                if (dur) { st<W>(dur, i, vr); st<W>(dui, i, vi); }
            }
#pragma unroll
            for (int k = 0; k < W; ++k) {
                accr[k] += tr.v[k] * xr.v[k] + ti.v[k] * xi.v[k];        // t o conj(u)
                acci[k] += ti.v[k] * xr.v[k] - tr.v[k] * xi.v[k];
            }
        }
    }
#pragma unroll
    for (int k = 0; k < W; ++k) {
        sr[threadIdx.y][threadIdx.x * W + k] = accr[k];
        si[threadIdx.y][threadIdx.x * W + k] = acci[k];
    }
    __syncthreads();
    // 32 * W columns of this block, summed over the 8 row lanes by the first 32 * W threads
    const int t = threadIdx.y * 32 + threadIdx.x;
    if (t < 32 * W) {
        int c = blockIdx.x * 32 * W + t;
        if (c < N) {
            float a = 0.f, d = 0.f;
#pragma unroll
            for (int k = 0; k < 8; ++k) { a += sr[k][t]; d += si[k][t]; }
            pr[(size_t) blockIdx.y * N + c] = a;
            pi[(size_t) blockIdx.y * N + c] = d;
        }
    }
    if (!done) return;                                   // a second launch sums the partial rows
    // The CTA that finishes last among those of this column block sums the partial rows, always in
    // chunk order (deterministic); nobody waits for anybody.
    __threadfence();
    __syncthreads();
    if (t == 0) s_last = atomicAdd(done + blockIdx.x, 1) == (int) gridDim.y - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const int chunks = gridDim.y;
    if constexpr (W == 4) {
        // 32 threads x 16 bytes cover the 128 columns, 8 lanes share the chunks: a lane's loop is chunks / 8 long
        // and its loads are independent, so the tail is a few L2 round trips instead of one per pair of chunks
        const int cx = (t & 31) * 4, lane8 = t >> 5;
        const int c = blockIdx.x * 128 + cx;
        float4 a = make_float4(0.f, 0.f, 0.f, 0.f), d = a;
        if (c < N) {
#pragma unroll 4
            for (int k = lane8; k < chunks; k += 8) {
                const float4 x = __ldcg(reinterpret_cast<const float4*>(pr + (size_t) k * N + c));
                const float4 y = __ldcg(reinterpret_cast<const float4*>(pi + (size_t) k * N + c));
                a.x += x.x; a.y += x.y; a.z += x.z; a.w += x.w;
                d.x += y.x; d.y += y.y; d.z += y.z; d.w += y.w;
            }
        }
        sr[lane8][cx] = a.x; sr[lane8][cx + 1] = a.y; sr[lane8][cx + 2] = a.z; sr[lane8][cx + 3] = a.w;
        si[lane8][cx] = d.x; si[lane8][cx + 1] = d.y; si[lane8][cx + 2] = d.z; si[lane8][cx + 3] = d.w;
        __syncthreads();
        if (t < 128) {
            const int cc = blockIdx.x * 128 + t;
            if (cc < N) {
                float e = 0.f, f = 0.f;
#pragma unroll
                for (int k = 0; k < 8; ++k) { e += sr[k][t]; f += si[k][t]; }
                if (accumulate_v) { e += dvr[cc]; f += dvi[cc]; }
                dvr[cc] = e; dvi[cc] = f;
            }
        }
    } else {
        const int cx = t % (32 * W), lane8 = t / (32 * W);        // 32 columns x 8 lanes
        constexpr int LANES = 256 / (32 * W);
        const int c = blockIdx.x * 32 * W + cx;
        float a = 0.f, d = 0.f;
        if (c < N)
            for (int k = lane8; k < chunks; k += LANES) {
                a += __ldcg(pr + (size_t) k * N + c);
                d += __ldcg(pi + (size_t) k * N + c);
            }
        sr[lane8][cx] = a;
        si[lane8][cx] = d;
        __syncthreads();
        if (lane8 == 0 && c < N) {
#pragma unroll
            for (int k = 1; k < LANES; ++k) { a += sr[k][cx]; d += si[k][cx]; }
            if (accumulate_v) { a += dvr[c]; d += dvi[c]; }
            dvr[c] = a; dvi[c] = d;
        }
    }
    if (t == 0) done[blockIdx.x] = 0;                    // ready for the next launch
}

// Stage 2: dv[n] (+)= sum_c partial[c][n], always in the same order (deterministic).
// Block = 32 columns x 8 chunk lanes: the chunk loop is 8 times shorter than one thread per column
// and the partial rows are read 128 contiguous bytes at a time.
__global__ void colreduce_stage2_k(const float* __restrict__ pr, const float* __restrict__ pi,
                                   float* __restrict__ dr, float* __restrict__ di, int accumulate,
                                   int chunks, int N) {
    cnb_pdl_enter();
    __shared__ float sr[8][33], si[8][33];
    int col = blockIdx.x * 32 + threadIdx.x;
    float a = 0.f, b = 0.f;
    if (col < N)
        for (int c = threadIdx.y; c < chunks; c += 8) { a += pr[(size_t) c * N + col]; b += pi[(size_t) c * N + col]; }
    sr[threadIdx.y][threadIdx.x] = a;
    si[threadIdx.y][threadIdx.x] = b;
    __syncthreads();
    if (threadIdx.y == 0 && col < N) {
#pragma unroll
        for (int k = 1; k < 8; ++k) { a += sr[k][threadIdx.x]; b += si[k][threadIdx.x]; }
        if (accumulate) { a += dr[col]; b += di[col]; }
        dr[col] = a; di[col] = b;
    }
}

// --------------------------------------------------------------------- CGelu
template <int W>
__global__ void gelu_fwd_k(const float* __restrict__ zr, const float* __restrict__ zi,
                           float* __restrict__ yr, float* __restrict__ yi, size_t total) {
    cnb_pdl_enter();
    size_t stride = (size_t) gridDim.x * blockDim.x * W;
    for (size_t i = ((size_t) blockIdx.x * blockDim.x + threadIdx.x) * W; i < total; i += stride) {
        Pack<W> a = ld<W>(zr, i), b = ld<W>(zi, i);
#pragma unroll
        for (int k = 0; k < W; ++k) { a.v[k] = gelu_f(a.v[k]); b.v[k] = gelu_f(b.v[k]); }
        st<W>(yr, i, a); st<W>(yi, i, b);
    }
}

template <int W>
__global__ void gelu_bwd_k(const float* __restrict__ gr, const float* __restrict__ gi,
                           const float* __restrict__ zr, const float* __restrict__ zi,
                           float* __restrict__ dr, float* __restrict__ di, int accumulate, size_t total) {
    cnb_pdl_enter();
    size_t stride = (size_t) gridDim.x * blockDim.x * W;
    for (size_t i = ((size_t) blockIdx.x * blockDim.x + threadIdx.x) * W; i < total; i += stride) {
        Pack<W> a = ld<W>(gr, i), b = ld<W>(gi, i), x = ld<W>(zr, i), y = ld<W>(zi, i), r, s;
        if (accumulate) { r = ld<W>(dr, i); s = ld<W>(di, i); }
#pragma unroll
        for (int k = 0; k < W; ++k) {
            // conj(g) (dx-dy) + g (dx+dy), dx, dy = gelu'(x) / 2, gelu'(y) / 2: component-wise products
            float nr = a.v[k] * dgelu_f(x.v[k]);
            float ni = b.v[k] * dgelu_f(y.v[k]);
            r.v[k] = accumulate ? r.v[k] + nr : nr;
            s.v[k] = accumulate ? s.v[k] + ni : ni;
        }
        st<W>(dr, i, r); st<W>(di, i, s);
    }
}

// sp != NULL: also emit the operand split of y (a split buffer with plane pitch `np`) that the
// tensor-core GEMM of the consuming Linear reads, saving that layer's separate split pass.
template <int W>
__global__ void hadamard_gelu_fwd_k(const float* __restrict__ ur, const float* __restrict__ ui,
                                    const float* __restrict__ hr, const float* __restrict__ hi,
                                    float* __restrict__ ar, float* __restrict__ ai,
                                    float* __restrict__ yr, float* __restrict__ yi, size_t total, int N,
                                    float* __restrict__ sp, size_t np) {
    cnb_pdl_enter();
    size_t stride = (size_t) gridDim.x * blockDim.x * W;
    for (size_t i = ((size_t) blockIdx.x * blockDim.x + threadIdx.x) * W; i < total; i += stride) {
        size_t j = i % N;
        Pack<W> a = ld<W>(ur, i), b = ld<W>(ui, i), c = ld<W>(hr, j), d = ld<W>(hi, j), r, s;
#pragma unroll
        for (int k = 0; k < W; ++k) {
            r.v[k] = a.v[k] * c.v[k] - b.v[k] * d.v[k];
            s.v[k] = a.v[k] * d.v[k] + b.v[k] * c.v[k];
        }
        st<W>(ar, i, r); st<W>(ai, i, s);
#pragma unroll
        for (int k = 0; k < W; ++k) { r.v[k] = gelu_f(r.v[k]); s.v[k] = gelu_f(s.v[k]); }
        st<W>(yr, i, r); st<W>(yi, i, s);
        if (sp) {
            const cnb_split_dst d0 = cnb_split_component(sp, np, 0), d1 = cnb_split_component(sp, np, 1);
            if constexpr (W == 4) {
                cnb_split_store4(d0, i, r.v[0], r.v[1], r.v[2], r.v[3]);
                cnb_split_store4(d1, i, s.v[0], s.v[1], s.v[2], s.v[3]);
            } else {
#pragma unroll
                for (int k = 0; k < W; ++k) { cnb_split_store1(d0, i + k, r.v[k]); cnb_split_store1(d1, i + k, s.v[k]); }
            }
        }
    }
}

// --------------------------------------------------------------------- CRelu
// y = z where re > 0 and im > 0, else 0; the backward passes g* through the same gate.
template <int W>
__global__ void crelu_k(const float* __restrict__ zr, const float* __restrict__ zi,
                        const float* __restrict__ sr, const float* __restrict__ si,
                        float* __restrict__ dr, float* __restrict__ di, int accumulate, size_t total) {
    cnb_pdl_enter();
    size_t stride = (size_t) gridDim.x * blockDim.x * W;
    for (size_t i = ((size_t) blockIdx.x * blockDim.x + threadIdx.x) * W; i < total; i += stride) {
        Pack<W> a = ld<W>(zr, i), b = ld<W>(zi, i), x = ld<W>(sr, i), y = ld<W>(si, i), r, s;
        if (accumulate) { r = ld<W>(dr, i); s = ld<W>(di, i); }
#pragma unroll
        for (int k = 0; k < W; ++k) {
            bool on = a.v[k] > 0.f && b.v[k] > 0.f;
            float vr = on ? x.v[k] : 0.f, vi = on ? y.v[k] : 0.f;
            r.v[k] = accumulate ? r.v[k] + vr : vr;
            s.v[k] = accumulate ? s.v[k] + vi : vi;
        }
        st<W>(dr, i, r); st<W>(di, i, s);
    }
}

// momentum-only "Adam" of the reference: m = beta m + (1-beta) g; w -= lr m / (1 - beta^(t+1)); g = 0
template <int W>
__global__ void adam_k(float* __restrict__ w, float* __restrict__ m, float* __restrict__ g, size_t total, float lr_hat,
                       float beta) {
    cnb_pdl_enter();
    size_t stride = (size_t) gridDim.x * blockDim.x * W;
    for (size_t i = ((size_t) blockIdx.x * blockDim.x + threadIdx.x) * W; i < total; i += stride) {
        Pack<W> a = ld<W>(w, i), b = ld<W>(m, i), c = ld<W>(g, i);
#pragma unroll
        for (int k = 0; k < W; ++k) {
            b.v[k] = b.v[k] * beta + (1.f - beta) * c.v[k];
            a.v[k] -= lr_hat * b.v[k];
            c.v[k] = 0.f;
        }
        st<W>(w, i, a); st<W>(m, i, b); st<W>(g, i, c);
    }
}

// ------------------------------------------------- Residual, pass-through, SGD
template <int W>
__global__ void add2_k(const float* __restrict__ ur, const float* __restrict__ ui,
                       const float* __restrict__ vr, const float* __restrict__ vi,
                       float* __restrict__ yr, float* __restrict__ yi, size_t total) {
    cnb_pdl_enter();
    size_t stride = (size_t) gridDim.x * blockDim.x * W;
    for (size_t i = ((size_t) blockIdx.x * blockDim.x + threadIdx.x) * W; i < total; i += stride) {
        Pack<W> a = ld<W>(ur, i), b = ld<W>(ui, i), c = ld<W>(vr, i), d = ld<W>(vi, i);
#pragma unroll
        for (int k = 0; k < W; ++k) { a.v[k] += c.v[k]; b.v[k] += d.v[k]; }
        st<W>(yr, i, a); st<W>(yi, i, b);
    }
}

template <int W>
__global__ void sgd_k(float* __restrict__ w, float* __restrict__ g, size_t total, float lr, int zero_grad) {
    cnb_pdl_enter();
    size_t stride = (size_t) gridDim.x * blockDim.x * W;
    for (size_t i = ((size_t) blockIdx.x * blockDim.x + threadIdx.x) * W; i < total; i += stride) {
        Pack<W> a = ld<W>(w, i), b = ld<W>(g, i);
#pragma unroll
        for (int k = 0; k < W; ++k) { a.v[k] -= lr * b.v[k]; b.v[k] = 0.f; }
        st<W>(w, i, a);
        if (zero_grad) st<W>(g, i, b);
    }
}

// The update with the operand split of the new values written in the same pass for the spans of the
// arena that are Linear weights (span begins and lengths are multiples of 4 floats).
struct SplitSpans {
    size_t begin[CNB_MAX_SPLIT_SPANS];
    size_t count[CNB_MAX_SPLIT_SPANS];
    cnb_split_dst dst[CNB_MAX_SPLIT_SPANS];
    int n;
};

__global__ void sgd_split_k(float* __restrict__ w, float* __restrict__ g, size_t total, float lr, int zero_grad,
                            const SplitSpans sp) {
    cnb_pdl_enter();
    size_t stride = (size_t) gridDim.x * blockDim.x * 4;
    for (size_t i = ((size_t) blockIdx.x * blockDim.x + threadIdx.x) * 4; i < total; i += stride) {
        Pack<4> a = ld<4>(w, i), b = ld<4>(g, i);
#pragma unroll
        for (int k = 0; k < 4; ++k) { a.v[k] -= lr * b.v[k]; b.v[k] = 0.f; }
        st<4>(w, i, a);
        if (zero_grad) st<4>(g, i, b);
        for (int s = 0; s < sp.n; ++s) {
            if (i >= sp.begin[s] && i < sp.begin[s] + sp.count[s]) {
                cnb_split_store4(sp.dst[s], i - sp.begin[s], a.v[0], a.v[1], a.v[2], a.v[3]);
                break;
            }
        }
    }
}

template <typename... P> bool all_aligned(P... p) { return (aligned16(p) && ...); }

int colreduce_launch(cnb_ctx* ctx, int mode, const float* gr, const float* gi, const float* ar, const float* ai,
                     const float* ur, const float* ui, const float* hr, const float* hi,
                     float* dur, float* dui, int acc_u, float* dvr, float* dvi, int acc_v,
                     int B, int N, cudaStream_t stm) {
    bool vec = (N % 4 == 0) && aligned16(gr) && aligned16(gi) && aligned16(ur) && aligned16(ui) &&
               (mode == 0 || (aligned16(ar) && aligned16(ai) && aligned16(hr) && aligned16(hi))) &&   // NULL is aligned
               (!dur || (aligned16(dur) && aligned16(dui)));
    int w = vec ? 4 : 1;
    int col_blocks = (N + 32 * w - 1) / (32 * w);
    // one full wave: as many row chunks as the resident CTAs of the whole device allow
    static int occ[4] = {0, 0, 0, 0};
    int& per_sm = occ[(mode ? 2 : 0) + (vec ? 1 : 0)];
    if (!per_sm) {
        cudaError_t e = mode ? (vec ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, colreduce_stage1_k<1, 4>, 256, 0)
                                    : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, colreduce_stage1_k<1, 1>, 256, 0))
                             : (vec ? cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, colreduce_stage1_k<0, 4>, 256, 0)
                                    : cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, colreduce_stage1_k<0, 1>, 256, 0));
        if (e != cudaSuccess || per_sm < 1) per_sm = 4;
    }
    int chunks = std::max(1, cnb::usable_sms(ctx) * per_sm / col_blocks);
    int max_chunks = (B + 7) / 8;
    if (chunks > max_chunks) chunks = max_chunks;
    if (chunks > 128) chunks = 128;
    if (chunks < 1) chunks = 1;
    int rows = (B + chunks - 1) / chunks;
    chunks = (B + rows - 1) / rows;
    float* part = nullptr;
    int rc = cnb::ensure_scratch(ctx, (size_t) chunks * N * 2 * sizeof(float), &part);
    if (rc != CNB_OK) return rc;
    float* pr = part;
    float* pi = part + (size_t) chunks * N;
    dim3 grid(col_blocks, chunks), block(32, 8);
    // up to 64 column blocks: the last CTA of each column block finishes the sum in the same launch
    int* done = (col_blocks <= 64 && ctx->d_counters) ? ctx->d_counters + 64 * (ctx->counter_set++ & 7) : nullptr;
#define CNB_COLREDUCE(MODE, W) cnb::launch(colreduce_stage1_k<MODE, W>, grid, block, 0, stm, 1, gr, gi, ar, ai, ur, ui, hr, hi, dur, dui, acc_u, pr, pi, B, N, rows, done, dvr, dvi, acc_v)
    if (mode == 0) { if (vec) CNB_COLREDUCE(0, 4); else CNB_COLREDUCE(0, 1); }
    else { if (vec) CNB_COLREDUCE(1, 4); else CNB_COLREDUCE(1, 1); }
#undef CNB_COLREDUCE
    CNB_LAUNCH_CHECK("colreduce_stage1");
    if (!done) {
        cnb::launch(colreduce_stage2_k, dim3((N + 31) / 32), dim3(32, 8), 0, stm, 1, pr, pi, dvr, dvi, acc_v, chunks, N);
        CNB_LAUNCH_CHECK("colreduce_stage2");
    }
    return CNB_OK;
}

}  // namespace


#define DISPATCH_W(vec_ok, KERNEL, total, ...)                                              \
    do {                                                                                    \
        if (vec_ok) {                                                                       \
            cnb::launch(KERNEL<4>, dim3(grid_for(((total) + 3) / 4, 256, ctx->sm_count)), dim3(256), 0, stm, 1, __VA_ARGS__); \
        } else {                                                                            \
            cnb::launch(KERNEL<1>, dim3(grid_for((total), 256, ctx->sm_count)), dim3(256), 0, stm, 1, __VA_ARGS__); \
        }                                                                                   \
        CNB_LAUNCH_CHECK(#KERNEL);                                                          \
    } while (0)

extern "C" {

int cnb_hadamard_fwd(cnb_ctx* ctx, const float* u_re, const float* u_im, const float* v_re, const float* v_im,
                     int v_batched, float* y_re, float* y_im, int B, int N, void* stream) {
    CNB_CHECK_ARG(ctx && u_re && u_im && v_re && v_im && y_re && y_im, "cnb_hadamard_fwd: null pointer");
    CNB_CHECK_ARG(B > 0 && N > 0, "cnb_hadamard_fwd: B=%d N=%d", B, N);
    cudaStream_t stm = cnb::S(stream);
    size_t total = (size_t) B * N;
    bool vec = (N % 4 == 0) && all_aligned(u_re, u_im, v_re, v_im, y_re, y_im);
    DISPATCH_W(vec, hadamard_fwd_k, total, u_re, u_im, v_re, v_im, v_batched, y_re, y_im, total, N);
    return CNB_OK;
}

int cnb_hadamard_bwd(cnb_ctx* ctx, const float* g_re, const float* g_im, const float* u_re, const float* u_im,
                     const float* v_re, const float* v_im, int v_batched, float* du_re, float* du_im,
                     int accumulate_u, float* dv_re, float* dv_im, int accumulate_v, int B, int N, void* stream) {
    CNB_CHECK_ARG(ctx && g_re && g_im && u_re && u_im && v_re && v_im, "cnb_hadamard_bwd: null pointer");
    CNB_CHECK_ARG(B > 0 && N > 0, "cnb_hadamard_bwd: B=%d N=%d", B, N);
    CNB_CHECK_ARG((du_re == nullptr) == (du_im == nullptr) && (dv_re == nullptr) == (dv_im == nullptr),
                  "cnb_hadamard_bwd: re/im output planes must be given in pairs");
    cudaStream_t stm = cnb::S(stream);
    size_t total = (size_t) B * N;
    if (du_re) {
        bool vec = (N % 4 == 0) && all_aligned(g_re, g_im, v_re, v_im, du_re, du_im);
        DISPATCH_W(vec, hadamard_bwd_elem_k, total, g_re, g_im, v_re, v_im, v_batched, du_re, du_im, accumulate_u,
                   total, N);
    }
    if (dv_re) {
        if (v_batched) {
            bool vec = (N % 4 == 0) && all_aligned(g_re, g_im, u_re, u_im, dv_re, dv_im);
            DISPATCH_W(vec, hadamard_bwd_elem_k, total, g_re, g_im, u_re, u_im, 1, dv_re, dv_im, accumulate_v,
                       total, N);
        } else {
            return colreduce_launch(ctx, 0, g_re, g_im, nullptr, nullptr, u_re, u_im, nullptr, nullptr, nullptr,
                                    nullptr, 0, dv_re, dv_im, accumulate_v, B, N, stm);
        }
    }
    return CNB_OK;
}

int cnb_gelu_fwd(cnb_ctx* ctx, const float* z_re, const float* z_im, float* y_re, float* y_im, size_t n,
                 void* stream) {
    CNB_CHECK_ARG(ctx && z_re && z_im && y_re && y_im && n > 0, "cnb_gelu_fwd: bad argument");
    cudaStream_t stm = cnb::S(stream);
    bool vec = (n % 4 == 0) && all_aligned(z_re, z_im, y_re, y_im);
    DISPATCH_W(vec, gelu_fwd_k, n, z_re, z_im, y_re, y_im, n);
    return CNB_OK;
}

int cnb_gelu_bwd(cnb_ctx* ctx, const float* g_re, const float* g_im, const float* z_re, const float* z_im,
                 float* dz_re, float* dz_im, size_t n, int accumulate, void* stream) {
    CNB_CHECK_ARG(ctx && g_re && g_im && z_re && z_im && dz_re && dz_im && n > 0, "cnb_gelu_bwd: bad argument");
    cudaStream_t stm = cnb::S(stream);
    bool vec = (n % 4 == 0) && all_aligned(g_re, g_im, z_re, z_im, dz_re, dz_im);
    DISPATCH_W(vec, gelu_bwd_k, n, g_re, g_im, z_re, z_im, dz_re, dz_im, accumulate, n);
    return CNB_OK;
}

int cnb_hadamard_gelu_fwd_split(cnb_ctx* ctx, const float* u_re, const float* u_im, const float* h_re,
                                const float* h_im, float* a_re, float* a_im, float* y_re, float* y_im,
                                float* y_split, int B, int N, void* stream) {
    CNB_CHECK_ARG(ctx && u_re && u_im && h_re && h_im && a_re && a_im && y_re && y_im,
                  "cnb_hadamard_gelu_fwd: null pointer");
    CNB_CHECK_ARG(B > 0 && N > 0, "cnb_hadamard_gelu_fwd: B=%d N=%d", B, N);
    cudaStream_t stm = cnb::S(stream);
    size_t total = (size_t) B * N;
    size_t np = (total + 63) & ~size_t(63);
    bool vec = (N % 4 == 0) && all_aligned(u_re, u_im, h_re, h_im, a_re, a_im, y_re, y_im, y_split);
    DISPATCH_W(vec, hadamard_gelu_fwd_k, total, u_re, u_im, h_re, h_im, a_re, a_im, y_re, y_im, total, N, y_split, np);
    return CNB_OK;
}

int cnb_hadamard_gelu_fwd(cnb_ctx* ctx, const float* u_re, const float* u_im, const float* h_re,
                          const float* h_im, float* a_re, float* a_im, float* y_re, float* y_im, int B, int N,
                          void* stream) {
    return cnb_hadamard_gelu_fwd_split(ctx, u_re, u_im, h_re, h_im, a_re, a_im, y_re, y_im, nullptr, B, N, stream);
}

int cnb_hadamard_gelu_bwd(cnb_ctx* ctx, const float* g_re, const float* g_im, const float* a_re,
                          const float* a_im, const float* u_re, const float* u_im, const float* h_re,
                          const float* h_im, float* du_re, float* du_im, int accumulate_u, float* dh_re,
                          float* dh_im, int accumulate_h, int B, int N, void* stream) {
    CNB_CHECK_ARG(ctx && g_re && g_im && u_re && u_im && h_re && h_im && dh_re && dh_im,
                  "cnb_hadamard_gelu_bwd: null pointer");
    CNB_CHECK_ARG((a_re == nullptr) == (a_im == nullptr), "cnb_hadamard_gelu_bwd: a planes must be a pair");
    CNB_CHECK_ARG((du_re == nullptr) == (du_im == nullptr), "cnb_hadamard_gelu_bwd: du planes must be a pair");
    CNB_CHECK_ARG(B > 0 && N > 0, "cnb_hadamard_gelu_bwd: B=%d N=%d", B, N);
    return colreduce_launch(ctx, 1, g_re, g_im, a_re, a_im, u_re, u_im, h_re, h_im, du_re, du_im, accumulate_u,
                            dh_re, dh_im, accumulate_h, B, N, cnb::S(stream));
}

int cnb_residual_fwd(cnb_ctx* ctx, const float* u_re, const float* u_im, const float* v_re, const float* v_im,
                     float* y_re, float* y_im, size_t n, void* stream) {
    CNB_CHECK_ARG(ctx && u_re && u_im && v_re && v_im && y_re && y_im && n > 0, "cnb_residual_fwd: bad argument");
    cudaStream_t stm = cnb::S(stream);
    bool vec = (n % 4 == 0) && all_aligned(u_re, u_im, v_re, v_im, y_re, y_im);
    DISPATCH_W(vec, add2_k, n, u_re, u_im, v_re, v_im, y_re, y_im, n);
    return CNB_OK;
}

int cnb_axpy(cnb_ctx* ctx, const float* src_re, const float* src_im, float* dst_re, float* dst_im, size_t n,
             int accumulate, void* stream) {
    CNB_CHECK_ARG(ctx && src_re && src_im && dst_re && dst_im && n > 0, "cnb_axpy: bad argument");
    cudaStream_t stm = cnb::S(stream);
    if (!accumulate) {
        CNB_CUDA(cudaMemcpyAsync(dst_re, src_re, n * sizeof(float), cudaMemcpyDeviceToDevice, stm));
        CNB_CUDA(cudaMemcpyAsync(dst_im, src_im, n * sizeof(float), cudaMemcpyDeviceToDevice, stm));
        return CNB_OK;
    }
    bool vec = (n % 4 == 0) && all_aligned(src_re, src_im, dst_re, dst_im);
    DISPATCH_W(vec, add2_k, n, src_re, src_im, dst_re, dst_im, dst_re, dst_im, n);
    return CNB_OK;
}

int cnb_crelu_fwd(cnb_ctx* ctx, const float* z_re, const float* z_im, float* y_re, float* y_im, size_t n,
                  void* stream) {
    CNB_CHECK_ARG(ctx && z_re && z_im && y_re && y_im && n > 0, "cnb_crelu_fwd: bad argument");
    cudaStream_t stm = cnb::S(stream);
    bool vec = (n % 4 == 0) && all_aligned(z_re, z_im, y_re, y_im);
    DISPATCH_W(vec, crelu_k, n, z_re, z_im, z_re, z_im, y_re, y_im, 0, n);
    return CNB_OK;
}

int cnb_crelu_bwd(cnb_ctx* ctx, const float* g_re, const float* g_im, const float* z_re, const float* z_im,
                  float* dz_re, float* dz_im, size_t n, int accumulate, void* stream) {
    CNB_CHECK_ARG(ctx && g_re && g_im && z_re && z_im && dz_re && dz_im && n > 0, "cnb_crelu_bwd: bad argument");
    cudaStream_t stm = cnb::S(stream);
    bool vec = (n % 4 == 0) && all_aligned(g_re, g_im, z_re, z_im, dz_re, dz_im);
    DISPATCH_W(vec, crelu_k, n, z_re, z_im, g_re, g_im, dz_re, dz_im, accumulate, n);
    return CNB_OK;
}

int cnb_adam_update(cnb_ctx* ctx, float* w, float* m, float* g, size_t n, float lr, float beta, int t,
                    void* stream) {
    CNB_CHECK_ARG(ctx && w && m && g && n > 0 && t >= 0, "cnb_adam_update: bad argument");
    CNB_CHECK_ARG(beta >= 0.f && beta < 1.f, "cnb_adam_update: beta=%f", beta);
    cudaStream_t stm = cnb::S(stream);
    float lr_hat = (float) ((double) lr / (1.0 - pow((double) beta, t + 1)));
    bool vec = (n % 4 == 0) && all_aligned(w, m, g);
    DISPATCH_W(vec, adam_k, n, w, m, g, n, lr_hat, beta);
    return CNB_OK;
}

int cnb_sgd_update(cnb_ctx* ctx, float* w, float* g, size_t n, float lr, int zero_grad, void* stream) {
    CNB_CHECK_ARG(ctx && w && g && n > 0, "cnb_sgd_update: bad argument");
    cudaStream_t stm = cnb::S(stream);
    bool vec = (n % 4 == 0) && all_aligned(w, g);
    DISPATCH_W(vec, sgd_k, n, w, g, n, lr, zero_grad);
    return CNB_OK;
}

int cnb_sgd_update_split(cnb_ctx* ctx, float* w, float* g, size_t n, float lr, int zero_grad,
                         const cnb_split_span* spans, int nspans, void* stream) {
    CNB_CHECK_ARG(ctx && w && g && n > 0 && n % 4 == 0 && all_aligned(w, g), "cnb_sgd_update_split: bad argument");
    CNB_CHECK_ARG(nspans >= 0 && nspans <= CNB_MAX_SPLIT_SPANS && (nspans == 0 || spans),
                  "cnb_sgd_update_split: %d spans (at most %d)", nspans, CNB_MAX_SPLIT_SPANS);
    SplitSpans sp;
    sp.n = nspans;
    for (int k = 0; k < nspans; ++k) {
        CNB_CHECK_ARG(spans[k].begin % 4 == 0 && spans[k].count % 4 == 0 && spans[k].begin + spans[k].count <= n &&
                      all_aligned(spans[k].hi, spans[k].h16, spans[k].l16) && spans[k].hi && spans[k].h16 && spans[k].l16,
                      "cnb_sgd_update_split: span %d is not a 16-byte aligned range of the arena", k);
        sp.begin[k] = spans[k].begin; sp.count[k] = spans[k].count;
        sp.dst[k].hi = spans[k].hi;
        sp.dst[k].h16 = static_cast<unsigned short*>(spans[k].h16);
        sp.dst[k].l16 = static_cast<unsigned short*>(spans[k].l16);
    }
    cudaStream_t stm = cnb::S(stream);
    size_t blocks = (n / 4 + 255) / 256, cap = (size_t) ctx->sm_count * 16;
    cnb::launch(sgd_split_k, dim3((unsigned) std::min(blocks, cap)), dim3(256), 0, stm, 1, w, g, n, lr, zero_grad, sp);
    CNB_LAUNCH_CHECK("sgd_split");
    return CNB_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------
// Hadamard backward without any allocation.
//
// Some hosts of this library are not allowed to allocate device memory at the point where
// they call it: a runtime that has already handed every byte of the device to its own pool
// and must not let a foreign cudaMalloc fail or fragment it, or a latency-critical loop that
// cannot afford the device-wide synchronisation cudaMalloc / cudaFree imply.  For those, this
// one entry point keeps the column-reduction partials in a fixed array that is part of the
// loaded module instead of in an arena: 2 MiB per GPU that loads the library, held until the
// process exits.  Limits: N <= CNB_STATIC_MAX_N, shared (non-batched) v only.
//
// In host code `g_static_partials` is only a handle for the symbol, not a device address, so
// its address is looked up with cudaGetSymbolAddress once per device (with that device
// current) and that pointer is what the kernels receive.
namespace {

constexpr int kStaticMaxN = 4096;
constexpr int kStaticMaxChunks = 64;
static __device__ __align__(256) float g_static_partials[2 * kStaticMaxChunks * kStaticMaxN];

struct StaticScratch {
    float* ptr = nullptr;
    int sm_count = 0;
};

int static_scratch_for_current_device(StaticScratch* out) {
    static StaticScratch per_device[64];
    static std::mutex mu;
    int dev = 0;
    CNB_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return cnb::set_error(CNB_ERR_ARG, "device ordinal %d out of range", dev);
    std::lock_guard<std::mutex> lock(mu);
    if (!per_device[dev].ptr) {
        float* p = nullptr;
        CNB_CUDA(cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_static_partials));
        int sms = 0;
        CNB_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        per_device[dev].sm_count = sms;
        per_device[dev].ptr = p;
    }
    *out = per_device[dev];
    return CNB_OK;
}

}  // namespace

extern "C" int cnb_hadamard_bwd_static(const float* g_re, const float* g_im, const float* u_re, const float* u_im,
                                       const float* v_re, const float* v_im, float* du_re, float* du_im,
                                       int accumulate_u, float* dv_re, float* dv_im, int accumulate_v, int B, int N,
                                       void* stream) {
    CNB_CHECK_ARG(g_re && g_im && u_re && u_im && v_re && v_im && dv_re && dv_im,
                  "cnb_hadamard_bwd_static: null pointer");
    CNB_CHECK_ARG((du_re == nullptr) == (du_im == nullptr), "cnb_hadamard_bwd_static: du planes must be a pair");
    CNB_CHECK_ARG(B > 0 && N > 0, "cnb_hadamard_bwd_static: B=%d N=%d", B, N);
    CNB_CHECK_ARG(N <= kStaticMaxN, "cnb_hadamard_bwd_static: N=%d exceeds the built-in scratch (N <= %d); "
                  "use cnb_hadamard_bwd with an arena", N, kStaticMaxN);
    StaticScratch sc;
    int rc = static_scratch_for_current_device(&sc);
    if (rc != CNB_OK) return rc;
    {   // the scratch belongs to the current device: kernels launched here must not be handed another GPU's planes
        int dev = -1;
        CNB_CUDA(cudaGetDevice(&dev));
        const void* probe[2] = {g_re, dv_re};
        for (const void* q : probe) {
            cudaPointerAttributes at;
            CNB_CUDA(cudaPointerGetAttributes(&at, q));
            CNB_CHECK_ARG((at.type == cudaMemoryTypeDevice || at.type == cudaMemoryTypeManaged) && at.device == dev,
                          "cnb_hadamard_bwd_static: the planes are not memory of the current device %d", dev);
        }
    }
    cudaStream_t stm = cnb::S(stream);
    size_t total = (size_t) B * N;
    if (du_re) {
        bool vec = (N % 4 == 0) && all_aligned(g_re, g_im, v_re, v_im, du_re, du_im);
        if (vec)
            hadamard_bwd_elem_k<4><<<grid_for((total + 3) / 4, 256, sc.sm_count), 256, 0, stm>>>(
                g_re, g_im, v_re, v_im, 0, du_re, du_im, accumulate_u, total, N);
        else
            hadamard_bwd_elem_k<1><<<grid_for(total, 256, sc.sm_count), 256, 0, stm>>>(
                g_re, g_im, v_re, v_im, 0, du_re, du_im, accumulate_u, total, N);
        CNB_LAUNCH_CHECK("hadamard_bwd_elem");
    }
    // 16-byte form (4 columns per thread) where the planes allow it, as the arena-backed entry does
    const bool vec = (N % 4 == 0) && all_aligned(g_re, g_im, u_re, u_im);
    const int w = vec ? 4 : 1;
    int col_blocks = (N + 32 * w - 1) / (32 * w);
    int chunks = (sc.sm_count * 4 + col_blocks - 1) / col_blocks;
    chunks = std::min(chunks, std::min((B + 7) / 8, kStaticMaxChunks));
    chunks = std::max(chunks, 1);
    int rows = (B + chunks - 1) / chunks;
    chunks = (B + rows - 1) / rows;
    // every partial that stage 2 reads is written by stage 1 of this call: nothing has to start at zero
    float* pr = sc.ptr;
    float* pi = sc.ptr + (size_t) kStaticMaxChunks * kStaticMaxN;
    dim3 grid(col_blocks, chunks), block(32, 8);
    if (vec)
        colreduce_stage1_k<0, 4><<<grid, block, 0, stm>>>(g_re, g_im, nullptr, nullptr, u_re, u_im, nullptr, nullptr,
                                                          nullptr, nullptr, 0, pr, pi, B, N, rows, nullptr, nullptr, nullptr, 0);
    else
        colreduce_stage1_k<0, 1><<<grid, block, 0, stm>>>(g_re, g_im, nullptr, nullptr, u_re, u_im, nullptr, nullptr,
                                                          nullptr, nullptr, 0, pr, pi, B, N, rows, nullptr, nullptr, nullptr, 0);
    CNB_LAUNCH_CHECK("colreduce_stage1");
    colreduce_stage2_k<<<(N + 31) / 32, dim3(32, 8), 0, stm>>>(pr, pi, dv_re, dv_im, accumulate_v, chunks, N);
    CNB_LAUNCH_CHECK("colreduce_stage2");
    return CNB_OK;
}
