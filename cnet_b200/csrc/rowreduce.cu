// Row reductions of the complex training step: L2 normalisation (the reference's
// "SoftMax") forward/backward and the fused CrossEntropy forward + backward seed.
// One CTA per sample row; warp-shuffle tree + one shared-memory hop.  Rows are read once
// for the reduction and once (from L2/L1) for the element-wise pass.
#include <initializer_list>

#include "common.cuh"

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Sum over the CTA; result valid in every thread.  blockDim.x is a multiple of 32, <= 1024.
__device__ __forceinline__ float block_sum(float v, float* smem) {
    v = warp_sum(v);
    int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    __syncthreads();
    if (lane == 0) smem[warp] = v;
    __syncthreads();
    float r = (lane < nw) ? smem[lane] : 0.f;
    r = warp_sum(r);
    return r;
}

__global__ void softmax_fwd_k(const float* __restrict__ zr, const float* __restrict__ zi,
                              float* __restrict__ yr, float* __restrict__ yi, float* __restrict__ inv_norm, int N) {
    cnb_pdl_enter();
    __shared__ float sm[32];
    size_t base = (size_t) blockIdx.x * N;
    float s = 0.f;
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
        float a = zr[base + i], b = zi[base + i];
        s += a * a + b * b;
    }
    s = block_sum(s, sm);
    float n = fmaxf(sqrtf(s), 1e-15f);
    float inv = 1.0f / n;
    if (threadIdx.x == 0) inv_norm[blockIdx.x] = inv;
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
        yr[base + i] = zr[base + i] * inv;
        yi[base + i] = zi[base + i] * inv;
    }
}

__global__ void softmax_bwd_k(const float* __restrict__ gr, const float* __restrict__ gi,
                              const float* __restrict__ zr, const float* __restrict__ zi,
                              const float* __restrict__ inv_norm, float* __restrict__ dr, float* __restrict__ di,
                              int N, int accumulate) {
    cnb_pdl_enter();
    __shared__ float sm[32];
    size_t base = (size_t) blockIdx.x * N;
    float s = 0.f;
    for (int i = threadIdx.x; i < N; i += blockDim.x)   // Re(g* conj(z))
        s += gr[base + i] * zr[base + i] + gi[base + i] * zi[base + i];
    s = block_sum(s, sm);
    float inv = inv_norm[blockIdx.x];
    float c = s * inv * inv * inv;
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
        float a = gr[base + i] * inv - zr[base + i] * c;
        float b = gi[base + i] * inv - zi[base + i] * c;
        if (accumulate) { a += dr[base + i]; b += di[base + i]; }
        dr[base + i] = a; di[base + i] = b;
    }
}

__global__ void crossent_k(const float* __restrict__ zr, const float* __restrict__ zi,
                           const int32_t* __restrict__ labels, float* __restrict__ loss,
                           float* __restrict__ dr, float* __restrict__ di, int M) {
    cnb_pdl_enter();
    __shared__ float sm[32];
    size_t base = (size_t) blockIdx.x * M;
    float s = 0.f;
    for (int i = threadIdx.x; i < M; i += blockDim.x) {
        float a = zr[base + i], b = zi[base + i];
        s += a * a + b * b;
    }
    s = block_sum(s, sm);
    float S = fmaxf(s, 1e-15f);
    int l = labels[blockIdx.x];
    l = min(max(l, 0), M - 1);
    float lr = zr[base + l], li = zi[base + l];
    float m2 = lr * lr + li * li;
    if (threadIdx.x == 0) loss[blockIdx.x] = -logf(fmaxf(m2 / S, 1e-15f));
    if (dr == nullptr) return;
    float m = fmaxf(m2, 1e-15f);
    float cl = -(S - m) / (m * S), co = 1.0f / S;
    for (int i = threadIdx.x; i < M; i += blockDim.x) {
        float c = (i == l) ? cl : co;
        dr[base + i] = zr[base + i] * c;
        di[base + i] = zi[base + i] * c;
    }
}

// L2Out: loss[b] = sum |z|^2; seed dz* = z
__global__ void l2out_k(const float* __restrict__ zr, const float* __restrict__ zi, float* __restrict__ loss,
                        float* __restrict__ dr, float* __restrict__ di, int N) {
    cnb_pdl_enter();
    __shared__ float sm[32];
    size_t base = (size_t) blockIdx.x * N;
    float s = 0.f;
    for (int i = threadIdx.x; i < N; i += blockDim.x) {
        float a = zr[base + i], b = zi[base + i];
        s += a * a + b * b;
        if (dr) { dr[base + i] = a; di[base + i] = b; }
    }
    s = block_sum(s, sm);
    if (threadIdx.x == 0) loss[blockIdx.x] = s;
}

// Register-cached forms for rows of up to 16-byte-aligned 4 * CACHE * blockDim floats: the row is read ONCE
// with 16-byte loads, kept in registers across the reduction, and the element-wise pass works from the
// registers (the two-pass kernels above read the row a second time; at 8192 columns that second read is
// what kept them at ~0.55 of the copy bandwidth).
constexpr int CACHE = 4;         // float4 per plane and thread

__device__ __forceinline__ float4 ld4(const float* p, size_t i) { return *reinterpret_cast<const float4*>(p + i); }
__device__ __forceinline__ void st4(float* p, size_t i, float4 v) { *reinterpret_cast<float4*>(p + i) = v; }
__device__ __forceinline__ float4 scale4(float4 a, float s) { return make_float4(a.x * s, a.y * s, a.z * s, a.w * s); }
__device__ __forceinline__ float dot4(float4 a, float4 b) { return a.x * b.x + a.y * b.y + a.z * b.z + a.w * b.w; }

__global__ void __launch_bounds__(512) softmax_fwd_cached_k(const float* __restrict__ zr, const float* __restrict__ zi,
                                                            float* __restrict__ yr, float* __restrict__ yi,
                                                            float* __restrict__ inv_norm, int N) {
    cnb_pdl_enter();
    __shared__ float sm[32];
    const size_t base = (size_t) blockIdx.x * N;
    float4 a[CACHE], b[CACHE];
    float s = 0.f;
#pragma unroll
    for (int v = 0; v < CACHE; ++v) {
        const int i = 4 * (threadIdx.x + v * blockDim.x);
        if (i < N) { a[v] = ld4(zr, base + i); b[v] = ld4(zi, base + i); s += dot4(a[v], a[v]) + dot4(b[v], b[v]); }
    }
    s = block_sum(s, sm);
    const float inv = 1.0f / fmaxf(sqrtf(s), 1e-15f);
    if (threadIdx.x == 0) inv_norm[blockIdx.x] = inv;
#pragma unroll
    for (int v = 0; v < CACHE; ++v) {
        const int i = 4 * (threadIdx.x + v * blockDim.x);
        if (i < N) { st4(yr, base + i, scale4(a[v], inv)); st4(yi, base + i, scale4(b[v], inv)); }
    }
}

__global__ void __launch_bounds__(512) softmax_bwd_cached_k(const float* __restrict__ gr, const float* __restrict__ gi,
                                                            const float* __restrict__ zr, const float* __restrict__ zi,
                                                            const float* __restrict__ inv_norm, float* __restrict__ dr,
                                                            float* __restrict__ di, int N, int accumulate) {
    cnb_pdl_enter();
    __shared__ float sm[32];
    const size_t base = (size_t) blockIdx.x * N;
    float4 a[CACHE], b[CACHE], x[CACHE], y[CACHE];
    float s = 0.f;
#pragma unroll
    for (int v = 0; v < CACHE; ++v) {
        const int i = 4 * (threadIdx.x + v * blockDim.x);
        if (i < N) {
            a[v] = ld4(gr, base + i); b[v] = ld4(gi, base + i); x[v] = ld4(zr, base + i); y[v] = ld4(zi, base + i);
            s += dot4(a[v], x[v]) + dot4(b[v], y[v]);            // Re(g* conj(z))
        }
    }
    s = block_sum(s, sm);
    const float inv = inv_norm[blockIdx.x];
    const float c = s * inv * inv * inv;
#pragma unroll
    for (int v = 0; v < CACHE; ++v) {
        const int i = 4 * (threadIdx.x + v * blockDim.x);
        if (i < N) {
            float4 p = make_float4(a[v].x * inv - x[v].x * c, a[v].y * inv - x[v].y * c, a[v].z * inv - x[v].z * c, a[v].w * inv - x[v].w * c);
            float4 q = make_float4(b[v].x * inv - y[v].x * c, b[v].y * inv - y[v].y * c, b[v].z * inv - y[v].z * c, b[v].w * inv - y[v].w * c);
            if (accumulate) {
                const float4 o = ld4(dr, base + i), w = ld4(di, base + i);
                p.x += o.x; p.y += o.y; p.z += o.z; p.w += o.w;
                q.x += w.x; q.y += w.y; q.z += w.z; q.w += w.w;
            }
            st4(dr, base + i, p); st4(di, base + i, q);
        }
    }
}

__global__ void __launch_bounds__(512) crossent_cached_k(const float* __restrict__ zr, const float* __restrict__ zi,
                                                         const int32_t* __restrict__ labels, float* __restrict__ loss,
                                                         float* __restrict__ dr, float* __restrict__ di, int M) {
    cnb_pdl_enter();
    __shared__ float sm[32];
    const size_t base = (size_t) blockIdx.x * M;
    float4 a[CACHE], b[CACHE];
    float s = 0.f;
#pragma unroll
    for (int v = 0; v < CACHE; ++v) {
        const int i = 4 * (threadIdx.x + v * blockDim.x);
        if (i < M) { a[v] = ld4(zr, base + i); b[v] = ld4(zi, base + i); s += dot4(a[v], a[v]) + dot4(b[v], b[v]); }
    }
    // the label's element is handed over by the thread that holds it (a global load after the reduction would
    // put an L2 round trip on every row's critical path)
    __shared__ float s_lab[2];
    int l = labels[blockIdx.x];
    l = min(max(l, 0), M - 1);
#pragma unroll
    for (int v = 0; v < CACHE; ++v) {
        const int i = 4 * (threadIdx.x + v * blockDim.x);
        if (i < M && l >= i && l < i + 4) {
            const int k = l - i;
            s_lab[0] = k == 0 ? a[v].x : k == 1 ? a[v].y : k == 2 ? a[v].z : a[v].w;
            s_lab[1] = k == 0 ? b[v].x : k == 1 ? b[v].y : k == 2 ? b[v].z : b[v].w;
        }
    }
    s = block_sum(s, sm);                                 // its barriers also publish s_lab
    const float S = fmaxf(s, 1e-15f);
    const float lr = s_lab[0], li = s_lab[1];
    const float m2 = lr * lr + li * li;
    if (threadIdx.x == 0) loss[blockIdx.x] = -logf(fmaxf(m2 / S, 1e-15f));
    if (dr == nullptr) return;
    const float m = fmaxf(m2, 1e-15f);
    const float cl = -(S - m) / (m * S), co = 1.0f / S;
#pragma unroll
    for (int v = 0; v < CACHE; ++v) {
        const int i = 4 * (threadIdx.x + v * blockDim.x);
        if (i < M) {
            // the label's own coefficient (selects, not an indexed component: that would put the row in local memory)
            const float c0 = (i == l) ? cl : co, c1 = (i + 1 == l) ? cl : co, c2 = (i + 2 == l) ? cl : co, c3 = (i + 3 == l) ? cl : co;
            st4(dr, base + i, make_float4(a[v].x * c0, a[v].y * c1, a[v].z * c2, a[v].w * c3));
            st4(di, base + i, make_float4(b[v].x * c0, b[v].y * c1, b[v].z * c2, b[v].w * c3));
        }
    }
}

// rows the cached kernels take: 16-byte aligned planes, N % 4 == 0, and the row fits the CTA's registers
inline bool cached_ok(int n, int threads, std::initializer_list<const void*> planes) {
    if (n % 4 || n < 1024 || n / 4 > threads * CACHE) return false;
    for (const void* p : planes) if (p && (reinterpret_cast<uintptr_t>(p) & 15)) return false;
    return true;
}

inline int threads_for(int n) {
    int t = 32;
    while (t < n / 4 && t < 512) t <<= 1;
    return t;
}

}  // namespace

extern "C" {

int cnb_softmax_fwd(cnb_ctx* ctx, const float* z_re, const float* z_im, float* y_re, float* y_im,
                    float* inv_norm, int B, int N, void* stream) {
    CNB_CHECK_ARG(ctx && z_re && z_im && y_re && y_im && inv_norm, "cnb_softmax_fwd: null pointer");
    CNB_CHECK_ARG(B > 0 && N > 0, "cnb_softmax_fwd: B=%d N=%d", B, N);
    if (cached_ok(N, threads_for(N), {z_re, z_im, y_re, y_im}))
        cnb::launch(softmax_fwd_cached_k, dim3(B), dim3(threads_for(N)), 0, cnb::S(stream), 1, z_re, z_im, y_re, y_im, inv_norm, N);
    else
        cnb::launch(softmax_fwd_k, dim3(B), dim3(threads_for(N)), 0, cnb::S(stream), 1, z_re, z_im, y_re, y_im, inv_norm, N);
    CNB_LAUNCH_CHECK("softmax_fwd");
    return CNB_OK;
}

int cnb_softmax_bwd(cnb_ctx* ctx, const float* g_re, const float* g_im, const float* z_re, const float* z_im,
                    const float* inv_norm, float* dz_re, float* dz_im, int B, int N, int accumulate,
                    void* stream) {
    CNB_CHECK_ARG(ctx && g_re && g_im && z_re && z_im && inv_norm && dz_re && dz_im,
                  "cnb_softmax_bwd: null pointer");
    CNB_CHECK_ARG(B > 0 && N > 0, "cnb_softmax_bwd: B=%d N=%d", B, N);
    if (cached_ok(N, threads_for(N), {g_re, g_im, z_re, z_im, dz_re, dz_im}))
        cnb::launch(softmax_bwd_cached_k, dim3(B), dim3(threads_for(N)), 0, cnb::S(stream), 1, g_re, g_im, z_re, z_im, inv_norm, dz_re, dz_im, N, accumulate);
    else
        cnb::launch(softmax_bwd_k, dim3(B), dim3(threads_for(N)), 0, cnb::S(stream), 1, g_re, g_im, z_re, z_im, inv_norm, dz_re, dz_im, N, accumulate);
    CNB_LAUNCH_CHECK("softmax_bwd");
    return CNB_OK;
}

int cnb_crossent_fwd_bwd(cnb_ctx* ctx, const float* z_re, const float* z_im, const int32_t* labels, float* loss,
                         float* dz_re, float* dz_im, int B, int M, void* stream) {
    CNB_CHECK_ARG(ctx && z_re && z_im && labels && loss, "cnb_crossent_fwd_bwd: null pointer");
    CNB_CHECK_ARG((dz_re == nullptr) == (dz_im == nullptr), "cnb_crossent_fwd_bwd: dz planes must be a pair");
    CNB_CHECK_ARG(B > 0 && M > 0, "cnb_crossent_fwd_bwd: B=%d M=%d", B, M);
    if (cached_ok(M, threads_for(M), {z_re, z_im, dz_re, dz_im}))
        cnb::launch(crossent_cached_k, dim3(B), dim3(threads_for(M)), 0, cnb::S(stream), 1, z_re, z_im, labels, loss, dz_re, dz_im, M);
    else
        cnb::launch(crossent_k, dim3(B), dim3(threads_for(M)), 0, cnb::S(stream), 1, z_re, z_im, labels, loss, dz_re, dz_im, M);
    CNB_LAUNCH_CHECK("crossent");
    return CNB_OK;
}

int cnb_l2out_fwd_bwd(cnb_ctx* ctx, const float* z_re, const float* z_im, float* loss, float* dz_re, float* dz_im,
                      int B, int N, void* stream) {
    CNB_CHECK_ARG(ctx && z_re && z_im && loss, "cnb_l2out_fwd_bwd: null pointer");
    CNB_CHECK_ARG((dz_re == nullptr) == (dz_im == nullptr), "cnb_l2out_fwd_bwd: dz planes must be a pair");
    CNB_CHECK_ARG(B > 0 && N > 0, "cnb_l2out_fwd_bwd: B=%d N=%d", B, N);
    cnb::launch(l2out_k, dim3(B), dim3(threads_for(N)), 0, cnb::S(stream), 1, z_re, z_im, loss, dz_re, dz_im, N);
    CNB_LAUNCH_CHECK("l2out");
    return CNB_OK;
}

}  // extern "C"
