// Complex Linear (forward, dX*, dW*) and FourierTrans as a complex GEMM against a
// twiddle matrix: shape dispatch between the tcgen05 tiles (split operands) and the fp32 SIMT tiles.
#include <algorithm>
#include <cmath>
#include <vector>

#include "common.cuh"

namespace {

// F[p,q] = N^-1/2 e^{-2 pi i (pq mod N)/N}, angles reduced exactly in integers and evaluated
// in double with sincospi; the matrix is symmetric.
__global__ void twiddle_k(float* __restrict__ fr, float* __restrict__ fi, int N) {
    size_t total = (size_t) N * N;
    double scale = 1.0 / sqrt((double) N);
    for (size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t) gridDim.x * blockDim.x) {
        long p = (long) (i / N), q = (long) (i % N);
        long r = (p * q) % N;
        double s, c;
        sincospi(-2.0 * (double) r / (double) N, &s, &c);
        fr[i] = (float) (c * scale);
        fi[i] = (float) (s * scale);
    }
}

// TriangFourier: the same matrix with the entries above the diagonal (q > p) zeroed
__global__ void tri_mask_k(float* __restrict__ fr, float* __restrict__ fi, int N) {
    size_t total = (size_t) N * N;
    for (size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t) gridDim.x * blockDim.x)
        if ((int) (i % N) > (int) (i / N)) { fr[i] = 0.f; fi[i] = 0.f; }
}

const int kTriKey = 1 << 28;    // twiddle-cache key offset of the triangular matrices

int get_twiddle(cnb_ctx* ctx, int key, cudaStream_t st, cnb_twiddle* out) {
    const int N = key & (kTriKey - 1);
    auto it = ctx->twiddles.find(key);
    if (it != ctx->twiddles.end()) { *out = it->second; return CNB_OK; }
    cnb_twiddle t;
    void* p = nullptr;
    int rc = cnb_alloc(ctx, (size_t) N * N * sizeof(float), &p);
    if (rc != CNB_OK) return rc;
    t.re = static_cast<float*>(p);
    rc = cnb_alloc(ctx, (size_t) N * N * sizeof(float), &p);
    if (rc != CNB_OK) return rc;
    t.im = static_cast<float*>(p);
    twiddle_k<<<ctx->sm_count * 4, 256, 0, st>>>(t.re, t.im, N);
    CNB_LAUNCH_CHECK("twiddle");
    if (key & kTriKey) {
        tri_mask_k<<<ctx->sm_count * 4, 256, 0, st>>>(t.re, t.im, N);
        CNB_LAUNCH_CHECK("tri_mask");
    }
    if (cnb::cgemm_tc_shape_ok(64, N, N) && (!cnb::fft_supported(N) || (key & kTriKey))) {
        // the matrix is a constant: where the GEMM is the transform's engine, its operand split is
        // made here, not by every product
        rc = cnb_alloc(ctx, cnb_split_floats((size_t) N * N) * sizeof(float), &p);
        if (rc != CNB_OK) return rc;
        t.split = static_cast<float*>(p);
        rc = cnb::split_planes(ctx, t.re, t.im, (size_t) N * N, t.split, st);
        if (rc != CNB_OK) return rc;
    }
    ctx->twiddles[key] = t;
    *out = t;
    return CNB_OK;
}

// X F^T (conj = 0) or G conj(F) (conj = 1) with F symmetric, so F itself is the K-major operand
int twiddle_product(cnb_ctx* ctx, const cnb_twiddle& t, const float* x_re, const float* x_im, float* y_re, float* y_im,
                    int B, int N, int conj, int accumulate, cudaStream_t st) {
    if (cnb::cgemm_tc_shape_ok(B, N, N)) {
        cnb::g_last_engine = 1;
        return cnb::cgemm_tc_run(ctx, x_re, x_im, 0, t.re, t.im, 0, conj, nullptr, nullptr, y_re, y_im, B, N, N,
                                 accumulate, st, t.split);
    }
    cnb::g_last_engine = 2;
    return cnb::cgemm_simt(ctx, x_re, x_im, N, 1, t.re, t.im, N, 1, conj, nullptr, nullptr, y_re, y_im, B, N, N,
                           accumulate, st);
}

}  // namespace

extern "C" {

int cnb_linear_fwd(cnb_ctx* ctx, const float* x_re, const float* x_im, const float* w_re, const float* w_im,
                   const float* res_re, const float* res_im, float* y_re, float* y_im, int B, int in, int out,
                   void* stream) {
    CNB_CHECK_ARG(ctx && x_re && x_im && w_re && w_im && y_re && y_im, "cnb_linear_fwd: null pointer");
    CNB_CHECK_ARG((res_re == nullptr) == (res_im == nullptr), "cnb_linear_fwd: residual planes must be a pair");
    CNB_CHECK_ARG(B > 0 && in > 0 && out > 0, "cnb_linear_fwd: B=%d in=%d out=%d", B, in, out);
    cudaStream_t st = cnb::S(stream);
    if (cnb::skinny_ok(B, in, out) && !res_re) {
        cnb::g_last_engine = 4;
        return cnb::skinny_fwd(ctx, x_re, x_im, w_re, w_im, y_re, y_im, B, in, out, st);
    }
    if (cnb::cgemm_tc_shape_ok(B, out, in)) {
        cnb::g_last_engine = 1;
        return cnb::cgemm_tc_nt(ctx, x_re, x_im, w_re, w_im, 0, res_re, res_im, y_re, y_im, B, out, in, 0, st);
    }
    cnb::g_last_engine = 2;
    return cnb::cgemm_simt(ctx, x_re, x_im, in, 1, w_re, w_im, in, 1, 0, res_re, res_im, y_re, y_im, B, out, in,
                           0, st);
}

int cnb_linear_bwd_x(cnb_ctx* ctx, const float* g_re, const float* g_im, const float* w_re, const float* w_im,
                     float* dx_re, float* dx_im, int B, int in, int out, int accumulate, void* stream) {
    CNB_CHECK_ARG(ctx && g_re && g_im && w_re && w_im && dx_re && dx_im, "cnb_linear_bwd_x: null pointer");
    CNB_CHECK_ARG(B > 0 && in > 0 && out > 0, "cnb_linear_bwd_x: B=%d in=%d out=%d", B, in, out);
    cudaStream_t st = cnb::S(stream);
    // dX*[b,i] = sum_o G[b,o] conj(W[o,i]) : M = B, N = in, K = out; B-operand(n=i,k=o) = W[o,i]
    if (cnb::skinny_ok(B, in, out)) {
        cnb::g_last_engine = 4;
        return cnb::skinny_bwd_x(ctx, g_re, g_im, w_re, w_im, dx_re, dx_im, B, in, out, accumulate, st);
    }
    if (cnb::cgemm_tc_shape_ok(B, in, out)) {
        // the B operand (n = i, k = o) is W stored [K = out, N = in]: transposed while it is split
        cnb::g_last_engine = 1;
        return cnb::cgemm_tc_run(ctx, g_re, g_im, 0, w_re, w_im, 1, 1, nullptr, nullptr, dx_re, dx_im, B, in, out,
                                 accumulate, st);
    }
    cnb::g_last_engine = 2;
    return cnb::cgemm_simt(ctx, g_re, g_im, out, 1, w_re, w_im, 1, in, 1, nullptr, nullptr, dx_re, dx_im, B, in,
                           out, accumulate, st);
}

int cnb_linear_bwd_w(cnb_ctx* ctx, const float* g_re, const float* g_im, const float* x_re, const float* x_im,
                     float* dw_re, float* dw_im, int B, int in, int out, int accumulate, void* stream) {
    CNB_CHECK_ARG(ctx && g_re && g_im && x_re && x_im && dw_re && dw_im, "cnb_linear_bwd_w: null pointer");
    CNB_CHECK_ARG(B > 0 && in > 0 && out > 0, "cnb_linear_bwd_w: B=%d in=%d out=%d", B, in, out);
    cudaStream_t st = cnb::S(stream);
    // dW*[o,i] = sum_b G[b,o] conj(X[b,i]) : M = out, N = in, K = B
    if (cnb::skinny_ok(B, in, out)) {
        cnb::g_last_engine = 4;
        return cnb::skinny_bwd_w(ctx, g_re, g_im, x_re, x_im, dw_re, dw_im, B, in, out, accumulate, st);
    }
    if (cnb::cgemm_tc_shape_ok(out, in, B)) {
        // both operands are stored [K = B, rows]: transposed while they are split
        cnb::g_last_engine = 1;
        return cnb::cgemm_tc_run(ctx, g_re, g_im, 1, x_re, x_im, 1, 1, nullptr, nullptr, dw_re, dw_im, out, in, B,
                                 accumulate, st);
    }
    cnb::g_last_engine = 2;
    return cnb::cgemm_simt(ctx, g_re, g_im, 1, out, x_re, x_im, 1, in, 1, nullptr, nullptr, dw_re, dw_im, out, in,
                           B, accumulate, st);
}

int cnb_dft_fwd(cnb_ctx* ctx, const float* x_re, const float* x_im, float* y_re, float* y_im, int B, int N,
                void* stream) {
    CNB_CHECK_ARG(ctx && x_re && x_im && y_re && y_im, "cnb_dft_fwd: null pointer");
    CNB_CHECK_ARG(B > 0 && N > 0 && N <= 16384, "cnb_dft_fwd: B=%d N=%d (N <= 16384)", B, N);
    if (cnb::fft_supported(N) && !ctx->force_dft_gemm) {
        cnb::g_last_engine = 3;
        return cnb::fft_run(ctx, x_re, x_im, y_re, y_im, B, N, 0, 0, cnb::S(stream));
    }
    cnb_twiddle t;
    int rc = get_twiddle(ctx, N, cnb::S(stream), &t);
    if (rc != CNB_OK) return rc;
    return twiddle_product(ctx, t, x_re, x_im, y_re, y_im, B, N, 0, 0, cnb::S(stream));
}

int cnb_dft_bwd(cnb_ctx* ctx, const float* g_re, const float* g_im, float* dx_re, float* dx_im, int B, int N,
                int accumulate, void* stream) {
    CNB_CHECK_ARG(ctx && g_re && g_im && dx_re && dx_im, "cnb_dft_bwd: null pointer");
    CNB_CHECK_ARG(B > 0 && N > 0 && N <= 16384, "cnb_dft_bwd: B=%d N=%d (N <= 16384)", B, N);
    cudaStream_t st = cnb::S(stream);
    if (cnb::fft_supported(N) && !ctx->force_dft_gemm) {
        cnb::g_last_engine = 3;
        return cnb::fft_run(ctx, g_re, g_im, dx_re, dx_im, B, N, 1, accumulate, st);
    }
    cnb_twiddle t;
    int rc = get_twiddle(ctx, N, st, &t);
    if (rc != CNB_OK) return rc;
    return twiddle_product(ctx, t, g_re, g_im, dx_re, dx_im, B, N, 1, accumulate, st);
}

/* Scratch the three Linear products and the column reductions of one layer may need. */
size_t cnb_linear_workspace(int B, int in, int out) {
    size_t w = 0;
    if (cnb::skinny_ok(B, in, out)) return cnb::skinny_workspace_bytes(B, in, out, 256);
    if (cnb::cgemm_tc_shape_ok(B, out, in)) w = std::max(w, cnb::cgemm_tc_workspace_bytes(B, out, in));
    if (cnb::cgemm_tc_shape_ok(B, in, out)) w = std::max(w, cnb::cgemm_tc_workspace_bytes(B, in, out));
    if (cnb::cgemm_tc_shape_ok(out, in, B)) w = std::max(w, cnb::cgemm_tc_workspace_bytes(out, in, B));
    return w;
}

/* ---- operands split once by the caller (fp32 hi, bf16 hi and lo), reused by several products ---- */
size_t cnb_split_floats(size_t n) { return 4 * ((n + 63) & ~size_t(63)); }

int cnb_split_planes(cnb_ctx* ctx, const float* re, const float* im, size_t n, float* split, void* stream) {
    CNB_CHECK_ARG(ctx && re && im && split && n > 0, "cnb_split_planes: bad argument");
    return cnb::split_planes(ctx, re, im, n, split, cnb::S(stream));
}

int cnb_linear_split_ok(int B, int in, int out) {
    return (B >= 64 && in >= 64 && out >= 64 && in % 64 == 0 && out % 64 == 0) ? 1 : 0;
}

namespace {
inline void planes_of(const float* split, size_t n, const float* p[4]) {
    size_t np = (n + 63) & ~size_t(63);
    for (int q = 0; q < 4; ++q) p[q] = split + q * np;
}
}  // namespace

int cnb_linear_fwd_split(cnb_ctx* ctx, const float* x_split, const float* w_split, const float* res_re,
                         const float* res_im, float* y_re, float* y_im, int B, int in, int out, void* stream) {
    CNB_CHECK_ARG(ctx && x_split && w_split && y_re && y_im, "cnb_linear_fwd_split: null pointer");
    CNB_CHECK_ARG(cnb_linear_split_ok(B, in, out), "cnb_linear_fwd_split: B=%d in=%d out=%d not eligible", B, in, out);
    const float *a[4], *b[4];
    planes_of(x_split, (size_t) B * in, a);
    planes_of(w_split, (size_t) out * in, b);
    cnb::g_last_engine = 1;
    return cnb::cgemm_tc_presplit(ctx, a, 0, b, 0, 0, res_re, res_im, y_re, y_im, B, out, in, 0, cnb::S(stream));
}

int cnb_linear_bwd_x_split(cnb_ctx* ctx, const float* g_split, const float* w_split, float* dx_re, float* dx_im,
                           int B, int in, int out, int accumulate, void* stream) {
    CNB_CHECK_ARG(ctx && g_split && w_split && dx_re && dx_im, "cnb_linear_bwd_x_split: null pointer");
    CNB_CHECK_ARG(cnb_linear_split_ok(B, in, out), "cnb_linear_bwd_x_split: B=%d in=%d out=%d not eligible", B, in, out);
    const float *a[4], *b[4];
    planes_of(g_split, (size_t) B * out, a);
    planes_of(w_split, (size_t) out * in, b);      // W [out, in] = [K, N]: MN-major B operand
    cnb::g_last_engine = 1;
    return cnb::cgemm_tc_presplit(ctx, a, 0, b, 1, 1, nullptr, nullptr, dx_re, dx_im, B, in, out, accumulate,
                                  cnb::S(stream));
}

int cnb_linear_bwd_w_split(cnb_ctx* ctx, const float* g_split, const float* x_split, float* dw_re, float* dw_im,
                           int B, int in, int out, int accumulate, void* stream) {
    CNB_CHECK_ARG(ctx && g_split && x_split && dw_re && dw_im, "cnb_linear_bwd_w_split: null pointer");
    CNB_CHECK_ARG(cnb_linear_split_ok(B, in, out), "cnb_linear_bwd_w_split: B=%d in=%d out=%d not eligible", B, in, out);
    const float *a[4], *b[4];
    planes_of(g_split, (size_t) B * out, a);       // G [B, out] = [K, M]: MN-major A operand
    planes_of(x_split, (size_t) B * in, b);        // X [B, in]  = [K, N]: MN-major B operand
    cnb::g_last_engine = 1;
    return cnb::cgemm_tc_presplit(ctx, a, 1, b, 1, 1, nullptr, nullptr, dw_re, dw_im, out, in, B, accumulate,
                                  cnb::S(stream));
}

int cnb_dft_fused_ok(int N) { return cnb::fft_supported(N) ? 1 : 0; }

int cnb_dft_hadamard_gelu_fwd(cnb_ctx* ctx, const float* x_re, const float* x_im, const float* h_re,
                              const float* h_im, float* u_re, float* u_im, float* y_re, float* y_im, float* y_split,
                              int B, int N, void* stream) {
    CNB_CHECK_ARG(ctx && x_re && x_im && h_re && h_im && u_re && u_im, "cnb_dft_hadamard_gelu_fwd: null pointer");
    CNB_CHECK_ARG((y_re == nullptr) == (y_im == nullptr) && (y_re || y_split),
                  "cnb_dft_hadamard_gelu_fwd: y planes must be a pair, and may only be left out when y_split is given");
    CNB_CHECK_ARG(B > 0 && cnb::fft_supported(N), "cnb_dft_hadamard_gelu_fwd: B=%d, N=%d is not an FFT-kernel length", B, N);
    cnb::g_last_engine = 3;
    return cnb::fft_hadamard_gelu(ctx, x_re, x_im, h_re, h_im, u_re, u_im, y_re, y_im, y_split, B, N, cnb::S(stream));
}

int cnb_tdft_fwd(cnb_ctx* ctx, const float* x_re, const float* x_im, float* y_re, float* y_im, int B, int N,
                 void* stream) {
    CNB_CHECK_ARG(ctx && x_re && x_im && y_re && y_im, "cnb_tdft_fwd: null pointer");
    CNB_CHECK_ARG(B > 0 && N > 0 && N <= 16384, "cnb_tdft_fwd: B=%d N=%d (N <= 16384)", B, N);
    cnb_twiddle t;
    int rc = get_twiddle(ctx, N | kTriKey, cnb::S(stream), &t);
    if (rc != CNB_OK) return rc;
    // the forward product takes the masked matrix as the Linear weight; it is not symmetric
    return twiddle_product(ctx, t, x_re, x_im, y_re, y_im, B, N, 0, 0, cnb::S(stream));
}

int cnb_tdft_bwd(cnb_ctx* ctx, const float* g_re, const float* g_im, float* dx_re, float* dx_im, int B, int N,
                 int accumulate, void* stream) {
    CNB_CHECK_ARG(ctx && g_re && g_im && dx_re && dx_im, "cnb_tdft_bwd: null pointer");
    CNB_CHECK_ARG(B > 0 && N > 0 && N <= 16384, "cnb_tdft_bwd: B=%d N=%d (N <= 16384)", B, N);
    cnb_twiddle t;
    int rc = get_twiddle(ctx, N | kTriKey, cnb::S(stream), &t);
    if (rc != CNB_OK) return rc;
    return cnb_linear_bwd_x(ctx, g_re, g_im, t.re, t.im, dx_re, dx_im, B, N, N, accumulate, stream);
}

int cnb_set_gemm_sm_limit(cnb_ctx* ctx, int max_ctas) {
    CNB_CHECK_ARG(ctx && max_ctas >= 0, "cnb_set_gemm_sm_limit: bad argument");
    ctx->gemm_cta_limit = max_ctas;
    return CNB_OK;
}

int cnb_set_dft_engine(cnb_ctx* ctx, int force_gemm) {
    CNB_CHECK_ARG(ctx, "cnb_set_dft_engine: null context");
    ctx->force_dft_gemm = force_gemm != 0;
    return CNB_OK;
}

int cnb_reserve_scratch(cnb_ctx* ctx, size_t bytes) {
    CNB_CHECK_ARG(ctx, "cnb_reserve_scratch: null context");
    float* p = nullptr;
    return cnb::ensure_scratch(ctx, bytes, &p);
}

}  // extern "C"
