// CEmbedding: row gather (forward) and scatter-add of dL/dz* rows (backward).
// One thread per 4 floats of an embedding row when D % 4 == 0 (16-byte accesses).
#include "common.cuh"

namespace {

template <int W>
__global__ void embed_fwd_k(const float* __restrict__ tr, const float* __restrict__ ti,
                            const int32_t* __restrict__ tok, float* __restrict__ orr, float* __restrict__ oi,
                            size_t rows, int D, int V) {
    cnb_pdl_enter();
    int per_row = D / W;
    size_t total = rows * per_row;
    for (size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t) gridDim.x * blockDim.x) {
        size_t row = i / per_row;
        int d = (int) (i % per_row) * W;
        int t = tok[row];
        size_t dst = row * D + d;
        if (t < 0 || t >= V) {
            if constexpr (W == 4) {
                *reinterpret_cast<float4*>(orr + dst) = make_float4(0.f, 0.f, 0.f, 0.f);
                *reinterpret_cast<float4*>(oi + dst) = make_float4(0.f, 0.f, 0.f, 0.f);
            } else { orr[dst] = 0.f; oi[dst] = 0.f; }
        } else {
            size_t src = (size_t) t * D + d;
            if constexpr (W == 4) {
                *reinterpret_cast<float4*>(orr + dst) = *reinterpret_cast<const float4*>(tr + src);
                *reinterpret_cast<float4*>(oi + dst) = *reinterpret_cast<const float4*>(ti + src);
            } else { orr[dst] = tr[src]; oi[dst] = ti[src]; }
        }
    }
}

// W = 4: a thread takes 4 consecutive floats of a gradient row (one 16-byte load per plane) and adds them to
// the table's gradient row with one 16-byte vector reduction per plane (red.global.add.v4.f32) instead of four
// scalar atomics.  Rows that hit the same table row are summed in arrival order: the sums differ by fp32
// reassociation from run to run (~1e-7 relative), as with the reference's own atomicAdd kernel
// (gpu/kernels.cpp:404-442).
template <int W>
__global__ void embed_bwd_k(const float* __restrict__ gr, const float* __restrict__ gi,
                            const int32_t* __restrict__ tok, float* __restrict__ dr, float* __restrict__ di,
                            size_t rows, int D, int V) {
    cnb_pdl_enter();
    const int per_row = D / W;
    const size_t total = rows * per_row;
    for (size_t i = (size_t) blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t) gridDim.x * blockDim.x) {
        const size_t row = i / per_row;
        const int d = (int) (i % per_row) * W;
        const int t = tok[row];
        if (t < 0 || t >= V) continue;
        const size_t src = row * D + d, dst = (size_t) t * D + d;
        if constexpr (W == 4) {
            const float4 a = *reinterpret_cast<const float4*>(gr + src), b = *reinterpret_cast<const float4*>(gi + src);
            atomicAdd(reinterpret_cast<float4*>(dr + dst), a);
            atomicAdd(reinterpret_cast<float4*>(di + dst), b);
        } else {
            atomicAdd(dr + dst, gr[src]);
            atomicAdd(di + dst, gi[src]);
        }
    }
}

}  // namespace

extern "C" {

int cnb_embed_fwd(cnb_ctx* ctx, const float* tab_re, const float* tab_im, const int32_t* tokens, float* out_re,
                  float* out_im, int B, int T, int D, int V, void* stream) {
    CNB_CHECK_ARG(ctx && tab_re && tab_im && tokens && out_re && out_im, "cnb_embed_fwd: null pointer");
    CNB_CHECK_ARG(B > 0 && T > 0 && D > 0 && V > 0, "cnb_embed_fwd: B=%d T=%d D=%d V=%d", B, T, D, V);
    size_t rows = (size_t) B * T;
    bool vec = (D % 4 == 0) && ((reinterpret_cast<uintptr_t>(tab_re) | reinterpret_cast<uintptr_t>(tab_im) |
                                 reinterpret_cast<uintptr_t>(out_re) | reinterpret_cast<uintptr_t>(out_im)) & 15) == 0;
    size_t items = rows * (vec ? D / 4 : D);
    size_t blocks = (items + 255) / 256, cap = (size_t) ctx->sm_count * 16;
    int grid = (int) (blocks < cap ? blocks : cap);
    if (vec) cnb::launch(embed_fwd_k<4>, dim3(grid), dim3(256), 0, cnb::S(stream), 1, tab_re, tab_im, tokens, out_re, out_im, rows, D, V);
    else cnb::launch(embed_fwd_k<1>, dim3(grid), dim3(256), 0, cnb::S(stream), 1, tab_re, tab_im, tokens, out_re, out_im, rows, D, V);
    CNB_LAUNCH_CHECK("embed_fwd");
    return CNB_OK;
}

int cnb_embed_bwd(cnb_ctx* ctx, const float* g_re, const float* g_im, const int32_t* tokens, float* dtab_re,
                  float* dtab_im, int B, int T, int D, int V, void* stream) {
    CNB_CHECK_ARG(ctx && g_re && g_im && tokens && dtab_re && dtab_im, "cnb_embed_bwd: null pointer");
    CNB_CHECK_ARG(B > 0 && T > 0 && D > 0 && V > 0, "cnb_embed_bwd: B=%d T=%d D=%d V=%d", B, T, D, V);
    size_t rows = (size_t) B * T;
    bool vec = (D % 4 == 0) && ((reinterpret_cast<uintptr_t>(g_re) | reinterpret_cast<uintptr_t>(g_im) |
                                 reinterpret_cast<uintptr_t>(dtab_re) | reinterpret_cast<uintptr_t>(dtab_im)) & 15) == 0;
    size_t items = rows * (vec ? D / 4 : D);
    size_t blocks = (items + 255) / 256, cap = (size_t) ctx->sm_count * 16;
    int grid = (int) (blocks < cap ? blocks : cap);
    if (vec) cnb::launch(embed_bwd_k<4>, dim3(grid), dim3(256), 0, cnb::S(stream), 1, g_re, g_im, tokens, dtab_re, dtab_im, rows, D, V);
    else cnb::launch(embed_bwd_k<1>, dim3(grid), dim3(256), 0, cnb::S(stream), 1, g_re, g_im, tokens, dtab_re, dtab_im, rows, D, V);
    CNB_LAUNCH_CHECK("embed_bwd");
    return CNB_OK;
}

}  // extern "C"
