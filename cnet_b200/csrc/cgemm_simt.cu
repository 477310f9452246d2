// fp32 SIMT complex GEMM on generic strides.  Serves the skinny heads (out = 10), ragged
// shapes that do not fit the tensor-core tiles, and the operand orientations of the
// Linear backward without staging copies.  64x64 output tile, 16-deep k-slab in shared
// memory, 256 threads each owning a 4x4 block of complex accumulators.
#include "common.cuh"

namespace {

constexpr int TM = 64, TN = 64, TK = 16;

__global__ void __launch_bounds__(256)
cgemm_simt_k(const float* __restrict__ a_re, const float* __restrict__ a_im, long sam, long sak,
             const float* __restrict__ b_re, const float* __restrict__ b_im, long sbn, long sbk, int conjB,
             const float* __restrict__ r_re, const float* __restrict__ r_im,
             float* __restrict__ d_re, float* __restrict__ d_im, int M, int N, int K, int accumulate) {
    cnb_pdl_enter();
    __shared__ float As_r[TK][TM + 4], As_i[TK][TM + 4], Bs_r[TK][TN + 4], Bs_i[TK][TN + 4];
    int tid = threadIdx.x;
    int m0 = blockIdx.y * TM, n0 = blockIdx.x * TN;
    int tx = tid & 15, ty = tid >> 4;          // 16 x 16 threads, 4x4 micro-tile each
    float cr[4][4] = {}, ci[4][4] = {};
    // loader mapping: pick the index that is contiguous in memory as the fast one
    bool a_kfast = (sak == 1), b_kfast = (sbk == 1);
    for (int k0 = 0; k0 < K; k0 += TK) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int e = tid + j * 256;             // 0..1023 = TM*TK
            int mm = a_kfast ? e / TK : e % TM;
            int kk = a_kfast ? e % TK : e / TM;
            int gm = m0 + mm, gk = k0 + kk;
            float vr = 0.f, vi = 0.f;
            if (gm < M && gk < K) { size_t o = (size_t) gm * sam + (size_t) gk * sak; vr = a_re[o]; vi = a_im[o]; }
            As_r[kk][mm] = vr; As_i[kk][mm] = vi;
            int nn = b_kfast ? e / TK : e % TN;
            kk = b_kfast ? e % TK : e / TN;
            int gn = n0 + nn; gk = k0 + kk;
            vr = 0.f; vi = 0.f;
            if (gn < N && gk < K) { size_t o = (size_t) gn * sbn + (size_t) gk * sbk; vr = b_re[o]; vi = b_im[o]; }
            Bs_r[kk][nn] = vr; Bs_i[kk][nn] = conjB ? -vi : vi;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < TK; ++kk) {
            float ar[4], ai[4], br[4], bi[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                ar[i] = As_r[kk][ty * 4 + i]; ai[i] = As_i[kk][ty * 4 + i];
                br[i] = Bs_r[kk][tx * 4 + i]; bi[i] = Bs_i[kk][tx * 4 + i];
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    cr[i][j] += ar[i] * br[j] - ai[i] * bi[j];
                    ci[i][j] += ar[i] * bi[j] + ai[i] * br[j];
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            int gn = n0 + tx * 4 + j;
            if (gn >= N) continue;
            size_t o = (size_t) gm * N + gn;
            float vr = cr[i][j], vi = ci[i][j];
            if (r_re) { vr += r_re[o]; vi += r_im[o]; }
            if (accumulate) { vr += d_re[o]; vi += d_im[o]; }
            d_re[o] = vr; d_im[o] = vi;
        }
    }
}

}  // namespace

namespace cnb {

int cgemm_simt(cnb_ctx* ctx, const float* a_re, const float* a_im, long sam, long sak, const float* b_re,
               const float* b_im, long sbn, long sbk, int conjB, const float* r_re, const float* r_im,
               float* d_re, float* d_im, int M, int N, int K, int accumulate, cudaStream_t st) {
    (void) ctx;
    dim3 grid((N + TN - 1) / TN, (M + TM - 1) / TM);
    cnb::launch(cgemm_simt_k, dim3(grid), dim3(256), 0, st, 1, a_re, a_im, sam, sak, b_re, b_im, sbn, sbk, conjB, r_re, r_im, d_re, d_im,
                                       M, N, K, accumulate);
    CNB_LAUNCH_CHECK("cgemm_simt");
    return CNB_OK;
}

}  // namespace cnb
