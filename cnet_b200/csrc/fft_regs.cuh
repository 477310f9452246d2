// Pieces shared by the FourierTrans kernels: twiddle constants, the in-register R-point FFT and
// the descriptor of the fused forward tail.
#pragma once
#include "common.cuh"

namespace cnb_fft {

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
                else if (t == 16) { re[i1] = -SIGN * di; im[i1] = SIGN * dr; }   // times SIGN * i
                else {
                    const float c = kCos64[t], s = SIGN * kSin64[t];   // e^{SIGN * 2 pi i t/64}
                    re[i1] = dr * c - di * s;
                    im[i1] = dr * s + di * c;
                }
            }
        }
    }
}

// Optional fused tail of the forward transform: Hadamard with a shared vector h, then CGelu.
struct FftEpilogue {
    const float* hr = nullptr;      // h planes [N]; NULL = plain transform
    const float* hi = nullptr;
    float* gr = nullptr;            // gelu(u o h) planes [B, N]; may be NULL when sp is given (hi + l16 is the value to 2^-19)
    float* gi = nullptr;
    float* sp = nullptr;            // operand split of that (a split buffer with plane pitch np) or NULL
    size_t np = 0;
};

}  // namespace cnb_fft

namespace cnb {
// N = 1024: persistent kernel fed and drained by bulk copies
// fresh_table: `tw` is written by the launch just before this one (the kernel reads it before it waits for its
// predecessor, so that one launch must be fully serialised)
int fft1024_pipe(cnb_ctx* ctx, const float* xr, const float* xi, float* yr, float* yi, const float2* tw, int B,
                 int inverse, int accumulate, const cnb_fft::FftEpilogue& ep, cudaStream_t st, bool fresh_table);
}  // namespace cnb
