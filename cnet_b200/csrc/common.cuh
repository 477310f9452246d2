// Shared declarations of the device library: context, error plumbing, launch helpers.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>
#include <algorithm>
#include <map>
#include <string>

#include "../../include/cnet_b200.h"

struct cnb_twiddle {
    float* re = nullptr;   // [N, N] planes, F[p,q] = N^-1/2 e^{-2 pi i pq/N}
    float* im = nullptr;
    float* split = nullptr;   // split buffer of the matrix (made once), or null when the tiles cannot take it
};

struct cnb_ctx {
    int device = 0;
    int sm_count = 148;
    char* base = nullptr;
    size_t size = 0;
    size_t used = 0;
    bool owns = false;
    int* d_status = nullptr;          // device error word (bounded waits report here)
    int* d_counters = nullptr;        // 8 sets of 64 "CTAs done" counters, zero between launches
    unsigned counter_set = 0;
    float* scratch = nullptr;         // column-reduction partials and GEMM operand staging
    size_t scratch_bytes = 0;
    std::map<int, cnb_twiddle> twiddles;
    int gemm_cta_limit = 0;           // > 0: the tensor-core GEMM uses at most this many CTAs (SMs)
    bool force_dft_gemm = false;      // FourierTrans as a GEMM even where the FFT kernel applies
};

namespace cnb {

int set_error(int code, const char* fmt, ...);
void count_launch();
int ensure_scratch(cnb_ctx* ctx, size_t bytes, float** out);
extern thread_local int g_last_engine;

inline cudaStream_t S(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// SMs a kernel sized as "one wave" should count on: all of them, or fewer while some are set aside for a
// collective's kernels (cnb_set_gemm_sm_limit); sized for the whole device such a kernel would run a second,
// nearly empty wave.
inline int usable_sms(const cnb_ctx* ctx) {
    return ctx->gemm_cta_limit > 0 && ctx->gemm_cta_limit < ctx->sm_count ? ctx->gemm_cta_limit : ctx->sm_count;
}

// fp32 SIMT complex GEMM on generic strides:
//   D[m,n] (+)= sum_k A(m,k) * (conjB ? conj(B(n,k)) : B(n,k)) (+ R[m,n])
//   A(m,k) = a[m*sam + k*sak], B(n,k) = b[n*sbn + k*sbk], D/R row-major with ld = N.
int cgemm_simt(cnb_ctx* ctx, const float* a_re, const float* a_im, long sam, long sak,
               const float* b_re, const float* b_im, long sbn, long sbk, int conjB,
               const float* r_re, const float* r_im, float* d_re, float* d_im,
               int M, int N, int K, int accumulate, cudaStream_t st);

// tcgen05 complex GEMM on split operands, K-major operands only:
//   D[m,n] (+)= sum_k A[m,k] * (conjB ? conj(B[n,k]) : B[n,k]) (+ R[m,n]); A [M,K], B [N,K] row-major.
// Returns CNB_ERR_UNSUPPORTED when the shape does not fit its tiles.
int cgemm_tc_nt(cnb_ctx* ctx, const float* a_re, const float* a_im,
                const float* b_re, const float* b_im, int conjB,
                const float* r_re, const float* r_im, float* d_re, float* d_im,
                int M, int N, int K, int accumulate, cudaStream_t st);
bool cgemm_tc_shape_ok(int M, int N, int K);
// General form: a_trans / b_trans = the source planes are stored [K, rows] (transposed while splitting).
int cgemm_tc_run(cnb_ctx* ctx, const float* a_re, const float* a_im, int a_trans, const float* b_re,
                 const float* b_im, int b_trans, int conjB, const float* r_re, const float* r_im, float* d_re,
                 float* d_im, int M, int N, int K, int accumulate, cudaStream_t st,
                 const float* b_split = nullptr);
size_t cgemm_tc_workspace_bytes(int M, int N, int K);
// Operands already split: a[q] / b[q] = slot q of the split buffer (see cnb_split_component below); major 0 =
// [rows, K], 1 = [K, rows].
int cgemm_tc_presplit(cnb_ctx* ctx, const float* const a[4], int a_mn, const float* const b[4], int b_mn, int conjB,
                      const float* r_re, const float* r_im, float* d_re, float* d_im, int M, int N, int K,
                      int accumulate, cudaStream_t st);
// split = 4 consecutive slots of pad64(n) floats (see cnb_split_component below)
int split_planes(cnb_ctx* ctx, const float* re, const float* im, size_t n, float* split, cudaStream_t st);

// Skinny Linear (out <= 16): HBM-bound fp32 kernels.
bool skinny_ok(int B, int in, int out);
size_t skinny_workspace_bytes(int B, int in, int out, int sm_count);
int skinny_fwd(cnb_ctx* ctx, const float* xr, const float* xi, const float* wr, const float* wi, float* yr, float* yi,
               int B, int in, int out, cudaStream_t st);
int skinny_bwd_x(cnb_ctx* ctx, const float* gr, const float* gi, const float* wr, const float* wi, float* dr,
                 float* di, int B, int in, int out, int accumulate, cudaStream_t st);
int skinny_bwd_w(cnb_ctx* ctx, const float* gr, const float* gi, const float* xr, const float* xi, float* dr,
                 float* di, int B, int in, int out, int accumulate, cudaStream_t st);

// Shared-memory FFT (N = 256, 1024, 4096); inverse = conjugate direction.
bool fft_supported(int N);
int fft_run(cnb_ctx* ctx, const float* xr, const float* xi, float* yr, float* yi, int B, int N, int inverse,
            int accumulate, cudaStream_t st);
// Forward FFT whose epilogue also applies Hadamard(h) -> CGelu: u = FFT(x) -> (ur, ui); y = gelu(u o h) ->
// (yr, yi) and, when sp != NULL, the operand split of y.
int fft_hadamard_gelu(cnb_ctx* ctx, const float* xr, const float* xi, const float* hr, const float* hi, float* ur,
                      float* ui, float* yr, float* yi, float* sp, int B, int N, cudaStream_t st);

}  // namespace cnb

// CGelu of the reference (impl/relu.h:119-131): tanh form; the derivative uses sech^2 = 1 - tanh^2.
// tanh(y) = 1 - 2 / (e^{2y} + 1) on the special-function unit: absolute error below 1e-7 (the
// approximate exp2 is good to 2^-22; both tails saturate to +-1 exactly), a third of tanhf's instructions.
__device__ __forceinline__ float cnb_tanh(float y) {
    return 1.0f - __fdividef(2.0f, __expf(2.0f * y) + 1.0f);
}

__device__ __forceinline__ float cnb_gelu(float x) {
    float t = cnb_tanh(0.7978845608028654f * (x + 0.044715f * x * x * x));
    return 0.5f * x * (1.0f + t);
}

__device__ __forceinline__ float cnb_dgelu(float x) {
    float x2 = x * x;
    float t = cnb_tanh(0.7978845608028654f * (x + 0.044715f * x * x2));
    float sech2 = 1.0f - t * t;
    return 0.5f * (1.0f + t) + 0.5f * x * sech2 * 0.7978845608028654f * (1.0f + 3.0f * 0.044715f * x2);
}

// The operand split of the tensor-core product.  x = hi + lo with hi = x cut to TF32 (low 13 mantissa bits
// cleared) and lo = x - hi, exact in fp32.  A product x.y is taken as hi.hi on the TF32 pipe plus the two cross
// terms hi.lo + lo.hi on the BF16 pipe, for which hi and lo are also kept rounded to bf16 (h16, l16).  A split
// buffer of n elements is four slots of np = pad64(n) floats:
//   slot 0: hi of the real plane (fp32)      slot 2: h16 of the real plane, then of the imaginary plane (bf16)
//   slot 1: hi of the imaginary plane        slot 3: l16 of the real plane, then of the imaginary plane
__device__ __forceinline__ float cnb_tf32_hi(float x) { return __uint_as_float(__float_as_uint(x) & 0xFFFFE000u); }
__device__ __forceinline__ unsigned short cnb_bf16_bits(float x) { return __bfloat16_as_ushort(__float2bfloat16_rn(x)); }

struct cnb_split_dst {
    float* hi;               // fp32 hi plane of this component (real or imaginary)
    unsigned short* h16;     // its bf16 planes
    unsigned short* l16;
};

// component c (0 = real, 1 = imaginary) of a split buffer with plane pitch np
__host__ __device__ __forceinline__ cnb_split_dst cnb_split_component(float* sp, size_t np, int c) {
    cnb_split_dst d;
    d.hi = sp + (size_t) c * np;
    d.h16 = reinterpret_cast<unsigned short*>(sp + 2 * np) + (size_t) c * np;
    d.l16 = reinterpret_cast<unsigned short*>(sp + 3 * np) + (size_t) c * np;
    return d;
}

__device__ __forceinline__ void cnb_split_store1(const cnb_split_dst& d, size_t i, float x) {
    const float h = cnb_tf32_hi(x);
    d.hi[i] = h;
    d.h16[i] = cnb_bf16_bits(h);
    d.l16[i] = cnb_bf16_bits(x - h);
}

// four consecutive elements, i % 4 == 0 (16-byte store of hi, 8-byte stores of the bf16 planes)
__device__ __forceinline__ void cnb_split_store4(const cnb_split_dst& d, size_t i, float x0, float x1, float x2, float x3) {
    const float h0 = cnb_tf32_hi(x0), h1 = cnb_tf32_hi(x1), h2 = cnb_tf32_hi(x2), h3 = cnb_tf32_hi(x3);
    *reinterpret_cast<float4*>(d.hi + i) = make_float4(h0, h1, h2, h3);
    uint2 a, b;
    a.x = (uint32_t) cnb_bf16_bits(h0) | ((uint32_t) cnb_bf16_bits(h1) << 16);
    a.y = (uint32_t) cnb_bf16_bits(h2) | ((uint32_t) cnb_bf16_bits(h3) << 16);
    b.x = (uint32_t) cnb_bf16_bits(x0 - h0) | ((uint32_t) cnb_bf16_bits(x1 - h1) << 16);
    b.y = (uint32_t) cnb_bf16_bits(x2 - h2) | ((uint32_t) cnb_bf16_bits(x3 - h3) << 16);
    *reinterpret_cast<uint2*>(d.h16 + i) = a;
    *reinterpret_cast<uint2*>(d.l16 + i) = b;
}

// Programmatic dependent launch.  Every kernel of the step is launched with the "programmatic stream
// serialization" attribute (cnb::launch below): it may be scheduled as soon as every CTA of the kernel before
// it in the stream has called cnb_pdl_trigger() (or exited), so its launch latency and its set-up (barriers,
// tensor memory, tables that no kernel writes) run under the predecessor's tail.  cnb_pdl_wait() returns when
// the predecessor grid has completed and its memory is visible: nothing a predecessor writes or reads may be
// touched before it.  Both are no-ops in a kernel launched the ordinary way.
__device__ __forceinline__ void cnb_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void cnb_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void cnb_pdl_enter() { cnb_pdl_trigger(); cnb_pdl_wait(); }

namespace cnb {

bool pdl_enabled();                // CNB_PDL=0 in the environment launches every kernel fully serialised

// Launch of a kernel that starts with cnb_pdl_enter() (or does its own trigger / wait); cluster > 1 adds a
// thread-block cluster of that many CTAs along x.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_ex(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, int cluster,
                             bool dependent, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[2];
    unsigned n = 0;
    if (dependent && pdl_enabled()) {
        at[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster > 1) {
        at[n].id = cudaLaunchAttributeClusterDimension;
        at[n].val.clusterDim.x = (unsigned) cluster;
        at[n].val.clusterDim.y = 1;
        at[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = at;
    cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, int cluster,
                          Args... args) {
    return launch_ex(kernel, grid, block, smem, st, cluster, true, args...);
}

}  // namespace cnb

#define CNB_CHECK_ARG(cond, ...) \
    do { if (!(cond)) return cnb::set_error(CNB_ERR_ARG, __VA_ARGS__); } while (0)

#define CNB_CUDA(call) \
    do { cudaError_t e_ = (call); \
         if (e_ != cudaSuccess) return cnb::set_error(CNB_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e_)); } while (0)

#define CNB_LAUNCH_CHECK(name) \
    do { cnb::count_launch(); cudaError_t e_ = cudaGetLastError(); \
         if (e_ != cudaSuccess) return cnb::set_error(CNB_ERR_CUDA, "launch of %s failed: %s", name, cudaGetErrorString(e_)); } while (0)
