// Context, device arena, copies and error reporting of the C ABI.
#include <atomic>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>

#include "common.cuh"

namespace cnb {

static thread_local char g_err[512] = "";
thread_local int g_last_engine = 0;
static std::atomic<unsigned long long> g_launches{0};

int set_error(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

void count_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

bool pdl_enabled() {
    static const bool on = [] { const char* e = getenv("CNB_PDL"); return !(e && e[0] == '0'); }();
    return on;
}

int ensure_scratch(cnb_ctx* ctx, size_t bytes, float** out) {
    if (bytes > ctx->scratch_bytes) {
        size_t want = bytes < (8u << 20) ? (8u << 20) : bytes;
        void* p = nullptr;
        int rc = cnb_alloc(ctx, want, &p);
        if (rc != CNB_OK) return rc;
        ctx->scratch = static_cast<float*>(p);
        ctx->scratch_bytes = want;
    }
    *out = ctx->scratch;
    return CNB_OK;
}

}  // namespace cnb

extern "C" {

const char* cnb_last_error(void) { return cnb::g_err; }

unsigned long long cnb_launch_count(void) { return cnb::g_launches.load(); }

int cnb_last_gemm_engine(void) { return cnb::g_last_engine; }

static int create_common(int device, void* arena, size_t bytes, bool owns, cnb_ctx** out) {
    CNB_CHECK_ARG(out != nullptr, "cnb_create: out is null");
    CNB_CHECK_ARG(bytes >= (1u << 16), "cnb_create: arena of %zu bytes is too small", bytes);
    int ndev = 0;
    CNB_CUDA(cudaGetDeviceCount(&ndev));
    CNB_CHECK_ARG(device >= 0 && device < ndev, "cnb_create: device %d of %d", device, ndev);
    CNB_CUDA(cudaSetDevice(device));
    cnb_ctx* c = new cnb_ctx();
    c->device = device;
    c->owns = owns;
    if (owns) {
        void* p = nullptr;
        cudaError_t e = cudaMalloc(&p, bytes);
        if (e != cudaSuccess) {
            delete c;
            return cnb::set_error(CNB_ERR_CUDA, "cudaMalloc of the %zu-byte arena failed: %s", bytes,
                                  cudaGetErrorString(e));
        }
        arena = p;
    }
    CNB_CHECK_ARG((reinterpret_cast<uintptr_t>(arena) & 255) == 0, "arena must be 256-byte aligned");
    c->base = static_cast<char*>(arena);
    c->size = bytes;
    cudaDeviceGetAttribute(&c->sm_count, cudaDevAttrMultiProcessorCount, device);
    void* st = nullptr;
    int rc = cnb_alloc(c, 4096, &st);                    // error word, then the completion counters of reductions
    if (rc != CNB_OK) { cnb_destroy(c); return rc; }
    c->d_status = static_cast<int*>(st);
    c->d_counters = c->d_status + 256;
    cudaMemset(c->d_status, 0, 4096);
    *out = c;
    return CNB_OK;
}

int cnb_create(int device, size_t arena_bytes, cnb_ctx** out) {
    return create_common(device, nullptr, arena_bytes, true, out);
}

int cnb_create_external(int device, void* arena, size_t arena_bytes, cnb_ctx** out) {
    CNB_CHECK_ARG(arena != nullptr, "cnb_create_external: arena is null");
    return create_common(device, arena, arena_bytes, false, out);
}

int cnb_destroy(cnb_ctx* ctx) {
    if (!ctx) return CNB_OK;
    if (ctx->owns && ctx->base) cudaFree(ctx->base);
    delete ctx;
    return CNB_OK;
}

int cnb_alloc(cnb_ctx* ctx, size_t bytes, void** out) {
    CNB_CHECK_ARG(ctx && out, "cnb_alloc: null argument");
    size_t need = (bytes + 255) & ~size_t(255);
    if (ctx->used + need > ctx->size)
        return cnb::set_error(CNB_ERR_ARENA, "arena exhausted: %zu used + %zu requested > %zu", ctx->used, need,
                              ctx->size);
    *out = ctx->base + ctx->used;
    ctx->used += need;
    return CNB_OK;
}

int cnb_reset(cnb_ctx* ctx) {
    CNB_CHECK_ARG(ctx, "cnb_reset: null context");
    ctx->used = 4096;           // keep the status word and the counters
    ctx->scratch = nullptr;
    ctx->scratch_bytes = 0;
    ctx->twiddles.clear();
    return CNB_OK;
}

size_t cnb_arena_used(const cnb_ctx* ctx) { return ctx ? ctx->used : 0; }
size_t cnb_arena_size(const cnb_ctx* ctx) { return ctx ? ctx->size : 0; }

int cnb_device_info(int device, int* sm_count, int* cc_major, int* cc_minor, size_t* total_mem) {
    cudaDeviceProp p;
    CNB_CUDA(cudaGetDeviceProperties(&p, device));
    if (sm_count) *sm_count = p.multiProcessorCount;
    if (cc_major) *cc_major = p.major;
    if (cc_minor) *cc_minor = p.minor;
    if (total_mem) *total_mem = p.totalGlobalMem;
    return CNB_OK;
}

int cnb_h2d(cnb_ctx* ctx, void* dst, const void* src, size_t bytes, void* stream) {
    CNB_CHECK_ARG(ctx && dst && src, "cnb_h2d: null argument");
    CNB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyHostToDevice, cnb::S(stream)));
    return CNB_OK;
}

int cnb_d2h(cnb_ctx* ctx, void* dst, const void* src, size_t bytes, void* stream) {
    CNB_CHECK_ARG(ctx && dst && src, "cnb_d2h: null argument");
    CNB_CUDA(cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToHost, cnb::S(stream)));
    CNB_CUDA(cudaStreamSynchronize(cnb::S(stream)));
    return CNB_OK;
}

int cnb_memset0(cnb_ctx* ctx, void* dst, size_t bytes, void* stream) {
    CNB_CHECK_ARG(ctx && dst, "cnb_memset0: null argument");
    CNB_CUDA(cudaMemsetAsync(dst, 0, bytes, cnb::S(stream)));
    return CNB_OK;
}

int cnb_sync(cnb_ctx* ctx, void* stream) {
    CNB_CHECK_ARG(ctx, "cnb_sync: null context");
    CNB_CUDA(cudaStreamSynchronize(cnb::S(stream)));
    return CNB_OK;
}

int cnb_check_device_status(cnb_ctx* ctx, void* stream) {
    CNB_CHECK_ARG(ctx, "cnb_check_device_status: null context");
    int h[2] = {0, 0};
    CNB_CUDA(cudaMemcpyAsync(h, ctx->d_status, sizeof(h), cudaMemcpyDeviceToHost, cnb::S(stream)));
    CNB_CUDA(cudaStreamSynchronize(cnb::S(stream)));
    if (h[0] != 0) {
        CNB_CUDA(cudaMemsetAsync(ctx->d_status, 0, 256, cnb::S(stream)));
        return cnb::set_error(CNB_ERR_DEVICE, "a kernel gave up a bounded wait (code %d, detail %d)", h[0], h[1]);
    }
    return CNB_OK;
}

}  // extern "C"
