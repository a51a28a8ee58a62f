// Per-device library state and error reporting.
//
// The reference aborts the process on any CUDA error (cuda/cuda_backend.c:15-34).  A shared
// library cannot do that to its host, so every entry point returns a code and keeps the
// message; a C caller that wants the reference's behaviour prints tb_last_error() and exits.
#include "common.h"

#include <cstdarg>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <set>
#include <string>

namespace tb {

static thread_local char g_err[1024] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

const char* last_error() { return g_err; }

static DeviceCtx g_ctx[64];
static std::mutex g_ctx_mutex;

int get_ctx(DeviceCtx** out) {
    int dev = -1;
    TB_CUDA(cudaGetDevice(&dev));
    TB_CHECK(dev >= 0 && dev < 64, "device ordinal %d out of range", dev);
    DeviceCtx* c = &g_ctx[dev];
    if (c->device != dev) {
        std::lock_guard<std::mutex> lock(g_ctx_mutex);
        if (c->device != dev) {
            cudaDeviceProp prop;
            TB_CUDA(cudaGetDeviceProperties(&prop, dev));
            TB_CHECK(prop.major == 10, "this library is built for sm_100a only; device %d is sm_%d%d", dev, prop.major,
                     prop.minor);
            c->sm_count = prop.multiProcessorCount;
            // TB_SM_RESERVE=n: the persistent kernels (one CTA per SM) leave n SMs free, e.g. for the
            // communication kernels of a data-parallel run, whose CTAs would otherwise hold up whole GEMMs
            if (const char* e = getenv("TB_SM_RESERVE")) {
                const int n = atoi(e);
                if (n > 0 && n < c->sm_count - 8) c->sm_count -= n;
            }
            TB_CUDA(cudaMalloc(&c->d_err, 1024));
            TB_CUDA(cudaMemset(c->d_err, 0, 1024));
            c->d_tickets = reinterpret_cast<unsigned int*>(c->d_err + 32);
            c->d_best = reinterpret_cast<unsigned long long*>(c->d_err + 64);
            c->scratch = nullptr;
            c->scratch_bytes = 0;
            c->launches = 0;
            c->device = dev;
        }
    }
    *out = c;
    return 0;
}

int ensure_scratch(DeviceCtx* ctx, size_t bytes) {
    if (bytes <= ctx->scratch_bytes) return 0;
    // growing: earlier work may still be reading the old buffer
    TB_CUDA(cudaDeviceSynchronize());
    if (ctx->scratch) TB_CUDA(cudaFree(ctx->scratch));
    ctx->scratch = nullptr;
    ctx->scratch_bytes = 0;
    size_t want = bytes + (bytes >> 2);
    want = (want + (1u << 20) - 1) & ~((size_t)(1u << 20) - 1);
    TB_CUDA(cudaMalloc(&ctx->scratch, want));
    ctx->scratch_bytes = want;
    return 0;
}

int pdl_mode() {
    static int mode = -1;
    if (mode < 0) {
        const char* e = getenv("TB_PDL");
        mode = getenv("TB_NO_PDL") ? 0 : (e ? atoi(e) : 2);
    }
    return mode;
}

const char* prof_intern(const char* text) {
    static std::set<std::string> pool;
    static std::mutex m;
    std::lock_guard<std::mutex> lock(m);
    return pool.insert(text).first->c_str();
}

void prof_mark(DeviceCtx* ctx, const char* tag, double flops, double bytes, cudaStream_t stream) {
    if (!ctx->prof_on) return;
    if (!ctx->prof) ctx->prof = new std::vector<ProfRec>();
    ProfRec r;
    r.tag = tag; r.flops = flops; r.bytes = bytes; r.ev_end = nullptr;
    if (cudaEventCreate(&r.ev) != cudaSuccess) return;
    cudaEventRecord(r.ev, stream);
    ctx->prof->push_back(r);
}

void prof_close(DeviceCtx* ctx, cudaStream_t stream) {
    if (!ctx->prof_on || !ctx->prof || ctx->prof->empty()) return;
    ProfRec& r = ctx->prof->back();
    if (r.ev_end != nullptr) return;
    if (cudaEventCreate(&r.ev_end) != cudaSuccess) { r.ev_end = nullptr; return; }
    cudaEventRecord(r.ev_end, stream);
}

int check_device_error(DeviceCtx* ctx, cudaStream_t stream) {
    int h = 0;
    TB_CUDA(cudaStreamSynchronize(stream));
    TB_CUDA(cudaMemcpy(&h, ctx->d_err, sizeof(int), cudaMemcpyDeviceToHost));
    if (h != 0) {
        // the ticket words and packed maxima behind the error word go back to zero as well: a kernel that
        // gave up may have left them half-way
        cudaMemset(ctx->d_err, 0, 1024);
        const char* who = h == 1 ? "TMA producer" : h == 2 ? "MMA issuer" : h == 3 ? "epilogue" : "kernel";
        set_error("a kernel gave up on a bounded wait (%s, code %d); its output is invalid", who, h);
        return -3;
    }
    return 0;
}

}  // namespace tb
