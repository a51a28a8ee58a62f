// extern "C" entry points declared in include/turkce_b200.h (library, memory and GEMM part).
#include "../../include/turkce_b200.h"
#include "common.h"

#include <cstring>
#include <map>
#include <mutex>
#include <string>

using namespace tb;

static inline cudaStream_t S(void* s) { return static_cast<cudaStream_t>(s); }

extern "C" {

int tb_init(int device) {
    TB_CUDA(cudaSetDevice(device));
    DeviceCtx* ctx;
    return get_ctx(&ctx);
}

int tb_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) return 0;
    return n;
}

const char* tb_last_error(void) { return last_error(); }

long long tb_launch_count(void) {
    DeviceCtx* ctx;
    if (get_ctx(&ctx) != 0) return -1;
    return ctx->launches;
}

int tb_check(void* stream) {
    DeviceCtx* ctx;
    TB_TRY(get_ctx(&ctx));
    return check_device_error(ctx, S(stream));
}

int tb_shutdown(void) {
    DeviceCtx* ctx;
    TB_TRY(get_ctx(&ctx));
    TB_CUDA(cudaDeviceSynchronize());
    if (ctx->scratch) TB_CUDA(cudaFree(ctx->scratch));
    ctx->scratch = nullptr;
    ctx->scratch_bytes = 0;
    return 0;
}

int tb_profile_begin(void) {
    DeviceCtx* ctx;
    TB_TRY(get_ctx(&ctx));
    if (ctx->prof) {
        for (auto& r : *ctx->prof) { cudaEventDestroy(r.ev); if (r.ev_end) cudaEventDestroy(r.ev_end); }
        ctx->prof->clear();
    }
    ctx->prof_on = true;
    return 0;
}

int tb_profile_end(void* stream, char* out, int cap) {
    DeviceCtx* ctx;
    TB_TRY(get_ctx(&ctx));
    ctx->prof_on = false;
    TB_CHECK(out != nullptr && cap > 0, "tb_profile_end: no output buffer");
    out[0] = 0;
    if (!ctx->prof || ctx->prof->empty()) return 0;
    cudaEvent_t last;
    TB_CUDA(cudaEventCreate(&last));
    TB_CUDA(cudaEventRecord(last, S(stream)));
    TB_CUDA(cudaEventSynchronize(last));
    struct Agg { long long n = 0; double ms = 0, flops = 0, bytes = 0; };
    std::map<std::string, Agg> agg;
    auto& v = *ctx->prof;
    for (size_t i = 0; i < v.size(); ++i) {
        float ms = 0.f;
        cudaEvent_t next = v[i].ev_end ? v[i].ev_end : ((i + 1 < v.size()) ? v[i + 1].ev : last);
        if (cudaEventElapsedTime(&ms, v[i].ev, next) != cudaSuccess) ms = 0.f;
        Agg& a = agg[v[i].tag];
        a.n++; a.ms += ms; a.flops += v[i].flops; a.bytes += v[i].bytes;
    }
    std::string text;
    char line[256];
    for (auto& kv : agg) {
        snprintf(line, sizeof(line), "%s %lld %.6f %.6e %.6e\n", kv.first.c_str(), kv.second.n, kv.second.ms,
                 kv.second.flops, kv.second.bytes);
        text += line;
    }
    for (auto& r : v) { cudaEventDestroy(r.ev); if (r.ev_end) cudaEventDestroy(r.ev_end); }
    v.clear();
    cudaEventDestroy(last);
    strncpy(out, text.c_str(), (size_t)cap - 1);
    out[cap - 1] = 0;
    return 0;
}

int tb_alloc(void** d_ptr, uint64_t bytes) { TB_CUDA(cudaMalloc(d_ptr, bytes)); return 0; }
int tb_free(void* d_ptr) { TB_CUDA(cudaFree(d_ptr)); return 0; }
int tb_h2d(void* d_dst, const void* h_src, uint64_t bytes) {
    TB_H2D_SYNC(d_dst, h_src, bytes);
    return 0;
}
int tb_d2h(void* h_dst, const void* d_src, uint64_t bytes) {
    TB_CUDA(cudaMemcpy(h_dst, d_src, bytes, cudaMemcpyDeviceToHost));
    return 0;
}
int tb_memset_zero(void* d_ptr, uint64_t bytes) { TB_CUDA(cudaMemset(d_ptr, 0, bytes)); return 0; }
int tb_sync(void) { TB_CUDA(cudaDeviceSynchronize()); return 0; }

int tb_pack_bf16(const float* d_src, void* d_dst, int rows, int cols, int64_t ld_src, int64_t ld_dst,
                 int batch, int64_t stride_src, int64_t stride_dst, void* stream) {
    DeviceCtx* ctx;
    TB_TRY(get_ctx(&ctx));
    return launch_pack_bf16(ctx, d_src, static_cast<bf16*>(d_dst), rows, cols, ld_src, ld_dst, batch, stride_src,
                            stride_dst, S(stream));
}

int tb_gemm_swiglu_bf16(const void* d_X, const void* d_W, const float* d_bias, int M, int F, int K, void* d_H,
                        void* d_GU, void* stream) {
    DeviceCtx* ctx;
    TB_TRY(get_ctx(&ctx));
    TB_CHECK(d_X && d_W && d_H, "tb_gemm_swiglu_bf16: NULL operand");
    TB_CHECK(M > 0 && K > 0 && F > 0 && F % 64 == 0 && K % 8 == 0,
             "tb_gemm_swiglu_bf16: d_ff must be a multiple of 64 and K a multiple of 8 (got F=%d K=%d)", F, K);
    GemmArgs a;
    a.kind = GEMM_NN; a.A = d_X; a.B = d_W; a.M = M; a.N = 2 * F; a.K = K; a.lda = K; a.ldb = 2 * F;
    a.bias = d_bias; a.splits = 1;
    a.swiglu_h = static_cast<bf16*>(d_H); a.ldh = F;
    a.swiglu_gu = static_cast<bf16*>(d_GU); a.ldgu = 2 * F;
    return launch_gemm_bf16(ctx, a, S(stream));
}

int tb_gemm_qkv_rope_bf16(const void* d_X, const void* d_W, const float* d_bias, const float* d_cos, const float* d_sin,
                          int B, int T, int H, int hd, void* d_QKV, void* stream) {
    DeviceCtx* ctx;
    TB_TRY(get_ctx(&ctx));
    TB_CHECK(d_X && d_W && d_cos && d_sin && d_QKV, "tb_gemm_qkv_rope_bf16: NULL operand");
    TB_CHECK(B > 0 && T > 0 && H > 0 && (hd == 32 || hd == 64) && T % 32 == 0,
             "tb_gemm_qkv_rope_bf16: head_dim must be 32 or 64 and T a multiple of 32 (got T=%d hd=%d)", T, hd);
    TB_CHECK((reinterpret_cast<uintptr_t>(d_cos) & 15u) == 0 && (reinterpret_cast<uintptr_t>(d_sin) & 15u) == 0,
             "tb_gemm_qkv_rope_bf16: the angle tables must be 16-byte aligned");
    const int D = H * hd;
    GemmArgs a;
    a.kind = GEMM_NN; a.A = d_X; a.B = d_W; a.M = B * T; a.N = 3 * D; a.K = D; a.lda = D; a.ldb = 3 * D;
    a.bias = d_bias; a.splits = 1;
    a.rope_qkv = static_cast<bf16*>(d_QKV); a.rope_cos = d_cos; a.rope_sin = d_sin;
    a.rope_T = T; a.rope_H = H; a.rope_hd = hd;
    return launch_gemm_bf16(ctx, a, S(stream));
}

int tb_decode_linear(const void* d_X16, const float* d_x32, const float* d_norm_w, float eps, const void* d_W,
                     const float* d_bias, const float* d_residual, float* d_y32, void* d_h16, int S, int N, int K,
                     void* stream) {
    DeviceCtx* ctx;
    TB_TRY(get_ctx(&ctx));
    TB_CHECK(d_W != nullptr, "tb_decode_linear: NULL weight matrix");
    TB_CHECK(decode_linear_supported(S, N, K, d_h16 != nullptr),
             "tb_decode_linear: needs 1 <= S <= 64, K a multiple of 64 up to 1024, N a multiple of 128 (d_ff a multiple of 64 "
             "with the SwiGLU output); got S=%d N=%d K=%d -- use tb_gemm_bf16 for other shapes", S, N, K);
    return launch_decode_linear(ctx, static_cast<const bf16*>(d_X16), d_x32, d_norm_w, eps, static_cast<const bf16*>(d_W),
                                d_bias, d_residual, d_y32, static_cast<bf16*>(d_h16), S, N, K, static_cast<cudaStream_t>(stream));
}

int tb_lmhead_argmax_bf16(const void* d_X, const void* d_E, int n_seqs, int V, int K, uint32_t* d_tok, float* d_logits,
                          int64_t ld_logits, int table_is_stable, void* stream) {
    DeviceCtx* ctx;
    TB_TRY(get_ctx(&ctx));
    TB_CHECK(d_X && d_E && d_tok, "tb_lmhead_argmax_bf16: NULL operand");
    TB_CHECK(lmhead_argmax_supported(ctx, n_seqs, V, K),
             "tb_lmhead_argmax_bf16: needs 1 <= S <= 64 and K a multiple of 64 small enough for one slice of E per SM "
             "(got S=%d V=%d K=%d); use tb_gemm_bf16 for other shapes", n_seqs, V, K);
    TB_CHECK(d_logits == nullptr || ld_logits >= V, "tb_lmhead_argmax_bf16: ld_logits < V");
    return launch_lmhead_argmax(ctx, static_cast<const bf16*>(d_X), static_cast<const bf16*>(d_E), n_seqs, V, K,
                                table_is_stable != 0, ctx->d_best, ctx->d_tickets, d_tok, nullptr, nullptr, 0, 0,
                                d_logits, ld_logits, S(stream));
}

int tb_gemm_bf16(int kind, const void* d_A, const void* d_B, int M, int N, int K,
                 int64_t lda, int64_t ldb, int batch, int64_t strideA, int64_t strideB,
                 float* d_C32, int64_t ldc32, int64_t strideC32,
                 void* d_C16, int64_t ldc16, int64_t strideC16,
                 const float* d_bias, const float* d_residual, int64_t ldr, int64_t strideR,
                 float alpha, float beta, int causal, int splits, int tile_n, void* stream) {
    DeviceCtx* ctx;
    TB_TRY(get_ctx(&ctx));
    TB_CHECK(kind >= 0 && kind <= 2, "unknown GEMM kind %d", kind);
    TB_CHECK(causal >= 0 && causal <= 3, "unknown causal mode %d", causal);
    GemmArgs a;
    a.kind = static_cast<GemmKind>(kind);
    a.A = static_cast<const bf16*>(d_A); a.B = static_cast<const bf16*>(d_B);
    a.M = M; a.N = N; a.K = K; a.lda = lda; a.ldb = ldb;
    a.batch = batch; a.strideA = strideA; a.strideB = strideB;
    a.C32 = d_C32; a.ldc32 = ldc32; a.strideC32 = strideC32;
    a.C16 = static_cast<bf16*>(d_C16); a.ldc16 = ldc16; a.strideC16 = strideC16;
    a.bias = d_bias; a.residual = d_residual; a.ldr = ldr; a.strideR = strideR;
    a.alpha = alpha; a.beta = beta;
    a.causal = static_cast<CausalMode>(causal);
    a.splits = splits; a.bn = tile_n;
    return launch_gemm_bf16(ctx, a, S(stream));
}

int tb_attention_fwd(const void* d_Q, const void* d_K, const void* d_V, void* d_att, float* d_lse, int B, int H, int T,
                     int hd, float scale, void* stream) {
    DeviceCtx* ctx;
    TB_TRY(get_ctx(&ctx));
    return launch_attention_fwd(ctx, static_cast<const bf16*>(d_Q), static_cast<const bf16*>(d_K),
                                static_cast<const bf16*>(d_V), static_cast<bf16*>(d_att), d_lse, B, H, T, hd, scale,
                                S(stream));
}

int tb_attention_bwd(const void* d_Q, const void* d_K, const void* d_V, const void* d_att, const void* d_datt,
                     const float* d_lse, float* d_delta, float* d_dQ, float* d_dK, float* d_dV, int B, int H, int T,
                     int hd, float scale, void* stream) {
    DeviceCtx* ctx;
    TB_TRY(get_ctx(&ctx));
    return launch_attention_bwd(ctx, static_cast<const bf16*>(d_Q), static_cast<const bf16*>(d_K),
                                static_cast<const bf16*>(d_V), static_cast<const bf16*>(d_att),
                                static_cast<const bf16*>(d_datt), d_lse, d_delta, d_dQ, d_dK, d_dV, B, H, T, hd, scale,
                                S(stream));
}

// GEMM on float32 matrices in the reference's storage format.
//   BF16: both operands are packed to bf16 in scratch memory, then the bf16 GEMM runs;
//   TF32: the float32 operands go to the tensor cores as they are (kind::tf32 reads the top 19 bits);
//         an operand whose rows are not 16-byte addressable is first copied with a padded leading dimension;
//   FP32: each operand is split into tf32-exact pieces hi + lo and the product is evaluated as
//         hi*hi + hi*lo + lo*hi in one TF32 GEMM over a 3x longer K (error ~2^-20 of the result).
static inline bool tma_ok_f32(const float* p, long long ld, int batch, long long stride) {
    return (reinterpret_cast<uintptr_t>(p) & 15u) == 0 && ld % 4 == 0 && (batch == 1 || stride % 4 == 0);
}

static int gemm_f32_impl(int kind, const float* A, const float* B, float* C, int M, int N, int K,
                         long long lda, long long ldb, long long ldc, int batch, long long sA, long long sB,
                         long long sC, float alpha, float beta, const float* bias, const float* residual,
                         int precision, cudaStream_t stream) {
    DeviceCtx* ctx;
    TB_TRY(get_ctx(&ctx));
    TB_CHECK(kind >= 0 && kind <= 2, "unknown GEMM kind %d", kind);
    TB_CHECK(precision >= TB_PREC_BF16 && precision <= TB_PREC_FP32, "unknown precision %d", precision);
    TB_CHECK(M > 0 && N > 0 && K > 0 && batch > 0, "GEMM dims must be positive");
    // stored shapes
    const int a_rows = (kind == TB_GEMM_TN) ? K : M, a_cols = (kind == TB_GEMM_TN) ? M : K;
    const int b_rows = (kind == TB_GEMM_NT) ? N : K, b_cols = (kind == TB_GEMM_NT) ? K : N;

    GemmArgs g;
    g.kind = static_cast<GemmKind>(kind);
    g.M = M; g.N = N; g.K = K;
    g.batch = batch;
    g.C32 = C; g.ldc32 = ldc; g.strideC32 = sC;
    g.bias = bias; g.residual = residual; g.ldr = ldc; g.strideR = sC;
    g.alpha = alpha; g.beta = beta;

    if (precision == TB_PREC_BF16) {
        const long long a_ld = round_up(a_cols, 8), b_ld = round_up(b_cols, 8);
        const long long a_stride = (long long)a_rows * a_ld, b_stride = (long long)b_rows * b_ld;
        const size_t a_bytes = round_up((size_t)a_stride * batch * 2, 256);
        const size_t b_bytes = round_up((size_t)b_stride * batch * 2, 256);
        g.lda = a_ld; g.ldb = b_ld; g.strideA = a_stride; g.strideB = b_stride;
        const int splits = residual ? 1 : choose_splits(ctx, g, (N <= 64) ? 64 : 128);
        g.splits = splits;
        const size_t ws_floats = splits > 1 ? (size_t)splits * batch * M * N : 0;
        TB_TRY(ensure_scratch(ctx, a_bytes + b_bytes + ws_floats * sizeof(float)));
        bf16* pa = static_cast<bf16*>(ctx->scratch);
        bf16* pb = reinterpret_cast<bf16*>(static_cast<char*>(ctx->scratch) + a_bytes);
        float* ws = reinterpret_cast<float*>(static_cast<char*>(ctx->scratch) + a_bytes + b_bytes);
        TB_TRY(launch_pack_bf16(ctx, A, pa, a_rows, a_cols, lda, a_ld, batch, sA, a_stride, stream));
        TB_TRY(launch_pack_bf16(ctx, B, pb, b_rows, b_cols, ldb, b_ld, batch, sB, b_stride, stream));
        g.A = pa; g.B = pb;
        return launch_gemm_bf16_ws(ctx, g, ws, ws_floats, stream);
    }

    g.tf32 = true;
    const bool split3 = precision == TB_PREC_FP32;
    // shapes of the operands the TF32 GEMM sees
    const bool a_cat_cols = kind != TB_GEMM_TN;      // A stored [M,K]: the three pieces sit side by side
    const bool b_cat_cols = kind == TB_GEMM_NT;      // B stored [N,K]
    const int a_rows2 = split3 && !a_cat_cols ? 3 * a_rows : a_rows, a_cols2 = split3 && a_cat_cols ? 3 * a_cols : a_cols;
    const int b_rows2 = split3 && !b_cat_cols ? 3 * b_rows : b_rows, b_cols2 = split3 && b_cat_cols ? 3 * b_cols : b_cols;
    const bool a_inplace = !split3 && tma_ok_f32(A, lda, batch, sA);
    const bool b_inplace = !split3 && tma_ok_f32(B, ldb, batch, sB);
    const long long a_ld = a_inplace ? lda : round_up(a_cols2, 4), b_ld = b_inplace ? ldb : round_up(b_cols2, 4);
    const long long a_stride = a_inplace ? sA : (long long)a_rows2 * a_ld;
    const long long b_stride = b_inplace ? sB : (long long)b_rows2 * b_ld;
    const size_t a_bytes = a_inplace ? 0 : round_up((size_t)a_stride * batch * 4, 256);
    const size_t b_bytes = b_inplace ? 0 : round_up((size_t)b_stride * batch * 4, 256);
    if (split3) g.K = 3 * K;
    g.lda = a_ld; g.ldb = b_ld; g.strideA = a_stride; g.strideB = b_stride;
    const int splits = residual ? 1 : choose_splits(ctx, g, (N <= 64) ? 64 : 128);
    g.splits = splits;
    const size_t ws_floats = splits > 1 ? (size_t)splits * batch * M * N : 0;
    TB_TRY(ensure_scratch(ctx, a_bytes + b_bytes + ws_floats * sizeof(float)));
    float* pa = static_cast<float*>(ctx->scratch);
    float* pb = reinterpret_cast<float*>(static_cast<char*>(ctx->scratch) + a_bytes);
    float* ws = reinterpret_cast<float*>(static_cast<char*>(ctx->scratch) + a_bytes + b_bytes);
    if (split3) {
        TB_TRY(launch_split3_f32(ctx, A, pa, a_rows, a_cols, lda, a_ld, a_cat_cols ? 1 : 0, 0, batch, sA, a_stride, stream));
        TB_TRY(launch_split3_f32(ctx, B, pb, b_rows, b_cols, ldb, b_ld, b_cat_cols ? 1 : 0, 1, batch, sB, b_stride, stream));
    } else {
        if (!a_inplace) TB_TRY(launch_copy_f32(ctx, A, pa, a_rows, a_cols, lda, a_ld, batch, sA, a_stride, stream));
        if (!b_inplace) TB_TRY(launch_copy_f32(ctx, B, pb, b_rows, b_cols, ldb, b_ld, batch, sB, b_stride, stream));
    }
    g.A = a_inplace ? static_cast<const void*>(A) : pa;
    g.B = b_inplace ? static_cast<const void*>(B) : pb;
    return launch_gemm_bf16_ws(ctx, g, ws, ws_floats, stream);
}

int tb_gemm_f32(int kind, const float* d_A, const float* d_B, float* d_C,
                int M, int N, int K, int lda, int ldb, int ldc,
                int batch, int64_t strideA, int64_t strideB, int64_t strideC,
                float alpha, float beta, int precision, void* stream) {
    return gemm_f32_impl(kind, d_A, d_B, d_C, M, N, K, lda, ldb, ldc, batch, strideA, strideB, strideC, alpha, beta,
                         nullptr, nullptr, precision, S(stream));
}

int tb_gemm_bias_f32(const float* d_A, const float* d_B, const float* d_bias, const float* d_residual,
                     float* d_C, int M, int N, int K, int precision, void* stream) {
    return gemm_f32_impl(TB_GEMM_NN, d_A, d_B, d_C, M, N, K, K, N, N, 1, 0, 0, 0, 1.0f, 0.0f, d_bias, d_residual,
                         precision, S(stream));
}

// gpu_matmul keeps three growable device buffers per worker slot and reuses them from call to call
// (model/gpu_ops.c:31-46,118-160); the slot of a call is the calling thread's (gpu_ops_set_worker_id stores it in a
// thread-local, :100-102).  Here every host thread that calls tb_matmul_host owns one such slot per device: buffers
// grow on demand and live until the thread ends, so the steady state allocates nothing, and threads never share a
// slot (no lock on the data path, as the reference's worker slots).
namespace {
struct MatmulSlot {
    int device = -1;
    float *dA = nullptr, *dB = nullptr, *dC = nullptr;
    size_t capA = 0, capB = 0, capC = 0;
    ~MatmulSlot() {
        if (device < 0) return;
        int cur = -1;
        if (cudaGetDevice(&cur) != cudaSuccess) return;      // the runtime is already shutting down
        cudaSetDevice(device);
        cudaFree(dA); cudaFree(dB); cudaFree(dC);
        cudaSetDevice(cur);
    }
};
thread_local MatmulSlot t_slots[8];

int grow(float** p, size_t* cap, size_t need) {
    if (need <= *cap) return 0;
    if (*p) TB_CUDA(cudaFree(*p));
    *p = nullptr; *cap = 0;
    const size_t want = need + need / 4;
    TB_CUDA(cudaMalloc(p, want * sizeof(float)));
    *cap = want;
    return 0;
}
}  // namespace

int tb_matmul_host(const float* h_A, const float* h_B, float* h_C, int M, int K, int N, int precision) {
    DeviceCtx* ctx;
    TB_TRY(get_ctx(&ctx));
    TB_CHECK(M > 0 && N > 0 && K > 0, "matmul dims must be positive");
    const size_t na = (size_t)M * K, nb = (size_t)K * N, nc = (size_t)M * N;
    MatmulSlot* slot = nullptr;
    for (MatmulSlot& s : t_slots)
        if (s.device == ctx->device || s.device < 0) { slot = &s; break; }
    TB_CHECK(slot != nullptr, "tb_matmul_host: this thread already uses 8 devices");
    slot->device = ctx->device;
    TB_TRY(grow(&slot->dA, &slot->capA, na));
    TB_TRY(grow(&slot->dB, &slot->capB, nb));
    TB_TRY(grow(&slot->dC, &slot->capC, nc));
    TB_H2D_SYNC(slot->dA, h_A, na * 4);
    TB_H2D_SYNC(slot->dB, h_B, nb * 4);
    // the library scratch (operand packing, split-K partials) is one per device: calls of different threads take turns
    static std::mutex gemm_mutex;
    std::lock_guard<std::mutex> lock(gemm_mutex);
    TB_TRY(gemm_f32_impl(TB_GEMM_NN, slot->dA, slot->dB, slot->dC, M, N, K, K, N, N, 1, 0, 0, 0, 1.0f, 0.0f, nullptr,
                         nullptr, precision, nullptr));
    TB_TRY(check_device_error(ctx, nullptr));
    TB_CUDA(cudaMemcpy(h_C, slot->dC, nc * 4, cudaMemcpyDeviceToHost));
    return 0;
}

}  // extern "C"
