// Autoregressive decoding with a KV cache for the same decoder the trainer trains.
//
// The reference has no KV cache: it re-runs lm_forward over the whole window for every generated
// token (training/generate.c:186-212, training/chat.c:139-165).  This engine computes the same
// function -- the logits of the last position given all earlier tokens -- incrementally: the
// prompt is processed once (prefill: the trainer's forward kernels, K and V written straight into
// the cache), then each step feeds one new token per sequence through M = S skinny GEMMs, a
// rotary kernel that appends to the cache, and an attention kernel that reads the cache.
// Greedy choice (argmax of the last logits row) stays on the device; one decode step is a CUDA
// graph that reads the current position from device memory, so generating n tokens is n graph
// launches and one copy of the result.
#include "../../include/turkce_b200.h"
#include "common.h"
#include "step_kernels.h"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "pcg32.h"

using namespace tb;

namespace {
enum { PK_ATTN_NORM = 0, PK_WQKV, PK_BQKV, PK_WO, PK_BO, PK_FFN_NORM, PK_WGU, PK_BGU, PK_WDOWN, PK_BDOWN };
}

struct TbDecoder {
    DeviceCtx* ctx = nullptr;
    int device = 0;
    cudaStream_t stream = nullptr;
    int V = 0, D = 0, H = 0, L = 0, F = 0, hd = 0, S = 0, cap = 0;
    long long Vp = 0;
    float eps = 1e-5f, scale = 0.f;
    std::vector<long long> offsets;
    long long total = 0;
    float* params = nullptr; bf16* params16 = nullptr;
    std::vector<bf16*> Kc, Vc;                 // per layer [S, H, cap, hd]
    // activations sized for the prefill (S * cap rows) and reused by the decode step (S rows)
    float *x = nullptr, *x2 = nullptr, *qkv = nullptr, *gu = nullptr, *r = nullptr, *logits = nullptr, *xl = nullptr;
    float* qdec = nullptr;                     // [S, H, hd] rotated query of the decode step
    bf16 *n = nullptr, *att = nullptr, *h = nullptr, *Q = nullptr;
    uint32_t *ids = nullptr, *tok = nullptr, *out = nullptr;
    int* pos = nullptr;
    DecodeMega* mega = nullptr;                // decode step of all layers as one cooperative kernel (default when the shape fits)
    bool lean_step = false;                    // decode step on decode_linear_kernel (norm / SwiGLU / residual fused)
    bool fused_head = false;                   // LM head with the greedy choice fused (no logits in HBM)
    unsigned long long* head_best = nullptr;   // packed per-sequence maxima of the fused head (zero between launches)
    unsigned int* head_ticket = nullptr;
    int head_rows = 0;                         // rows of g->n the most recent head() normalised
    float *cos_t = nullptr, *sin_t = nullptr;
    uint32_t* h_pinned = nullptr;
    float* splitk_ws = nullptr; size_t splitk_floats = 0;
    int prompt_len = 0, generated = 0;
    float temperature = 0.f;                   // > 0: temperature sampling with the uniforms in sample_u
    double* sample_u = nullptr;                // [cap, S]: draw of sequence s for generated token i at i * S + s
    cudaGraphExec_t step_graph = nullptr;
    int step_state = 0;
    long long step_launches = 0;
    std::vector<void*> allocs;
};

namespace {

template <typename T>
int dalloc(TbDecoder* g, T** p, size_t count) {
    void* q = nullptr;
    TB_CUDA(cudaMalloc(&q, std::max<size_t>(count, 1) * sizeof(T)));
    g->allocs.push_back(q);
    *p = static_cast<T*>(q);
    return 0;
}

inline long long pidx(int layer, int k) { return 1 + 10LL * layer + k; }
inline float* P32(TbDecoder* g, long long i) { return g->params + g->offsets[i]; }
inline bf16* P16(TbDecoder* g, long long i) { return g->params16 + g->offsets[i]; }

// C[M,N] = A[M,K] @ W[K,N] + bias (+ residual), float32 out
int linear(TbDecoder* g, const bf16* A, const bf16* W, const float* bias, const float* residual, float* C, int M,
           int N, int K) {
    GemmArgs a;
    a.kind = GEMM_NN; a.A = A; a.B = W; a.M = M; a.N = N; a.K = K; a.lda = K; a.ldb = N;
    a.C32 = C; a.ldc32 = N; a.bias = bias; a.residual = residual; a.ldr = N;
    a.splits = 1;
    return launch_gemm_bf16_ws(g->ctx, a, g->splitk_ws, g->splitk_floats, g->stream);
}

// the rest of a layer after attention, and the head; rows = number of token rows in flight
int layer_tail(TbDecoder* g, int l, int rows) {
    DeviceCtx* c = g->ctx; cudaStream_t st = g->stream;
    const int D = g->D, F = g->F;
    TB_TRY(linear(g, g->att, P16(g, pidx(l, PK_WO)), P32(g, pidx(l, PK_BO)), g->x, g->x2, rows, D, D));
    TB_TRY(launch_rmsnorm_fwd(c, g->x2, P32(g, pidx(l, PK_FFN_NORM)), g->n, g->r, rows, D, g->eps, st));
    if (F % 64 == 0 && getenv("TB_NO_FUSED_SWIGLU") == nullptr) {
        GemmArgs s;       // h = silu(gate) * up in the projection's epilogue; gate|up themselves are not kept
        s.kind = GEMM_NN; s.A = g->n; s.B = P16(g, pidx(l, PK_WGU)); s.M = rows; s.N = 2 * F; s.K = D; s.lda = D;
        s.ldb = 2 * F; s.bias = P32(g, pidx(l, PK_BGU)); s.splits = 1; s.swiglu_h = g->h; s.ldh = F;
        TB_TRY(launch_gemm_bf16_ws(c, s, g->splitk_ws, g->splitk_floats, st));
    } else {
        TB_TRY(linear(g, g->n, P16(g, pidx(l, PK_WGU)), P32(g, pidx(l, PK_BGU)), nullptr, g->gu, rows, 2 * F, D));
        TB_TRY(launch_swiglu_fwd(c, g->gu, g->h, rows, F, st));
    }
    TB_TRY(linear(g, g->h, P16(g, pidx(l, PK_WDOWN)), P32(g, pidx(l, PK_BDOWN)), g->x2, g->x, rows, D, F));
    return 0;
}

// logits [rows, Vp] of the normalised rows in g->n (tied LM head)
int head_logits(TbDecoder* g, int rows) {
    GemmArgs a;
    a.kind = GEMM_NT; a.A = g->n; a.B = P16(g, 0); a.M = rows; a.N = g->V; a.K = g->D; a.lda = g->D; a.ldb = g->D;
    a.C32 = g->logits; a.ldc32 = g->Vp; a.splits = 1; a.pad_cols_writable = true;
    return launch_gemm_bf16_ws(g->ctx, a, g->splitk_ws, g->splitk_floats, g->stream);
}

// final norm of `rows` rows of src, tied LM head, greedy choice
int head(TbDecoder* g, const float* src, int rows, int advance_pos) {
    DeviceCtx* c = g->ctx; cudaStream_t st = g->stream;
    TB_TRY(launch_rmsnorm_fwd(c, src, P32(g, pidx(g->L, 0)), g->n, g->r, rows, g->D, g->eps, st));
    g->head_rows = rows;
    if (g->temperature > 0.f) {
        TB_TRY(head_logits(g, rows));
        return launch_sample_rows(c, g->logits, g->sample_u, g->temperature, g->tok, g->out, g->pos, rows, g->V, g->Vp,
                                  g->cap, advance_pos, st);
    }
    if (g->fused_head)
        return launch_lmhead_argmax(c, g->n, P16(g, 0), rows, g->V, g->D, true, g->head_best, g->head_ticket,
                                    g->tok, g->out, g->pos, g->cap, advance_pos, nullptr, 0, st);
    TB_TRY(head_logits(g, rows));
    return launch_argmax_rows(c, g->logits, g->tok, g->out, g->pos, rows, g->V, g->Vp, g->cap, advance_pos, st);
}

int decode_step_body(TbDecoder* g) {
    DeviceCtx* c = g->ctx; cudaStream_t st = g->stream;
    const int S = g->S, D = g->D, H = g->H, hd = g->hd;
    const bool split_rope = getenv("TB_DECODE_SPLIT_ROPE") != nullptr;    // the two-kernel form, for comparison
    if (g->mega) {
        // all layers in one cooperative kernel (embedding gather included), then the head as usual
        TB_TRY(launch_decode_mega(c, g->mega, g->tok, g->pos, g->cos_t, g->sin_t, g->x, g->x2, g->qkv, g->att, g->h, st));
        return head(g, g->x, S, 1);
    }
    TB_TRY(launch_embed_fwd(c, P32(g, 0), g->tok, g->x, S, D, st));
    for (int l = 0; l < g->L; ++l) {
        if (g->lean_step) {
            // five launches per layer: [RMSNorm + QKV] [rotary + cache append + attention] [out-projection + residual]
            // [RMSNorm + gate|up + SwiGLU] [down + residual]
            TB_TRY(launch_decode_linear(c, nullptr, g->x, P32(g, pidx(l, PK_ATTN_NORM)), g->eps, P16(g, pidx(l, PK_WQKV)),
                                        P32(g, pidx(l, PK_BQKV)), nullptr, g->qkv, nullptr, S, 3 * D, D, st));
            TB_TRY(launch_rope_attn_decode(c, g->qkv, g->cos_t, g->sin_t, g->Kc[l], g->Vc[l], g->att, g->pos, S, H, hd,
                                           g->cap, g->scale, st));
            TB_TRY(launch_decode_linear(c, g->att, nullptr, nullptr, 0.f, P16(g, pidx(l, PK_WO)), P32(g, pidx(l, PK_BO)),
                                        g->x, g->x2, nullptr, S, D, D, st));
            TB_TRY(launch_decode_linear(c, nullptr, g->x2, P32(g, pidx(l, PK_FFN_NORM)), g->eps, P16(g, pidx(l, PK_WGU)),
                                        P32(g, pidx(l, PK_BGU)), nullptr, nullptr, g->h, S, 2 * g->F, D, st));
            TB_TRY(launch_decode_linear(c, g->h, nullptr, nullptr, 0.f, P16(g, pidx(l, PK_WDOWN)), P32(g, pidx(l, PK_BDOWN)),
                                        g->x2, g->x, nullptr, S, D, g->F, st));
            continue;
        }
        TB_TRY(launch_rmsnorm_fwd(c, g->x, P32(g, pidx(l, PK_ATTN_NORM)), g->n, g->r, S, D, g->eps, st));
        TB_TRY(linear(g, g->n, P16(g, pidx(l, PK_WQKV)), P32(g, pidx(l, PK_BQKV)), nullptr, g->qkv, S, 3 * D, D));
        if (split_rope) {
            TB_TRY(launch_rope_decode(c, g->qkv, g->cos_t, g->sin_t, g->qdec, g->Kc[l], g->Vc[l], g->pos, S, H, hd, g->cap, st));
            TB_TRY(launch_attn_decode(c, g->qdec, g->Kc[l], g->Vc[l], g->att, g->pos, S, H, hd, g->cap, g->scale, st));
        } else {
            TB_TRY(launch_rope_attn_decode(c, g->qkv, g->cos_t, g->sin_t, g->Kc[l], g->Vc[l], g->att, g->pos, S, H, hd,
                                           g->cap, g->scale, st));
        }
        TB_TRY(layer_tail(g, l, S));
    }
    return head(g, g->x, S, 1);
}

}  // namespace

extern "C" {

int tb_decoder_create(TbDecoder** out, int V, int D, int H, int L, int F, int max_seqs, int max_len, float eps,
                      void* stream) {
    TB_CHECK(out != nullptr, "tb_decoder_create: out is NULL");
    TB_CHECK(V > 0 && D > 0 && H > 0 && L >= 0 && F > 0 && max_seqs > 0 && max_len > 1, "decoder dims must be positive");
    TB_CHECK(D % H == 0 && D % 8 == 0 && F % 8 == 0 && (D / H) % 8 == 0 && (D / H) <= 64,
             "d_model, d_ff, head_dim must be multiples of 8 and head_dim <= 64");
    TbDecoder* g = new TbDecoder();
    TB_TRY(get_ctx(&g->ctx));
    g->device = g->ctx->device;
    g->stream = static_cast<cudaStream_t>(stream);
    if (g->stream == nullptr) TB_CUDA(cudaStreamCreateWithFlags(&g->stream, cudaStreamNonBlocking));
    g->V = V; g->D = D; g->H = H; g->L = L; g->F = F; g->hd = D / H; g->S = max_seqs; g->cap = max_len;
    g->Vp = round_up(V, 8);
    g->eps = eps;
    g->scale = 1.0f / sqrtf((float)g->hd);
    auto push = [&](long long n) { g->offsets.push_back(g->total); g->total += n; };
    push((long long)V * D);
    for (int l = 0; l < L; ++l) {
        push(D); push((long long)D * 3 * D); push(3LL * D); push((long long)D * D); push(D);
        push(D); push((long long)D * 2 * F); push(2LL * F); push((long long)F * D); push(D);
    }
    push(D);
    const size_t S = max_seqs, N = S * (size_t)max_len;
    TB_TRY(dalloc(g, &g->params, g->total)); TB_TRY(dalloc(g, &g->params16, g->total));
    g->Kc.resize(L); g->Vc.resize(L);
    for (int l = 0; l < L; ++l) {
        TB_TRY(dalloc(g, &g->Kc[l], N * D)); TB_TRY(dalloc(g, &g->Vc[l], N * D));
        TB_CUDA(cudaMemset(g->Kc[l], 0, N * D * 2)); TB_CUDA(cudaMemset(g->Vc[l], 0, N * D * 2));
    }
    TB_TRY(dalloc(g, &g->x, N * D)); TB_TRY(dalloc(g, &g->x2, N * D)); TB_TRY(dalloc(g, &g->qkv, N * 3 * D));
    TB_TRY(dalloc(g, &g->gu, N * 2 * F)); TB_TRY(dalloc(g, &g->r, N)); TB_TRY(dalloc(g, &g->xl, S * D));
    TB_TRY(dalloc(g, &g->logits, S * g->Vp)); TB_TRY(dalloc(g, &g->qdec, S * D));
    g->fused_head = getenv("TB_NO_FUSED_LMHEAD") == nullptr && lmhead_argmax_supported(g->ctx, (int)S, V, D);
    // TB_DECODE_LEAN=1: the decode step on decode_linear_kernel (RMSNorm, SwiGLU and residual fused: 63 launches per
    // token instead of 87).  Off by default: it measures slower (640-700 against 572 us per step of 64 sequences); a
    // CTA that streams a whole 128-column slab by itself gets only 10-25 B/clk out of HBM, and the per-CTA RMSNorm
    // prologue (3 us on 8 warps) sits on the critical path.
    g->lean_step = getenv("TB_DECODE_LEAN") != nullptr && getenv("TB_DECODE_SPLIT_ROPE") == nullptr &&
                   decode_linear_supported((int)S, 3 * D, D, false) && decode_linear_supported((int)S, D, D, false) &&
                   decode_linear_supported((int)S, 2 * F, D, true) && decode_linear_supported((int)S, D, F, false) && D % 4 == 0;
    // One cooperative kernel for the layers of a decode step (TB_DECODE_NO_MEGA=1: the launch-per-kernel path)
    if (L > 0 && getenv("TB_DECODE_NO_MEGA") == nullptr && !g->lean_step &&
        decode_mega_supported(g->ctx, (int)S, D, H, F, max_len))
        TB_TRY(decode_mega_create(g->ctx, &g->mega, (int)S, D, H, F, L, max_len, eps, g->scale));
    if (g->fused_head) {
        TB_TRY(dalloc(g, &g->head_best, 64)); TB_CUDA(cudaMemset(g->head_best, 0, 64 * sizeof(unsigned long long)));
        TB_TRY(dalloc(g, &g->head_ticket, 1)); TB_CUDA(cudaMemset(g->head_ticket, 0, sizeof(unsigned int)));
    }
    TB_TRY(dalloc(g, &g->n, N * D)); TB_TRY(dalloc(g, &g->att, N * D)); TB_TRY(dalloc(g, &g->h, N * F));
    TB_TRY(dalloc(g, &g->Q, N * D));
    TB_TRY(dalloc(g, &g->ids, N)); TB_TRY(dalloc(g, &g->tok, S)); TB_TRY(dalloc(g, &g->out, N));
    TB_TRY(dalloc(g, &g->pos, 2));      // {position of the next token, tokens generated}
    g->splitk_floats = 4u << 20;
    TB_TRY(dalloc(g, &g->splitk_ws, g->splitk_floats));
    TB_CUDA(cudaMallocHost(&g->h_pinned, (N + 4) * 4));
    {
        const int half = g->hd / 2;
        std::vector<float> ct((size_t)max_len * half), sn((size_t)max_len * half);
        for (int p = 0; p < max_len; ++p)
            for (int k = 0; k < half; ++k) {
                const float theta = powf(10000.0f, -(2.0f * (float)k) / (float)g->hd);
                const float angle = (float)p * theta;
                ct[(size_t)p * half + k] = cosf(angle);
                sn[(size_t)p * half + k] = sinf(angle);
            }
        TB_TRY(dalloc(g, &g->cos_t, ct.size())); TB_TRY(dalloc(g, &g->sin_t, sn.size()));
        TB_H2D_SYNC(g->cos_t, ct.data(), ct.size() * 4);
        TB_H2D_SYNC(g->sin_t, sn.data(), sn.size() * 4);
    }
    *out = g;
    return 0;
}

int tb_decoder_destroy(TbDecoder* g) {
    if (!g) return 0;
    cudaDeviceSynchronize();
    if (g->step_graph) cudaGraphExecDestroy(g->step_graph);
    for (void* p : g->allocs) cudaFree(p);
    decode_mega_destroy(g->mega);
    cudaFreeHost(g->h_pinned);
    delete g;
    return 0;
}

int64_t tb_decoder_total_scalars(const TbDecoder* g) { return g->total; }

int tb_decoder_upload(TbDecoder* g, const float* h_flat) {
    TB_CUDA(cudaStreamSynchronize(g->stream));
    TB_H2D_SYNC(g->params, h_flat, (size_t)g->total * 4);
    TB_CHECK(g->total < (1LL << 31), "model too large for the single-row pack");
    TB_TRY(launch_pack_bf16(g->ctx, g->params, g->params16, 1, (int)g->total, g->total, g->total, 1, 0, 0, g->stream));
    if (g->mega)
        TB_TRY(decode_mega_set_weights(g->ctx, g->mega, g->params, g->params16, g->offsets.data(), g->Kc.data(), g->Vc.data(),
                                       g->stream));
    TB_CUDA(cudaStreamSynchronize(g->stream));
    return 0;
}

// Processes the prompts (S sequences x prompt_len tokens, row-major), fills the KV cache and
// chooses the first new token of every sequence.
int tb_decoder_prefill(TbDecoder* g, const uint32_t* h_ids, int prompt_len) {
    TB_CUDA(cudaSetDevice(g->device));
    TB_CHECK(prompt_len >= 1 && prompt_len < g->cap, "prompt length %d must be in [1, %d)", prompt_len, g->cap);
    DeviceCtx* c = g->ctx; cudaStream_t st = g->stream;
    const int S = g->S, T = prompt_len, N = S * T, D = g->D, H = g->H, hd = g->hd;
    for (int i = 0; i < N; ++i) TB_CHECK(h_ids[i] < (uint32_t)g->V, "token id out of range at position %d", i);
    std::memcpy(g->h_pinned, h_ids, (size_t)N * 4);
    TB_CUDA(cudaMemcpyAsync(g->ids, g->h_pinned, (size_t)N * 4, cudaMemcpyHostToDevice, st));
    g->prompt_len = T; g->generated = 0;
    int* h_state = reinterpret_cast<int*>(g->h_pinned + N);
    h_state[0] = T; h_state[1] = 0;
    TB_CUDA(cudaMemcpyAsync(g->pos, h_state, 2 * sizeof(int), cudaMemcpyHostToDevice, st));
    TB_TRY(launch_embed_fwd(c, P32(g, 0), g->ids, g->x, N, D, st));
    for (int l = 0; l < g->L; ++l) {
        TB_TRY(launch_rmsnorm_fwd(c, g->x, P32(g, pidx(l, PK_ATTN_NORM)), g->n, g->r, N, D, g->eps, st));
        TB_TRY(linear(g, g->n, P16(g, pidx(l, PK_WQKV)), P32(g, pidx(l, PK_BQKV)), nullptr, g->qkv, N, 3 * D, D));
        TB_TRY(launch_rope_split(c, g->qkv, g->cos_t, g->sin_t, g->Q, g->Kc[l], g->Vc[l], S, T, H, hd, g->cap, st));
        TB_TRY(launch_attention_fwd(c, g->Q, g->Kc[l], g->Vc[l], g->att, nullptr, S, H, T, hd, g->scale, st, g->cap));
        TB_TRY(layer_tail(g, l, N));
    }
    TB_TRY(launch_gather_last_rows(c, g->x, g->xl, S, T, D, st));
    // the first generated token sits at position prompt_len; *pos stays there for the first decode step
    TB_TRY(head(g, g->xl, S, 0));
    g->generated = 1;
    return 0;
}

int tb_decoder_set_sampling(TbDecoder* g, float temperature, uint64_t seed, uint64_t seq) {
    TB_CHECK(g, "tb_decoder_set_sampling: null decoder");
    TB_CUDA(cudaSetDevice(g->device));
    TB_CUDA(cudaStreamSynchronize(g->stream));
    if (g->step_graph) {                       // the captured step holds the other head: capture again
        cudaGraphExecDestroy(g->step_graph);
        g->step_graph = nullptr;
    }
    g->step_state = 0;
    g->temperature = temperature > 0.f ? temperature : 0.f;
    if (g->temperature > 0.f) {
        if (!g->sample_u) TB_TRY(dalloc(g, &g->sample_u, (size_t)g->cap * g->S));
        TB_CHECK(g->logits, "tb_decoder_set_sampling: this decoder was created without a logits buffer");
        std::vector<double> u((size_t)g->cap * g->S);
        for (int s = 0; s < g->S; ++s) {
            Pcg32 rng(seed, seq + (uint64_t)s);
            for (int i = 0; i < g->cap; ++i) u[(size_t)i * g->S + s] = rng.uniform();
        }
        TB_H2D_SYNC(g->sample_u, u.data(), u.size() * sizeof(double));
    }
    return 0;
}

// Generates n more tokens per sequence (greedy or sampled); the tokens stay on the device until read.
int tb_decoder_generate(TbDecoder* g, int n) {
    TB_CUDA(cudaSetDevice(g->device));
    TB_CHECK(g->generated >= 1, "tb_decoder_generate: call tb_decoder_prefill first");
    TB_CHECK(g->prompt_len + g->generated + n <= g->cap + 1, "cache capacity %d exceeded", g->cap);
    // (with the one-kernel step there are three launches per token: nothing for a graph to save)
    const bool use_graph = getenv("TB_NO_GRAPH") == nullptr && !g->ctx->prof_on && g->mega == nullptr;
    for (int i = 0; i < n; ++i) {
        if (!use_graph || g->step_state == 0) {
            TB_TRY(decode_step_body(g));
            if (use_graph) g->step_state = 1;
        } else if (g->step_state == 1) {
            const long long before = g->ctx->launches;
            TB_CUDA(cudaStreamBeginCapture(g->stream, cudaStreamCaptureModeRelaxed));
            const int rc = decode_step_body(g);
            cudaGraph_t graph = nullptr;
            const cudaError_t e = cudaStreamEndCapture(g->stream, &graph);
            if (rc != 0) { if (graph) cudaGraphDestroy(graph); return rc; }
            TB_CUDA(e);
            g->step_launches = g->ctx->launches - before;
            TB_CUDA(cudaGraphInstantiate(&g->step_graph, graph, 0));
            cudaGraphDestroy(graph);
            g->step_state = 2;
            TB_CUDA(cudaGraphLaunch(g->step_graph, g->stream));
        } else {
            TB_CUDA(cudaGraphLaunch(g->step_graph, g->stream));
            g->ctx->launches += g->step_launches;
        }
        g->generated++;
    }
    return 0;
}

// Copies the generated tokens [S, count] (count = tokens generated so far) to the host.
int tb_decoder_read_tokens(TbDecoder* g, uint32_t* h_out, int count) {
    TB_CHECK(count >= 0 && count <= g->generated, "only %d tokens have been generated", g->generated);
    TB_TRY(check_device_error(g->ctx, g->stream));
    std::vector<uint32_t> tmp((size_t)g->S * g->cap);
    TB_CUDA(cudaMemcpy(tmp.data(), g->out, tmp.size() * 4, cudaMemcpyDeviceToHost));
    for (int s = 0; s < g->S; ++s)
        for (int i = 0; i < count; ++i) h_out[(size_t)s * count + i] = tmp[(size_t)s * g->cap + i];
    return 0;
}

// Logits [S, V] of the most recent step (for parity tests).  The fused head never stores them:
// they are formed here, on request, from the step's normalised hidden states.
int tb_decoder_read_logits(TbDecoder* g, float* h_logits) {
    TB_CHECK(g->head_rows > 0, "tb_decoder_read_logits: no step has run yet");
    if (g->fused_head) TB_TRY(head_logits(g, g->head_rows));
    TB_CUDA(cudaStreamSynchronize(g->stream));
    TB_TRY(check_device_error(g->ctx, g->stream));
    std::vector<float> tmp((size_t)g->S * g->Vp);
    TB_CUDA(cudaMemcpy(tmp.data(), g->logits, tmp.size() * 4, cudaMemcpyDeviceToHost));
    for (int s = 0; s < g->S; ++s) std::memcpy(h_logits + (size_t)s * g->V, tmp.data() + (size_t)s * g->Vp, (size_t)g->V * 4);
    return 0;
}

void* tb_decoder_stream(TbDecoder* g) { return g->stream; }

}  // extern "C"
