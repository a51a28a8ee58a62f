// GPU-resident trainer: the whole decoder's forward, backward and Adam on one device, with
// the schedule and the flat parameter layout of the reference's GpuTrainer
// (model/gpu_train.c:144-529, model/gpu_train.h:33-125) and this library's kernels underneath.
//
// Differences from the reference that do not change the function computed:
//  * every GEMM operand lives in bf16 in HBM (weights as a shadow copy refreshed by Adam,
//    activations written in bf16 by the kernel that produces them), so the tensor cores read
//    through TMA with no conversion pass; residual stream, logits, gradients and Adam state
//    stay float32;
//  * the weight-gradient (TN) GEMMs run on tensor cores with deterministic split-K instead of
//    the reference's FP32 SIMT kernel;
//  * attention skips the masked upper triangle (exact: the reference's -1e9 mask underflows to
//    0 after exp) and P*V writes the merged [B*T, D] layout directly;
//  * the gradient norm and clip factor are reduced on the device, so a full training step
//    needs one host read (the loss rows) instead of three.
#include "../../include/turkce_b200.h"
#include "common.h"
#include "step_kernels.h"
#include "trainer_internal.h"

#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <vector>

using namespace tb;

namespace {

enum { PK_ATTN_NORM = 0, PK_WQKV, PK_BQKV, PK_WO, PK_BO, PK_FFN_NORM, PK_WGU, PK_BGU, PK_WDOWN, PK_BDOWN };

struct LayerActs {
    float *n1_32 = nullptr, *n2_32 = nullptr, *h32 = nullptr;    // TF32 mode: float32 GEMM operands
    float* x_in;  bf16* n1; float* r1;
    bf16 *Q, *K, *V, *P, *att;     // P [BH,T,T] only on the unfused attention path
    float* lse;                    // [BH,T] on the fused path
    float* x2;    bf16* n2; float* r2;
    float* gu;    bf16* h;   // gu: gate|up projection (unfused SwiGLU path)
    bf16* gu16;              // gate|up in bf16, written by the fused SwiGLU GEMM epilogue
};

}  // namespace

struct TbTrainer {
    DeviceCtx* ctx = nullptr;
    int device = 0;
    cudaStream_t stream = nullptr;
    int V = 0, D = 0, H = 0, L = 0, F = 0, T = 0, B = 0, N = 0, hd = 0;
    long long Vp = 0;   // logits leading dimension (V rounded up to 8)
    long long Tp = 0;   // score-matrix leading dimension (T rounded up to 8)
    float eps = 1e-5f;
    float scale = 0.f;

    std::vector<long long> offsets, numels;
    long long total = 0, padded = 0;
    float *params = nullptr, *grads = nullptr, *adam_m = nullptr, *adam_v = nullptr;
    bf16* params16 = nullptr;

    std::vector<LayerActs> layers;
    float* x_final = nullptr; bf16* nf = nullptr; float* rf = nullptr;
    float* logits = nullptr; bf16* dlogits = nullptr;   // logits only exist without the fused cross-entropy
    float *ce_stats = nullptr, *ce_zt = nullptr, *ce_lse = nullptr;

    float *qkv = nullptr, *S = nullptr, *dP = nullptr, *dn = nullptr, *dres = nullptr, *wtmp = nullptr, *dh = nullptr;
    float *dQ = nullptr, *dK = nullptr, *dV = nullptr;
    bf16 *dres16 = nullptr, *dgu = nullptr, *datt = nullptr, *dO = nullptr, *dS = nullptr, *dqkv = nullptr;
    float* colsum_partial = nullptr;
    float* colsum_partial2 = nullptr;       // for the column sum that runs on the weight gradients' stream
    float* norm_scratch = nullptr;
    float* swiglu_scratch = nullptr;
    float* splitk_ws = nullptr; size_t splitk_floats = 0;

    uint32_t *ids = nullptr, *targets = nullptr;
    uint32_t *order = nullptr, *seg_start = nullptr, *seg_token = nullptr, *seg_meta = nullptr;   // one buffer
    float* embed_partial = nullptr;
    unsigned int* embed_tickets = nullptr;
    float *loss_rows = nullptr, *cos_t = nullptr, *sin_t = nullptr;
    float* norm_partial = nullptr; float* scalars = nullptr; double* norm64 = nullptr;

    // pinned host staging
    uint32_t *h_ids = nullptr, *h_targets = nullptr, *h_seg = nullptr;
    float* h_loss_rows = nullptr; double* h_norm = nullptr;
    cudaEvent_t staged = nullptr; bool staged_pending = false;   // behind the last copy out of the pinned buffers
    int nseg = 0;
    uint32_t* nseg_dev = nullptr;
    std::vector<void*> allocs;

    // CUDA graphs: each segment of the step (forward, head backward, one layer's backward, ...) is
    // run eagerly once, captured on its second use and replayed afterwards.
    struct Segment { int state = 0; cudaGraphExec_t exec = nullptr; long long launches = 0; };
    std::vector<Segment> segments;
    bool graphs_on = true;
    bool fused_attention = true;   // head_dim <= 64: scores stay on chip
    bool fused_rope = true;        // T % 32 == 0, head_dim 32 or 64: rotation and head split in the QKV GEMM epilogue
    bool fused_ce = true;          // cross-entropy inside the LM-head GEMM epilogues: no [N, V] logits
    bool fused_dswiglu = false;    // SwiGLU backward in the epilogue of the down-projection's input-gradient GEMM
    bool fused_swiglu = true;      // d_ff % 64 == 0: silu(gate) * up formed in the gate|up GEMM's epilogue
    // TF32 mode (TB_PREC_TF32): every linear-layer GEMM (forward, dX, dW, LM head) reads float32 operands as tf32
    // (kind::tf32); weights are the float32 masters, activations and gradients that feed a GEMM are kept in float32.
    // The attention core stays the fused bf16 kernel (the reference's attention products are bf16 as well);
    // its outputs are widened.  The fused epilogues are those of the bf16 path and are switched off here.
    bool tf32 = false;
    float *nf32 = nullptr, *dlogits32 = nullptr, *dgu32 = nullptr, *dqkv32 = nullptr, *att32 = nullptr;
    float* att_delta = nullptr;
    bf16* att_ds = nullptr;        // dS blocks on their way from the dK/dV kernel to the dQ kernel
    bool owns_stream = false;
    // The weight-gradient product of a linear layer and its input-gradient product read the same dY and depend on
    // nothing of each other: they run side by side, the first on a second stream, each on half of the SMs.  (Measured
    // per pair in a graph, M = 8192: 29.3 -> 23.0, 19.2 -> 14.7, 46.3 -> 42.1, 29.3 -> 23.5 us; without the cap on the
    // CTAs the two persistent kernels only take each other's SMs and nothing is gained.)
    cudaStream_t side = nullptr;
    cudaEvent_t ev_fork = nullptr, ev_done[4] = {nullptr, nullptr, nullptr, nullptr};   // after each of a layer's four dW
    int pair_ctas = 0;             // CTAs per product of such a pair; 0 = one after the other
    int pair_ctas_down = 0;        // CTAs of the down-projection's input-gradient product when it carries SwiGLU backward
    cudaEvent_t ev_zero = nullptr; bool zero_pending = false;     // the gradient buffer is being cleared on `side`
};

namespace {

template <typename T>
int dalloc(TbTrainer* g, T** p, size_t count) {
    void* q = nullptr;
    TB_CUDA(cudaMalloc(&q, std::max<size_t>(count, 1) * sizeof(T)));
    g->allocs.push_back(q);
    *p = static_cast<T*>(q);
    return 0;
}

constexpr int kCeTile = 256;      // tile width of the LM-head products with the fused cross-entropy (a CTA pair)

inline long long pidx(int layer, int k) { return 1 + 10LL * layer + k; }
inline float* P32(TbTrainer* g, long long i) { return g->params + g->offsets[i]; }
inline bf16* P16(TbTrainer* g, long long i) { return g->params16 + g->offsets[i]; }
inline float* G32(TbTrainer* g, long long i) { return g->grads + g->offsets[i]; }

int gemm(TbTrainer* g, GemmArgs& a) {
    return launch_gemm_bf16_ws(g->ctx, a, g->splitk_ws, g->splitk_floats, g->stream);
}

// side-by-side pairs are off while every launch is timed (the events assume one stream)
inline bool pair_on(const TbTrainer* g) { return g->pair_ctas > 0 && !g->ctx->prof_on; }

// C[M,N] = A[M,K] @ W[K,N] + bias (+ residual): the reference's bf16_gemm_bias (gpu_train.c:103-107).
// Operands are bf16, or float32 read as tf32 in the TF32 mode.
int linear_fwd(TbTrainer* g, const void* A, const void* W, const float* bias, const float* residual, float* C32,
               bf16* C16, int M, int N, int K) {
    GemmArgs a;
    a.kind = GEMM_NN; a.A = A; a.B = W; a.M = M; a.N = N; a.K = K; a.lda = K; a.ldb = N;
    a.C32 = C32; a.ldc32 = N; a.C16 = C16; a.ldc16 = N;
    a.bias = bias; a.residual = residual; a.ldr = N;
    a.splits = 1; a.tf32 = g->tf32;
    return gemm(g, a);
}

// dX[M,K] = dY[M,N] @ W[K,N]^T : the reference's bf16_gemm1(GEMM_NT) (gpu_train.c:419,427,434,463)
int linear_dx(TbTrainer* g, const void* dY, const void* W, float* dX32, bf16* dX16, int M, int N, int K) {
    GemmArgs a;
    a.kind = GEMM_NT; a.A = dY; a.B = W; a.M = M; a.N = K; a.K = N; a.lda = N; a.ldb = N;
    a.C32 = dX32; a.ldc32 = K; a.C16 = dX16; a.ldc16 = K;
    a.splits = 1; a.tf32 = g->tf32;
    if (pair_on(g)) a.max_ctas = g->pair_ctas;
    return gemm(g, a);
}

// dW[K,N] += X[M,K]^T @ dY[M,N] : the reference's gemm1(GEMM_TN, beta=1) (gpu_train.c:417,425,432,461)
// Issued on the second stream when the pair runs side by side (linear_dx follows on the main stream); which = 0..3
// numbers the layer's four weight gradients (down, gate|up, out, qkv).  The main stream does not wait at once: the
// memory-bound kernels that follow the input-gradient product run beside the tail of the weight-gradient product,
// and pair_wait(which) stands in front of the first kernel that overwrites an operand of that product.
// The split-K workspace is the weight gradients' alone (they are in order on their stream); no other product of the
// step splits K.
int linear_dw(TbTrainer* g, const void* X, const void* dY, float* dW, int M, int N, int K, int which) {
    GemmArgs a;
    a.kind = GEMM_TN; a.A = X; a.B = dY; a.M = K; a.N = N; a.K = M; a.lda = K; a.ldb = N;
    a.C32 = dW; a.ldc32 = N; a.beta = 1.0f;
    a.splits = 0; a.tf32 = g->tf32;
    if (!pair_on(g)) return gemm(g, a);
    a.max_ctas = g->ctx->sm_count - ((which == 0 && g->fused_dswiglu) ? g->pair_ctas_down : g->pair_ctas);
    TB_CUDA(cudaEventRecord(g->ev_fork, g->stream));
    TB_CUDA(cudaStreamWaitEvent(g->side, g->ev_fork, 0));
    TB_TRY(launch_gemm_bf16_ws(g->ctx, a, g->splitk_ws, g->splitk_floats, g->side));
    TB_CUDA(cudaEventRecord(g->ev_done[which], g->side));
    return 0;
}
// everything the main stream launches from here on comes after weight-gradient product `which` of this layer
int pair_wait(TbTrainer* g, int which) {
    if (!pair_on(g)) return 0;
    TB_CUDA(cudaStreamWaitEvent(g->stream, g->ev_done[which], 0));
    return 0;
}

// the weight matrix of parameter i as a GEMM operand: the bf16 shadow, or the float32 master in the TF32 mode
inline const void* WOP(TbTrainer* g, long long i) {
    return g->tf32 ? static_cast<const void*>(P32(g, i)) : static_cast<const void*>(P16(g, i));
}

int forward(TbTrainer* g, bool want_grad) {
    DeviceCtx* c = g->ctx;
    cudaStream_t st = g->stream;
    const int N = g->N, D = g->D, F = g->F, T = g->T, V = g->V, H = g->H, hd = g->hd, B = g->B;
    const int BH = B * H;
    const long long Tp = g->Tp, sTT = (long long)T * Tp, sThd = (long long)T * hd;

    float* x0 = g->L > 0 ? g->layers[0].x_in : g->x_final;
    TB_TRY(launch_embed_fwd(c, P32(g, 0), g->ids, x0, N, D, st));

    for (int l = 0; l < g->L; ++l) {
        LayerActs& a = g->layers[l];
        float* x_out = (l + 1 < g->L) ? g->layers[l + 1].x_in : g->x_final;
        TB_TRY(launch_rmsnorm_fwd(c, a.x_in, P32(g, pidx(l, PK_ATTN_NORM)), a.n1, a.r1, N, D, g->eps, st, a.n1_32));
        if (g->fused_rope) {
            // QKV projection; q and k rotated and all three stored per head as bf16 by the GEMM epilogue
            GemmArgs s;
            s.kind = GEMM_NN; s.A = a.n1; s.B = P16(g, pidx(l, PK_WQKV)); s.M = N; s.N = 3 * D; s.K = D; s.lda = D;
            s.ldb = 3 * D; s.bias = P32(g, pidx(l, PK_BQKV)); s.splits = 1;
            s.rope_qkv = a.Q; s.rope_cos = g->cos_t; s.rope_sin = g->sin_t; s.rope_T = T; s.rope_H = H; s.rope_hd = hd;
            if (const char* e = getenv("TB_ROPE_BN")) s.bn = atoi(e);
            TB_TRY(gemm(g, s));
        } else {
            TB_TRY(linear_fwd(g, g->tf32 ? (const void*)a.n1_32 : (const void*)a.n1, WOP(g, pidx(l, PK_WQKV)),
                              P32(g, pidx(l, PK_BQKV)), nullptr, g->qkv, nullptr, N, 3 * D, D));
            TB_TRY(launch_rope_split(c, g->qkv, g->cos_t, g->sin_t, a.Q, a.K, a.V, B, T, H, hd, T, st));
        }
        if (g->fused_attention) {
            TB_TRY(launch_attention_fwd(c, a.Q, a.K, a.V, a.att, a.lse, B, H, T, hd, g->scale, st));
        } else {
            {   // S = Q K^T per (batch, head), lower-triangular tiles only
                GemmArgs s;
                s.kind = GEMM_NT; s.A = a.Q; s.B = a.K; s.M = T; s.N = T; s.K = hd; s.lda = hd; s.ldb = hd;
                s.batch = BH; s.strideA = sThd; s.strideB = sThd;
                s.C32 = g->S; s.ldc32 = Tp; s.strideC32 = sTT;
                s.causal = CAUSAL_SKIP_UPPER; s.splits = 1;
                TB_TRY(gemm(g, s));
            }
            TB_TRY(launch_attn_softmax_fwd(c, g->S, a.P, BH, T, Tp, g->scale, st));
            {   // att[b*T+t, h*hd+d] = sum_j P[j] V[j,d], written straight into the merged layout
                GemmArgs o;
                o.kind = GEMM_NN; o.A = a.P; o.B = a.V; o.M = T; o.N = hd; o.K = T; o.lda = Tp; o.ldb = hd;
                o.batch = BH; o.strideA = sTT; o.strideB = sThd;
                o.C16 = a.att; o.ldc16 = D; o.c_inner = H; o.strideC16 = (long long)T * D; o.strideC16_in = hd;
                o.causal = CAUSAL_K_PREFIX; o.splits = 1;
                TB_TRY(gemm(g, o));
            }
        }
        if (g->tf32) TB_TRY(launch_widen_bf16(c, a.att, g->att32, (long long)N * D, st));
        TB_TRY(linear_fwd(g, g->tf32 ? (const void*)g->att32 : (const void*)a.att, WOP(g, pidx(l, PK_WO)),
                          P32(g, pidx(l, PK_BO)), a.x_in, a.x2, nullptr, N, D, D));
        TB_TRY(launch_rmsnorm_fwd(c, a.x2, P32(g, pidx(l, PK_FFN_NORM)), a.n2, a.r2, N, D, g->eps, st, a.n2_32));
        if (g->fused_swiglu) {
            // gate|up projection with h = silu(gate) * up formed in the GEMM epilogue; gate|up kept in bf16
            GemmArgs s;
            s.kind = GEMM_NN; s.A = a.n2; s.B = P16(g, pidx(l, PK_WGU)); s.M = N; s.N = 2 * F; s.K = D; s.lda = D;
            s.ldb = 2 * F; s.bias = P32(g, pidx(l, PK_BGU)); s.splits = 1;
            s.swiglu_h = a.h; s.ldh = F; s.swiglu_gu = a.gu16; s.ldgu = 2 * F;
            TB_TRY(gemm(g, s));
        } else {
            TB_TRY(linear_fwd(g, g->tf32 ? (const void*)a.n2_32 : (const void*)a.n2, WOP(g, pidx(l, PK_WGU)),
                              P32(g, pidx(l, PK_BGU)), nullptr, a.gu, nullptr, N, 2 * F, D));
            TB_TRY(launch_swiglu_fwd(c, a.gu, g->tf32 ? nullptr : a.h, N, F, st, a.h32));
        }
        TB_TRY(linear_fwd(g, g->tf32 ? (const void*)a.h32 : (const void*)a.h, WOP(g, pidx(l, PK_WDOWN)),
                          P32(g, pidx(l, PK_BDOWN)), a.x2, x_out, nullptr, N, D, F));
    }

    const long long p_final = pidx(g->L, 0);
    TB_TRY(launch_rmsnorm_fwd(c, g->x_final, P32(g, p_final), g->nf, g->rf, N, D, g->eps, st, g->nf32));
    if (g->fused_ce) {
        // logits = nf @ E^T (tied head, gpu_train.c:378) never reach HBM: pass 1 keeps per-tile softmax
        // statistics and the target logit, their combination is the loss; pass 2 forms the product again
        // and stores (softmax - onehot) / N directly (gpu_train.c:381)
        GemmArgs a;
        a.kind = GEMM_NT; a.A = g->nf; a.B = P16(g, 0); a.M = N; a.N = V; a.K = D; a.lda = D; a.ldb = D;
        a.splits = 1; a.bn = kCeTile; a.ce_targets = g->targets;
        GemmArgs s1 = a;
        s1.ce_mode = 1; s1.ce_stats = g->ce_stats; s1.ce_ztarget = g->ce_zt;
        TB_TRY(gemm(g, s1));
        TB_TRY(launch_ce_combine(c, g->ce_stats, 2 * ((V + kCeTile - 1) / kCeTile), N, g->ce_zt, g->ce_lse, g->loss_rows, st));
        if (want_grad) {
            GemmArgs s2 = a;
            s2.ce_mode = 2; s2.ce_lse = g->ce_lse; s2.ce_scale = 1.0f / (float)N;
            s2.C16 = g->dlogits; s2.ldc16 = g->Vp; s2.pad_cols_writable = true;
            TB_TRY(gemm(g, s2));
        }
        return 0;
    }
    {   // logits = nf @ E^T (tied head): gpu_train.c:378
        GemmArgs a;
        a.kind = GEMM_NT; a.A = g->tf32 ? (const void*)g->nf32 : (const void*)g->nf; a.B = WOP(g, 0);
        a.M = N; a.N = V; a.K = D; a.lda = D; a.ldb = D; a.tf32 = g->tf32;
        a.C32 = g->logits; a.ldc32 = g->Vp; a.splits = 1; a.pad_cols_writable = true;
        TB_TRY(gemm(g, a));
    }
    TB_TRY(launch_cross_entropy(c, g->logits, g->targets, g->loss_rows, (want_grad && !g->tf32) ? g->dlogits : nullptr, N, V,
                                g->Vp, 1.0f / (float)N, st, (want_grad && g->tf32) ? g->dlogits32 : nullptr));
    return 0;
}

int backward_head(TbTrainer* g) {
    DeviceCtx* c = g->ctx;
    cudaStream_t st = g->stream;
    const int N = g->N, D = g->D, V = g->V;
    const long long p_final = pidx(g->L, 0);
    {   // dE += dlogits^T @ nf  (gpu_train.c:403)
        GemmArgs a;
        a.kind = GEMM_TN; a.A = g->tf32 ? (const void*)g->dlogits32 : (const void*)g->dlogits;
        a.B = g->tf32 ? (const void*)g->nf32 : (const void*)g->nf; a.tf32 = g->tf32;
        a.M = V; a.N = D; a.K = N; a.lda = g->Vp; a.ldb = D;
        a.C32 = G32(g, 0); a.ldc32 = D; a.beta = 1.0f; a.splits = 1;
        TB_TRY(gemm(g, a));
    }
    {   // dnf = dlogits @ E  (gpu_train.c:404)
        GemmArgs a;
        a.kind = GEMM_NN; a.A = g->tf32 ? (const void*)g->dlogits32 : (const void*)g->dlogits; a.B = WOP(g, 0);
        a.tf32 = g->tf32; a.M = N; a.N = D; a.K = V; a.lda = g->Vp; a.ldb = D;
        a.C32 = g->dn; a.ldc32 = D; a.splits = 0;         // (two splits on 256 x 384 pair tiles when D <= 384, else one)
        TB_TRY(gemm(g, a));
    }
    // dres (the gradient of the last layer's output) also yields that layer's b_down gradient
    TB_TRY(launch_rmsnorm_bwd_dw(c, g->x_final, P32(g, p_final), g->rf, g->dn, g->dres, g->dres16, G32(g, p_final),
                                 g->L > 0 ? G32(g, pidx(g->L - 1, PK_BDOWN)) : nullptr, g->norm_scratch, N, D, 0, st));
    return 0;
}

int backward_layer(TbTrainer* g, int l) {
    DeviceCtx* c = g->ctx;
    cudaStream_t st = g->stream;
    const int N = g->N, D = g->D, F = g->F, T = g->T, H = g->H, hd = g->hd, B = g->B;
    const int BH = B * H;
    const long long Tp = g->Tp, sTT = (long long)T * Tp, sThd = (long long)T * hd;
    LayerActs& a = g->layers[l];

    // the gradient of the residual stream as a GEMM operand: bf16 copy, or the float32 buffer itself (TF32 mode)
    const void* dres_op = g->tf32 ? (const void*)g->dres : (const void*)g->dres16;
    // ---- FFN: x3 = x2 + (h @ Wd + bd); dres = dx3
    TB_TRY(linear_dw(g, g->tf32 ? (const void*)a.h32 : (const void*)a.h, dres_op, G32(g, pidx(l, PK_WDOWN)), N, D, F, 0));
    // (b_down's gradient, the column sum of dres, was produced together with dres)
    if (g->fused_dswiglu) {
        // dh = dres @ Wd^T never reaches HBM: the product's epilogue turns each tile into dgu with the saved gate|up
        // projection; the gate|up bias gradient (the column sums of dgu) is taken beside the next products
        GemmArgs x;
        x.kind = GEMM_NT; x.A = g->dres16; x.B = WOP(g, pidx(l, PK_WDOWN)); x.M = N; x.N = F; x.K = D; x.lda = D; x.ldb = D;
        x.splits = 1; x.dsw_gu = a.gu16; x.dsw_dgu = g->dgu; x.ldgu = 2 * F;
        if (pair_on(g)) x.max_ctas = g->pair_ctas_down;
        TB_TRY(gemm(g, x));
    } else {
    TB_TRY(linear_dx(g, dres_op, WOP(g, pidx(l, PK_WDOWN)), g->dh, nullptr, N, D, F));
    // (fused path: the gate|up bias gradient, the column sums of dgu, comes out of the same kernel)
    if (g->fused_swiglu)
        TB_TRY(launch_swiglu_bwd_colsum(c, a.gu16, g->dh, g->dgu, G32(g, pidx(l, PK_BGU)), g->swiglu_scratch, N, F, st));
    else TB_TRY(launch_swiglu_bwd(c, a.gu, g->dh, g->tf32 ? nullptr : g->dgu, N, F, st, g->dgu32));
    }
    const void* dgu_op = g->tf32 ? (const void*)g->dgu32 : (const void*)g->dgu;
    TB_TRY(linear_dw(g, g->tf32 ? (const void*)a.n2_32 : (const void*)a.n2, dgu_op, G32(g, pidx(l, PK_WGU)), N, 2 * F, D, 1));
    if (g->fused_dswiglu) {
        // on the weight gradients' stream when the pair runs side by side (in order behind the product above and ahead
        // of the layer's last weight gradient, whose event the layer's end waits for); with a scratch buffer of its
        // own, because the main stream's column sum of dqkv may run at the same time
        cudaStream_t cs = pair_on(g) ? g->side : st;
        TB_TRY(launch_colsum_bf16(c, g->dgu, G32(g, pidx(l, PK_BGU)), g->colsum_partial2, N, 2 * F, cs));
    }
    if (!g->fused_swiglu) {
        if (g->tf32) TB_TRY(launch_colsum_f32(c, g->dgu32, G32(g, pidx(l, PK_BGU)), g->colsum_partial, N, 2 * F, st));
        else TB_TRY(launch_colsum_bf16(c, g->dgu, G32(g, pidx(l, PK_BGU)), g->colsum_partial, N, 2 * F, st));
    }
    TB_TRY(linear_dx(g, dgu_op, WOP(g, pidx(l, PK_WGU)), g->dn, nullptr, N, 2 * F, D));
    TB_TRY(pair_wait(g, 0));           // the norm backward overwrites dres16, which the down-projection's dW reads
    TB_TRY(launch_rmsnorm_bwd_dw(c, a.x2, P32(g, pidx(l, PK_FFN_NORM)), a.r2, g->dn, g->dres, g->dres16,
                                 G32(g, pidx(l, PK_FFN_NORM)), G32(g, pidx(l, PK_BO)), g->norm_scratch, N, D, 1, st));

    // ---- attention: x2 = x + (att @ Wo + bo); dres = dx2
    if (g->tf32) TB_TRY(launch_widen_bf16(c, a.att, g->att32, (long long)N * D, st));
    TB_TRY(linear_dw(g, g->tf32 ? (const void*)g->att32 : (const void*)a.att, dres_op, G32(g, pidx(l, PK_WO)), N, D, D, 2));
    // (bo's gradient came with dres as well)
    TB_TRY(linear_dx(g, dres_op, WOP(g, pidx(l, PK_WO)), nullptr, g->datt, N, D, D));
    if (g->fused_attention) {
        // dQ, dK, dV leave the kernels rotated back and merged as bf16 dqkv [N, 3D]
        TB_TRY(launch_attention_bwd(c, a.Q, a.K, a.V, a.att, g->datt, a.lse, g->att_delta, nullptr, nullptr, nullptr, B,
                                    H, T, hd, g->scale, st, g->dqkv, g->cos_t, g->sin_t, g->att_ds));
    } else {
    TB_TRY(launch_heads_split(c, g->datt, g->dO, B, T, H, hd, st));
    {   // dV = P^T dO
        GemmArgs v;
        v.kind = GEMM_TN; v.A = a.P; v.B = g->dO; v.M = T; v.N = hd; v.K = T; v.lda = Tp; v.ldb = hd;
        v.batch = BH; v.strideA = sTT; v.strideB = sThd;
        v.C32 = g->dV; v.ldc32 = hd; v.strideC32 = sThd; v.causal = CAUSAL_K_SUFFIX; v.splits = 1;
        TB_TRY(gemm(g, v));
    }
    {   // dP = dO V^T
        GemmArgs p;
        p.kind = GEMM_NT; p.A = g->dO; p.B = a.V; p.M = T; p.N = T; p.K = hd; p.lda = hd; p.ldb = hd;
        p.batch = BH; p.strideA = sThd; p.strideB = sThd;
        p.C32 = g->dP; p.ldc32 = Tp; p.strideC32 = sTT; p.causal = CAUSAL_SKIP_UPPER; p.splits = 1;
        TB_TRY(gemm(g, p));
    }
    TB_TRY(launch_attn_softmax_bwd(c, a.P, g->dP, g->dS, BH, T, Tp, g->scale, st));
    {   // dQ = dS K
        GemmArgs q;
        q.kind = GEMM_NN; q.A = g->dS; q.B = a.K; q.M = T; q.N = hd; q.K = T; q.lda = Tp; q.ldb = hd;
        q.batch = BH; q.strideA = sTT; q.strideB = sThd;
        q.C32 = g->dQ; q.ldc32 = hd; q.strideC32 = sThd; q.causal = CAUSAL_K_PREFIX; q.splits = 1;
        TB_TRY(gemm(g, q));
    }
    {   // dK = dS^T Q
        GemmArgs k;
        k.kind = GEMM_TN; k.A = g->dS; k.B = a.Q; k.M = T; k.N = hd; k.K = T; k.lda = Tp; k.ldb = hd;
        k.batch = BH; k.strideA = sTT; k.strideB = sThd;
        k.C32 = g->dK; k.ldc32 = hd; k.strideC32 = sThd; k.causal = CAUSAL_K_SUFFIX; k.splits = 1;
        TB_TRY(gemm(g, k));
    }
    TB_TRY(launch_rope_merge_bwd(c, g->dQ, g->dK, g->dV, g->cos_t, g->sin_t, g->dqkv, B, T, H, hd, st));
    }
    if (g->tf32) TB_TRY(launch_widen_bf16(c, g->dqkv, g->dqkv32, (long long)N * 3 * D, st));
    const void* dqkv_op = g->tf32 ? (const void*)g->dqkv32 : (const void*)g->dqkv;
    TB_TRY(linear_dw(g, g->tf32 ? (const void*)a.n1_32 : (const void*)a.n1, dqkv_op, G32(g, pidx(l, PK_WQKV)), N, 3 * D, D, 3));
    TB_TRY(launch_colsum_bf16(c, g->dqkv, G32(g, pidx(l, PK_BQKV)), g->colsum_partial, N, 3 * D, st));
    TB_TRY(linear_dx(g, dqkv_op, WOP(g, pidx(l, PK_WQKV)), g->dn, nullptr, N, 3 * D, D));
    TB_TRY(pair_wait(g, 2));           // the norm backward overwrites dres16, which the out-projection's dW reads
    TB_TRY(launch_rmsnorm_bwd_dw(c, a.x_in, P32(g, pidx(l, PK_ATTN_NORM)), a.r1, g->dn, g->dres, g->dres16,
                                 G32(g, pidx(l, PK_ATTN_NORM)), l > 0 ? G32(g, pidx(l - 1, PK_BDOWN)) : nullptr,
                                 g->norm_scratch, N, D, 1, st));
    // the layer below overwrites dgu and dqkv; a graph of this layer alone must end with the second stream joined
    TB_TRY(pair_wait(g, 3));
    return 0;
}

int backward_embed(TbTrainer* g) {
    return launch_embed_bwd(g->ctx, g->dres, g->order, g->seg_start, g->seg_token, g->seg_meta, g->nseg_dev, g->N,
                            g->embed_partial, g->embed_tickets, G32(g, 0),
                            g->D, g->stream);
}

enum { SEG_FWD_TRAIN = 0, SEG_FWD_EVAL, SEG_HEAD_BWD, SEG_EMBED_BWD, SEG_ZERO, SEG_STEP, SEG_BWD_ALL, SEG_LAYER0 };

// Runs `body` (a fixed sequence of launches on g->stream): eagerly the first time, under stream
// capture the second time, as a graph launch from then on.
template <typename Body>
int run_segment(TbTrainer* g, int id, Body body) {
    if (!g->graphs_on || g->ctx->prof_on) return body();
    if ((int)g->segments.size() <= id) g->segments.resize(id + 1);
    TbTrainer::Segment& s = g->segments[id];
    if (s.state == 0) { s.state = 1; return body(); }
    if (s.state == 1) {
        const long long before = g->ctx->launches;
        TB_CUDA(cudaStreamBeginCapture(g->stream, cudaStreamCaptureModeRelaxed));
        const int rc = body();
        cudaGraph_t graph = nullptr;
        const cudaError_t e = cudaStreamEndCapture(g->stream, &graph);
        if (rc != 0) { if (graph) cudaGraphDestroy(graph); return rc; }
        TB_CUDA(e);
        s.launches = g->ctx->launches - before;
        TB_CUDA(cudaGraphInstantiate(&s.exec, graph, 0));
        cudaGraphDestroy(graph);
        s.state = 2;
        TB_CUDA(cudaGraphLaunch(s.exec, g->stream));
        return 0;
    }
    TB_CUDA(cudaGraphLaunch(s.exec, g->stream));
    g->ctx->launches += s.launches;
    return 0;
}

// Stages ids/targets through pinned memory and starts their copy to the device.
int stage_inputs(TbTrainer* g, const uint32_t* ids, const uint32_t* targets) {
    const size_t bytes = (size_t)g->N * sizeof(uint32_t);
    for (int i = 0; i < g->N; ++i)
        TB_CHECK(ids[i] < (uint32_t)g->V && targets[i] < (uint32_t)g->V, "token id out of range at position %d", i);
    // the pinned staging buffers are reused: the copies of the previous batch (micro-batches of one optimiser
    // step follow each other without a host synchronisation) must have left them
    if (g->staged_pending) { TB_CUDA(cudaEventSynchronize(g->staged)); g->staged_pending = false; }
    std::memcpy(g->h_ids, ids, bytes);
    std::memcpy(g->h_targets, targets, bytes);
    TB_CUDA(cudaMemcpyAsync(g->ids, g->h_ids, bytes, cudaMemcpyHostToDevice, g->stream));
    TB_CUDA(cudaMemcpyAsync(g->targets, g->h_targets, bytes, cudaMemcpyHostToDevice, g->stream));
    TB_CUDA(cudaEventRecord(g->staged, g->stream));
    g->staged_pending = true;
    return 0;
}

// Rows grouped by token (ties in ascending position) for the embedding gradient; runs of one token
// are cut into chunks of kEmbedChunk rows (see embed_bwd_kernel).  One pinned buffer, one copy:
// [order N][chunk start N+1][chunk token N][chunk meta 3N][number of chunks 1].
int stage_segments(TbTrainer* g) {
    const int N = g->N;
    std::vector<uint64_t> keys(N);
    for (int i = 0; i < N; ++i) keys[i] = ((uint64_t)g->h_ids[i] << 32) | (uint32_t)i;
    std::sort(keys.begin(), keys.end());
    uint32_t* order = g->h_seg;
    uint32_t* seg_start = g->h_seg + N;
    uint32_t* seg_token = g->h_seg + 2 * N + 1;
    uint32_t* meta = g->h_seg + 3 * N + 1;
    for (int i = 0; i < N; ++i) order[i] = (uint32_t)(keys[i] & 0xffffffffu);
    int nseg = 0;
    uint32_t slot = 0;
    for (int i = 0; i < N;) {
        const uint32_t tok = (uint32_t)(keys[i] >> 32);
        int j = i;
        while (j < N && (uint32_t)(keys[j] >> 32) == tok) ++j;
        const uint32_t chunks = (uint32_t)((j - i + kEmbedChunk - 1) / kEmbedChunk);
        for (uint32_t c = 0; c < chunks; ++c) {
            seg_start[nseg] = (uint32_t)(i + (int)c * kEmbedChunk);
            seg_token[nseg] = tok;
            meta[3 * nseg] = chunks > 1 ? slot : 0xffffffffu;
            meta[3 * nseg + 1] = c;
            meta[3 * nseg + 2] = chunks;
            ++nseg;
        }
        if (chunks > 1) slot += chunks;
        i = j;
    }
    TB_CHECK((int)slot <= embed_partial_slots(N), "embedding gradient: %u partial slots exceed the buffer", slot);
    for (int i = nseg; i <= N; ++i) seg_start[i] = (uint32_t)N;
    g->nseg = nseg;
    g->h_seg[6 * N + 1] = (uint32_t)nseg;
    TB_CUDA(cudaMemcpyAsync(g->order, g->h_seg, (size_t)(6 * N + 2) * sizeof(uint32_t), cudaMemcpyHostToDevice,
                            g->stream));
    TB_CUDA(cudaEventRecord(g->staged, g->stream));
    g->staged_pending = true;
    return 0;
}

// mean over the T rows of each sequence, then over sequences (gpu_train.c:478-487)
float mean_loss_host(const TbTrainer* g) {
    float loss_sum = 0.0f;
    for (int b = 0; b < g->B; ++b) {
        float s = 0.0f;
        for (int t = 0; t < g->T; ++t) s += g->h_loss_rows[(size_t)b * g->T + t];
        loss_sum += s / (float)g->T;
    }
    return loss_sum / (float)g->B;
}

int read_loss(TbTrainer* g, float* loss_out) {
    TB_CUDA(cudaMemcpyAsync(g->h_loss_rows, g->loss_rows, (size_t)g->N * sizeof(float), cudaMemcpyDeviceToHost,
                            g->stream));
    TB_TRY(check_device_error(g->ctx, g->stream));
    if (loss_out) *loss_out = mean_loss_host(g);
    return 0;
}

int adam_launch(TbTrainer* g, uint64_t t, float lr, float b1, float b2, float eps, float grad_scale,
                const float* dev_scale) {
    const float bc1 = 1.0f - powf(b1, (float)t);
    const float bc2 = 1.0f - powf(b2, (float)t);
    return launch_adam(g->ctx, g->params, g->params16, g->grads, g->adam_m, g->adam_v, g->total, lr, b1, b2, eps, bc1,
                       bc2, grad_scale, dev_scale, g->stream);
}

}  // namespace

namespace tb {
int trainer_grads_ready(TbTrainer* g) {
    if (g->zero_pending) {
        TB_CUDA(cudaStreamWaitEvent(g->stream, g->ev_zero, 0));
        g->zero_pending = false;
    }
    return 0;
}

int trainer_view(TbTrainer* g, TrainerView* v) {
    TB_CHECK(g != nullptr && v != nullptr, "trainer_view: null argument");
    v->ctx = g->ctx; v->stream = g->stream; v->device = g->device;
    v->total = g->total; v->padded = g->padded;
    v->params = g->params; v->grads = g->grads; v->adam_m = g->adam_m; v->adam_v = g->adam_v; v->params16 = g->params16;
    v->loss_rows = g->loss_rows; v->B = g->B; v->T = g->T; v->L = g->L;
    v->norm_partial = g->norm_partial; v->scalars = g->scalars; v->norm64 = g->norm64; v->h_norm = g->h_norm;
    return 0;
}
}  // namespace tb

extern "C" {

int tb_trainer_create(TbTrainer** out, int V, int D, int H, int L, int F, int T, int B, float eps, void* stream) {
    return tb_trainer_create_prec(out, V, D, H, L, F, T, B, eps, TB_PREC_BF16, stream);
}

int tb_trainer_create_prec(TbTrainer** out, int V, int D, int H, int L, int F, int T, int B, float eps, int precision,
                           void* stream) {
    TB_CHECK(out != nullptr, "tb_trainer_create: out is NULL");
    TB_CHECK(precision == TB_PREC_BF16 || precision == TB_PREC_TF32,
             "the trainer runs its GEMMs in BF16 or TF32 mode (precision %d is not available: there is no fallback)", precision);
    TB_CHECK(V > 0 && D > 0 && H > 0 && L >= 0 && F > 0 && T > 0 && B > 0, "trainer dims must be positive");
    TB_CHECK(D % H == 0, "d_model %d not divisible by heads %d", D, H);
    TB_CHECK(D % 8 == 0 && F % 8 == 0 && (D / H) % 8 == 0,
             "d_model, d_ff and head_dim must be multiples of 8 (16-byte rows for TMA); got D=%d F=%d hd=%d", D, F,
             D / H);
    TbTrainer* g = new TbTrainer();
    TB_TRY(get_ctx(&g->ctx));
    g->device = g->ctx->device;
    g->stream = static_cast<cudaStream_t>(stream);
    if (g->stream == nullptr) {
        // the legacy default stream cannot be captured into a graph: work on a stream of our own
        TB_CUDA(cudaStreamCreateWithFlags(&g->stream, cudaStreamNonBlocking));
        g->owns_stream = true;
    }
    g->tf32 = precision == TB_PREC_TF32;
    g->graphs_on = getenv("TB_NO_GRAPH") == nullptr;
    g->fused_attention = (D / H) <= 64 && getenv("TB_NO_FUSED_ATTENTION") == nullptr;
    TB_CHECK(!g->tf32 || g->fused_attention, "the TF32 mode needs head_dim <= 64 (the attention core is the fused bf16 kernel)");
    g->fused_swiglu = !g->tf32 && F % 64 == 0 && getenv("TB_NO_FUSED_SWIGLU") == nullptr;
    g->fused_dswiglu = g->fused_swiglu && getenv("TB_NO_FUSED_DSWIGLU") == nullptr;
    g->fused_rope = !g->tf32 && T % 32 == 0 && (D / H == 32 || D / H == 64) && getenv("TB_NO_FUSED_ROPE") == nullptr;
    g->V = V; g->D = D; g->H = H; g->L = L; g->F = F; g->T = T; g->B = B; g->N = B * T; g->hd = D / H;
    g->Vp = round_up(V, 8);
    g->Tp = round_up(T, 8);
    g->eps = eps;
    g->scale = 1.0f / sqrtf((float)g->hd);

    // flat layout in lm_collect_params order (model/lm_model.c:84-98)
    auto push = [&](long long n) { g->offsets.push_back(g->total); g->numels.push_back(n); g->total += n; };
    push((long long)V * D);
    for (int l = 0; l < L; ++l) {
        push(D); push((long long)D * 3 * D); push(3LL * D); push((long long)D * D); push(D);
        push(D); push((long long)D * 2 * F); push(2LL * F); push((long long)F * D); push(D);
    }
    push(D);

    const size_t N = g->N, BHT = (size_t)B * H * T;
    const size_t Tp = (size_t)g->Tp;
    // the flat buffers carry kFlatPad spare scalars behind the last parameter: the data-parallel step keeps
    // the rank's loss there (so one collective sums gradients and loss) and rounds its per-rank slices up
    g->padded = g->total + kFlatPad;
    TB_TRY(dalloc(g, &g->params, g->padded)); TB_TRY(dalloc(g, &g->grads, g->padded));
    TB_TRY(dalloc(g, &g->adam_m, g->padded)); TB_TRY(dalloc(g, &g->adam_v, g->padded));
    TB_TRY(dalloc(g, &g->params16, g->padded));
    TB_CUDA(cudaMemset(g->params, 0, g->padded * 4)); TB_CUDA(cudaMemset(g->grads, 0, g->padded * 4));
    TB_CUDA(cudaMemset(g->adam_m, 0, g->padded * 4)); TB_CUDA(cudaMemset(g->adam_v, 0, g->padded * 4));
    TB_CUDA(cudaMemset(g->params16, 0, g->padded * 2));

    g->layers.resize(L);
    for (int l = 0; l < L; ++l) {
        LayerActs& a = g->layers[l];
        TB_TRY(dalloc(g, &a.x_in, N * D)); TB_TRY(dalloc(g, &a.n1, N * D)); TB_TRY(dalloc(g, &a.r1, N));
        TB_TRY(dalloc(g, &a.Q, 3 * N * D));          // Q, K, V back to back: one 5-D store map covers them
        a.K = a.Q + N * D; a.V = a.K + N * D;
        if (g->fused_attention) { a.P = nullptr; TB_TRY(dalloc(g, &a.lse, BHT)); }
        else { a.lse = nullptr; TB_TRY(dalloc(g, &a.P, BHT * Tp)); }
        TB_TRY(dalloc(g, &a.att, N * D));
        TB_TRY(dalloc(g, &a.x2, N * D)); TB_TRY(dalloc(g, &a.n2, N * D)); TB_TRY(dalloc(g, &a.r2, N));
        a.gu = nullptr; a.gu16 = nullptr;
        if (g->fused_swiglu) TB_TRY(dalloc(g, &a.gu16, N * 2 * F));
        else TB_TRY(dalloc(g, &a.gu, N * 2 * F));
        TB_TRY(dalloc(g, &a.h, N * F));
        if (g->tf32) {
            TB_TRY(dalloc(g, &a.n1_32, N * D)); TB_TRY(dalloc(g, &a.n2_32, N * D)); TB_TRY(dalloc(g, &a.h32, N * F));
        }
    }
    TB_TRY(dalloc(g, &g->x_final, N * D)); TB_TRY(dalloc(g, &g->nf, N * D)); TB_TRY(dalloc(g, &g->rf, N));
    g->fused_ce = !g->tf32 && getenv("TB_NO_FUSED_CE") == nullptr;
    if (g->tf32) {
        TB_TRY(dalloc(g, &g->nf32, N * D)); TB_TRY(dalloc(g, &g->dlogits32, N * g->Vp));
        TB_TRY(dalloc(g, &g->dgu32, N * 2 * F)); TB_TRY(dalloc(g, &g->dqkv32, N * 3 * D)); TB_TRY(dalloc(g, &g->att32, N * D));
        TB_CUDA(cudaMemset(g->dlogits32, 0, N * g->Vp * 4));      // the padding columns stay zero
    }
    if (g->fused_ce) {
        TB_TRY(dalloc(g, &g->ce_stats, (size_t)2 * ((V + kCeTile - 1) / kCeTile) * N * 2));
        TB_TRY(dalloc(g, &g->ce_zt, N)); TB_TRY(dalloc(g, &g->ce_lse, N));
    } else {
        TB_TRY(dalloc(g, &g->logits, N * g->Vp));
    }
    TB_TRY(dalloc(g, &g->dlogits, N * g->Vp));
    TB_TRY(dalloc(g, &g->qkv, N * 3 * D));
    if (g->fused_attention) {
        TB_TRY(dalloc(g, &g->att_delta, BHT));
        TB_TRY(dalloc(g, &g->att_ds, attention_bwd_ds_bytes(B, H, T) / sizeof(bf16)));
    } else {
        TB_TRY(dalloc(g, &g->S, BHT * Tp)); TB_TRY(dalloc(g, &g->dP, BHT * Tp));
    }
    TB_TRY(dalloc(g, &g->dn, N * D)); TB_TRY(dalloc(g, &g->dres, N * D)); TB_TRY(dalloc(g, &g->wtmp, N * D));
    TB_TRY(dalloc(g, &g->dh, N * F));
    TB_TRY(dalloc(g, &g->dQ, N * D)); TB_TRY(dalloc(g, &g->dK, N * D)); TB_TRY(dalloc(g, &g->dV, N * D));
    TB_TRY(dalloc(g, &g->dres16, N * D)); TB_TRY(dalloc(g, &g->dgu, N * 2 * F)); TB_TRY(dalloc(g, &g->datt, N * D));
    TB_TRY(dalloc(g, &g->dqkv, N * 3 * D));
    if (!g->fused_attention) { TB_TRY(dalloc(g, &g->dO, N * D)); TB_TRY(dalloc(g, &g->dS, BHT * Tp)); }
    TB_CHECK(D <= 1024, "d_model up to 1024 is supported (got %d)", D);
    {
        const size_t nc = colsum_partial_floats(std::max(3 * D, 2 * F)), nn = rmsnorm_bwd_scratch_floats(D);
        TB_TRY(dalloc(g, &g->colsum_partial, nc));
        TB_TRY(dalloc(g, &g->colsum_partial2, nc));
        TB_CUDA(cudaMemset(g->colsum_partial2, 0, nc * 4));
        TB_TRY(dalloc(g, &g->norm_scratch, nn));
        TB_TRY(dalloc(g, &g->swiglu_scratch, swiglu_bwd_scratch_floats(F)));
        TB_CUDA(cudaMemset(g->colsum_partial, 0, nc * 4));     // ticket words start at zero
        TB_CUDA(cudaMemset(g->norm_scratch, 0, nn * 4));
    }
    // dS and P rows are read by whole 128-tiles: start them from zero so never-written tails are finite
    if (!g->fused_attention) {
        TB_CUDA(cudaMemset(g->dS, 0, BHT * Tp * 2));
        for (int l = 0; l < L; ++l) TB_CUDA(cudaMemset(g->layers[l].P, 0, BHT * Tp * 2));
    }

    // split-K partials for the weight-gradient GEMMs: the largest is [D, 2F] or [D, 3D] or [F, D]
    {
        // a split count never exceeds SMs / tiles, so splits * M * N stays below about one 128x128
        // tile per SM, plus one unsplit copy of the largest weight matrix for rounding slack
        size_t biggest = std::max({(size_t)D * 2 * F, (size_t)D * 3 * D, (size_t)F * D, (size_t)D * D});
        g->splitk_floats = biggest + 2 * (size_t)g->ctx->sm_count * 128 * 128;
        // the LM head's input gradient [N, D] may run split along K on 256-row pair tiles: splits <= pairs / tiles, so
        // splits * N * D stays below one 256-row slab per CTA pair (plus the unsplit size for rounding slack)
        g->splitk_floats = std::max(g->splitk_floats, ((size_t)g->ctx->sm_count / 2 + 2) * 256 * (size_t)D + 2 * (size_t)N * D);
        TB_TRY(dalloc(g, &g->splitk_ws, g->splitk_floats));
    }

    TB_TRY(dalloc(g, &g->ids, N)); TB_TRY(dalloc(g, &g->targets, N)); 
    TB_TRY(dalloc(g, &g->order, 6 * N + 2));          // order | chunk start | chunk token | chunk meta | count
    g->seg_start = g->order + N; g->seg_token = g->order + 2 * N + 1; g->seg_meta = g->order + 3 * N + 1;
    g->nseg_dev = g->order + 6 * N + 1;
    TB_TRY(dalloc(g, &g->embed_partial, (size_t)embed_partial_slots((int)N) * D));
    TB_TRY(dalloc(g, &g->embed_tickets, (size_t)embed_partial_slots((int)N)));
    TB_CUDA(cudaMemset(g->embed_tickets, 0, (size_t)embed_partial_slots((int)N) * sizeof(unsigned int)));
    TB_TRY(dalloc(g, &g->loss_rows, N));
    TB_TRY(dalloc(g, &g->norm_partial, (size_t)kNormBlocks)); TB_TRY(dalloc(g, &g->scalars, 4));
    TB_TRY(dalloc(g, &g->norm64, 1));
    TB_CUDA(cudaMallocHost(&g->h_ids, N * 4)); TB_CUDA(cudaMallocHost(&g->h_targets, N * 4));
    TB_CUDA(cudaMallocHost(&g->h_seg, (6 * N + 4) * 4)); TB_CUDA(cudaMallocHost(&g->h_loss_rows, N * 4));
    TB_CUDA(cudaMallocHost(&g->h_norm, sizeof(double)));
    TB_CUDA(cudaEventCreateWithFlags(&g->staged, cudaEventDisableTiming));
    if (getenv("TB_NO_DW_PAIR") == nullptr) {
        TB_CUDA(cudaStreamCreateWithFlags(&g->side, cudaStreamNonBlocking));
        TB_CUDA(cudaEventCreateWithFlags(&g->ev_fork, cudaEventDisableTiming));
        for (int i = 0; i < 4; ++i) TB_CUDA(cudaEventCreateWithFlags(&g->ev_done[i], cudaEventDisableTiming));
        TB_CUDA(cudaEventCreateWithFlags(&g->ev_zero, cudaEventDisableTiming));
        g->pair_ctas = g->ctx->sm_count / 2;
        if (const char* e = getenv("TB_DW_PAIR_CTAS")) {
            const int v = atoi(e);
            if (v >= 8 && v <= g->ctx->sm_count - 8) g->pair_ctas = v;
        }
        // the input-gradient product of the down-projection carries SwiGLU backward in its epilogue and takes 5/8 of
        // the SMs (measured on the benchmark step: 74 CTAs 5.27 ms, 82 5.27, 90 5.18, 98 5.18, 104 5.11 against 5.09 at 90
        // on a second GPU)
        g->pair_ctas_down = g->fused_dswiglu ? g->ctx->sm_count * 5 / 8 : g->pair_ctas;
        if (const char* e = getenv("TB_DSW_PAIR_CTAS")) {
            const int v = atoi(e);
            if (v >= 8 && v <= g->ctx->sm_count - 8) g->pair_ctas_down = v;
        }
    }

    // RoPE tables [T, hd/2] (model/rope.c:4-18), built on the host in float32
    {
        const int half = g->hd / 2;
        std::vector<float> ct((size_t)T * half), sn((size_t)T * half);
        for (int pos = 0; pos < T; ++pos)
            for (int k = 0; k < half; ++k) {
                const float exponent = -(2.0f * (float)k) / (float)g->hd;
                const float theta = powf(10000.0f, exponent);
                const float angle = (float)pos * theta;
                ct[(size_t)pos * half + k] = cosf(angle);
                sn[(size_t)pos * half + k] = sinf(angle);
            }
        TB_TRY(dalloc(g, &g->cos_t, ct.size())); TB_TRY(dalloc(g, &g->sin_t, sn.size()));
        TB_H2D_SYNC(g->cos_t, ct.data(), ct.size() * 4);
        TB_H2D_SYNC(g->sin_t, sn.data(), sn.size() * 4);
    }
    *out = g;
    return 0;
}

int tb_trainer_destroy(TbTrainer* g) {
    if (!g) return 0;
    cudaDeviceSynchronize();
    for (auto& sgm : g->segments) if (sgm.exec) cudaGraphExecDestroy(sgm.exec);
    if (g->owns_stream) cudaStreamDestroy(g->stream);
    for (void* p : g->allocs) cudaFree(p);
    cudaFreeHost(g->h_ids); cudaFreeHost(g->h_targets); cudaFreeHost(g->h_seg);
    cudaFreeHost(g->h_loss_rows); cudaFreeHost(g->h_norm);
    if (g->staged) cudaEventDestroy(g->staged);
    if (g->ev_fork) cudaEventDestroy(g->ev_fork);
    for (int i = 0; i < 4; ++i) if (g->ev_done[i]) cudaEventDestroy(g->ev_done[i]);
    if (g->ev_zero) cudaEventDestroy(g->ev_zero);
    if (g->side) cudaStreamDestroy(g->side);
    delete g;
    return 0;
}

int64_t tb_trainer_total_scalars(const TbTrainer* g) { return g->total; }
int tb_trainer_num_params(const TbTrainer* g) { return (int)g->offsets.size(); }

int tb_trainer_dims(const TbTrainer* g, int* V, int* D, int* H, int* L, int* F, int* T, int* B) {
    TB_CHECK(g, "tb_trainer_dims: null trainer");
    if (V) *V = g->V;
    if (D) *D = g->D;
    if (H) *H = g->H;
    if (L) *L = g->L;
    if (F) *F = g->F;
    if (T) *T = g->T;
    if (B) *B = g->B;
    return 0;
}

int tb_trainer_param_layout(const TbTrainer* g, int64_t* offsets, int64_t* numels) {
    for (size_t i = 0; i < g->offsets.size(); ++i) { offsets[i] = g->offsets[i]; numels[i] = g->numels[i]; }
    return 0;
}

static float* flat_ptr(TbTrainer* g, int which) {
    switch (which) { case 0: return g->params; case 1: return g->grads; case 2: return g->adam_m; case 3: return g->adam_v; }
    return nullptr;
}

void* tb_trainer_device_ptr(TbTrainer* g, int which) { return flat_ptr(g, which); }

int tb_trainer_upload(TbTrainer* g, int which, const float* h_flat) {
    float* d = flat_ptr(g, which);
    TB_CHECK(d != nullptr, "tb_trainer_upload: unknown buffer %d", which);
    TB_CUDA(cudaStreamSynchronize(g->stream));
    TB_H2D_SYNC(d, h_flat, (size_t)g->total * 4);
    if (which == 0) {
        // refresh the bf16 shadow copy the GEMMs read
        TB_CHECK(g->total < (1LL << 31), "model too large for the single-row pack");
        TB_TRY(launch_pack_bf16(g->ctx, g->params, g->params16, 1, (int)g->total, g->total, g->total, 1, 0, 0,
                                g->stream));
        TB_CUDA(cudaStreamSynchronize(g->stream));
    }
    return 0;
}

int tb_trainer_download(TbTrainer* g, int which, float* h_flat) {
    float* d = flat_ptr(g, which);
    TB_CHECK(d != nullptr, "tb_trainer_download: unknown buffer %d", which);
    TB_CUDA(cudaStreamSynchronize(g->stream));
    TB_CUDA(cudaMemcpy(h_flat, d, (size_t)g->total * 4, cudaMemcpyDeviceToHost));
    return 0;
}

// The clearing (134 MB, ~25 us) runs on the second stream, beside the forward pass, which does not touch the
// gradients; trainer_grads_ready stands in front of the first writer.
int tb_trainer_zero_grads(TbTrainer* g) {
    if (g->side == nullptr || g->ctx->prof_on) {
        TB_CUDA(cudaMemsetAsync(g->grads, 0, (size_t)g->padded * 4, g->stream));
        return 0;
    }
    TB_CUDA(cudaEventRecord(g->ev_fork, g->stream));          // after whatever still reads or writes the buffer
    TB_CUDA(cudaStreamWaitEvent(g->side, g->ev_fork, 0));
    TB_CUDA(cudaMemsetAsync(g->grads, 0, (size_t)g->padded * 4, g->side));
    TB_CUDA(cudaEventRecord(g->ev_zero, g->side));
    g->zero_pending = true;
    return 0;
}


void* tb_trainer_stream(TbTrainer* g) { return g->stream; }

int tb_trainer_forward(TbTrainer* g, const uint32_t* h_ids, const uint32_t* h_targets, int want_grad) {
    TB_CUDA(cudaSetDevice(g->device));
    TB_TRY(stage_inputs(g, h_ids, h_targets));
    const bool wg = want_grad != 0;
    TB_TRY(run_segment(g, wg ? SEG_FWD_TRAIN : SEG_FWD_EVAL, [&]() { return forward(g, wg); }));
    if (want_grad) TB_TRY(stage_segments(g));
    return 0;
}

int tb_trainer_set_inputs(TbTrainer* g, const uint32_t* h_ids, const uint32_t* h_targets) {
    TB_CUDA(cudaSetDevice(g->device));
    TB_TRY(stage_inputs(g, h_ids, h_targets));
    TB_TRY(stage_segments(g));
    TB_CUDA(cudaStreamSynchronize(g->stream));
    return 0;
}

int tb_trainer_step_resident(TbTrainer* g, uint64_t t, float lr, float beta1, float beta2, float eps,
                             float max_norm) {
    TB_CHECK(g->nseg > 0, "tb_trainer_step_resident: call tb_trainer_set_inputs first");
    // zeroing, forward and the whole backward are one graph (a single-GPU step has no reason to stop between
    // layers); the optimiser's scalars change every step, so clip + Adam stay ordinary launches
    TB_TRY(run_segment(g, SEG_STEP, [&]() {
        if (pair_on(g)) {          // cleared beside the forward pass (inside the same graph)
            TB_CUDA(cudaEventRecord(g->ev_fork, g->stream));
            TB_CUDA(cudaStreamWaitEvent(g->side, g->ev_fork, 0));
            TB_CUDA(cudaMemsetAsync(g->grads, 0, (size_t)g->padded * 4, g->side));
            TB_CUDA(cudaEventRecord(g->ev_done[0], g->side));
            TB_TRY(forward(g, true));
            TB_CUDA(cudaStreamWaitEvent(g->stream, g->ev_done[0], 0));
        } else {
            TB_CUDA(cudaMemsetAsync(g->grads, 0, (size_t)g->padded * 4, g->stream));
            TB_TRY(forward(g, true));
        }
        TB_TRY(backward_head(g));
        for (int l = g->L - 1; l >= 0; --l) TB_TRY(backward_layer(g, l));
        return backward_embed(g);
    }));
    return tb_trainer_clip_adam_async(g, t, lr, beta1, beta2, eps, max_norm, 1.0f);
}

int tb_trainer_forward_resident(TbTrainer* g, int want_grad) {
    TB_CHECK(g->nseg > 0, "tb_trainer_forward_resident: call tb_trainer_set_inputs first");
    const bool wg = want_grad != 0;
    return run_segment(g, wg ? SEG_FWD_TRAIN : SEG_FWD_EVAL, [&]() { return forward(g, wg); });
}

int tb_trainer_last_norm(TbTrainer* g, double* norm_out) {
    TB_CUDA(cudaStreamSynchronize(g->stream));
    *norm_out = *g->h_norm;
    return 0;
}

int tb_trainer_backward_head(TbTrainer* g) {
    TB_TRY(trainer_grads_ready(g));
    return run_segment(g, SEG_HEAD_BWD, [&]() { return backward_head(g); });
}
int tb_trainer_backward_layer(TbTrainer* g, int layer) {
    TB_CHECK(layer >= 0 && layer < g->L, "layer %d out of range", layer);
    return run_segment(g, SEG_LAYER0 + layer, [&]() { return backward_layer(g, layer); });
}
int tb_trainer_backward_embed(TbTrainer* g) {
    return run_segment(g, SEG_EMBED_BWD, [&]() { return backward_embed(g); });
}
static int backward_all_segment(TbTrainer* g) {
    TB_TRY(trainer_grads_ready(g));
    return run_segment(g, SEG_BWD_ALL, [&]() {
        TB_TRY(backward_head(g));
        for (int l = g->L - 1; l >= 0; --l) TB_TRY(backward_layer(g, l));
        return backward_embed(g);
    });
}
int tb_trainer_read_loss(TbTrainer* g, float* loss_out) { return read_loss(g, loss_out); }

int tb_trainer_forward_backward(TbTrainer* g, const uint32_t* h_ids, const uint32_t* h_targets, float* loss_out) {
    TB_CUDA(cudaSetDevice(g->device));
    TB_TRY(tb_trainer_zero_grads(g));
    TB_TRY(tb_trainer_forward(g, h_ids, h_targets, 1));
    TB_TRY(backward_all_segment(g));
    return read_loss(g, loss_out);
}

int tb_trainer_eval_loss(TbTrainer* g, const uint32_t* h_ids, const uint32_t* h_targets, float* loss_out) {
    TB_CUDA(cudaSetDevice(g->device));
    TB_TRY(tb_trainer_forward(g, h_ids, h_targets, 0));
    return read_loss(g, loss_out);
}

int tb_trainer_grad_norm(TbTrainer* g, double* norm_out) {
    TB_TRY(trainer_grads_ready(g));
    TB_TRY(launch_sumsq_partial(g->ctx, g->grads, g->total, g->norm_partial, g->stream));
    TB_TRY(launch_clip_scale(g->ctx, g->norm_partial, 0.0f, 1.0f, g->scalars, g->norm64, g->stream));
    TB_CUDA(cudaMemcpyAsync(g->h_norm, g->norm64, sizeof(double), cudaMemcpyDeviceToHost, g->stream));
    TB_CUDA(cudaStreamSynchronize(g->stream));
    *norm_out = *g->h_norm;
    return 0;
}

int tb_trainer_adam_step_scaled(TbTrainer* g, uint64_t t, float lr, float beta1, float beta2, float eps,
                                float grad_scale) {
    TB_CHECK(t >= 1, "Adam step counter starts at 1");
    TB_TRY(adam_launch(g, t, lr, beta1, beta2, eps, grad_scale, nullptr));
    TB_CUDA(cudaStreamSynchronize(g->stream));
    return 0;
}

int tb_trainer_clip_adam_async(TbTrainer* g, uint64_t t, float lr, float beta1, float beta2, float eps,
                               float max_norm, float grad_scale) {
    TB_CHECK(t >= 1, "Adam step counter starts at 1");
    TB_TRY(trainer_grads_ready(g));
    TB_TRY(launch_sumsq_partial(g->ctx, g->grads, g->total, g->norm_partial, g->stream));
    TB_TRY(launch_clip_scale(g->ctx, g->norm_partial, max_norm, grad_scale, g->scalars, g->norm64, g->stream));
    TB_CUDA(cudaMemcpyAsync(g->h_norm, g->norm64, sizeof(double), cudaMemcpyDeviceToHost, g->stream));
    return adam_launch(g, t, lr, beta1, beta2, eps, grad_scale, g->scalars);
}

int tb_trainer_train_step(TbTrainer* g, const uint32_t* h_ids, const uint32_t* h_targets, uint64_t t, float lr,
                          float beta1, float beta2, float eps, float max_norm, float* loss_out, double* norm_out) {
    TB_CUDA(cudaSetDevice(g->device));
    TB_TRY(tb_trainer_zero_grads(g));
    TB_TRY(tb_trainer_forward(g, h_ids, h_targets, 1));
    TB_TRY(backward_all_segment(g));
    TB_TRY(tb_trainer_clip_adam_async(g, t, lr, beta1, beta2, eps, max_norm, 1.0f));
    TB_TRY(read_loss(g, loss_out));
    if (norm_out) *norm_out = *g->h_norm;
    return 0;
}

}  // extern "C"

namespace tb {
int trainer_backward_all(TbTrainer* g) { return backward_all_segment(g); }
}  // namespace tb
