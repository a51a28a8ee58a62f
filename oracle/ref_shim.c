/* TEST INFRASTRUCTURE ONLY -- never linked into or called by the product library.
 *
 * Plain-C entry points (for ctypes) around the UNMODIFIED reference sources,
 * which the recipe in oracle/Makefile compiles from where they lie in the
 * reference checkout into oracle/_ref/libref.so.  Nothing here restates the
 * reference's arithmetic: every function forwards to a reference function
 * (cited per function, paths relative to the reference project).
 *
 * The GPU half of the reference (model/gpu_ops.c, cuda/cuda_backend.c) needs
 * libcuda and a device; it is left out of this library and its five entry
 * points are stubbed at the bottom so that lm_forward(..., use_gpu=0) links.
 */
#include "runtime/types.h"
#include "runtime/memory.h"
#include "runtime/prng.h"
#include "runtime/mathlib.h"
#include "tensor/tensor.h"
#include "autograd/node.h"
#include "model/lm_model.h"
#include "model/attention.h"
#include "model/feedforward.h"
#include "model/rope.h"
#include "model/loss.h"
#include "model/model_ops.h"
#include "model/gpu_ops.h"
#include "training/adam.h"
#include "training/data_parallel.h"
#include "training/checkpoint.h"
#include "training/lr_schedule.h"

#include <stdlib.h>
#include <string.h>
#include <stdio.h>

/* ---- stubs for the reference's GPU matmul operator (model/gpu_ops.h:23-60) ---- */
void gpu_ops_init(Allocator* scratch, const char* ptx_path) { (void)scratch; (void)ptx_path; }
void gpu_ops_shutdown(void) {}
void gpu_ops_init_workers(Allocator* scratch, const char* ptx_path, u32 n) { (void)scratch; (void)ptx_path; (void)n; }
void gpu_ops_set_worker_id(i32 worker_id) { (void)worker_id; }
Node* node_matmul2d_gpu(Allocator* alloc, Node* a, Node* b) {
    (void)alloc; (void)a; (void)b;
    fprintf(stderr, "ref_shim: node_matmul2d_gpu is not available in the CPU-only reference build\n");
    abort();
}
void gpu_ops_debug_stats(f64* s, u32* c) { if (s) *s = 0; if (c) *c = 0; }
void gpu_ops_debug_reset(void) {}

/* ---- seeded inputs: runtime/prng.c:19-94 ---- */
void ref_gaussian_fill(float* out, u64 n, u64 seed, u64 seq, double mean, double std) {
    PCGState rng = pcg_seed(seed, seq);
    for (u64 i = 0; i < n; i++) out[i] = (f32)pcg_gaussian(&rng, mean, std);
}

void ref_uniform_fill(double* out, u64 n, u64 seed, u64 seq) {
    PCGState rng = pcg_seed(seed, seq);
    for (u64 i = 0; i < n; i++) out[i] = pcg_uniform(&rng);
}

void ref_range_fill(u32* out, u64 n, u64 seed, u64 seq, i64 lo, i64 hi) {
    PCGState rng = pcg_seed(seed, seq);
    for (u64 i = 0; i < n; i++) out[i] = (u32)pcg_range_i64(&rng, lo, hi);
}

/* ---- tensor_matmul2d on strided views: tensor/tensor.c:351-373 ---- */
void ref_matmul2d(const float* A, u64 M, u64 K, i64 sa0, i64 sa1,
                  const float* B, u64 N, i64 sb0, i64 sb1, float* C) {
    Allocator alloc = allocator_create((M * N + 1024) * sizeof(f32) + (1ull << 20));
    Tensor a; memset(&a, 0, sizeof(a));
    a.data = (f32*)A; a.shape[0] = M; a.shape[1] = K; a.strides[0] = sa0; a.strides[1] = sa1;
    a.ndim = 2; a.numel = M * K; a.owns_data = FALSE;
    Tensor b; memset(&b, 0, sizeof(b));
    b.data = (f32*)B; b.shape[0] = K; b.shape[1] = N; b.strides[0] = sb0; b.strides[1] = sb1;
    b.ndim = 2; b.numel = K * N; b.owns_data = FALSE;
    Tensor c = tensor_matmul2d(&alloc, &a, &b);
    memcpy(C, c.data, M * N * sizeof(f32));
    allocator_destroy(&alloc);
}

/* ---- node_matmul2d forward + backward_matmul2d: autograd/node.c:116-135 ----
 * dC is the upstream gradient; dA, dB receive the accumulated gradients. */
void ref_matmul2d_fwd_bwd(const float* A, const float* B, const float* dC,
                          u64 M, u64 K, u64 N, float* C, float* dA, float* dB) {
    Allocator alloc = allocator_create(8 * (M * K + K * N + M * N) * sizeof(f32) + (4ull << 20));
    u64 sa[2] = { M, K }, sb[2] = { K, N };
    Tensor ta = tensor_create(&alloc, sa, 2); memcpy(ta.data, A, M * K * sizeof(f32));
    Tensor tb = tensor_create(&alloc, sb, 2); memcpy(tb.data, B, K * N * sizeof(f32));
    Node* na = node_leaf(&alloc, ta, TRUE);
    Node* nb = node_leaf(&alloc, tb, TRUE);
    Node* nc = node_matmul2d(&alloc, na, nb);
    memcpy(C, nc->value.data, M * N * sizeof(f32));
    memcpy(nc->grad.data, dC, M * N * sizeof(f32));
    nc->backward_fn(nc, &alloc);
    memcpy(dA, na->grad.data, M * K * sizeof(f32));
    memcpy(dB, nb->grad.data, K * N * sizeof(f32));
    allocator_destroy(&alloc);
}

/* ---- RoPE tables: model/rope.c:4-18 ---- */
void ref_rope_tables(u64 T, u64 hd, float base, float* cos_out, float* sin_out) {
    Allocator alloc = allocator_create(4 * T * hd * sizeof(f32) + (1ull << 20));
    u64 sh[2] = { T, hd / 2 };
    Tensor c = tensor_create(&alloc, sh, 2), s = tensor_create(&alloc, sh, 2);
    rope_build_tables(&c, &s, T, hd, base);
    memcpy(cos_out, c.data, c.numel * sizeof(f32));
    memcpy(sin_out, s.data, s.numel * sizeof(f32));
    allocator_destroy(&alloc);
}

/* ---- scalar math the trainer uses on the host ---- */
float ref_sqrtf(float x) { return m_sqrtf(x); }
float ref_powf(float a, float b) { return m_powf(a, b); }
float ref_expf(float x) { return m_expf(x); }
double ref_sqrt(double x) { return m_sqrt(x); }

/* ---- whole-model handle: lm_init (model/lm_model.c:39-60), lm_collect_params
 * (:84-98), adam_create/adam_step (training/adam.c) ---- */
typedef struct RefLM {
    Allocator alloc;
    LMModel model;
    Node* params[LM_MAX_LAYERS * 12 + 2];
    u32 np;
    AdamOptimizer opt;
    u32 F;
} RefLM;

RefLM* ref_lm_create(u32 V, u32 D, u32 H, u32 L, u32 F, float eps, u64 seed, u64 seq, u64 arena_bytes) {
    RefLM* r = (RefLM*)calloc(1, sizeof(RefLM));
    r->alloc = allocator_create(arena_bytes);
    PCGState rng = pcg_seed(seed, seq);
    r->model = lm_init(&r->alloc, &rng, V, D, H, L, F, eps);
    r->np = lm_collect_params(&r->model, r->params);
    r->opt = adam_create(&r->alloc, r->params, r->np, 3e-4f, 0.9f, 0.999f, 1e-8f);
    r->F = F;
    return r;
}

void ref_lm_destroy(RefLM* r) { allocator_destroy(&r->alloc); free(r); }

u32 ref_lm_num_params(RefLM* r) { return r->np; }
u64 ref_lm_param_numel(RefLM* r, u32 i) { return r->params[i]->value.numel; }

u64 ref_lm_total_scalars(RefLM* r) {
    u64 n = 0;
    for (u32 i = 0; i < r->np; i++) n += r->params[i]->value.numel;
    return n;
}

/* which: 0 = values, 1 = grads, 2 = adam m, 3 = adam v; flat in lm_collect_params order */
static f32* ref_lm_ptr(RefLM* r, u32 i, int which) {
    switch (which) {
        case 0: return r->params[i]->value.data;
        case 1: return r->params[i]->grad.data;
        case 2: return r->opt.m[i].data;
        default: return r->opt.v[i].data;
    }
}

void ref_lm_get(RefLM* r, int which, float* flat) {
    u64 off = 0;
    for (u32 i = 0; i < r->np; i++) {
        u64 n = r->params[i]->value.numel;
        memcpy(flat + off, ref_lm_ptr(r, i, which), n * sizeof(f32));
        off += n;
    }
}

void ref_lm_set(RefLM* r, int which, const float* flat) {
    u64 off = 0;
    for (u32 i = 0; i < r->np; i++) {
        u64 n = r->params[i]->value.numel;
        memcpy(ref_lm_ptr(r, i, which), flat + off, n * sizeof(f32));
        off += n;
    }
}

/* One production CPU step: adam_zero_grad + data_parallel_step
 * (training/data_parallel.c:119-163), CPU matmuls only.  Leaves the mean
 * gradients in the params; returns the mean loss. */
float ref_lm_dp_step(RefLM* r, const u32* tokens, u64 num_tokens, u64 T, u32 workers,
                     u64 seed_base, u64 step_arena_bytes) {
    adam_zero_grad(&r->opt);
    return data_parallel_step(&r->model, r->params, r->np, tokens, num_tokens, T,
                              step_arena_bytes, workers, seed_base, 0, 0);
}

/* Window selection used by both the CPU workers (data_parallel.c:73-77) and the
 * GPU trainer (model/gpu_train.c:296-307): sequence w draws its start from
 * pcg_seed(seed_base*1000003+w, 99+w). */
void ref_sample_batch(const u32* tokens, u64 num_tokens, u32 T, u32 B, u64 seed_base,
                      u32* ids_out, u32* targets_out) {
    i64 max_start = (i64)(num_tokens - T - 1);
    for (u32 w = 0; w < B; w++) {
        PCGState rng = pcg_seed(seed_base * 1000003ull + w, 99ull + w);
        i64 start = pcg_range_i64(&rng, 0, max_start);
        for (u32 t = 0; t < T; t++) {
            ids_out[(u64)w * T + t] = tokens[start + t];
            targets_out[(u64)w * T + t] = tokens[start + t + 1];
        }
    }
}

void ref_lm_adam_step(RefLM* r, float lr) { r->opt.lr = lr; adam_step(&r->opt); }
u64 ref_lm_adam_t(RefLM* r) { return r->opt.t; }
void ref_lm_set_adam_t(RefLM* r, u64 t) { r->opt.t = t; }

/* checkpoint_save / checkpoint_load: training/checkpoint.c:24-135.  Return the reference's bool32. */
int ref_lm_checkpoint_save(RefLM* r, const char* path, int with_opt) {
    return (int)checkpoint_save(path, r->params, r->np, with_opt ? &r->opt : NULL_PTR);
}
int ref_lm_checkpoint_load(RefLM* r, const char* path, int with_opt) {
    Allocator scratch = allocator_create(ref_lm_total_scalars(r) * 3 * sizeof(f32) + (16ull << 20));
    int ok = (int)checkpoint_load(&scratch, path, r->params, r->np, with_opt ? &r->opt : NULL_PTR);
    allocator_destroy(&scratch);
    return ok;
}

/* lr_warmup_cosine: training/lr_schedule.c:6-15 */
float ref_lr_warmup_cosine(u64 step, u64 warmup, u64 total, float peak, float min_lr) {
    return lr_warmup_cosine(step, warmup, total, peak, min_lr);
}

/* lm_forward (model/lm_model.c:62-82) on a batch of B stacked sequences;
 * writes logits [B*T, V].  Used as the decode oracle (full recompute). */
void ref_lm_forward_logits(RefLM* r, const u32* ids, u32 B, u64 T, float* logits_out, u64 arena_bytes) {
    Allocator a = allocator_create(arena_bytes);
    u64 hd = r->model.d_model / r->model.num_heads;
    u64 cs[2] = { T, hd / 2 };
    Tensor c = tensor_create(&a, cs, 2), s = tensor_create(&a, cs, 2);
    rope_build_tables(&c, &s, T, hd, 10000.0f);
    u64 ms[2] = { T, T };
    Tensor mask = tensor_create(&a, ms, 2);
    build_causal_mask(&mask);
    Node* logits = lm_forward(&a, &r->model, ids, B, T, node_leaf(&a, c, FALSE), node_leaf(&a, s, FALSE),
                              node_leaf(&a, mask, FALSE), 0, 0);
    memcpy(logits_out, logits->value.data, (u64)B * T * r->model.vocab_size * sizeof(f32));
    allocator_destroy(&a);
}

/* causal_self_attention (model/attention.c:17-68) forward + backward for one
 * layer's attention block: x [B*T, D], weights as in AttentionWeights.
 * dout is the upstream gradient of the block output. */
void ref_attention_fwd_bwd(const float* x, const float* w_qkv, const float* b_qkv,
                           const float* wo, const float* bo, const float* dout,
                           u32 B, u64 T, u32 H, u32 D,
                           float* out, float* dx, float* dw_qkv, float* db_qkv, float* dwo, float* dbo,
                           u64 arena_bytes) {
    Allocator a = allocator_create(arena_bytes);
    u64 N = (u64)B * T, hd = D / H;
    u64 sx[2] = { N, D }, sw[2] = { D, 3ull * D }, sb[1] = { 3ull * D }, so[2] = { D, D }, sbo[1] = { D };
    Tensor tx = tensor_create(&a, sx, 2);   memcpy(tx.data, x, N * D * 4);
    Tensor tw = tensor_create(&a, sw, 2);   memcpy(tw.data, w_qkv, (u64)D * 3 * D * 4);
    Tensor tb = tensor_create(&a, sb, 1);   memcpy(tb.data, b_qkv, 3ull * D * 4);
    Tensor two = tensor_create(&a, so, 2);  memcpy(two.data, wo, (u64)D * D * 4);
    Tensor tbo = tensor_create(&a, sbo, 1); memcpy(tbo.data, bo, (u64)D * 4);
    AttentionWeights w;
    Node* nx = node_leaf(&a, tx, TRUE);
    w.w_qkv = node_leaf(&a, tw, TRUE); w.b_qkv = node_leaf(&a, tb, TRUE);
    w.wo = node_leaf(&a, two, TRUE);   w.bo = node_leaf(&a, tbo, TRUE);
    u64 cs[2] = { T, hd / 2 };
    Tensor c = tensor_create(&a, cs, 2), s = tensor_create(&a, cs, 2);
    rope_build_tables(&c, &s, T, hd, 10000.0f);
    u64 ms[2] = { T, T };
    Tensor mask = tensor_create(&a, ms, 2);
    build_causal_mask(&mask);
    Node* y = causal_self_attention(&a, nx, &w, H, B, T, node_leaf(&a, c, FALSE), node_leaf(&a, s, FALSE),
                                    node_leaf(&a, mask, FALSE), 0);
    memcpy(out, y->value.data, N * D * 4);
    /* loss = sum(y * dout) seeds exactly dout as the upstream gradient */
    Tensor td = tensor_create(&a, sx, 2); memcpy(td.data, dout, N * D * 4);
    Node* loss = node_sum_all(&a, node_mul(&a, y, node_leaf(&a, td, FALSE)));
    backward(&a, loss);
    memcpy(dx, nx->grad.data, N * D * 4);
    memcpy(dw_qkv, w.w_qkv->grad.data, (u64)D * 3 * D * 4);
    memcpy(db_qkv, w.b_qkv->grad.data, 3ull * D * 4);
    memcpy(dwo, w.wo->grad.data, (u64)D * D * 4);
    memcpy(dbo, w.bo->grad.data, (u64)D * 4);
    allocator_destroy(&a);
}

/* swiglu_feedforward (model/feedforward.c:5-17) forward + backward. */
void ref_ffn_fwd_bwd(const float* x, const float* w_gu, const float* b_gu,
                     const float* w_down, const float* b_down, const float* dout,
                     u64 N, u32 D, u32 F,
                     float* out, float* dx, float* dw_gu, float* db_gu, float* dw_down, float* db_down,
                     u64 arena_bytes) {
    Allocator a = allocator_create(arena_bytes);
    u64 sx[2] = { N, D }, sg[2] = { D, 2ull * F }, sbg[1] = { 2ull * F }, sd[2] = { F, D }, sbd[1] = { D };
    Tensor tx = tensor_create(&a, sx, 2);   memcpy(tx.data, x, N * D * 4);
    Tensor tg = tensor_create(&a, sg, 2);   memcpy(tg.data, w_gu, (u64)D * 2 * F * 4);
    Tensor tbg = tensor_create(&a, sbg, 1); memcpy(tbg.data, b_gu, 2ull * F * 4);
    Tensor tdn = tensor_create(&a, sd, 2);  memcpy(tdn.data, w_down, (u64)F * D * 4);
    Tensor tbd = tensor_create(&a, sbd, 1); memcpy(tbd.data, b_down, (u64)D * 4);
    FeedForwardWeights w;
    Node* nx = node_leaf(&a, tx, TRUE);
    w.w_gate_up = node_leaf(&a, tg, TRUE); w.b_gate_up = node_leaf(&a, tbg, TRUE);
    w.w_down = node_leaf(&a, tdn, TRUE);   w.b_down = node_leaf(&a, tbd, TRUE);
    Node* y = swiglu_feedforward(&a, nx, &w, 0);
    memcpy(out, y->value.data, N * D * 4);
    Tensor td = tensor_create(&a, sx, 2); memcpy(td.data, dout, N * D * 4);
    Node* loss = node_sum_all(&a, node_mul(&a, y, node_leaf(&a, td, FALSE)));
    backward(&a, loss);
    memcpy(dx, nx->grad.data, N * D * 4);
    memcpy(dw_gu, w.w_gate_up->grad.data, (u64)D * 2 * F * 4);
    memcpy(db_gu, w.b_gate_up->grad.data, 2ull * F * 4);
    memcpy(dw_down, w.w_down->grad.data, (u64)F * D * 4);
    memcpy(db_down, w.b_down->grad.data, (u64)D * 4);
    allocator_destroy(&a);
}
