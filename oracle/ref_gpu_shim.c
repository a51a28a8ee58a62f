/* TEST INFRASTRUCTURE ONLY -- never linked into or called by the product library.
 *
 * Plain-C entry points (for ctypes) around the reference's UNMODIFIED GPU-resident trainer
 * (model/gpu_train.c, cuda/cuda_backend.c, model/gpu_ops.c), which the recipe in
 * oracle/Makefile compiles from where the sources lie into oracle/_ref/librefgpu.so, next to
 * oracle/_ref/train_kernels.cubin = the reference's own cuda/train_kernels.cu compiled by nvcc
 * for sm_100a.  It gives the GPU tests the reference's own trainer as the full-size oracle (the
 * CPU path needs hours per step at 8 x 1024 tokens) and gives the measurements the kernels this
 * library replaces, running on the same B200.
 *
 * Nothing here restates the reference's arithmetic.  The one exception is the 3-line launch
 * geometry of the reference's static helper bf16_gemm_bias (model/gpu_train.c:103-107), which
 * refgpu_time_gemm_bias repeats in order to time that kernel alone.
 *
 * The reference creates a CUDA context of its own (cuCtxCreate_v2, cuda/cuda_backend.c:75) and
 * makes it current on every call: load this library in a process that uses no other CUDA
 * runtime state (oracle/ref_gpu.py runs as a child process for that reason).
 */
#include "runtime/types.h"
#include "runtime/memory.h"
#include "runtime/prng.h"
#include "runtime/timer.h"
#include "tensor/tensor.h"
#include "autograd/node.h"
#include "model/lm_model.h"
#include "model/gpu_train.h"
#include "cuda/cuda_backend.h"
#include "training/adam.h"
#include "training/lr_schedule.h"

#include <stdlib.h>
#include <string.h>

typedef struct RefGpu {
    Allocator alloc;
    LMModel model;
    Node* params[LM_MAX_LAYERS * 12 + 2];
    u32 np;
    AdamOptimizer opt;
    GpuTrainer gt;
    u32 B, T;
} RefGpu;

/* lm_init (model/lm_model.c:39-60) + lm_collect_params (:84-98) + adam_create (training/adam.c) +
 * gpu_trainer_create (model/gpu_train.c:144-251), in the order training/train_lm_gpu.c uses. */
RefGpu* refgpu_create(u32 V, u32 D, u32 H, u32 L, u32 F, float eps, u64 seed, u64 seq,
                      u32 B, u32 T, const char* module_path, u64 arena_bytes) {
    RefGpu* r = (RefGpu*)calloc(1, sizeof(RefGpu));
    r->alloc = allocator_create(arena_bytes);
    PCGState rng = pcg_seed(seed, seq);
    r->model = lm_init(&r->alloc, &rng, V, D, H, L, F, eps);
    r->np = lm_collect_params(&r->model, r->params);
    r->opt = adam_create(&r->alloc, r->params, r->np, 3e-4f, 0.9f, 0.999f, 1e-8f);
    r->B = B; r->T = T;
    r->gt = gpu_trainer_create(&r->alloc, module_path, &r->model, r->params, r->np, B, T);
    gpu_trainer_upload(&r->gt, r->params, &r->opt);
    return r;
}

void refgpu_destroy(RefGpu* r) {
    gpu_trainer_destroy(&r->gt);
    allocator_destroy(&r->alloc);
    free(r);
}

u64 refgpu_total_scalars(RefGpu* r) { return r->gt.total_scalars; }

static f32* refgpu_ptr(RefGpu* r, u32 i, int which) {
    switch (which) {
        case 0: return r->params[i]->value.data;
        case 1: return r->params[i]->grad.data;
        case 2: return r->opt.m[i].data;
        default: return r->opt.v[i].data;
    }
}

/* which: 0 = values, 1 = grads, 2 = adam m, 3 = adam v; flat, lm_collect_params order.
 * set: host mirror <- flat, then gpu_trainer_upload / gpu_trainer_upload_grads. */
void refgpu_set(RefGpu* r, int which, const float* flat) {
    u64 off = 0;
    for (u32 i = 0; i < r->np; i++) {
        u64 n = r->params[i]->value.numel;
        memcpy(refgpu_ptr(r, i, which), flat + off, n * sizeof(f32));
        off += n;
    }
    if (which == 1) gpu_trainer_upload_grads(&r->gt, r->params);
    else gpu_trainer_upload(&r->gt, r->params, &r->opt);
}

/* get: gpu_trainer_download / gpu_trainer_download_grads, then host mirror -> flat. */
void refgpu_get(RefGpu* r, int which, float* flat) {
    if (which == 1) gpu_trainer_download_grads(&r->gt, r->params);
    else gpu_trainer_download(&r->gt, r->params, &r->opt);
    u64 off = 0;
    for (u32 i = 0; i < r->np; i++) {
        u64 n = r->params[i]->value.numel;
        memcpy(flat + off, refgpu_ptr(r, i, which), n * sizeof(f32));
        off += n;
    }
}

float refgpu_forward_backward(RefGpu* r, const u32* ids, const u32* targets) {
    return gpu_trainer_forward_backward(&r->gt, ids, targets);
}
float refgpu_eval_loss(RefGpu* r, const u32* ids, const u32* targets) {
    return gpu_trainer_eval_loss(&r->gt, ids, targets);
}
double refgpu_grad_norm(RefGpu* r) { return gpu_trainer_grad_norm(&r->gt); }

void refgpu_adam_scaled(RefGpu* r, float lr, float grad_scale) {
    r->opt.lr = lr;
    gpu_trainer_adam_step_scaled(&r->gt, &r->opt, grad_scale);
}

void refgpu_sample_batch(const u32* tokens, u64 num_tokens, u32 T, u32 B, u64 seed_base,
                         u32* ids_out, u32* targets_out) {
    gpu_trainer_sample_batch(tokens, num_tokens, T, B, seed_base, ids_out, targets_out);
}

float refgpu_lr(u32 step, u32 warmup, u32 total, float peak, float min_lr) {
    return lr_warmup_cosine(step, warmup, total, peak, min_lr);
}

/* The body of the training loop of training/train_lm_gpu.c:212-223 for `steps` steps starting at
 * `step0`: schedule, window sampling with seed 2026 + step, forward+backward, global-norm clip,
 * scaled Adam.  losses_out[steps]; returns the wall-clock seconds of the loop (timer_now_seconds,
 * as the reference measures itself). */
double refgpu_train_loop(RefGpu* r, const u32* tokens, u64 num_tokens, u32 step0, u32 steps,
                         u32 warmup, u32 total_steps, float peak_lr, float min_lr, float clip,
                         float* losses_out, double* norms_out) {
    u64 n = (u64)r->B * r->T;
    u32* ids = (u32*)malloc(n * sizeof(u32));
    u32* tgt = (u32*)malloc(n * sizeof(u32));
    f64 t0 = timer_now_seconds();
    for (u32 s = 0; s < steps; s++) {
        u32 step = step0 + s;
        r->opt.lr = lr_warmup_cosine(step, warmup, total_steps, peak_lr, min_lr);
        gpu_trainer_sample_batch(tokens, num_tokens, r->T, r->B, 2026ull + step, ids, tgt);
        f32 loss = gpu_trainer_forward_backward(&r->gt, ids, tgt);
        f64 norm = gpu_trainer_grad_norm(&r->gt);
        f32 scale = (norm > clip) ? (f32)(clip / norm) : 1.0f;
        gpu_trainer_adam_step_scaled(&r->gt, &r->opt, scale);
        losses_out[s] = loss;
        if (norms_out) norms_out[s] = norm;
    }
    f64 t1 = timer_now_seconds();
    free(ids); free(tgt);
    return t1 - t0;
}

/* Times the reference's fused projection kernel k_bf16_gemm_nn_bias (cuda/train_kernels.cu:226-329)
 * alone: C[M,N] = A[M,K] @ B[K,N] + bias (+ residual), float32 in HBM, launched with the geometry
 * of bf16_gemm_bias (model/gpu_train.c:103-107).  Buffers hold zeros.  Returns seconds per launch
 * over `iters` back-to-back launches between two cuda_sync calls. */
double refgpu_time_gemm_bias(RefGpu* r, i32 M, i32 N, i32 K, int with_residual, int iters) {
    cuda_set_current(&r->gt.cuda);
    CUdeviceptr A = cuda_alloc((u64)M * K * 4), B = cuda_alloc((u64)K * N * 4);
    CUdeviceptr C = cuda_alloc((u64)M * N * 4), bias = cuda_alloc((u64)N * 4);
    CUdeviceptr res = with_residual ? cuda_alloc((u64)M * N * 4) : 0;
    cuda_memset_zero(A, (u64)M * K * 4); cuda_memset_zero(B, (u64)K * N * 4);
    cuda_memset_zero(bias, (u64)N * 4);
    if (res) cuda_memset_zero(res, (u64)M * N * 4);
    void* args[] = { &A, &B, &bias, &res, &C, &M, &N, &K };
    for (int i = 0; i < 3; i++)
        cuda_launch(r->gt.k_bf16_gemm_nn_bias, (u32)((N + 63) / 64), (u32)((M + 63) / 64), 1, 256, 1, 1, 0, args);
    cuda_sync();
    f64 t0 = timer_now_seconds();
    for (int i = 0; i < iters; i++)
        cuda_launch(r->gt.k_bf16_gemm_nn_bias, (u32)((N + 63) / 64), (u32)((M + 63) / 64), 1, 256, 1, 1, 0, args);
    cuda_sync();
    f64 t1 = timer_now_seconds();
    cuda_free(A); cuda_free(B); cuda_free(C); cuda_free(bias);
    if (res) cuda_free(res);
    return (t1 - t0) / (f64)iters;
}

/* The same for the general kernels k_bf16_gemm_{nn,nt,tn} / k_gemm_{nn,nt,tn}
 * (cuda/train_kernels.cu:110-193,343-467) with the geometry of bf16_gemm / gemm
 * (model/gpu_train.c:45-83).  kind: 0 NN, 1 NT, 2 TN; fp32_kernel != 0 picks k_gemm_*. */
double refgpu_time_gemm(RefGpu* r, int kind, int fp32_kernel, i32 M, i32 N, i32 K, u32 batch, int iters) {
    cuda_set_current(&r->gt.cuda);
    u64 na = (u64)M * K * batch, nb = (u64)K * N * batch, nc = (u64)M * N * batch;
    CUdeviceptr A = cuda_alloc(na * 4), B = cuda_alloc(nb * 4), C = cuda_alloc(nc * 4);
    cuda_memset_zero(A, na * 4); cuda_memset_zero(B, nb * 4); cuda_memset_zero(C, nc * 4);
    i32 lda = (kind == 2) ? M : K, ldb = (kind == 1) ? K : N, ldc = N;
    i64 sA = (i64)M * K, sB = (i64)K * N, sC = (i64)M * N;
    f32 alpha = 1.0f, beta = 0.0f;
    CUfunction f;
    if (fp32_kernel) f = (kind == 0) ? r->gt.k_gemm_nn : (kind == 1) ? r->gt.k_gemm_nt : r->gt.k_gemm_tn;
    else f = (kind == 0) ? r->gt.k_bf16_gemm_nn : (kind == 1) ? r->gt.k_bf16_gemm_nt : r->gt.k_bf16_gemm_tn;
    void* args[] = { &A, &B, &C, &M, &N, &K, &lda, &ldb, &ldc, &sA, &sB, &sC, &alpha, &beta };
    u32 bx = fp32_kernel ? 16 : 256, by = fp32_kernel ? 16 : 1;
    for (int i = 0; i < 2; i++)
        cuda_launch(f, (u32)((N + 63) / 64), (u32)((M + 63) / 64), batch, bx, by, 1, 0, args);
    cuda_sync();
    f64 t0 = timer_now_seconds();
    for (int i = 0; i < iters; i++)
        cuda_launch(f, (u32)((N + 63) / 64), (u32)((M + 63) / 64), batch, bx, by, 1, 0, args);
    cuda_sync();
    f64 t1 = timer_now_seconds();
    cuda_free(A); cuda_free(B); cuda_free(C);
    return (t1 - t0) / (f64)iters;
}

/* One GEMM launch through the reference's unmodified loader, with ANY module image: cuda_init (module load with
 * cuModuleLoadData, cuda/cuda_backend.c:56-107), cuda_get_kernel (:103-107), cuda_alloc / cuda_h2d, cuda_launch
 * (cuLaunchKernel on the NULL stream with the reference's void** parameter convention, :150-153), cuda_d2h.  The
 * caller gives the entry name, the host matrices and the launch geometry (the test computes it the way the reference's
 * static helpers do, model/gpu_train.c:45-118, cuda/cuda_backend.c:141-148).
 * form 0: the 14-parameter list of k_gemm_* / k_bf16_gemm_* (cuda/train_kernels.cu:187-188);
 * form 1: k_bf16_gemm_nn_bias(A, B, bias, residual, C, M, N, K) (:226-228), bias / residual may be NULL;
 * form 2: k_matmul(A, B, C, M, K, N) (cuda/kernels.cu:35).
 * C holds the initial output (read when beta != 0) and receives the result.  iters > 1 repeats the launch and the
 * function returns the seconds per launch of the repeated part (timer_now_seconds around cuda_sync), else 0. */
double refcuda_gemm(const char* module_path, const char* entry, int form,
                    const float* A, u64 nA, const float* B, u64 nB, const float* bias, const float* residual,
                    float* C, u64 nC, i32 M, i32 N, i32 K, i32 lda, i32 ldb, i32 ldc,
                    i64 sA, i64 sB, i64 sC, f32 alpha, f32 beta,
                    u32 gx, u32 gy, u32 gz, u32 bx, u32 by, int iters) {
    Allocator alloc = allocator_create(64ull << 20);
    CudaCtx ctx = cuda_init(&alloc, module_path);
    CUfunction f = cuda_get_kernel(&ctx, entry);
    CUdeviceptr dA = cuda_alloc(nA * 4), dB = cuda_alloc(nB * 4), dC = cuda_alloc(nC * 4);
    CUdeviceptr dbias = 0, dres = 0;
    cuda_h2d(dA, A, nA * 4); cuda_h2d(dB, B, nB * 4); cuda_h2d(dC, C, nC * 4);
    if (bias) { dbias = cuda_alloc((u64)N * 4); cuda_h2d(dbias, bias, (u64)N * 4); }
    if (residual) { dres = cuda_alloc(nC * 4); cuda_h2d(dres, residual, nC * 4); }
    void* args0[] = { &dA, &dB, &dC, &M, &N, &K, &lda, &ldb, &ldc, &sA, &sB, &sC, &alpha, &beta };
    void* args1[] = { &dA, &dB, &dbias, &dres, &dC, &M, &N, &K };
    void* args2[] = { &dA, &dB, &dC, &M, &K, &N };
    void** args = form == 0 ? args0 : form == 1 ? args1 : args2;
    cuda_launch(f, gx, gy, gz, bx, by, 1, 0, args);
    cuda_sync();
    cuda_d2h(C, dC, nC * 4);
    double sec = 0.0;
    if (iters > 1) {
        f64 t0 = timer_now_seconds();
        for (int i = 0; i < iters; i++) cuda_launch(f, gx, gy, gz, bx, by, 1, 0, args);
        cuda_sync();
        sec = (timer_now_seconds() - t0) / (f64)iters;
    }
    cuda_free(dA); cuda_free(dB); cuda_free(dC);
    if (dbias) cuda_free(dbias);
    if (dres) cuda_free(dres);
    cuda_shutdown(&ctx);
    allocator_destroy(&alloc);
    return sec;
}

/* The C-ABI route inside the reference's own context: cuda_init creates a context with cuCtxCreate and makes it
 * current (cuda/cuda_backend.c:56-107); the product library (libturkce_b200.so, CUDA runtime API) is then loaded and
 * its float32 entry point tb_gemm_bias_f32 is called on CUdeviceptr values from cuda_alloc -- the call the binding
 * stub of bf16_gemm_bias makes (model/gpu_train.c:103-107).  Returns the library's return code; tb_last_error's
 * text is copied to err (cap bytes). */
#include <dlfcn.h>
#include <stdio.h>
int refcuda_call_tb_gemm_bias(const char* module_path, const char* libtb_path, const float* A, const float* B,
                              const float* bias, const float* residual, float* C, i32 M, i32 N, i32 K, char* err, int cap) {
    Allocator alloc = allocator_create(64ull << 20);
    CudaCtx ctx = cuda_init(&alloc, module_path);
    void* h = dlopen(libtb_path, RTLD_NOW | RTLD_LOCAL);
    if (!h) { snprintf(err, cap, "dlopen failed: %s", dlerror()); return -100; }
    typedef int (*GemmBiasFn)(const float*, const float*, const float*, const float*, float*, int, int, int, int, void*);
    typedef int (*CheckFn)(void*);
    typedef const char* (*ErrFn)(void);
    GemmBiasFn gemm_bias = (GemmBiasFn)dlsym(h, "tb_gemm_bias_f32");
    CheckFn check_fn = (CheckFn)dlsym(h, "tb_check");
    ErrFn last_error = (ErrFn)dlsym(h, "tb_last_error");
    if (!gemm_bias || !check_fn || !last_error) { snprintf(err, cap, "symbols missing"); return -101; }
    CUdeviceptr dA = cuda_alloc((u64)M * K * 4), dB = cuda_alloc((u64)K * N * 4), dC = cuda_alloc((u64)M * N * 4);
    CUdeviceptr dbias = cuda_alloc((u64)N * 4), dres = cuda_alloc((u64)M * N * 4);
    cuda_h2d(dA, A, (u64)M * K * 4); cuda_h2d(dB, B, (u64)K * N * 4);
    cuda_h2d(dbias, bias, (u64)N * 4); cuda_h2d(dres, residual, (u64)M * N * 4);
    int rc = gemm_bias((const float*)dA, (const float*)dB, (const float*)dbias, (const float*)dres, (float*)dC, M, N, K,
                       0 /* TB_PREC_BF16 */, NULL);
    if (rc == 0) rc = check_fn(NULL);
    if (rc != 0) snprintf(err, cap, "%s", last_error());
    cuda_sync();
    if (rc == 0) cuda_d2h(C, dC, (u64)M * N * 4);
    cuda_free(dA); cuda_free(dB); cuda_free(dC); cuda_free(dbias); cuda_free(dres);
    cuda_shutdown(&ctx);
    allocator_destroy(&alloc);
    return rc;
}
