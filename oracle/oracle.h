/* TEST INFRASTRUCTURE ONLY.  CPU restatement (plain C) of the reference's
 * algorithms on the matrix-multiplication hot path.  Only tests/, the smoke
 * check and the bench's cpu_baseline / reference arm may load this library;
 * the product library never does.
 *
 * Parity of this restatement is PINNED: tests/test_oracle_pins.py checks it
 * bit-for-bit against the reference's own known-answer tests and against the
 * reference's CPU sources compiled unmodified (oracle/_ref/libref.so), and
 * against fixtures under tests/golden/ generated from that library.
 *
 * All matrices are row-major float32.  Citations give the reference file:line
 * each function follows (paths relative to the reference project).
 */
#ifndef ORACLE_H
#define ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* operand rounding applied to A and B before the multiply (accumulate is always
 * a single float32 accumulator walked in k order, tensor/tensor.c:351-373) */
enum { ORC_FP32 = 0, ORC_BF16 = 1, ORC_TF32 = 2 };

/* cuda/train_kernels.cu:207-212: round-to-nearest-even to bfloat16, returned
 * widened back to float32. No NaN/Inf special case, as in the reference. */
float orc_bf16_round(float f);
/* tcgen05 kind::tf32 reads the top 19 bits of a float32 operand: truncation. */
float orc_tf32_trunc(float f);
void orc_round_array(const float* in, float* out, int64_t n, int mode);

/* General GEMM with the interface of gemm_body / bf16_gemm_body
 * (cuda/train_kernels.cu:110-193, :343-467):
 *   C = alpha * op(A) @ op(B) + beta * C,  batch matrices at element strides.
 *   ta=0: A stored [M,K] (lda)   ta=1: A stored [K,M]
 *   tb=0: B stored [K,N] (ldb)   tb=1: B stored [N,K]
 * With alpha=1, beta=0, mode=ORC_FP32 the result is bit-identical to
 * tensor_matmul2d on the corresponding (possibly transposed) views. */
void orc_gemm(int ta, int tb, const float* A, const float* B, float* C,
              int M, int N, int K, int lda, int ldb, int ldc,
              int batch, int64_t sA, int64_t sB, int64_t sC,
              float alpha, float beta, int mode);

/* Same product accumulated in float64 (ground truth for error attribution). */
void orc_gemm_f64(int ta, int tb, const float* A, const float* B, double* C,
                  int M, int N, int K, int lda, int ldb, int ldc);

/* k_bf16_gemm_nn_bias (cuda/train_kernels.cu:226-329):
 * C = A[M,K] @ B[K,N] + bias[N] (+ residual[M,N]); NULL disables a term. */
void orc_gemm_bias(const float* A, const float* B, const float* bias, const float* residual,
                   float* C, int M, int N, int K, int mode);

/* k_colsum_acc (cuda/train_kernels.cu:518-531): out[c] += sum_r in[r,c]. */
void orc_colsum_acc(const float* in, float* out, int rows, int cols);

/* k_rmsnorm_fwd / k_rmsnorm_bwd (cuda/train_kernels.cu:535-569;
 * model/model_ops.c:52-80). bwd: dx += ..., dw += sum_rows(dy*x*r). */
void orc_rmsnorm_fwd(const float* x, const float* w, float* out, float* rinv, int rows, int cols, float eps);
void orc_rmsnorm_bwd(const float* x, const float* w, const float* rinv, const float* dy,
                     float* dx, float* dw, int rows, int cols);

/* model/rope.c:4-18 */
void orc_rope_tables(int T, int hd, float base, float* cos_t, float* sin_t);

/* k_qkv_rope_split / k_qkv_rope_merge_bwd (cuda/train_kernels.cu:573-626):
 * qkv [B*T, 3D] <-> Q,K (rotated), V in [B,H,T,hd]. */
void orc_qkv_rope_split(const float* qkv, const float* cos_t, const float* sin_t,
                        float* Q, float* K, float* V, int B, int T, int H, int hd);
void orc_qkv_rope_merge_bwd(const float* dQ, const float* dK, const float* dV,
                            const float* cos_t, const float* sin_t, float* dqkv,
                            int B, int T, int H, int hd);

/* Causal attention on head-major Q,K,V [BH,T,hd] (model/attention.c:32-60;
 * cuda/train_kernels.cu:631-664; model/gpu_train.c:346-358,435-455):
 * S = Q K^T * scale + mask(-1e9 above the diagonal), P = softmax(S), O = P V.
 * P_out may be NULL. mode rounds the MMA operands (Q,K,P,V / dO,dS). */
void orc_attention_fwd(const float* Q, const float* K, const float* V, float* O, float* P_out,
                       int BH, int T, int hd, float scale, int mode);
void orc_attention_bwd(const float* Q, const float* K, const float* V, const float* dO,
                       float* dQ, float* dK, float* dV,
                       int BH, int T, int hd, float scale, int mode);

/* k_heads_merge / k_heads_split (cuda/train_kernels.cu:667-692) */
void orc_heads_merge(const float* O, float* out, int B, int T, int H, int hd);
void orc_heads_split(const float* dout, float* dO, int B, int T, int H, int hd);

/* k_swiglu_fwd / k_swiglu_bwd (cuda/train_kernels.cu:695-721; model/feedforward.c:9-14) */
void orc_swiglu_fwd(const float* gu, float* h, int rows, int F);
void orc_swiglu_bwd(const float* gu, const float* dh, float* dgu, int rows, int F);

/* k_embed_fwd / k_embed_bwd (cuda/train_kernels.cu:724-740) */
void orc_embed_fwd(const float* E, const uint32_t* ids, float* x, int rows, int D);
void orc_embed_bwd(const float* dx, const uint32_t* ids, float* dE, int rows, int D);

/* k_cross_entropy (cuda/train_kernels.cu:747-772; model/loss.c:31-73):
 * loss_rows[n], logits <- (softmax - onehot) * grad_scale in place. */
void orc_cross_entropy(float* logits, const uint32_t* targets, float* loss_rows,
                       int rows, int V, int ld, float grad_scale);

/* k_adam (cuda/train_kernels.cu:787-800; training/adam.c:38-53) */
void orc_adam(float* p, const float* g, float* m, float* v, int64_t n,
              float lr, float b1, float b2, float eps, float bc1, float bc2, float grad_scale);

/* gpu_trainer_grad_norm (model/gpu_train.c:502-512): sqrt of the f64 sum. */
double orc_grad_norm(const float* g, int64_t n);

/* Whole model: the schedule of gpu_forward + gpu_backward
 * (model/gpu_train.c:312-474) with flat params/grads in lm_collect_params
 * order (model/lm_model.c:84-98).  mode rounds GEMM operands the way the
 * reference GPU trainer does (BF16 everywhere except the TN weight-gradient
 * GEMMs, which stay FP32: gpu_train.c:417,425,432,461 -- mode_dw rounds
 * those); ORC_FP32 = no rounding.
 * grads may be NULL (forward + loss only). Returns the mean loss
 * (mean over T inside a sequence, then over sequences: gpu_train.c:478-487).
 * logits_out (optional) receives the [B*T, V] logits before the loss. */
typedef struct OrcModelCfg {
    int V, D, H, L, F, T, B;
    float eps;
} OrcModelCfg;

int64_t orc_model_total_scalars(const OrcModelCfg* c);
float orc_model_forward_backward(const OrcModelCfg* c, const float* params,
                                 const uint32_t* ids, const uint32_t* targets,
                                 float* grads, float* logits_out, int mode, int mode_dw);

/* timing helper for the bench's cpu_baseline: number of worker threads in use */
int orc_num_threads(void);
void orc_set_num_threads(int n);

#ifdef __cplusplus
}
#endif
#endif
