/* turkce_b200 -- C ABI of the sm_100a matrix-multiplication hot path.
 *
 * Plain pointers and sizes only.  Every pointer named d_* is a CUDA device pointer
 * on the current device; h_* is host memory.  `stream` is a cudaStream_t passed as
 * void* (NULL = the default stream).  Every function returns 0 on success; on
 * failure it returns non-zero and tb_last_error() gives the message.  The reference
 * treats every CUDA error as fatal (cuda/cuda_backend.c:15-34): a C caller keeps that
 * behaviour by printing tb_last_error() and exiting on a non-zero return.
 *
 * Citations name the reference interface each entry point replaces
 * (paths relative to the reference project).
 */
#ifndef TURKCE_B200_H
#define TURKCE_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GEMM kinds: the reference's GemmKind (model/gpu_train.c:41) */
#define TB_GEMM_NN 0   /* A [M,K] lda, B [K,N] ldb */
#define TB_GEMM_NT 1   /* A [M,K] lda, B [N,K] ldb */
#define TB_GEMM_TN 2   /* A [K,M] lda, B [K,N] ldb */

/* operand precision of the tensor-core product; accumulation is always FP32.
 * BF16: operands rounded to bf16 (kind::f16).  TF32: float32 operands read as tf32 (kind::tf32).
 * FP32: each operand split into two tf32-exact pieces and multiplied as hi*hi + hi*lo + lo*hi
 * (three TF32 products in one accumulator): about 2^-20 relative error, for the <= 1e-5 bound. */
#define TB_PREC_BF16 0
#define TB_PREC_TF32 1
#define TB_PREC_FP32 2

/* causal structure of batched square attention products (see tb_gemm_bf16) */
#define TB_CAUSAL_NONE 0
#define TB_CAUSAL_SKIP_UPPER 1
#define TB_CAUSAL_K_PREFIX 2
#define TB_CAUSAL_K_SUFFIX 3

/* ---- library / device ------------------------------------------------------ */

/* cuda_init_on_device + cuda_set_current (cuda/cuda_backend.h:19-40): selects the
 * device for the calling thread and creates the library's per-device state. */
int tb_init(int device);
/* cuda_device_count (cuda/cuda_backend.h:27) */
int tb_device_count(void);
const char* tb_last_error(void);
/* Number of kernels this library has launched on the current device so far. */
long long tb_launch_count(void);
/* Waits for `stream` and reports a kernel that gave up on a bounded wait. */
int tb_check(void* stream);
/* cuda_shutdown (cuda/cuda_backend.h:33): frees the library's scratch memory. */
int tb_shutdown(void);
/* Per-launch timing with CUDA events (the reference only has wall-clock counters,
 * model/gpu_ops.c:57-68).  Between begin and end every launch of this library on the
 * current device is timed; end writes one text line per kernel:
 * "<name> <launches> <total ms> <algorithmic flops> <algorithmic bytes>". */
int tb_profile_begin(void);
int tb_profile_end(void* stream, char* out, int cap);

/* cuda_alloc / cuda_free / cuda_h2d / cuda_d2h / cuda_memset_zero / cuda_sync
 * (cuda/cuda_backend.h:42-65) for C callers that have no other CUDA runtime. */
int tb_alloc(void** d_ptr, uint64_t bytes);
int tb_free(void* d_ptr);
int tb_h2d(void* d_dst, const void* h_src, uint64_t bytes);
int tb_d2h(void* h_dst, const void* d_src, uint64_t bytes);
int tb_memset_zero(void* d_ptr, uint64_t bytes);
int tb_sync(void);

/* ---- GEMM on float32 device matrices (the reference's storage format) ------- */

/* gemm() / bf16_gemm() host helpers and the k_gemm_{nn,nt,tn} / k_bf16_gemm_{nn,nt,tn}
 * kernels they launch (model/gpu_train.c:45-78; cuda/train_kernels.cu:187-193, :343-467):
 *   C = alpha * op(A) @ op(B) + beta * C   for `batch` matrices at element strides.
 * Operands are rounded to `precision` (bf16: round-to-nearest-even, as
 * cuda/train_kernels.cu:207-212) on the way into the tensor cores. */
int tb_gemm_f32(int kind, const float* d_A, const float* d_B, float* d_C,
                int M, int N, int K, int lda, int ldb, int ldc,
                int batch, int64_t strideA, int64_t strideB, int64_t strideC,
                float alpha, float beta, int precision, void* stream);

/* bf16_gemm_bias() and k_bf16_gemm_nn_bias (model/gpu_train.c:103-107;
 * cuda/train_kernels.cu:226-329): C[M,N] = A[M,K] @ B[K,N] + bias[N] (+ residual[M,N]);
 * a NULL bias or residual is skipped. All matrices contiguous. */
int tb_gemm_bias_f32(const float* d_A, const float* d_B, const float* d_bias, const float* d_residual,
                     float* d_C, int M, int N, int K, int precision, void* stream);

/* gpu_matmul() behind node_matmul2d_gpu, and k_matmul (model/gpu_ops.c:118-160;
 * cuda/kernels.cu:35-65): host matrices in, host matrix out, copies included.
 * C[M,N] = A[M,K] @ B[K,N], all contiguous row-major float32 in host memory.
 * Like the reference's worker slots (model/gpu_ops.c:31-46,78-102) every calling host thread keeps its own three
 * device buffers per device, grown on demand and reused, so repeated calls allocate nothing; threads may call
 * concurrently (the product itself is serialised per process: the library's scratch is one per device). */
int tb_matmul_host(const float* h_A, const float* h_B, float* h_C, int M, int K, int N, int precision);

/* ---- GEMM on bf16 device matrices (native format of this library) ----------- */

/* Same product on operands already in bf16 (leading dimensions and batch strides must
 * be multiples of 8 elements, pointers 16-byte aligned).  Either or both outputs may
 * be given: d_C32 float32 (beta applies to its previous contents), d_C16 bf16.
 * bias [N] and residual [M,N] (float32, leading dimension ldr, batch stride strideR)
 * are optional.  `causal` restricts batched square attention products to the lower
 * triangle: SKIP_UPPER leaves output tiles wholly above the diagonal unwritten;
 * K_PREFIX / K_SUFFIX shorten the k range for a lower-triangular A / transposed A.
 * splits: 0 = chosen by the library; >1 = split-K with fixed-order partial sums
 * (bitwise reproducible, as the reference requires: cuda/train_kernels.cu:17-20). */
int tb_gemm_bf16(int kind, const void* d_A, const void* d_B, int M, int N, int K,
                 int64_t lda, int64_t ldb, int batch, int64_t strideA, int64_t strideB,
                 float* d_C32, int64_t ldc32, int64_t strideC32,
                 void* d_C16, int64_t ldc16, int64_t strideC16,
                 const float* d_bias, const float* d_residual, int64_t ldr, int64_t strideR,
                 float alpha, float beta, int causal, int splits, int tile_n, void* stream);

/* No counterpart in the reference.  The split-K form of tb_gemm_bf16 for hosts that must not
 * allocate device memory: processes whose HBM is wholly owned by another allocator, and loops
 * that cannot take cudaMalloc's device-wide synchronisation.  It calls no cudaMalloc / cudaFree
 * and no allocating library routine; the per-split partial sums go to a 16 MiB array built into
 * the library image (held by every GPU that loads the library until the process exits), so
 * splits * M * N must not exceed 4,194,304 floats -- larger problems are rejected with an error.
 *   C32 = alpha * op(A) @ op(B) [+ bias] [+ beta * C32],  one matrix, bf16 operands as tb_gemm_bf16.
 * splits: 0 = chosen by the library, else the number of K splits (partials are added in split
 * order: bitwise reproducible).  wait != 0: the call waits for `stream` and returns non-zero if a
 * kernel gave up on a bounded wait; wait == 0: fully asynchronous.
 * The first call on a device looks up the array's device address (cudaGetSymbolAddress) and
 * queries device attributes; make that first call before any stream capture begins.  (That set-up is
 * guarded by a mutex: two host threads may make their first calls at the same time.)
 * All calls on a device share the one array and one status word: two calls whose kernels can
 * overlap on the GPU (different streams, no ordering between them) race on them.  Every call clears the
 * status word on its stream before it launches, so a caller that passes wait == 0 must read the word
 * with tb_gemm_bf16_splitk_static_status before its next call, or a time-out goes unreported
 * (tb_check reads a different word and allocates on first use). */
int tb_gemm_bf16_splitk_static(int kind, const void* d_A, const void* d_B, int M, int N, int K,
                               int64_t lda, int64_t ldb, float* d_C32, int64_t ldc32,
                               const float* d_bias, float alpha, float beta, int splits, int wait, void* stream);

/* No counterpart in the reference.  Waits for `stream` and returns non-zero if a kernel of an earlier
 * tb_gemm_bf16_splitk_static call on this device gave up on a bounded wait.  Allocates nothing. */
int tb_gemm_bf16_splitk_static_status(void* stream);

/* float32 [rows, cols] (ld_src) -> bf16 [rows, cols] (ld_dst), `batch` matrices. */
int tb_pack_bf16(const float* d_src, void* d_dst, int rows, int cols, int64_t ld_src, int64_t ld_dst,
                 int batch, int64_t stride_src, int64_t stride_dst, void* stream);

/* Gate|up projection of the SwiGLU feed-forward with the activation fused into the GEMM epilogue:
 * [g | u] = X[M,K] . W[K,2F] + bias[2F] (gate columns [0,F), up columns [F,2F)), H[M,F] = silu(g) * u.
 * Replaces bf16_gemm_bias (model/gpu_train.c:364) followed by k_swiglu_fwd (cuda/train_kernels.cu:695-707;
 * CPU definition model/feedforward.c:9-14) without the float32 [M,2F] projection in HBM.  X, W bf16 row-major;
 * H bf16 [M,F]; GU (optional, bf16 [M,2F]) keeps g and u for the backward pass.  F must be a multiple of 64. */
int tb_gemm_swiglu_bf16(const void* d_X, const void* d_W, const float* d_bias, int M, int F, int K, void* d_H,
                        void* d_GU, void* stream);

/* QKV projection with the position embedding and the head split fused into the GEMM epilogue:
 * bf16_gemm_bias (model/gpu_train.c:338) followed by k_qkv_rope_split (model/gpu_train.c:339-343,
 * cuda/train_kernels.cu:573-597; CPU definition model/attention.c:26-29,50-53 with model/rope.c:20-47).
 *   qkv = X[B*T, D] . W[D, 3D] + bias[3D]   (D = H*hd; row n holds q | k | v of token n, head h at column h*hd)
 * q and k are rotated pairwise ((2k, 2k+1) by the angle of (position, k), tables cos/sin [T, hd/2] float32),
 * and all three leave as bf16 in d_QKV = [3][B][H][T][hd] (Q, K, V back to back, the layout tb_attention_fwd
 * reads).  X, W bf16 row-major; hd 32 or 64; T a multiple of 32; tables 16-byte aligned. */
int tb_gemm_qkv_rope_bf16(const void* d_X, const void* d_W, const float* d_bias, const float* d_cos, const float* d_sin,
                          int B, int T, int H, int hd, void* d_QKV, void* stream);

/* One linear layer of a decode step for S <= 64 sequences (the reference has no decode path: its generator re-runs
 * lm_forward per token, training/generate.c:186-212; the products are the layer's projections, model/attention.c:26,67
 * and model/feedforward.c:9-16, with model_ops.c's RMSNorm in front of the QKV and gate|up projections):
 *   Y[S, N] = X[S, K] . W[K, N] + bias[N] (+ residual[S, N])             d_y32 float32
 *   or, with d_h16 given (N = 2F): H[S, F] = silu(g + b_g) * (u + b_u)    d_h16 bf16, [g | u] = X W
 * X is either bf16 (d_X16) or float32 rows (d_x32) that the kernel normalises itself: X = x * rsqrt(mean x^2 + eps) * w.
 * W bf16 row-major; K a multiple of 64 up to 1024; N a multiple of 128 (F a multiple of 64).  A weight-streaming
 * kernel: the slab of W a CTA needs is requested before the previous kernel of the stream has finished. */
int tb_decode_linear(const void* d_X16, const float* d_x32, const float* d_norm_w, float eps, const void* d_W,
                     const float* d_bias, const float* d_residual, float* d_y32, void* d_h16, int S, int N, int K,
                     void* stream);

/* Decode-time LM head with the greedy choice fused: d_tok[s] = argmax_v <X[s,:], E[v,:]> (lowest index
 * on ties) for 1 <= S <= 64 rows of X [S, K] bf16 against the tied embedding table E [V, K] bf16, K a
 * multiple of 64.  The [S, V] logits (lm_forward's last rows, model/lm_model.c:72-81, whose argmax
 * model/generate.c:204-206 takes when sampling is off) are not written unless d_logits is given
 * (float32 [S, ld_logits]).  E is streamed from HBM exactly once; uses the library scratch buffer.
 * table_is_stable != 0 promises that no earlier work still running on the stream writes E (weights
 * during generation): the kernel then starts streaming E while that work finishes.  Calls that can
 * overlap on the GPU (different streams) must not share a device: they share one ticket word. */
int tb_lmhead_argmax_bf16(const void* d_X, const void* d_E, int S, int V, int K, uint32_t* d_tok, float* d_logits,
                          int64_t ld_logits, int table_is_stable, void* stream);

/* ---- fused causal attention ---------------------------------------------------- */

/* The per-head attention contractions of the reference's GPU trainer in one kernel: QK^T
 * (k_bf16_gemm_nt), causal softmax (k_attn_softmax_fwd), P V (k_bf16_gemm_nn) and k_heads_merge
 * (model/gpu_train.c:346-358; cuda/train_kernels.cu:631-651, :667-678).
 * d_Q, d_K, d_V: bf16 [B*H, T, hd] with RoPE applied (the output layout of k_qkv_rope_split),
 * hd <= 64 and a multiple of 8.  d_att: bf16 [B*T, H*hd] (heads merged).  d_lse: float [B*H, T],
 * log of the row's sum of exponentials, kept for the backward pass in place of P [B,H,T,T]. */
int tb_attention_fwd(const void* d_Q, const void* d_K, const void* d_V, void* d_att, float* d_lse, int B, int H, int T,
                     int hd, float scale, void* stream);
/* Backward of the same chain: k_heads_split, the dV / dP / dQ / dK products and
 * k_attn_softmax_bwd (model/gpu_train.c:435-455; cuda/train_kernels.cu:655-664, :681-692).
 * d_att, d_datt: bf16 [B*T, H*hd] (forward output and its gradient); d_delta: float scratch
 * [B*H, T]; d_dQ, d_dK, d_dV: float [B*H, T, hd] (gradients of the rotated Q, K and of V). */
int tb_attention_bwd(const void* d_Q, const void* d_K, const void* d_V, const void* d_att, const void* d_datt,
                     const float* d_lse, float* d_delta, float* d_dQ, float* d_dK, float* d_dV, int B, int H, int T,
                     int hd, float scale, void* stream);

/* ---- GPU-resident trainer ---------------------------------------------------- */

/* GpuTrainer (model/gpu_train.h:51-80).  Parameters, gradients and Adam state are flat
 * float32 buffers in lm_collect_params order (model/lm_model.c:84-98): embedding [V,D];
 * per layer attn_norm [D], w_qkv [D,3D], b_qkv [3D], wo [D,D], bo [D], ffn_norm [D],
 * w_gate_up [D,2F], b_gate_up [2F], w_down [F,D], b_down [D]; final_norm [D]. */
typedef struct TbTrainer TbTrainer;

/* gpu_trainer_create (model/gpu_train.h:86-92): the architecture comes as numbers instead of
 * an LMModel*, the weights through tb_trainer_upload.  d_model, d_ff and head_dim must be
 * multiples of 8.  All work of this trainer is issued on `stream`. */
int tb_trainer_create(TbTrainer** out, int V, int D, int H, int L, int F, int T, int B, float eps, void* stream);
/* The same with the operand precision of the linear-layer GEMMs (forward, dX, dW and the LM head) chosen:
 * TB_PREC_BF16 (what tb_trainer_create gives) or TB_PREC_TF32 -- float32 weights and activations read by the
 * tensor cores as tf32 (kind::tf32), float32 accumulation; the attention core stays the fused bf16 kernel in
 * both (the reference's attention products are bf16: model/gpu_train.c:346-353).  Other values are rejected. */
int tb_trainer_create_prec(TbTrainer** out, int V, int D, int H, int L, int F, int T, int B, float eps, int precision,
                           void* stream);
/* gpu_trainer_destroy (model/gpu_train.h:93) */
int tb_trainer_destroy(TbTrainer* g);
int64_t tb_trainer_total_scalars(const TbTrainer* g);
int tb_trainer_num_params(const TbTrainer* g);                       /* 10*L + 2 */
int tb_trainer_param_layout(const TbTrainer* g, int64_t* offsets, int64_t* numels);
/* The architecture and step shape the trainer was created with (any pointer may be NULL). */
int tb_trainer_dims(const TbTrainer* g, int* V, int* D, int* H, int* L, int* F, int* T, int* B);

/* `which` selects a flat buffer: 0 parameters, 1 gradients, 2 Adam m, 3 Adam v.
 * gpu_trainer_upload / gpu_trainer_upload_grads (model/gpu_train.h:97,103) */
int tb_trainer_upload(TbTrainer* g, int which, const float* h_flat);
/* gpu_trainer_download / gpu_trainer_download_grads (model/gpu_train.h:99,101) */
int tb_trainer_download(TbTrainer* g, int which, float* h_flat);
/* Device address of a flat buffer (for a collective over the gradients). */
void* tb_trainer_device_ptr(TbTrainer* g, int which);
/* The cudaStream_t all of this trainer's work is issued on: the one given to tb_trainer_create,
 * or a stream of the trainer's own when that was NULL (the step is replayed from CUDA graphs,
 * which cannot be captured on the default stream). */
void* tb_trainer_stream(TbTrainer* g);

/* gpu_trainer_forward_backward (model/gpu_train.h:114): zeroes the gradients, runs forward and
 * backward on host ids/targets [B*T], returns the mean loss (mean inside a sequence, then over
 * sequences) and leaves the mean gradients on the device. */
int tb_trainer_forward_backward(TbTrainer* g, const uint32_t* h_ids, const uint32_t* h_targets, float* loss_out);
/* gpu_trainer_eval_loss (model/gpu_train.h:119): forward only; bit-identical to the loss of
 * tb_trainer_forward_backward on the same input. */
int tb_trainer_eval_loss(TbTrainer* g, const uint32_t* h_ids, const uint32_t* h_targets, float* loss_out);
/* gpu_trainer_grad_norm (model/gpu_train.h:122): global L2 norm, fixed summation order. */
int tb_trainer_grad_norm(TbTrainer* g, double* norm_out);
/* gpu_trainer_adam_step_scaled (model/gpu_train.h:125) with the optimiser's scalars passed in;
 * t is the step counter after the increment (first step: 1). grad_scale 1 = gpu_trainer_adam_step. */
int tb_trainer_adam_step_scaled(TbTrainer* g, uint64_t t, float lr, float beta1, float beta2, float eps,
                                float grad_scale);
/* One iteration of the training loop (training/train_lm_gpu.c:212-223): forward, backward,
 * gradient norm, clip to max_norm (<= 0: no clipping) and Adam, with a single host read. */
int tb_trainer_train_step(TbTrainer* g, const uint32_t* h_ids, const uint32_t* h_targets, uint64_t t, float lr,
                          float beta1, float beta2, float eps, float max_norm, float* loss_out, double* norm_out);

/* The same step in pieces, so that a data-parallel caller can start the all-reduce of a
 * layer's gradients while the layers below are still in backward (the multi-GPU extension of
 * training/data_parallel.c:119-163).  Order: zero_grads, forward(want_grad=1), backward_head,
 * backward_layer(L-1 .. 0), backward_embed, [all-reduce], clip_adam_async, read_loss. */
int tb_trainer_zero_grads(TbTrainer* g);
int tb_trainer_forward(TbTrainer* g, const uint32_t* h_ids, const uint32_t* h_targets, int want_grad);
int tb_trainer_backward_head(TbTrainer* g);
int tb_trainer_backward_layer(TbTrainer* g, int layer);
int tb_trainer_backward_embed(TbTrainer* g);
/* grad_scale multiplies the gradients before the norm is taken and clipped (1/world_size after a sum over
 * ranks, 1/micro-batches after accumulation): the reported and clipped norm is that of the averaged gradients. */
int tb_trainer_clip_adam_async(TbTrainer* g, uint64_t t, float lr, float beta1, float beta2, float eps,
                               float max_norm, float grad_scale);
int tb_trainer_read_loss(TbTrainer* g, float* loss_out);
/* Copies host ids/targets to the device (and prepares the embedding-gradient row order)
 * without running anything; tb_trainer_step_resident then runs complete training steps on
 * those device-resident inputs with no host transfer and no host synchronisation. */
int tb_trainer_set_inputs(TbTrainer* g, const uint32_t* h_ids, const uint32_t* h_targets);
int tb_trainer_step_resident(TbTrainer* g, uint64_t t, float lr, float beta1, float beta2, float eps,
                             float max_norm);
/* Forward on the device-resident inputs (the staged form of tb_trainer_step_resident). */
int tb_trainer_forward_resident(TbTrainer* g, int want_grad);
/* Gradient norm computed by the last tb_trainer_clip_adam_async (waits for the stream). */
int tb_trainer_last_norm(TbTrainer* g, double* norm_out);

/* ---- the training loop around the trainer (host code) ---------------------------- */

/* gpu_trainer_sample_batch (model/gpu_train.h:108-109, model/gpu_train.c:296-307; the same windows as the
 * CPU workers of training/data_parallel.c:73-77): sequence w of the batch starts at a position drawn from
 * PCG32 seeded (seed_base * 1000003 + w, stream 99 + w), uniformly in [0, num_tokens - T - 1); targets are
 * the ids shifted by one.  ids_out, targets_out: [B * T].  Host memory only. */
int tb_sample_batch(const uint32_t* tokens, uint64_t num_tokens, int T, int B, uint64_t seed_base,
                    uint32_t* ids_out, uint32_t* targets_out);
/* Sequences [first_sequence, first_sequence + count) of the same step: what one rank of a data-parallel job
 * draws.  A sequence's window depends on its index in the GLOBAL batch only (the reference's worker w,
 * training/data_parallel.c:132-133), so the set of windows of a step does not depend on the number of ranks. */
int tb_sample_batch_range(const uint32_t* tokens, uint64_t num_tokens, int T, int first_sequence, int count,
                          uint64_t seed_base, uint32_t* ids_out, uint32_t* targets_out);
/* n draws of pcg_uniform (runtime/prng.c:34-37) from the generator seeded (seed, seq): [0, 1) in steps of 2^-32. */
int tb_pcg_uniform_fill(uint64_t seed, uint64_t seq, uint64_t n, double* out);
/* lr_warmup_cosine (training/lr_schedule.c:6-15): peak * (step + 1) / warmup during warm-up, then a
 * cosine from peak to min over the remaining steps. */
float tb_lr_warmup_cosine(uint64_t step, uint64_t warmup_steps, uint64_t total_steps, float peak_lr, float min_lr);
/* checkpoint_save / checkpoint_load (training/checkpoint.h:6-12,30-41) on the trainer's device state, in the
 * reference's "TRLM" version-1 file format, byte for byte: header, per tensor [ndim][shape][values], then,
 * with_optimizer != 0, per tensor Adam m and v, then the step counter.  Save writes <path>.tmp and renames
 * it; load validates the whole file against the model before it touches the trainer, and with_optimizer != 0
 * requires the optimiser state to be in the file.  A checkpoint written by the reference loads here and
 * the other way round. */
int tb_checkpoint_save(const char* path, TbTrainer* g, int with_optimizer, uint64_t adam_t);
int tb_checkpoint_load(const char* path, TbTrainer* g, int with_optimizer, uint64_t* adam_t_out);
/* The loop of training/train_lm_gpu.c:212-223 for steps [start_step, start_step + num_steps): schedule,
 * windows drawn with seed 2026 + step, forward, backward, global-norm clip at max_norm, Adam.  *adam_t is
 * the optimiser's step counter (incremented per step).  The next step's windows are drawn on the host while
 * the device runs the current step; ids travel through pinned memory; the loss read-back is the only host
 * synchronisation of a step.  losses_out / norms_out: [num_steps] or NULL. */
int tb_trainer_run(TbTrainer* g, const uint32_t* tokens, uint64_t num_tokens, uint32_t start_step, uint32_t num_steps,
                   uint32_t warmup_steps, uint32_t total_steps, float peak_lr, float min_lr, float max_norm,
                   float beta1, float beta2, float eps, uint64_t* adam_t, float* losses_out, double* norms_out);

/* ---- data parallelism over the GPUs of one box ----------------------------------------- */

/* The multi-GPU extension of data_parallel_step (training/data_parallel.h:20-35, training/data_parallel.c:119-163).
 * The reference hands one sequence to each CPU worker thread, adds the workers' gradients in a fixed order,
 * divides by the worker count (dp_reduce_run, :102-117) and averages the workers' losses.  Here a worker is a
 * rank: one process or host thread per GPU, each with its own TbTrainer (a full replica, created with the
 * per-rank batch), and the flat float32 gradient buffers are summed over the ranks by NCCL over NVLink;
 * 1 / ranks is folded into Adam's gradient scale, and every rank ends the step with bit-identical weights.
 * NCCL is loaded at run time (libnccl.so.2, or the path in TB_NCCL_LIB); one rank alone needs no NCCL. */
typedef struct TbDp TbDp;
#define TB_DP_ALLREDUCE 0   /* one all-reduce of the flat gradient buffer (the loss rides in a spare slot) */
#define TB_DP_SHARDED   1   /* reduce-scatter, Adam on this rank's 1/ranks slice, all-gather of the weights */
#define TB_DP_OVERLAP   2   /* the all-reduce in per-layer buckets on a side stream, under the rest of the backward pass */
/* Rank 0 calls this and hands the 128 bytes to every rank (through whatever channel launched them). */
int tb_dp_unique_id(void* id_out_128_bytes);
/* Collective over the ranks (creates the NCCL communicator); unique_id may be NULL when world == 1. */
int tb_dp_create(TbDp** out, TbTrainer* g, const void* unique_id, int rank, int world, int mode);
int tb_dp_destroy(TbDp* dp);
/* Host arithmetic of TB_DP_SHARDED: the slice [first, first + count) of the flat buffers that `rank` owns, and the
 * chunk (scalars per rank in the reduce-scatter / all-gather, a multiple of 8).  The slices tile [0, total). */
int tb_dp_slice(int64_t total, int world, int rank, int64_t* chunk, int64_t* first, int64_t* count);
int tb_dp_info(const TbDp* dp, int* rank, int* world, int* mode, int* nccl_version);
/* One optimiser step: data_parallel_step + the clipped Adam step of the training loop
 * (training/train_lm.c:184-194, training/train_lm_gpu.c:212-223).  h_ids / h_targets hold this rank's
 * `micro_batches` batches of B * T tokens back to back; their gradients accumulate in the flat buffer (every
 * backward kernel adds, as the reference's do), the ranks' sums are combined once, and
 * 1 / (ranks * micro_batches) scales the gradients before the norm is taken and clipped at max_norm.
 * loss_out: mean loss over all ranks and micro-batches; norm_out: the global gradient norm.  With one rank
 * and one micro-batch the step equals tb_trainer_train_step bit for bit. */
int tb_dp_step(TbDp* dp, const uint32_t* h_ids, const uint32_t* h_targets, int micro_batches, uint64_t t, float lr,
               float beta1, float beta2, float eps, float max_norm, float* loss_out, double* norm_out);
/* The same step on the device-resident inputs of tb_trainer_set_inputs: no host transfer, no host
 * synchronisation; tb_dp_last_result waits for the stream and returns that step's loss and norm. */
int tb_dp_step_resident(TbDp* dp, uint64_t t, float lr, float beta1, float beta2, float eps, float max_norm);
int tb_dp_last_result(TbDp* dp, float* loss_out, double* norm_out);

/* ---- decoding with a KV cache --------------------------------------------------- */

/* The reference generates by re-running lm_forward over the whole window for every new token
 * (training/generate.c:186-212, training/chat.c:139-165) and has no KV cache; this engine computes
 * the same last-row logits incrementally.  The next token is the greedy choice (argmax) unless
 * tb_decoder_set_sampling selects the reference's temperature sampling.  max_seqs sequences are decoded in lockstep, each with room for max_len
 * positions; the parameters are the trainer's flat float32 layout. */
typedef struct TbDecoder TbDecoder;
int tb_decoder_create(TbDecoder** out, int V, int D, int H, int L, int F, int max_seqs, int max_len, float eps,
                      void* stream);
int tb_decoder_destroy(TbDecoder* g);
int64_t tb_decoder_total_scalars(const TbDecoder* g);
int tb_decoder_upload(TbDecoder* g, const float* h_flat);
/* h_ids: [max_seqs, prompt_len] prompt tokens; fills the cache and chooses the first new token. */
int tb_decoder_prefill(TbDecoder* g, const uint32_t* h_ids, int prompt_len);
/* sample_next (training/generate.c:57-73): with temperature > 0 every next token (the prefill's included) is
 * drawn from softmax(logits / temperature) by inverse CDF in ascending token order, float64 running sum.
 * Sequence s uses the PCG32 stream (seed, seq + s), one pcg_uniform per generated token -- (4242, 7) is the
 * reference generator's stream for its single sequence.  temperature <= 0 goes back to greedy.  Call before
 * tb_decoder_prefill; the sampled head writes the [S, V] logits (the greedy head does not). */
int tb_decoder_set_sampling(TbDecoder* g, float temperature, uint64_t seed, uint64_t seq);
/* n more tokens per sequence; asynchronous (one CUDA-graph launch per token). */
int tb_decoder_generate(TbDecoder* g, int n);
/* h_out: [max_seqs, count], the first `count` generated tokens of every sequence (waits). */
int tb_decoder_read_tokens(TbDecoder* g, uint32_t* h_out, int count);
/* h_logits: [max_seqs, V], the logits the most recent token was chosen from (waits). */
int tb_decoder_read_logits(TbDecoder* g, float* h_logits);
void* tb_decoder_stream(TbDecoder* g);

#ifdef __cplusplus
}
#endif
#endif /* TURKCE_B200_H */
