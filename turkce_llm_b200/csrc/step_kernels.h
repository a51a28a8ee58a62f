// Launchers of the kernels that complete a training step around the GEMMs: embedding,
// RMSNorm, RoPE split/merge, causal softmax, SwiGLU, cross-entropy, column sums, gradient
// norm and Adam.  All are bandwidth-bound row or element kernels; activations that feed a
// GEMM are written in bf16 so the tensor cores read them through TMA without a conversion
// pass.  None uses atomics: every reduction has a fixed order, so a step is bitwise
// reproducible (the reference's rule: cuda/train_kernels.cu:17-20).
#pragma once
#include "common.h"

namespace tb {

int launch_embed_fwd(DeviceCtx*, const float* E, const uint32_t* ids, float* x, int rows, int D, cudaStream_t);
// (out32, when given, receives the same values unrounded; out may then be NULL)
int launch_rmsnorm_fwd(DeviceCtx*, const float* x, const float* w, bf16* out, float* rinv, int rows, int cols,
                       float eps, cudaStream_t, float* out32 = nullptr);
// dx (+)= rmsnorm backward; dx16 = bf16(dx); wtmp[n,j] = dy*x*r (summed over rows by colsum)
int launch_rmsnorm_bwd(DeviceCtx*, const float* x, const float* w, const float* rinv, const float* dy, float* dx,
                       bf16* dx16, float* wtmp, int rows, int cols, int accumulate, cudaStream_t);
// the same with two column sums fused (fixed order): the norm-weight gradient dw[j] += sum_rows dy*x*r
// and, when db is given, db[j] += sum_rows dx[row, j] (the bias gradient of the layer that produced
// this residual stream).  scratch needs rmsnorm_bwd_scratch_floats(cols) floats, first 64 words zero.
size_t rmsnorm_bwd_scratch_floats(int cols);
int launch_rmsnorm_bwd_dw(DeviceCtx*, const float* x, const float* w, const float* rinv, const float* dy, float* dx,
                          bf16* dx16, float* dw, float* db, float* scratch, int rows, int cols, int accumulate,
                          cudaStream_t);
// Q [B,H,T,hd]; K, V [B,H,kv_cap,hd] (kv_cap = T for the trainer, the cache capacity for prefill)
int launch_rope_split(DeviceCtx*, const float* qkv, const float* cos_t, const float* sin_t, bf16* Q, bf16* K, bf16* V,
                      int B, int T, int H, int hd, int kv_cap, cudaStream_t);
// ---- decode with a KV cache [S, H, cap, hd] (bf16); *pos is the position of the new token
int launch_rope_decode(DeviceCtx*, const float* qkv, const float* cos_t, const float* sin_t, float* Q, bf16* Kc,
                       bf16* Vc, const int* pos, int S, int H, int hd, int cap, cudaStream_t);
int launch_attn_decode(DeviceCtx*, const float* Q, const bf16* Kc, const bf16* Vc, bf16* att, const int* pos, int S,
                       int H, int hd, int cap, float scale, cudaStream_t);
int launch_gather_last_rows(DeviceCtx*, const float* in, float* out, int S, int T, int D, cudaStream_t);
// state = {position of the next token, tokens generated so far} in device memory
int launch_rope_attn_decode(DeviceCtx*, const float* qkv, const float* cos_t, const float* sin_t, bf16* Kc, bf16* Vc,
                            bf16* att, const int* pos, int S, int H, int hd, int cap, float scale, cudaStream_t);
int launch_sample_rows(DeviceCtx*, const float* logits, const double* u, float temperature, uint32_t* tok,
                       uint32_t* out, int* state, int S, int V, long long ld, int out_ld, int advance_pos, cudaStream_t);
int launch_argmax_rows(DeviceCtx*, const float* logits, uint32_t* tok, uint32_t* out, int* state, int S, int V,
                       long long ld, int out_ld, int advance_pos, cudaStream_t);
int launch_rope_merge_bwd(DeviceCtx*, const float* dQ, const float* dK, const float* dV, const float* cos_t,
                          const float* sin_t, bf16* dqkv, int B, int T, int H, int hd, cudaStream_t);
// S [BH*T rows, leading dimension ld >= T] fp32 (entries j<=i valid) -> P bf16, same shape
// (zero from the diagonal to the end of its 128-tile)
int launch_attn_softmax_fwd(DeviceCtx*, const float* S, bf16* P, int BH, int T, long long ld, float scale,
                            cudaStream_t);
int launch_attn_softmax_bwd(DeviceCtx*, const bf16* P, const float* dP, bf16* dS, int BH, int T, long long ld,
                            float scale, cudaStream_t);
int launch_heads_split(DeviceCtx*, const bf16* dout, bf16* dO, int B, int T, int H, int hd, cudaStream_t);
// (h32 / dgu32, when given, receive the float32 values; the bf16 output may then be NULL)
int launch_swiglu_fwd(DeviceCtx*, const float* gu, bf16* h, int rows, int F, cudaStream_t, float* h32 = nullptr);
int launch_swiglu_bwd(DeviceCtx*, const float* gu, const float* dh, bf16* dgu, int rows, int F, cudaStream_t,
                      float* dgu32 = nullptr);
// the same with gate|up kept in bf16 by the fused SwiGLU GEMM epilogue
int launch_swiglu_bwd_bf16(DeviceCtx*, const bf16* gu, const float* dh, bf16* dgu, int rows, int F, cudaStream_t);
// ... and with the gate|up bias gradient (dbias[2F] += column sums of dgu) produced on the way;
// scratch holds swiglu_bwd_scratch_floats(F) floats
size_t swiglu_bwd_scratch_floats(int F);
int launch_swiglu_bwd_colsum(DeviceCtx*, const bf16* gu, const float* dh, bf16* dgu, float* dbias, float* scratch,
                             int rows, int F, cudaStream_t);
// logits [rows, ld] fp32 -> loss_rows, dlogits bf16 [rows, ld] = (softmax - onehot) * grad_scale
// combines the per-tile softmax statistics of the fused LM-head GEMM (GemmArgs::ce_mode 1):
// lse[row] and loss_rows[row] = lse - ztarget[row]; stats is [parts][rows] pairs (max, sum exp)
int launch_ce_combine(DeviceCtx*, const float* stats, int parts, int rows, const float* ztarget, float* lse,
                      float* loss_rows, cudaStream_t);
int launch_cross_entropy(DeviceCtx*, const float* logits, const uint32_t* targets, float* loss_rows, bf16* dlogits,
                         int rows, int V, long long ld, float grad_scale, cudaStream_t, float* dlogits32 = nullptr);
// out[c] += sum_r in[r,c]; in is fp32 or bf16; partial needs colsum_partial_floats(cols) floats, zeroed once
size_t colsum_partial_floats(int cols);
int launch_colsum_f32(DeviceCtx*, const float* in, float* out, float* partial, int rows, int cols, cudaStream_t);
int launch_colsum_bf16(DeviceCtx*, const bf16* in, float* out, float* partial, int rows, int cols, cudaStream_t);
// dE[token] += sum of dx rows of that token.  Rows sorted by token; each run cut into chunks of at most
// kEmbedChunk rows (seg_start/seg_token per chunk, meta = {first partial slot | 0xffffffff, chunk index,
// chunks in run}); nseg = number of chunks, in device memory; rows = launch size = number of rows.
// partial: embed_partial_slots(rows) * D floats; tickets: embed_partial_slots(rows) words, zero.
constexpr int kEmbedChunk = 16;
inline int embed_partial_slots(int rows) { return 2 * (rows / kEmbedChunk) + 2; }
int launch_embed_bwd(DeviceCtx*, const float* dx, const uint32_t* order, const uint32_t* seg_start,
                     const uint32_t* seg_token, const uint32_t* meta, const uint32_t* nseg, int rows, float* partial,
                     unsigned int* tickets, float* dE, int D, cudaStream_t);
constexpr int kNormBlocks = 1024;
int launch_sumsq_partial(DeviceCtx*, const float* x, long long n, float* partial, cudaStream_t);
// scalars[0] = norm (as float), scalars[1] = min(1, max_norm / norm) (1 when max_norm <= 0); norm64 = norm
int launch_clip_scale(DeviceCtx*, const float* partial, float max_norm, float grad_scale, float* scalars,
                      double* norm64, cudaStream_t);
// Adam; gradient is multiplied by grad_scale * (*dev_scale if given); writes the bf16 shadow copy too
int launch_adam(DeviceCtx*, float* p, bf16* p16, const float* g, float* m, float* v, long long n, float lr, float b1,
                float b2, float eps, float bc1, float bc2, float grad_scale, const float* dev_scale, cudaStream_t);

}  // namespace tb
