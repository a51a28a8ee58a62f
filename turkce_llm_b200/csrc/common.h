// Shared host-side declarations of the library: error reporting, the per-device
// context (scratch memory, error word, driver entry points) and the launchers the
// C-ABI layer and the trainer call.
#pragma once
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <vector>

namespace tb {

typedef __nv_bfloat16 bf16;

// ---- errors: every entry point returns 0 on success; the message of the last
// failure on the calling thread is kept for tb_last_error().
void set_error(const char* fmt, ...);
const char* last_error();

#define TB_CUDA(expr)                                                                        \
    do {                                                                                     \
        cudaError_t _e = (expr);                                                             \
        if (_e != cudaSuccess) {                                                             \
            tb::set_error("[CUDA] %s -> %s: %s (%s:%d)", #expr, cudaGetErrorName(_e),        \
                          cudaGetErrorString(_e), __FILE__, __LINE__);                       \
            return -1;                                                                       \
        }                                                                                    \
    } while (0)

#define TB_CHECK(cond, ...)                  \
    do {                                     \
        if (!(cond)) {                       \
            tb::set_error(__VA_ARGS__);      \
            return -2;                       \
        }                                    \
    } while (0)

#define TB_TRY(expr)              \
    do {                          \
        int _r = (expr);          \
        if (_r != 0) return _r;   \
    } while (0)

// cudaMemcpy from pageable host memory may return once the data sits in the driver's staging buffer, before
// the DMA into device memory (ordered on the legacy default stream) has finished.  The work of this library runs
// on non-blocking streams, which do not wait for that stream: wait for it here, so that a kernel launched right
// after an upload never reads the old contents.
#define TB_H2D_SYNC(dst, src, bytes)                                             \
    do {                                                                         \
        TB_CUDA(cudaMemcpy((dst), (src), (bytes), cudaMemcpyHostToDevice));      \
        TB_CUDA(cudaStreamSynchronize(cudaStreamLegacy));                        \
    } while (0)

// ---- optional per-launch timing: one event in front of a launch (prof_mark) and one behind it
// (prof_close); the difference is the kernel's own time even when the host is the bottleneck.
struct ProfRec { const char* tag; cudaEvent_t ev; cudaEvent_t ev_end; double flops; double bytes; };

// ---- per-device context
struct DeviceCtx {
    int device = -1;
    int sm_count = 0;
    int* d_err = nullptr;
    // device error word written by kernels whose bounded waits ran out
    unsigned int* d_tickets = nullptr;   // 32 zeroed words behind the error word, for single-launch tickets
    unsigned long long* d_best = nullptr; // 64 zeroed words for the fused LM head's packed maxima
    void* scratch = nullptr;       // growable scratch (operand packing, split-K partials)
    size_t scratch_bytes = 0;
    long long launches = 0;        // kernels launched by this library on this device
    bool prof_on = false;
    std::vector<ProfRec>* prof = nullptr;
};

// Records a timing mark when profiling is on (no-op otherwise).
void prof_mark(DeviceCtx* ctx, const char* tag, double flops, double bytes, cudaStream_t stream);
// Records the closing event of the last mark (no-op when profiling is off).
void prof_close(DeviceCtx* ctx, cudaStream_t stream);
// Returns a pointer that stays valid for the life of the process (for composed tags).
const char* prof_intern(const char* text);

// Returns the context of the current device, creating it on first use.
int get_ctx(DeviceCtx** out);
// Makes sure the scratch buffer holds at least `bytes`; may reallocate (synchronises).
int ensure_scratch(DeviceCtx* ctx, size_t bytes);
// Reads and clears the device error word (synchronises the stream first).
int check_device_error(DeviceCtx* ctx, cudaStream_t stream);

// ---- GEMM on BF16 operands (gemm_tcgen05.cu)
enum GemmKind { GEMM_NN = 0, GEMM_NT = 1, GEMM_TN = 2 };
enum CausalMode {
    CAUSAL_NONE = 0,
    CAUSAL_SKIP_UPPER = 1,   // square score-shaped output: tiles wholly above the diagonal are not computed
    CAUSAL_K_PREFIX = 2,     // A is lower-triangular [M,K]: k runs only to the end of the tile's rows
    CAUSAL_K_SUFFIX = 3      // op(A) = A^T of a lower-triangular matrix: k starts at the tile's first row
};

struct GemmArgs {
    GemmKind kind = GEMM_NN;
    const void* A = nullptr;   // NN/NT: [M,K] lda   TN: [K,M] lda   (bf16, or float32 when tf32 is set)
    const void* B = nullptr;   // NN/TN: [K,N] ldb   NT: [N,K] ldb
    int M = 0, N = 0, K = 0;
    long long lda = 0, ldb = 0;
    int batch = 1;
    long long strideA = 0, strideB = 0;     // elements
    // outputs: either or both
    float* C32 = nullptr; long long ldc32 = 0, strideC32 = 0, strideC32_in = 0;
    bf16* C16 = nullptr;  long long ldc16 = 0, strideC16 = 0, strideC16_in = 0;
    int c_inner = 1;   // >1: output of batch z goes to (z / c_inner) * strideC + (z % c_inner) * strideC_in
    const float* bias = nullptr;            // [N]
    const float* residual = nullptr; long long ldr = 0, strideR = 0;   // [M,N] fp32
    float alpha = 1.0f, beta = 0.0f;        // beta applies to the previous contents of C32
    CausalMode causal = CAUSAL_NONE;
    int splits = 0;                         // 0 = choose; >1 uses scratch for fixed-order partial sums
    int bn = 0;                             // 0 = choose tile width (64, 128 or 192; 256 = a CTA pair on a 256 x 256 tile)
    int max_ctas = 0;                       // > 0: at most this many CTAs (two products that share the SMs side by side)
    // SwiGLU backward in the epilogue (bf16 NT product with N = F, the input gradient of the down-projection): the
    // product dh [M, F] is not stored; with the saved gate|up projection dsw_gu [M, 2F] (leading dimension ldgu) the
    // tile leaves as dsw_dgu [M, 2F] (same leading dimension): dg = dh u s (1 + g (1 - s)), du = dh g s, s = sigmoid(g).
    // F must be a multiple of 64.
    const bf16* dsw_gu = nullptr;
    bf16* dsw_dgu = nullptr;
    bool tf32 = false;                      // operands are float32 in memory and enter the tensor cores as tf32
    bool pad_cols_writable = false;         // columns N .. round_up(N, 16 bytes) of each output row are padding
    // Fused SwiGLU epilogue (kind NN, N = 2F with gate columns [0,F) and up columns [F,2F), F % 64 == 0):
    // h[M,F] = silu(g) * u with g, u = the product (+bias) -- the activation the reference computes in
    // k_swiglu_fwd from the stored projection (cuda/train_kernels.cu:695-707).  Each tile pairs 64 gate
    // columns with their 64 up columns.  swiglu_gu (optional, bf16 [M,2F]) keeps g and u for the backward pass.
    bf16* swiglu_h = nullptr;  long long ldh = 0;
    bf16* swiglu_gu = nullptr; long long ldgu = 0;
    // Cross-entropy fused into the LM-head product (kind NT, bn = 192 or 256, no other output), so that the
    // [M, N] logits never exist in HBM (the reference writes them and k_cross_entropy reads them back,
    // model/gpu_train.c:378-381, cuda/train_kernels.cu:742-775).
    //   ce_mode 1: per row and per half tile (bn/2 columns), max and sum of exp(z - max) -> ce_stats
    //              [2 * ceil(N/bn)][M] float2, and the target's logit -> ce_ztarget[M]
    //   ce_mode 2: the product is formed again and leaves as C16 = (exp(z - ce_lse[row]) - onehot) * ce_scale
    // QKV projection with the position embedding fused (kind NN, N = 3*H*hd, hd 32 or 64, T % 32 == 0, M = B*T):
    // instead of the float32 [M, 3D] projection and k_qkv_rope_split (cuda/train_kernels.cu:573-597), the
    // epilogue rotates the interleaved pairs of the q and k columns with the [T, hd/2] tables and stores
    // bf16 tiles straight into rope_qkv = [3][B][H][T][hd] (Q, K, V of equal size, back to back)
    bf16* rope_qkv = nullptr;
    const float* rope_cos = nullptr; const float* rope_sin = nullptr;
    int rope_T = 0, rope_H = 0, rope_hd = 0;
    int ce_mode = 0;
    const uint32_t* ce_targets = nullptr;
    float* ce_stats = nullptr;
    float* ce_ztarget = nullptr;
    const float* ce_lse = nullptr;
    float ce_scale = 1.0f;
};

int launch_gemm_bf16(DeviceCtx* ctx, const GemmArgs& a, cudaStream_t stream);
// split-K with caller-provided partial-sum storage (needs splits*batch*M*N floats)
int launch_gemm_bf16_ws(DeviceCtx* ctx, const GemmArgs& a, float* workspace, size_t workspace_floats,
                        cudaStream_t stream);
int choose_splits(const DeviceCtx* ctx, const GemmArgs& a, int bn);
// TMA map over a bf16 matrix seen as (inner, rows, batch) with a 64-element x box_rows box, 128B swizzle
int make_operand_map(CUtensorMap* map, const bf16* ptr, long long inner, long long rows, long long ld, int batch,
                     long long batch_stride, int box_rows);
// the same over a float32 matrix: 32-element x box_rows box
int make_operand_map_f32(CUtensorMap* map, const float* ptr, long long inner, long long rows, long long ld, int batch,
                         long long batch_stride, int box_rows);
// the same over a 4-level view (inner, rows, batch0, batch1) -- e.g. one head of a [B*T, H*hd] matrix
int make_operand_map4(CUtensorMap* map, const bf16* ptr, long long inner, long long rows, long long ld,
                      long long n0, long long stride0, long long n1, long long stride1, int box_rows);

// ---- fused causal attention (attention.cu); Q, K, V bf16 [B*H, T, hd] (hd <= 64, multiple of 8)
// forward: att bf16 [B*T, H*hd] (heads merged), lse float [B*H, T] (natural-log sum of exponentials)
// (lse may be NULL; kv_rows_per_head > T when K and V live in a KV cache with that many rows per head)
int launch_attention_fwd(DeviceCtx* ctx, const bf16* Q, const bf16* K, const bf16* V, bf16* att, float* lse, int B,
                         int H, int T, int hd, float scale, cudaStream_t stream, long long kv_rows_per_head = 0);
// backward: datt bf16 [B*T, H*hd] -> dQ, dK, dV float [B*H, T, hd]; delta is float scratch [B*H, T]
int launch_attention_bwd(DeviceCtx* ctx, const bf16* Q, const bf16* K, const bf16* V, const bf16* att,
                         const bf16* datt, const float* lse, float* delta, float* dQ, float* dK, float* dV, int B,
                         int H, int T, int hd, float scale, cudaStream_t stream, bf16* dqkv = nullptr,
                         const float* cos_t = nullptr, const float* sin_t = nullptr, bf16* ds_blocks = nullptr);
// (dqkv given: the gradients leave merged as bf16 [B*T, 3*H*hd] with the inverse rotation of the position
//  embedding applied to dQ and dK; dQ, dK, dV are then unused and may be NULL.
//  ds_blocks: attention_bwd_ds_bytes(B, H, T) bytes through which the dK/dV kernel hands the dS blocks to the dQ
//  kernel (lower-triangular 128 x 128 blocks, bf16); NULL = the context's growable scratch)
size_t attention_bwd_ds_bytes(int B, int H, int T);

// ---- the decode step of all layers as one cooperative kernel (decode_mega.cu)
struct DecodeMega;
bool decode_mega_supported(const DeviceCtx* ctx, int S, int D, int H, int F, int cap);
int decode_mega_create(DeviceCtx* ctx, DecodeMega** out, int S, int D, int H, int F, int L, int cap, float eps, float scale);
void decode_mega_destroy(DecodeMega* m);
// slab copies of the weights + the per-layer pointer table; offsets = the flat parameter offsets (embedding first)
int decode_mega_set_weights(DeviceCtx* ctx, DecodeMega* m, const float* params, const bf16* params16, const long long* offsets,
                            bf16* const* Kc, bf16* const* Vc, cudaStream_t st);
// x (float32 [S, D]) = the last layer's output for the tokens tok at position *pos; K and V rows appended to the caches
int launch_decode_mega(DeviceCtx* ctx, DecodeMega* m, const uint32_t* tok, const int* pos, const float* cos_t, const float* sin_t,
                       float* x, float* x2, float* qkv, bf16* att, bf16* h, cudaStream_t st);

// ---- operand packing (pack.cu)
// float32 [rows, cols] -> float32 copy with another leading dimension (makes a matrix TMA-addressable)
int launch_copy_f32(DeviceCtx* ctx, const float* src, float* dst, int rows, int cols, long long ld_src,
                    long long ld_dst, int batch, long long stride_src, long long stride_dst, cudaStream_t stream);
// float32 x -> three tf32-exact pieces for the 3xTF32 product: hi = x truncated to tf32, lo = x - hi.
// along_cols: dst [rows, 3*cols] = [p0 | p1 | p2], else dst [3*rows, cols] = [p0 ; p1 ; p2];
// pattern 0: (hi, hi, lo)   pattern 1: (hi, lo, hi)
int launch_split3_f32(DeviceCtx* ctx, const float* src, float* dst, int rows, int cols, long long ld_src,
                      long long ld_dst, int along_cols, int pattern, int batch, long long stride_src,
                      long long stride_dst, cudaStream_t stream);
// float32 [rows, cols] (ld) -> bf16 [rows, cols] (ld_out), batched
// Decode-time LM head with fused greedy choice (lmhead_decode.cu): tok[s] = argmax_v <X[s,:], E[v,:]>,
// S <= 64 rows of X [S, K] bf16, E [V, K] bf16; best (64 words) and ticket (1 word) are zeroed device
// memory that no concurrent launch shares (the kernel leaves them zero).  table_is_stable: E is not written by
// earlier work of the stream, so its loads may start before that work has finished.
// Also stores the token as out[s, state[1]] and advances state = {position, generated} like launch_argmax_rows
// (out and state may be NULL).  logits (optional, [S, ld_logits] float32) receives the full products.
bool lmhead_argmax_supported(const DeviceCtx* ctx, int S, int V, int K);
int lmhead_argmax_ctas(const DeviceCtx* ctx, int S, int V, int K);
int launch_lmhead_argmax(DeviceCtx* ctx, const bf16* X, const bf16* E, int S, int V, int K, bool table_is_stable,
                         unsigned long long* best, unsigned int* ticket, uint32_t* tok, uint32_t* out, int* state,
                         int out_ld, int advance_pos, float* logits, long long ld_logits, cudaStream_t st);

// Linear layer of a decode step for S <= 64 rows (decode_linear.cu): y32 [S, N] = X W + bias (+ residual), or with
// h16 given (N = 2F) h16 [S, F] = silu(gate) * up.  X is bf16 [S, K], or x32 float32 [S, K] with the RMSNorm
// (norm_w, eps) fused in front.  W bf16 [K, N] row-major.  N % 128 == 0 (F % 64 == 0), K % 64 == 0, K <= 1024.
bool decode_linear_supported(int S, int N, int K, bool swiglu);
int launch_decode_linear(DeviceCtx* ctx, const bf16* X16, const float* x32, const float* norm_w, float eps, const bf16* W,
                         const float* bias, const float* residual, float* y32, bf16* h16, int S, int N, int K,
                         cudaStream_t st);

int launch_pack_bf16(DeviceCtx* ctx, const float* src, bf16* dst, int rows, int cols, long long ld_src,
                     long long ld_dst, int batch, long long stride_src, long long stride_dst, cudaStream_t stream);

// bf16 -> float32, n elements (n % 4 == 0)
int launch_widen_bf16(DeviceCtx* ctx, const bf16* src, float* dst, long long n, cudaStream_t stream);

static inline long long round_up(long long x, long long m) { return (x + m - 1) / m * m; }

// ---- launches with programmatic dependent launch: the next kernel of the stream may be scheduled
// and run its prologue while this one drains; every kernel of this library therefore executes
// pdl_wait() before it touches global memory (a no-op for a launch without the attribute).
int pdl_mode();     // 0 off, 1 every launch, 2 only launches with >= 64 KB of dynamic shared memory

// cluster_x > 1: thread-block clusters of that many CTAs along x (the grid must be a multiple of it)
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel_cluster(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                         cudaStream_t stream, int cluster_x, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int n = 0;
    const int mode = pdl_mode();
    if (mode == 1 || (mode == 2 && smem >= 65536)) {
        attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cluster_x > 1) {
        attr[n].id = cudaLaunchAttributeClusterDimension;
        attr[n].val.clusterDim.x = (unsigned)cluster_x; attr[n].val.clusterDim.y = 1; attr[n].val.clusterDim.z = 1;
        ++n;
    }
    cfg.attrs = n ? attr : nullptr;
    cfg.numAttrs = (unsigned)n;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                 Args&&... args) {
    return launch_kernel_cluster(kernel, grid, block, smem, stream, 1, static_cast<Args&&>(args)...);
}

#ifdef __CUDACC__
// waits until every kernel this launch depends on has completed and its writes are visible
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// lets the next kernel of the stream start launching
__device__ __forceinline__ void pdl_launch_dependents_now() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
#ifndef TB_PDL_STEP_LATE
    pdl_launch_dependents_now();
#endif
}
#endif

}  // namespace tb
