// Linear layers of a decode step: Y[S, N] = f(X)[S, K] . W[K, N] + bias (+ residual) for S <= 64 sequences.
//
// The reference has no decode path (it re-runs lm_forward over the whole window per token,
// training/generate.c:186-212); the products are those of its layer: the QKV, output, gate|up and down projections
// (model/attention.c:26,67, model/feedforward.c:9-16) with the RMSNorm in front of the first and third
// (model/transformer_block.c:7-15, model/model_ops.c) and the SwiGLU behind the third (model/feedforward.c:9-14).
//
// With 64 rows these products are pure weight streaming (0.3 - 1.6 MB per matrix) and a step is bound by the number
// and latency of its launches, so this kernel is built to start its weight stream at once and to carry its neighbours:
//   * a CTA owns 128 output columns; the weight slab W[:, n0:n0+128] is the M = 128 operand of tcgen05.mma (MN-major
//     tiles straight from the row-major matrix), the activations are the N = 64 operand, the accumulator
//     [128 columns x 64 sequences] lives in 64 TMEM columns;
//   * every TMA load of the slab that fits the ring is issued before griddepcontrol.wait: the weights do not
//     depend on the previous kernel, so they stream while it drains;
//   * the RMSNorm of the input is fused in front (each CTA normalises the 64 rows itself, the arithmetic of
//     rmsnorm_fwd_vec_kernel, and writes the bf16 operand straight into its swizzled shared-memory tile), and the
//     bias, the residual add and silu(gate) * up are fused behind.
// One decode layer is five launches of 3 - 16 CTAs instead of seven launches of the general persistent GEMM.
// Measured on a B200 (cycle stamps inside the kernel, weights cold in HBM): set-up 0.9 us, the RMSNorm prologue of 64
// rows on 8 warps 3.0 us, a 98 KB slab arrives at 10 - 25 B/clk per SM, the epilogue takes 2 us; a launch is 8 - 10 us
// against 6 us for the general kernel, which spreads the same weights over twice as many SMs.  The decoder therefore
// uses this kernel only on request (TB_DECODE_LEAN=1).
#include "common.h"
#include "ptx.cuh"

#include <algorithm>
#include <cstdlib>

namespace tb {

namespace {

constexpr int DL_THREADS = 256;
constexpr int DL_SEQ = 64;                   // sequences = UMMA N
constexpr int DL_COLS = 128;                 // output columns per CTA = UMMA M
constexpr int DL_BK = 64;                    // bf16 elements of one 128-byte row
constexpr int DL_X_SLICE = DL_SEQ * 128;     // one K slice of the activations
constexpr int DL_W_BOX = DL_BK * 128;        // one 64 (columns) x 64 (k) box of the weights
constexpr int DL_W_SLICE = 2 * DL_W_BOX;     // one K slice of the slab
constexpr int DL_HEADER = 1024;
constexpr int DL_MAX_RING = 8;
constexpr int DL_MAX_KBLOCKS = 16;           // K <= 1024
constexpr int DL_MAX_SMEM = 227 * 1024;
constexpr int DL_PART_LD = 68;               // floats per parked accumulator row: 16-byte rows, conflict-free

struct DecLinParams {
    int S, K, N, kblocks, ring;
    int ks;                    // K splits: a cluster of ks CTAs shares one slab, each taking kblocks K slices; rank 0
                               // adds the partial accumulators in rank order through distributed shared memory
    int norm;                  // 1: X = RMSNorm(x32) formed here; 0: X bf16 by TMA
    const float* x32; const float* norm_w; float eps;
    int swiglu, F;             // 1: the slab pairs 64 gate columns with their 64 up columns, output h16 [S, F]
    const float* bias; const float* residual;
    float* y32; bf16* h16;
    int* err;
};

// RMSNorm of the 64 input rows into the K-major 128-byte-swizzle operand tile: y = x * r * w with
// r = 1 / sqrt(mean(x^2) + eps) -- the arithmetic and summation order of rmsnorm_fwd_vec_kernel (lane owns columns
// 4 * (lane + 32 k) .. + 3, xor-shuffle tree over the lanes).  One warp takes rows warp, warp + 8, ...; four rows are
// in flight at a time so that their loads and reductions overlap.  Element k of row s goes to slice k / 64 at
// s * 128 + ((chunk ^ (s & 7)) << 4), chunk = (k % 64) / 8; a CTA of a K split keeps only its own K range.
template <int NV>
__device__ __forceinline__ void norm_rows(const DecLinParams& p, uint8_t* sX, int kb0, int warp, int lane) {
    const int K = p.K;
    float4 wv[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int j = 4 * (lane + 32 * k);
        wv[k] = j < K ? __ldg(reinterpret_cast<const float4*>(p.norm_w + j)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    constexpr int ROWS = DL_SEQ / (DL_THREADS / 32);      // 8 rows per warp
    constexpr int BATCH = NV <= 4 ? 4 : 2;
#pragma unroll 1
    for (int b0 = 0; b0 < ROWS; b0 += BATCH) {
        float4 xv[BATCH][NV];
        float ss[BATCH];
#pragma unroll
        for (int b = 0; b < BATCH; ++b) {
            const int s = warp + 8 * (b0 + b);
            const float* xr = p.x32 + (long long)s * K;
#pragma unroll
            for (int k = 0; k < NV; ++k) {
                const int j = 4 * (lane + 32 * k);
                xv[b][k] = (s < p.S && j < K) ? __ldg(reinterpret_cast<const float4*>(xr + j)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
#pragma unroll
        for (int b = 0; b < BATCH; ++b) {
            float a = 0.0f;
#pragma unroll
            for (int k = 0; k < NV; ++k)
                a += xv[b][k].x * xv[b][k].x + xv[b][k].y * xv[b][k].y + xv[b][k].z * xv[b][k].z + xv[b][k].w * xv[b][k].w;
            ss[b] = a;
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
            for (int b = 0; b < BATCH; ++b) ss[b] += __shfl_xor_sync(0xffffffffu, ss[b], o);
        }
#pragma unroll
        for (int b = 0; b < BATCH; ++b) {
            const int s = warp + 8 * (b0 + b);
            const float ms = ss[b] / (float)K;
            const float r = 1.0f / (float)sqrt((double)(ms + p.eps));
#pragma unroll
            for (int k = 0; k < NV; ++k) {
                const int j = 4 * (lane + 32 * k);
                const int jl = j - kb0 * DL_BK;                      // position inside this CTA's K range
                if (j < K && jl >= 0 && jl < p.kblocks * DL_BK) {
                    __nv_bfloat162 lo = __floats2bfloat162_rn(xv[b][k].x * r * wv[k].x, xv[b][k].y * r * wv[k].y);
                    __nv_bfloat162 hi = __floats2bfloat162_rn(xv[b][k].z * r * wv[k].z, xv[b][k].w * r * wv[k].w);
                    uint2 pk;
                    pk.x = *reinterpret_cast<uint32_t*>(&lo); pk.y = *reinterpret_cast<uint32_t*>(&hi);
                    const int chunk = (jl & 63) >> 3;
                    *reinterpret_cast<uint2*>(sX + (jl >> 6) * DL_X_SLICE + s * 128 + ((chunk ^ (s & 7)) << 4) + (jl & 7) * 2) = pk;
                }
            }
        }
    }
}

__global__ void __launch_bounds__(DL_THREADS, 1)
decode_linear_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX,
                     const DecLinParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    uint64_t* w_full = bars;                          // [ring]
    uint64_t* w_empty = bars + DL_MAX_RING;           // [ring]
    uint64_t* x_bar = bars + 2 * DL_MAX_RING;
    uint64_t* acc_bar = bars + 2 * DL_MAX_RING + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * DL_MAX_RING + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    uint8_t* sX = smem + DL_HEADER;                                  // [kblocks][64 rows][128 B]
    uint8_t* sW = sX + p.kblocks * DL_X_SLICE;                       // [ring][2 boxes][64 k][128 B]
    float* exch = reinterpret_cast<float*>(sW);                      // SwiGLU: up values [64 units][65], over the consumed ring
    float* part = reinterpret_cast<float*>(sW);                      // K splits: this CTA's accumulator [128][68], likewise

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int rank = p.ks > 1 ? (int)cluster_ctarank() : 0;          // which K range of the slab
    const int slab = (int)blockIdx.x / p.ks;
    const int kb0 = rank * p.kblocks;                                // first K slice of this CTA (p.kblocks = slices per CTA)
    const int n0 = slab * DL_COLS;
    // first column of the two 64-column boxes of this CTA's slab
    const int box_col0 = p.swiglu ? slab * 64 : n0;
    const int box_col1 = p.swiglu ? p.F + slab * 64 : n0 + 64;

    if (tid == 0) {
        for (int i = 0; i < p.ring; ++i) { mbar_init(&w_full[i], 1); mbar_init(&w_empty[i], 1); }
        mbar_init(x_bar, 1);
        mbar_init(acc_bar, 1);
        *abort_flag = 0;
        fence_mbar_init();
        // the first `ring` slices of the slab, before the fence on the previous kernel: weights are not its output
        const int first = p.ring < p.kblocks ? p.ring : p.kblocks;
        for (int kb = 0; kb < first; ++kb) {
            mbar_expect_tx(&w_full[kb], DL_W_SLICE);
            tma_load_3d(sW + kb * DL_W_SLICE, &tmW, &w_full[kb], box_col0, (kb0 + kb) * DL_BK, 0);
            tma_load_3d(sW + kb * DL_W_SLICE + DL_W_BOX, &tmW, &w_full[kb], box_col1, (kb0 + kb) * DL_BK, 0);
        }
        if (!p.norm) tma_prefetch_desc(&tmX);
    }
    if (warp == 1) { tmem_alloc(tmem_slot, 64); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();                      // the activations come from the previous kernel of the stream

    if (p.norm) {
        if (p.K <= 384) norm_rows<3>(p, sX, kb0, warp, lane);
        else if (p.K <= 512) norm_rows<4>(p, sX, kb0, warp, lane);
        else norm_rows<8>(p, sX, kb0, warp, lane);
        fence_proxy_async();          // the tensor core reads the tile through the async proxy
    }
    __syncthreads();

    if (warp == 0 && lane == 0) {
        // ---- producer: the activations (when they arrive as bf16) and the rest of the slab
        bool ok = true;
        if (!p.norm) {
            mbar_expect_tx(x_bar, (uint32_t)(p.kblocks * DL_X_SLICE));
            for (int kb = 0; kb < p.kblocks; ++kb) tma_load_3d(sX + kb * DL_X_SLICE, &tmX, x_bar, (kb0 + kb) * DL_BK, 0, 0);
        }
        for (int kb = p.ring; kb < p.kblocks && ok; ++kb) {
            const int slot = kb % p.ring;
            const uint32_t phase = (uint32_t)(kb / p.ring - 1) & 1u;          // the (kb / ring)-th reuse of the slot
            if (!mbar_wait(&w_empty[slot], phase, abort_flag)) { ok = false; break; }
            mbar_expect_tx(&w_full[slot], DL_W_SLICE);
            tma_load_3d(sW + slot * DL_W_SLICE, &tmW, &w_full[slot], box_col0, (kb0 + kb) * DL_BK, 0);
            tma_load_3d(sW + slot * DL_W_SLICE + DL_W_BOX, &tmW, &w_full[slot], box_col1, (kb0 + kb) * DL_BK, 0);
        }
        pdl_launch_dependents_now();
        if (!ok) { *abort_flag = 1; atomicExch(p.err, 51); }
    } else if (warp == 1 && lane == 0) {
        // ---- MMA issuer: D[128 columns, 64 sequences] += W_slab^T (MN-major) . X^T (K-major)
        const uint32_t idesc = umma_idesc(1u, 1u, 0u, DL_COLS, DL_SEQ);
        bool ok = p.norm ? true : mbar_wait(x_bar, 0u, abort_flag);
        for (int kb = 0; kb < p.kblocks && ok; ++kb) {
            const int slot = kb % p.ring;
            if (!mbar_wait(&w_full[slot], (uint32_t)(kb / p.ring) & 1u, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t w_addr = smem_u32(sW + slot * DL_W_SLICE);
            const uint32_t x_addr = smem_u32(sX + kb * DL_X_SLICE);
#pragma unroll
            for (int k = 0; k < 4; ++k)       // 16 k per UMMA: 16 rows of 128 B in the MN-major slab, 32 B in the K-major tile
                umma_bf16(tmem_base, umma_desc_sw128(w_addr + k * 2048, DL_W_BOX, 1024), umma_desc_sw128(x_addr + k * 32, 16, 1024),
                          idesc, (kb | k) != 0 ? 1u : 0u);
            umma_commit(&w_empty[slot]);
        }
        if (ok) umma_commit(acc_bar);
        else { *abort_flag = 1; atomicExch(p.err, 52); }
    }
    __syncwarp();

    // ---- epilogue: thread = output column (accumulator lane), 64 sequences in registers
    const bool done = mbar_wait(acc_bar, 0u, abort_flag);
    tc_fence_after();
    float v[DL_SEQ];
    if (done && warp < 4) {
        uint32_t a0[32], a1[32];
        const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16);
        tmem_ld32(taddr, a0);
        tmem_ld32(taddr + 32, a1);
        tmem_ld_wait();
#pragma unroll
        for (int s = 0; s < 32; ++s) { v[s] = __uint_as_float(a0[s]); v[32 + s] = __uint_as_float(a1[s]); }
    }
    tc_fence_before();
    if (p.ks > 1) {
        // ranks 1.. park their accumulators in their own shared memory (the ring is consumed); rank 0 adds them in rank
        // order (a fixed order: the result does not depend on timing); nobody leaves before rank 0 has read
        __syncthreads();
        if (rank != 0 && done && warp < 4) {
#pragma unroll
            for (int s = 0; s < DL_SEQ; s += 4)
                *reinterpret_cast<float4*>(part + tid * DL_PART_LD + s) = make_float4(v[s], v[s + 1], v[s + 2], v[s + 3]);
        }
        cluster_sync();
        if (rank == 0 && done && warp < 4) {
            const uint32_t mine = smem_u32(part + tid * DL_PART_LD);
            for (int r = 1; r < p.ks; ++r) {
                uint32_t peer;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(peer) : "r"(mine), "r"((uint32_t)r));
                float4 x[DL_SEQ / 4];
#pragma unroll
                for (int s = 0; s < DL_SEQ / 4; ++s)      // all sixteen loads of a rank in flight, then the additions in order
                    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                                 : "=f"(x[s].x), "=f"(x[s].y), "=f"(x[s].z), "=f"(x[s].w) : "r"(peer + 16u * (uint32_t)s));
#pragma unroll
                for (int s = 0; s < DL_SEQ / 4; ++s) {
                    v[4 * s] += x[s].x; v[4 * s + 1] += x[s].y; v[4 * s + 2] += x[s].z; v[4 * s + 3] += x[s].w;
                }
            }
        }
        cluster_sync();
    }
    if (!p.swiglu) {
        if (done && warp < 4 && rank == 0) {
            const int n = n0 + tid;
            if (n < p.N) {
                const float b = p.bias ? __ldg(p.bias + n) : 0.0f;
                if (p.residual) {      // all residual loads in flight before the first store (the output may alias nothing,
                                       // but the compiler cannot know: it would order every load behind the store before it)
                    float rr[DL_SEQ];
#pragma unroll
                    for (int s = 0; s < DL_SEQ; ++s) rr[s] = s < p.S ? __ldg(p.residual + (long long)s * p.N + n) : 0.0f;
#pragma unroll
                    for (int s = 0; s < DL_SEQ; ++s) v[s] = (v[s] + b) + rr[s];      // accumulator + bias + residual, in that order
                } else {
#pragma unroll
                    for (int s = 0; s < DL_SEQ; ++s) v[s] += b;
                }
#pragma unroll
                for (int s = 0; s < DL_SEQ; ++s)
                    if (s < p.S) p.y32[(long long)s * p.N + n] = v[s];
            }
        }
        __syncthreads();
    } else {
        // accumulator rows 0..63 hold the gate columns of 64 hidden units, rows 64..127 their up columns: the up half
        // goes through shared memory (the ring is consumed by now) to the thread that holds the unit's gate values
        const int unit = slab * 64 + (tid & 63);
        __syncthreads();                                      // every role has left the ring
        if (done && warp >= 2 && warp < 4) {
            const float bu = p.bias ? __ldg(p.bias + p.F + unit) : 0.0f;
#pragma unroll
            for (int s = 0; s < DL_SEQ; ++s) exch[(tid - 64) * 65 + s] = v[s] + bu;
        }
        __syncthreads();
        if (done && warp < 2) {
            const float bg = p.bias ? __ldg(p.bias + unit) : 0.0f;
#pragma unroll
            for (int s = 0; s < DL_SEQ; ++s) {
                if (s < p.S) {
                    const float g = v[s] + bg, u = exch[tid * 65 + s];
                    // the sigmoid of the fused SwiGLU GEMM epilogue: ex2.approx and an approximate reciprocal
                    const float sg = __fdividef(1.0f, 1.0f + ex2_approx(-g * 1.4426950408889634f));
                    p.h16[(long long)s * p.F + unit] = __float2bfloat16_rn(g * sg * u);
                }
            }
        }
        __syncthreads();
    }
    if (*abort_flag) {
        // a bounded wait ran out: give copies in flight time to land before the CTA's shared memory is released
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 64); }
}

}  // namespace

bool decode_linear_supported(int S, int N, int K, bool swiglu) {
    if (S < 1 || S > DL_SEQ || K < DL_BK || K % DL_BK != 0 || K / DL_BK > DL_MAX_KBLOCKS) return false;
    if (swiglu) return N % 2 == 0 && (N / 2) % 64 == 0;
    return N % DL_COLS == 0;
}

// X: bf16 [S, K] (x32 == nullptr), or x32 float32 [S, K] normalised here with norm_w and eps.  W: bf16 [K, N] row-major.
// Plain: y32 [S, N] = X W + bias (+ residual [S, N]).  SwiGLU (h16 given): N = 2F, h16 [S, F] = silu(g + b_g) * (u + b_u).
int launch_decode_linear(DeviceCtx* ctx, const bf16* X16, const float* x32, const float* norm_w, float eps, const bf16* W,
                         const float* bias, const float* residual, float* y32, bf16* h16, int S, int N, int K,
                         cudaStream_t st) {
    const bool swiglu = h16 != nullptr;
    TB_CHECK(decode_linear_supported(S, N, K, swiglu), "decode linear: unsupported shape S=%d N=%d K=%d", S, N, K);
    TB_CHECK((X16 != nullptr) != (x32 != nullptr), "decode linear: give the input either as bf16 or as float32 to normalise");
    TB_CHECK(x32 == nullptr || (norm_w != nullptr && K % 4 == 0 && (reinterpret_cast<uintptr_t>(x32) & 15u) == 0 &&
                                (reinterpret_cast<uintptr_t>(norm_w) & 15u) == 0),
             "decode linear: the float32 input and the norm weights must be 16-byte aligned");
    DecLinParams p;
    p.S = S; p.K = K; p.N = N;
    const int kblocks_total = K / DL_BK;
    const int slabs = swiglu ? (N / 2) / 64 : N / DL_COLS;
    // K splits: few slabs with a long K (the down projection: 3 slabs of 1024 x 128) would leave the weight stream to
    // three SMs; a cluster of ks CTAs per slab shares it.  The largest divisor of the slice count that keeps at least
    // two slices per CTA and at most 16 CTAs in all.
    int ks = 1;
    if (!swiglu && getenv("TB_DECODE_NO_KSPLIT") == nullptr) {
        for (int c = 2; c <= 8; ++c)
            if (kblocks_total % c == 0 && kblocks_total / c >= 2 && slabs * c <= 16) ks = c;
    }
    p.ks = ks;
    p.kblocks = kblocks_total / ks;
    const long long x_bytes = (long long)p.kblocks * DL_X_SLICE;
    long long ring = (DL_MAX_SMEM - DL_HEADER - 1024 - x_bytes) / DL_W_SLICE;
    if (ring > p.kblocks) ring = p.kblocks;
    if (ring > DL_MAX_RING) ring = DL_MAX_RING;
    TB_CHECK(ring >= 2 || ring == p.kblocks, "decode linear: K=%d leaves no room for the weight ring", K);
    p.ring = (int)ring;
    p.norm = x32 != nullptr ? 1 : 0; p.x32 = x32; p.norm_w = norm_w; p.eps = eps;
    p.swiglu = swiglu ? 1 : 0; p.F = swiglu ? N / 2 : 0;
    p.bias = bias; p.residual = residual; p.y32 = y32; p.h16 = h16; p.err = ctx->d_err;
    TB_CHECK(swiglu || y32 != nullptr, "decode linear: no output");
    // the SwiGLU exchange buffer (64 x 65 floats) and the K-split accumulators (128 x 68 floats) lie over the ring
    const long long over = swiglu ? 64 * 65 * 4 : (ks > 1 ? 128 * DL_PART_LD * 4 : 0);
    size_t smem = DL_HEADER + 1024 + (size_t)x_bytes + (size_t)std::max<long long>(ring * DL_W_SLICE, over);
    TB_CHECK(smem <= (size_t)DL_MAX_SMEM, "decode linear: %zu bytes of shared memory", smem);
    CUtensorMap tmW, tmX;
    TB_TRY(make_operand_map(&tmW, W, N, K, N, 1, 0, DL_BK));
    if (X16) TB_TRY(make_operand_map(&tmX, X16, K, S, K, 1, 0, DL_SEQ));
    else tmX = tmW;
    static bool attr_set[64] = {false};
    if (!attr_set[ctx->device & 63]) {
        TB_CUDA(cudaFuncSetAttribute(decode_linear_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DL_MAX_SMEM));
        attr_set[ctx->device & 63] = true;
    }
    const int ctas = slabs * ks;
    const double bytes = 2.0 * K * N + (x32 ? 4.0 : 2.0) * S * K + (swiglu ? 2.0 * S * (N / 2) : 4.0 * S * N) +
                         (residual ? 4.0 * S * N : 0.0);
    prof_mark(ctx, swiglu ? "decode_linear_swiglu" : (x32 ? "decode_linear_norm" : "decode_linear"), 2.0 * S * (double)N * K, bytes, st);
    TB_CUDA(launch_kernel_cluster(decode_linear_kernel, dim3(ctas), dim3(DL_THREADS), smem, st, ks, tmW, tmX, p));
    TB_CUDA(cudaGetLastError());
    ctx->launches++;
    prof_close(ctx, st);
    return 0;
}

}  // namespace tb
