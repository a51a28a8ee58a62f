// Fused causal attention for sm_100a: S = Q K^T and O = P V on tcgen05 tensor cores with the
// score tile kept in TMEM, the softmax done in registers and P handed to the second product
// through shared memory -- the [T, T] score and probability matrices never exist in HBM.
//
// Replaces the reference's chain k_bf16_gemm_nt (QK^T) -> k_attn_softmax_fwd -> k_bf16_gemm_nn
// (P V) -> k_heads_merge and its backward counterpart (model/gpu_train.c:346-358, :435-455;
// cuda/train_kernels.cu:631-692), which stores P [B,H,T,T] in float32 per layer.
//
// Semantics are the reference's (model/attention.c:32-60): scores * 1/sqrt(hd), keys after the
// query excluded, softmax over the row, times V.  The reference adds -1e9 to the excluded scores;
// after exp in float32 that is exactly 0, so excluding them is the same function.  The softmax is
// evaluated block-wise with a running maximum (the result is the same softmax; rounding of P to
// bf16 happens against the running maximum instead of the final one).
//
// Layouts: Q, K, V bf16 [B*H, T, hd] (RoPE already applied), hd <= 64 and a multiple of 8 (rows
// are padded to 64 columns with zeros by the TMA loads).  Output bf16 [B*T, H*hd] (heads merged)
// plus the row-wise log-sum-exp, which is all the backward pass needs to rebuild P.
#include "common.h"
#include "ptx.cuh"

#include <cstdlib>

namespace tb {

constexpr int ATT_BM = 128;       // queries per CTA
constexpr int ATT_BN = 128;       // keys per step
constexpr int ATT_HD = 64;        // padded head dimension
constexpr int TILE_BYTES = 128 * 64 * 2;   // one [128, 64] bf16 tile, 128-byte rows

// Shared-memory descriptors are built once per tile, outside the issue loops (one thread issues every
// UMMA of the CTA, so each instruction it spends per UMMA delays the tensor pipe); the loops only add
// to the start-address field (low 14 bits, 16-byte units; never carries below 256 KB).
// K-major operand tile [rows, 64] (128-byte rows, 128B swizzle): advance 32 bytes per K=16
__device__ __forceinline__ uint64_t kmajor_tile(uint32_t tile_addr) { return umma_desc_sw128(tile_addr, 16, 1024); }
// the same tile read as an MN-major operand (64 MN elements contiguous, K = rows): 16 rows per K=16;
// lbo = bytes between consecutive 64-wide MN blocks
__device__ __forceinline__ uint64_t mnmajor_tile(uint32_t tile_addr, uint32_t lbo) {
    return umma_desc_sw128(tile_addr, lbo, 1024);
}
constexpr uint64_t KSTEP = 32 >> 4;          // descriptor units per K=16 step of a K-major tile
constexpr uint64_t MNSTEP = 2048 >> 4;       // ... of an MN-major tile (16 rows of 128 bytes)
constexpr uint64_t TILESTEP = (128 * 64 * 2) >> 4;   // one [128, 64] bf16 tile

// 2^x on the special-function unit (one instruction; 2^-inf = 0)
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Two float32 results per issue slot (fma.rn.f32x2 and friends, sm_100): the softmax warps of these kernels are
// bound by instruction issue (about 2,000 cycles per 128 x 128 block for 64 scores per thread), not by a unit.
__device__ __forceinline__ float2 pair_of(uint32_t a, uint32_t b) { return make_float2(__uint_as_float(a), __uint_as_float(b)); }


// 32 consecutive values of row r -> bf16 in a [128 x 128] operand stored as two [128 x 64] tiles
__device__ __forceinline__ void store_chunk_bf16(uint8_t* tiles, int r, int c, const float (&x)[32]) {
    uint8_t* row = tiles + (c >> 1) * TILE_BYTES + r * 128;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        uint4 pk;
        __nv_bfloat162 h0 = __floats2bfloat162_rn(x[8 * g + 0], x[8 * g + 1]);
        __nv_bfloat162 h1 = __floats2bfloat162_rn(x[8 * g + 2], x[8 * g + 3]);
        __nv_bfloat162 h2 = __floats2bfloat162_rn(x[8 * g + 4], x[8 * g + 5]);
        __nv_bfloat162 h3 = __floats2bfloat162_rn(x[8 * g + 6], x[8 * g + 7]);
        pk.x = *reinterpret_cast<uint32_t*>(&h0); pk.y = *reinterpret_cast<uint32_t*>(&h1);
        pk.z = *reinterpret_cast<uint32_t*>(&h2); pk.w = *reinterpret_cast<uint32_t*>(&h3);
        const int chunk = (c & 1) * 4 + g;
        *reinterpret_cast<uint4*>(row + ((chunk ^ (r & 7)) << 4)) = pk;
    }
}

struct AttFwdParams {
    int T, H, hd, D;
    int nq;                 // query blocks per head
    float scale_log2;       // 1/sqrt(hd) * log2(e)
    bf16* att;              // [B*T, D]
    float* lse;             // [B*H, T]
    int* err;
};

// ------------------------------------------------------------------------------------ forward
// CTA = 6 warps: TMA producer, MMA issuer (owns TMEM: two score buffers of 64 key columns and two
// P V buffers of 64 head-dim columns), four softmax warps (thread = query row).  Keys are taken in
// half blocks of 64 and the steps are software-pipelined: while the softmax warps work on half block
// i, the tensor core computes the scores of i+1 and P V of i-1.  Two CTAs fit per SM on top of that.
__global__ void __launch_bounds__(192, 2)
attention_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                     const AttFwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    uint8_t* sQ = smem;                          // 16 KB
    uint8_t* sK = smem + TILE_BYTES;             // 2 x 16 KB
    uint8_t* sV = smem + 3 * TILE_BYTES;         // 2 x 16 KB
    uint8_t* sP = smem + 5 * TILE_BYTES;         // 2 x 16 KB: keys 0-63 | keys 64-127
    // the request is exactly 1 KB + 7 tiles (two CTAs per SM): the barriers go behind the tiles when
    // the alignment pad leaves room there (the usual case: pad 0), else into the pad itself
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint64_t* bars = reinterpret_cast<uint64_t*>(pad <= 768u ? smem + 7 * TILE_BYTES : smem_raw);
    uint64_t* q_full = bars;          // 1
    uint64_t* k_full = bars + 1;      // 2: K tile of 128 keys in stage s
    uint64_t* v_full = bars + 3;      // 2
    uint64_t* kv_empty = bars + 5;    // 2
    uint64_t* s_full = bars + 7;      // 2: score buffer b holds Q K^T of a 64-key half block
    uint64_t* s_free = bars + 9;      // 2
    uint64_t* p_full = bars + 11;     // 2: probability buffer b written
    uint64_t* o_full = bars + 13;     // 2: P V of a half block landed in output buffer b
    uint64_t* o_free = bars + 15;     // 2
    uint64_t* out_full = bars + 18;   // 4 arrivals: the output tile is staged in shared memory
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 17);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // blocks are handed out x fastest: all heads' heaviest (last) query block first, the lightest last,
    // so the long CTAs start together and the short ones fill the tail
    const int qb = p.nq - 1 - (int)blockIdx.y;
    const int bh = blockIdx.x;
    const int q0 = qb * ATT_BM;
    const int nkv = qb + 1;                           // key blocks 0..qb

    if (threadIdx.x == 0) {
        mbar_init(q_full, 1);
        for (int i = 0; i < 2; ++i) { mbar_init(&k_full[i], 1); mbar_init(&v_full[i], 1); mbar_init(&kv_empty[i], 1); }
        for (int i = 0; i < 2; ++i) {
            mbar_init(&s_full[i], 1); mbar_init(&s_free[i], 4); mbar_init(&p_full[i], 4);
            mbar_init(&o_full[i], 1); mbar_init(&o_free[i], 4);
        }
        mbar_init(out_full, 4);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) { tmem_alloc(tmem_slot, 256); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();                 // everything above is independent of earlier kernels' results
    // TMEM: two score buffers of 64 key columns, two output buffers of 64 head-dim columns
    const uint32_t tS = tmem_base, tO = tmem_base + 128;
    const int nsub = 2 * nkv;                         // 64-key half blocks

    if (warp == 0) {
        if (lane == 0) {
            bool ok = true;
            mbar_expect_tx(q_full, TILE_BYTES);
            tma_load_3d(sQ, &tmQ, q_full, 0, q0, bh);
            for (int j = 0; j < nkv && ok; ++j) {
                const int s = j & 1;
                if (!mbar_wait(&kv_empty[s], (uint32_t)((j >> 1) & 1) ^ 1u, abort_flag)) { ok = false; break; }
                mbar_expect_tx(&k_full[s], TILE_BYTES);
                tma_load_3d(sK + s * TILE_BYTES, &tmK, &k_full[s], 0, j * ATT_BN, bh);
                mbar_expect_tx(&v_full[s], TILE_BYTES);
                tma_load_3d(sV + s * TILE_BYTES, &tmV, &v_full[s], 0, j * ATT_BN, bh);
            }
            pdl_launch_dependents_now();     // all loads issued: the next kernel may start its prologue
            if (!ok) { *abort_flag = 1; atomicExch(p.err, 11); }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // Half blocks of 64 keys, software-pipelined: the scores of half block i+2 are issued as soon
            // as the softmax warps have drained buffer i&1, so the tensor core works on Q K^T (i+1, i+2)
            // and P V (i-1) while the softmax of i runs -- no step waits for a full round trip.
            const uint32_t idesc_s = umma_idesc(1u, 0u, 0u, ATT_BM, 64);         // Q K^T: both K-major
            const uint32_t idesc_o = umma_idesc(1u, 0u, 1u, ATT_BM, ATT_HD);     // P V: V is MN-major
            const uint64_t dQ = kmajor_tile(smem_u32(sQ)), dK0 = kmajor_tile(smem_u32(sK)), dP0 = kmajor_tile(smem_u32(sP));
            const uint64_t dV0 = mnmajor_tile(smem_u32(sV), TILE_BYTES);
            bool ok = mbar_wait(q_full, 0, abort_flag);
            auto issue_scores = [&](int i) -> bool {
                const int j = i >> 1, st = j & 1, b = i & 1;
                if (b == 0 && !mbar_wait(&k_full[st], (uint32_t)((j >> 1) & 1), abort_flag)) return false;
                if (!mbar_wait(&s_free[b], (uint32_t)((i >> 1) & 1) ^ 1u, abort_flag)) return false;
                tc_fence_after();
                const uint64_t dK = dK0 + (uint64_t)st * TILESTEP + (uint64_t)b * (TILESTEP / 2);   // keys 64b.. of the tile
#pragma unroll
                for (int k = 0; k < ATT_HD / 16; ++k)
                    umma_bf16(tS + (uint32_t)(b * 64), dQ + k * KSTEP, dK + k * KSTEP, idesc_s, k > 0 ? 1u : 0u);
                umma_commit(&s_full[b]);
                return true;
            };
            if (ok) ok = issue_scores(0);
            if (ok && nsub > 1) ok = issue_scores(1);
            for (int i = 0; i < nsub && ok; ++i) {
                const int j = i >> 1, st = j & 1, b = i & 1;
                const uint32_t par = (uint32_t)((i >> 1) & 1);
                if (!mbar_wait(&p_full[b], par, abort_flag)) { ok = false; break; }
                if (b == 0 && !mbar_wait(&v_full[st], (uint32_t)((j >> 1) & 1), abort_flag)) { ok = false; break; }
                if (!mbar_wait(&o_free[b], par ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint64_t dP = dP0 + (uint64_t)b * TILESTEP;
                const uint64_t dV = dV0 + (uint64_t)st * TILESTEP + (uint64_t)b * (4 * MNSTEP);
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    umma_bf16(tO + (uint32_t)(b * 64), dP + k * KSTEP, dV + k * MNSTEP, idesc_o, k > 0 ? 1u : 0u);
                umma_commit(&o_full[b]);
                if (b == 1) umma_commit(&kv_empty[st]);          // both halves of the K/V tile are consumed
                if (i + 2 < nsub) ok = issue_scores(i + 2);
            }
            if (!ok) { *abort_flag = 1; atomicExch(p.err, 12); }
        }
    } else {
        const int q = warp & 3;
        const int r = q * 32 + lane;                 // row of the tile = TMEM lane
        const int qi = q0 + r;                       // query position
        const uint32_t lane_base = (uint32_t)(q * 32) << 16;
        float m = -INFINITY, l = 0.0f;
        float O[ATT_HD];
#pragma unroll
        for (int d = 0; d < ATT_HD; ++d) O[d] = 0.0f;
        bool ok = true;
        float alpha_prev = 0.0f;                     // rescale factor of the half block whose P V is still due
        // adds P V of half block i (output buffer i&1) into the running output: O = O * alpha_i + P_i V_i
        uint32_t va[32], vb[32];                     // one half block's scores (or one P V result) per row
        auto accumulate = [&](int i, float alpha) -> bool {
            const int b = i & 1;
            if (!mbar_wait(&o_full[b], (uint32_t)((i >> 1) & 1), abort_flag)) return false;
            tc_fence_after();
            tmem_ld32(tO + lane_base + (uint32_t)(b * 64), va);
            tmem_ld32(tO + lane_base + (uint32_t)(b * 64 + 32), vb);
            tmem_ld_wait();
            const float2 al2 = make_float2(alpha, alpha);
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
                const float2 o0 = __ffma2_rn(make_float2(O[e], O[e + 1]), al2, pair_of(va[e], va[e + 1]));
                const float2 o1 = __ffma2_rn(make_float2(O[32 + e], O[33 + e]), al2, pair_of(vb[e], vb[e + 1]));
                O[e] = o0.x; O[e + 1] = o0.y; O[32 + e] = o1.x; O[33 + e] = o1.y;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&o_free[b]);
            return true;
        };
        for (int i = 0; i < nsub && ok; ++i) {
            const int b = i & 1;
            if (!mbar_wait(&s_full[b], (uint32_t)((i >> 1) & 1), abort_flag)) { ok = false; break; }
            tc_fence_after();
            const bool diag = ((i >> 1) == qb);
            const int k0 = (i >> 1) * ATT_BN + b * 64;
            const uint32_t ts = tS + lane_base + (uint32_t)(b * 64);
            // all 64 scores of the row in one TMEM round trip; the registers are reused for the probabilities
            tmem_ld32(ts, va);
            tmem_ld32(ts + 32, vb);
            tmem_ld_wait();
            const int lim = diag ? qi - k0 : 64;               // columns e <= lim are allowed
            float mx = -INFINITY;
            if (diag) {
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    mx = fmaxf(mx, e <= lim ? __uint_as_float(va[e]) : -INFINITY);
                    mx = fmaxf(mx, e + 32 <= lim ? __uint_as_float(vb[e]) : -INFINITY);
                }
            } else {
                // four chains instead of one of 32 dependent maxima
                float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
                for (int e = 0; e < 32; e += 4) {
                    m0 = fmaxf(m0, fmaxf(__uint_as_float(va[e]), __uint_as_float(vb[e])));
                    m1 = fmaxf(m1, fmaxf(__uint_as_float(va[e + 1]), __uint_as_float(vb[e + 1])));
                    m2 = fmaxf(m2, fmaxf(__uint_as_float(va[e + 2]), __uint_as_float(vb[e + 2])));
                    m3 = fmaxf(m3, fmaxf(__uint_as_float(va[e + 3]), __uint_as_float(vb[e + 3])));
                }
                mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
            }
            const float m_new = fmaxf(m, mx * p.scale_log2);
            const float alpha = fast_exp2(m - m_new);        // 0 on the first block (m = -inf)
            l *= alpha;
            // p = 2^(s*c - m), row sum, bf16 P into shared memory (K-major, 128B swizzle)
            float pa[32], pb[32];
            const float2 c2 = make_float2(p.scale_log2, p.scale_log2), nm2 = make_float2(-m_new, -m_new);
            float2 la = make_float2(0.f, 0.f), lb = make_float2(0.f, 0.f);
#pragma unroll
            for (int e = 0; e < 32; e += 2) {
                const float2 xa = __ffma2_rn(pair_of(va[e], va[e + 1]), c2, nm2);
                const float2 xb = __ffma2_rn(pair_of(vb[e], vb[e + 1]), c2, nm2);
                pa[e] = fast_exp2(xa.x); pa[e + 1] = fast_exp2(xa.y);
                pb[e] = fast_exp2(xb.x); pb[e + 1] = fast_exp2(xb.y);
                if (diag) {
                    pa[e] = e <= lim ? pa[e] : 0.0f;           pa[e + 1] = e + 1 <= lim ? pa[e + 1] : 0.0f;
                    pb[e] = e + 32 <= lim ? pb[e] : 0.0f;      pb[e + 1] = e + 33 <= lim ? pb[e + 1] : 0.0f;
                }
                la = __fadd2_rn(la, make_float2(pa[e], pa[e + 1]));
                lb = __fadd2_rn(lb, make_float2(pb[e], pb[e + 1]));
            }
            l += (la.x + la.y) + (lb.x + lb.y);
            store_chunk_bf16(sP, r, 2 * b, pa);
            store_chunk_bf16(sP, r, 2 * b + 1, pb);
            tc_fence_before();
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) { mbar_arrive(&s_free[b]); mbar_arrive(&p_full[b]); }
            // the previous half block's P V has had this whole softmax to finish: add it now
            if (i > 0) ok = accumulate(i - 1, alpha_prev);
            alpha_prev = alpha;
            m = m_new;
        }
        if (ok) ok = accumulate(nsub - 1, alpha_prev);
        if (ok) {
            // O / l as bf16 into the Q tile (every product has completed), one TMA store for the 128 rows: a thread per
            // row storing to global memory directly touches 32 different rows per instruction
            const float inv = 1.0f / l;
            const int b = bh / p.H, h = bh % p.H;
            if (qi < p.T) {
                uint8_t* row = sQ + r * 128;
#pragma unroll
                for (int d = 0; d < ATT_HD; d += 8) {
                    if (d >= p.hd) break;
                    uint4 pk;
                    __nv_bfloat162 h0 = __floats2bfloat162_rn(O[d + 0] * inv, O[d + 1] * inv);
                    __nv_bfloat162 h1 = __floats2bfloat162_rn(O[d + 2] * inv, O[d + 3] * inv);
                    __nv_bfloat162 h2 = __floats2bfloat162_rn(O[d + 4] * inv, O[d + 5] * inv);
                    __nv_bfloat162 h3 = __floats2bfloat162_rn(O[d + 6] * inv, O[d + 7] * inv);
                    pk.x = *reinterpret_cast<uint32_t*>(&h0); pk.y = *reinterpret_cast<uint32_t*>(&h1);
                    pk.z = *reinterpret_cast<uint32_t*>(&h2); pk.w = *reinterpret_cast<uint32_t*>(&h3);
                    *reinterpret_cast<uint4*>(row + (((d >> 3) ^ (r & 7)) << 4)) = pk;
                }
                if (p.lse) p.lse[(long long)bh * p.T + qi] = (m + log2f(l)) * 0.6931471805599453f;
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(out_full);
            if (q == 0 && lane == 0) {
                if (mbar_wait(out_full, 0, abort_flag)) {
                    tma_store_4d(&tmO, sQ, 0, q0, h, b);          // rows past T are clipped
                    tma_store_commit();
                    tma_store_wait_read<0>();
                } else ok = false;
            }
        }
        if (!ok && lane == 0) { *abort_flag = 1; atomicExch(p.err, 13); }
    }

    __syncwarp();
    if (*abort_flag) for (int i = 0; i < 64; ++i) __nanosleep(1000);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 256); }
}

// ----------------------------------------------------------------------------------- backward
// With P rebuilt from the saved log-sum-exp (P = exp(S*scale - lse)) the backward is, per head,
//   dV = P^T dO,  dP = dO V^T,  dS = P * (dP - delta) * scale,  dQ = dS K,  dK = dS^T Q,
// delta[i] = <dO_i, O_i>  (the reference's k_attn_softmax_bwd row dot <dP, P>, since O = P V).
// Two kernels keep every sum in a fixed order without atomics: one owns a key block and walks the
// query blocks below the diagonal (dK, dV), the other owns a query block and walks its key blocks
// (dQ); both recompute S and dP on the tensor cores.

__global__ void attention_delta_kernel(const bf16* __restrict__ att, const bf16* __restrict__ datt,
                                       float* __restrict__ delta, int B, int T, int H, int hd) {
    pdl_wait();
    pdl_launch_dependents();
    const long long total = (long long)B * T * H;
    const int D = H * hd;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int h = (int)(i % H);
        const long long n = i / H;
        const int t = (int)(n % T);
        const long long b = n / T;
        const bf16* o = att + n * D + h * hd;
        const bf16* d = datt + n * D + h * hd;
        float s = 0.0f;
        for (int k = 0; k < hd; k += 8) {
            const uint4 ov = *reinterpret_cast<const uint4*>(o + k);
            const uint4 dv = *reinterpret_cast<const uint4*>(d + k);
            const __nv_bfloat162* o2 = reinterpret_cast<const __nv_bfloat162*>(&ov);
            const __nv_bfloat162* d2 = reinterpret_cast<const __nv_bfloat162*>(&dv);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 a = __bfloat1622float2(o2[e]), c = __bfloat1622float2(d2[e]);
                s += a.x * c.x;
                s += a.y * c.y;
            }
        }
        delta[(b * H + h) * T + t] = s;
    }
}

struct AttBwdParams {
    int T, H, hd;
    int nq;
    float scale, scale_log2;
    const float* lse;       // [B*H, T]
    const float* delta;     // [B*H, T]
    float* dQ; float* dK; float* dV;     // [B*H, T, hd]
    // merged output (optional, replaces dQ/dK/dV): dqkv bf16 [B*T, 3*H*hd] with the inverse rotation of
    // the position embedding applied to dQ and dK on the way out (the reference's k_qkv_rope_merge_bwd,
    // cuda/train_kernels.cu:600-626); cos_t/sin_t are the [T, hd/2] tables
    bf16* dqkv; const float* cos_t; const float* sin_t;
    // dS hand-off between the two kernels: the dK/dV kernel stores each [128 q x 128 keys] block of dS' = P * (dP - delta)
    // (bf16, the 32 KB shared-memory image it feeds its own tensor-core product with) at block index
    // bh * nq*(nq+1)/2 + qb*(qb+1)/2 + kb; the dQ kernel reads the blocks back and only forms dQ = sum_kb dS' K.
    // (Recomputing S, dP and the exponentials there instead cost a second pass over the 2^x unit, the busiest one.)
    bf16* ds;
    int* err;
};
constexpr int DS_BLOCK_BYTES = 2 * TILE_BYTES;

// The rotation tables of one row for 32 consecutive head-dim values (16 pairs) starting at d0: fetched before the
// wait for the accumulators, in one batch (loads placed between the stores of a row would each wait for the
// store before them, since the compiler cannot tell the tables from the output).
struct RopeRow { float4 c[4], s[4]; };
__device__ __forceinline__ void load_rope_row(RopeRow& t, const float* cs, const float* sn, int d0, int hd) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        if (d0 + 8 * g < hd) {
            t.c[g] = *reinterpret_cast<const float4*>(cs + ((d0 + 8 * g) >> 1));
            t.s[g] = *reinterpret_cast<const float4*>(sn + ((d0 + 8 * g) >> 1));
        } else {
            t.c[g] = make_float4(1.f, 1.f, 1.f, 1.f);
            t.s[g] = make_float4(0.f, 0.f, 0.f, 0.f);
        }
    }
}

// 32 consecutive head-dim values of one row (first index d0), times mul, optionally through the inverse rotation of
// the interleaved pairs (2k, 2k+1): out = (a*c + b*s, -a*s + b*c), as bf16 into row r of a [128 x 64] tile in shared
// memory (128-byte rows, 128B swizzle), from where one TMA store writes the whole tile: a thread per row storing to global memory directly touches 32 different
// rows per instruction (one 16-byte piece each), which took ~4,500 cycles per CTA.
__device__ __forceinline__ void stage_row_bf16(uint8_t* tile, int r, const uint32_t (&v)[32], int d0, int hd,
                                               const RopeRow* rot, float mul) {
    uint8_t* row = tile + r * 128;
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        const int e = 8 * g;
        if (d0 + e >= hd) break;
        float o[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] = __uint_as_float(v[e + j]) * mul;
        if (rot != nullptr) {
            const float4 c4 = rot->c[g], s4 = rot->s[g];
            const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float a = o[2 * j], b = o[2 * j + 1];
                o[2 * j] = a * cc[j] + b * ss[j];
                o[2 * j + 1] = -a * ss[j] + b * cc[j];
            }
        }
        uint4 pk;
        __nv_bfloat162 h0 = __floats2bfloat162_rn(o[0], o[1]), h1 = __floats2bfloat162_rn(o[2], o[3]);
        __nv_bfloat162 h2 = __floats2bfloat162_rn(o[4], o[5]), h3 = __floats2bfloat162_rn(o[6], o[7]);
        pk.x = *reinterpret_cast<uint32_t*>(&h0); pk.y = *reinterpret_cast<uint32_t*>(&h1);
        pk.z = *reinterpret_cast<uint32_t*>(&h2); pk.w = *reinterpret_cast<uint32_t*>(&h3);
        const int chunk = (d0 >> 3) + g;
        *reinterpret_cast<uint4*>(row + ((chunk ^ (r & 7)) << 4)) = pk;
    }
}

// 32 float32 values times mul into row r of a [128 x 32] float32 tile (128-byte rows, 128B swizzle) for a TMA store
__device__ __forceinline__ void stage_row_f32(uint8_t* tile, int r, const uint32_t (&v)[32], float mul) {
    uint8_t* row = tile + r * 128;
#pragma unroll
    for (int g = 0; g < 8; ++g)
        *reinterpret_cast<float4*>(row + ((g ^ (r & 7)) << 4)) =
            make_float4(__uint_as_float(v[4 * g]) * mul, __uint_as_float(v[4 * g + 1]) * mul,
                        __uint_as_float(v[4 * g + 2]) * mul, __uint_as_float(v[4 * g + 3]) * mul);
}

// P = 2^(s*c - lse) and dS' = P * (dP - delta) of 32 scores of one row, two per instruction.  The factor 1/sqrt(hd)
// of dS is applied to the accumulated dQ and dK instead (they are linear in dS).  lim: columns e <= lim are allowed.
__device__ __forceinline__ void p_and_ds(const uint32_t (&sv)[32], const uint32_t (&dv)[32], float scale_log2, float lse2,
                                         float dl, bool diag, int lim, float (&P)[32], float (&dS)[32]) {
    const float2 c2 = make_float2(scale_log2, scale_log2), nl2 = make_float2(-lse2, -lse2), nd2 = make_float2(-dl, -dl);
#pragma unroll
    for (int e = 0; e < 32; e += 2) {
        const float2 x = __ffma2_rn(pair_of(sv[e], sv[e + 1]), c2, nl2);
        float p0 = fast_exp2(x.x), p1 = fast_exp2(x.y);
        if (diag) { p0 = e <= lim ? p0 : 0.0f; p1 = e + 1 <= lim ? p1 : 0.0f; }
        const float2 d = __fmul2_rn(make_float2(p0, p1), __fadd2_rn(pair_of(dv[e], dv[e + 1]), nd2));
        P[e] = p0; P[e + 1] = p1;
        dS[e] = d.x; dS[e + 1] = d.y;
    }
}

constexpr int ATT_BWD_STAGES = 2;       // stages of the (Q, dO) pair in the dK/dV kernel
constexpr int ATT_BWD_THREADS = 352;     // TMA warp, score-MMA warp, 8 compute warps, gradient-MMA warp
// (two issuing threads on different schedulers: one thread cannot issue a block's 24 UMMAs as fast as the
//  tensor pipe retires them while eight compute warps compete for the same issue slots)

// dK, dV of one key block: walks the query blocks qb = kb .. nq-1.
__global__ void __launch_bounds__(ATT_BWD_THREADS, 1)
attention_bwd_dkdv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                          const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmdO,
                          const __grid_constant__ CUtensorMap tmoK, const __grid_constant__ CUtensorMap tmoV,
                          const AttBwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    uint8_t* sK = smem;
    uint8_t* sV = smem + TILE_BYTES;
    uint8_t* sQ = smem + 2 * TILE_BYTES;                              // ATT_BWD_STAGES stages
    uint8_t* sdO = smem + (2 + ATT_BWD_STAGES) * TILE_BYTES;          // ATT_BWD_STAGES stages
    uint8_t* sP = smem + (2 + 2 * ATT_BWD_STAGES) * TILE_BYTES;       // [128 q, 128 keys] as two tiles
    uint8_t* sdS = smem + (4 + 2 * ATT_BWD_STAGES) * TILE_BYTES;      // same, two buffers (one is being stored to HBM)
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + (8 + 2 * ATT_BWD_STAGES) * TILE_BYTES);
    uint64_t* kv_full = bars;          // 1
    uint64_t* qdo_full = bars + 1;     // ATT_BWD_STAGES
    uint64_t* qdo_empty = bars + 5;    // ATT_BWD_STAGES
    uint64_t* sdp_full = bars + 9;
    uint64_t* sdp_free = bars + 10;    // 8 arrivals
    uint64_t* pds_full = bars + 11;    // 8 arrivals
    uint64_t* pds_free = bars + 12;
    uint64_t* acc_full = bars + 13;
    uint64_t* out_full = bars + 14;    // 8 arrivals: the output tile is staged in shared memory
    uint64_t* ds_stored = bars + 16;   // 2: the bulk store of dS buffer b has read it
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int kb = blockIdx.y;                 // early key blocks have the most query blocks: all heads' first
    const int bh = blockIdx.x;
    const int b = bh / p.H, h = bh % p.H;
    const int k0 = kb * ATT_BN;
    const int niter = p.nq - kb;

    if (threadIdx.x == 0) {
        mbar_init(kv_full, 1);
        for (int i = 0; i < ATT_BWD_STAGES; ++i) { mbar_init(&qdo_full[i], 1); mbar_init(&qdo_empty[i], 1); }
        mbar_init(sdp_full, 1); mbar_init(sdp_free, 8); mbar_init(pds_full, 8); mbar_init(pds_free, 1);
        mbar_init(acc_full, 1); mbar_init(out_full, 8);
        mbar_init(&ds_stored[0], 1); mbar_init(&ds_stored[1], 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();                 // everything above is independent of earlier kernels' results
    const uint32_t tS = tmem_base, tdP = tmem_base + 128, tdV = tmem_base + 256, tdK = tmem_base + 320;

    if (warp == 0) {
        if (lane == 0) {
            bool ok = true;
            mbar_expect_tx(kv_full, 2 * TILE_BYTES);
            tma_load_3d(sK, &tmK, kv_full, 0, k0, bh);
            tma_load_3d(sV, &tmV, kv_full, 0, k0, bh);
            for (int it = 0; it < niter && ok; ++it) {
                const int s = it % ATT_BWD_STAGES;
                if (!mbar_wait(&qdo_empty[s], (uint32_t)((it / ATT_BWD_STAGES) & 1) ^ 1u, abort_flag)) { ok = false; break; }
                const int q0 = (kb + it) * ATT_BM;
                mbar_expect_tx(&qdo_full[s], 2 * TILE_BYTES);
                tma_load_3d(sQ + s * TILE_BYTES, &tmQ, &qdo_full[s], 0, q0, bh);
                tma_load_4d(sdO + s * TILE_BYTES, &tmdO, &qdo_full[s], 0, q0, h, b);
            }
            pdl_launch_dependents_now();     // all loads issued: the next kernel may start its prologue
            if (!ok) { *abort_flag = 1; atomicExch(p.err, 21); }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t id_s = umma_idesc(1u, 0u, 0u, 128, 128);      // Q K^T, dO V^T
            const uint64_t dKk = kmajor_tile(smem_u32(sK)), dVk = kmajor_tile(smem_u32(sV));
            const uint64_t dQk0 = kmajor_tile(smem_u32(sQ)), ddOk0 = kmajor_tile(smem_u32(sdO));
            bool ok = mbar_wait(kv_full, 0, abort_flag);
            // S = Q K^T and dP = dO V^T of query block `it`; may run ahead of the accumulation of it-1
            // because the compute warps free the two score tiles as soon as they hold them in registers
            auto issue_sdp = [&](int it) -> bool {
                const int s = it % ATT_BWD_STAGES;
                const uint64_t dQk = dQk0 + (uint64_t)s * TILESTEP, ddOk = ddOk0 + (uint64_t)s * TILESTEP;
                if (!mbar_wait(&qdo_full[s], (uint32_t)((it / ATT_BWD_STAGES) & 1), abort_flag)) return false;
                if (!mbar_wait(sdp_free, (uint32_t)(it & 1) ^ 1u, abort_flag)) return false;
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_bf16(tS, dQk + k * KSTEP, dKk + k * KSTEP, id_s, k > 0 ? 1u : 0u);
#pragma unroll
                for (int k = 0; k < 4; ++k) umma_bf16(tdP, ddOk + k * KSTEP, dVk + k * KSTEP, id_s, k > 0 ? 1u : 0u);
                umma_commit(sdp_full);
                return true;
            };
            if (ok) ok = issue_sdp(0);
            for (int it = 0; it + 1 < niter && ok; ++it) ok = issue_sdp(it + 1);
            if (!ok) { *abort_flag = 1; atomicExch(p.err, 22); }
        }
    } else if (warp == 10) {
        // second issuer: dV += P^T dO and dK += dS^T Q once the compute warps have written P and dS
        if (lane == 0) {
            const uint32_t id_t = umma_idesc(1u, 1u, 1u, 128, 64);       // both operands MN-major
            const uint64_t dPm = mnmajor_tile(smem_u32(sP), TILE_BYTES), ddSm0 = mnmajor_tile(smem_u32(sdS), TILE_BYTES);
            const long long nblk = (long long)p.nq * (p.nq + 1) / 2;
            const uint64_t dQm0 = mnmajor_tile(smem_u32(sQ), TILE_BYTES), ddOm0 = mnmajor_tile(smem_u32(sdO), TILE_BYTES);
            bool ok = true;
            for (int it = 0; it < niter && ok; ++it) {
                const int s = it % ATT_BWD_STAGES;
                const uint64_t dQm = dQm0 + (uint64_t)s * TILESTEP, ddOm = ddOm0 + (uint64_t)s * TILESTEP;
                if (!mbar_wait(&qdo_full[s], (uint32_t)((it / ATT_BWD_STAGES) & 1), abort_flag)) { ok = false; break; }
                if (!mbar_wait(pds_full, (uint32_t)(it & 1), abort_flag)) { ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    umma_bf16(tdV, dPm + k * MNSTEP, ddOm + k * MNSTEP, id_t, (it > 0 || k > 0) ? 1u : 0u);
                const uint64_t ddSm = ddSm0 + (uint64_t)(it & 1) * (2 * TILESTEP);
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    umma_bf16(tdK, ddSm + k * MNSTEP, dQm + k * MNSTEP, id_t, (it > 0 || k > 0) ? 1u : 0u);
                umma_commit(pds_free);
                // S and dP of this block (the other issuer's) completed before the compute warps could sign
                // pds_full, so this commit covers every read of the stage
                umma_commit(&qdo_empty[s]);
                if (it == niter - 1) umma_commit(acc_full);      // the epilogue need not wait for the store below
                // the dS block leaves for the dQ kernel as it lies in shared memory; its buffer is written again two
                // steps from now, and this thread has nothing else to do until the next block is ready.  Not before the
                // products above have completed: a 32 KB read of shared memory beside them delays pds_free, which the
                // compute warps need ~900 cycles after they sign pds_full
                if (!mbar_wait(pds_free, (uint32_t)(it & 1), abort_flag)) { ok = false; break; }
                {
                    const int qb = kb + it;
                    uint8_t* dst = reinterpret_cast<uint8_t*>(p.ds) +
                                   ((long long)bh * nblk + (long long)qb * (qb + 1) / 2 + kb) * DS_BLOCK_BYTES;
                    bulk_store(dst, sdS + (it & 1) * DS_BLOCK_BYTES, DS_BLOCK_BYTES);
                    tma_store_commit();
                    tma_store_wait_read<0>();
                    mbar_arrive(&ds_stored[it & 1]);
                }
            }
            if (!ok) { *abort_flag = 1; atomicExch(p.err, 24); }
        }
    } else {
        const int q = warp & 3;
        const int half = (warp - 2) >> 2;             // which 64 key columns this warp handles
        const int r = q * 32 + lane;                  // query row inside the block
        const uint32_t lane_base = (uint32_t)(q * 32) << 16;
        bool ok = true;
        // the row's log-sum-exp and delta of the NEXT query block are fetched while this one is worked on
        float lse_next = INFINITY, dl_next = 0.0f;
        {
            const int qi0 = kb * ATT_BM + r;
            if (qi0 < p.T) { lse_next = p.lse[(long long)bh * p.T + qi0] * 1.4426950408889634f; dl_next = p.delta[(long long)bh * p.T + qi0]; }
        }
        for (int it = 0; it < niter && ok; ++it) {
            const uint32_t pi = (uint32_t)(it & 1);
            const int qb = kb + it;
            const int qi = qb * ATT_BM + r;
            const bool diag = (qb == kb);
            const float lse2 = lse_next, dl = dl_next;            // +inf for rows past T: P = 0
            lse_next = INFINITY; dl_next = 0.0f;
            if (it + 1 < niter && qi + ATT_BM < p.T) {
                lse_next = p.lse[(long long)bh * p.T + qi + ATT_BM] * 1.4426950408889634f;
                dl_next = p.delta[(long long)bh * p.T + qi + ATT_BM];
            }
            if (!mbar_wait(sdp_full, pi, abort_flag)) { ok = false; break; }
            tc_fence_after();
            // this thread's 64 scores and 64 dP values in one TMEM round trip, then the tiles are free
            uint32_t sv0[32], sv1[32], dv0[32], dv1[32];
            tmem_ld32(tS + lane_base + (half * 2) * 32, sv0);
            tmem_ld32(tS + lane_base + (half * 2 + 1) * 32, sv1);
            tmem_ld32(tdP + lane_base + (half * 2) * 32, dv0);
            tmem_ld32(tdP + lane_base + (half * 2 + 1) * 32, dv1);
            tmem_ld_wait();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(sdp_free);
            // rows past T get lse2 = +inf, i.e. P = 0; the diagonal block masks keys after the query
            float P[32], dS[32];
            p_and_ds(sv0, dv0, p.scale_log2, lse2, dl, diag, diag ? qi - (k0 + (half * 2) * 32) : 32, P, dS);
            if (!mbar_wait(pds_free, pi ^ 1u, abort_flag)) { ok = false; break; }     // previous P, dS consumed
            uint8_t* sdS_it = sdS + pi * DS_BLOCK_BYTES;                                // and this buffer's block stored
            if (!mbar_wait(&ds_stored[pi], (uint32_t)((it >> 1) & 1) ^ 1u, abort_flag)) { ok = false; break; }
            store_chunk_bf16(sP, r, half * 2, P);
            store_chunk_bf16(sdS_it, r, half * 2, dS);
            p_and_ds(sv1, dv1, p.scale_log2, lse2, dl, diag, diag ? qi - (k0 + (half * 2 + 1) * 32) : 32, P, dS);
            store_chunk_bf16(sP, r, half * 2 + 1, P);
            store_chunk_bf16(sdS_it, r, half * 2 + 1, dS);
            tc_fence_before();
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(pds_full);
        }
        const int kj = k0 + r;                        // key row of the accumulators
        RopeRow rot;                                  // fetched while the last products finish
        if (ok && kj < p.T && p.dqkv != nullptr)
            load_rope_row(rot, p.cos_t + (long long)kj * (p.hd >> 1), p.sin_t + (long long)kj * (p.hd >> 1), half * 32, p.hd);
        if (ok) {
            if (!mbar_wait(acc_full, 0, abort_flag)) ok = false;
        }
        if (ok) {
            tc_fence_after();
            uint32_t v[32], w[32];
            tmem_ld32(tdV + lane_base + half * 32, v);
            tmem_ld32(tdK + lane_base + half * 32, w);
            tmem_ld_wait();
            if (p.dqkv != nullptr) {
                // the P and dS tiles are free (every product has completed): dK into the first, dV into the second
                if (kj < p.T) {
                    stage_row_bf16(sP, r, w, half * 32, p.hd, &rot, p.scale);
                    stage_row_bf16(sP + TILE_BYTES, r, v, half * 32, p.hd, nullptr, 1.0f);
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(out_full);
                if (warp == 2 && lane == 0) {
                    if (mbar_wait(out_full, 0, abort_flag)) {
                        tma_store_4d(&tmoK, sP, 0, k0, h, b);              // rows past T are clipped
                        tma_store_4d(&tmoV, sP + TILE_BYTES, 0, k0, h, b);
                        tma_store_commit();
                        tma_store_wait_read<0>();
                    } else ok = false;
                }
            } else {
                // separate float32 outputs [B*H, T, hd]: dK into the two P tiles (head-dim columns 0-31 | 32-63), dV
                // into the two Q stages (a dS buffer may still be on its way out); tmoK / tmoV are float32 maps here
                if (kj < p.T && half * 32 < p.hd) {
                    stage_row_f32(sP + half * TILE_BYTES, r, w, p.scale);
                    stage_row_f32(sQ + half * TILE_BYTES, r, v, 1.0f);
                }
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(out_full);
                if (warp == 2 && lane == 0) {
                    if (mbar_wait(out_full, 0, abort_flag)) {
                        for (int c = 0; c * 32 < p.hd; ++c) {
                            tma_store_3d(&tmoK, sP + c * TILE_BYTES, c * 32, k0, bh);
                            tma_store_3d(&tmoV, sQ + c * TILE_BYTES, c * 32, k0, bh);
                        }
                        tma_store_commit();
                        tma_store_wait_read<0>();
                    } else ok = false;
                }
            }
        }
        if (!ok && lane == 0) { *abort_flag = 1; atomicExch(p.err, 23); }
    }

    __syncwarp();
    if (*abort_flag) for (int i = 0; i < 64; ++i) __nanosleep(1000);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// dQ of one query block: dQ = scale * sum over its key blocks kb = 0 .. qb of dS'(qb, kb) K(kb), the dS' blocks read
// back as the dK/dV kernel stored them.  No exponentials and no compute warps in the loop: a loader, a tensor-core
// issuer and four epilogue warps (thread = query row); two stages of 48 KB, so two CTAs share an SM and the prologue
// and epilogue of one hide behind the loop of the other.  Sums are formed in key-block order: fixed, no atomics.
constexpr int ATT_DQ_THREADS = 192;
constexpr int ATT_DQ_STAGES = 2;
constexpr int ATT_DQ_STAGE_BYTES = DS_BLOCK_BYTES + TILE_BYTES;

__global__ void __launch_bounds__(ATT_DQ_THREADS, 2)
attention_bwd_dq_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmoQ,
                        const AttBwdParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t pad = (1024u - (raw_addr & 1023u)) & 1023u;
    uint8_t* smem = smem_raw + pad;
    // stage s: dS block (two [128 x 64] tiles) then the K tile.  The request is 1 KB + the stages: the barriers go
    // behind the stages when the alignment pad leaves room there (the usual case: pad 0), else into the pad itself
    uint64_t* bars = reinterpret_cast<uint64_t*>(pad <= 768u ? smem + ATT_DQ_STAGES * ATT_DQ_STAGE_BYTES : smem_raw);
    uint64_t* full = bars;             // ATT_DQ_STAGES
    uint64_t* empty = bars + 2;        // ATT_DQ_STAGES
    uint64_t* acc_full = bars + 4;
    uint64_t* out_full = bars + 5;     // 4 arrivals
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 6);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int qb = p.nq - 1 - (int)blockIdx.y;       // heaviest query blocks of all heads first
    const int bh = blockIdx.x;
    const int b = bh / p.H, h = bh % p.H;
    const int q0 = qb * ATT_BM;
    const int niter = qb + 1;

    if (threadIdx.x == 0) {
        for (int i = 0; i < ATT_DQ_STAGES; ++i) { mbar_init(&full[i], 1); mbar_init(&empty[i], 1); }
        mbar_init(acc_full, 1); mbar_init(out_full, 4);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) { tmem_alloc(tmem_slot, 64); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tdQ = *tmem_slot;
    pdl_wait();                 // everything above is independent of earlier kernels' results

    if (warp == 0) {
        if (lane == 0) {
            bool ok = true;
            const long long nblk = (long long)p.nq * (p.nq + 1) / 2;
            const uint8_t* src = reinterpret_cast<const uint8_t*>(p.ds) +
                                 ((long long)bh * nblk + (long long)qb * (qb + 1) / 2) * DS_BLOCK_BYTES;
            for (int it = 0; it < niter && ok; ++it) {
                const int s = it % ATT_DQ_STAGES;
                if (!mbar_wait(&empty[s], (uint32_t)((it / ATT_DQ_STAGES) & 1) ^ 1u, abort_flag)) { ok = false; break; }
                uint8_t* st = smem + s * ATT_DQ_STAGE_BYTES;
                mbar_expect_tx(&full[s], ATT_DQ_STAGE_BYTES);
                bulk_load(st, src + (long long)it * DS_BLOCK_BYTES, DS_BLOCK_BYTES, &full[s]);
                tma_load_3d(st + DS_BLOCK_BYTES, &tmK, &full[s], 0, it * ATT_BN, bh);
            }
            pdl_launch_dependents_now();     // all loads issued: the next kernel may start its prologue
            if (!ok) { *abort_flag = 1; atomicExch(p.err, 31); }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t id_q = umma_idesc(1u, 0u, 1u, 128, 64);       // dS (K-major) x K block (MN-major)
            bool ok = true;
            for (int it = 0; it < niter && ok; ++it) {
                const int s = it % ATT_DQ_STAGES;
                const uint32_t st = smem_u32(smem + s * ATT_DQ_STAGE_BYTES);
                const uint64_t ddSk = kmajor_tile(st);
                const uint64_t dKm = mnmajor_tile(st + DS_BLOCK_BYTES, TILE_BYTES);
                if (!mbar_wait(&full[s], (uint32_t)((it / ATT_DQ_STAGES) & 1), abort_flag)) { ok = false; break; }
                tc_fence_after();
#pragma unroll
                for (int k = 0; k < 8; ++k)
                    umma_bf16(tdQ, ddSk + (uint64_t)(k >> 2) * TILESTEP + (uint64_t)(k & 3) * KSTEP, dKm + k * MNSTEP, id_q,
                              (it > 0 || k > 0) ? 1u : 0u);
                umma_commit(&empty[s]);
            }
            if (ok) umma_commit(acc_full);
            if (!ok) { *abort_flag = 1; atomicExch(p.err, 32); }
        }
    } else {
        const int q = warp & 3;
        const int r = q * 32 + lane;
        const int qi = q0 + r;
        const bool valid = qi < p.T;
        const uint32_t lane_base = (uint32_t)(q * 32) << 16;
        bool ok = true;
        RopeRow rot0, rot1;                           // fetched while the products run
        if (valid && p.dqkv != nullptr) {
            const float* cs = p.cos_t + (long long)qi * (p.hd >> 1);
            const float* sn = p.sin_t + (long long)qi * (p.hd >> 1);
            load_rope_row(rot0, cs, sn, 0, p.hd);
            load_rope_row(rot1, cs, sn, 32, p.hd);
        }
        if (!mbar_wait(acc_full, 0, abort_flag)) ok = false;
        if (ok) {
            tc_fence_after();
            uint32_t v0[32], v1[32];
            tmem_ld32(tdQ + lane_base, v0);
            tmem_ld32(tdQ + lane_base + 32, v1);
            tmem_ld_wait();
            uint8_t* out = smem;                      // stage 0 is free: every product has completed
            if (p.dqkv != nullptr) {
                if (valid) {
                    stage_row_bf16(out, r, v0, 0, p.hd, &rot0, p.scale);
                    stage_row_bf16(out, r, v1, 32, p.hd, &rot1, p.scale);
                }
            } else if (valid) {                       // float32 dQ [B*H, T, hd]
                stage_row_f32(out, r, v0, p.scale);
                if (p.hd > 32) stage_row_f32(out + TILE_BYTES, r, v1, p.scale);
            }
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(out_full);
            if (q == 0 && lane == 0) {
                if (mbar_wait(out_full, 0, abort_flag)) {
                    if (p.dqkv != nullptr) tma_store_4d(&tmoQ, out, 0, q0, h, b);          // rows past T are clipped
                    else for (int c = 0; c * 32 < p.hd; ++c) tma_store_3d(&tmoQ, out + c * TILE_BYTES, c * 32, q0, bh);
                    tma_store_commit();
                    tma_store_wait_read<0>();
                } else ok = false;
            }
        }
        if (!ok && lane == 0) { *abort_flag = 1; atomicExch(p.err, 33); }
    }

    __syncwarp();
    if (*abort_flag) for (int i = 0; i < 64; ++i) __nanosleep(1000);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) { tc_fence_after(); tmem_dealloc(tdQ, 64); }
}

constexpr int ATT_DKDV_SMEM = 1024 + (8 + 2 * ATT_BWD_STAGES) * TILE_BYTES + 256;
constexpr int ATT_DQ_SMEM = 1024 + ATT_DQ_STAGES * ATT_DQ_STAGE_BYTES;

size_t attention_bwd_ds_bytes(int B, int H, int T) {
    const long long nq = (T + ATT_BM - 1) / ATT_BM;
    return (size_t)((long long)B * H * (nq * (nq + 1) / 2) * DS_BLOCK_BYTES);
}

int launch_attention_bwd(DeviceCtx* ctx, const bf16* Q, const bf16* K, const bf16* V, const bf16* att,
                         const bf16* datt, const float* lse, float* delta, float* dQ, float* dK, float* dV, int B,
                         int H, int T, int hd, float scale, cudaStream_t stream, bf16* dqkv, const float* cos_t,
                         const float* sin_t, bf16* ds_blocks) {
    TB_CHECK(hd > 0 && hd <= ATT_HD && hd % 8 == 0, "fused attention needs head_dim <= 64 and a multiple of 8 (got %d)", hd);
    TB_CHECK(dqkv != nullptr ? (cos_t && sin_t && (reinterpret_cast<uintptr_t>(dqkv) & 15u) == 0) : (dQ && dK && dV),
             "attention backward needs either dQ, dK, dV or the merged output with the rotation tables");
    TB_CHECK(B > 0 && H > 0 && T > 0, "attention dims must be positive");
    const int BH = B * H, D = H * hd;
    CUtensorMap tmQ, tmK, tmV, tmdO;
    TB_TRY(make_operand_map(&tmQ, Q, hd, T, hd, BH, (long long)T * hd, 128));
    TB_TRY(make_operand_map(&tmK, K, hd, T, hd, BH, (long long)T * hd, 128));
    TB_TRY(make_operand_map(&tmV, V, hd, T, hd, BH, (long long)T * hd, 128));
    TB_TRY(make_operand_map4(&tmdO, datt, hd, T, D, H, hd, B, (long long)T * D, 128));
    // the merged output dqkv [B*T, 3D] as three (hd, T, H, B) views for the tile stores
    CUtensorMap tmoQ = tmdO, tmoK = tmdO, tmoV = tmdO;
    if (dqkv != nullptr) {
        TB_TRY(make_operand_map4(&tmoQ, dqkv, hd, T, 3LL * D, H, hd, B, (long long)T * 3 * D, 128));
        TB_TRY(make_operand_map4(&tmoK, dqkv + D, hd, T, 3LL * D, H, hd, B, (long long)T * 3 * D, 128));
        TB_TRY(make_operand_map4(&tmoV, dqkv + 2 * D, hd, T, 3LL * D, H, hd, B, (long long)T * 3 * D, 128));
    } else {
        TB_TRY(make_operand_map_f32(&tmoQ, dQ, hd, T, hd, BH, (long long)T * hd, 128));
        TB_TRY(make_operand_map_f32(&tmoK, dK, hd, T, hd, BH, (long long)T * hd, 128));
        TB_TRY(make_operand_map_f32(&tmoV, dV, hd, T, hd, BH, (long long)T * hd, 128));
    }
    AttBwdParams p;
    p.T = T; p.H = H; p.hd = hd; p.nq = (T + ATT_BM - 1) / ATT_BM;
    p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
    p.lse = lse; p.delta = delta; p.dQ = dQ; p.dK = dK; p.dV = dV; p.err = ctx->d_err;
    p.dqkv = dqkv; p.cos_t = cos_t; p.sin_t = sin_t;
    if (ds_blocks == nullptr) {      // no caller-owned buffer for the dS blocks: the context's scratch
        TB_TRY(ensure_scratch(ctx, attention_bwd_ds_bytes(B, H, T)));
        ds_blocks = reinterpret_cast<bf16*>(ctx->scratch);
    }
    TB_CHECK((reinterpret_cast<uintptr_t>(ds_blocks) & 15u) == 0, "the dS block buffer must be 16-byte aligned");
    p.ds = ds_blocks;
    static bool attr_set[64] = {false};
    if (!attr_set[ctx->device & 63]) {
        TB_CUDA(cudaFuncSetAttribute(attention_bwd_dkdv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_DKDV_SMEM));
        TB_CUDA(cudaFuncSetAttribute(attention_bwd_dq_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_DQ_SMEM));
        attr_set[ctx->device & 63] = true;
    }
    {
        const long long total = (long long)B * T * H;
        long long blocks = (total + 255) / 256;
        if (blocks > 16LL * ctx->sm_count) blocks = 16LL * ctx->sm_count;
        prof_mark(ctx, "attention_delta", 0.0, 0.0, stream);
        TB_CUDA(launch_kernel(attention_delta_kernel, dim3((int)blocks), dim3(256), 0, stream, att, datt, delta, B, T, H, hd));
        TB_CUDA(cudaGetLastError());
        ctx->launches++;
        prof_close(ctx, stream);
    }
    dim3 grid(BH, p.nq);
    const double tri = (double)BH * T * (double)T * hd;      // one lower-triangular product = tri flops
    prof_mark(ctx, "attention_bwd_dkdv", 4.0 * tri, (double)BH * T * hd * (2.0 * 4 + 8.0), stream);
    TB_CUDA(launch_kernel(attention_bwd_dkdv_kernel, dim3(grid), dim3(ATT_BWD_THREADS), ATT_DKDV_SMEM, stream, tmQ, tmK, tmV, tmdO, tmoK, tmoV, p));
    TB_CUDA(cudaGetLastError());
    ctx->launches++;
    prof_close(ctx, stream);
    prof_mark(ctx, "attention_bwd_dq", 1.0 * tri, (double)BH * T * hd * (2.0 * 4 + 4.0), stream);
    TB_CUDA(launch_kernel(attention_bwd_dq_kernel, dim3(grid), dim3(ATT_DQ_THREADS), ATT_DQ_SMEM, stream, tmK, tmoQ, p));
    TB_CUDA(cudaGetLastError());
    ctx->launches++;
    prof_close(ctx, stream);
    return 0;
}

constexpr int ATT_FWD_SMEM = 1024 + 7 * TILE_BYTES;

int launch_attention_fwd(DeviceCtx* ctx, const bf16* Q, const bf16* K, const bf16* V, bf16* att, float* lse, int B,
                         int H, int T, int hd, float scale, cudaStream_t stream, long long kv_rows_per_head) {
    TB_CHECK(hd > 0 && hd <= ATT_HD && hd % 8 == 0, "fused attention needs head_dim <= 64 and a multiple of 8 (got %d)", hd);
    TB_CHECK(B > 0 && H > 0 && T > 0, "attention dims must be positive");
    const int BH = B * H;
    CUtensorMap tmQ, tmK, tmV;
    TB_TRY(make_operand_map(&tmQ, Q, hd, T, hd, BH, (long long)T * hd, ATT_BM));
    const long long kv_rows = kv_rows_per_head > 0 ? kv_rows_per_head : T;      // a KV cache has room for more rows
    TB_TRY(make_operand_map(&tmK, K, hd, T, hd, BH, kv_rows * hd, ATT_BN));
    TB_TRY(make_operand_map(&tmV, V, hd, T, hd, BH, kv_rows * hd, ATT_BN));
    CUtensorMap tmO;        // att [B*T, D] as (hd, T, H, B) for the tile store
    TB_TRY(make_operand_map4(&tmO, att, hd, T, (long long)H * hd, H, hd, B, (long long)T * H * hd, ATT_BM));
    AttFwdParams p;
    p.T = T; p.H = H; p.hd = hd; p.D = H * hd;
    p.nq = (T + ATT_BM - 1) / ATT_BM;
    p.scale_log2 = scale * 1.4426950408889634f;
    p.att = att; p.lse = lse; p.err = ctx->d_err;
    static bool attr_set[64] = {false};
    if (!attr_set[ctx->device & 63]) {
        TB_CUDA(cudaFuncSetAttribute(attention_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ATT_FWD_SMEM));
        attr_set[ctx->device & 63] = true;
    }
    dim3 grid(BH, p.nq);
    // algorithmic work: the lower triangle of two products of 2*T*T*hd flops each
    prof_mark(ctx, "attention_fwd", 2.0 * (double)BH * T * (double)T * hd, (double)BH * T * hd * 2.0 * 4.0, stream);
    TB_CUDA(launch_kernel(attention_fwd_kernel, dim3(grid), dim3(192), ATT_FWD_SMEM, stream, tmQ, tmK, tmV, tmO, p));
    TB_CUDA(cudaGetLastError());
    ctx->launches++;
    prof_close(ctx, stream);
    return 0;
}

}  // namespace tb

