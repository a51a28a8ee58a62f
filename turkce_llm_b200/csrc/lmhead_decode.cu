// Decode-time LM head with the greedy choice fused: tok[s] = argmax_v <x_s, E_v> for up to 64
// sequences, without writing the [S, V] logits.
//
// The reference has no decode path of its own; its generator recomputes lm_forward over the whole
// window and takes the last row (model/generate.c:204-206, model/lm_model.c:72-81: logits =
// RMSNorm(x) . E^T with the tied embedding table E [V, D]).  At 64 sequences this product is
// bound by streaming E (24.4 MB in bf16 for V = 31,769, D = 384) from HBM once.
//
// Shape of the kernel: the vocabulary is cut into one contiguous slice of rows per CTA (one CTA
// per SM), small enough that the whole slice [rows, D] sits in shared memory.  Each CTA issues all
// of its TMA loads at once (so every SM has its full share of the table in flight from the first
// microsecond), multiplies the slice -- as the M = 128 operand -- by the 64 hidden states on the
// tensor cores (tcgen05, accumulator [128 vocabulary rows x 64 sequences] in TMEM), turns the
// accumulator through shared memory and scans it per sequence.  Each CTA's winners go into one
// packed 64-bit maximum per sequence in global memory (order-independent: the largest value wins,
// among equals the lowest index, as the unfused argmax does); the CTA that finishes last (a ticket)
// publishes the tokens, advances the decoder's position state and clears the maxima.
#include "common.h"
#include "ptx.cuh"

namespace tb {

namespace {

constexpr int LH_THREADS = 256;
constexpr int LH_SEQ = 64;          // sequences per launch = UMMA N
constexpr int LH_BK = 64;           // bf16 elements per 128-byte row
constexpr int LH_XK_BYTES = LH_SEQ * 128;   // one K slice of the hidden states
constexpr int LH_STAGE_LD = 260;    // floats per staged sequence: 256 rows + 4 (16-byte loads of 8 sequences hit 32 banks)
constexpr int LH_MAX_SMEM = 227 * 1024;
constexpr int LH_HEADER_BYTES = 8192;
constexpr int LH_MAX_KBLOCKS = 64;

struct LmHeadParams {
    int V, S, kblocks, rows_per_cta, box_rows;
    int early_table;          // the table is not written by earlier kernels of the stream: load it before the fence
    unsigned long long* best; // [64] packed (value key, ~index) maxima over the CTAs; zero between launches
    unsigned int* ticket;     // zero between launches
    uint32_t* tok;            // [S]
    uint32_t* out;            // optional [S, out_ld]: generated tokens
    int* state;               // optional {position of the next token, tokens generated}
    int out_ld, advance_pos;
    float* logits;            // optional [S, ld_logits]
    long long ld_logits;
    int* err;
};

__global__ void __launch_bounds__(LH_THREADS, 1)
lmhead_argmax_kernel(const __grid_constant__ CUtensorMap tmE, const __grid_constant__ CUtensorMap tmX,
                     const LmHeadParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);
    // header (barriers, TMEM slot, reduction arrays) | table slice | hidden states | padding: the
    // second 128-row operand chunk of the last K slice is read past the slice's own rows (those
    // accumulator rows are never looked at), and that read must stay inside the allocation
    const int e_bytes = p.box_rows * 128;                       // one K slice of this CTA's rows
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem);
    uint8_t* sE = smem + LH_HEADER_BYTES;                        // [kblocks][box_rows][128 B]
    uint8_t* sX = sE + p.kblocks * e_bytes;                      // [kblocks][64][128 B]
    uint64_t* full_bar = bars;                                   // [kblocks]: one K slice of the table
    uint64_t* x_bar = bars + p.kblocks;                          // the hidden states
    uint64_t* acc_bar = bars + p.kblocks + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + p.kblocks + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    int* is_last = reinterpret_cast<int*>(tmem_slot + 2);
    float* red_val = reinterpret_cast<float*>(tmem_slot + 4);    // [4 segments][64]
    uint32_t* red_row = tmem_slot + 4 + 4 * LH_SEQ;              // [4 segments][64]

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int row0 = blockIdx.x * p.rows_per_cta;
    const int rows_here = min(p.rows_per_cta, p.V - row0);
    const int nchunks = (p.box_rows + 127) / 128;

    if (threadIdx.x == 0) {
        for (int i = 0; i < p.kblocks; ++i) mbar_init(&full_bar[i], 1);
        mbar_init(x_bar, 1);
        mbar_init(acc_bar, 1);
        *abort_flag = 0;
        fence_mbar_init();
        if (p.early_table) {
            // every table load of this CTA at once, before the fence on earlier kernels: the weights do not
            // depend on them, so the stream of the table overlaps the previous kernel's tail
            for (int kb = 0; kb < p.kblocks; ++kb) {
                mbar_expect_tx(&full_bar[kb], (uint32_t)e_bytes);
                tma_load_3d(sE + kb * e_bytes, &tmE, &full_bar[kb], kb * LH_BK, row0, 0);
            }
        }
        tma_prefetch_desc(&tmX);
    }
    if (warp == 1) { tmem_alloc(tmem_slot, 128); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    pdl_wait();                 // the hidden states come from the previous kernel of the stream

    if (warp == 0 && lane == 0) {
        mbar_expect_tx(x_bar, (uint32_t)(p.kblocks * LH_XK_BYTES));
        for (int kb = 0; kb < p.kblocks; ++kb) tma_load_3d(sX + kb * LH_XK_BYTES, &tmX, x_bar, kb * LH_BK, 0, 0);
        if (!p.early_table) {
            for (int kb = 0; kb < p.kblocks; ++kb) {
                mbar_expect_tx(&full_bar[kb], (uint32_t)e_bytes);
                tma_load_3d(sE + kb * e_bytes, &tmE, &full_bar[kb], kb * LH_BK, row0, 0);
            }
        }
        pdl_launch_dependents_now();
    } else if (warp == 1 && lane == 0) {
        const uint32_t idesc = umma_idesc(1u, 0u, 0u, 128, LH_SEQ);
        bool ok = mbar_wait(x_bar, 0u, abort_flag);
        for (int kb = 0; kb < p.kblocks && ok; ++kb) {
            if (!mbar_wait(&full_bar[kb], 0u, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const uint32_t e_addr = smem_u32(sE + kb * e_bytes);
            const uint32_t x_addr = smem_u32(sX + kb * LH_XK_BYTES);
            for (int c = 0; c < nchunks; ++c) {
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    umma_bf16(tmem_base + (uint32_t)(c * LH_SEQ), umma_desc_sw128(e_addr + c * 16384 + k * 32, 16, 1024),
                              umma_desc_sw128(x_addr + k * 32, 16, 1024), idesc, (kb | k) != 0 ? 1u : 0u);
            }
        }
        if (ok) umma_commit(acc_bar);
        else { *abort_flag = 1; atomicExch(p.err, 41); }
    }
    __syncwarp();

    // ---- accumulator [vocabulary row (lane), sequence (column)] -> shared memory, sequence-major
    // (over the consumed table slice): lanes write consecutive addresses, readers take 4 rows per load
    const bool done = mbar_wait(acc_bar, 0u, abort_flag);
    tc_fence_after();
    float* stage = reinterpret_cast<float*>(sE);
    const int chunk = warp >> 2, q = warp & 3;
    if (done && chunk < nchunks) {
        const int r = chunk * 128 + q * 32 + lane;
        const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(chunk * LH_SEQ);
        uint32_t v0[32], v1[32];
        tmem_ld32(taddr, v0);
        tmem_ld32(taddr + 32, v1);
        tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) {
            stage[c * LH_STAGE_LD + r] = __uint_as_float(v0[c]);
            stage[(32 + c) * LH_STAGE_LD + r] = __uint_as_float(v1[c]);
        }
    }
    tc_fence_before();
    // a CTA whose wait ran out skips the scan but still takes its ticket below, so that the ticket word and
    // the maxima are back at zero when the launch ends (the error word tells the host the tokens are invalid)
    const int all_done = __syncthreads_and(done ? 1 : 0);
    if (warp == 1) tmem_dealloc(tmem_base, 128);

    if (all_done) {
    // ---- per sequence: 4 threads scan a quarter of the rows each, four rows per load, in four
    // independent chains (row mod 4); every comparison prefers the lower row on equal values
    {
        const int s = threadIdx.x & (LH_SEQ - 1), seg = threadIdx.x >> 6;
        const int seg_len = ((rows_here + 15) >> 4) << 2;              // multiple of 4 rows
        const int r0 = seg * seg_len, r1 = min(r0 + seg_len, rows_here);
        const float* src = stage + s * LH_STAGE_LD;
        // every chain starts on a row of this CTA with the lowest key, so that a sequence whose products are
        // all NaN or -inf (diverged weights) still yields a token inside the vocabulary
        float bv[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        int br[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) br[j] = r0 + j < r1 ? r0 + j : (r0 < r1 ? r0 : 0);
        for (int r = r0; r < r1; r += 4) {
            const float4 v = *reinterpret_cast<const float4*>(src + r);
            const float e[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (r + j < r1 && e[j] > bv[j]) { bv[j] = e[j]; br[j] = r + j; }      // false for NaN
        }
#pragma unroll
        for (int j = 1; j < 4; ++j)
            if (bv[j] > bv[0] || (bv[j] == bv[0] && br[j] < br[0])) { bv[0] = bv[j]; br[0] = br[j]; }
        red_val[seg * LH_SEQ + s] = bv[0];
        red_row[seg * LH_SEQ + s] = (uint32_t)br[0];
    }
    if (p.logits != nullptr) {
        // optional: the products themselves
        for (int s = 0; s < p.S; ++s)
            for (int rr = threadIdx.x; rr < rows_here; rr += LH_THREADS)
                p.logits[(long long)s * p.ld_logits + row0 + rr] = stage[s * LH_STAGE_LD + rr];
    }
    __syncthreads();

    // ---- this CTA's winners (segments hold ascending row ranges: strict > keeps the lowest row on ties)
    // go into one packed maximum per sequence: value as an order-preserving key in the high word, the
    // complemented index in the low word, so the largest value wins and among equals the lowest index
    // -- whatever order the CTAs arrive in
    if (threadIdx.x < LH_SEQ) {
        const int s = threadIdx.x;
        float best = red_val[s];
        uint32_t row = red_row[s];
#pragma unroll
        for (int seg = 1; seg < 4; ++seg) {
            const float v = red_val[seg * LH_SEQ + s];
            if (v > best) { best = v; row = red_row[seg * LH_SEQ + s]; }
        }
        const uint32_t b = __float_as_uint(best + 0.0f);                       // -0 -> +0
        const uint32_t key = (b & 0x80000000u) ? ~b : (b | 0x80000000u);
        atomicMax(p.best + s, ((unsigned long long)key << 32) | (unsigned long long)(0xffffffffu - ((uint32_t)row0 + row)));
        __threadfence();
    }
    }   // all_done
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int t = atomicAdd(p.ticket, 1u);
        *is_last = (t == gridDim.x - 1u) ? 1 : 0;
        if (t == gridDim.x - 1u) *p.ticket = 0u;                 // ready for the next launch
    }
    __syncthreads();
    if (!*is_last) return;
    __threadfence();

    // ---- the last CTA to finish publishes the choices and clears the maxima for the next launch
    const int generated = p.state != nullptr ? p.state[1] : 0;
    if (threadIdx.x < LH_SEQ) {
        const int s = threadIdx.x;
        const unsigned long long packed = __ldcg(p.best + s);
        p.best[s] = 0ull;
        if (s < p.S) {
            uint32_t idx = 0xffffffffu - (uint32_t)(packed & 0xffffffffull);
            if (idx >= (uint32_t)p.V) idx = 0u;      // only after an aborted launch: keep the fed-back token in range
            p.tok[s] = idx;
            if (p.out != nullptr) p.out[(long long)s * p.out_ld + generated] = idx;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && p.state != nullptr) {
        p.state[1] = generated + 1;
        if (p.advance_pos) p.state[0] += 1;
    }
}

struct LmHeadPlan { int ctas, rows_per_cta, box_rows, kblocks; size_t smem; };

bool plan(const DeviceCtx* ctx, int S, int V, int K, LmHeadPlan* out) {
    if (S < 1 || S > LH_SEQ || V < 1 || K < LH_BK || K % LH_BK != 0 || K / LH_BK > LH_MAX_KBLOCKS) return false;
    LmHeadPlan pl;
    pl.kblocks = K / LH_BK;
    // most rows whose slice (plus header, hidden states and 1 KB of alignment slack) fits
    const long long fixed = LH_HEADER_BYTES + (long long)pl.kblocks * LH_XK_BYTES + 1024;
    long long max_rows = (LH_MAX_SMEM - fixed) / ((long long)pl.kblocks * 128);
    max_rows = std::min<long long>(max_rows, 256) / 8 * 8;
    if (max_rows < 8) return false;
    int rows = (V + ctx->sm_count - 1) / ctx->sm_count;
    if (rows > max_rows) rows = (int)max_rows;
    pl.ctas = (V + rows - 1) / rows;
    pl.rows_per_cta = rows;
    pl.box_rows = (int)round_up(rows, 8);
    const long long nchunks = (pl.box_rows + 127) / 128;
    const long long e_bytes = (long long)pl.box_rows * 128;
    const long long data = (long long)pl.kblocks * (e_bytes + LH_XK_BYTES);
    // operand reads reach (kblocks-1) slices + whole 128-row chunks; the staged accumulator lies over the data
    const long long reach = std::max((long long)(pl.kblocks - 1) * e_bytes + nchunks * 16384,
                                     (long long)LH_SEQ * LH_STAGE_LD * 4);
    pl.smem = (size_t)(LH_HEADER_BYTES + std::max(data, reach) + 1024);
    if (pl.smem > (size_t)LH_MAX_SMEM) return false;
    *out = pl;
    return true;
}

}  // namespace

bool lmhead_argmax_supported(const DeviceCtx* ctx, int S, int V, int K) {
    LmHeadPlan pl;
    return plan(ctx, S, V, K, &pl);
}

int lmhead_argmax_ctas(const DeviceCtx* ctx, int S, int V, int K) {
    LmHeadPlan pl;
    return plan(ctx, S, V, K, &pl) ? pl.ctas : 0;
}

int launch_lmhead_argmax(DeviceCtx* ctx, const bf16* X, const bf16* E, int S, int V, int K, bool table_is_stable,
                         unsigned long long* best, unsigned int* ticket, uint32_t* tok, uint32_t* out, int* state,
                         int out_ld, int advance_pos, float* logits, long long ld_logits, cudaStream_t st) {
    LmHeadPlan pl;
    TB_CHECK(plan(ctx, S, V, K, &pl), "fused LM head: unsupported shape S=%d V=%d K=%d", S, V, K);
    CUtensorMap tmE, tmX;
    TB_TRY(make_operand_map(&tmE, E, K, V, K, 1, 0, pl.box_rows));
    TB_TRY(make_operand_map(&tmX, X, K, S, K, 1, 0, LH_SEQ));
    LmHeadParams p;
    p.V = V; p.S = S; p.kblocks = pl.kblocks; p.rows_per_cta = pl.rows_per_cta; p.box_rows = pl.box_rows;
    p.early_table = table_is_stable ? 1 : 0;
    p.best = best; p.ticket = ticket; p.tok = tok; p.out = out; p.state = state;
    p.out_ld = out_ld; p.advance_pos = advance_pos;
    p.logits = logits; p.ld_logits = ld_logits; p.err = ctx->d_err;
    static bool attr_set[64] = {false};
    if (!attr_set[ctx->device & 63]) {
        TB_CUDA(cudaFuncSetAttribute(lmhead_argmax_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, LH_MAX_SMEM));
        attr_set[ctx->device & 63] = true;
    }
    const double bytes = 2.0 * V * K + 2.0 * S * K;
    prof_mark(ctx, "lmhead_argmax", 2.0 * S * (double)V * K, bytes, st);
    TB_CUDA(launch_kernel(lmhead_argmax_kernel, dim3(pl.ctas), dim3(LH_THREADS), pl.smem, st, tmE, tmX, p));
    ctx->launches++;
    prof_close(ctx, st);
    return 0;
}

}  // namespace tb
