// Persistent TMA + tcgen05 GEMM for sm_100a on BF16 operands with FP32 accumulation in TMEM.
//
//   C = alpha * op(A) * op(B) [+ bias] [+ residual] [+ beta * C]
//
// replaces the reference's gemm_body / bf16_gemm_body / k_bf16_gemm_nn_bias
// (cuda/train_kernels.cu:110-193, :226-329, :343-467).  One kernel covers NN, NT and TN:
// a transposed operand is not transposed in memory, it is described to the tensor core
// as an MN-major shared-memory tile instead of a K-major one.
//
// CTA = 6 warps, one CTA per SM, tiles 128 x BN handed out round-robin:
//   warp 0     TMA producer: 64-wide K slices of A and B into a ring of 128B-swizzled stages
//   warp 1     owns TMEM (2 accumulators of BN columns) and issues tcgen05.mma (one lane)
//   warps 2-5  epilogue: tcgen05.ld -> registers -> per-warp shared staging -> coalesced
//              global stores with bias / residual / beta*C / bf16 copy fused
// The two accumulators let the epilogue of tile i overlap the main loop of tile i+1,
// which matters because K is only 384..1024 here (6..16 slices per tile).
//
// Split-K (weight gradients: small M,N, K = tokens) writes one partial tile per split into
// scratch memory; reduce_splits_kernel then adds the partials in split order, so the result
// does not depend on scheduling (the reference forbids atomics: train_kernels.cu:17-20).
#include "../../include/turkce_b200.h"
#include "common.h"
#include "ptx.cuh"

#include <cstdlib>
#include <cstring>
#include <mutex>
#include <cstring>

namespace tb {

constexpr int BM = 128;
constexpr int BK = 64;              // bf16 elements of one 128-byte swizzle row
constexpr int BK_TF32 = 32;         // float32 elements of one 128-byte swizzle row (kind::tf32 operands)
constexpr int ROW_BYTES = 128;
constexpr int NUM_THREADS = 320;      // TMA warp, MMA warp, 8 epilogue warps
constexpr int EPI_WARPS = 8;
constexpr int STAGE_LD = 36;        // floats per staging row (32 + 4 pad: conflict-free float4 access)

// PAIR: two CTAs of a cluster share a 256 x BN tile (cta_group::2): each loads its own 128 rows of A and
// BN/2 columns of B, so a CTA's shared-memory traffic per output element drops by BN/(128 + BN/2)/(BN/(128+BN)).
// BN = 384 (PAIR, B stored [K, N]): for products with N <= 384 and a long K (the LM-head gradients): one tile spans
// the whole N, 40 KB per K slice feed 768 tensor-core cycles (53 B/clk against 64 for 256 x 256 with half of the
// second tile empty).  The tensor core takes N <= 256, so a K step is three instructions of 128 columns; each CTA
// loads the 64-column boxes at n0 + 128 j + 64 rank, which keeps accumulator column = output column.  One accumulator.
template <int BN, bool PAIR = false> struct GemmCfg {
    static constexpr int BN_LOCAL = PAIR ? BN / 2 : BN;   // columns of B this CTA loads
    static constexpr int A_BYTES = BM * ROW_BYTES;      // one K slice: 128-byte rows for either operand type
    static constexpr int B_BYTES = BN_LOCAL * ROW_BYTES;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr int STAGES = (PAIR && BN == 384) ? 3 : PAIR ? 4 : (BN == 192) ? 3 : (BN == 128) ? 4 : 5;
    // per epilogue warp: 2 output buffers + 1 residual buffer of 32 rows x 128 B (TMA path);
    // the generic path uses the front of the same region (32 x 36 floats per warp)
    static constexpr int EPI_WARP_BYTES = 3 * 4096;
    static constexpr int STAGING_BYTES = EPI_WARPS * EPI_WARP_BYTES;
    static constexpr int BAR_BYTES = 512;
    static constexpr int SMEM_BYTES = 1024 + STAGES * STAGE_BYTES + STAGING_BYTES + BAR_BYTES;
    static constexpr int TMEM_COLS = (2 * BN <= 128) ? 128 : (2 * BN <= 256) ? 256 : 512;   // power of two
    // accumulators in TMEM: two (the epilogue of tile i overlaps the main loop of tile i+1) unless one fills it
    static constexpr int NBUF = (2 * BN <= 512) ? 2 : 1;
};

struct GemmParams {
    int M, N, K;
    int batch, splits;
    int mt, nt;                 // tiles along M, N
    int kb_total, kb_per;       // K slices in all, and per split
    int a_mn, b_mn;             // 1 = operand tile is MN-major (stored transposed)
    int causal;
    float* C32; long long ldc32, strideC32, strideC32_in;
    bf16* C16; long long ldc16, strideC16, strideC16_in;
    int c_inner;                // output batch index z -> (z / c_inner) * stride + (z % c_inner) * stride_in
    const float* bias;
    const float* residual; long long ldr, strideR;
    float alpha, beta;
    int vec32, vec16, vecr;     // 16-byte (8-byte for bf16) vector access allowed
    int tma_mode;               // 0: generic epilogue; 1: fp32 tile stores by TMA; 2: bf16 tile stores by TMA;
                                // 3: SwiGLU (tmC = h [M,F] bf16, tmR = gate|up [M,2F] bf16 when keep_gu)
                                // 4: softmax statistics only (cross-entropy pass 1), nothing stored
                                // 5: bf16 tiles into [3][B][H][T][hd] with q, k rotated (tmC is a 5-D map)
    const float* rope_cos; const float* rope_sin; int rope_T, rope_H, rope_hd;
    int ce_mode;                // 2: bf16 tile stores carry (exp(z - lse[row]) - onehot) * ce_scale
    const uint32_t* ce_targets; float* ce_stats; float* ce_ztarget; const float* ce_lse; float ce_scale;
    int pair_off;               // mode 3: F; tile columns [0,BN/2) are gate columns n0/2.., [BN/2,BN) up columns F + n0/2..
    int keep_gu;
    int wide16;                 // bf16 tiles leave two 32-column chunks at a time: 32 rows x 128 bytes per store through the
                                // 64-column map (tmR; with dsw: tmC), a last odd chunk through the 32-column map tmC
    int dsw;                    // SwiGLU backward: the product is dh; tmR = saved gate|up [M,2F] bf16, tmC = dgu [M,2F] bf16
    int tma_res;                // TMA path: add res_scale * (tile of tmR) -- the residual, or the old C for beta
    float res_scale;
    int bias_vec;               // bias pointer is 16-byte aligned
    int* err;
};

// Built with -DTB_GEMM_STAMPS (TB_NVCC_FLAGS of the build script), every CTA records %globaltimer at the points of its
// life named in tb_debug_gemm_stamps' header comment; `python bench.py --only timeline ...` prints them.  Off by default.
#ifdef TB_GEMM_STAMPS
__device__ unsigned long long g_gemm_stamps[160][16];
__device__ __forceinline__ void gemm_stamp(int slot) {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    if (blockIdx.x < 160) g_gemm_stamps[blockIdx.x][slot] = t;
}
#define TS(slot) gemm_stamp(slot)
#else
#define TS(slot) do { } while (0)
#endif

struct TileCoord { int z, s, m0, n0, kb0, kb1; bool skip; };

template <int BN, int BKE, int TILE_M = BM>
__device__ __forceinline__ TileCoord tile_of(const GemmParams& p, int t, int row_off = 0) {
    TileCoord c;
    // (integer divisions by run-time values cost ~100 cycles each on the path to a tile's first load: the K-slice
    // counts come from the host, and the common single-split, single-batch launch skips two more)
    const int n_idx = t % p.nt; t /= p.nt;
    int m_idx = t;
    c.s = 0; c.z = 0;
    if (p.batch * p.splits != 1) {
        m_idx = t % p.mt; t /= p.mt;
        c.s = t % p.splits;
        c.z = t / p.splits;
    }
    c.m0 = m_idx * TILE_M + row_off;
    c.n0 = n_idx * BN;
    const int kb_total = p.kb_total;
    const int kb_per = p.kb_per;
    c.kb0 = c.s * kb_per;
    c.kb1 = min(kb_total, c.kb0 + kb_per);
    c.skip = false;
    if (p.causal == CAUSAL_SKIP_UPPER) {
        c.skip = c.n0 > c.m0 + BM - 1;
    } else if (p.causal == CAUSAL_K_PREFIX) {
        c.kb1 = min(c.kb1, (c.m0 + BM + BKE - 1) / BKE);
    } else if (p.causal == CAUSAL_K_SUFFIX) {
        c.kb0 = max(c.kb0, c.m0 / BKE);
    }
    if (c.kb1 < c.kb0) c.kb1 = c.kb0;   // empty range: the accumulator is treated as zero
    return c;
}

// TF32 = true: float32 operands in shared memory, kind::tf32 (the tensor core reads the top 19 bits),
// K slices of 32 elements; everything else is shared with the bf16 path.
// EPI: the epilogue the instantiation is compiled for.  EPI_ANY keeps every mode behind run-time checks (one kernel
// for all of them: its epilogue loop then steps over the code of the modes it does not run, ~40 KB of instructions, and
// a 32-column chunk costs ~0.15 us more in instruction fetches); the other values fix the mode at compile time and
// drop the rest -- measured on an [8192 x 384 x 1152] launch: last tile's epilogue 2.42 -> 1.89 us (float32 out),
// 2.02 -> 1.54 us (bf16 out).
enum { EPI_ANY = 0, EPI_F32, EPI_BF16, EPI_SWIGLU, EPI_CE1, EPI_ROPE, EPI_CE2, EPI_DSW };

template <int BN, bool TF32, bool PAIR = false, int EPI = EPI_ANY>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const __grid_constant__ CUtensorMap tmR,
                 const GemmParams p) {
    static_assert(!(PAIR && TF32), "CTA pairs are built for bf16 operands only");
    using Cfg = GemmCfg<BN, PAIR>;
    constexpr int STAGES = Cfg::STAGES;
    constexpr int NBUF = Cfg::NBUF;
    constexpr int BNL = Cfg::BN_LOCAL;
    static_assert(BN != 384 || PAIR, "384-column tiles are built for CTA pairs");
    constexpr int TILE_M = PAIR ? 2 * BM : BM;
    // PAIR: rank in the CTA pair; rank 0 issues the UMMAs and owns the barriers the loads are counted on
    const uint32_t rank = PAIR ? cluster_ctarank() : 0u;
    const int row_off = (int)rank * BM;
    const int worker = PAIR ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int nworkers = PAIR ? (int)(gridDim.x >> 1) : (int)gridDim.x;
    constexpr int BKE = TF32 ? BK_TF32 : BK;           // elements per K slice
    constexpr int MNW = TF32 ? 32 : 64;                // elements per 128-byte row of an MN-major box
    constexpr int MN_BOX_BYTES = BKE * ROW_BYTES;      // one MN-major box: BKE rows of 128 bytes
    constexpr int MN_STEP = (TF32 ? 8 : 16) * ROW_BYTES;   // rows consumed by one UMMA (K = 8 or 16)

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    uint8_t* smem = smem_raw + ((1024u - (raw_addr & 1023u)) & 1023u);

    uint8_t* stage_base = smem;
    float* staging = reinterpret_cast<float*>(smem + STAGES * Cfg::STAGE_BYTES);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + STAGES * Cfg::STAGE_BYTES + Cfg::STAGING_BYTES);
    uint64_t* full_bar = bars;                    // [STAGES]
    uint64_t* empty_bar = bars + STAGES;          // [STAGES]
    uint64_t* acc_full = bars + 2 * STAGES;       // [2]
    uint64_t* acc_empty = bars + 2 * STAGES + 2;  // [2]
    uint64_t* res_bar = bars + 2 * STAGES + 4;    // [EPI_WARPS]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * STAGES + 4 + EPI_WARPS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int total_tiles = p.batch * p.splits * p.mt * p.nt;
    // the epilogue mode: constants in a specialised instantiation, the launch's parameters in the general one
    constexpr bool ANY = EPI == EPI_ANY;
    const bool m_generic = ANY && p.tma_mode == 0;                       // predicated stores, any alignment
    const bool m_f32 = ANY ? p.tma_mode == 1 : EPI == EPI_F32;           // float32 tiles by TMA
    const bool m_swiglu = ANY ? p.tma_mode == 3 : EPI == EPI_SWIGLU;
    const bool m_ce1 = ANY ? p.tma_mode == 4 : EPI == EPI_CE1;
    const bool m_rope = ANY ? p.tma_mode == 5 : EPI == EPI_ROPE;
    const bool m_ce2 = ANY ? p.ce_mode == 2 : EPI == EPI_CE2;
    const bool m_dsw = ANY ? p.dsw != 0 : EPI == EPI_DSW;
    const bool m_res = (ANY || EPI == EPI_F32) && p.tma_res != 0;        // a residual / previous-C tile only with float32 tiles
    const bool m_bias = (ANY || EPI == EPI_F32 || EPI == EPI_BF16 || EPI == EPI_ROPE) && p.bias != nullptr;
    const bool m_wide = (ANY || EPI == EPI_BF16 || EPI == EPI_ROPE || EPI == EPI_CE2) ? p.wide16 != 0 : EPI == EPI_DSW;
    if (threadIdx.x == 0) TS(0);

    // Prologue: nothing here reads or writes memory an earlier kernel of the stream produces, so it
    // may overlap that kernel's tail (programmatic dependent launch); pdl_wait() below is the fence.
    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmA);
        tma_prefetch_desc(&tmB);
        if (!m_generic && !m_ce1) tma_prefetch_desc(&tmC);
        for (int i = 0; i < STAGES; ++i) { mbar_init(&full_bar[i], 1); mbar_init(&empty_bar[i], 1); }
        for (int i = 0; i < 2; ++i) { mbar_init(&acc_full[i], 1); mbar_init(&acc_empty[i], PAIR ? 2 * EPI_WARPS : EPI_WARPS); }
        for (int i = 0; i < EPI_WARPS; ++i) mbar_init(&res_bar[i], 1);
        *abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        if (PAIR) { tmem_alloc_pair(tmem_slot, Cfg::TMEM_COLS); tmem_relinquish_pair(); }
        else      { tmem_alloc(tmem_slot, Cfg::TMEM_COLS); tmem_relinquish(); }
    }
    // every role's first tile, worked out while the barriers and the tensor memory are being set up
    const TileCoord c_first = tile_of<BN, BKE, TILE_M>(p, worker < total_tiles ? worker : 0, row_off);
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync();          // both CTAs' barriers exist before either signals the other's
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) TS(1);
    pdl_wait();

    if (warp == 0) {
        // ------------------------------------------------------------ TMA producer
        if (lane == 0) {
            int stage = 0; uint32_t phase = 0;
            bool ok = true;
            for (int t = worker; t < total_tiles && ok; t += nworkers) {
                const TileCoord c = t == worker ? c_first : tile_of<BN, BKE, TILE_M>(p, t, row_off);
                if (c.skip) continue;
                for (int kb = c.kb0; kb < c.kb1; ++kb) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) { ok = false; break; }
                    uint8_t* sA = stage_base + stage * Cfg::STAGE_BYTES;
                    uint8_t* sB = sA + Cfg::A_BYTES;
                    // PAIR: both CTAs' bytes are counted on rank 0's barrier, which alone arms it
                    if (!PAIR) mbar_expect_tx(&full_bar[stage], Cfg::STAGE_BYTES);
                    else if (rank == 0) mbar_expect_tx(&full_bar[stage], 2 * Cfg::STAGE_BYTES);
                    auto load = [&](void* dst, const CUtensorMap* map, int x, int y, int z) {
                        if (PAIR) tma_load_3d_pair(dst, map, &full_bar[stage], x, y, z);
                        else tma_load_3d(dst, map, &full_bar[stage], x, y, z);
                    };
                    if (!p.a_mn) {
                        load(sA, &tmA, kb * BKE, c.m0, c.z);
                    } else {
#pragma unroll
                        for (int j = 0; j < BM / MNW; ++j) load(sA + j * MN_BOX_BYTES, &tmA, c.m0 + j * MNW, kb * BKE, c.z);
                    }
                    const int nb0 = c.n0 + (int)rank * BNL;          // first B column this CTA loads
                    if (!p.b_mn) {
                        load(sB, &tmB, kb * BKE, nb0, c.z);
                    } else {
#pragma unroll
                        for (int j = 0; j < BNL / MNW; ++j) {
                            int n = BN == 384 ? c.n0 + 128 * j + 64 * (int)rank : nb0 + j * MNW;
                            if (m_swiglu) {            // paired tile: first half gate columns, second half their up columns
                                const int jj = (int)rank * (BNL / MNW) + j;      // box index inside the whole tile
                                n = (c.n0 >> 1) + (jj < BN / MNW / 2 ? jj * MNW : p.pair_off + (jj - BN / MNW / 2) * MNW);
                            }
                            load(sB + j * MN_BOX_BYTES, &tmB, n, kb * BKE, c.z);
                        }
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                    if (t == worker && kb == c.kb0) TS(2);
                }
            }
            TS(3);
            if (PAIR && ok) {
                // every release of a stage must have arrived (from rank 0's commits) before this CTA may exit
                for (int i = 0; i < STAGES && ok; ++i) {
                    if (!mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag)) ok = false;
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            pdl_launch_dependents_now();     // all loads issued: the next kernel may start its prologue
            if (!ok) { *abort_flag = 1; atomicExch(p.err, 1); }
        }
    } else if (warp == 1) {
        // -------------------------------------------------------------- MMA issuer (PAIR: rank 0 for both CTAs)
        if (lane == 0 && rank == 0) {
            constexpr int UMMA_N = BN == 384 ? 128 : BN;       // columns per tensor-core instruction
            constexpr int NSUB = BN / UMMA_N;
            const uint32_t idesc = umma_idesc(TF32 ? 2u : 1u, (uint32_t)p.a_mn, (uint32_t)p.b_mn, TILE_M, UMMA_N);
            // (BN = 384: instruction j takes the j-th 64-column box of B in either CTA and accumulator columns 128 j ..)
            constexpr uint64_t B_SUB_STEP = (uint64_t)(MN_BOX_BYTES >> 4);
            // Shared-memory descriptors are built once: the descriptor of stage 0, the step between stages
            // and the step between the four UMMAs of a K slice are all that changes (the start address sits
            // in the low 14 bits, in 16-byte units, and never carries out of them below 256 KB).  One thread
            // issues every UMMA of the CTA, so its instruction count per UMMA bounds the tensor pipe.
            const uint32_t a_addr0 = smem_u32(stage_base);
            const uint32_t b_addr0 = a_addr0 + Cfg::A_BYTES;
            const uint64_t a_desc0 = !p.a_mn ? umma_desc_sw128(a_addr0, 16, 1024)
                                     : TF32  ? umma_desc_mn32(a_addr0, MN_BOX_BYTES)
                                             : umma_desc_sw128(a_addr0, MN_BOX_BYTES, 1024);
            const uint64_t b_desc0 = !p.b_mn ? umma_desc_sw128(b_addr0, 16, 1024)
                                     : TF32  ? umma_desc_mn32(b_addr0, MN_BOX_BYTES)
                                             : umma_desc_sw128(b_addr0, MN_BOX_BYTES, 1024);
            const uint64_t a_kstep = (uint64_t)((!p.a_mn ? 32 : MN_STEP) >> 4);
            const uint64_t b_kstep = (uint64_t)((!p.b_mn ? 32 : MN_STEP) >> 4);
            constexpr uint64_t STAGE_STEP = (uint64_t)(Cfg::STAGE_BYTES >> 4);
            uint64_t a_desc = a_desc0, b_desc = b_desc0;
            int stage = 0; uint32_t phase = 0;
            int it = 0;
            bool ok = true;
            for (int t = worker; t < total_tiles && ok; t += nworkers) {
                const TileCoord c = t == worker ? c_first : tile_of<BN, BKE, TILE_M>(p, t, row_off);
                if (c.skip) continue;
                const int buf = it % NBUF;
                const uint32_t acc_phase = (uint32_t)(it / NBUF) & 1u;
                if (!mbar_wait(&acc_empty[buf], acc_phase ^ 1u, abort_flag)) { ok = false; break; }
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(buf * BN);
                for (int kb = c.kb0; kb < c.kb1; ++kb) {
                    if (!mbar_wait(&full_bar[stage], phase, abort_flag)) { ok = false; break; }
                    if (it == 0 && kb == c.kb0) TS(4);
                    tc_fence_after();
#pragma unroll
                    for (int k = 0; k < 4; ++k) {          // 4 UMMAs of 32 bytes of K per 128-byte slice
                        if (TF32)      umma_tf32(d_tmem, a_desc + k * a_kstep, b_desc + k * b_kstep, idesc, (kb > c.kb0 || k > 0) ? 1u : 0u);
                        else if (PAIR) {
#pragma unroll
                            for (int j = 0; j < NSUB; ++j)
                                umma_bf16_pair(d_tmem + (uint32_t)(j * UMMA_N), a_desc + k * a_kstep, b_desc + k * b_kstep + j * B_SUB_STEP,
                                               idesc, (kb > c.kb0 || k > 0) ? 1u : 0u);
                        }
                        else           umma_bf16(d_tmem, a_desc + k * a_kstep, b_desc + k * b_kstep, idesc, (kb > c.kb0 || k > 0) ? 1u : 0u);
                    }
                    if (PAIR) umma_commit_pair(&empty_bar[stage]);   // stage reusable (in both CTAs) once these MMAs have read it
                    else      umma_commit(&empty_bar[stage]);
                    a_desc += STAGE_STEP; b_desc += STAGE_STEP;
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; a_desc = a_desc0; b_desc = b_desc0; }
                }
                if (!ok) break;
                if (PAIR) umma_commit_pair(&acc_full[buf]);      // accumulator complete (each CTA reads its own 128 rows)
                else      umma_commit(&acc_full[buf]);
                if (it == 0) TS(5);
                ++it;
            }
            TS(6);
            if (!ok) { *abort_flag = 1; atomicExch(p.err, 2); }
        }
    } else if (!m_generic) {
        // ------------------------------------------------ epilogue, tile stores by TMA
        // Per 32-column chunk: tcgen05.ld -> registers (+bias, +scaled residual tile) -> this warp's
        // 32 x 128 B staging buffer in the 128B-swizzle pattern -> one TMA store (clipped at the
        // matrix edge by the hardware).  Two buffers per warp: the store of chunk i drains while
        // chunk i+1 is produced; the residual tile of chunk i+1 is fetched by TMA meanwhile.
        const int q = warp & 3;                  // TMEM lane quarter this warp may read
        const int ew = warp - 2;                 // 0..7; warps ew and ew+4 share a quarter
        const int half = ew >> 2;                // which half of the tile's column chunks
        uint8_t* obuf = reinterpret_cast<uint8_t*>(staging) + ew * Cfg::EPI_WARP_BYTES;
        uint8_t* rbuf = obuf + 8192;
        uint64_t* rbar = res_bar + ew;
        constexpr int NCH = BN / 64;             // chunks of 32 columns per warp and tile
        uint32_t cnt = 0;                        // chunks produced so far (selects the output buffer)
        uint32_t rphase = 0;
        int it = 0;
        bool ok = true;
        for (int t = worker; t < total_tiles && ok; t += nworkers) {
            const TileCoord c = t == worker ? c_first : tile_of<BN, BKE, TILE_M>(p, t, row_off);
            if (c.skip) continue;
            const int buf = it % NBUF;
            const uint32_t acc_phase = (uint32_t)(it / NBUF) & 1u;
            const bool have_acc = c.kb1 > c.kb0;
            const int zc = c.z * p.splits + c.s;
            const int zo = zc / p.c_inner, zi = zc % p.c_inner;
            const int gm0 = c.m0 + q * 32;
            const bool rows_in = gm0 < p.M;
            if (m_ce1) {
                // Cross-entropy pass 1: running max and sum of exponentials of this warp's 32 rows over its
                // half of the tile's columns (online update per 32-column chunk); nothing leaves but the pair
                if (!mbar_wait(&acc_full[buf], acc_phase, abort_flag)) { ok = false; break; }
                tc_fence_after();
                constexpr float LOG2E = 1.4426950408889634f;
                const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN + half * (BN / 2));
                const int row = gm0 + lane;
                const int tgt = row < p.M ? (int)__ldg(p.ce_targets + row) : -1;
                float m_run = -INFINITY, s_run = 0.0f, zt = 0.0f;
                bool has_t = false;
#pragma unroll 1
                for (int ch = 0; ch < NCH; ++ch) {
                    const int gn0 = c.n0 + half * (BN / 2) + ch * 32;
                    if (gn0 >= p.N) break;
                    uint32_t v[32];
                    tmem_ld32(t_row + (uint32_t)(ch * 32), v);
                    tmem_ld_wait();
                    float cm = -INFINITY;
                    const bool full = gn0 + 32 <= p.N;
                    if (full) {
                        // four independent chains instead of one of 32 dependent maxima
                        float c0 = __uint_as_float(v[0]), c1 = __uint_as_float(v[1]), c2 = __uint_as_float(v[2]), c3 = __uint_as_float(v[3]);
#pragma unroll
                        for (int j = 4; j < 32; j += 4) {
                            c0 = fmaxf(c0, __uint_as_float(v[j]));     c1 = fmaxf(c1, __uint_as_float(v[j + 1]));
                            c2 = fmaxf(c2, __uint_as_float(v[j + 2])); c3 = fmaxf(c3, __uint_as_float(v[j + 3]));
                        }
                        cm = fmaxf(fmaxf(c0, c1), fmaxf(c2, c3));
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) cm = fmaxf(cm, gn0 + j < p.N ? __uint_as_float(v[j]) : -INFINITY);
                    }
                    if (tgt >= gn0 && tgt < gn0 + 32) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) if (gn0 + j == tgt) zt = __uint_as_float(v[j]);
                        has_t = true;
                    }
                    const float m_new = fmaxf(m_run, cm);
                    const float mb = m_new * LOG2E;
                    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
                    if (full) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            s0 += ex2_approx(__uint_as_float(v[j])     * LOG2E - mb);
                            s1 += ex2_approx(__uint_as_float(v[j + 1]) * LOG2E - mb);
                            s2 += ex2_approx(__uint_as_float(v[j + 2]) * LOG2E - mb);
                            s3 += ex2_approx(__uint_as_float(v[j + 3]) * LOG2E - mb);
                        }
                    } else
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        s0 += gn0 + j     < p.N ? ex2_approx(__uint_as_float(v[j])     * LOG2E - mb) : 0.0f;
                        s1 += gn0 + j + 1 < p.N ? ex2_approx(__uint_as_float(v[j + 1]) * LOG2E - mb) : 0.0f;
                        s2 += gn0 + j + 2 < p.N ? ex2_approx(__uint_as_float(v[j + 2]) * LOG2E - mb) : 0.0f;
                        s3 += gn0 + j + 3 < p.N ? ex2_approx(__uint_as_float(v[j + 3]) * LOG2E - mb) : 0.0f;
                    }
                    s_run = s_run * ex2_approx((m_run - m_new) * LOG2E) + ((s0 + s1) + (s2 + s3));
                    m_run = m_new;
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) { if (PAIR) mbar_arrive_leader(&acc_empty[buf]); else mbar_arrive(&acc_empty[buf]); }
                if (row < p.M) {
                    float2* dst = reinterpret_cast<float2*>(p.ce_stats) + ((size_t)((c.n0 / BN) * 2 + half) * p.M + row);
                    *dst = make_float2(m_run, s_run);           // (-inf, 0) for a half with no column inside N
                    if (has_t) p.ce_ztarget[row] = zt;
                }
                ++it;
                continue;
            }
            if (m_swiglu) {
                // SwiGLU: this warp owns 32 rows x BN/4 hidden units: gate in accumulator columns half*BN/4..,
                // up in columns BN/2 + half*BN/4..; h = silu(g) * u leaves as bf16, g and u (bf16) on request
                if (!mbar_wait(&acc_full[buf], acc_phase, abort_flag)) { ok = false; break; }
                tc_fence_after();
#pragma unroll 1
                for (int ch = 0; ch < BN / 128; ++ch) {
                    const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) +
                                           (uint32_t)(buf * BN + half * (BN / 4) + ch * 32);
                    uint32_t gr[32], ur[32];
                    tmem_ld32(t_row, gr);
                    tmem_ld32(t_row + (uint32_t)(BN / 2), ur);
                    tmem_ld_wait();
                    if (ch == BN / 128 - 1) {
                        tc_fence_before();
                        __syncwarp();
                        if (lane == 0) { if (PAIR) mbar_arrive_leader(&acc_empty[buf]); else mbar_arrive(&acc_empty[buf]); }
                    }
                    const int hj0 = (c.n0 >> 1) + half * (BN / 4) + ch * 32;     // first hidden unit of this chunk
                    float gv[32], uv[32], hv[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) { gv[j] = __uint_as_float(gr[j]); uv[j] = __uint_as_float(ur[j]); }
                    if (p.bias) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            gv[j] += __ldg(p.bias + hj0 + j);
                            uv[j] += __ldg(p.bias + p.pair_off + hj0 + j);
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        // sigmoid from ex2.approx and an approximate reciprocal (relative error ~1e-6, far below bf16's)
                        const float sg = __fdividef(1.0f, 1.0f + ex2_approx(-gv[j] * 1.4426950408889634f));
                        hv[j] = gv[j] * sg * uv[j];
                    }
                    // wide16 (256-column tiles: two chunks per warp): both chunks fill one set of buffers with rows of
                    // 128 bytes and leave together through 64-column maps
                    const bool second = p.wide16 && ch == 1;
                    if (lane == 0 && !second) tma_store_wait_read<0>(); // the previous stores have left the buffers
                    __syncwarp();
                    auto stage_bf16 = [&](uint8_t* base, const float (&o)[32]) {
                        uint8_t* orow = base + lane * (p.wide16 ? 128 : 64);     // 32 x 64 B, 64B swizzle (wide: 128 B, 128B)
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            uint4 pk;
                            __nv_bfloat162 h0 = __floats2bfloat162_rn(o[8 * j + 0], o[8 * j + 1]);
                            __nv_bfloat162 h1 = __floats2bfloat162_rn(o[8 * j + 2], o[8 * j + 3]);
                            __nv_bfloat162 h2 = __floats2bfloat162_rn(o[8 * j + 4], o[8 * j + 5]);
                            __nv_bfloat162 h3 = __floats2bfloat162_rn(o[8 * j + 6], o[8 * j + 7]);
                            pk.x = *reinterpret_cast<uint32_t*>(&h0); pk.y = *reinterpret_cast<uint32_t*>(&h1);
                            pk.z = *reinterpret_cast<uint32_t*>(&h2); pk.w = *reinterpret_cast<uint32_t*>(&h3);
                            const int so = p.wide16 ? (((second ? 4 : 0) + j) ^ (lane & 7)) << 4 : (j ^ ((lane >> 1) & 3)) << 4;
                            *reinterpret_cast<uint4*>(orow + so) = pk;
                        }
                    };
                    stage_bf16(obuf, hv);
                    if (p.keep_gu) { stage_bf16(obuf + 4096, gv); stage_bf16(rbuf, uv); }
                    if (p.wide16 && !second) continue;
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0) {
                        if (rows_in) {
                            const int hs = p.wide16 ? hj0 - 32 : hj0;
                            tma_store_4d(&tmC, obuf, hs, gm0, 0, 0);
                            if (p.keep_gu) {
                                tma_store_4d(&tmR, obuf + 4096, hs, gm0, 0, 0);
                                tma_store_4d(&tmR, rbuf, p.pair_off + hs, gm0, 0, 0);
                            }
                        }
                        tma_store_commit();
                    }
                }
                ++it;
                continue;
            }
            const int col0 = c.n0 + half * (BN / 2);
            // mode 5: position of this thread's row, and of the 32-row chunk, inside its sequence (once per tile)
            const int rope_D = p.rope_H * p.rope_hd, rope_shift = p.rope_hd == 64 ? 6 : 5;
            int rope_b = 0, rope_t0 = 0, rope_t = 0;
            if (m_rope) { rope_b = gm0 / p.rope_T; rope_t0 = gm0 - rope_b * p.rope_T; rope_t = rope_t0 + lane; }
            if (m_res && lane == 0 && rows_in && col0 < p.N) {
                mbar_expect_tx(rbar, 4096);
                tma_load_4d(rbuf, &tmR, rbar, col0, gm0, 0, c.z);
            }
            // SwiGLU backward: g and u of chunk ch + 1 are fetched while chunk ch is computed
            auto dsw_fetch = [&](int ch) {
                mbar_expect_tx(rbar, 4096);
                tma_load_4d(rbuf, &tmR, rbar, col0 + ch * 32, gm0, 0, 0);
                tma_load_4d(rbuf + 2048, &tmR, rbar, p.pair_off + col0 + ch * 32, gm0, 0, 0);
            };
            if (m_dsw && lane == 0 && rows_in && col0 < p.N) dsw_fetch(0);
            if (!mbar_wait(&acc_full[buf], acc_phase, abort_flag)) { ok = false; break; }
            if (warp == 2 && lane == 0 && it == 0) TS(7);
            tc_fence_after();
            const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN + half * (BN / 2));
#pragma unroll 1
            for (int ch = 0; ch < NCH; ++ch) {
                // a store unit is one chunk, or in wide16 mode a pair of chunks (an odd last chunk stays alone);
                // with dsw a unit fills both output buffers (dg | du), else the units alternate between them
                const bool paired = m_wide && ((ch & 1) || ch + 1 < NCH);
                const bool second = paired && (ch & 1);
                const uint32_t b = m_dsw ? 0u : (cnt & 1u);
                const int gn0 = col0 + ch * 32;
                const bool active = rows_in && gn0 < p.N;
                if (lane == 0 && !second) {                   // the unit's output buffer has been read out
                    if (m_dsw) tma_store_wait_read<0>(); else tma_store_wait_read<1>();
                }
                __syncwarp();
                uint32_t v[32];
                if (have_acc) {
                    tmem_ld32(t_row + (uint32_t)(ch * 32), v);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = 0u;
                }
                float o[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) o[j] = __uint_as_float(v[j]) * p.alpha;
                if (m_bias) {
                    if (p.bias_vec && gn0 + 32 <= p.N) {
                        const float4* b4 = reinterpret_cast<const float4*>(p.bias + gn0);
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float4 bb = __ldg(b4 + j);
                            o[4 * j] += bb.x; o[4 * j + 1] += bb.y; o[4 * j + 2] += bb.z; o[4 * j + 3] += bb.w;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) if (gn0 + j < p.N) o[j] += __ldg(p.bias + gn0 + j);
                    }
                }
                if (m_res && active) {
                    if (!mbar_wait(rbar, rphase, abort_flag)) { ok = false; break; }
                    rphase ^= 1u;
                    const uint8_t* rrow = rbuf + lane * 128;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const float4 r4 = *reinterpret_cast<const float4*>(rrow + ((j ^ (lane & 7)) << 4));
                        o[4 * j] += p.res_scale * r4.x; o[4 * j + 1] += p.res_scale * r4.y;
                        o[4 * j + 2] += p.res_scale * r4.z; o[4 * j + 3] += p.res_scale * r4.w;
                    }
                    // the residual buffer is free again: fetch the next chunk's tile into it
                    fence_proxy_async();
                    __syncwarp();
                    if (lane == 0 && ch + 1 < NCH && gn0 + 32 < p.N) {
                        mbar_expect_tx(rbar, 4096);
                        tma_load_4d(rbuf, &tmR, rbar, gn0 + 32, gm0, 0, c.z);
                    }
                }
                if (m_rope) {
                    // position embedding on the q and k columns: pairs (2k, 2k+1) of a head rotate by the
                    // angle of (position, k); this chunk is 32 consecutive head-dim values of one head
                    if (gn0 < 2 * rope_D) {
                        const int d0 = (gn0 - (gn0 >= rope_D ? rope_D : 0)) & (p.rope_hd - 1);
                        const long long off = (long long)rope_t * (p.rope_hd >> 1) + (d0 >> 1);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float4 c4 = __ldg(reinterpret_cast<const float4*>(p.rope_cos + off) + j);
                            const float4 s4 = __ldg(reinterpret_cast<const float4*>(p.rope_sin + off) + j);
                            const float cc[4] = {c4.x, c4.y, c4.z, c4.w}, ss[4] = {s4.x, s4.y, s4.z, s4.w};
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float a0 = o[8 * j + 2 * i], b0 = o[8 * j + 2 * i + 1];
                                o[8 * j + 2 * i] = a0 * cc[i] - b0 * ss[i];
                                o[8 * j + 2 * i + 1] = a0 * ss[i] + b0 * cc[i];
                            }
                        }
                    }
                }
                if (m_ce2) {
                    // cross-entropy pass 2: the logits turn into their gradient before they are stored
                    constexpr float LOG2E = 1.4426950408889634f;
                    const int row = gm0 + lane;
                    const float lb = row < p.M ? __ldg(p.ce_lse + row) * LOG2E : 0.0f;
                    const int tgt = row < p.M ? (int)__ldg(p.ce_targets + row) : -1;
                    if (gn0 + 32 <= p.N && (tgt < gn0 || tgt >= gn0 + 32)) {
                        // a whole chunk without the row's target column (all but one chunk of a row, and the ragged last)
#pragma unroll
                        for (int j = 0; j < 32; ++j) o[j] = ex2_approx(o[j] * LOG2E - lb) * p.ce_scale;
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j) {
                            float pr = gn0 + j < p.N ? ex2_approx(o[j] * LOG2E - lb) : 0.0f;
                            if (gn0 + j == tgt) pr -= 1.0f;
                            o[j] = pr * p.ce_scale;
                        }
                    }
                }
                if (m_dsw) {
                    // SwiGLU backward (the reference's k_swiglu_bwd on the product's tile, cuda/train_kernels.cu:709-721):
                    // o = dh (zero in rows past M, whose operand rows the tile loads fill with zeros); with the saved
                    // g, u of the same rows and hidden units, a = g s, s = sigmoid(g):
                    //   dg = dh u (s + a - a s),  du = dh a
                    // leave as bf16 boxes of dgu at columns gn0 and F + gn0
                    if (active) {
                        if (!mbar_wait(rbar, rphase, abort_flag)) { ok = false; break; }
                        rphase ^= 1u;
                        constexpr float NLOG2E = -1.4426950408889634f;
                        const uint8_t* grow = rbuf + lane * 64;
                        // paired: dg rows of 128 bytes in obuf, du rows in obuf + 4096; alone: 64-byte rows, du at + 2048
                        uint8_t* orow = obuf + lane * (paired ? 128 : 64);
                        const int uoff = paired ? 4096 : 2048;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int sw = (j ^ ((lane >> 1) & 3)) << 4;
                            const int so = paired ? (((second ? 4 : 0) + j) ^ (lane & 7)) << 4 : sw;
                            const uint4 g4 = *reinterpret_cast<const uint4*>(grow + sw);
                            const uint4 u4 = *reinterpret_cast<const uint4*>(grow + 2048 + sw);
                            const uint32_t gw[4] = {g4.x, g4.y, g4.z, g4.w}, uw[4] = {u4.x, u4.y, u4.z, u4.w};
                            uint32_t pg[4], pu[4];
#pragma unroll
                            for (int e = 0; e < 4; ++e) {
                                const float2 gg = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&gw[e]));
                                const float2 uu = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&uw[e]));
                                const float d0 = o[8 * j + 2 * e], d1 = o[8 * j + 2 * e + 1];
                                const float s0 = __fdividef(1.0f, 1.0f + ex2_approx(gg.x * NLOG2E));
                                const float s1 = __fdividef(1.0f, 1.0f + ex2_approx(gg.y * NLOG2E));
                                const float a0 = gg.x * s0, a1 = gg.y * s1;
                                const float q0 = fmaf(-a0, s0, a0) + s0, q1 = fmaf(-a1, s1, a1) + s1;
                                __nv_bfloat162 hg = __floats2bfloat162_rn(d0 * uu.x * q0, d1 * uu.y * q1);
                                __nv_bfloat162 hu = __floats2bfloat162_rn(d0 * a0, d1 * a1);
                                pg[e] = *reinterpret_cast<uint32_t*>(&hg); pu[e] = *reinterpret_cast<uint32_t*>(&hu);
                            }
                            *reinterpret_cast<uint4*>(orow + so) = make_uint4(pg[0], pg[1], pg[2], pg[3]);
                            *reinterpret_cast<uint4*>(orow + uoff + so) = make_uint4(pu[0], pu[1], pu[2], pu[3]);
                        }
                        // the g / u buffer is free again: fetch the next chunk's boxes into it
                        fence_proxy_async();
                        __syncwarp();
                        if (lane == 0 && ch + 1 < NCH && gn0 + 32 < p.N) dsw_fetch(ch + 1);
                    }
                } else if (m_f32) {
                    uint8_t* orow = obuf + b * 4096 + lane * 128;
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        *reinterpret_cast<float4*>(orow + ((j ^ (lane & 7)) << 4)) =
                            make_float4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
                } else {
                    uint8_t* orow = obuf + b * 4096 + lane * (paired ? 128 : 64);
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        uint4 pk;
                        __nv_bfloat162 h0 = __floats2bfloat162_rn(o[8 * j + 0], o[8 * j + 1]);
                        __nv_bfloat162 h1 = __floats2bfloat162_rn(o[8 * j + 2], o[8 * j + 3]);
                        __nv_bfloat162 h2 = __floats2bfloat162_rn(o[8 * j + 4], o[8 * j + 5]);
                        __nv_bfloat162 h3 = __floats2bfloat162_rn(o[8 * j + 6], o[8 * j + 7]);
                        pk.x = *reinterpret_cast<uint32_t*>(&h0); pk.y = *reinterpret_cast<uint32_t*>(&h1);
                        pk.z = *reinterpret_cast<uint32_t*>(&h2); pk.w = *reinterpret_cast<uint32_t*>(&h3);
                        const int so = paired ? (((second ? 4 : 0) + j) ^ (lane & 7)) << 4 : (j ^ ((lane >> 1) & 3)) << 4;
                        *reinterpret_cast<uint4*>(orow + so) = pk;
                    }
                }
                if (paired && !second) continue;              // the unit leaves after its second chunk
                fence_proxy_async();
                __syncwarp();
                if (lane == 0 && paired) {
                    // rows of 128 bytes: columns gn0 - 32 .. gn0 + 31 (what lies past N is clipped by the hardware)
                    if (rows_in && gn0 - 32 < p.N) {
                        if (m_rope) {                         // the pair is one head's 64 values of 32 positions
                            const int g0 = gn0 - 32;
                            const int which = g0 >= 2 * rope_D ? 2 : (g0 >= rope_D ? 1 : 0);
                            tma_store_5d(&tmC, obuf + b * 4096, 0, rope_t0, (g0 - which * rope_D) >> 6, rope_b, which);
                        } else if (m_dsw) {
                            tma_store_4d(&tmC, obuf, gn0 - 32, gm0, 0, 0);
                            tma_store_4d(&tmC, obuf + 4096, p.pair_off + gn0 - 32, gm0, 0, 0);
                        } else {
                            tma_store_4d(&tmR, obuf + b * 4096, gn0 - 32, gm0, zi, zo);
                        }
                    }
                    tma_store_commit();
                } else if (lane == 0) {
                    if (active && m_rope) {
                        const int which = gn0 >= 2 * rope_D ? 2 : (gn0 >= rope_D ? 1 : 0);
                        const int cin = gn0 - which * rope_D;
                        tma_store_5d(&tmC, obuf + b * 4096, cin & (p.rope_hd - 1), rope_t0, cin >> rope_shift, rope_b, which);
                    } else if (active && m_dsw) {
                        tma_store_4d(&tmC, obuf + b * 4096, gn0, gm0, 0, 0);
                        tma_store_4d(&tmC, obuf + b * 4096 + 2048, p.pair_off + gn0, gm0, 0, 0);
                    } else if (active) {
                        tma_store_4d(&tmC, obuf + b * 4096, gn0, gm0, zi, zo);
                    }
                    tma_store_commit();
                }
                ++cnt;
            }
            if (!ok) break;
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { if (PAIR) mbar_arrive_leader(&acc_empty[buf]); else mbar_arrive(&acc_empty[buf]); }
            if (warp == 2 && lane == 0) { if (it == 0) TS(8); TS(9); }
            ++it;
        }
        if (lane == 0) tma_store_wait_read<0>();
        if (warp == 2 && lane == 0) TS(10);
        if (!ok && lane == 0) { *abort_flag = 1; atomicExch(p.err, 3); }
    } else {
        // ------------------------------------------- epilogue, generic (any alignment)
        const int q = warp & 3;                        // TMEM lane quarter this warp may read
        const int half = (warp - 2) >> 2;              // warps w and w+4 share a quarter: even / odd chunks
        float* stg = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(staging) + (warp - 2) * Cfg::EPI_WARP_BYTES);
        const int r_sub = lane >> 3;                   // 0..3
        const int cg = lane & 7;                       // 0..7 -> columns 4*cg..4*cg+3
        int it = 0;
        bool ok = true;
        for (int t = worker; t < total_tiles && ok; t += nworkers) {
            const TileCoord c = t == worker ? c_first : tile_of<BN, BKE, TILE_M>(p, t, row_off);
            if (c.skip) continue;
            const int buf = it % NBUF;
            const uint32_t acc_phase = (uint32_t)(it / NBUF) & 1u;
            const bool have_acc = c.kb1 > c.kb0;
            if (!mbar_wait(&acc_full[buf], acc_phase, abort_flag)) { ok = false; break; }
            tc_fence_after();
            const long long zc = (long long)c.z * p.splits + c.s;
            const long long zo = zc / p.c_inner, zi = zc % p.c_inner;
            float* C32 = p.C32 ? p.C32 + zo * p.strideC32 + zi * p.strideC32_in : nullptr;
            bf16* C16 = p.C16 ? p.C16 + zo * p.strideC16 + zi * p.strideC16_in : nullptr;
            const float* R = p.residual ? p.residual + (long long)c.z * p.strideR : nullptr;
            const uint32_t t_row = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(buf * BN);

#pragma unroll 1
            for (int ch = half; ch < BN / 32; ch += 2) {
                uint32_t v[32];
                if (have_acc) {
                    tmem_ld32(t_row + (uint32_t)(ch * 32), v);
                    tmem_ld_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = 0u;
                }
                float* srow = stg + lane * STAGE_LD;
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    float4 f;
                    f.x = __uint_as_float(v[4 * j + 0]); f.y = __uint_as_float(v[4 * j + 1]);
                    f.z = __uint_as_float(v[4 * j + 2]); f.w = __uint_as_float(v[4 * j + 3]);
                    *reinterpret_cast<float4*>(srow + 4 * j) = f;
                }
                __syncwarp();
                const int gn = c.n0 + ch * 32 + 4 * cg;
                float bias4[4] = {0.f, 0.f, 0.f, 0.f};
                if (p.bias) {
#pragma unroll
                    for (int e = 0; e < 4; ++e) if (gn + e < p.N) bias4[e] = p.bias[gn + e];
                }
#pragma unroll 2
                for (int itr = 0; itr < 8; ++itr) {
                    const int row = itr * 4 + r_sub;
                    const int gm = c.m0 + q * 32 + row;
                    if (gm >= p.M || gn >= p.N) continue;
                    const float4 x = *reinterpret_cast<const float4*>(stg + row * STAGE_LD + 4 * cg);
                    float o[4] = {x.x * p.alpha + bias4[0], x.y * p.alpha + bias4[1],
                                  x.z * p.alpha + bias4[2], x.w * p.alpha + bias4[3]};
                    const bool full4 = gn + 3 < p.N;
                    if (R) {
                        const float* rp = R + (long long)gm * p.ldr + gn;
                        if (full4 && p.vecr) {
                            const float4 r4 = *reinterpret_cast<const float4*>(rp);
                            o[0] += r4.x; o[1] += r4.y; o[2] += r4.z; o[3] += r4.w;
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e) if (gn + e < p.N) o[e] += rp[e];
                        }
                    }
                    if (C32) {
                        float* cp = C32 + (long long)gm * p.ldc32 + gn;
                        if (full4 && p.vec32) {
                            if (p.beta != 0.0f) {
                                const float4 c4 = *reinterpret_cast<const float4*>(cp);
                                o[0] += p.beta * c4.x; o[1] += p.beta * c4.y; o[2] += p.beta * c4.z; o[3] += p.beta * c4.w;
                            }
                            *reinterpret_cast<float4*>(cp) = make_float4(o[0], o[1], o[2], o[3]);
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e) if (gn + e < p.N) {
                                if (p.beta != 0.0f) o[e] += p.beta * cp[e];
                                cp[e] = o[e];
                            }
                        }
                    }
                    if (C16) {
                        bf16* hp = C16 + (long long)gm * p.ldc16 + gn;
                        if (full4 && p.vec16) {
                            __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]);
                            __nv_bfloat162 hi = __floats2bfloat162_rn(o[2], o[3]);
                            uint2 pk;
                            pk.x = *reinterpret_cast<uint32_t*>(&lo);
                            pk.y = *reinterpret_cast<uint32_t*>(&hi);
                            *reinterpret_cast<uint2*>(hp) = pk;
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; ++e) if (gn + e < p.N) hp[e] = __float2bfloat16_rn(o[e]);
                        }
                    }
                }
                __syncwarp();
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) { if (PAIR) mbar_arrive_leader(&acc_empty[buf]); else mbar_arrive(&acc_empty[buf]); }
            ++it;
        }
        if (!ok && lane == 0) { *abort_flag = 1; atomicExch(p.err, 3); }
    }

    // ---------------------------------------------------------------- teardown
    __syncwarp();
    if (*abort_flag) {
        // a bounded wait ran out: give copies in flight time to land before the CTA's
        // shared memory is released
        for (int i = 0; i < 64; ++i) __nanosleep(1000);
    }
    tc_fence_before();
    __syncthreads();
    if (PAIR) cluster_sync();          // the other CTA has read its accumulators and needs none of this CTA's barriers any more
    if (warp == 1) {
        tc_fence_after();
        if (PAIR) tmem_dealloc_pair(tmem_base, Cfg::TMEM_COLS);
        else tmem_dealloc(tmem_base, Cfg::TMEM_COLS);
    }
}

// Adds split-K partials in split order: out = sum_s part[s] (+ bias) (+ beta * out).  Loads of four
// splits are issued together; the additions stay in split order.
template <int VEC>
__global__ void reduce_splits_kernel(const float* __restrict__ part, float* __restrict__ out,
                                     bf16* __restrict__ out16, int M, int N, long long ldc32, long long ldc16,
                                     int splits, long long strideC32, long long strideC16, float beta,
                                     const float* __restrict__ bias) {
    pdl_wait();
    pdl_launch_dependents();
    const long long per = (long long)M * N;
    const int z = blockIdx.y;
    const long long nvec = per / VEC;
    for (long long iv = (long long)blockIdx.x * blockDim.x + threadIdx.x; iv < nvec;
         iv += (long long)gridDim.x * blockDim.x) {
        const long long i = iv * VEC;
        const int r = (int)(i / N), cidx = (int)(i % N);
        const float* src = part + ((long long)z * splits) * per + i;
        float s[VEC];
#pragma unroll
        for (int e = 0; e < VEC; ++e) s[e] = 0.0f;
        int k = 0;
        for (; k + 4 <= splits; k += 4) {
            float v[4][VEC];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                if (VEC == 4) {
                    const float4 t = *reinterpret_cast<const float4*>(src + (long long)(k + u) * per);
                    v[u][0] = t.x; v[u][1 % VEC] = t.y; v[u][2 % VEC] = t.z; v[u][3 % VEC] = t.w;
                } else {
                    v[u][0] = src[(long long)(k + u) * per];
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u)
#pragma unroll
                for (int e = 0; e < VEC; ++e) s[e] += v[u][e];
        }
        for (; k < splits; ++k) {
            if (VEC == 4) {
                const float4 t = *reinterpret_cast<const float4*>(src + (long long)k * per);
                s[0] += t.x; s[1 % VEC] += t.y; s[2 % VEC] += t.z; s[3 % VEC] += t.w;
            } else {
                s[0] += src[(long long)k * per];
            }
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            if (bias) s[e] += bias[cidx + e];
            if (out) {
                float* o = out + (long long)z * strideC32 + (long long)r * ldc32 + cidx + e;
                if (beta != 0.0f) s[e] += beta * *o;
                *o = s[e];
            }
            if (out16) out16[(long long)z * strideC16 + (long long)r * ldc16 + cidx + e] = __float2bfloat16_rn(s[e]);
        }
    }
}

// ===================================================================== host side

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_driver_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            return nullptr;
        fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

// Host-side cache of encoded tensor maps, keyed by everything that goes into one (address, extents, strides,
// box, types): a training loop or a caller of the eager entry points presents the same few dozen matrices
// again and again, and a map depends on nothing but those numbers, so a hit can never be stale.
// Direct-mapped, 1024 entries, one mutex; a miss costs the driver call it replaces.
struct MapKey {
    uint64_t v[20];
    bool operator==(const MapKey& o) const { return memcmp(v, o.v, sizeof(v)) == 0; }
};
struct MapEntry { MapKey key; CUtensorMap map; bool used; };
static MapEntry g_map_cache[1024];
static std::mutex g_map_mutex;

static CUresult encode_cached(CUtensorMap* map, CUtensorMapDataType dtype, cuuint32_t rank, void* ptr,
                              const cuuint64_t* dims, const cuuint64_t* strides, const cuuint32_t* box,
                              const cuuint32_t* estr, CUtensorMapInterleave il, CUtensorMapSwizzle sw,
                              CUtensorMapL2promotion l2, CUtensorMapFloatOOBfill oob) {
    EncodeTiledFn fn = get_driver_encode_fn();
    if (fn == nullptr) return CUDA_ERROR_NOT_SUPPORTED;
    if (rank > 5) return fn(map, dtype, rank, ptr, dims, strides, box, estr, il, sw, l2, oob);
    MapKey k;
    memset(&k, 0, sizeof(k));
    k.v[0] = reinterpret_cast<uint64_t>(ptr);
    k.v[1] = ((uint64_t)dtype << 40) | ((uint64_t)rank << 32) | ((uint64_t)il << 24) | ((uint64_t)sw << 16) |
             ((uint64_t)l2 << 8) | (uint64_t)oob;
    for (cuuint32_t i = 0; i < rank; ++i) {
        k.v[2 + i] = dims[i];
        k.v[12 + i] = ((uint64_t)box[i] << 32) | estr[i];
        if (i + 1 < rank) k.v[7 + i] = strides[i];
    }
    uint64_t h = 1469598103934665603ull;
    for (int i = 0; i < 20; ++i) { h ^= k.v[i]; h *= 1099511628211ull; }
    MapEntry& e = g_map_cache[(h ^ (h >> 29)) & 1023u];
    {
        std::lock_guard<std::mutex> lock(g_map_mutex);
        if (e.used && e.key == k) { *map = e.map; return CUDA_SUCCESS; }
    }
    const CUresult r = fn(map, dtype, rank, ptr, dims, strides, box, estr, il, sw, l2, oob);
    if (r == CUDA_SUCCESS) {
        std::lock_guard<std::mutex> lock(g_map_mutex);
        e.key = k; e.map = *map; e.used = true;
    }
    return r;
}

static EncodeTiledFn get_encode_fn() { return get_driver_encode_fn() ? &encode_cached : nullptr; }

// 3-D view (inner, rows, batch) of a bf16 matrix with a 64-element (128-byte) inner box.
int make_operand_map(CUtensorMap* map, const bf16* ptr, long long inner, long long rows, long long ld, int batch,
                     long long batch_stride, int box_rows);
static int make_operand_map_es(CUtensorMap* map, const void* ptr, int es, long long inner, long long rows,
                               long long ld, int batch, long long batch_stride, int box_rows, bool mn_major = false);
int make_operand_map(CUtensorMap* map, const bf16* ptr, long long inner, long long rows, long long ld,
                     int batch, long long batch_stride, int box_rows) {
    return make_operand_map_es(map, ptr, 2, inner, rows, ld, batch, batch_stride, box_rows);
}
// es = 2: bf16, 64-element rows; es = 4: float32 (read as tf32), 32-element rows
static int make_operand_map_es(CUtensorMap* map, const void* ptr, int es, long long inner, long long rows,
                               long long ld, int batch, long long batch_stride, int box_rows, bool mn_major) {
    EncodeTiledFn enc = get_encode_fn();
    TB_CHECK(enc != nullptr, "cuTensorMapEncodeTiled entry point not available");
    TB_CHECK((reinterpret_cast<uintptr_t>(ptr) & 15u) == 0, "GEMM operand must be 16-byte aligned");
    TB_CHECK((ld * es) % 16 == 0, "GEMM operand leading dimension must be a multiple of 16 bytes (got %lld elements of %d bytes)",
             ld, es);
    TB_CHECK(batch == 1 || (batch_stride * es) % 16 == 0, "GEMM batch stride must be a multiple of 16 bytes");
    cuuint64_t dims[3] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)batch};
    cuuint64_t bs = batch > 1 ? (cuuint64_t)batch_stride * es : (cuuint64_t)rows * (cuuint64_t)ld * es;
    if (bs == 0) bs = 16;
    cuuint64_t strides[2] = {(cuuint64_t)ld * es, bs};
    cuuint32_t box[3] = {(cuuint32_t)(ROW_BYTES / es), (cuuint32_t)box_rows, 1u};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r = enc(map, es == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3,
                     const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     (es == 4 && mn_major) ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B : CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TB_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled failed with code %d (inner=%lld rows=%lld ld=%lld batch=%d)",
             (int)r, inner, rows, ld, batch);
    return 0;
}

int make_operand_map_f32(CUtensorMap* map, const float* ptr, long long inner, long long rows, long long ld, int batch,
                         long long batch_stride, int box_rows) {
    return make_operand_map_es(map, ptr, 4, inner, rows, ld, batch, batch_stride, box_rows);
}

int make_operand_map4(CUtensorMap* map, const bf16* ptr, long long inner, long long rows, long long ld,
                      long long n0, long long stride0, long long n1, long long stride1, int box_rows) {
    EncodeTiledFn enc = get_encode_fn();
    TB_CHECK(enc != nullptr, "cuTensorMapEncodeTiled entry point not available");
    TB_CHECK((reinterpret_cast<uintptr_t>(ptr) & 15u) == 0 && (ld * 2) % 16 == 0 && (stride0 * 2) % 16 == 0 &&
                 (stride1 * 2) % 16 == 0,
             "attention operand must be 16-byte aligned with strides that are multiples of 8 elements");
    cuuint64_t dims[4] = {(cuuint64_t)inner, (cuuint64_t)rows, (cuuint64_t)n0, (cuuint64_t)n1};
    cuuint64_t s0 = n0 > 1 ? (cuuint64_t)stride0 * 2 : (cuuint64_t)ld * 2 * (cuuint64_t)rows;
    cuuint64_t s1 = n1 > 1 ? (cuuint64_t)stride1 * 2 : (cuuint64_t)ld * 2 * (cuuint64_t)rows;
    cuuint64_t strides[3] = {(cuuint64_t)ld * 2, s0, s1};
    cuuint32_t box[4] = {64u, (cuuint32_t)box_rows, 1u, 1u};
    cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<bf16*>(ptr), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TB_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (4-D operand) failed with code %d", (int)r);
    return 0;
}

// 4-D view (columns, rows, inner batch, outer batch) of an output or residual matrix with a
// 32 x 32 element box: 128-byte rows for float32 (128B swizzle), 64-byte rows for bf16 (64B swizzle).
// wide (bf16 only): a 64 x 32 element box, 128-byte rows with the 128B swizzle.
static int make_map_out(CUtensorMap* map, const void* ptr, int elem_bytes, long long cols, long long rows,
                        long long ld, long long inner, long long stride_in, long long outer, long long stride_out,
                        bool wide = false) {
    EncodeTiledFn enc = get_encode_fn();
    TB_CHECK(enc != nullptr, "cuTensorMapEncodeTiled entry point not available");
    const cuuint64_t row_bytes = (cuuint64_t)ld * elem_bytes;
    cuuint64_t s_in = inner > 1 ? (cuuint64_t)stride_in * elem_bytes : row_bytes * (cuuint64_t)rows;
    cuuint64_t s_out = outer > 1 ? (cuuint64_t)stride_out * elem_bytes : row_bytes * (cuuint64_t)rows;
    if (s_in == 0) s_in = 16;
    if (s_out == 0) s_out = 16;
    cuuint64_t dims[4] = {(cuuint64_t)cols, (cuuint64_t)rows, (cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t strides[3] = {row_bytes, s_in, s_out};
    cuuint32_t box[4] = {wide ? 64u : 32u, 32u, 1u, 1u};
    cuuint32_t estr[4] = {1u, 1u, 1u, 1u};
    CUresult r = enc(map, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4,
                     const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     (elem_bytes == 4 || wide) ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                     CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    TB_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (output) failed with code %d (cols=%lld rows=%lld ld=%lld)",
             (int)r, cols, rows, ld);
    return 0;
}

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

static int pick_bn(const DeviceCtx* ctx, const GemmArgs& a) {
    // time ~ waves x tile width x a factor for how often a tile re-reads its operands from L2
    // (flops per operand byte: 43 for 128x64, 64 for 128x128, 77 for 128x192, 128 for a CTA pair on 256x256).
    // 256 = a CTA pair on a 256 x 256 tile: per output element a CTA pulls 0.6x the operand bytes of a
    // 128 x 192 tile through its L2 port (the limit of the main loop); its waves are counted in CTA pairs.
    const bool pair_ok = !a.tf32 && a.batch == 1 && a.causal == CAUSAL_NONE && a.c_inner <= 1 && a.M >= 512 &&
                         getenv("TB_GEMM_NO_PAIR") == nullptr;
    const long long mt = (a.M + BM - 1) / BM;
    auto cost_of = [&](int width) -> double {
        static const double factor[4] = {1.30, 1.00, 0.95, 0.70};
        if (width == 256) {
            const long long tiles = ((a.M + 2 * BM - 1) / (2 * BM)) * ((a.N + 255) / 256);
            const long long pairs = ctx->sm_count / 2;
            // a narrow output wastes part of the second 256-wide column of tiles; only a long K loop pays for that
            const double narrow = (a.N < 512 && a.K < 4096) ? 1.15 : 1.0;
            return (double)((tiles + pairs - 1) / pairs) * 256 * factor[3] * narrow;
        }
        const long long tiles = mt * ((a.N + width - 1) / width) * a.batch;
        return (double)((tiles + ctx->sm_count - 1) / ctx->sm_count) * width * factor[width / 64 - 1];
    };
    if (a.swiglu_h)      // paired gate/up tile: 128 wide, or 256 wide on a CTA pair
        return ((a.bn == 256 || (a.bn == 0 && pair_ok && cost_of(256) < cost_of(128))) && a.N % 256 == 0) ? 256 : 128;
    if (a.dsw_dgu) return (a.bn == 256 || (a.bn == 0 && pair_ok)) ? 256 : 128;      // its chunks leave in pairs
    if (a.ce_mode != 0) return a.bn == 256 ? 256 : 192;     // the statistics are laid out per tile of this width
    if (a.bn == 64 || a.bn == 128 || a.bn == 192 || a.bn == 256 || a.bn == 384) return a.bn;
    // one 256 x 384 pair tile over the whole N where K is long (the LM-head gradients: dE 225 -> ~125 us)
    if (pair_ok && a.kind != GEMM_NT && a.N > 256 && a.N <= 384 && a.K >= 4096 && !a.swiglu_h && !a.rope_qkv &&
        getenv("TB_GEMM_NO_384") == nullptr)
        return 384;
    if (a.N <= 64) return 64;
    const long long t128 = mt * ((a.N + 127) / 128) * a.batch;
    if (t128 * 2 <= ctx->sm_count && a.K >= 16 * (a.tf32 ? BK_TF32 : BK)) {
        // split-K will fill the machine.  With at least 16 tiles of 192 columns the wider tile wins (fewer operand
        // bytes per flop through the SM's L2 port): measured on the weight-gradient products at K = 8192,
        // [384 x 1152] 15.2 us against 17.5, [384 x 2048] 22.1 against 23.9, [1024 x 384] 14.9 against 16.0
        const long long t192 = mt * ((a.N + 191) / 192) * a.batch;
        return (!a.tf32 && t192 >= 16) ? 192 : 128;
    }
    const int widths[4] = {64, 128, 192, 256};
    int best = 128;
    double best_cost = 1e30;
    for (int i = 0; i < (pair_ok ? 4 : 3); ++i) {
        const double cost = cost_of(widths[i]);
        if (cost < best_cost - 1e-9) { best_cost = cost; best = widths[i]; }
    }
    if (a.causal != CAUSAL_NONE && best == 192) best = 128;     // the causal tile rules assume 64 | 128 columns
    return best;
}

int choose_splits(const DeviceCtx* ctx, const GemmArgs& a, int bn) {
    if (a.causal != CAUSAL_NONE) return 1;
    const int tile_m = bn >= 256 ? 2 * BM : BM;                     // a CTA pair owns 256 rows
    const int sms = (a.max_ctas > 0 && a.max_ctas < ctx->sm_count) ? a.max_ctas : ctx->sm_count;
    const int workers = bn >= 256 ? sms / 2 : sms;
    const long long tiles = (long long)((a.M + tile_m - 1) / tile_m) * ((a.N + bn - 1) / bn) * a.batch;
    const int bke = a.tf32 ? BK_TF32 : BK;
    const int kb_total = (a.K + bke - 1) / bke;
    if (tiles * 2 > workers || kb_total < 16) return 1;
    int s = (int)(workers / tiles);
    if (s > kb_total / 4) s = kb_total / 4;     // at least 4 K slices per split
    if (s < 1) s = 1;
    const int kb_per = (kb_total + s - 1) / s;
    return (kb_total + kb_per - 1) / kb_per;     // no empty split
}

template <int BN, bool TF32, bool PAIR = false, int EPI = EPI_ANY>
static int launch_impl(DeviceCtx* ctx, const GemmArgs& a, const GemmParams& p, const CUtensorMap& tmA,
                       const CUtensorMap& tmB, const CUtensorMap& tmC, const CUtensorMap& tmR,
                       cudaStream_t stream) {
    using Cfg = GemmCfg<BN, PAIR>;
    static bool attr_set[64] = {false};
    if (!attr_set[ctx->device & 63]) {
        TB_CUDA(cudaFuncSetAttribute(gemm_bf16_kernel<BN, TF32, PAIR, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     Cfg::SMEM_BYTES));
        attr_set[ctx->device & 63] = true;
    }
    const long long total = (long long)p.batch * p.splits * p.mt * p.nt;
    const int sms = (a.max_ctas > 0 && a.max_ctas < ctx->sm_count) ? a.max_ctas : ctx->sm_count;
    int grid;
    if (PAIR) {
        const long long pairs = sms / 2;
        grid = 2 * (int)(total < pairs ? total : pairs);      // one cluster of two CTAs per tile in flight
    } else {
        grid = (int)(total < sms ? total : sms);
    }
    if (grid < 1) grid = PAIR ? 2 : 1;
    TB_CUDA(launch_kernel_cluster((gemm_bf16_kernel<BN, TF32, PAIR, EPI>), dim3(grid), dim3(NUM_THREADS), Cfg::SMEM_BYTES,
                                  stream, PAIR ? 2 : 1, tmA, tmB, tmC, tmR, p));
    TB_CUDA(cudaGetLastError());
    ctx->launches++;
    prof_close(ctx, stream);
    return 0;
}

// The instantiation compiled for the launch's epilogue where one exists (bf16 operands; the fused epilogues on the tile
// widths the trainer uses them with), else the general kernel.
template <int BN, bool PAIR>
static int launch_bf16(DeviceCtx* ctx, const GemmArgs& a, const GemmParams& p, const CUtensorMap& tmA,
                       const CUtensorMap& tmB, const CUtensorMap& tmC, const CUtensorMap& tmR, cudaStream_t stream) {
    static const bool general_only = getenv("TB_GEMM_GENERAL_KERNEL") != nullptr;
    int epi = EPI_ANY;
    if (!general_only) {
        switch (p.tma_mode) {
            case 1: epi = EPI_F32; break;
            case 2: epi = p.ce_mode == 2 ? EPI_CE2 : p.dsw ? EPI_DSW : EPI_BF16; break;
            case 3: epi = EPI_SWIGLU; break;
            case 4: epi = EPI_CE1; break;
            case 5: epi = EPI_ROPE; break;
            default: break;
        }
    }
    if (epi == EPI_F32) return launch_impl<BN, false, PAIR, EPI_F32>(ctx, a, p, tmA, tmB, tmC, tmR, stream);
    if (epi == EPI_BF16) return launch_impl<BN, false, PAIR, EPI_BF16>(ctx, a, p, tmA, tmB, tmC, tmR, stream);
    if constexpr (BN == 128 || BN == 256) {
        if (epi == EPI_SWIGLU) return launch_impl<BN, false, PAIR, EPI_SWIGLU>(ctx, a, p, tmA, tmB, tmC, tmR, stream);
        if (epi == EPI_DSW) return launch_impl<BN, false, PAIR, EPI_DSW>(ctx, a, p, tmA, tmB, tmC, tmR, stream);
    }
    if constexpr (BN == 192 || BN == 256) {
        if (epi == EPI_CE1) return launch_impl<BN, false, PAIR, EPI_CE1>(ctx, a, p, tmA, tmB, tmC, tmR, stream);
        if (epi == EPI_CE2) return launch_impl<BN, false, PAIR, EPI_CE2>(ctx, a, p, tmA, tmB, tmC, tmR, stream);
    }
    if constexpr (BN == 128) {
        if (epi == EPI_ROPE) return launch_impl<BN, false, PAIR, EPI_ROPE>(ctx, a, p, tmA, tmB, tmC, tmR, stream);
    }
    return launch_impl<BN, false, PAIR, EPI_ANY>(ctx, a, p, tmA, tmB, tmC, tmR, stream);
}

static int launch_core(DeviceCtx* ctx, const GemmArgs& a, int bn, int splits, float* ws, cudaStream_t stream) {
    TB_CHECK(a.M > 0 && a.N > 0 && a.K > 0 && a.batch > 0, "GEMM dims must be positive (M=%d N=%d K=%d batch=%d)",
             a.M, a.N, a.K, a.batch);
    TB_CHECK(a.A && a.B && (a.C32 || a.C16 || a.swiglu_h || a.ce_mode == 1 || a.rope_qkv || a.dsw_dgu),
             "GEMM needs A, B and at least one output");
    if (a.rope_qkv) {
        TB_CHECK(a.kind == GEMM_NN && !a.tf32 && a.batch == 1 && splits == 1 && a.alpha == 1.0f && a.beta == 0.0f &&
                     !a.residual && !a.C32 && !a.C16 && !a.swiglu_h && a.ce_mode == 0 && a.causal == CAUSAL_NONE &&
                     a.rope_cos && a.rope_sin && (a.rope_hd == 32 || a.rope_hd == 64) && a.rope_T > 0 &&
                     a.rope_T % 32 == 0 && a.M % a.rope_T == 0 && a.N == 3 * a.rope_H * a.rope_hd && aligned16(a.rope_qkv),
                 "fused QKV + position-embedding GEMM: needs a plain NN bf16 product with N = 3*H*hd, hd 32 or 64, T %% 32 == 0");
    }
    if (a.ce_mode != 0) {
        TB_CHECK(a.kind == GEMM_NT && !a.tf32 && a.batch == 1 && (bn == 192 || bn == 256) && splits == 1 && a.alpha == 1.0f &&
                     a.beta == 0.0f && !a.bias && !a.residual && !a.C32 && !a.swiglu_h && a.causal == CAUSAL_NONE && a.ce_targets,
                 "fused cross-entropy GEMM: needs a plain NT bf16 product with 192-column tiles and the targets");
        if (a.ce_mode == 1) TB_CHECK(a.ce_stats && a.ce_ztarget && !a.C16, "cross-entropy pass 1 writes statistics only");
        else TB_CHECK(a.ce_mode == 2 && a.ce_lse && a.C16, "cross-entropy pass 2 needs the row log-sum-exp and a bf16 output");
    }
    if (a.dsw_dgu) {
        TB_CHECK(!a.tf32 && a.batch == 1 && splits == 1 && a.alpha == 1.0f && a.beta == 0.0f && !a.bias && !a.residual &&
                     !a.C32 && !a.C16 && !a.swiglu_h && a.ce_mode == 0 && !a.rope_qkv && a.causal == CAUSAL_NONE &&
                     a.dsw_gu && a.N % 64 == 0 && a.ldgu % 8 == 0 && a.ldgu >= 2 * a.N &&
                     aligned16(a.dsw_gu) && aligned16(a.dsw_dgu),
                 "SwiGLU-backward GEMM: needs a plain bf16 product with N = F (a multiple of 64), the saved gate|up "
                 "projection and the output, 16-byte aligned with ldgu %% 8 == 0");
    }
    const bool swiglu = a.swiglu_h != nullptr;
    if (swiglu) {
        TB_CHECK(a.kind == GEMM_NN && !a.tf32 && a.batch == 1 && (bn == 128 || bn == 256) && splits == 1 && a.N % bn == 0 &&
                     a.residual == nullptr && a.alpha == 1.0f && a.beta == 0.0f && !a.C32 && !a.C16 && a.causal == CAUSAL_NONE,
                 "fused SwiGLU GEMM: needs a plain NN bf16 product with N = 2F, F a multiple of 64 (got N=%d)", a.N);
        TB_CHECK(aligned16(a.swiglu_h) && a.ldh % 8 == 0 && (!a.swiglu_gu || (aligned16(a.swiglu_gu) && a.ldgu % 8 == 0)),
                 "fused SwiGLU GEMM: outputs must be 16-byte aligned with leading dimensions that are multiples of 8");
    }
    const int a_mn = (a.kind == GEMM_TN) ? 1 : 0;
    const int b_mn = (a.kind == GEMM_NT) ? 0 : 1;
    CUtensorMap tmA, tmB;
    const int es = a.tf32 ? 4 : 2;
    const int bke = a.tf32 ? BK_TF32 : BK;
    if (!a_mn) TB_TRY(make_operand_map_es(&tmA, a.A, es, a.K, a.M, a.lda, a.batch, a.strideA, BM));
    else       TB_TRY(make_operand_map_es(&tmA, a.A, es, a.M, a.K, a.lda, a.batch, a.strideA, bke, true));
    const bool pair = bn == 256 || bn == 384;
    if (pair)
        TB_CHECK(!a.tf32 && a.batch == 1 && a.causal == CAUSAL_NONE && a.c_inner <= 1,
                 "256-wide CTA-pair tiles take one plain bf16 product (no batch, no causal mode)");
    if (bn == 384)
        TB_CHECK(b_mn && !a.swiglu_h && a.ce_mode == 0 && !a.rope_qkv,
                 "384-wide CTA-pair tiles take B stored [K, N] (kinds NN and TN) and a plain epilogue");
    if (!b_mn) TB_TRY(make_operand_map_es(&tmB, a.B, es, a.K, a.N, a.ldb, a.batch, a.strideB, pair ? bn / 2 : bn));
    else       TB_TRY(make_operand_map_es(&tmB, a.B, es, a.N, a.K, a.ldb, a.batch, a.strideB, bke, true));

    GemmParams p;
    p.M = a.M; p.N = a.N; p.K = a.K; p.batch = a.batch; p.splits = splits;
    p.mt = pair ? (a.M + 2 * BM - 1) / (2 * BM) : (a.M + BM - 1) / BM;      // a pair owns 256 rows
    p.nt = (a.N + bn - 1) / bn;
    p.kb_total = (a.K + bke - 1) / bke;
    p.kb_per = (p.kb_total + splits - 1) / splits;
    p.a_mn = a_mn; p.b_mn = b_mn; p.causal = (int)a.causal;
    p.dsw = 0; p.wide16 = 0;
    p.err = ctx->d_err;
    if (splits > 1) {
        // partial tiles, one [M,N] slab per (batch, split); everything else happens in the reduction
        TB_CHECK(a.c_inner <= 1, "split-K GEMM does not take a two-level output batch stride");
        p.C32 = ws; p.ldc32 = a.N; p.strideC32 = (long long)a.M * a.N; p.strideC32_in = 0;
        p.C16 = nullptr; p.ldc16 = 0; p.strideC16 = 0; p.strideC16_in = 0;
        p.c_inner = 1;
        p.bias = nullptr; p.residual = nullptr; p.ldr = 0; p.strideR = 0;
        p.alpha = a.alpha; p.beta = 0.0f;
    } else {
        p.C32 = a.C32; p.ldc32 = a.ldc32; p.strideC32 = a.strideC32; p.strideC32_in = a.strideC32_in;
        p.C16 = a.C16; p.ldc16 = a.ldc16; p.strideC16 = a.strideC16; p.strideC16_in = a.strideC16_in;
        p.c_inner = a.c_inner > 1 ? a.c_inner : 1;
        p.bias = a.bias; p.residual = a.residual; p.ldr = a.ldr; p.strideR = a.strideR;
        p.alpha = a.alpha; p.beta = a.beta;
    }
    p.vec32 = p.C32 && (reinterpret_cast<uintptr_t>(p.C32) % 16 == 0) && p.ldc32 % 4 == 0 && p.strideC32 % 4 == 0 &&
              p.strideC32_in % 4 == 0;
    p.vec16 = p.C16 && (reinterpret_cast<uintptr_t>(p.C16) % 8 == 0) && p.ldc16 % 4 == 0 && p.strideC16 % 4 == 0 &&
              p.strideC16_in % 4 == 0;
    p.vecr = p.residual && (reinterpret_cast<uintptr_t>(p.residual) % 16 == 0) && p.ldr % 4 == 0 && p.strideR % 4 == 0;

    // Tile stores by TMA when the output (and the residual / previous C) is 16-byte addressable
    CUtensorMap tmC, tmR;
    memset(&tmC, 0, sizeof(tmC));
    memset(&tmR, 0, sizeof(tmR));
    p.tma_mode = 0; p.tma_res = 0; p.res_scale = 0.0f;
    p.pair_off = 0; p.keep_gu = 0;
    p.ce_mode = a.ce_mode; p.ce_targets = a.ce_targets; p.ce_stats = a.ce_stats; p.ce_ztarget = a.ce_ztarget;
    p.ce_lse = a.ce_lse; p.ce_scale = a.ce_scale;
    p.bias_vec = p.bias && aligned16(p.bias);
    p.rope_cos = a.rope_cos; p.rope_sin = a.rope_sin; p.rope_T = a.rope_T; p.rope_H = a.rope_H; p.rope_hd = a.rope_hd;
    if (a.ce_mode == 1) {
        p.tma_mode = 4;
    } else if (a.rope_qkv) {
        EncodeTiledFn enc = get_encode_fn();
        TB_CHECK(enc != nullptr, "cuTensorMapEncodeTiled entry point not available");
        const cuuint64_t hd = (cuuint64_t)a.rope_hd, T = (cuuint64_t)a.rope_T, H = (cuuint64_t)a.rope_H, Bn = (cuuint64_t)(a.M / a.rope_T);
        cuuint64_t dims[5] = {hd, T, H, Bn, 3};
        cuuint64_t strides[4] = {hd * 2, T * hd * 2, H * T * hd * 2, Bn * H * T * hd * 2};
        // head dim 64 on 128- or 256-column tiles: a warp's chunk pairs are whole heads and leave in rows of 128 bytes
        const bool wide = a.rope_hd == 64 && (bn == 128 || bn == 256) && getenv("TB_GEMM_NO_WIDE16") == nullptr;
        cuuint32_t box[5] = {wide ? 64u : 32u, 32u, 1u, 1u, 1u};
        cuuint32_t estr[5] = {1u, 1u, 1u, 1u, 1u};
        CUresult r = enc(&tmC, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 5, a.rope_qkv, dims, strides, box, estr,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, wide ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                         CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        p.wide16 = wide ? 1 : 0;
        TB_CHECK(r == CUDA_SUCCESS, "cuTensorMapEncodeTiled (QKV output) failed with code %d", (int)r);
        p.tma_mode = 5;
    } else if (a.dsw_dgu) {
        TB_CHECK(bn == 128 || bn == 256, "SwiGLU-backward GEMM: tiles of 128 or 256 columns (chunks leave in pairs)");
        TB_TRY(make_map_out(&tmC, a.dsw_dgu, 2, 2 * a.N, a.M, a.ldgu, 1, 0, 1, 0, true));
        TB_TRY(make_map_out(&tmR, a.dsw_gu, 2, 2 * a.N, a.M, a.ldgu, 1, 0, 1, 0));
        p.tma_mode = 2; p.dsw = 1; p.wide16 = 1; p.pair_off = a.N;
    } else if (swiglu) {
        const int F = a.N / 2;
        // 256-column tiles: a warp's two chunks are 64 adjacent hidden units and leave in rows of 128 bytes
        const bool wide = bn == 256 && F % 64 == 0 && getenv("TB_GEMM_NO_WIDE16") == nullptr;
        TB_TRY(make_map_out(&tmC, a.swiglu_h, 2, F, a.M, a.ldh, 1, 0, 1, 0, wide));
        if (a.swiglu_gu) TB_TRY(make_map_out(&tmR, a.swiglu_gu, 2, a.N, a.M, a.ldgu, 1, 0, 1, 0, wide));
        else tmR = tmC;
        p.wide16 = wide ? 1 : 0;
        p.tma_mode = 3; p.pair_off = F; p.keep_gu = a.swiglu_gu ? 1 : 0;
    } else {
        const bool one_out = (p.C32 != nullptr) != (p.C16 != nullptr);
        const int es = p.C32 ? 4 : 2;
        const void* cptr = p.C32 ? (const void*)p.C32 : (const void*)p.C16;
        const long long ld = p.C32 ? p.ldc32 : p.ldc16;
        const long long so = p.C32 ? p.strideC32 : p.strideC16;
        const long long si = p.C32 ? p.strideC32_in : p.strideC16_in;
        const long long nz = (long long)p.batch * p.splits;
        const bool has_res = p.residual != nullptr;
        const bool has_beta = p.C32 != nullptr && p.beta != 0.0f;
        // TMA stores work in 16-byte units: a row end that is not on such a boundary would spill
        // zeros into the next few elements, so it needs the caller's word that those are padding
        const bool row_end_ok = ((long long)p.N * es) % 16 == 0 || a.pad_cols_writable;
        bool ok = one_out && row_end_ok && aligned16(cptr) && (ld * es) % 16 == 0 && (so * es) % 16 == 0 && (si * es) % 16 == 0 &&
                  nz % p.c_inner == 0 && !getenv("TB_GEMM_GENERIC_EPILOGUE");
        if (has_res && has_beta) ok = false;
        if ((has_res || has_beta) && (p.C32 == nullptr || p.c_inner > 1)) ok = false;
        if (has_res && !(aligned16(p.residual) && (p.ldr * 4) % 16 == 0 && (p.strideR * 4) % 16 == 0)) ok = false;
        TB_CHECK(ok || a.ce_mode == 0, "fused cross-entropy GEMM: the bf16 output must be 16-byte aligned with padded rows");
        if (ok) {
            TB_TRY(make_map_out(&tmC, cptr, es, p.N, p.M, ld, p.c_inner, si, nz / p.c_inner, so));
            if (has_res) {
                TB_TRY(make_map_out(&tmR, p.residual, 4, p.N, p.M, p.ldr, 1, 0, p.batch, p.strideR));
                p.tma_res = 1; p.res_scale = 1.0f;
            } else if (has_beta) {
                tmR = tmC;
                p.tma_res = 1; p.res_scale = p.beta;
            }
            p.tma_mode = p.C32 ? 1 : 2;
            if (!p.C32 && bn >= 128 && getenv("TB_GEMM_NO_WIDE16") == nullptr) {
                // bf16 tiles leave in rows of 128 bytes (two chunks per store); tmR is free: no residual with a bf16 output
                TB_TRY(make_map_out(&tmR, cptr, es, p.N, p.M, ld, p.c_inner, si, nz / p.c_inner, so, true));
                p.wide16 = 1;
            }
        }
    }
    {
        // algorithmic work: the causal products touch only the lower triangle (half the MACs)
        const double macs = (double)a.M * a.N * a.K * a.batch * (a.causal != CAUSAL_NONE ? 0.5 : 1.0);
        const double out_bytes = a.rope_qkv ? 2.0 * a.M * a.N
                                 : a.ce_mode == 1 ? 16.0 * a.M * ((a.N + 191) / 192)
                                 : a.dsw_dgu   ? 8.0 * a.M * a.N          // g, u read and dg, du written, bf16
                                 : swiglu      ? (double)a.M * a.N * (a.swiglu_gu ? 3.0 : 1.0)
                                        : (double)a.M * a.N * a.batch * ((a.C32 ? 4.0 : 0.0) + (a.C16 ? 2.0 : 0.0)) *
                                              (a.causal == CAUSAL_SKIP_UPPER ? 0.5 : 1.0);
        const double in_bytes = 2.0 * a.batch * ((double)a.M * a.K + (double)a.K * a.N) *
                                (a.causal == CAUSAL_K_PREFIX || a.causal == CAUSAL_K_SUFFIX ? 0.75 : 1.0);
        if (ctx->prof_on) {
            char tag[128];
            static const char* kn[3] = {"NN", "NT", "TN"};
            snprintf(tag, sizeof(tag), "%s:%s:%dx%dx%d:b%d:s%d:c%d:bn%d%s", a.tf32 ? "gemm_tf32" : "gemm_bf16",
                     kn[(int)a.kind], a.M, a.N, a.K, a.batch, splits, (int)a.causal, bn, swiglu ? ":swiglu" : a.rope_qkv ? ":rope" : a.ce_mode == 1 ? ":ce_stats" : a.ce_mode == 2 ? ":ce_grad" : "");
            // the second cross-entropy pass repeats pass 1's product: its flops are not algorithmic work
            prof_mark(ctx, prof_intern(tag), a.ce_mode == 2 ? 0.0 : 2.0 * macs, in_bytes + out_bytes, stream);
        }
    }
    if (pair && bn == 384) {
        TB_TRY((launch_bf16<384, true>(ctx, a, p, tmA, tmB, tmC, tmR, stream)));
    } else if (pair) {
        TB_TRY((launch_bf16<256, true>(ctx, a, p, tmA, tmB, tmC, tmR, stream)));
    } else if (a.tf32) {
        // (float32 operands read as tf32: plain float32 / bf16 tiles have instantiations of their own, the rest is general)
        static const bool general_only = getenv("TB_GEMM_GENERAL_KERNEL") != nullptr;
        const int epi = general_only ? EPI_ANY : p.tma_mode == 1 ? EPI_F32 : (p.tma_mode == 2 && p.ce_mode == 0 && !p.dsw) ? EPI_BF16 : EPI_ANY;
#define TB_TF32_LAUNCH(W)                                                                                              \
        (epi == EPI_F32    ? launch_impl<W, true, false, EPI_F32>(ctx, a, p, tmA, tmB, tmC, tmR, stream)                 \
         : epi == EPI_BF16 ? launch_impl<W, true, false, EPI_BF16>(ctx, a, p, tmA, tmB, tmC, tmR, stream)                \
                           : launch_impl<W, true, false, EPI_ANY>(ctx, a, p, tmA, tmB, tmC, tmR, stream))
        if (bn == 64)       TB_TRY(TB_TF32_LAUNCH(64));
        else if (bn == 192) TB_TRY(TB_TF32_LAUNCH(192));
        else                TB_TRY(TB_TF32_LAUNCH(128));
#undef TB_TF32_LAUNCH
    } else {
        if (bn == 64)       TB_TRY((launch_bf16<64, false>(ctx, a, p, tmA, tmB, tmC, tmR, stream)));
        else if (bn == 192) TB_TRY((launch_bf16<192, false>(ctx, a, p, tmA, tmB, tmC, tmR, stream)));
        else                TB_TRY((launch_bf16<128, false>(ctx, a, p, tmA, tmB, tmC, tmR, stream)));
    }

    if (splits > 1) {
        TB_CHECK(a.residual == nullptr, "split-K GEMM does not take a residual operand");
        const long long per = (long long)a.M * a.N;
        const bool vec4 = a.N % 4 == 0;      // a float4 never straddles a row; partial slabs are 16-byte aligned
        const long long nvec = vec4 ? per / 4 : per;
        int blocks = (int)((nvec + 255) / 256);
        if (blocks > 8 * ctx->sm_count) blocks = 8 * ctx->sm_count;
        if (blocks < 1) blocks = 1;
        dim3 grid(blocks, a.batch);
        prof_mark(ctx, "splitk_reduce", 0.0, (double)(splits + 2) * per * a.batch * 4.0, stream);
        if (vec4)
            TB_CUDA(launch_kernel((reduce_splits_kernel<4>), dim3(grid), dim3(256), 0, stream, ws, a.C32, a.C16, a.M, a.N, a.ldc32, a.ldc16, splits, a.strideC32, a.strideC16, a.beta, a.bias));
        else
            TB_CUDA(launch_kernel((reduce_splits_kernel<1>), dim3(grid), dim3(256), 0, stream, ws, a.C32, a.C16, a.M, a.N, a.ldc32, a.ldc16, splits, a.strideC32, a.strideC16, a.beta, a.bias));
        TB_CUDA(cudaGetLastError());
        ctx->launches++;
        prof_close(ctx, stream);
    }
    return 0;
}

// Forms that cannot be split along K run unsplit: fused epilogues, a residual operand, and the causal modes
// (a skipped tile writes no partial slab, and the causal k ranges are per tile).  A split count beyond the
// number of K slices would leave empty splits.
static int check_splits(const GemmArgs& a, int* splits) {
    if (a.residual || a.c_inner > 1 || a.swiglu_h || a.ce_mode != 0 || a.rope_qkv || a.causal != CAUSAL_NONE) *splits = 1;
    const int bke = a.tf32 ? BK_TF32 : BK;
    const int kb_total = (a.K + bke - 1) / bke;
    TB_CHECK(*splits <= kb_total, "splits=%d exceeds the %d K slices of %d elements this product has", *splits, kb_total, bke);
    return 0;
}

int launch_gemm_bf16(DeviceCtx* ctx, const GemmArgs& a, cudaStream_t stream) {
    const int bn = pick_bn(ctx, a);
    int splits = a.splits > 0 ? a.splits : choose_splits(ctx, a, bn);
    TB_TRY(check_splits(a, &splits));
    float* ws = nullptr;
    if (splits > 1) {
        const size_t need = (size_t)splits * a.batch * a.M * a.N * sizeof(float);
        TB_TRY(ensure_scratch(ctx, need));
        ws = static_cast<float*>(ctx->scratch);
    }
    return launch_core(ctx, a, bn, splits, ws, stream);
}

int launch_gemm_bf16_ws(DeviceCtx* ctx, const GemmArgs& a, float* workspace, size_t workspace_floats,
                        cudaStream_t stream) {
    const int bn = pick_bn(ctx, a);
    int splits = a.splits > 0 ? a.splits : choose_splits(ctx, a, bn);
    TB_TRY(check_splits(a, &splits));
    if (splits > 1) {
        const size_t need = (size_t)splits * a.batch * a.M * a.N;
        TB_CHECK(workspace != nullptr && workspace_floats >= need,
                 "split-K workspace too small: need %zu floats, have %zu", need, workspace_floats);
    }
    return launch_core(ctx, a, bn, splits, workspace, stream);
}

// =====================================================================================
// Split-K GEMM that allocates nothing.
//
// Some hosts of this library must not call cudaMalloc at all: a process whose device memory is
// entirely owned by another allocator (a framework's caching pool that has reserved the card, a
// fixed partition handed to a service), and loops that cannot afford cudaMalloc's device-wide
// synchronisation because other streams are in flight.  For them the split-K partial sums live in
// a fixed array inside the library image instead of the growable scratch buffer, and the word that
// reports a timed-out wait lives beside it.  Every GPU that loads the library carries the array
// (16 MiB) until the process exits.
//
// In host code `g_static_partials` is only a stand-in for the symbol: its device address is looked
// up once per device with cudaGetSymbolAddress and that address is what the kernels receive.
constexpr size_t kStaticPartialFloats = 4u * 1024u * 1024u;   // 16 MiB: split count x batch x M x N floats
static __device__ __align__(256) float g_static_partials[kStaticPartialFloats];
static __device__ int g_static_status;

namespace {
struct StaticSetup {
    bool done = false;
    float* partials = nullptr;   // device address of g_static_partials on this device
    int* status = nullptr;       // device address of g_static_status
    int sm_count = 0;
};
StaticSetup g_static_setup[64];
std::mutex g_static_mutex;

int static_setup(int dev, StaticSetup** out) {
    TB_CHECK(dev >= 0 && dev < 64, "device ordinal %d out of range", dev);
    StaticSetup* s = &g_static_setup[dev];
    std::lock_guard<std::mutex> lock(g_static_mutex);     // two host threads may make the first call together
    if (!s->done) {
        void* p = nullptr;
        TB_CUDA(cudaGetSymbolAddress(&p, g_static_partials));
        s->partials = static_cast<float*>(p);
        TB_CUDA(cudaGetSymbolAddress(&p, g_static_status));
        s->status = static_cast<int*>(p);
        int major = 0;
        TB_CUDA(cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev));
        TB_CHECK(major == 10, "this library is built for sm_100a only; device %d has compute capability %d.x", dev,
                 major);
        TB_CUDA(cudaDeviceGetAttribute(&s->sm_count, cudaDevAttrMultiProcessorCount, dev));
        s->done = true;
    }
    *out = s;
    return 0;
}
}  // namespace

}  // namespace tb

#ifdef TB_GEMM_STAMPS
// host[160][16] <- the stamps of the last launch (ns of %globaltimer; 0 = not reached), then cleared.  Slots per CTA:
// 0 entry, 1 barriers and tensor memory set up, 2 first tile's first loads issued, 3 all loads issued, 4 first operands
// arrived, 5 first tile's products committed, 6 last tile's products committed, 7 epilogue sees the first accumulator,
// 8 first tile stored, 9 last tile stored, 10 the stores have left shared memory.  (TMA-store epilogue, warp 2.)
extern "C" int tb_debug_gemm_stamps(unsigned long long* host) {
    int rc = (int)cudaMemcpyFromSymbol(host, tb::g_gemm_stamps, sizeof(tb::g_gemm_stamps));
    static unsigned long long zero[160][16];
    rc |= (int)cudaMemcpyToSymbol(tb::g_gemm_stamps, zero, sizeof(zero));
    return rc;
}
#endif

extern "C" int tb_gemm_bf16_splitk_static(int kind, const void* d_A, const void* d_B, int M, int N, int K,
                                          int64_t lda, int64_t ldb, float* d_C32, int64_t ldc32,
                                          const float* d_bias, float alpha, float beta, int splits, int wait,
                                          void* stream) {
    using namespace tb;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int dev = -1;
    TB_CUDA(cudaGetDevice(&dev));
    StaticSetup* s = nullptr;
    TB_TRY(static_setup(dev, &s));
    TB_CHECK(kind >= 0 && kind <= 2, "unknown GEMM kind %d", kind);
    TB_CHECK(d_C32 != nullptr, "tb_gemm_bf16_splitk_static writes a float32 output: d_C32 is NULL");

    // a context on the stack: nothing here owns device memory
    DeviceCtx ctx;
    ctx.device = dev;
    ctx.sm_count = s->sm_count;
    ctx.d_err = s->status;

    GemmArgs a;
    a.kind = static_cast<GemmKind>(kind);
    a.A = static_cast<const bf16*>(d_A); a.B = static_cast<const bf16*>(d_B);
    a.M = M; a.N = N; a.K = K; a.lda = lda; a.ldb = ldb;
    a.C32 = d_C32; a.ldc32 = ldc32;
    a.bias = d_bias; a.alpha = alpha; a.beta = beta;
    TB_CHECK(M > 0 && N > 0 && K > 0, "GEMM dims must be positive (M=%d N=%d K=%d)", M, N, K);
    const int bn = pick_bn(&ctx, a);
    if (splits <= 0) splits = choose_splits(&ctx, a, bn);
    const int kb_total = (K + BK - 1) / BK;
    TB_CHECK(splits <= kb_total, "splits=%d exceeds the %d K slices of 64 this problem has", splits, kb_total);
    const size_t need = splits > 1 ? (size_t)splits * (size_t)M * (size_t)N : 0;
    TB_CHECK(need <= kStaticPartialFloats,
             "tb_gemm_bf16_splitk_static: splits*M*N = %zu floats exceeds the built-in scratch of %zu floats "
             "(16 MiB); use fewer splits or tb_gemm_bf16",
             need, kStaticPartialFloats);
    // the status word keeps the previous call's value: clear it; the partial sums need no clearing,
    // every element the reduction reads is written by this call's tiles first
    TB_CUDA(cudaMemsetAsync(s->status, 0, sizeof(int), st));
    a.splits = splits;
    TB_TRY(launch_core(&ctx, a, bn, splits, s->partials, st));
    if (wait) {
        int h = 0;
        TB_CUDA(cudaStreamSynchronize(st));
        TB_CUDA(cudaMemcpy(&h, s->status, sizeof(int), cudaMemcpyDeviceToHost));
        TB_CHECK(h == 0, "tb_gemm_bf16_splitk_static: a kernel gave up on a bounded wait (code %d); output invalid", h);
    }
    return 0;
}

extern "C" int tb_gemm_bf16_splitk_static_status(void* stream) {
    using namespace tb;
    int dev = -1;
    TB_CUDA(cudaGetDevice(&dev));
    StaticSetup* s = nullptr;
    TB_TRY(static_setup(dev, &s));
    int h = 0;
    TB_CUDA(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    TB_CUDA(cudaMemcpy(&h, s->status, sizeof(int), cudaMemcpyDeviceToHost));
    TB_CHECK(h == 0, "tb_gemm_bf16_splitk_static: a kernel gave up on a bounded wait (code %d); output invalid", h);
    return 0;
}
