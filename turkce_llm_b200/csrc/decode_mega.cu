// One decode step of all layers in ONE cooperative kernel: 148 CTAs (one per SM) walk the phases of every layer
//   [RMSNorm + QKV] -> [rotary + cache append + cache attention] -> [out-projection + residual]
//   -> [RMSNorm + gate|up + SwiGLU] -> [down-projection + residual]
// and meet at a grid barrier after each.  The step of 64 sequences moves 67 MB of weights and ~0.2 GB of cache, 40 us
// at the HBM rate, but as 87 dependent launches it took 570 us: every launch pays its ramp (tensor maps, TMEM, first
// bytes) and its tail.  Here a phase costs a barrier (~1 us) plus the load of the 64 activation rows every CTA needs;
// the weights of the next phase are fetched while the CTA waits at the barrier.
//
// Products: M = 64 rows is far below what tcgen05 wants (the tile would be 64 x 8 columns per CTA) and the step is
// bound by latency and bytes, not flops, so the products are warp-level mma.sync (m16n8k16, bf16 in, float32
// accumulate) on operands in shared memory: a CTA owns slabs of 8 output columns (144 + 48 + 128 + 48 slabs per
// layer at D = 384, F = 1024), the four 16-row tiles go to four warps, two warp groups split K and are added in a
// fixed order.  Weights are kept in a second copy laid out per slab ([slab][8 or 16 columns][K], K contiguous) so that
// a slab is one contiguous read.  Arithmetic mirrors the launch-per-kernel path (same RMSNorm summation order, bf16
// operands, float32 bias/residual, the same sigmoid), which stays the fallback for shapes this kernel does not take.
//
// Replaces, for the decode step, the reference's re-run of lm_forward over the whole window per generated token
// (training/generate.c:186-212).
#include "common.h"
#include "ptx.cuh"
#include "step_kernels.h"

#include <cuda_bf16.h>

#include <cstring>
#include <vector>

namespace tb {

namespace {

constexpr int MEGA_THREADS = 256;
constexpr int MEGA_ROWS = 64;            // sequences per step (rows of every product)
constexpr int MEGA_SPIN_LIMIT = 1 << 22;   // polls of the grid barrier before the kernel gives up (~ a second)

struct MegaLayer {
    const float *attn_norm, *bqkv, *bo, *ffn_norm, *bgu, *bdown;
    const bf16 *wqkv, *wo, *wgu, *wdown;          // slab layout
    bf16 *Kc, *Vc;                                  // [S, H, cap, hd]
    const CUtensorMap *mapK, *mapV;                 // (hd, cap, S*H) views of the caches: 64-row boxes, 128B swizzle
};

struct MegaParams {
    int S, D, H, hd, F, L, cap;
    float eps, scale;
    const float* embed;            // float32 embedding table [V, D]
    const uint32_t* tok;           // [S] current tokens
    const int* pos;                // position of the current token
    const MegaLayer* layers;
    const float *cos_t, *sin_t;
    float *x, *x2, *qkv;           // [S, D], [S, D], [S, 3D]
    bf16 *att, *h;                 // [64, D + 8], [64, F + 8]: padded rows, rows >= S zero (the kernel's own buffers)
    unsigned int* barrier;         // zero at launch
    int* err;
};

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void ldmatrix_x2(uint32_t (&r)[2], const void* p) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];" : "=r"(r[0]), "=r"(r[1]) : "r"(smem_u32(p)));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// Grid barrier number `index` (0, 1, ...) of this launch: every CTA adds one to the counter and waits until it
// holds (index + 1) * gridDim.x.  Bounded: after MEGA_SPIN_LIMIT polls the CTA records error 41 and returns false,
// and every other CTA follows (they time out as well or see the error word).
__device__ __forceinline__ bool grid_barrier(const MegaParams& p, int index, int* sh_flag) {
    // the phase's ordinary stores to shared memory come before the bulk copies that overwrite it after the barrier
    fence_proxy_async();
    __syncthreads();
    if (threadIdx.x == 0) {
        // release + add without waiting for the old value to come back
        asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(p.barrier) : "memory");
        const unsigned int target = (unsigned int)(index + 1) * gridDim.x;
        int ok = 1;
        int polls = 0;
        while (true) {
            unsigned int v;
            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p.barrier) : "memory");
            if (v >= target) break;
            if (++polls > MEGA_SPIN_LIMIT || (polls & 1023) == 0 && *reinterpret_cast<volatile int*>(p.err) != 0) {
                atomicCAS(p.err, 0, 41);
                ok = 0;
                break;
            }
        }
        *sh_flag = ok;
    }
    __syncthreads();
    return *sh_flag != 0;
}

// ---- operand loads -------------------------------------------------------------------------------------------
// All loads are bulk copies (cp.async.bulk, one row or one block per instruction) counted on an mbarrier: 16-byte
// cp.async pieces issued by the threads delivered 11-17 bytes per clock to an SM (96 KB took 8,600 cycles).
// A load is requested by begin_*(...) and awaited by mbar_wait on its barrier with the parity the caller tracks.
// The last ordinary access of the destination lies before a grid barrier (which fences and synchronises).

// a bf16 activation written by other CTAs in the previous phase, stored with padded rows [64][K + 8] in global memory
// too, so that ONE bulk copy fills the operand tile (a copy per row cost ~35 cycles of issue each)
__device__ __forceinline__ void begin_x_bf16(bf16* Xs, int KP, const bf16* src, uint64_t* bar) {
    if (threadIdx.x == 0) {
        mbar_expect_tx(bar, (uint32_t)(MEGA_ROWS * KP * 2));
        bulk_load(Xs, src, (uint32_t)(MEGA_ROWS * KP * 2), bar);
    }
}

// float32 rows (x, or the embedding rows of the current tokens in layer 0) -> stage [S][D]
__device__ __forceinline__ void begin_x_f32(float* stage, const MegaParams& p, const float* x, bool from_embed, uint64_t* bar) {
    if (threadIdx.x == 0) mbar_expect_tx(bar, (uint32_t)(p.S * p.D * 4));
    if (from_embed) {
        if ((int)threadIdx.x < p.S)
            bulk_load(stage + threadIdx.x * p.D, p.embed + (long long)p.tok[threadIdx.x] * p.D, (uint32_t)(p.D * 4), bar);
    } else if (threadIdx.x == 0) {
        bulk_load(stage, x, (uint32_t)(p.S * p.D * 4), bar);
    }
}

// RMSNorm of the staged rows -> bf16 Xs.  The summation order is the one of rmsnorm_fwd_vec_kernel: lane owns columns
// 4 * (lane + 32 k), k ascending, then the butterfly.  A warp works on its eight rows at once: one row is a chain of
// dependent steps (sum, shuffles, square root, scaling) of ~600 cycles.
template <int NV>
__device__ __forceinline__ void norm_staged(bf16* Xs, int KP, const float* stage, const MegaParams& p, const float* w) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int D = p.D;
    constexpr int WARPS = MEGA_THREADS / 32, RU = 8;
    float4 wv[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) wv[k] = __ldg(reinterpret_cast<const float4*>(w + 4 * (lane + 32 * k)));
    for (int r0 = warp; r0 < MEGA_ROWS; r0 += RU * WARPS) {
        float4 xv[RU][NV];
        float ss[RU];
#pragma unroll
        for (int u = 0; u < RU; ++u) {
            const int r = r0 + u * WARPS;
            ss[u] = 0.0f;
#pragma unroll
            for (int k = 0; k < NV; ++k) {
                xv[u][k] = r < p.S ? *reinterpret_cast<const float4*>(stage + r * D + 4 * (lane + 32 * k)) : make_float4(0.f, 0.f, 0.f, 0.f);
                ss[u] += xv[u][k].x * xv[u][k].x + xv[u][k].y * xv[u][k].y + xv[u][k].z * xv[u][k].z + xv[u][k].w * xv[u][k].w;
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1)
#pragma unroll
            for (int u = 0; u < RU; ++u) ss[u] += __shfl_xor_sync(0xffffffffu, ss[u], o);
        // 1 / sqrt(mean + eps): the launch-per-kernel path takes the square root in double and rounds it to float, which
        // is the correctly rounded float square root (53 bits exceed 2 * 24 + 2); __fsqrt_rn gives the same bits
        // without the double-precision pipe, which cost ~250 cycles per row here
#pragma unroll
        for (int u = 0; u < RU; ++u) {
            const int r = r0 + u * WARPS;
            const float rr = 1.0f / __fsqrt_rn(ss[u] / (float)D + p.eps);
#pragma unroll
            for (int k = 0; k < NV; ++k) {
                const float4 v = xv[u][k];
                __nv_bfloat162 lo = __floats2bfloat162_rn(v.x * rr * wv[k].x, v.y * rr * wv[k].y);
                __nv_bfloat162 hi = __floats2bfloat162_rn(v.z * rr * wv[k].z, v.w * rr * wv[k].w);
                uint2 pk;
                pk.x = *reinterpret_cast<uint32_t*>(&lo); pk.y = *reinterpret_cast<uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(Xs + r * KP + 4 * (lane + 32 * k)) = pk;
            }
        }
    }
}

// one slab of weights ([ncols][K + 8] bf16, rows padded like the tile) -> Ws: one bulk copy
__device__ __forceinline__ void begin_w_slab(bf16* Ws, int KP, const bf16* slab, int ncols, uint64_t* bar) {
    if (threadIdx.x == 0) {
        mbar_expect_tx(bar, (uint32_t)(ncols * KP * 2));
        bulk_load(Ws, slab, (uint32_t)(ncols * KP * 2), bar);
    }
}

// C[64][8 * NT] = Xs[64][K] * Ws[8 * NT][K]^T: warp w takes rows 16 * (w & 3) and half (w >> 2) of K; the halves land
// in Cs[2][64][16] and are added by the caller (half 0 + half 1).
template <int NT>
__device__ __forceinline__ void slab_product(const bf16* Xs, const bf16* Ws, int KP, int K, float* Cs) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int mt = warp & 3, kh = warp >> 2;
    const int ksteps = K >> 4, kper = ksteps >> 1;
    float acc[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) { acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.0f; }
    const bf16* arow = Xs + (mt * 16 + (lane & 15)) * KP + (lane >> 4) * 8;
    const bf16* brow = Ws + (lane & 7) * KP + ((lane >> 3) & 1) * 8;
    for (int ks = kh * kper; ks < (kh + 1) * kper; ++ks) {
        uint32_t a[4];
        ldmatrix_x4(a, arow + ks * 16);
#pragma unroll
        for (int n = 0; n < NT; ++n) {
            uint32_t b[2];
            ldmatrix_x2(b, brow + n * 8 * KP + ks * 16);
            mma_bf16(acc[n], a, b);
        }
    }
    float* c = Cs + kh * (MEGA_ROWS * 16);
    const int r = mt * 16 + (lane >> 2), cc = (lane & 3) * 2;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        c[r * 16 + n * 8 + cc] = acc[n][0];
        c[r * 16 + n * 8 + cc + 1] = acc[n][1];
        c[(r + 8) * 16 + n * 8 + cc] = acc[n][2];
        c[(r + 8) * 16 + n * 8 + cc + 1] = acc[n][3];
    }
}

// ---- rotary embedding of the new q and k, cache append, attention over the cache ------------------------------
// The function of rope_attn_decode_kernel (the launch-per-kernel path) for up to three (sequence, head) pairs of a
// CTA at a time.  The cache rows of the pairs are brought into shared memory by TMA (64-row boxes, 128B swizzle):
// the keys of the first pairs are requested before the grid barrier in front of this phase (rows written by earlier
// steps do not depend on this one), the values while the softmax runs.  Scores and the weighted sum of the values are
// warp-level mma.sync products over those tiles -- as SIMT loops they took ~5,000 cycles each for 3 x 256 keys.
// The float32 operand of each product (q, then the exponentials) enters as a bf16 pair hi + lo in two columns / rows
// of the fragment, so the products keep float32 accuracy on that side (the cache rows are bf16 anyway).
constexpr int ATT_ITEMS = 3;
constexpr int KV_BOX_ROWS = 64;
constexpr int KV_BOX_BYTES = KV_BOX_ROWS * 128;

struct AttSmem {
    float* scratch;        // per pair: q [hd] | pr [cap rounded up to 16] | red [32] | vnew [hd] | e_hi, e_lo [cap16 bf16 each]
    uint8_t* tiles;        // [items][blocks][64 rows x 128 B] staged cache rows, 1024-byte aligned
    uint64_t* bar;         // staged rows have landed
    int items;             // pairs per round (1 .. ATT_ITEMS): what fits
    int blocks;            // boxes per pair: ceil(cap / 64)
};
__host__ __device__ inline int att_cap16(int cap) { return (cap + 15) & ~15; }
__host__ __device__ inline int att_per_floats(int hd, int cap) { return hd + att_cap16(cap) + 32 + hd + att_cap16(cap); }

// byte address of (row r, 16-byte piece j) of a pair's tile
__device__ __forceinline__ const uint8_t* tile_piece(const uint8_t* tile, int r, int j) {
    return tile + (r >> 6) * KV_BOX_BYTES + (r & 63) * 128 + ((j ^ (r & 7)) << 4);
}

// requests the boxes that hold rows [0, rows) of the keys (or values) of the pairs.  rows = position + 1 rounded up to
// 16: the products read whole 16-row tiles, so the rows behind the newest one must hold finite numbers (the cache
// is zero-filled at creation and only ever holds finite values; rows past its end are zero-filled by the copy)
__device__ __forceinline__ void begin_cache_tiles(const AttSmem& a, const CUtensorMap* map, const int* items, int n, int rows) {
    const int nblk = (rows + KV_BOX_ROWS - 1) / KV_BOX_ROWS;
    if (threadIdx.x == 0) mbar_expect_tx(a.bar, (uint32_t)(n * nblk * KV_BOX_BYTES));
    if ((int)threadIdx.x < n * nblk) {
        const int i = threadIdx.x / nblk, blk = threadIdx.x % nblk;
        tma_load_3d(a.tiles + ((size_t)i * a.blocks + blk) * KV_BOX_BYTES, map, a.bar, 0, blk * KV_BOX_ROWS, items[i]);
    }
}

__device__ __forceinline__ uint32_t pack_bf16(float x, float y) {
    __nv_bfloat162 v = __floats2bfloat162_rn(x, y);
    return *reinterpret_cast<uint32_t*>(&v);
}
// x = hi + lo with hi = bf16(x), lo = bf16(x - hi)
__device__ __forceinline__ void split_bf16(float x, float& hi, float& lo) {
    hi = __bfloat162float(__float2bfloat16_rn(x));
    lo = x - hi;
}

// returns false when a bounded wait gave up
__device__ bool attend_items(const MegaParams& p, const MegaLayer& ly, const int* items, int n, int t, const AttSmem& a,
                             bool keys_requested, uint32_t& parity, volatile int* abort_sh) {
    const int hd = p.hd, H = p.H, D = H * hd, half = hd >> 1;
    const int L = t + 1, L16 = (L + 15) & ~15;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int per = att_per_floats(hd, p.cap), cap16 = att_cap16(p.cap);
    float* sh = a.scratch;
    fence_proxy_async();                                     // (row t of the previous pairs' tiles was an ordinary store)
    __syncthreads();                                         // the scratch and tiles of the previous pairs are no longer read
    if (!keys_requested) begin_cache_tiles(a, ly.mapK, items, n, L16);
    // rotary embedding of the new q and k, new cache row: pair i on threads [i * half, (i + 1) * half)
    __nv_bfloat162 kn = __floats2bfloat162_rn(0.f, 0.f);
    {
        const int i = tid / half, k = tid % half;
        if (i < n) {
            const int sq = items[i] / H, h = items[i] % H;
            const float* row = p.qkv + (long long)sq * 3 * D + h * hd + 2 * k;
            const float c = p.cos_t[t * half + k], sn = p.sin_t[t * half + k];
            const float2 qq = __ldcg(reinterpret_cast<const float2*>(row));
            const float2 kk = __ldcg(reinterpret_cast<const float2*>(row + D));
            const float2 v = __ldcg(reinterpret_cast<const float2*>(row + 2 * D));
            float* q = sh + i * per;
            q[2 * k] = qq.x * c - qq.y * sn;
            q[2 * k + 1] = qq.x * sn + qq.y * c;
            const long long o = (long long)items[i] * p.cap * hd + (long long)t * hd + 2 * k;
            kn = __floats2bfloat162_rn(kk.x * c - kk.y * sn, kk.x * sn + kk.y * c);
            const __nv_bfloat162 vn = __floats2bfloat162_rn(v.x, v.y);
            *reinterpret_cast<__nv_bfloat162*>(ly.Kc + o) = kn;
            *reinterpret_cast<__nv_bfloat162*>(ly.Vc + o) = vn;
            *reinterpret_cast<__nv_bfloat162*>(sh + i * per + hd + cap16 + 32 + k) = vn;      // vnew, as bf16 pairs
        }
        // the weights behind the last key take part in the value product: zero
        for (int j = tid; j < n * 16; j += MEGA_THREADS) {
            const int ii = j >> 4, l = L16 - 16 + (j & 15);
            bf16* ehi = reinterpret_cast<bf16*>(sh + ii * per + hd + cap16 + 32 + hd);
            if (l >= L) { ehi[l] = __float2bfloat16_rn(0.0f); ehi[cap16 + l] = __float2bfloat16_rn(0.0f); }
        }
    }
    if (!mbar_wait(a.bar, parity, abort_sh)) return false;
    parity ^= 1u;
    // row t of the key tiles is this step's: written after the copy (whose box may cover it with the old contents)
    {
        const int i = tid / half, k = tid % half;
        if (i < n)
            *reinterpret_cast<__nv_bfloat162*>(const_cast<uint8_t*>(tile_piece(a.tiles + (size_t)i * a.blocks * KV_BOX_BYTES, t, k >> 2)) + (k & 3) * 4) = kn;
    }
    __syncthreads();
    // scores: s[l] = scale * <q, K[l]>, one mma tile = 16 keys; columns 0 | 1 of the B fragment hold q_hi | q_lo
    // (built once per pair: lanes 0-3 hold column 0, lanes 4-7 column 1, the other columns are zero)
    const int mtiles = L16 >> 4;
    uint32_t bq[ATT_ITEMS][4][2];
    {
        // every lane computes (without branches, so that the twelve short chains overlap); lanes 8-31 keep zeros
        const int k0 = (lane & 3) * 2;
#pragma unroll
        for (int i = 0; i < ATT_ITEMS; ++i) {
            const float* q = sh + (i < n ? i : 0) * per;
#pragma unroll
            for (int ks = 0; ks < 4; ++ks) {
                const int kk = ks < (hd >> 4) ? ks * 16 + k0 : k0;
                float h0, l0, h1, l1, h8, l8, h9, l9;
                split_bf16(q[kk], h0, l0); split_bf16(q[kk + 1], h1, l1);
                split_bf16(q[kk + 8], h8, l8); split_bf16(q[kk + 9], h9, l9);
                const uint32_t hi0 = pack_bf16(h0, h1), lo0 = pack_bf16(l0, l1);
                const uint32_t hi8 = pack_bf16(h8, h9), lo8 = pack_bf16(l8, l9);
                bq[i][ks][0] = lane < 4 ? hi0 : lane < 8 ? lo0 : 0u;
                bq[i][ks][1] = lane < 4 ? hi8 : lane < 8 ? lo8 : 0u;
            }
        }
    }
    float mx[ATT_ITEMS];
#pragma unroll
    for (int i = 0; i < ATT_ITEMS; ++i) mx[i] = -3.0e38f;
    // the pairs of a key tile are worked on together: their products are independent chains
    for (int mt = warp; mt < mtiles; mt += MEGA_THREADS / 32) {
        float acc[ATT_ITEMS][4];
#pragma unroll
        for (int i = 0; i < ATT_ITEMS; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.0f; }
        const int r = mt * 16 + (lane & 15);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
            if (ks < (hd >> 4)) {
#pragma unroll
                for (int i = 0; i < ATT_ITEMS; ++i) {
                    if (i < n) {
                        uint32_t af[4];
                        ldmatrix_x4(af, tile_piece(a.tiles + (size_t)i * a.blocks * KV_BOX_BYTES, r, ks * 2 + (lane >> 4)));
                        mma_bf16(acc[i], af, bq[i][ks]);
                    }
                }
            }
        }
        if ((lane & 3) == 0) {
            const int r0 = mt * 16 + (lane >> 2), r1 = r0 + 8;
#pragma unroll
            for (int i = 0; i < ATT_ITEMS; ++i) {
                if (i < n) {
                    const float s0 = (acc[i][0] + acc[i][1]) * p.scale, s1 = (acc[i][2] + acc[i][3]) * p.scale;
                    if (r0 < L) { sh[i * per + hd + r0] = s0; mx[i] = fmaxf(mx[i], s0); }
                    if (r1 < L) { sh[i * per + hd + r1] = s1; mx[i] = fmaxf(mx[i], s1); }
                }
            }
        }
    }
    // block maxima of the pairs
#pragma unroll
    for (int i = 0; i < ATT_ITEMS; ++i) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], o));
        if (lane == 0) sh[i * per + hd + cap16 + warp] = mx[i];
    }
    fence_proxy_async();
    __syncthreads();                                         // every key tile has been read
    // the values take the place of the keys while the softmax runs
    begin_cache_tiles(a, ly.mapV, items, n, L16);
    float sum[ATT_ITEMS];
#pragma unroll
    for (int i = 0; i < ATT_ITEMS; ++i) {
        const float* red = sh + i * per + hd + cap16;
        float m = red[0];
        for (int w = 1; w < MEGA_THREADS / 32; ++w) m = fmaxf(m, red[w]);
        mx[i] = m;
        sum[i] = 0.0f;
    }
    for (int l = tid; l < L; l += MEGA_THREADS) {
#pragma unroll
        for (int i = 0; i < ATT_ITEMS; ++i) {
            if (i < n) {
                const float e = expf(sh[i * per + hd + l] - mx[i]);
                sum[i] += e;
                float eh, el;
                split_bf16(e, eh, el);
                bf16* ehi = reinterpret_cast<bf16*>(sh + i * per + hd + cap16 + 32 + hd);
                ehi[l] = __float2bfloat16_rn(eh);
                ehi[cap16 + l] = __float2bfloat16_rn(el);
            }
        }
    }
#pragma unroll
    for (int i = 0; i < ATT_ITEMS; ++i) {
        sum[i] = warp_sum_f(sum[i]);
        if (lane == 0) sh[i * per + hd + cap16 + 16 + warp] = sum[i];
    }
    if (!mbar_wait(a.bar, parity, abort_sh)) return false;
    parity ^= 1u;
    {
        const int i = tid / half, k = tid % half;
        if (i < n)
            *reinterpret_cast<__nv_bfloat162*>(const_cast<uint8_t*>(tile_piece(a.tiles + (size_t)i * a.blocks * KV_BOX_BYTES, t, k >> 2)) + (k & 3) * 4) =
                *reinterpret_cast<const __nv_bfloat162*>(sh + i * per + hd + cap16 + 32 + k);
    }
    __syncthreads();
    // out[d] = sum_l e[l] V[l][d] / sum_l e[l] as out^T = V^T e: the A fragment (16 head-dim columns x 16 keys) comes
    // transposed out of the row-major value tile, columns 0 | 1 of the B fragment hold e_hi | e_lo.  (With e as the A
    // operand only 2 of its 16 rows would be used and twice as many mma were needed; an mma.sync costs a warp ~100
    // cycles here.)  The warps split the keys; their partial sums are added in warp order.
    const int dtiles = hd >> 4;
    {
        float acc[ATT_ITEMS][4][4];
#pragma unroll
        for (int i = 0; i < ATT_ITEMS; ++i)
#pragma unroll
            for (int m = 0; m < 4; ++m) { acc[i][m][0] = acc[i][m][1] = acc[i][m][2] = acc[i][m][3] = 0.0f; }
        for (int kt = warp; kt < mtiles; kt += MEGA_THREADS / 32) {
            const int k0 = kt * 16 + (lane & 3) * 2;
            const int key = kt * 16 + ((lane >> 4) << 3) + (lane & 7);
#pragma unroll
            for (int i = 0; i < ATT_ITEMS; ++i) {
                if (i < n) {
                    const uint8_t* tile = a.tiles + (size_t)i * a.blocks * KV_BOX_BYTES;
                    const bf16* ew = reinterpret_cast<const bf16*>(sh + i * per + hd + cap16 + 32 + hd) + (lane >= 4 ? cap16 : 0);
                    uint32_t be[2] = {0u, 0u};
                    if (lane < 8) {
                        be[0] = *reinterpret_cast<const uint32_t*>(ew + k0);
                        be[1] = *reinterpret_cast<const uint32_t*>(ew + k0 + 8);
                    }
#pragma unroll
                    for (int m = 0; m < 4; ++m) {
                        if (m < dtiles) {
                            uint32_t av[4];
                            asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                                         : "=r"(av[0]), "=r"(av[1]), "=r"(av[2]), "=r"(av[3])
                                         : "r"(smem_u32(tile_piece(tile, key, m * 2 + ((lane >> 3) & 1)))));
                            mma_bf16(acc[i][m], av, be);
                        }
                    }
                }
            }
        }
        // partial sums of this warp
        float* part = sh + ATT_ITEMS * per;                   // [8 warps][ATT_ITEMS][hd], behind the pairs' scratch
        if ((lane & 3) == 0) {
#pragma unroll
            for (int i = 0; i < ATT_ITEMS; ++i)
#pragma unroll
                for (int m = 0; m < 4; ++m)
                    if (i < n && m < dtiles) {
                        float* dst = part + (warp * ATT_ITEMS + i) * hd + m * 16 + (lane >> 2);
                        dst[0] = acc[i][m][0] + acc[i][m][1];
                        dst[8] = acc[i][m][2] + acc[i][m][3];
                    }
        }
    }
    __syncthreads();
    {
        const int i = tid / hd, d = tid % hd;
        if (i < n) {
            const float* red = sh + i * per + hd + cap16 + 16;
            float tot = red[0];
            for (int w = 1; w < MEGA_THREADS / 32; ++w) tot += red[w];
            const float* part = sh + ATT_ITEMS * per;
            float o = part[i * hd + d];
            for (int w = 1; w < MEGA_THREADS / 32; ++w) o += part[(w * ATT_ITEMS + i) * hd + d];
            const int sq = items[i] / H, h = items[i] % H;
            p.att[(long long)sq * (D + 8) + h * hd + d] = __float2bfloat16_rn(o / tot);
        }
    }
    return true;
}

// ---- the kernel ----------------------------------------------------------------------------------------------
// Shared memory: Ws [16][Kmax + 8] bf16 | Cs [2][64][16] float | flag | X region.  The X region holds the operand tile
// [64][K + 8] bf16 of the phase (K = D or F), behind it (RMSNorm phases) the float32 rows on their way in, or the
// scratch of the attention phase.
__host__ __device__ inline size_t mega_fixed_bytes(int D, int F) {
    const int kmax = D > F ? D : F;
    return (size_t)16 * (kmax + 8) * 2 + 2 * MEGA_ROWS * 16 * 4 + 48;       // Ws | Cs | flag, three mbarriers
}
__host__ __device__ inline size_t att_scratch_bytes(int hd, int cap) {
    return ((size_t)ATT_ITEMS * att_per_floats(hd, cap) + (size_t)(MEGA_THREADS / 32) * ATT_ITEMS * hd) * 4;    // + value partials
}
__host__ __device__ inline int att_blocks(int cap) { return (att_cap16(cap) + KV_BOX_ROWS - 1) / KV_BOX_ROWS; }
__host__ __device__ inline size_t mega_gemm_region_bytes(int D, int F) {
    const size_t tile_f = (size_t)MEGA_ROWS * (F + 8) * 2;
    const size_t norm = (size_t)MEGA_ROWS * (D + 8) * 2 + (size_t)MEGA_ROWS * D * 4;
    return tile_f > norm ? tile_f : norm;
}
// (sequence, head) pairs whose cache tiles fit beside the scratch (0: none -- the kernel is not used).  The tiles
// start on a 1024-byte boundary, so a kilobyte of slack is counted.
__host__ __device__ inline int mega_att_items(int D, int F, int hd, int cap) {
    const size_t budget = 225 * 1024 - mega_fixed_bytes(D, F);
    const size_t need0 = att_scratch_bytes(hd, cap) + 1024;
    if (need0 >= budget) return 0;
    const size_t n = (budget - need0) / ((size_t)att_blocks(cap) * KV_BOX_BYTES);
    return n > ATT_ITEMS ? ATT_ITEMS : (int)n;
}
__host__ __device__ inline size_t mega_x_region_bytes(int D, int F, int hd, int cap) {
    const size_t att = att_scratch_bytes(hd, cap) + 1024 + (size_t)mega_att_items(D, F, hd, cap) * att_blocks(cap) * KV_BOX_BYTES;
    const size_t m = mega_gemm_region_bytes(D, F);
    return m > att ? m : att;
}
__host__ __device__ inline size_t mega_smem_bytes(int D, int F, int hd, int cap) {
    return mega_fixed_bytes(D, F) + mega_x_region_bytes(D, F, hd, cap);
}

template <int NV>
__global__ void __launch_bounds__(MEGA_THREADS, 1) decode_layers_kernel(const MegaParams p) {
    extern __shared__ __align__(16) uint8_t smem_raw[];
    const int D = p.D, F = p.F, S = p.S;
    const int kmax = D > F ? D : F;
    const int KD = D + 8, KF = F + 8;                  // padded rows of the operand tiles (conflict-free ldmatrix)
    bf16* Ws = reinterpret_cast<bf16*>(smem_raw);                                  // [16][K + 8] of the phase
    float* Cs = reinterpret_cast<float*>(smem_raw + (size_t)16 * (kmax + 8) * 2);    // [2][64][16]
    int* sh_flag = reinterpret_cast<int*>(Cs + 2 * MEGA_ROWS * 16);
    uint64_t* bar_x = reinterpret_cast<uint64_t*>(sh_flag + 4);                    // activation rows have landed
    uint64_t* bar_w = bar_x + 1;                                                   // weight slab has landed
    bf16* Xs = reinterpret_cast<bf16*>(bar_x + 4);
    float* stage = reinterpret_cast<float*>(Xs + MEGA_ROWS * KD);                  // float32 rows of the RMSNorm phases
    AttSmem att;                                                                   // the attention phase reuses the X region
    att.scratch = reinterpret_cast<float*>(Xs);
    {
        const uint32_t after = smem_u32(Xs) + (uint32_t)att_scratch_bytes(p.hd, p.cap);
        att.tiles = reinterpret_cast<uint8_t*>(Xs) + att_scratch_bytes(p.hd, p.cap) + ((1024u - (after & 1023u)) & 1023u);
    }
    att.bar = bar_x + 2;
    att.items = mega_att_items(D, F, p.hd, p.cap);
    att.blocks = att_blocks(p.cap);
    volatile int* abort_sh = sh_flag + 1;
    const int tid = threadIdx.x;
    const int cta = blockIdx.x, ncta = gridDim.x;
    const int t = *p.pos;
    int nbar = 0;
    uint32_t px = 0, pw = 0, pk = 0;                   // parities of the next completion of bar_x, bar_w, att.bar

    if (tid == 0) { mbar_init(bar_x, 1); mbar_init(bar_w, 1); mbar_init(att.bar, 1); *abort_sh = 0; fence_mbar_init(); }
    __syncthreads();

    const int slabs_qkv = 3 * D / 8, slabs_o = D / 8, slabs_gu = F / 8, slabs_down = D / 8;
    // a bounded wait gave up: record it and leave (the other CTAs follow at their next grid barrier)
#define MEGA_WAIT(bar, parity)                                                   \
    do {                                                                         \
        if (!mbar_wait(bar, parity, abort_sh)) { atomicCAS(p.err, 0, 42); *abort_sh = 1; return; } \
        parity ^= 1u;                                                            \
    } while (0)

    // weights of the first phase
    if (cta < slabs_qkv) begin_w_slab(Ws, KD, p.layers[0].wqkv + (long long)cta * 8 * KD, 8, bar_w);

    for (int l = 0; l < p.L; ++l) {
        const MegaLayer ly = p.layers[l];
        // ------------------------------------------------------------- RMSNorm + QKV projection
        if (cta < slabs_qkv) {
            begin_x_f32(stage, p, p.x, l == 0, bar_x);
            // (what the epilogue of this CTA's first slab adds is requested now: thread = column c of rows r0, r0 + 32)
            const float pre_b = __ldg(ly.bqkv + cta * 8 + (tid & 7));
            MEGA_WAIT(bar_x, px);
            norm_staged<NV>(Xs, KD, stage, p, ly.attn_norm);
            for (int slab = cta; slab < slabs_qkv; slab += ncta) {
                if (slab != cta) { __syncthreads(); begin_w_slab(Ws, KD, ly.wqkv + (long long)slab * 8 * KD, 8, bar_w); }
                MEGA_WAIT(bar_w, pw);
                __syncthreads();
                slab_product<1>(Xs, Ws, KD, D, Cs);
                __syncthreads();
                for (int i = tid; i < MEGA_ROWS * 8; i += MEGA_THREADS) {
                    const int r = i >> 3, c = i & 7, col = slab * 8 + c;
                    if (r < S) p.qkv[(long long)r * 3 * D + col] = Cs[r * 16 + c] + Cs[MEGA_ROWS * 16 + r * 16 + c] + (slab == cta ? pre_b : __ldg(ly.bqkv + col));
                }
            }
            __syncthreads();
        }
        if (cta < slabs_o) begin_w_slab(Ws, KD, ly.wo + (long long)cta * 8 * KD, 8, bar_w);       // for the phase after next
        // the keys of this CTA's first (sequence, head) pairs: rows of earlier steps can come in during the barrier
        int items0[ATT_ITEMS];
        int n0 = 0;
#pragma unroll
        for (int i = 0; i < ATT_ITEMS; ++i) {
            items0[i] = cta + i * ncta;
            if (i < att.items && items0[i] < S * p.H) n0 = i + 1;
        }
        if (n0 > 0) {
            fence_proxy_async();                      // this phase's ordinary stores into the region come first
            __syncthreads();
            begin_cache_tiles(att, ly.mapK, items0, n0, (t + 16) & ~15);
        }
        if (!grid_barrier(p, nbar++, sh_flag)) return;
        // ------------------------------------------------------------- rotary + cache append + attention
        // (the out-projection weights requested above land in Ws, which this phase leaves alone)
        for (int first = cta; first < S * p.H; first += att.items * ncta) {
            int items[ATT_ITEMS];
            int n = 0;
#pragma unroll
            for (int i = 0; i < ATT_ITEMS; ++i) {
                items[i] = first + i * ncta;
                if (i < att.items && items[i] < S * p.H) n = i + 1;
            }
            if (!attend_items(p, ly, items, n, t, att, first == cta, pk, abort_sh)) { atomicCAS(p.err, 0, 43); *abort_sh = 1; return; }
        }
        if (!grid_barrier(p, nbar++, sh_flag)) return;
        // ------------------------------------------------------------- out-projection + residual -> x2
        if (cta < slabs_o) {
            begin_x_bf16(Xs, KD, p.att, bar_x);
            const int pc = cta * 8 + (tid & 7), pr0 = tid >> 3;
            const float pre_b = __ldg(ly.bo + pc);
            float pre_r[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int r = pr0 + 32 * u;
                pre_r[u] = r < S ? (l == 0 ? __ldg(p.embed + (long long)p.tok[r] * D + pc) : __ldcg(p.x + (long long)r * D + pc)) : 0.0f;
            }
            MEGA_WAIT(bar_x, px);
            for (int slab = cta; slab < slabs_o; slab += ncta) {
                if (slab != cta) { __syncthreads(); begin_w_slab(Ws, KD, ly.wo + (long long)slab * 8 * KD, 8, bar_w); }
                MEGA_WAIT(bar_w, pw);
                __syncthreads();
                slab_product<1>(Xs, Ws, KD, D, Cs);
                __syncthreads();
                for (int i = tid; i < MEGA_ROWS * 8; i += MEGA_THREADS) {
                    const int r = i >> 3, c = i & 7, col = slab * 8 + c;
                    if (r < S) {
                        const bool pre = slab == cta;
                        const float res = pre ? (i >= MEGA_THREADS ? pre_r[1] : pre_r[0])
                                              : (l == 0 ? __ldg(p.embed + (long long)p.tok[r] * D + col) : __ldcg(p.x + (long long)r * D + col));
                        p.x2[(long long)r * D + col] = Cs[r * 16 + c] + Cs[MEGA_ROWS * 16 + r * 16 + c] + (pre ? pre_b : __ldg(ly.bo + col)) + res;
                    }
                }
            }
            __syncthreads();
        }
        if (cta < slabs_gu) begin_w_slab(Ws, KD, ly.wgu + (long long)cta * 16 * KD, 16, bar_w);
        if (!grid_barrier(p, nbar++, sh_flag)) return;
        // ------------------------------------------------------------- RMSNorm + gate|up projection + SwiGLU -> h
        if (cta < slabs_gu) {
            begin_x_f32(stage, p, p.x2, false, bar_x);
            const float pre_bg = __ldg(ly.bgu + cta * 8 + (tid & 7)), pre_bu = __ldg(ly.bgu + F + cta * 8 + (tid & 7));
            MEGA_WAIT(bar_x, px);
            norm_staged<NV>(Xs, KD, stage, p, ly.ffn_norm);
            for (int slab = cta; slab < slabs_gu; slab += ncta) {
                if (slab != cta) { __syncthreads(); begin_w_slab(Ws, KD, ly.wgu + (long long)slab * 16 * KD, 16, bar_w); }
                MEGA_WAIT(bar_w, pw);
                __syncthreads();
                slab_product<2>(Xs, Ws, KD, D, Cs);
                __syncthreads();
                for (int i = tid; i < MEGA_ROWS * 8; i += MEGA_THREADS) {
                    const int r = i >> 3, c = i & 7, col = slab * 8 + c;
                    if (r < S) {
                        const float gv = Cs[r * 16 + c] + Cs[MEGA_ROWS * 16 + r * 16 + c] + (slab == cta ? pre_bg : __ldg(ly.bgu + col));
                        const float uv = Cs[r * 16 + 8 + c] + Cs[MEGA_ROWS * 16 + r * 16 + 8 + c] + (slab == cta ? pre_bu : __ldg(ly.bgu + F + col));
                        const float sg = __fdividef(1.0f, 1.0f + ex2_approx(-gv * 1.4426950408889634f));
                        p.h[(long long)r * KF + col] = __float2bfloat16_rn(gv * sg * uv);
                    }
                }
            }
            __syncthreads();
        }
        if (cta < slabs_down) begin_w_slab(Ws, KF, ly.wdown + (long long)cta * 8 * KF, 8, bar_w);
        if (!grid_barrier(p, nbar++, sh_flag)) return;
        // ------------------------------------------------------------- down-projection + residual -> x
        if (cta < slabs_down) {
            begin_x_bf16(Xs, KF, p.h, bar_x);
            const int pc = cta * 8 + (tid & 7), pr0 = tid >> 3;
            const float pre_b = __ldg(ly.bdown + pc);
            float pre_r[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) pre_r[u] = pr0 + 32 * u < S ? __ldcg(p.x2 + (long long)(pr0 + 32 * u) * D + pc) : 0.0f;
            MEGA_WAIT(bar_x, px);
            for (int slab = cta; slab < slabs_down; slab += ncta) {
                if (slab != cta) { __syncthreads(); begin_w_slab(Ws, KF, ly.wdown + (long long)slab * 8 * KF, 8, bar_w); }
                MEGA_WAIT(bar_w, pw);
                __syncthreads();
                slab_product<1>(Xs, Ws, KF, F, Cs);
                __syncthreads();
                for (int i = tid; i < MEGA_ROWS * 8; i += MEGA_THREADS) {
                    const int r = i >> 3, c = i & 7, col = slab * 8 + c;
                    if (r < S) {
                        const bool pre = slab == cta;
                        p.x[(long long)r * D + col] = Cs[r * 16 + c] + Cs[MEGA_ROWS * 16 + r * 16 + c] + (pre ? pre_b : __ldg(ly.bdown + col)) +
                                                      (pre ? (i >= MEGA_THREADS ? pre_r[1] : pre_r[0]) : __ldcg(p.x2 + (long long)r * D + col));
                    }
                }
            }
            __syncthreads();
        }
        if (l + 1 < p.L) {
            if (cta < slabs_qkv) begin_w_slab(Ws, KD, p.layers[l + 1].wqkv + (long long)cta * 8 * KD, 8, bar_w);
            if (!grid_barrier(p, nbar++, sh_flag)) return;
        }
    }
#undef MEGA_WAIT
}

// W [K][N] (row-major bf16) -> slabs [N/8][8][K + 8] (8 zero columns behind every row); pair_off > 0: slabs of 16 rows,
// columns 8j.. then pair_off + 8j..
__global__ void slab_layout_kernel(const bf16* __restrict__ W, bf16* __restrict__ out, int K, int N, int pair_off) {
    const int rows_per = pair_off > 0 ? 16 : 8;
    const int nslab = (pair_off > 0 ? pair_off : N) / 8;
    const int KP = K + 8;
    const long long total = (long long)nslab * rows_per * KP;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int k = (int)(i % KP);
        const int r = (int)((i / KP) % rows_per);
        const int slab = (int)(i / ((long long)KP * rows_per));
        const int col = r < 8 ? slab * 8 + r : pair_off + slab * 8 + (r - 8);
        out[i] = k < K ? W[(long long)k * N + col] : __float2bfloat16_rn(0.0f);
    }
}

}  // namespace

struct DecodeMega {
    MegaParams p;
    MegaLayer* d_layers = nullptr;
    bf16* wt = nullptr;
    bf16 *att = nullptr, *h = nullptr;         // [64][D + 8], [64][F + 8]
    CUtensorMap* d_maps = nullptr;             // [L][2]: K and V cache views
    unsigned int* barrier = nullptr;
    size_t smem = 0;
    int grid = 0, nv = 0;
};

bool decode_mega_supported(const DeviceCtx* ctx, int S, int D, int H, int F, int cap) {
    const int hd = H > 0 ? D / H : 0;
    if (S < 1 || S > MEGA_ROWS || D % 128 != 0 || D > 1024 || F % 32 != 0 || F > 1024) return false;
    if (hd < 16 || hd > 64 || hd % 16 != 0) return false;                       // k-steps of 16 head-dim columns
    if (MEGA_THREADS / hd < ATT_ITEMS) return false;                            // thread ranges of the pairs
    if (mega_att_items(D, F, hd, cap) < 1 || ATT_ITEMS * att_blocks(cap) > MEGA_THREADS) return false;
    return mega_smem_bytes(D, F, hd, cap) <= 225 * 1024 && ctx->sm_count >= 8;
}

size_t decode_mega_weight_scalars(int D, int F, int L) {
    return (size_t)L * ((size_t)(D + 8) * 3 * D + (size_t)(D + 8) * D + (size_t)(D + 8) * 2 * F + (size_t)(F + 8) * D);
}

int decode_mega_create(DeviceCtx* ctx, DecodeMega** out, int S, int D, int H, int F, int L, int cap, float eps, float scale) {
    DecodeMega* m = new DecodeMega();
    std::memset(&m->p, 0, sizeof(m->p));
    m->p.S = S; m->p.D = D; m->p.H = H; m->p.hd = D / H; m->p.F = F; m->p.L = L; m->p.cap = cap; m->p.eps = eps; m->p.scale = scale;
    m->p.err = ctx->d_err;
    m->smem = mega_smem_bytes(D, F, D / H, cap);
    m->nv = D / 128;
    m->grid = ctx->sm_count;
    TB_CUDA(cudaMalloc(&m->d_layers, sizeof(MegaLayer) * (size_t)(L > 0 ? L : 1)));
    TB_CUDA(cudaMalloc(&m->wt, decode_mega_weight_scalars(D, F, L > 0 ? L : 1) * sizeof(bf16)));
    TB_CUDA(cudaMalloc(&m->barrier, 256));
    TB_CUDA(cudaMemset(m->barrier, 0, 256));
    TB_CUDA(cudaMalloc(&m->d_maps, sizeof(CUtensorMap) * 2 * (size_t)(L > 0 ? L : 1)));
    TB_CUDA(cudaMalloc(&m->att, (size_t)MEGA_ROWS * (D + 8) * sizeof(bf16)));
    TB_CUDA(cudaMemset(m->att, 0, (size_t)MEGA_ROWS * (D + 8) * sizeof(bf16)));
    TB_CUDA(cudaMalloc(&m->h, (size_t)MEGA_ROWS * (F + 8) * sizeof(bf16)));
    TB_CUDA(cudaMemset(m->h, 0, (size_t)MEGA_ROWS * (F + 8) * sizeof(bf16)));
    m->p.layers = m->d_layers;
    m->p.barrier = m->barrier;
    *out = m;
    return 0;
}

void decode_mega_destroy(DecodeMega* m) {
    if (!m) return;
    cudaFree(m->d_layers); cudaFree(m->wt); cudaFree(m->barrier); cudaFree(m->att); cudaFree(m->h); cudaFree(m->d_maps);
    delete m;
}

// (Re)builds the slab copies of the weights and the per-layer pointer table; call after every weight upload.
int decode_mega_set_weights(DeviceCtx* ctx, DecodeMega* m, const float* params, const bf16* params16, const long long* offsets,
                            bf16* const* Kc, bf16* const* Vc, cudaStream_t st) {
    const int D = m->p.D, F = m->p.F, L = m->p.L;
    std::vector<MegaLayer> hl((size_t)(L > 0 ? L : 1));
    std::vector<CUtensorMap> hmaps(2 * (size_t)(L > 0 ? L : 1));
    bf16* w = m->wt;
    for (int l = 0; l < L; ++l) {
        const long long* o = offsets + 1 + 10LL * l;
        MegaLayer& y = hl[l];
        y.attn_norm = params + o[0]; y.bqkv = params + o[2]; y.bo = params + o[4]; y.ffn_norm = params + o[5];
        y.bgu = params + o[7]; y.bdown = params + o[9];
        y.Kc = Kc[l]; y.Vc = Vc[l];
        TB_TRY(make_operand_map(&hmaps[2 * l], Kc[l], m->p.hd, m->p.cap, m->p.hd, m->p.S * m->p.H, (long long)m->p.cap * m->p.hd, KV_BOX_ROWS));
        TB_TRY(make_operand_map(&hmaps[2 * l + 1], Vc[l], m->p.hd, m->p.cap, m->p.hd, m->p.S * m->p.H, (long long)m->p.cap * m->p.hd, KV_BOX_ROWS));
        y.mapK = m->d_maps + 2 * l; y.mapV = m->d_maps + 2 * l + 1;
        auto relayout = [&](const bf16* src, int K, int N, int pair_off, const bf16** dst) -> int {
            const long long total = (long long)(K + 8) * N;
            int blocks = (int)((total + 255) / 256);
            if (blocks > 16 * ctx->sm_count) blocks = 16 * ctx->sm_count;
            slab_layout_kernel<<<blocks, 256, 0, st>>>(src, w, K, N, pair_off);
            TB_CUDA(cudaGetLastError());
            *dst = w;
            w += total;
            return 0;
        };
        TB_TRY(relayout(params16 + o[1], D, 3 * D, 0, &y.wqkv));
        TB_TRY(relayout(params16 + o[3], D, D, 0, &y.wo));
        TB_TRY(relayout(params16 + o[6], D, 2 * F, F, &y.wgu));
        TB_TRY(relayout(params16 + o[8], F, D, 0, &y.wdown));
    }
    TB_CUDA(cudaMemcpyAsync(m->d_maps, hmaps.data(), sizeof(CUtensorMap) * hmaps.size(), cudaMemcpyHostToDevice, st));
    TB_CUDA(cudaMemcpyAsync(m->d_layers, hl.data(), sizeof(MegaLayer) * hl.size(), cudaMemcpyHostToDevice, st));
    TB_CUDA(cudaStreamSynchronize(st));          // hl goes out of scope
    m->p.embed = params;
    return 0;
}

int launch_decode_mega(DeviceCtx* ctx, DecodeMega* m, const uint32_t* tok, const int* pos, const float* cos_t, const float* sin_t,
                       float* x, float* x2, float* qkv, bf16* att, bf16* h, cudaStream_t st) {
    MegaParams p = m->p;
    p.tok = tok; p.pos = pos; p.cos_t = cos_t; p.sin_t = sin_t; p.x = x; p.x2 = x2; p.qkv = qkv; p.att = m->att; p.h = m->h;
    TB_CUDA(cudaMemsetAsync(m->barrier, 0, sizeof(unsigned int), st));
    void (*kernel)(const MegaParams) = nullptr;
    switch (m->nv) {
        case 1: kernel = decode_layers_kernel<1>; break;
        case 2: kernel = decode_layers_kernel<2>; break;
        case 3: kernel = decode_layers_kernel<3>; break;
        case 4: kernel = decode_layers_kernel<4>; break;
        case 5: kernel = decode_layers_kernel<5>; break;
        case 6: kernel = decode_layers_kernel<6>; break;
        case 7: kernel = decode_layers_kernel<7>; break;
        default: kernel = decode_layers_kernel<8>; break;
    }
    static bool attr_set[64][9] = {};
    if (!attr_set[ctx->device & 63][m->nv]) {
        TB_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)m->smem));
        int per_sm = 0;
        TB_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, MEGA_THREADS, m->smem));
        TB_CHECK(per_sm >= 1, "the decode-step kernel does not fit an SM (%zu bytes of shared memory)", m->smem);
        attr_set[ctx->device & 63][m->nv] = true;
    }
    // a cooperative launch: the CTAs wait for one another at the grid barriers, so all of them must be resident
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(m->grid); cfg.blockDim = dim3(MEGA_THREADS); cfg.dynamicSmemBytes = m->smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    prof_mark(ctx, "decode_layers", 0.0, 0.0, st);
    TB_CUDA(cudaLaunchKernelEx(&cfg, kernel, p));
    ctx->launches++;
    prof_close(ctx, st);
    return 0;
}

}  // namespace tb

