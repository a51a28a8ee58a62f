// The GEMM family under the reference's own kernel names and parameter lists, for the reference's Driver-API
// loader: compiled to an sm_100a cubin (nvcc -cubin), the image loads through the reference's unmodified
// cuda_init / cuda_get_kernel / cuda_launch (cuda/cuda_backend.c:36-107,150-153), and every entry accepts the launch
// geometry the reference's host helpers use (model/gpu_train.c:45-118, cuda/cuda_backend.c:141-148):
//
//   k_matmul(A, B, C, M, K, N)                                  grid (ceil(N/16), ceil(M/16)), block 16 x 16   (cuda/kernels.cu:35)
//   k_gemm_{nn,nt,tn}(A, B, C, M, N, K, lda, ldb, ldc, strideA, strideB, strideC, alpha, beta)
//                                                               grid (ceil(N/64), ceil(M/64), batch), block 16 x 16   (cuda/train_kernels.cu:187-193)
//   k_bf16_gemm_{nn,nt,tn,tn_small}(same list)                  grid (ceil(N/64), ceil(M/64), batch), block 256       (:464-467)
//   k_bf16_gemm_nn_bias(A, B, bias, residual, C, M, N, K)       grid (ceil(N/64), ceil(M/64)), block 256              (:226-228)
//
// These signatures pass raw float32 pointers with arbitrary leading dimensions and no tensor maps, and the host
// launches 256 threads with no dynamic shared memory, so this is the non-TMA form of the kernel: the CTA's threads
// load float32 tiles with ordinary global loads (the next K slice travels in registers while the tensor core works on
// the current one), round them to bf16 (round-to-nearest-even, the reference's f32_to_bf16, cuda/train_kernels.cu:207-212)
// or keep them as tf32 for the k_gemm_* entries (float32 SIMT kernels in the reference), write them into shared memory
// in the K-major 128-byte-swizzle layout, and one thread issues tcgen05.mma on a 128 x 64 accumulator in TMEM.
// The reference's grid has one CTA per 64 x 64 (16 x 16 for k_matmul) output block: the CTA whose block is the
// top-left corner of a 128 x 64 tile computes the whole tile, the others return at once.
//
// The TMA-fed persistent kernel of this library (gemm_tcgen05.cu) needs host-built CUtensorMap parameters and its own
// grid, which the reference's launch helpers cannot supply; it is reached through the C ABI instead (turkce_b200.h).
#include "../ptx.cuh"

#include <cuda_bf16.h>

namespace tbk {

using namespace tb;

constexpr int TM = 128;             // output rows per working CTA
constexpr int TN = 64;              // output columns per working CTA

// 1 after a launch in which a wait on the tensor core ran out (readable with cuModuleGetGlobal); never reset here.
__device__ int tb_gemm_status;

struct Operand { const float* p; long long rs, ks; };     // element (row, k) at p[row * rs + k * ks]

// One thread's share of a K slice: NV consecutive k of one tile row, converted and stored as 16-byte chunks of the
// row's 128-byte line; chunk c of row r lives at r * 128 + ((c ^ (r & 7)) << 4)  (the 128-byte swizzle).
template <int NV, bool TF32>
struct Share {
    float v[NV];
    __device__ __forceinline__ void load(const Operand& o, int row, int rows_valid, int k, int k_valid, bool vec) {
        if (row >= rows_valid) {
#pragma unroll
            for (int j = 0; j < NV; ++j) v[j] = 0.0f;
            return;
        }
        const float* src = o.p + (long long)row * o.rs + (long long)k * o.ks;
        if (vec && k + NV <= k_valid) {          // k is the contiguous direction and the run is 16-byte addressable
#pragma unroll
            for (int j = 0; j < NV; j += 4) {
                const float4 f = __ldg(reinterpret_cast<const float4*>(src + j));
                v[j] = f.x; v[j + 1] = f.y; v[j + 2] = f.z; v[j + 3] = f.w;
            }
        } else {
#pragma unroll
            for (int j = 0; j < NV; ++j) v[j] = k + j < k_valid ? __ldg(src + (long long)j * o.ks) : 0.0f;
        }
    }
    // first_chunk: index of this share's first 16-byte chunk inside the row
    __device__ __forceinline__ void store(uint8_t* tile, int row, int first_chunk) const {
        uint8_t* line = tile + row * 128;
        if (TF32) {
#pragma unroll
            for (int c = 0; c < NV / 4; ++c)
                *reinterpret_cast<float4*>(line + (((first_chunk + c) ^ (row & 7)) << 4)) =
                    make_float4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
        } else {
#pragma unroll
            for (int c = 0; c < NV / 8; ++c) {
                uint4 pk;
                __nv_bfloat162 h0 = __floats2bfloat162_rn(v[8 * c + 0], v[8 * c + 1]);
                __nv_bfloat162 h1 = __floats2bfloat162_rn(v[8 * c + 2], v[8 * c + 3]);
                __nv_bfloat162 h2 = __floats2bfloat162_rn(v[8 * c + 4], v[8 * c + 5]);
                __nv_bfloat162 h3 = __floats2bfloat162_rn(v[8 * c + 6], v[8 * c + 7]);
                pk.x = *reinterpret_cast<uint32_t*>(&h0); pk.y = *reinterpret_cast<uint32_t*>(&h1);
                pk.z = *reinterpret_cast<uint32_t*>(&h2); pk.w = *reinterpret_cast<uint32_t*>(&h3);
                *reinterpret_cast<uint4*>(line + (((first_chunk + c) ^ (row & 7)) << 4)) = pk;
            }
        }
    }
};

// C[z] = alpha * op(A[z]) op(B[z]) (+ bias[n]) (+ residual[m, n]) (+ beta * C[z]) on the tile whose top-left output
// block this CTA owns.  TA / TB: the operand is stored transposed (A as [K, M], B as [N, K]).  `unit`: output rows and
// columns per CTA of the caller's grid (64, or 16 for k_matmul).
template <int TA, int TB, bool TF32>
__device__ __forceinline__ void gemm_tile(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C,
                                          int M, int N, int K, long long lda, long long ldb, long long ldc,
                                          long long strideA, long long strideB, long long strideC, float alpha, float beta,
                                          const float* __restrict__ bias, const float* __restrict__ residual, int unit) {
    const int m0 = (int)blockIdx.y * unit, n0 = (int)blockIdx.x * unit;
    if ((m0 % TM) != 0 || (n0 % TN) != 0) return;       // another CTA's tile covers this block
    constexpr int BKE = TF32 ? 32 : 64;                   // elements per 128-byte K slice
    constexpr int NVA = BKE / 2, NVB = BKE / 4;           // values per thread and slice: A half a row, B a quarter
    __shared__ __align__(1024) uint8_t tiles[TM * 128 + TN * 128];
    __shared__ __align__(8) uint64_t mma_bar;
    __shared__ uint32_t tmem_slot;
    __shared__ int abort_flag;
    uint8_t* sA = tiles;
    uint8_t* sB = tiles + TM * 128;
    const int tid = (int)(threadIdx.y * blockDim.x + threadIdx.x);
    const int warp = tid >> 5, lane = tid & 31;
    const long long z = blockIdx.z;
    A += z * strideA; B += z * strideB; C += z * strideC;
    if (residual) residual += z * strideC;

    if (tid == 0) { mbar_init(&mma_bar, 1); abort_flag = 0; fence_mbar_init(); }
    if (warp == 0) { tmem_alloc(&tmem_slot, 64); tmem_relinquish(); }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = tmem_slot;

    // who loads what: a thread owns (row, part) of each operand tile; with k contiguous in memory neighbouring threads
    // take the parts of one row, with the row index contiguous they take neighbouring rows (coalesced either way)
    const Operand oa = TA ? Operand{A, 1, lda} : Operand{A, lda, 1};
    const Operand ob = TB ? Operand{B, ldb, 1} : Operand{B, 1, ldb};          // row of the B tile = output column n
    const int a_row = TA ? tid % TM : tid / 2, a_part = TA ? tid / TM : tid % 2;
    const int b_row = TB ? tid / 4 : tid % TN, b_part = TB ? tid % 4 : tid / TN;
    const bool a_vec = !TA && (lda % 4 == 0) && (strideA % 4 == 0) && ((reinterpret_cast<unsigned long long>(A) & 15ull) == 0);
    const bool b_vec = TB && (ldb % 4 == 0) && (strideB % 4 == 0) && ((reinterpret_cast<unsigned long long>(B) & 15ull) == 0);
    const int a_rows_valid = M - m0, b_rows_valid = N - n0;
    const Operand oa_t{oa.p + (long long)m0 * oa.rs, oa.rs, oa.ks};
    const Operand ob_t{ob.p + (long long)n0 * ob.rs, ob.rs, ob.ks};
    Share<NVA, TF32> ra;
    Share<NVB, TF32> rb;
    const int nk = (K + BKE - 1) / BKE;
    const uint32_t idesc = umma_idesc(TF32 ? 2u : 1u, 0u, 0u, TM, TN);
    ra.load(oa_t, a_row, a_rows_valid, a_part * NVA, K, a_vec);
    rb.load(ob_t, b_row, b_rows_valid, b_part * NVB, K, b_vec);
    bool ok = true;
    for (int kb = 0; kb < nk; ++kb) {
        if (kb > 0 && !mbar_wait(&mma_bar, (uint32_t)(kb - 1) & 1u, &abort_flag)) { ok = false; break; }   // slice kb-1 consumed
        ra.store(sA, a_row, a_part * (TF32 ? NVA / 4 : NVA / 8));
        rb.store(sB, b_row, b_part * (TF32 ? NVB / 4 : NVB / 8));
        fence_proxy_async();                 // the tensor core reads shared memory through the async proxy
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
            const uint32_t a_addr = smem_u32(sA), b_addr = smem_u32(sB);
#pragma unroll
            for (int k = 0; k < 4; ++k) {     // 32 bytes of K per UMMA (16 bf16 or 8 tf32)
                const uint64_t da = umma_desc_sw128(a_addr + k * 32, 16, 1024), db = umma_desc_sw128(b_addr + k * 32, 16, 1024);
                if (TF32) umma_tf32(tmem_base, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
                else      umma_bf16(tmem_base, da, db, idesc, (kb | k) != 0 ? 1u : 0u);
            }
            umma_commit(&mma_bar);
        }
        if (kb + 1 < nk) {                   // the next slice travels while the tensor core works
            const int k = (kb + 1) * BKE;
            ra.load(oa_t, a_row, a_rows_valid, k + a_part * NVA, K, a_vec);
            rb.load(ob_t, b_row, b_rows_valid, k + b_part * NVB, K, b_vec);
        }
    }
    if (ok && nk > 0 && !mbar_wait(&mma_bar, (uint32_t)(nk - 1) & 1u, &abort_flag)) ok = false;
    if (!ok) { abort_flag = 1; tb_gemm_status = 1; }
    tc_fence_after();

    // epilogue: warp w reads accumulator rows (w % 4) * 32 + lane, columns (w / 4) * 32 .. + 31
    if (ok) {
        const int row = m0 + (warp & 3) * 32 + lane;
        const int col0 = n0 + (warp >> 2) * 32;
        uint32_t acc[32];
        if (nk > 0) {
            tmem_ld32(tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)((warp >> 2) * 32), acc);
            tmem_ld_wait();
        } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) acc[j] = 0u;
        }
        if (row < M && col0 < N) {
            float* crow = C + (long long)row * ldc + col0;
            const float* rrow = residual ? residual + (long long)row * ldc + col0 : nullptr;
            const bool full = col0 + 32 <= N;
            const bool cvec = full && (ldc % 4 == 0) && (strideC % 4 == 0) && ((reinterpret_cast<unsigned long long>(C) & 15ull) == 0);
            float o[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) o[j] = alpha * __uint_as_float(acc[j]);
            if (bias) {
#pragma unroll
                for (int j = 0; j < 32; ++j) if (col0 + j < N) o[j] += __ldg(bias + col0 + j);
            }
            if (cvec) {
                const bool rvec = rrow && ((reinterpret_cast<unsigned long long>(residual) & 15ull) == 0);
#pragma unroll
                for (int j = 0; j < 32; j += 4) {
                    if (rrow) {
                        if (rvec) { const float4 r = __ldg(reinterpret_cast<const float4*>(rrow + j)); o[j] += r.x; o[j + 1] += r.y; o[j + 2] += r.z; o[j + 3] += r.w; }
                        else { o[j] += rrow[j]; o[j + 1] += rrow[j + 1]; o[j + 2] += rrow[j + 2]; o[j + 3] += rrow[j + 3]; }
                    }
                    if (beta != 0.0f) {
                        const float4 c = *reinterpret_cast<const float4*>(crow + j);
                        o[j] += beta * c.x; o[j + 1] += beta * c.y; o[j + 2] += beta * c.z; o[j + 3] += beta * c.w;
                    }
                    *reinterpret_cast<float4*>(crow + j) = make_float4(o[j], o[j + 1], o[j + 2], o[j + 3]);
                }
            } else {
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    if (col0 + j < N) {
                        float x = o[j];
                        if (rrow) x += rrow[j];
                        if (beta != 0.0f) x += beta * crow[j];
                        crow[j] = x;
                    }
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) { tc_fence_after(); tmem_dealloc(tmem_base, 64); }
}

}  // namespace tbk

#define TBK_GEMM_ARGS                                                                                         \
    const float *__restrict__ A, const float *__restrict__ B, float *__restrict__ C, int M, int N, int K, int lda, int ldb, \
        int ldc, long long strideA, long long strideB, long long strideC, float alpha, float beta
#define TBK_GEMM_PASS A, B, C, M, N, K, lda, ldb, ldc, strideA, strideB, strideC, alpha, beta, nullptr, nullptr

// float32 storage, bf16 operands (the reference's mma.sync kernels, cuda/train_kernels.cu:343-467)
extern "C" __global__ void __launch_bounds__(256) k_bf16_gemm_nn(TBK_GEMM_ARGS) { tbk::gemm_tile<0, 0, false>(TBK_GEMM_PASS, 64); }
extern "C" __global__ void __launch_bounds__(256) k_bf16_gemm_nt(TBK_GEMM_ARGS) { tbk::gemm_tile<0, 1, false>(TBK_GEMM_PASS, 64); }
extern "C" __global__ void __launch_bounds__(256) k_bf16_gemm_tn(TBK_GEMM_ARGS) { tbk::gemm_tile<1, 0, false>(TBK_GEMM_PASS, 64); }
// (never launched by the reference's host code, cuda/train_kernels.cu:199-205; kept because gpu_trainer_create looks it up)
extern "C" __global__ void __launch_bounds__(256) k_bf16_gemm_tn_small(TBK_GEMM_ARGS) { tbk::gemm_tile<1, 0, false>(TBK_GEMM_PASS, 32); }
// float32 SIMT kernels in the reference (cuda/train_kernels.cu:110-193): float32 operands read as tf32 here
extern "C" __global__ void __launch_bounds__(256) k_gemm_nn(TBK_GEMM_ARGS) { tbk::gemm_tile<0, 0, true>(TBK_GEMM_PASS, 64); }
extern "C" __global__ void __launch_bounds__(256) k_gemm_nt(TBK_GEMM_ARGS) { tbk::gemm_tile<0, 1, true>(TBK_GEMM_PASS, 64); }
extern "C" __global__ void __launch_bounds__(256) k_gemm_tn(TBK_GEMM_ARGS) { tbk::gemm_tile<1, 0, true>(TBK_GEMM_PASS, 64); }

// C = A B + bias (+ residual), all contiguous; a null bias or residual is skipped (cuda/train_kernels.cu:226-329)
extern "C" __global__ void __launch_bounds__(256)
k_bf16_gemm_nn_bias(const float* __restrict__ A, const float* __restrict__ B, const float* __restrict__ bias,
                    const float* __restrict__ residual, float* __restrict__ C, int M, int N, int K) {
    tbk::gemm_tile<0, 0, false>(A, B, C, M, N, K, K, N, N, 0, 0, 0, 1.0f, 0.0f, bias, residual, 64);
}

// C[M,N] = A[M,K] B[K,N], float32 (cuda/kernels.cu:35-65; note the M, K, N order); launched on 16 x 16 blocks
extern "C" __global__ void __launch_bounds__(256)
k_matmul(const float* __restrict__ A, const float* __restrict__ B, float* __restrict__ C, int M, int K, int N) {
    tbk::gemm_tile<0, 0, true>(A, B, C, M, N, K, K, N, N, 0, 0, 0, 1.0f, 0.0f, nullptr, nullptr, 16);
}
