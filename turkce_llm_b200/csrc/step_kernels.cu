// Row / element kernels that complete a training step (see step_kernels.h).
// Formulas follow the reference's kernels (cuda/train_kernels.cu:503-800) and the CPU
// definitions they mirror (model/model_ops.c, model/rope.c, model/loss.c, training/adam.c);
// the parallel decomposition is this library's own: one warp per row with shuffle
// reductions instead of one 256-thread block per row with shared-memory trees.
#include "step_kernels.h"

#include <cstdlib>

namespace tb {

static inline int grid_for(long long work, int block, const DeviceCtx* ctx, int per_sm = 16) {
    long long b = (work + block - 1) / block;
    const long long cap = (long long)per_sm * ctx->sm_count;
    if (b > cap) b = cap;
    return (int)(b < 1 ? 1 : b);
}

#define TB_LAUNCHED(ctx)            \
    do {                            \
        TB_CUDA(cudaGetLastError()); \
        (ctx)->launches++;          \
        prof_close((ctx), st);      \
    } while (0)

__device__ __forceinline__ float exp2f_approx(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ------------------------------------------------------------------ embedding
__global__ void embed_fwd_kernel(const float* __restrict__ E, const uint32_t* __restrict__ ids,
                                 float* __restrict__ x, long long total, int D) {
    pdl_wait();
    pdl_launch_dependents();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long n = i / D;
        const int j = (int)(i % D);
        x[i] = E[(long long)ids[n] * D + j];     // ids are range-checked by whoever writes them (host or argmax)
    }
}

int launch_embed_fwd(DeviceCtx* ctx, const float* E, const uint32_t* ids, float* x, int rows, int D,
                     cudaStream_t st) {
    const long long total = (long long)rows * D;
    prof_mark(ctx, "embed_fwd", 0.0, 0.0, st);
    TB_CUDA(launch_kernel(embed_fwd_kernel, dim3(grid_for(total, 256, ctx)), dim3(256), 0, st, E, ids, x, total, D));
    TB_LAUNCHED(ctx);
    return 0;
}

// Embedding gradient.  The host sorts the rows by token (ties by position) and cuts every run of
// equal tokens into chunks of at most kEmbedChunk rows; one block per chunk adds its rows in
// ascending position.  A run of one chunk adds straight into dE[token]; a longer run (a frequent
// token) parks each chunk's sum in `partial`, and the block that takes the run's last ticket adds
// the chunk sums in chunk order, so the result does not depend on which block finishes last.
// meta[3c..3c+2] = {first partial slot of the run or 0xffffffff, chunk index in the run, chunks in the run}.
// The grid has one block per row; blocks past the number of chunks (read from device memory, so
// that the launch shape does not depend on the batch) return at once.
__global__ void embed_bwd_kernel(const float* __restrict__ dx, const uint32_t* __restrict__ order,
                                 const uint32_t* __restrict__ seg_start, const uint32_t* __restrict__ seg_token,
                                 const uint32_t* __restrict__ meta, const uint32_t* __restrict__ nseg,
                                 float* __restrict__ partial, unsigned int* __restrict__ tickets,
                                 float* __restrict__ dE, int D) {
    pdl_wait();
    pdl_launch_dependents();
    const uint32_t seg = blockIdx.x;
    if (seg >= *nseg) return;
    __shared__ uint32_t rows[kEmbedChunk];
    __shared__ int is_last;
    const uint32_t r0 = seg_start[seg], r1 = seg_start[seg + 1];
    const int n = (int)(r1 - r0);
    const long long tok = seg_token[seg];
    const uint32_t slot0 = meta[3 * seg], idx = meta[3 * seg + 1], count = meta[3 * seg + 2];
    if ((int)threadIdx.x < n) rows[threadIdx.x] = order[r0 + threadIdx.x];
    __syncthreads();
    float* dst = slot0 == 0xffffffffu ? dE + tok * D : partial + (long long)(slot0 + idx) * D;
    for (int j = threadIdx.x; j < D; j += blockDim.x) {
        float acc = 0.0f;
        for (int r = 0; r < n; ++r) acc += dx[(long long)rows[r] * D + j];
        if (slot0 == 0xffffffffu) dst[j] += acc; else dst[j] = acc;
    }
    if (slot0 == 0xffffffffu) return;
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned int t = atomicAdd(&tickets[slot0], 1u);
        is_last = (t == count - 1u);
        if (is_last) tickets[slot0] = 0u;              // ready for the next step
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    for (int j = threadIdx.x; j < D; j += blockDim.x) {
        float acc = 0.0f;
        for (uint32_t c = 0; c < count; ++c) acc += __ldcg(partial + (long long)(slot0 + c) * D + j);
        dE[tok * D + j] += acc;
    }
}

int launch_embed_bwd(DeviceCtx* ctx, const float* dx, const uint32_t* order, const uint32_t* seg_start,
                     const uint32_t* seg_token, const uint32_t* meta, const uint32_t* nseg, int rows, float* partial,
                     unsigned int* tickets, float* dE, int D, cudaStream_t st) {
    if (rows <= 0) return 0;
    const int threads = D >= 256 ? 256 : (D >= 128 ? 128 : 64);
    prof_mark(ctx, "embed_bwd", 0.0, 0.0, st);
    TB_CUDA(launch_kernel(embed_bwd_kernel, dim3(rows), dim3(threads), 0, st, dx, order, seg_start, seg_token, meta,
                          nseg, partial, tickets, dE, D));
    TB_LAUNCHED(ctx);
    return 0;
}

// -------------------------------------------------------------------- RMSNorm
// y = x * r * w,  r = 1/sqrt(mean(x^2) + eps)   (model/model_ops.c; eps inside the root)
__global__ void rmsnorm_fwd_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                   bf16* __restrict__ out, float* __restrict__ out32, float* __restrict__ rinv,
                                   int rows, int cols, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int wpb = blockDim.x >> 5;
    for (long long row = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); row < rows;
         row += (long long)gridDim.x * wpb) {
        const float* xr = x + row * cols;
        float ss = 0.0f;
        for (int i = lane; i < cols; i += 32) ss += xr[i] * xr[i];
        ss = warp_sum(ss);
        const float ms = ss / (float)cols;
        const float r = 1.0f / (float)sqrt((double)(ms + eps));
        if (lane == 0) rinv[row] = r;
        for (int i = lane; i < cols; i += 32) {
            const float y = xr[i] * r * w[i];
            if (out) out[row * cols + i] = __float2bfloat16_rn(y);
            if (out32) out32[row * cols + i] = y;
        }
    }
}

// the same with 16-byte loads and 8-byte stores (cols % 4 == 0, cols <= 4 * 32 * NV)
template <int NV>
__global__ void rmsnorm_fwd_vec_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                       bf16* __restrict__ out, float* __restrict__ out32, float* __restrict__ rinv,
                                       int rows, int cols, float eps) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int wpb = blockDim.x >> 5;
    for (long long row = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); row < rows;
         row += (long long)gridDim.x * wpb) {
        const float* xr = x + row * cols;
        float4 xv[NV];
        float ss = 0.0f;
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int j = 4 * (lane + 32 * k);
            xv[k] = j < cols ? *reinterpret_cast<const float4*>(xr + j) : make_float4(0.f, 0.f, 0.f, 0.f);
            ss += xv[k].x * xv[k].x + xv[k].y * xv[k].y + xv[k].z * xv[k].z + xv[k].w * xv[k].w;
        }
        ss = warp_sum(ss);
        const float ms = ss / (float)cols;
        const float r = 1.0f / (float)sqrt((double)(ms + eps));
        if (lane == 0) rinv[row] = r;
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int j = 4 * (lane + 32 * k);
            if (j < cols) {
                const float4 wv = *reinterpret_cast<const float4*>(w + j);
                const float4 y = make_float4(xv[k].x * r * wv.x, xv[k].y * r * wv.y, xv[k].z * r * wv.z, xv[k].w * r * wv.w);
                if (out) {
                    __nv_bfloat162 lo = __floats2bfloat162_rn(y.x, y.y);
                    __nv_bfloat162 hi = __floats2bfloat162_rn(y.z, y.w);
                    uint2 pk;
                    pk.x = *reinterpret_cast<uint32_t*>(&lo); pk.y = *reinterpret_cast<uint32_t*>(&hi);
                    *reinterpret_cast<uint2*>(out + row * cols + j) = pk;
                }
                if (out32) *reinterpret_cast<float4*>(out32 + row * cols + j) = y;
            }
        }
    }
}

int launch_rmsnorm_fwd(DeviceCtx* ctx, const float* x, const float* w, bf16* out, float* rinv, int rows, int cols,
                       float eps, cudaStream_t st, float* out32) {
    prof_mark(ctx, "rmsnorm_fwd", 0.0, 0.0, st);
    if (cols % 4 == 0 && cols <= 384 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0 && (reinterpret_cast<uintptr_t>(w) & 15u) == 0 &&
        (reinterpret_cast<uintptr_t>(out) & 7u) == 0 && (reinterpret_cast<uintptr_t>(out32) & 15u) == 0)
        TB_CUDA(launch_kernel(rmsnorm_fwd_vec_kernel<3>, dim3(grid_for(rows, 8, ctx)), dim3(256), 0, st, x, w, out, out32, rinv, rows, cols, eps));
    else
        TB_CUDA(launch_kernel(rmsnorm_fwd_kernel, dim3(grid_for(rows, 8, ctx)), dim3(256), 0, st, x, w, out, out32, rinv, rows, cols, eps));
    TB_LAUNCHED(ctx);
    return 0;
}

// dx[j] (+)= w[j]*r*dy[j] - (r^3/cols) * x[j] * S,  S = sum_j dy*w*x ;  wtmp[j] = dy[j]*x[j]*r
__global__ void rmsnorm_bwd_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                   const float* __restrict__ rinv, const float* __restrict__ dy,
                                   float* __restrict__ dx, bf16* __restrict__ dx16, float* __restrict__ wtmp,
                                   int rows, int cols, int accumulate) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int wpb = blockDim.x >> 5;
    for (long long row = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); row < rows;
         row += (long long)gridDim.x * wpb) {
        const float* xr = x + row * cols;
        const float* dyr = dy + row * cols;
        const float r = rinv[row];
        float S = 0.0f;
        for (int i = lane; i < cols; i += 32) S += dyr[i] * w[i] * xr[i];
        S = warp_sum(S);
        const float k = (r * r * r) / (float)cols;
        for (int j = lane; j < cols; j += 32) {
            const long long o = row * cols + j;
            float v = w[j] * r * dyr[j] - k * xr[j] * S;
            if (accumulate) v += dx[o];
            dx[o] = v;
            dx16[o] = __float2bfloat16_rn(v);
            wtmp[o] = dyr[j] * xr[j] * r;
        }
    }
}

// Same row math, plus the norm-weight gradient dw[j] += sum_rows dy*x*r without the [rows, cols]
// temporary: each warp keeps its rows' column sums in registers, the block adds its warps in warp
// order and writes one partial row; norm_partial_sum_kernel then adds the partial rows in block
// order.  NC = ceil(cols / 32) columns per lane.
template <int NC>
__global__ void rmsnorm_bwd_dw_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                      const float* __restrict__ rinv, const float* __restrict__ dy,
                                      float* __restrict__ dx, bf16* __restrict__ dx16,
                                      float* __restrict__ partial, int rows, int cols, int accumulate) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float sh_part[];      // [warps][2 * cols]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wpb = blockDim.x >> 5;
    // every partial row is [norm-weight sums | column sums of dx], 2*cols floats
    const int pc = 2 * cols;
    float acc[NC], accb[NC];
#pragma unroll
    for (int k = 0; k < NC; ++k) { acc[k] = 0.0f; accb[k] = 0.0f; }
    for (long long row = (long long)blockIdx.x * wpb + warp; row < rows; row += (long long)gridDim.x * wpb) {
        const float* xr = x + row * cols;
        const float* dyr = dy + row * cols;
        const float r = rinv[row];
        float xv[NC], dv[NC], wv[NC], ov[NC];
        float S = 0.0f;
#pragma unroll
        for (int k = 0; k < NC; ++k) {
            const int j = lane + 32 * k;
            const bool in = j < cols;
            xv[k] = in ? xr[j] : 0.0f;
            dv[k] = in ? dyr[j] : 0.0f;
            wv[k] = in ? w[j] : 0.0f;
            ov[k] = (in && accumulate) ? dx[row * cols + j] : 0.0f;
        }
#pragma unroll
        for (int k = 0; k < NC; ++k) S += dv[k] * wv[k] * xv[k];
        S = warp_sum(S);
        const float kk = (r * r * r) / (float)cols;
#pragma unroll
        for (int k = 0; k < NC; ++k) {
            const int j = lane + 32 * k;
            if (j < cols) {
                const long long o = row * cols + j;
                const float v = wv[k] * r * dv[k] - kk * xv[k] * S + ov[k];
                dx[o] = v;
                dx16[o] = __float2bfloat16_rn(v);
                acc[k] += dv[k] * xv[k] * r;
                accb[k] += v;
            }
        }
    }
#pragma unroll
    for (int k = 0; k < NC; ++k) {
        const int j = lane + 32 * k;
        if (j < cols) { sh_part[warp * pc + j] = acc[k]; sh_part[warp * pc + cols + j] = accb[k]; }
    }
    __syncthreads();
    for (int j = threadIdx.x; j < pc; j += blockDim.x) {
        float t = sh_part[j];
        for (int k = 1; k < wpb; ++k) t += sh_part[k * pc + j];
        partial[(long long)blockIdx.x * pc + j] = t;
    }
}

// The same kernel with 16-byte accesses: lane owns columns 4*(lane + 32k) .. +3 (cols % 4 == 0), which cuts
// the load/store instruction count by four -- the kernel is bound by memory requests, not by arithmetic.
template <int NV>
__global__ void rmsnorm_bwd_dw_vec_kernel(const float* __restrict__ x, const float* __restrict__ w,
                                          const float* __restrict__ rinv, const float* __restrict__ dy,
                                          float* __restrict__ dx, bf16* __restrict__ dx16,
                                          float* __restrict__ partial, int rows, int cols, int accumulate) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float sh_part[];      // [warps][2 * cols]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int wpb = blockDim.x >> 5;
    const int pc = 2 * cols;
    float4 acc[NV], accb[NV], wv[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int j = 4 * (lane + 32 * k);
        acc[k] = make_float4(0.f, 0.f, 0.f, 0.f); accb[k] = acc[k];
        wv[k] = j < cols ? *reinterpret_cast<const float4*>(w + j) : acc[k];
    }
    for (long long row = (long long)blockIdx.x * wpb + warp; row < rows; row += (long long)gridDim.x * wpb) {
        const float* xr = x + row * cols;
        const float* dyr = dy + row * cols;
        float* dxr = dx + row * cols;
        const float r = rinv[row];
        float4 xv[NV], dv[NV], ov[NV];
        const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int j = 4 * (lane + 32 * k);
            const bool in = j < cols;
            xv[k] = in ? *reinterpret_cast<const float4*>(xr + j) : z;
            dv[k] = in ? *reinterpret_cast<const float4*>(dyr + j) : z;
            ov[k] = (in && accumulate) ? *reinterpret_cast<const float4*>(dxr + j) : z;
        }
        float S = 0.0f;
#pragma unroll
        for (int k = 0; k < NV; ++k)
            S += dv[k].x * wv[k].x * xv[k].x + dv[k].y * wv[k].y * xv[k].y + dv[k].z * wv[k].z * xv[k].z +
                 dv[k].w * wv[k].w * xv[k].w;
        S = warp_sum(S);
        const float kk = (r * r * r) / (float)cols * S;
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            const int j = 4 * (lane + 32 * k);
            if (j < cols) {
                float4 v;
                v.x = wv[k].x * r * dv[k].x - kk * xv[k].x + ov[k].x;
                v.y = wv[k].y * r * dv[k].y - kk * xv[k].y + ov[k].y;
                v.z = wv[k].z * r * dv[k].z - kk * xv[k].z + ov[k].z;
                v.w = wv[k].w * r * dv[k].w - kk * xv[k].w + ov[k].w;
                *reinterpret_cast<float4*>(dxr + j) = v;
                __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y), hi = __floats2bfloat162_rn(v.z, v.w);
                uint2 pk;
                pk.x = *reinterpret_cast<uint32_t*>(&lo); pk.y = *reinterpret_cast<uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(dx16 + row * cols + j) = pk;
                acc[k].x += dv[k].x * xv[k].x * r; acc[k].y += dv[k].y * xv[k].y * r;
                acc[k].z += dv[k].z * xv[k].z * r; acc[k].w += dv[k].w * xv[k].w * r;
                accb[k].x += v.x; accb[k].y += v.y; accb[k].z += v.z; accb[k].w += v.w;
            }
        }
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        const int j = 4 * (lane + 32 * k);
        if (j < cols) {
            *reinterpret_cast<float4*>(sh_part + warp * pc + j) = acc[k];
            *reinterpret_cast<float4*>(sh_part + warp * pc + cols + j) = accb[k];
        }
    }
    __syncthreads();
    for (int j = threadIdx.x; j < pc; j += blockDim.x) {
        float t = sh_part[j];
        for (int k = 1; k < wpb; ++k) t += sh_part[k * pc + j];
        partial[(long long)blockIdx.x * pc + j] = t;
    }
}

// dw[j] += sum over the partial rows (block order), db likewise: one block per 32 columns, each
// warp adds up to 32 consecutive partial rows (all loads in flight at once), warp 0 adds the warps.
__global__ void norm_partial_sum_kernel(const float* __restrict__ partial, int nb, int pc, int cols,
                                        float* __restrict__ dw, float* __restrict__ db) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float sh[32][33];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    const int j = blockIdx.x * 32 + lane;
    const int per = (nb + nw - 1) / nw;              // <= 32 by the launch
    float v[32];
#pragma unroll
    for (int k = 0; k < 32; ++k) {
        const int r = warp * per + k;
        v[k] = (k < per && r < nb && j < pc) ? __ldcg(&partial[(long long)r * pc + j]) : 0.0f;
    }
    float t = v[0];
#pragma unroll
    for (int k = 1; k < 32; ++k) t += v[k];
    sh[warp][lane] = t;
    __syncthreads();
    if (warp == 0 && j < pc) {
        float s = sh[0][lane];
        for (int k = 1; k < nw; ++k) s += sh[k][lane];
        if (j < cols) dw[j] += s;
        else if (db) db[j - cols] += s;
    }
}

constexpr int kNormBwdBlocks = 512;      // partial rows of the fused norm-weight gradient
constexpr int kNormBwdWarps = 16;        // rows in flight per block

size_t rmsnorm_bwd_scratch_floats(int cols) { return 64 + (size_t)(kNormBwdBlocks + 32) * cols * 2; }

int launch_rmsnorm_bwd_dw(DeviceCtx* ctx, const float* x, const float* w, const float* rinv, const float* dy,
                          float* dx, bf16* dx16, float* dw, float* db, float* scratch, int rows, int cols,
                          int accumulate, cudaStream_t st) {
    TB_CHECK(cols <= 1024, "fused RMSNorm backward supports at most 1024 columns (got %d)", cols);
    const int warps = cols <= 384 ? kNormBwdWarps : 8;       // the wide variant holds whole rows in 255 registers
    const size_t smem = (size_t)warps * 2 * cols * sizeof(float);
    static bool attr_set[64] = {false};
    if (!attr_set[ctx->device & 63]) {
        TB_CUDA(cudaFuncSetAttribute(rmsnorm_bwd_dw_kernel<12>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     kNormBwdWarps * 2 * 384 * (int)sizeof(float)));
        TB_CUDA(cudaFuncSetAttribute(rmsnorm_bwd_dw_vec_kernel<3>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     kNormBwdWarps * 2 * 384 * (int)sizeof(float)));
        TB_CUDA(cudaFuncSetAttribute(rmsnorm_bwd_dw_kernel<32>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     8 * 2 * 1024 * (int)sizeof(float)));
        attr_set[ctx->device & 63] = true;
    }
    int blocks = (rows + warps - 1) / warps;
    // Three quarters of the SMs, a warp walking several rows: in the training step this kernel runs beside a
    // weight-gradient GEMM on the second stream, and a grid that fills every SM (one row per warp, 512 blocks) only
    // takes that GEMM's SMs.  Measured on the benchmark step (148 SMs): 512 blocks 4.69 ms, 296 4.65, 148 4.62, 111 4.58,
    // 74 4.63 -- although alone the kernel is fastest at 148 (16.6 us with its events against 18.1 at 111, 19.4 at 512).
    static const int cap_env = getenv("TB_NORM_BLOCKS") ? atoi(getenv("TB_NORM_BLOCKS")) : 0;
    const int cap = cap_env >= 16 ? cap_env : ctx->sm_count * 3 / 4;
    if (blocks > kNormBwdBlocks) blocks = kNormBwdBlocks;
    if (blocks > cap) blocks = cap;
    float* partial = scratch + 64;
    const int pc = 2 * cols;
    prof_mark(ctx, "rmsnorm_bwd", 0.0, 0.0, st);
    if (cols % 4 == 0 && cols <= 384)
        TB_CUDA(launch_kernel((rmsnorm_bwd_dw_vec_kernel<3>), dim3(blocks), dim3(32 * warps), smem, st, x, w, rinv, dy, dx, dx16, partial, rows, cols, accumulate));
    else if (cols <= 384)
        TB_CUDA(launch_kernel((rmsnorm_bwd_dw_kernel<12>), dim3(blocks), dim3(32 * warps), smem, st, x, w, rinv, dy, dx, dx16, partial, rows, cols, accumulate));
    else
        TB_CUDA(launch_kernel((rmsnorm_bwd_dw_kernel<32>), dim3(blocks), dim3(32 * warps), smem, st, x, w, rinv, dy, dx, dx16, partial, rows, cols, accumulate));
    TB_LAUNCHED(ctx);
    prof_mark(ctx, "rmsnorm_bwd_sum", 0.0, 0.0, st);
    TB_CUDA(launch_kernel(norm_partial_sum_kernel, dim3((pc + 31) / 32), dim3(32 * ((blocks + 31) / 32)), 0, st, (const float*)partial, blocks, pc, cols, dw, db));
    TB_LAUNCHED(ctx);
    return 0;
}

int launch_rmsnorm_bwd(DeviceCtx* ctx, const float* x, const float* w, const float* rinv, const float* dy, float* dx,
                       bf16* dx16, float* wtmp, int rows, int cols, int accumulate, cudaStream_t st) {
    prof_mark(ctx, "rmsnorm_bwd", 0.0, 0.0, st);
    TB_CUDA(launch_kernel(rmsnorm_bwd_kernel, dim3(grid_for(rows, 8, ctx)), dim3(256), 0, st, x, w, rinv, dy, dx, dx16, wtmp, rows, cols, accumulate));
    TB_LAUNCHED(ctx);
    return 0;
}

// ----------------------------------------------------------------------- RoPE
// qkv [B*T, 3D] -> Q, K rotated on interleaved pairs (2k, 2k+1), V copied; all [B,H,T,hd] bf16
__global__ void rope_split_kernel(const float* __restrict__ qkv, const float* __restrict__ cos_t,
                                  const float* __restrict__ sin_t, bf16* __restrict__ Q, bf16* __restrict__ K,
                                  bf16* __restrict__ V, int B, int T, int H, int hd, int kv_cap) {
    pdl_wait();
    pdl_launch_dependents();
    const int half = hd >> 1;
    const int D = H * hd;
    const long long total = (long long)B * T * H * half;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int k = (int)(i % half);
        long long rest = i / half;
        const int h = (int)(rest % H);
        const long long n = rest / H;
        const int t = (int)(n % T);
        const long long b = n / T;
        const float* row = qkv + n * 3LL * D;
        const int c0 = h * hd + 2 * k;
        const float c = cos_t[t * half + k], s = sin_t[t * half + k];
        const long long o = ((b * H + h) * T + t) * hd + 2 * k;
        const long long okv = ((b * H + h) * (long long)kv_cap + t) * hd + 2 * k;     // K/V rows have room for kv_cap positions
        const float2 q = *reinterpret_cast<const float2*>(row + c0);
        const float2 kk = *reinterpret_cast<const float2*>(row + D + c0);
        const float2 v = *reinterpret_cast<const float2*>(row + 2 * D + c0);
        *reinterpret_cast<__nv_bfloat162*>(Q + o) = __floats2bfloat162_rn(q.x * c - q.y * s, q.x * s + q.y * c);
        *reinterpret_cast<__nv_bfloat162*>(K + okv) = __floats2bfloat162_rn(kk.x * c - kk.y * s, kk.x * s + kk.y * c);
        *reinterpret_cast<__nv_bfloat162*>(V + okv) = __floats2bfloat162_rn(v.x, v.y);
    }
}

int launch_rope_split(DeviceCtx* ctx, const float* qkv, const float* cos_t, const float* sin_t, bf16* Q, bf16* K,
                      bf16* V, int B, int T, int H, int hd, int kv_cap, cudaStream_t st) {
    TB_CHECK(hd % 2 == 0, "head dim must be even");
    const long long total = (long long)B * T * H * (hd / 2);
    prof_mark(ctx, "rope_split", 0.0, 0.0, st);
    TB_CUDA(launch_kernel(rope_split_kernel, dim3(grid_for(total, 256, ctx)), dim3(256), 0, st, qkv, cos_t, sin_t, Q, K, V, B, T, H, hd, kv_cap));
    TB_LAUNCHED(ctx);
    return 0;
}

// inverse rotation of dQ, dK and merge with dV into dqkv [B*T, 3D] (bf16)
__global__ void rope_merge_bwd_kernel(const float* __restrict__ dQ, const float* __restrict__ dK,
                                      const float* __restrict__ dV, const float* __restrict__ cos_t,
                                      const float* __restrict__ sin_t, bf16* __restrict__ dqkv, int B, int T, int H,
                                      int hd) {
    pdl_wait();
    pdl_launch_dependents();
    const int half = hd >> 1;
    const int D = H * hd;
    const long long total = (long long)B * T * H * half;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int k = (int)(i % half);
        long long rest = i / half;
        const int h = (int)(rest % H);
        const long long n = rest / H;
        const int t = (int)(n % T);
        const long long b = n / T;
        bf16* row = dqkv + n * 3LL * D;
        const int c0 = h * hd + 2 * k;
        const float c = cos_t[t * half + k], s = sin_t[t * half + k];
        const long long o = ((b * H + h) * T + t) * hd + 2 * k;
        const float2 a = *reinterpret_cast<const float2*>(dQ + o);
        const float2 bb = *reinterpret_cast<const float2*>(dK + o);
        const float2 v = *reinterpret_cast<const float2*>(dV + o);
        *reinterpret_cast<__nv_bfloat162*>(row + c0) = __floats2bfloat162_rn(a.x * c + a.y * s, -a.x * s + a.y * c);
        *reinterpret_cast<__nv_bfloat162*>(row + D + c0) =
            __floats2bfloat162_rn(bb.x * c + bb.y * s, -bb.x * s + bb.y * c);
        *reinterpret_cast<__nv_bfloat162*>(row + 2 * D + c0) = __floats2bfloat162_rn(v.x, v.y);
    }
}

int launch_rope_merge_bwd(DeviceCtx* ctx, const float* dQ, const float* dK, const float* dV, const float* cos_t,
                          const float* sin_t, bf16* dqkv, int B, int T, int H, int hd, cudaStream_t st) {
    const long long total = (long long)B * T * H * (hd / 2);
    prof_mark(ctx, "rope_merge_bwd", 0.0, 0.0, st);
    TB_CUDA(launch_kernel(rope_merge_bwd_kernel, dim3(grid_for(total, 256, ctx)), dim3(256), 0, st, dQ, dK, dV, cos_t, sin_t, dqkv, B, T, H, hd));
    TB_LAUNCHED(ctx);
    return 0;
}

__device__ __forceinline__ float block_reduce(float v, float* sh, bool is_max);

// ------------------------------------------------------- decode (one new token per sequence)
// qkv [S, 3D] of the new tokens at position *pos: rotated q -> Q [S, H, hd] (float32), rotated k and
// v -> the KV cache [S, H, cap, hd] (bf16) at row *pos.
__global__ void rope_decode_kernel(const float* __restrict__ qkv, const float* __restrict__ cos_t,
                                   const float* __restrict__ sin_t, float* __restrict__ Q, bf16* __restrict__ Kc,
                                   bf16* __restrict__ Vc, const int* __restrict__ pos, int S, int H, int hd, int cap) {
    pdl_wait();
    pdl_launch_dependents();
    const int half = hd >> 1, D = H * hd;
    const int t = *pos;
    const int total = S * H * half;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int k = i % half;
        const int h = (i / half) % H;
        const int sq = i / (half * H);
        const float* row = qkv + (long long)sq * 3 * D;
        const int c0 = h * hd + 2 * k;
        const float c = cos_t[t * half + k], sn = sin_t[t * half + k];
        const float2 q = *reinterpret_cast<const float2*>(row + c0);
        const float2 kk = *reinterpret_cast<const float2*>(row + D + c0);
        const float2 v = *reinterpret_cast<const float2*>(row + 2 * D + c0);
        *reinterpret_cast<float2*>(Q + ((long long)sq * H + h) * hd + 2 * k) = make_float2(q.x * c - q.y * sn, q.x * sn + q.y * c);
        const long long o = (((long long)sq * H + h) * cap + t) * hd + 2 * k;
        *reinterpret_cast<__nv_bfloat162*>(Kc + o) = __floats2bfloat162_rn(kk.x * c - kk.y * sn, kk.x * sn + kk.y * c);
        *reinterpret_cast<__nv_bfloat162*>(Vc + o) = __floats2bfloat162_rn(v.x, v.y);
    }
}

int launch_rope_decode(DeviceCtx* ctx, const float* qkv, const float* cos_t, const float* sin_t, float* Q, bf16* Kc,
                       bf16* Vc, const int* pos, int S, int H, int hd, int cap, cudaStream_t st) {
    const int total = S * H * (hd / 2);
    prof_mark(ctx, "rope_decode", 0.0, 0.0, st);
    TB_CUDA(launch_kernel(rope_decode_kernel, dim3(grid_for(total, 128, ctx)), dim3(128), 0, st, qkv, cos_t, sin_t, Q, Kc, Vc, pos, S, H, hd, cap));
    TB_LAUNCHED(ctx);
    return 0;
}

// One block per (sequence, head): scores of the new query against cache rows 0..*pos, softmax, P V.
// The same function as a full causal forward restricted to its last row (model/attention.c:55-60).
__global__ void attn_decode_kernel(const float* __restrict__ Q, const bf16* __restrict__ Kc,
                                   const bf16* __restrict__ Vc, bf16* __restrict__ att, const int* __restrict__ pos,
                                   int H, int hd, int cap, float scale) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float sh[];            // q [hd] | p [cap] | red [32] | part [groups][hd]
    float* q = sh;
    float* p = sh + hd;
    float* red = p + cap;
    float* part = red + 32;
    const int h = blockIdx.x, sq = blockIdx.y;
    const int L = *pos + 1;
    const int tid = threadIdx.x, nt = blockDim.x;
    const bf16* Kb = Kc + ((long long)sq * H + h) * cap * hd;
    const bf16* Vb = Vc + ((long long)sq * H + h) * cap * hd;
    for (int d = tid; d < hd; d += nt) q[d] = Q[((long long)sq * H + h) * hd + d];
    __syncthreads();
    float mx = -3.0e38f;
    for (int l = tid; l < L; l += nt) {
        const bf16* kr = Kb + (long long)l * hd;
        float s = 0.0f;
        for (int d = 0; d < hd; d += 8) {
            const uint4 kv = *reinterpret_cast<const uint4*>(kr + d);
            const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&kv);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(k2[e]);
                s += q[d + 2 * e] * f.x;
                s += q[d + 2 * e + 1] * f.y;
            }
        }
        s *= scale;
        p[l] = s;
        mx = fmaxf(mx, s);
    }
    mx = block_reduce(mx, red, true);
    float sum = 0.0f;
    for (int l = tid; l < L; l += nt) {
        const float e = expf(p[l] - mx);
        p[l] = e;
        sum += e;
    }
    sum = block_reduce(sum, red, false);
    // output: thread (g, c) adds keys g, g+G, ... for head dims 4c..4c+3 (one 8-byte load per key); the G
    // partial sums are added in group order
    const int C = hd >> 2;                   // threads per key group
    const int G = nt / C;
    const int g = tid / C, c4 = (tid % C) * 4;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    if (g < G) {
        for (int l = g; l < L; l += G) {
            const uint2 v = *reinterpret_cast<const uint2*>(Vb + (long long)l * hd + c4);
            const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
            const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
            const float w = p[l];
            a0 += w * lo.x; a1 += w * lo.y; a2 += w * hi.x; a3 += w * hi.y;
        }
        float* dst = part + g * hd + c4;
        dst[0] = a0; dst[1] = a1; dst[2] = a2; dst[3] = a3;
    }
    __syncthreads();
    if (tid < hd) {
        float o = part[tid];
        for (int k = 1; k < G; ++k) o += part[k * hd + tid];
        att[(long long)sq * (H * hd) + h * hd + tid] = __float2bfloat16_rn(o / sum);
    }
}

int launch_attn_decode(DeviceCtx* ctx, const float* Q, const bf16* Kc, const bf16* Vc, bf16* att, const int* pos, int S,
                       int H, int hd, int cap, float scale, cudaStream_t st) {
    TB_CHECK(hd <= 128 && hd % 8 == 0, "decode attention needs head_dim <= 128 and a multiple of 8");
    TB_CHECK(hd % 4 == 0, "decode attention needs a head_dim that is a multiple of 4");
    const int threads = 256 / (hd / 4) * (hd / 4) >= 64 ? 256 / (hd / 4) * (hd / 4) : 64;     // whole key groups of hd/4 threads
    const int groups = threads / (hd / 4);
    const size_t smem = (size_t)(hd + cap + 32 + groups * hd) * sizeof(float);
    TB_CHECK(smem <= 48 * 1024, "KV cache capacity %d too large for the decode attention kernel", cap);
    dim3 grid(H, S);
    prof_mark(ctx, "attn_decode", 0.0, 0.0, st);
    TB_CUDA(launch_kernel(attn_decode_kernel, dim3(grid), dim3(threads), smem, st, Q, Kc, Vc, att, pos, H, hd, cap, scale));
    TB_LAUNCHED(ctx);
    return 0;
}

// rope_decode_kernel and attn_decode_kernel in one launch: the block of (sequence, head) rotates its own slice of
// the new token's q and k, appends k and v to its own cache rows (no other block reads them in this launch),
// and attends over rows 0..*pos.  Kc and Vc are written and read here, so they are neither const nor restrict.
__global__ void rope_attn_decode_kernel(const float* __restrict__ qkv, const float* __restrict__ cos_t,
                                        const float* __restrict__ sin_t, bf16* Kc, bf16* Vc, bf16* __restrict__ att,
                                        const int* __restrict__ pos, int H, int hd, int cap, float scale) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float sh[];            // q [hd] | p [cap] | red [32] | part [groups][hd]
    float* q = sh;
    float* p = sh + hd;
    float* red = p + cap;
    float* part = red + 32;
    const int h = blockIdx.x, sq = blockIdx.y;
    const int t = *pos;
    const int L = t + 1;
    const int tid = threadIdx.x, nt = blockDim.x;
    const int half = hd >> 1, D = H * hd;
    bf16* Kb = Kc + ((long long)sq * H + h) * cap * hd;
    bf16* Vb = Vc + ((long long)sq * H + h) * cap * hd;
    for (int k = tid; k < half; k += nt) {
        const float* row = qkv + (long long)sq * 3 * D + h * hd + 2 * k;
        const float c = cos_t[t * half + k], sn = sin_t[t * half + k];
        const float2 qq = *reinterpret_cast<const float2*>(row);
        const float2 kk = *reinterpret_cast<const float2*>(row + D);
        const float2 v = *reinterpret_cast<const float2*>(row + 2 * D);
        q[2 * k] = qq.x * c - qq.y * sn;
        q[2 * k + 1] = qq.x * sn + qq.y * c;
        const long long o = (long long)t * hd + 2 * k;
        *reinterpret_cast<__nv_bfloat162*>(Kb + o) = __floats2bfloat162_rn(kk.x * c - kk.y * sn, kk.x * sn + kk.y * c);
        *reinterpret_cast<__nv_bfloat162*>(Vb + o) = __floats2bfloat162_rn(v.x, v.y);
    }
    __syncthreads();                         // the new cache row is visible to the whole block
    float mx = -3.0e38f;
    for (int l = tid; l < L; l += nt) {
        const bf16* kr = Kb + (long long)l * hd;
        float s = 0.0f;
        for (int d = 0; d < hd; d += 8) {
            const uint4 kv = *reinterpret_cast<const uint4*>(kr + d);
            const __nv_bfloat162* k2 = reinterpret_cast<const __nv_bfloat162*>(&kv);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __bfloat1622float2(k2[e]);
                s += q[d + 2 * e] * f.x;
                s += q[d + 2 * e + 1] * f.y;
            }
        }
        s *= scale;
        p[l] = s;
        mx = fmaxf(mx, s);
    }
    mx = block_reduce(mx, red, true);
    float sum = 0.0f;
    for (int l = tid; l < L; l += nt) {
        const float e = expf(p[l] - mx);
        p[l] = e;
        sum += e;
    }
    sum = block_reduce(sum, red, false);
    const int C = hd >> 2;
    const int G = nt / C;
    const int g = tid / C, c4 = (tid % C) * 4;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    if (g < G) {
        for (int l = g; l < L; l += G) {
            const uint2 v = *reinterpret_cast<const uint2*>(Vb + (long long)l * hd + c4);
            const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
            const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
            const float w = p[l];
            a0 += w * lo.x; a1 += w * lo.y; a2 += w * hi.x; a3 += w * hi.y;
        }
        float* dst = part + g * hd + c4;
        dst[0] = a0; dst[1] = a1; dst[2] = a2; dst[3] = a3;
    }
    __syncthreads();
    if (tid < hd) {
        float o = part[tid];
        for (int k = 1; k < G; ++k) o += part[k * hd + tid];
        att[(long long)sq * (H * hd) + h * hd + tid] = __float2bfloat16_rn(o / sum);
    }
}

int launch_rope_attn_decode(DeviceCtx* ctx, const float* qkv, const float* cos_t, const float* sin_t, bf16* Kc, bf16* Vc,
                            bf16* att, const int* pos, int S, int H, int hd, int cap, float scale, cudaStream_t st) {
    TB_CHECK(hd <= 128 && hd % 8 == 0, "decode attention needs head_dim <= 128 and a multiple of 8");
    const int threads = 256 / (hd / 4) * (hd / 4) >= 64 ? 256 / (hd / 4) * (hd / 4) : 64;
    const int groups = threads / (hd / 4);
    const size_t smem = (size_t)(hd + cap + 32 + groups * hd) * sizeof(float);
    TB_CHECK(smem <= 48 * 1024, "KV cache capacity %d too large for the decode attention kernel", cap);
    dim3 grid(H, S);
    prof_mark(ctx, "rope_attn_decode", 0.0, 0.0, st);
    TB_CUDA(launch_kernel(rope_attn_decode_kernel, dim3(grid), dim3(threads), smem, st, qkv, cos_t, sin_t, Kc, Vc, att, pos,
                          H, hd, cap, scale));
    TB_LAUNCHED(ctx);
    return 0;
}

// out[i, :] = in[idx(i), :] for the last position of every sequence: idx(i) = i*T + T-1
__global__ void gather_last_rows_kernel(const float* __restrict__ in, float* __restrict__ out, int S, int T, int D) {
    pdl_wait();
    pdl_launch_dependents();
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < S * D; i += gridDim.x * blockDim.x) {
        const int sq = i / D, j = i % D;
        out[i] = in[((long long)sq * T + T - 1) * D + j];
    }
}

int launch_gather_last_rows(DeviceCtx* ctx, const float* in, float* out, int S, int T, int D, cudaStream_t st) {
    prof_mark(ctx, "gather_last_rows", 0.0, 0.0, st);
    TB_CUDA(launch_kernel(gather_last_rows_kernel, dim3(grid_for((long long)S * D, 256, ctx)), dim3(256), 0, st, in, out, S, T, D));
    TB_LAUNCHED(ctx);
    return 0;
}

// Greedy choice: tok[s] = argmax_j logits[s, j] (lowest index on ties), also stored as generated
// token number state[1] of sequence s.  state = {position of the next token, tokens generated}.
__global__ void argmax_rows_kernel(const float* __restrict__ logits, uint32_t* __restrict__ tok,
                                   uint32_t* __restrict__ out, const int* __restrict__ state, int V, long long ld,
                                   int out_ld) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float bv[32];
    __shared__ int bi[32];
    const int sq = blockIdx.x;
    const float* z = logits + (long long)sq * ld;
    // a row of NaN or -inf logits (diverged weights) must still yield a token inside [0, V): the
    // comparison key of such a value is the lowest one, and the search starts from this thread's first column
    float best = -INFINITY;
    int idx = threadIdx.x < V ? (int)threadIdx.x : 0;
    for (int j = threadIdx.x; j < V; j += blockDim.x) {
        float v = z[j];
        if (!(v == v)) v = -INFINITY;
        if (v > best || (v == best && j < idx)) { best = v; idx = j; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ov > best || (ov == best && oi < idx)) { best = ov; idx = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { bv[warp] = best; bi[warp] = idx; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
            if (bv[w] > best || (bv[w] == best && bi[w] < idx)) { best = bv[w]; idx = bi[w]; }
        tok[sq] = (uint32_t)idx;
        if (out) out[(long long)sq * out_ld + state[1]] = (uint32_t)idx;
    }
}

// after a step: one more token generated; the position advances once the token has been fed
__global__ void advance_state_kernel(int* __restrict__ state, int advance_pos) {
    pdl_wait();
    pdl_launch_dependents();
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        state[1] += 1;
        if (advance_pos) state[0] += 1;
    }
}

int launch_argmax_rows(DeviceCtx* ctx, const float* logits, uint32_t* tok, uint32_t* out, int* state, int S, int V,
                       long long ld, int out_ld, int advance_pos, cudaStream_t st) {
    prof_mark(ctx, "argmax_rows", 0.0, 0.0, st);
    TB_CUDA(launch_kernel(argmax_rows_kernel, dim3(S), dim3(1024), 0, st, logits, tok, out, state, V, ld, out_ld));
    TB_LAUNCHED(ctx);
    prof_mark(ctx, "advance_state", 0.0, 0.0, st);
    TB_CUDA(launch_kernel(advance_state_kernel, dim3(1), dim3(32), 0, st, state, advance_pos));
    TB_LAUNCHED(ctx);
    return 0;
}

// Temperature sampling, sample_next of the reference's generator (training/generate.c:57-73):
// e_j = exp((z_j - max z) / temperature) in float32, r = u * sum_j e_j, the token is the first j whose running
// sum (float64, ascending j) reaches r; the last index if none does.  One block per sequence; thread t owns the
// contiguous columns [t * per, (t + 1) * per), so that the running sum is formed in ascending order: per-thread
// sums in column order, an exclusive scan over the threads in thread order.  u[state[1] * S + s] is the uniform
// draw of sequence s for generated token number state[1].
__global__ void __launch_bounds__(1024, 1)
sample_rows_kernel(const float* __restrict__ logits, const double* __restrict__ u, float temperature,
                   uint32_t* __restrict__ tok, uint32_t* __restrict__ out, const int* __restrict__ state, int S, int V,
                   long long ld, int out_ld) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float wmax[32];
    __shared__ double wsum[32];
    __shared__ int wfirst[32];
    const int sq = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float* z = logits + (long long)sq * ld;
    float mx = -3.0e38f;
    for (int j = tid; j < V; j += blockDim.x) mx = fmaxf(mx, z[j]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) wmax[warp] = mx;
    __syncthreads();
    mx = wmax[0];
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) mx = fmaxf(mx, wmax[w]);

    const int per = (V + (int)blockDim.x - 1) / (int)blockDim.x;
    const int j0 = min(tid * per, V), j1 = min(j0 + per, V);
    double local = 0.0;
    for (int j = j0; j < j1; ++j) local += (double)expf((z[j] - mx) / temperature);
    // inclusive scan inside the warp, then the warps' totals in warp order
    double incl = local;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const double v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) wsum[warp] = incl;
    __syncthreads();
    double before = 0.0, total = 0.0;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) {
        if (w < warp) before += wsum[w];
        total += wsum[w];
    }
    const double r = u[(long long)state[1] * S + sq] * total;
    double c = before + (incl - local);
    int first = 0x7fffffff;
    if (c + local >= r || j1 == V) {          // the crossing can only lie in a chunk whose end reaches r
        for (int j = j0; j < j1; ++j) {
            c += (double)expf((z[j] - mx) / temperature);
            if (c >= r) { first = j; break; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) first = min(first, __shfl_xor_sync(0xffffffffu, first, o));
    if (lane == 0) wfirst[warp] = first;
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w) first = min(first, wfirst[w]);
        if (first == 0x7fffffff) first = V - 1;
        tok[sq] = (uint32_t)first;
        if (out) out[(long long)sq * out_ld + state[1]] = (uint32_t)first;
    }
}

int launch_sample_rows(DeviceCtx* ctx, const float* logits, const double* u, float temperature, uint32_t* tok,
                       uint32_t* out, int* state, int S, int V, long long ld, int out_ld, int advance_pos,
                       cudaStream_t st) {
    prof_mark(ctx, "sample_rows", 0.0, 0.0, st);
    TB_CUDA(launch_kernel(sample_rows_kernel, dim3(S), dim3(1024), 0, st, logits, u, temperature, tok, out,
                          (const int*)state, S, V, ld, out_ld));
    TB_LAUNCHED(ctx);
    prof_mark(ctx, "advance_state", 0.0, 0.0, st);
    TB_CUDA(launch_kernel(advance_state_kernel, dim3(1), dim3(32), 0, st, state, advance_pos));
    TB_LAUNCHED(ctx);
    return 0;
}

// ------------------------------------------------------------- causal softmax
// Row i of a [T,T] score matrix: p_j = softmax_j(s_j * scale) over j <= i.  The reference adds
// -1e9 to j > i (model/attention.c:11), which underflows to exactly 0 after exp in float32, so
// leaving those entries out is the same function.  Zeros are written from i+1 to the end of the
// 128-wide tile that holds the diagonal: the following GEMMs read whole tiles up to there.
__global__ void attn_softmax_fwd_kernel(const float* __restrict__ S, bf16* __restrict__ P, long long rows, int T,
                                        long long ld, float scale) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int wpb = blockDim.x >> 5;
    for (long long row = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); row < rows;
         row += (long long)gridDim.x * wpb) {
        const int i = (int)(row % T);
        const float* s = S + row * ld;
        bf16* p = P + row * ld;
        float mx = -3.0e38f;
        for (int j = lane; j <= i; j += 32) mx = fmaxf(mx, s[j] * scale);
        mx = warp_max(mx);
        float sum = 0.0f;
        for (int j = lane; j <= i; j += 32) sum += expf(s[j] * scale - mx);
        sum = warp_sum(sum);
        for (int j = lane; j <= i; j += 32) p[j] = __float2bfloat16_rn(expf(s[j] * scale - mx) / sum);
        const int end = min(T, ((i >> 7) + 1) << 7);
        for (int j = i + 1 + lane; j < end; j += 32) p[j] = __float2bfloat16_rn(0.0f);
    }
}

int launch_attn_softmax_fwd(DeviceCtx* ctx, const float* S, bf16* P, int BH, int T, long long ld, float scale,
                            cudaStream_t st) {
    const long long rows = (long long)BH * T;
    prof_mark(ctx, "attn_softmax_fwd", 0.0, 0.0, st);
    TB_CUDA(launch_kernel(attn_softmax_fwd_kernel, dim3(grid_for(rows, 8, ctx, 32)), dim3(256), 0, st, S, P, rows, T, ld, scale));
    TB_LAUNCHED(ctx);
    return 0;
}

// dS = P * (dP - <dP, P>) * scale   (softmax backward then the score scale)
__global__ void attn_softmax_bwd_kernel(const bf16* __restrict__ P, const float* __restrict__ dP,
                                        bf16* __restrict__ dS, long long rows, int T, long long ld, float scale) {
    pdl_wait();
    pdl_launch_dependents();
    const int lane = threadIdx.x & 31;
    const int wpb = blockDim.x >> 5;
    for (long long row = (long long)blockIdx.x * wpb + (threadIdx.x >> 5); row < rows;
         row += (long long)gridDim.x * wpb) {
        const int i = (int)(row % T);
        const bf16* p = P + row * ld;
        const float* d = dP + row * ld;
        bf16* o = dS + row * ld;
        float dot = 0.0f;
        for (int j = lane; j <= i; j += 32) dot += d[j] * __bfloat162float(p[j]);
        dot = warp_sum(dot);
        for (int j = lane; j <= i; j += 32) o[j] = __float2bfloat16_rn(__bfloat162float(p[j]) * (d[j] - dot) * scale);
        const int end = min(T, ((i >> 7) + 1) << 7);
        for (int j = i + 1 + lane; j < end; j += 32) o[j] = __float2bfloat16_rn(0.0f);
    }
}

int launch_attn_softmax_bwd(DeviceCtx* ctx, const bf16* P, const float* dP, bf16* dS, int BH, int T, long long ld,
                            float scale, cudaStream_t st) {
    const long long rows = (long long)BH * T;
    prof_mark(ctx, "attn_softmax_bwd", 0.0, 0.0, st);
    TB_CUDA(launch_kernel(attn_softmax_bwd_kernel, dim3(grid_for(rows, 8, ctx, 32)), dim3(256), 0, st, P, dP, dS, rows, T, ld, scale));
    TB_LAUNCHED(ctx);
    return 0;
}

// dout [B*T, H*hd] -> dO [B,H,T,hd]
__global__ void heads_split_kernel(const bf16* __restrict__ dout, bf16* __restrict__ dO, int B, int T, int H,
                                   int hd) {
    pdl_wait();
    pdl_launch_dependents();
    const long long total = (long long)B * T * H * hd;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int d = (int)(i % hd);
        long long rest = i / hd;
        const int h = (int)(rest % H);
        const long long n = rest / H;
        const int t = (int)(n % T);
        const long long b = n / T;
        dO[((b * H + h) * T + t) * hd + d] = dout[i];
    }
}

int launch_heads_split(DeviceCtx* ctx, const bf16* dout, bf16* dO, int B, int T, int H, int hd, cudaStream_t st) {
    const long long total = (long long)B * T * H * hd;
    prof_mark(ctx, "heads_split", 0.0, 0.0, st);
    TB_CUDA(launch_kernel(heads_split_kernel, dim3(grid_for(total, 256, ctx)), dim3(256), 0, st, dout, dO, B, T, H, hd));
    TB_LAUNCHED(ctx);
    return 0;
}

// --------------------------------------------------------------------- SwiGLU
// h = g * sigmoid(g) * u with g = gu[:, :F], u = gu[:, F:]   (model/feedforward.c:9-14)
__global__ void swiglu_fwd_kernel(const float* __restrict__ gu, bf16* __restrict__ h, float* __restrict__ h32,
                                  long long total4, int F) {
    pdl_wait();
    pdl_launch_dependents();
    const int F4 = F >> 2;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total4;
         i += (long long)gridDim.x * blockDim.x) {
        const long long n = i / F4;
        const int j = (int)(i % F4) << 2;
        const float4 g = *reinterpret_cast<const float4*>(gu + n * 2 * F + j);
        const float4 u = *reinterpret_cast<const float4*>(gu + n * 2 * F + F + j);
        const float gg[4] = {g.x, g.y, g.z, g.w}, uu[4] = {u.x, u.y, u.z, u.w};
        float o[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float sg = 1.0f / (1.0f + expf(-gg[e]));
            o[e] = gg[e] * sg * uu[e];
        }
        if (h) {
            __nv_bfloat162 lo = __floats2bfloat162_rn(o[0], o[1]), hi = __floats2bfloat162_rn(o[2], o[3]);
            uint2 pk;
            pk.x = *reinterpret_cast<uint32_t*>(&lo); pk.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(h + n * F + j) = pk;
        }
        if (h32) *reinterpret_cast<float4*>(h32 + n * F + j) = make_float4(o[0], o[1], o[2], o[3]);
    }
}

int launch_swiglu_fwd(DeviceCtx* ctx, const float* gu, bf16* h, int rows, int F, cudaStream_t st, float* h32) {
    TB_CHECK(F % 4 == 0, "d_ff must be a multiple of 4");
    const long long total = (long long)rows * (F / 4);
    prof_mark(ctx, "swiglu_fwd", 0.0, 0.0, st);
    TB_CUDA(launch_kernel(swiglu_fwd_kernel, dim3(grid_for(total, 256, ctx)), dim3(256), 0, st, gu, h, h32, total, F));
    TB_LAUNCHED(ctx);
    return 0;
}

// dg = dh*u*(sg + g*sg*(1-sg)),  du = dh*g*sg
template <typename TG> struct Load4;
template <> struct Load4<float> {
    static __device__ __forceinline__ void at(const float* p, float (&o)[4]) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        o[0] = v.x; o[1] = v.y; o[2] = v.z; o[3] = v.w;
    }
};
template <> struct Load4<bf16> {
    static __device__ __forceinline__ void at(const bf16* p, float (&o)[4]) {
        const uint2 v = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&v.x);
        const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
        o[0] = __low2float(lo); o[1] = __high2float(lo); o[2] = __low2float(hi); o[3] = __high2float(hi);
    }
};

// TG = float: the stored projection; TG = bf16: the copy the fused SwiGLU GEMM epilogue keeps
template <typename TG>
__global__ void swiglu_bwd_kernel(const TG* __restrict__ gu, const float* __restrict__ dh,
                                  bf16* __restrict__ dgu, float* __restrict__ dgu32, long long total4, int F) {
    pdl_wait();
    pdl_launch_dependents();
    const int F4 = F >> 2;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total4;
         i += (long long)gridDim.x * blockDim.x) {
        const long long n = i / F4;
        const int j = (int)(i % F4) << 2;
        float gg[4], uu[4];
        Load4<TG>::at(gu + n * 2 * F + j, gg);
        Load4<TG>::at(gu + n * 2 * F + F + j, uu);
        const float4 d4 = *reinterpret_cast<const float4*>(dh + n * F + j);
        const float dd[4] = {d4.x, d4.y, d4.z, d4.w};
        float og[4], ou[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float sg = 1.0f / (1.0f + expf(-gg[e]));
            const float dsilu = dd[e] * uu[e];
            og[e] = dsilu * sg + dsilu * gg[e] * sg * (1.0f - sg);
            ou[e] = dd[e] * gg[e] * sg;
        }
        if (dgu) {
            __nv_bfloat162 a = __floats2bfloat162_rn(og[0], og[1]), b = __floats2bfloat162_rn(og[2], og[3]);
            __nv_bfloat162 c = __floats2bfloat162_rn(ou[0], ou[1]), d = __floats2bfloat162_rn(ou[2], ou[3]);
            uint2 pg, pu;
            pg.x = *reinterpret_cast<uint32_t*>(&a); pg.y = *reinterpret_cast<uint32_t*>(&b);
            pu.x = *reinterpret_cast<uint32_t*>(&c); pu.y = *reinterpret_cast<uint32_t*>(&d);
            *reinterpret_cast<uint2*>(dgu + n * 2 * F + j) = pg;
            *reinterpret_cast<uint2*>(dgu + n * 2 * F + F + j) = pu;
        }
        if (dgu32) {
            *reinterpret_cast<float4*>(dgu32 + n * 2 * F + j) = make_float4(og[0], og[1], og[2], og[3]);
            *reinterpret_cast<float4*>(dgu32 + n * 2 * F + F + j) = make_float4(ou[0], ou[1], ou[2], ou[3]);
        }
    }
}

int launch_swiglu_bwd(DeviceCtx* ctx, const float* gu, const float* dh, bf16* dgu, int rows, int F, cudaStream_t st,
                      float* dgu32) {
    TB_CHECK(F % 4 == 0, "d_ff must be a multiple of 4");
    const long long total = (long long)rows * (F / 4);
    prof_mark(ctx, "swiglu_bwd", 0.0, 0.0, st);
    TB_CUDA(launch_kernel(swiglu_bwd_kernel<float>, dim3(grid_for(total, 256, ctx)), dim3(256), 0, st, gu, dh, dgu, dgu32, total, F));
    TB_LAUNCHED(ctx);
    return 0;
}

int launch_swiglu_bwd_bf16(DeviceCtx* ctx, const bf16* gu, const float* dh, bf16* dgu, int rows, int F, cudaStream_t st) {
    TB_CHECK(F % 4 == 0, "d_ff must be a multiple of 4");
    const long long total = (long long)rows * (F / 4);
    prof_mark(ctx, "swiglu_bwd", 0.0, 0.0, st);
    TB_CUDA(launch_kernel(swiglu_bwd_kernel<bf16>, dim3(grid_for(total, 256, ctx)), dim3(256), 0, st, gu, dh, dgu, (float*)nullptr, total, F));
    TB_LAUNCHED(ctx);
    return 0;
}

// The same backward with the bias gradient of the gate|up projection (column sums of dgu, the reference's
// k_colsum_acc on it, cuda/train_kernels.cu:518-531) taken on the way: a thread owns four hidden units (four
// gate and four up columns) and walks its block's rows, so the eight column sums stay in its registers; each
// block leaves one partial row [2F] (sums of the bf16-rounded values, exactly what a column sum of dgu would
// add) and norm_partial_sum_kernel adds the partial rows in block order.
__global__ void swiglu_bwd_colsum_kernel(const bf16* __restrict__ gu, const float* __restrict__ dh,
                                         bf16* __restrict__ dgu, float* __restrict__ partial, int rows, int F) {
    pdl_wait();
    pdl_launch_dependents();
    const int rows_per = (rows + gridDim.x - 1) / gridDim.x;
    const int r0 = blockIdx.x * rows_per, r1 = min(rows, r0 + rows_per);
    for (int j = threadIdx.x * 4; j < F; j += blockDim.x * 4) {
        float sg_[4] = {0.f, 0.f, 0.f, 0.f}, su_[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 4
        for (int n = r0; n < r1; ++n) {
            float gg[4], uu[4];
            Load4<bf16>::at(gu + (long long)n * 2 * F + j, gg);
            Load4<bf16>::at(gu + (long long)n * 2 * F + F + j, uu);
            const float4 d4 = *reinterpret_cast<const float4*>(dh + (long long)n * F + j);
            const float dd[4] = {d4.x, d4.y, d4.z, d4.w};
            bf16 og[4], ou[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float sg = __fdividef(1.0f, 1.0f + exp2f_approx(-gg[e] * 1.4426950408889634f));   // ~1e-6 relative, far below bf16's
                const float dsilu = dd[e] * uu[e];
                og[e] = __float2bfloat16_rn(dsilu * sg + dsilu * gg[e] * sg * (1.0f - sg));
                ou[e] = __float2bfloat16_rn(dd[e] * gg[e] * sg);
                sg_[e] += __bfloat162float(og[e]);
                su_[e] += __bfloat162float(ou[e]);
            }
            uint2 pg, pu;
            __nv_bfloat162 a = __halves2bfloat162(og[0], og[1]), b = __halves2bfloat162(og[2], og[3]);
            __nv_bfloat162 c = __halves2bfloat162(ou[0], ou[1]), d = __halves2bfloat162(ou[2], ou[3]);
            pg.x = *reinterpret_cast<uint32_t*>(&a); pg.y = *reinterpret_cast<uint32_t*>(&b);
            pu.x = *reinterpret_cast<uint32_t*>(&c); pu.y = *reinterpret_cast<uint32_t*>(&d);
            *reinterpret_cast<uint2*>(dgu + (long long)n * 2 * F + j) = pg;
            *reinterpret_cast<uint2*>(dgu + (long long)n * 2 * F + F + j) = pu;
        }
        float* prow = partial + (long long)blockIdx.x * 2 * F;
        *reinterpret_cast<float4*>(prow + j) = make_float4(sg_[0], sg_[1], sg_[2], sg_[3]);
        *reinterpret_cast<float4*>(prow + F + j) = make_float4(su_[0], su_[1], su_[2], su_[3]);
    }
}

size_t swiglu_bwd_scratch_floats(int F) { return 64 + (size_t)kNormBwdBlocks * 2 * F; }

int launch_swiglu_bwd_colsum(DeviceCtx* ctx, const bf16* gu, const float* dh, bf16* dgu, float* dbias,
                             float* scratch, int rows, int F, cudaStream_t st) {
    TB_CHECK(F % 4 == 0, "d_ff must be a multiple of 4");
    int blocks = rows < kNormBwdBlocks ? rows : kNormBwdBlocks;
    float* partial = scratch + 64;
    const int threads = F / 4 >= 256 ? 256 : ((F / 4 + 31) / 32) * 32;
    prof_mark(ctx, "swiglu_bwd", 0.0, 0.0, st);
    TB_CUDA(launch_kernel(swiglu_bwd_colsum_kernel, dim3(blocks), dim3(threads), 0, st, gu, dh, dgu, partial, rows, F));
    TB_LAUNCHED(ctx);
    // blocks past the last row leave no partial row: only ceil(rows / rows_per) rows are valid
    const int rows_per = (rows + blocks - 1) / blocks;
    const int nb = (rows + rows_per - 1) / rows_per;
    prof_mark(ctx, "colsum_partials", 0.0, 0.0, st);
    TB_CUDA(launch_kernel(norm_partial_sum_kernel, dim3((2 * F + 31) / 32), dim3(32 * ((nb + 31) / 32)), 0, st,
                          (const float*)partial, nb, 2 * F, 2 * F, dbias, (float*)nullptr));
    TB_LAUNCHED(ctx);
    return 0;
}

// -------------------------------------------------------------- cross-entropy
__device__ __forceinline__ float block_reduce(float v, float* sh, bool is_max) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
    v = is_max ? warp_max(v) : warp_sum(v);
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    float r = sh[0];
    for (int k = 1; k < nw; ++k) r = is_max ? fmaxf(r, sh[k]) : r + sh[k];
    __syncthreads();
    return r;
}

// loss = log(sum exp(z - max)) + max - z[target];  dlogits = (softmax - onehot) * grad_scale
__global__ void cross_entropy_kernel(const float* __restrict__ logits, const uint32_t* __restrict__ targets,
                                     float* __restrict__ loss_rows, bf16* __restrict__ dlogits,
                                     float* __restrict__ dlogits32, int V, long long ld, float grad_scale) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float sh[32];
    const long long row = blockIdx.x;
    const float* z = logits + row * ld;
    const int t = (int)targets[row];
    float mx = -3.0e38f;
    for (int j = threadIdx.x; j < V; j += blockDim.x) mx = fmaxf(mx, z[j]);
    mx = block_reduce(mx, sh, true);
    float sum = 0.0f;
    for (int j = threadIdx.x; j < V; j += blockDim.x) sum += expf(z[j] - mx);
    sum = block_reduce(sum, sh, false);
    if (threadIdx.x == 0) loss_rows[row] = (float)log((double)sum) + mx - z[t];
    if (dlogits || dlogits32) {
        const float inv = 1.0f / sum;
        for (int j = threadIdx.x; j < V; j += blockDim.x) {
            float p = expf(z[j] - mx) * inv;
            if (j == t) p -= 1.0f;
            if (dlogits) dlogits[row * ld + j] = __float2bfloat16_rn(p * grad_scale);
            if (dlogits32) dlogits32[row * ld + j] = p * grad_scale;
        }
    }
}

// One read of the row: 1024 threads hold up to 32 logits each in registers (V <= 32768).
__global__ void __launch_bounds__(1024, 1)
cross_entropy_row_kernel(const float* __restrict__ logits, const uint32_t* __restrict__ targets,
                         float* __restrict__ loss_rows, bf16* __restrict__ dlogits, float* __restrict__ dlogits32, int V,
                         long long ld, float grad_scale) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float sh[32];
    const long long row = blockIdx.x;
    const float* z = logits + row * ld;
    const int t = (int)targets[row];
    float v[32];
    float mx = -3.0e38f;
#pragma unroll
    for (int k = 0; k < 32; ++k) {
        const int j = threadIdx.x + k * 1024;
        v[k] = j < V ? z[j] : -3.0e38f;
        mx = fmaxf(mx, v[k]);
    }
    mx = block_reduce(mx, sh, true);
    float sum = 0.0f;
#pragma unroll
    for (int k = 0; k < 32; ++k) {
        const int j = threadIdx.x + k * 1024;
        v[k] = j < V ? expf(v[k] - mx) : 0.0f;
        sum += v[k];
    }
    sum = block_reduce(sum, sh, false);
    if (threadIdx.x == 0) loss_rows[row] = (float)log((double)sum) + mx - z[t];
    if (dlogits || dlogits32) {
        const float inv = 1.0f / sum;
#pragma unroll
        for (int k = 0; k < 32; ++k) {
            const int j = threadIdx.x + k * 1024;
            if (j < V) {
                float p = v[k] * inv;
                if (j == t) p -= 1.0f;
                if (dlogits) dlogits[row * ld + j] = __float2bfloat16_rn(p * grad_scale);
                if (dlogits32) dlogits32[row * ld + j] = p * grad_scale;
            }
        }
    }
}

// Second half of the cross-entropy fused into the LM-head GEMM: the GEMM epilogue leaves, per row, `parts`
// pairs (max, sum exp(z - max)) over column ranges; their combination is the row's log-sum-exp, and
// loss = lse - z[target] (model/loss.c:31-73).  32 rows per block, 8 threads per row each taking every
// 8th pair in order, combined in thread order.
__global__ void ce_combine_kernel(const float2* __restrict__ stats, int parts, int rows,
                                  const float* __restrict__ ztarget, float* __restrict__ lse_out,
                                  float* __restrict__ loss_rows) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float shm[8][33], shs[8][33];
    const int rl = threadIdx.x & 31, g = threadIdx.x >> 5;
    const int row = blockIdx.x * 32 + rl;
    float m = -INFINITY, s = 0.0f;
    if (row < rows) {
        for (int t = g; t < parts; t += 8) {
            const float2 v = stats[(size_t)t * rows + row];
            if (v.x > -INFINITY) {
                const float mn = fmaxf(m, v.x);
                s = s * expf(m - mn) + v.y * expf(v.x - mn);
                m = mn;
            }
        }
    }
    shm[g][rl] = m; shs[g][rl] = s;
    __syncthreads();
    if (g == 0 && row < rows) {
        for (int k = 1; k < 8; ++k) {
            const float mk = shm[k][rl], sk = shs[k][rl];
            if (mk > -INFINITY) {
                const float mn = fmaxf(m, mk);
                s = s * expf(m - mn) + sk * expf(mk - mn);
                m = mn;
            }
        }
        const float lse = (float)log((double)s) + m;
        lse_out[row] = lse;
        loss_rows[row] = lse - ztarget[row];
    }
}

int launch_ce_combine(DeviceCtx* ctx, const float* stats, int parts, int rows, const float* ztarget, float* lse,
                      float* loss_rows, cudaStream_t st) {
    prof_mark(ctx, "ce_combine", 0.0, 0.0, st);
    TB_CUDA(launch_kernel(ce_combine_kernel, dim3((rows + 31) / 32), dim3(256), 0, st,
                          reinterpret_cast<const float2*>(stats), parts, rows, ztarget, lse, loss_rows));
    TB_LAUNCHED(ctx);
    return 0;
}

int launch_cross_entropy(DeviceCtx* ctx, const float* logits, const uint32_t* targets, float* loss_rows,
                         bf16* dlogits, int rows, int V, long long ld, float grad_scale, cudaStream_t st,
                         float* dlogits32) {
    prof_mark(ctx, "cross_entropy", 0.0, 0.0, st);
    if (V > 4096 && V <= 32768)
        TB_CUDA(launch_kernel(cross_entropy_row_kernel, dim3(rows), dim3(1024), 0, st, logits, targets, loss_rows, dlogits, dlogits32, V, ld, grad_scale));
    else
        TB_CUDA(launch_kernel(cross_entropy_kernel, dim3(rows), dim3(512), 0, st, logits, targets, loss_rows, dlogits, dlogits32, V, ld, grad_scale));
    TB_LAUNCHED(ctx);
    return 0;
}

// ---------------------------------------------------------------- column sums
// Stage 1: block (32 columns x 8 row-lanes) sums its chunk of rows -> partial[chunk][c];
// stage 2: out[c] += partial[0][c] + partial[1][c] + ... in chunk order.
constexpr int kColsumChunks = 64;

// scratch of a column sum: kTicketWords ticket words (one per 32-column group; they must start at
// zero and every launch leaves them at zero) followed by the partial sums [chunks][cols]
constexpr int kTicketWords = 256;
size_t colsum_partial_floats(int cols) { return (size_t)kTicketWords + (size_t)kColsumChunks * cols; }

template <typename T>
__device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

// One launch: every block writes the partial of its row chunk, takes a ticket, and the block that
// draws the last ticket of a 32-column group adds that group's partials in chunk order.  The
// ticket only decides WHO does the final sum, never its order, so the result is reproducible.
// Column sums of a [rows, cols] matrix, out[c] += sum_r in[r, c], in one launch.  A block owns 64
// columns (thread = 2 adjacent columns) x one chunk of rows; it writes the partial of its chunk,
// takes a ticket, and the block that draws the last ticket of a column group adds that group's
// partials in chunk order.  The ticket only decides WHO does the final sum, never its order.
__device__ __forceinline__ float2 load2(const float* p) { return *reinterpret_cast<const float2*>(p); }
__device__ __forceinline__ float2 load2(const bf16* p) {
    return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
}

// eight adjacent columns of one row (16 bytes of bf16, 32 bytes of float32)
__device__ __forceinline__ void load8(const float* p, float (&o)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
__device__ __forceinline__ void load8(const bf16* p, float (&o)[8]) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&w[k]));
        o[2 * k] = f.x; o[2 * k + 1] = f.y;
    }
}

// CW columns per thread (8 with 16-byte loads when cols % 8 == 0, else 2): a block owns 32 * CW columns x one
// chunk of rows; lane ty walks rows r0 + ty, + 8, ... with four loads in flight.
template <typename T, int CW>
__global__ void colsum_kernel(const T* __restrict__ in, float* __restrict__ out, float* __restrict__ partial,
                              unsigned int* __restrict__ tickets, int rows, int cols) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float part[8][32 * CW + 1];
    __shared__ int is_last;
    const int tx = threadIdx.x, ty = threadIdx.y;
    const int c = (blockIdx.x * 32 + tx) * CW;        // cols is a multiple of CW (checked by the launcher)
    const int chunk = blockIdx.y;
    const int per = (rows + kColsumChunks - 1) / kColsumChunks;
    const int r0 = chunk * per, r1 = min(rows, r0 + per);
    float s[CW];
#pragma unroll
    for (int e = 0; e < CW; ++e) s[e] = 0.0f;
    auto fetch = [&](int r, float (&o)[CW]) {
        if constexpr (CW == 8) {
            load8(in + (long long)r * cols + c, o);
        } else {
            const float2 v = load2(in + (long long)r * cols + c);
            o[0] = v.x; o[1] = v.y;
        }
    };
    if (c < cols) {
        int r = r0 + ty;
        for (; r + 24 < r1; r += 32) {               // four independent loads in flight
            float a[CW], b[CW], d[CW], e4[CW];
            fetch(r, a); fetch(r + 8, b); fetch(r + 16, d); fetch(r + 24, e4);
#pragma unroll
            for (int e = 0; e < CW; ++e) { s[e] += a[e]; s[e] += b[e]; s[e] += d[e]; s[e] += e4[e]; }
        }
        for (; r < r1; r += 8) {
            float a[CW];
            fetch(r, a);
#pragma unroll
            for (int e = 0; e < CW; ++e) s[e] += a[e];
        }
    }
#pragma unroll
    for (int e = 0; e < CW; ++e) part[ty][tx * CW + e] = s[e];
    __syncthreads();
    // the eight row-lanes of a column are added in lane order by one thread per column
    for (int j = ty * 32 + tx; j < 32 * CW; j += 256) {
        const int col = blockIdx.x * 32 * CW + j;
        if (col < cols) {
            float t = part[0][j];
#pragma unroll
            for (int k = 1; k < 8; ++k) t += part[k][j];
            partial[(long long)chunk * cols + col] = t;
        }
    }
    __threadfence();
    __syncthreads();
    if (tx == 0 && ty == 0) is_last = (atomicAdd(&tickets[blockIdx.x], 1u) == (unsigned)kColsumChunks - 1u);
    __syncthreads();
    if (is_last) {
        __threadfence();
        // the block that drew the last ticket of this column group adds the chunk partials in chunk order
        for (int j = ty * 32 + tx; j < 32 * CW; j += 256) {
            const int col = blockIdx.x * 32 * CW + j;
            if (col < cols) {
                float v[kColsumChunks];
#pragma unroll
                for (int k = 0; k < kColsumChunks; ++k) v[k] = __ldcg(&partial[(long long)k * cols + col]);
                float t = v[0];
#pragma unroll
                for (int k = 1; k < kColsumChunks; ++k) t += v[k];
                out[col] += t;
            }
        }
        if (tx == 0 && ty == 0) tickets[blockIdx.x] = 0u;     // ready for the next launch
    }
}

template <typename T>
static int colsum_impl(DeviceCtx* ctx, const T* in, float* out, float* partial, int rows, int cols, cudaStream_t st) {
    TB_CHECK((cols + 63) / 64 <= kTicketWords, "column sum supports at most %d columns", kTicketWords * 64);
    TB_CHECK(cols % 2 == 0, "column sum needs an even number of columns (got %d)", cols);
    unsigned int* tickets = reinterpret_cast<unsigned int*>(partial);
    prof_mark(ctx, "colsum", 0.0, 0.0, st);
    const bool wide = cols % 8 == 0 && (reinterpret_cast<uintptr_t>(in) & 15u) == 0;
    if (wide) {
        dim3 grid((cols + 255) / 256, kColsumChunks), block(32, 8);
        TB_CUDA(launch_kernel((colsum_kernel<T, 8>), dim3(grid), dim3(block), 0, st, in, out, partial + kTicketWords, tickets, rows, cols));
    } else {
        dim3 grid((cols + 63) / 64, kColsumChunks), block(32, 8);
        TB_CUDA(launch_kernel((colsum_kernel<T, 2>), dim3(grid), dim3(block), 0, st, in, out, partial + kTicketWords, tickets, rows, cols));
    }
    TB_LAUNCHED(ctx);
    return 0;
}

int launch_colsum_f32(DeviceCtx* ctx, const float* in, float* out, float* partial, int rows, int cols,
                      cudaStream_t st) {
    return colsum_impl<float>(ctx, in, out, partial, rows, cols, st);
}
int launch_colsum_bf16(DeviceCtx* ctx, const bf16* in, float* out, float* partial, int rows, int cols,
                       cudaStream_t st) {
    return colsum_impl<bf16>(ctx, in, out, partial, rows, cols, st);
}

// ------------------------------------------------------- gradient norm, Adam
__global__ void sumsq_partial_kernel(const float* __restrict__ x, long long n, float* __restrict__ partial) {
    pdl_wait();
    pdl_launch_dependents();
    __shared__ float sh[32];
    float s = 0.0f;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x)
        s += x[i] * x[i];
    s = block_reduce(s, sh, false);
    if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

int launch_sumsq_partial(DeviceCtx* ctx, const float* x, long long n, float* partial, cudaStream_t st) {
    prof_mark(ctx, "sumsq_partial", 0.0, 0.0, st);
    TB_CUDA(launch_kernel(sumsq_partial_kernel, dim3(kNormBlocks), dim3(256), 0, st, x, n, partial));
    TB_LAUNCHED(ctx);
    return 0;
}

// The reference sums the block partials on the host in float64 (model/gpu_train.c:508-511); one
// warp does that sum here so the step needs no host round trip: each lane adds a contiguous run of
// partials, then a fixed shuffle tree combines the lanes (same order every run).
__global__ void clip_scale_kernel(const float* __restrict__ partial, float max_norm, float grad_scale,
                                  float* __restrict__ scalars, double* __restrict__ norm64) {
    pdl_wait();
    pdl_launch_dependents();
    if (blockIdx.x != 0 || threadIdx.x >= 32) return;
    constexpr int PER = kNormBlocks / 32;
    static_assert(kNormBlocks % 32 == 0, "one contiguous run of partials per lane");
    float v[PER];
#pragma unroll
    for (int i = 0; i < PER; ++i) v[i] = partial[threadIdx.x * PER + i];
    double ss = 0.0;
#pragma unroll
    for (int i = 0; i < PER; ++i) ss += (double)v[i];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (threadIdx.x != 0) return;
    // the norm that is clipped is that of the gradients Adam will see: after grad_scale (1 / ranks after a sum
    // over ranks, 1 / micro-batches after accumulation), as the reference clips its averaged gradients
    const double norm = sqrt(ss) * (double)grad_scale;
    *norm64 = norm;
    scalars[0] = (float)norm;
    scalars[1] = (max_norm > 0.0f && norm > (double)max_norm) ? (float)((double)max_norm / norm) : 1.0f;
}

int launch_clip_scale(DeviceCtx* ctx, const float* partial, float max_norm, float grad_scale, float* scalars,
                      double* norm64, cudaStream_t st) {
    prof_mark(ctx, "clip_scale", 0.0, 0.0, st);
    TB_CUDA(launch_kernel(clip_scale_kernel, dim3(1), dim3(32), 0, st, partial, max_norm, grad_scale, scalars, norm64));
    TB_LAUNCHED(ctx);
    return 0;
}

// m = b1*m + (1-b1)*g; v = b2*v + (1-b2)*g^2; p -= lr * (m/bc1) / (sqrt(v/bc2) + eps)
// (training/adam.c:38-53).  The square root is IEEE sqrtf.
__global__ void adam_kernel(float* __restrict__ p, bf16* __restrict__ p16, const float* __restrict__ g,
                            float* __restrict__ m, float* __restrict__ v, long long n, float lr, float b1, float b2,
                            float eps, float bc1, float bc2, float grad_scale, const float* __restrict__ dev_scale) {
    pdl_wait();
    pdl_launch_dependents();
    const float gs = dev_scale ? grad_scale * dev_scale[1] : grad_scale;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n;
         i += (long long)gridDim.x * blockDim.x) {
        const float gi = g[i] * gs;
        const float mi = b1 * m[i] + (1.0f - b1) * gi;
        const float vi = b2 * v[i] + (1.0f - b2) * gi * gi;
        m[i] = mi;
        v[i] = vi;
        const float m_hat = mi / bc1;
        const float v_hat = vi / bc2;
        const float pi = p[i] - lr * m_hat / (sqrtf(v_hat) + eps);
        p[i] = pi;
        if (p16) p16[i] = __float2bfloat16_rn(pi);
    }
}

// The same update on four consecutive parameters per thread (16-byte loads and stores; the arithmetic of an
// element is that of adam_kernel, so the results are bit-identical).  n4 = n / 4 groups.
__global__ void adam_vec4_kernel(float4* __restrict__ p, uint2* __restrict__ p16, const float4* __restrict__ g,
                                 float4* __restrict__ m, float4* __restrict__ v, long long n4, float lr, float b1,
                                 float b2, float eps, float bc1, float bc2, float grad_scale,
                                 const float* __restrict__ dev_scale) {
    pdl_wait();
    pdl_launch_dependents();
    const float gs = dev_scale ? grad_scale * dev_scale[1] : grad_scale;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4;
         i += (long long)gridDim.x * blockDim.x) {
        const float4 g4 = g[i], m4 = m[i], v4 = v[i], p4 = p[i];
        const float gg[4] = {g4.x, g4.y, g4.z, g4.w}, mm[4] = {m4.x, m4.y, m4.z, m4.w};
        const float vv[4] = {v4.x, v4.y, v4.z, v4.w}, pp[4] = {p4.x, p4.y, p4.z, p4.w};
        float mo[4], vo[4], po[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const float gi = gg[k] * gs;
            const float mi = b1 * mm[k] + (1.0f - b1) * gi;
            const float vi = b2 * vv[k] + (1.0f - b2) * gi * gi;
            mo[k] = mi;
            vo[k] = vi;
            const float m_hat = mi / bc1;
            const float v_hat = vi / bc2;
            po[k] = pp[k] - lr * m_hat / (sqrtf(v_hat) + eps);
        }
        m[i] = make_float4(mo[0], mo[1], mo[2], mo[3]);
        v[i] = make_float4(vo[0], vo[1], vo[2], vo[3]);
        p[i] = make_float4(po[0], po[1], po[2], po[3]);
        if (p16) {
            const __nv_bfloat162 lo = __floats2bfloat162_rn(po[0], po[1]), hi = __floats2bfloat162_rn(po[2], po[3]);
            uint2 pk;
            pk.x = *reinterpret_cast<const uint32_t*>(&lo);
            pk.y = *reinterpret_cast<const uint32_t*>(&hi);
            p16[i] = pk;
        }
    }
}

int launch_adam(DeviceCtx* ctx, float* p, bf16* p16, const float* g, float* m, float* v, long long n, float lr,
                float b1, float b2, float eps, float bc1, float bc2, float grad_scale, const float* dev_scale,
                cudaStream_t st) {
    prof_mark(ctx, "adam", 0.0, 0.0, st);
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15u) == 0; };
    const long long n4 = (al16(p) && al16(g) && al16(m) && al16(v) && (!p16 || (reinterpret_cast<uintptr_t>(p16) & 7u) == 0))
                             ? n / 4 : 0;
    if (n4 > 0) {
        TB_CUDA(launch_kernel(adam_vec4_kernel, dim3(grid_for(n4, 256, ctx, 32)), dim3(256), 0, st,
                              reinterpret_cast<float4*>(p), reinterpret_cast<uint2*>(p16), reinterpret_cast<const float4*>(g),
                              reinterpret_cast<float4*>(m), reinterpret_cast<float4*>(v), n4, lr, b1, b2, eps, bc1, bc2,
                              grad_scale, dev_scale));
        TB_LAUNCHED(ctx);
    }
    const long long done = n4 * 4;
    if (done < n) {       // the last n % 4 parameters (or everything, when a buffer is not 16-byte aligned)
        TB_CUDA(launch_kernel(adam_kernel, dim3(grid_for(n - done, 256, ctx, 32)), dim3(256), 0, st, p + done,
                              p16 ? p16 + done : p16, g + done, m + done, v + done, n - done, lr, b1, b2, eps, bc1, bc2,
                              grad_scale, dev_scale));
        TB_LAUNCHED(ctx);
    }
    return 0;
}

}  // namespace tb
