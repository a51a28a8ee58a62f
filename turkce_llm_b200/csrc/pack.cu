// float32 -> bf16 operand packing for callers that keep their matrices in float32, as the
// reference does (its kernels convert while staging tiles: cuda/train_kernels.cu:256-263).
// Rounding is round-to-nearest-even, the same as the reference's f32_to_bf16
// (cuda/train_kernels.cu:207-212) on every finite input.
//
// The packed copy gets a leading dimension that is a multiple of 8 elements so that TMA can
// address it whatever the source's leading dimension was (the 31,769-column logits included).
#include "common.h"

namespace tb {

__global__ void pack_bf16_kernel(const float* __restrict__ src, bf16* __restrict__ dst, int rows, int cols,
                                 long long ld_src, long long ld_dst, long long stride_src, long long stride_dst,
                                 int vec) {
    pdl_wait();
    pdl_launch_dependents();
    const int z = blockIdx.z;
    const float* s = src + (long long)z * stride_src;
    bf16* d = dst + (long long)z * stride_dst;
    if (vec) {
        const int c4 = cols >> 2;
        const long long total = (long long)rows * c4;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
             i += (long long)gridDim.x * blockDim.x) {
            const long long r = i / c4;
            const int c = (int)(i % c4) << 2;
            const float4 v = *reinterpret_cast<const float4*>(s + r * ld_src + c);
            __nv_bfloat162 lo = __floats2bfloat162_rn(v.x, v.y);
            __nv_bfloat162 hi = __floats2bfloat162_rn(v.z, v.w);
            uint2 pk;
            pk.x = *reinterpret_cast<uint32_t*>(&lo);
            pk.y = *reinterpret_cast<uint32_t*>(&hi);
            *reinterpret_cast<uint2*>(d + r * ld_dst + c) = pk;
        }
    } else {
        const long long total = (long long)rows * cols;
        for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
             i += (long long)gridDim.x * blockDim.x) {
            const long long r = i / cols;
            const int c = (int)(i % cols);
            d[r * ld_dst + c] = __float2bfloat16_rn(s[r * ld_src + c]);
        }
    }
}

int launch_pack_bf16(DeviceCtx* ctx, const float* src, bf16* dst, int rows, int cols, long long ld_src,
                     long long ld_dst, int batch, long long stride_src, long long stride_dst, cudaStream_t stream) {
    TB_CHECK(rows > 0 && cols > 0 && batch > 0, "pack: empty matrix");
    const int vec = (cols % 4 == 0) && (ld_src % 4 == 0) && (ld_dst % 4 == 0) && (stride_src % 4 == 0) &&
                    (stride_dst % 4 == 0) && (reinterpret_cast<uintptr_t>(src) % 16 == 0) &&
                    (reinterpret_cast<uintptr_t>(dst) % 8 == 0);
    const long long work = (long long)rows * (vec ? cols / 4 : cols);
    long long blocks = (work + 255) / 256;
    const long long cap = 8LL * ctx->sm_count;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    dim3 grid((unsigned)blocks, 1, (unsigned)batch);
    prof_mark(ctx, "pack_bf16", 0.0, (double)rows * cols * batch * 6.0, stream);
    TB_CUDA(launch_kernel(pack_bf16_kernel, dim3(grid), dim3(256), 0, stream, src, dst, rows, cols, ld_src, ld_dst, stride_src, stride_dst, vec));
    TB_CUDA(cudaGetLastError());
    ctx->launches++;
    prof_close(ctx, stream);
    return 0;
}

__global__ void copy_f32_kernel(const float* __restrict__ src, float* __restrict__ dst, int rows, int cols,
                                long long ld_src, long long ld_dst, long long stride_src, long long stride_dst) {
    pdl_wait();
    pdl_launch_dependents();
    const float* s = src + (long long)blockIdx.z * stride_src;
    float* d = dst + (long long)blockIdx.z * stride_dst;
    const long long total = (long long)rows * cols;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cols;
        const int c = (int)(i % cols);
        d[r * ld_dst + c] = s[r * ld_src + c];
    }
}

int launch_copy_f32(DeviceCtx* ctx, const float* src, float* dst, int rows, int cols, long long ld_src,
                    long long ld_dst, int batch, long long stride_src, long long stride_dst, cudaStream_t stream) {
    TB_CHECK(rows > 0 && cols > 0 && batch > 0, "copy: empty matrix");
    long long blocks = ((long long)rows * cols + 255) / 256;
    if (blocks > 8LL * ctx->sm_count) blocks = 8LL * ctx->sm_count;
    dim3 grid((unsigned)blocks, 1, (unsigned)batch);
    prof_mark(ctx, "copy_f32", 0.0, (double)rows * cols * batch * 8.0, stream);
    TB_CUDA(launch_kernel(copy_f32_kernel, dim3(grid), dim3(256), 0, stream, src, dst, rows, cols, ld_src, ld_dst, stride_src, stride_dst));
    TB_CUDA(cudaGetLastError());
    ctx->launches++;
    prof_close(ctx, stream);
    return 0;
}

// hi keeps the 19 bits a tf32 operand has (sign, 8 exponent, 10 mantissa); lo = x - hi is exact in
// float32 and itself enters the tensor core truncated to tf32, which loses about 2^-21 of x.
__global__ void split3_f32_kernel(const float* __restrict__ src, float* __restrict__ dst, int rows, int cols,
                                  long long ld_src, long long ld_dst, int along_cols, int pattern,
                                  long long stride_src, long long stride_dst) {
    pdl_wait();
    pdl_launch_dependents();
    const float* s = src + (long long)blockIdx.z * stride_src;
    float* d = dst + (long long)blockIdx.z * stride_dst;
    const long long total = (long long)rows * cols;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cols;
        const int c = (int)(i % cols);
        const float x = s[r * ld_src + c];
        const float hi = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
        const float lo = x - hi;
        const float p1 = pattern == 0 ? hi : lo;
        const float p2 = pattern == 0 ? lo : hi;
        if (along_cols) {
            d[r * ld_dst + c] = hi;
            d[r * ld_dst + cols + c] = p1;
            d[r * ld_dst + 2LL * cols + c] = p2;
        } else {
            d[r * ld_dst + c] = hi;
            d[(r + rows) * ld_dst + c] = p1;
            d[(r + 2LL * rows) * ld_dst + c] = p2;
        }
    }
}

int launch_split3_f32(DeviceCtx* ctx, const float* src, float* dst, int rows, int cols, long long ld_src,
                      long long ld_dst, int along_cols, int pattern, int batch, long long stride_src,
                      long long stride_dst, cudaStream_t stream) {
    TB_CHECK(rows > 0 && cols > 0 && batch > 0, "split: empty matrix");
    long long blocks = ((long long)rows * cols + 255) / 256;
    if (blocks > 8LL * ctx->sm_count) blocks = 8LL * ctx->sm_count;
    dim3 grid((unsigned)blocks, 1, (unsigned)batch);
    prof_mark(ctx, "split3_f32", 0.0, (double)rows * cols * batch * 16.0, stream);
    TB_CUDA(launch_kernel(split3_f32_kernel, dim3(grid), dim3(256), 0, stream, src, dst, rows, cols, ld_src, ld_dst, along_cols, pattern, stride_src, stride_dst));
    TB_CUDA(cudaGetLastError());
    ctx->launches++;
    prof_close(ctx, stream);
    return 0;
}

}  // namespace tb

namespace tb {

// bf16 -> float32 (exact): the TF32 mode of the trainer widens the outputs of the attention kernels, which
// stay bf16, before they enter a float32-operand GEMM.  n must be a multiple of 4, pointers 16-byte aligned.
__global__ void widen_bf16_kernel(const uint2* __restrict__ src, float4* __restrict__ dst, long long n4) {
    pdl_wait();
    pdl_launch_dependents();
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
        const uint2 v = src[i];
        const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&v.x);
        const __nv_bfloat162 hi = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
        dst[i] = make_float4(__low2float(lo), __high2float(lo), __low2float(hi), __high2float(hi));
    }
}

int launch_widen_bf16(DeviceCtx* ctx, const bf16* src, float* dst, long long n, cudaStream_t stream) {
    TB_CHECK(n > 0 && n % 4 == 0, "widen: element count must be a positive multiple of 4");
    long long blocks = (n / 4 + 255) / 256;
    if (blocks > 8LL * ctx->sm_count) blocks = 8LL * ctx->sm_count;
    prof_mark(ctx, "widen_bf16", 0.0, (double)n * 6.0, stream);
    TB_CUDA(launch_kernel(widen_bf16_kernel, dim3((unsigned)blocks), dim3(256), 0, stream,
                          reinterpret_cast<const uint2*>(src), reinterpret_cast<float4*>(dst), n / 4));
    TB_CUDA(cudaGetLastError());
    ctx->launches++;
    prof_close(ctx, stream);
    return 0;
}

}  // namespace tb
