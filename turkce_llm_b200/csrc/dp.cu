// Data-parallel training step over the GPUs of one box: the multi-GPU extension of the reference's
// data_parallel_step (training/data_parallel.c:119-163).
//
// The reference runs one sequence per CPU worker thread on a shadow model, then adds the workers' gradients in
// a fixed order and divides by the worker count (dp_reduce_run, :102-117), and averages the workers' losses
// (:150-162).  Here a worker is a rank: one process (or host thread) per GPU, each with a full replica in its
// own TbTrainer.  A step is: every rank runs forward and backward on its own sequences; the flat float32
// gradient buffers (lm_collect_params order, 33,490,176 scalars = 134 MB for the 12-layer model) are summed
// over the ranks by NCCL over NVLink; 1 / ranks is folded into Adam's gradient scale; every rank applies the
// same clip factor and the same Adam update, so the replicas stay bit-identical.
//
// Two ways to combine (tb_dp_create's `mode`):
//   TB_DP_ALLREDUCE  one ncclAllReduce of the flat buffer; the rank's mean loss rides in a spare slot behind the
//                    last gradient, so the same collective averages the loss; every rank runs the whole Adam.
//   TB_DP_SHARDED    ncclReduceScatter: each rank receives the summed gradients of its contiguous 1/ranks slice
//                    only, adds up its share of the squared norm, one two-scalar all-reduce (float64) combines the
//                    norm and the loss, the rank runs Adam on its slice, and ncclAllGather returns the updated
//                    float32 weights of all slices; the bf16 shadow weights are re-formed locally.
//   TB_DP_OVERLAP    the all-reduce in per-layer buckets on a side stream while the layers below are still in backward
//                    (a layer's ten tensors are contiguous in the flat buffer and final once its backward has run;
//                    the final norm and the loss slot go first, the tied embedding, which receives gradient from the
//                    LM head first and from the token lookup last, goes last); the optimiser waits for the last bucket.
// Kernels of this library never touch another GPU's memory: all exchange is NCCL's.
//
// NCCL is looked up at run time (dlopen of libnccl.so.2, the copy the host process already has loaded if any),
// in the way the reference binds the CUDA driver by hand (cuda/driver_api.h:19-64): a process that never creates
// a communicator (one rank) needs no NCCL at all.
#include "../../include/turkce_b200.h"
#include "common.h"
#include "step_kernels.h"
#include "trainer_internal.h"

#include <dlfcn.h>
#include <nccl.h>

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

using namespace tb;

namespace {

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*ReduceScatter)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    ncclResult_t (*GetVersion)(int*) = nullptr;
};

NcclApi g_nccl;
std::mutex g_nccl_mutex;

int load_nccl() {
    std::lock_guard<std::mutex> lock(g_nccl_mutex);
    if (g_nccl.handle) return 0;
    const char* names[3] = {getenv("TB_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    void* h = nullptr;
    for (const char* n : names) {
        if (n == nullptr || *n == 0) continue;
        h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (h) break;
    }
    TB_CHECK(h != nullptr, "NCCL not found: dlopen(libnccl.so.2) failed (%s); set TB_NCCL_LIB to its path", dlerror());
#define TB_SYM(field, name)                                                       \
    do {                                                                          \
        *reinterpret_cast<void**>(&g_nccl.field) = dlsym(h, name);                \
        TB_CHECK(g_nccl.field != nullptr, "NCCL symbol %s not found", name);      \
    } while (0)
    TB_SYM(GetUniqueId, "ncclGetUniqueId");
    TB_SYM(CommInitRank, "ncclCommInitRank");
    TB_SYM(CommDestroy, "ncclCommDestroy");
    TB_SYM(AllReduce, "ncclAllReduce");
    TB_SYM(ReduceScatter, "ncclReduceScatter");
    TB_SYM(AllGather, "ncclAllGather");
    TB_SYM(GetErrorString, "ncclGetErrorString");
    TB_SYM(GetVersion, "ncclGetVersion");
#undef TB_SYM
    g_nccl.handle = h;
    return 0;
}

#define TB_NCCL(expr)                                                                              \
    do {                                                                                           \
        ncclResult_t _r = (expr);                                                                  \
        if (_r != ncclSuccess) {                                                                   \
            tb::set_error("[NCCL] %s -> %s (%s:%d)", #expr, g_nccl.GetErrorString(_r), __FILE__, __LINE__); \
            return -4;                                                                             \
        }                                                                                          \
    } while (0)

// Mean loss of this rank's batch, in the order the host code uses (mean inside a sequence, then over the
// sequences: model/gpu_train.c:478-487), written or added to *slot.  Each warp takes sequences in turn: its lanes
// fetch 32 consecutive rows at a time (one coalesced load) and lane 0 adds them in row order, so the sum is the
// sequential float32 sum of the host loop.
__global__ void loss_mean_kernel(const float* __restrict__ loss_rows, int B, int T, float* __restrict__ slot, int accumulate) {
    pdl_wait();
    pdl_launch_dependents();
    extern __shared__ float per_seq[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    for (int b = warp; b < B; b += nwarps) {
        const float* r = loss_rows + (size_t)b * T;
        float s = 0.0f;
        for (int t0 = 0; t0 < T; t0 += 128) {
            float v[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) v[k] = t0 + k * 32 + lane < T ? r[t0 + k * 32 + lane] : 0.0f;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int n = min(32, T - (t0 + k * 32));
                if (n == 32) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) s += __shfl_sync(0xffffffffu, v[k], j);   // every lane forms the same sum
                } else {
                    for (int j = 0; j < n; ++j) s += __shfl_sync(0xffffffffu, v[k], j);
                }
            }
        }
        if (lane == 0) per_seq[b] = s / (float)T;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        float sum = 0.0f;
        for (int b = 0; b < B; ++b) sum += per_seq[b];
        const float mean = sum / (float)B;
        *slot = accumulate ? *slot + mean : mean;
    }
}

// pair[0] = sum of the rank's kNormBlocks partial sums of squares in float64 (contiguous runs per lane, then a
// fixed shuffle tree: the order clip_scale_kernel uses), pair[1] = the rank's loss.
__global__ void sumsq_pair_kernel(const float* __restrict__ partial, const float* __restrict__ loss_slot,
                                  double* __restrict__ pair) {
    pdl_wait();
    pdl_launch_dependents();
    if (blockIdx.x != 0 || threadIdx.x >= 32) return;
    constexpr int PER = kNormBlocks / 32;
    double ss = 0.0;
    for (int i = 0; i < PER; ++i) ss += (double)partial[threadIdx.x * PER + i];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (threadIdx.x == 0) { pair[0] = ss; pair[1] = (double)*loss_slot; }
}

// From the squared norm summed over all ranks' slices: scalars[0] = norm, scalars[1] = clip factor (the same
// arithmetic as clip_scale_kernel from its sum on).
__global__ void clip_from_pair_kernel(const double* __restrict__ pair, float max_norm, float grad_scale,
                                      float* __restrict__ scalars, double* __restrict__ norm64) {
    pdl_wait();
    pdl_launch_dependents();
    if (blockIdx.x != 0 || threadIdx.x != 0) return;
    const double norm = sqrt(pair[0]) * (double)grad_scale;
    *norm64 = norm;
    scalars[0] = (float)norm;
    scalars[1] = (max_norm > 0.0f && norm > (double)max_norm) ? (float)((double)max_norm / norm) : 1.0f;
}

}  // namespace

struct TbDp {
    TbTrainer* g = nullptr;
    TrainerView v;
    int rank = 0, world = 1, mode = TB_DP_ALLREDUCE;
    ncclComm_t comm = nullptr;
    long long chunk = 0, lo = 0, own = 0;   // sharded mode: slice [lo, lo + own) of the flat buffers
    cudaStream_t side = nullptr;            // overlap mode: the stream the bucket all-reduces run on
    cudaEvent_t ev_ready = nullptr, ev_done = nullptr;
    std::vector<long long> bucket_lo, bucket_hi;      // [0] final norm (+ loss slot), [1 + i] layer L-1-i, [L + 1] embedding
    double* d_pair = nullptr;               // {sum of squares, loss} for the two-scalar all-reduce
    double* h_pair = nullptr;               // pinned
    float* h_loss = nullptr;                // pinned
};

namespace {

// overlap mode: bucket b is final on the trainer's stream now; reduce it on the side stream
int reduce_bucket(TbDp* dp, size_t b) {
    const TrainerView& v = dp->v;
    TB_CUDA(cudaEventRecord(dp->ev_ready, v.stream));
    TB_CUDA(cudaStreamWaitEvent(dp->side, dp->ev_ready, 0));
    float* p = v.grads + dp->bucket_lo[b];
    TB_NCCL(g_nccl.AllReduce(p, p, (size_t)(dp->bucket_hi[b] - dp->bucket_lo[b]), ncclFloat32, ncclSum, dp->comm, dp->side));
    return 0;
}

// The backward pass of one batch.  reduce: this is the step's last micro-batch and the mode is TB_DP_OVERLAP.
int backward_all(TbDp* dp, bool reduce = false) {
    if (!reduce) return trainer_backward_all(dp->g);      // no collective between the layers: one graph
    size_t b = 0;
    TB_TRY(tb_trainer_backward_head(dp->g));
    if (reduce) TB_TRY(reduce_bucket(dp, b++));
    for (int l = dp->v.L - 1; l >= 0; --l) {
        TB_TRY(tb_trainer_backward_layer(dp->g, l));
        if (reduce) TB_TRY(reduce_bucket(dp, b++));
    }
    TB_TRY(tb_trainer_backward_embed(dp->g));
    if (reduce) {
        TB_TRY(reduce_bucket(dp, b++));
        // the optimiser (on the trainer's stream) waits for the last bucket
        TB_CUDA(cudaEventRecord(dp->ev_done, dp->side));
        TB_CUDA(cudaStreamWaitEvent(dp->v.stream, dp->ev_done, 0));
    }
    return 0;
}

int mean_loss_to_slot(TbDp* dp, int accumulate) {
    const TrainerView& v = dp->v;
    TB_TRY(trainer_grads_ready(dp->g));        // the slot lies in the gradient buffer, which may still be being cleared
    const int threads = 32 * (v.B < 32 ? v.B : 32);          // one warp per sequence, up to 32 warps
    prof_mark(v.ctx, "loss_mean", 0.0, 0.0, v.stream);
    TB_CUDA(launch_kernel(loss_mean_kernel, dim3(1), dim3(threads), (size_t)v.B * sizeof(float), v.stream, v.loss_rows,
                          v.B, v.T, v.grads + v.total, accumulate));
    TB_CUDA(cudaGetLastError());
    v.ctx->launches++;
    prof_close(v.ctx, v.stream);
    return 0;
}

// Everything between the last backward kernel and the end of the optimiser step.  `parts` = micro-batches
// accumulated in the gradient buffer and in the loss slot.
int combine_and_update(TbDp* dp, uint64_t t, float lr, float b1, float b2, float eps, float max_norm, int parts) {
    const TrainerView& v = dp->v;
    const float scale = 1.0f / ((float)dp->world * (float)parts);
    if (dp->world == 1 || dp->mode == TB_DP_ALLREDUCE || dp->mode == TB_DP_OVERLAP) {
        if (dp->world > 1 && dp->mode == TB_DP_ALLREDUCE)      // gradients and the loss slot behind them in one collective
            TB_NCCL(g_nccl.AllReduce(v.grads, v.grads, (size_t)v.total + 1, ncclFloat32, ncclSum, dp->comm, v.stream));
        TB_TRY(tb_trainer_clip_adam_async(dp->g, t, lr, b1, b2, eps, max_norm, scale));
        TB_CUDA(cudaMemcpyAsync(dp->h_loss, v.grads + v.total, sizeof(float), cudaMemcpyDeviceToHost, v.stream));
        return 0;
    }
    // sharded: this rank's slice of the summed gradients, its share of the squared norm, Adam on the slice
    TB_NCCL(g_nccl.ReduceScatter(v.grads, v.grads + dp->lo, (size_t)dp->chunk, ncclFloat32, ncclSum, dp->comm, v.stream));
    if (dp->own > 0) {
        TB_TRY(launch_sumsq_partial(v.ctx, v.grads + dp->lo, dp->own, v.norm_partial, v.stream));
    } else {
        TB_CUDA(cudaMemsetAsync(v.norm_partial, 0, kNormBlocks * sizeof(float), v.stream));
    }
    TB_CUDA(launch_kernel(sumsq_pair_kernel, dim3(1), dim3(32), 0, v.stream, (const float*)v.norm_partial,
                          (const float*)(v.grads + v.total), dp->d_pair));
    TB_NCCL(g_nccl.AllReduce(dp->d_pair, dp->d_pair, 2, ncclFloat64, ncclSum, dp->comm, v.stream));
    TB_CUDA(launch_kernel(clip_from_pair_kernel, dim3(1), dim3(32), 0, v.stream, (const double*)dp->d_pair, max_norm, scale,
                          v.scalars, v.norm64));
    TB_CUDA(cudaGetLastError());
    v.ctx->launches += 2;
    TB_CUDA(cudaMemcpyAsync(v.h_norm, v.norm64, sizeof(double), cudaMemcpyDeviceToHost, v.stream));
    TB_CUDA(cudaMemcpyAsync(dp->h_pair, dp->d_pair, 2 * sizeof(double), cudaMemcpyDeviceToHost, v.stream));
    if (dp->own > 0) {
        const float bc1 = 1.0f - powf(b1, (float)t), bc2 = 1.0f - powf(b2, (float)t);
        TB_TRY(launch_adam(v.ctx, v.params + dp->lo, v.params16 + dp->lo, v.grads + dp->lo, v.adam_m + dp->lo,
                           v.adam_v + dp->lo, dp->own, lr, b1, b2, eps, bc1, bc2, scale, v.scalars, v.stream));
    }
    TB_NCCL(g_nccl.AllGather(v.params + dp->lo, v.params, (size_t)dp->chunk, ncclFloat32, dp->comm, v.stream));
    // the bf16 shadow of the other ranks' slices (and, again, of this one) from the gathered float32 weights
    TB_TRY(launch_pack_bf16(v.ctx, v.params, v.params16, 1, (int)v.total, v.total, v.total, 1, 0, 0, v.stream));
    return 0;
}

int finish(TbDp* dp, int parts, float* loss_out, double* norm_out) {
    const TrainerView& v = dp->v;
    TB_TRY(check_device_error(v.ctx, v.stream));      // waits for the stream
    float loss;
    if (dp->world > 1 && dp->mode == TB_DP_SHARDED) loss = (float)(dp->h_pair[1] / ((double)dp->world * parts));
    else loss = *dp->h_loss / ((float)dp->world * (float)parts);
    if (loss_out) *loss_out = loss;
    if (norm_out) *norm_out = *v.h_norm;
    return 0;
}

}  // namespace

extern "C" {

int tb_dp_unique_id(void* id_out_128_bytes) {
    TB_CHECK(id_out_128_bytes != nullptr, "tb_dp_unique_id: NULL output");
    TB_TRY(load_nccl());
    static_assert(sizeof(ncclUniqueId) == 128, "ncclUniqueId is 128 bytes");
    ncclUniqueId id;
    TB_NCCL(g_nccl.GetUniqueId(&id));
    memcpy(id_out_128_bytes, &id, sizeof(id));
    return 0;
}

int tb_dp_slice(int64_t total, int world, int rank, int64_t* chunk, int64_t* first, int64_t* count) {
    TB_CHECK(total > 0 && world >= 1 && rank >= 0 && rank < world, "tb_dp_slice: rank %d of %d over %lld scalars", rank, world,
             (long long)total);
    // equal chunks of a multiple of 8 scalars (16-byte boundaries in float32 and in bf16); the last ranks' chunks may
    // reach past the last parameter into the padding of the flat buffers, and own fewer (or no) parameters
    const int64_t c = round_up((total + world - 1) / world, 8);
    const int64_t lo = c * rank;
    const int64_t hi = lo + c < total ? lo + c : total;
    if (chunk) *chunk = c;
    if (first) *first = lo;
    if (count) *count = hi > lo ? hi - lo : 0;
    return 0;
}

int tb_dp_create(TbDp** out, TbTrainer* g, const void* unique_id, int rank, int world, int mode) {
    TB_CHECK(out != nullptr && g != nullptr, "tb_dp_create: NULL argument");
    TB_CHECK(world >= 1 && rank >= 0 && rank < world, "tb_dp_create: rank %d of %d", rank, world);
    TB_CHECK(mode == TB_DP_ALLREDUCE || mode == TB_DP_SHARDED || mode == TB_DP_OVERLAP, "tb_dp_create: unknown mode %d", mode);
    TbDp* dp = new TbDp();
    dp->g = g; dp->rank = rank; dp->world = world; dp->mode = mode;
    TB_TRY(trainer_view(g, &dp->v));
    TB_CUDA(cudaSetDevice(dp->v.device));
    TB_CUDA(cudaMallocHost(&dp->h_loss, sizeof(float)));
    TB_CUDA(cudaMallocHost(&dp->h_pair, 2 * sizeof(double)));
    TB_CUDA(cudaMalloc(&dp->d_pair, 2 * sizeof(double)));
    *dp->h_loss = 0.0f; dp->h_pair[0] = dp->h_pair[1] = 0.0;
    int64_t chunk = 0, lo = 0, own = 0;
    TB_TRY(tb_dp_slice(dp->v.total, world, rank, &chunk, &lo, &own));
    dp->chunk = chunk; dp->lo = lo; dp->own = own;
    TB_CHECK(dp->chunk * world <= dp->v.padded, "tb_dp_create: %d ranks need %lld scalars, the flat buffers hold %lld",
             world, dp->chunk * world, dp->v.padded);
    if (world > 1 && mode == TB_DP_OVERLAP) {
        TB_CUDA(cudaStreamCreateWithFlags(&dp->side, cudaStreamNonBlocking));
        TB_CUDA(cudaEventCreateWithFlags(&dp->ev_ready, cudaEventDisableTiming));
        TB_CUDA(cudaEventCreateWithFlags(&dp->ev_done, cudaEventDisableTiming));
        const int np = tb_trainer_num_params(g);
        std::vector<int64_t> off(np), num(np);
        TB_TRY(tb_trainer_param_layout(g, off.data(), num.data()));
        const int L = dp->v.L;
        dp->bucket_lo.push_back(off[np - 1]); dp->bucket_hi.push_back(dp->v.total + 1);      // final norm + the loss slot
        for (int l = L - 1; l >= 0; --l) {
            dp->bucket_lo.push_back(off[1 + 10 * l]);
            dp->bucket_hi.push_back(l + 1 < L ? off[1 + 10 * (l + 1)] : off[np - 1]);
        }
        dp->bucket_lo.push_back(0); dp->bucket_hi.push_back(np > 1 ? off[1] : dp->v.total);
    }
    if (world > 1) {
        TB_CHECK(unique_id != nullptr, "tb_dp_create: %d ranks need the 128-byte id from tb_dp_unique_id", world);
        TB_TRY(load_nccl());
        ncclUniqueId id;
        memcpy(&id, unique_id, sizeof(id));
        TB_NCCL(g_nccl.CommInitRank(&dp->comm, world, id, rank));
    }
    *out = dp;
    return 0;
}

int tb_dp_destroy(TbDp* dp) {
    if (!dp) return 0;
    cudaSetDevice(dp->v.device);
    cudaStreamSynchronize(dp->v.stream);
    if (dp->side) cudaStreamSynchronize(dp->side);
    if (dp->comm) g_nccl.CommDestroy(dp->comm);
    if (dp->side) cudaStreamDestroy(dp->side);
    if (dp->ev_ready) cudaEventDestroy(dp->ev_ready);
    if (dp->ev_done) cudaEventDestroy(dp->ev_done);
    cudaFreeHost(dp->h_loss); cudaFreeHost(dp->h_pair); cudaFree(dp->d_pair);
    delete dp;
    return 0;
}

int tb_dp_info(const TbDp* dp, int* rank, int* world, int* mode, int* nccl_version) {
    TB_CHECK(dp != nullptr, "tb_dp_info: NULL handle");
    if (rank) *rank = dp->rank;
    if (world) *world = dp->world;
    if (mode) *mode = dp->mode;
    if (nccl_version) {
        *nccl_version = 0;
        if (g_nccl.handle) g_nccl.GetVersion(nccl_version);
    }
    return 0;
}

int tb_dp_step(TbDp* dp, const uint32_t* h_ids, const uint32_t* h_targets, int micro_batches, uint64_t t, float lr,
               float beta1, float beta2, float eps, float max_norm, float* loss_out, double* norm_out) {
    TB_CHECK(dp != nullptr && h_ids != nullptr && h_targets != nullptr, "tb_dp_step: NULL argument");
    TB_CHECK(micro_batches >= 1, "tb_dp_step: micro_batches must be at least 1");
    const TrainerView& v = dp->v;
    TB_CUDA(cudaSetDevice(v.device));
    const size_t n = (size_t)v.B * v.T;
    TB_TRY(tb_trainer_zero_grads(dp->g));          // also clears the loss slot
    const bool overlap = dp->world > 1 && dp->mode == TB_DP_OVERLAP;
    for (int i = 0; i < micro_batches; ++i) {
        TB_TRY(tb_trainer_forward(dp->g, h_ids + i * n, h_targets + i * n, 1));
        TB_TRY(mean_loss_to_slot(dp, 1));          // the loss rows are final after the forward pass
        TB_TRY(backward_all(dp, overlap && i + 1 == micro_batches));
    }
    TB_TRY(combine_and_update(dp, t, lr, beta1, beta2, eps, max_norm, micro_batches));
    return finish(dp, micro_batches, loss_out, norm_out);
}

int tb_dp_step_resident(TbDp* dp, uint64_t t, float lr, float beta1, float beta2, float eps, float max_norm) {
    TB_CHECK(dp != nullptr, "tb_dp_step_resident: NULL handle");
    TB_CUDA(cudaSetDevice(dp->v.device));
    TB_TRY(tb_trainer_zero_grads(dp->g));
    TB_TRY(tb_trainer_forward_resident(dp->g, 1));
    TB_TRY(mean_loss_to_slot(dp, 1));
    TB_TRY(backward_all(dp, dp->world > 1 && dp->mode == TB_DP_OVERLAP));
    return combine_and_update(dp, t, lr, beta1, beta2, eps, max_norm, 1);
}

int tb_dp_last_result(TbDp* dp, float* loss_out, double* norm_out) {
    TB_CHECK(dp != nullptr, "tb_dp_last_result: NULL handle");
    return finish(dp, 1, loss_out, norm_out);
}

}  // extern "C"
