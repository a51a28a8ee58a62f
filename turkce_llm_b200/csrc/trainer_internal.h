// What the data-parallel step (dp.cu) needs to see of a trainer (trainer.cu): the flat buffers, the stream all
// of the trainer's work is issued on, and the small device words of the clip + Adam sequence.
#pragma once
#include "common.h"

struct TbTrainer;

namespace tb {

// spare scalars behind the last parameter of every flat buffer (see tb_trainer_create)
constexpr long long kFlatPad = 1024;

struct TrainerView {
    DeviceCtx* ctx; cudaStream_t stream; int device;
    long long total, padded;
    float *params, *grads, *adam_m, *adam_v; bf16* params16;
    float* loss_rows; int B, T, L;
    float* norm_partial; float* scalars; double* norm64; double* h_norm;
};

int trainer_view(TbTrainer* g, TrainerView* out);

}  // namespace tb
