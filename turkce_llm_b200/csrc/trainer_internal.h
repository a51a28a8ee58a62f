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
// tb_trainer_zero_grads may clear the gradient buffer on the trainer's second stream while the forward pass runs;
// whoever writes into the flat gradient buffer (or its loss slot) first calls this before.
int trainer_grads_ready(TbTrainer* g);
// head, layers L-1 .. 0 and embedding backward as ONE graph (tb_trainer_backward_head / _layer / _embed are a graph each,
// for a caller that puts collectives between them)
int trainer_backward_all(TbTrainer* g);

}  // namespace tb
