// Host side of the training loop around TbTrainer: window sampling, learning-rate schedule,
// checkpoints in the reference's file format, and the loop itself.  Mirrors what the reference's
// training/train_lm_gpu.c does around gpu_trainer_*; no kernels here.
#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>
#include <vector>

#include "common.h"
#include "pcg32.h"
#include "turkce_b200.h"

namespace {

using tb::Pcg32;

struct Dims { int V, D, H, L, F, T, B; };

int get_dims(const TbTrainer* g, Dims* d) { return tb_trainer_dims(g, &d->V, &d->D, &d->H, &d->L, &d->F, &d->T, &d->B); }

// Shape of parameter i in lm_collect_params order (model/lm_model.c:21-60,84-98): matrices are 2-D,
// biases and norm weights 1-D.
int param_shape(const Dims& d, int i, uint64_t shape[2]) {
    const int last = 10 * d.L + 1;
    if (i == 0) { shape[0] = d.V; shape[1] = d.D; return 2; }
    if (i == last) { shape[0] = d.D; return 1; }
    switch ((i - 1) % 10) {
        case 0: case 4: case 5: case 9: shape[0] = d.D; return 1;          // attn_norm, bo, ffn_norm, b_down
        case 1: shape[0] = d.D; shape[1] = 3ull * d.D; return 2;            // w_qkv
        case 2: shape[0] = 3ull * d.D; return 1;                            // b_qkv
        case 3: shape[0] = d.D; shape[1] = d.D; return 2;                   // wo
        case 6: shape[0] = d.D; shape[1] = 2ull * d.F; return 2;            // w_gate_up
        case 7: shape[0] = 2ull * d.F; return 1;                            // b_gate_up
        default: shape[0] = d.F; shape[1] = d.D; return 2;                  // w_down
    }
}

struct File {
    FILE* f = nullptr;
    ~File() { if (f) fclose(f); }
};

}  // namespace

extern "C" {

int tb_sample_batch_range(const uint32_t* tokens, uint64_t num_tokens, int T, int first_sequence, int count,
                          uint64_t seed_base, uint32_t* ids_out, uint32_t* targets_out) {
    TB_CHECK(tokens && ids_out && targets_out, "tb_sample_batch: null pointer");
    TB_CHECK(T > 0 && count > 0 && first_sequence >= 0 && num_tokens > (uint64_t)T + 1,
             "tb_sample_batch: %llu tokens cannot hold a window of %d + 1", (unsigned long long)num_tokens, T);
    const int64_t max_start = (int64_t)(num_tokens - (uint64_t)T - 1);
    for (int i = 0; i < count; ++i) {
        const uint64_t w = (uint64_t)first_sequence + (uint64_t)i;
        Pcg32 rng(seed_base * 1000003ull + w, 99ull + w);
        const int64_t start = rng.range(0, max_start);
        std::memcpy(ids_out + (size_t)i * T, tokens + start, (size_t)T * sizeof(uint32_t));
        std::memcpy(targets_out + (size_t)i * T, tokens + start + 1, (size_t)T * sizeof(uint32_t));
    }
    return 0;
}

int tb_sample_batch(const uint32_t* tokens, uint64_t num_tokens, int T, int B, uint64_t seed_base,
                    uint32_t* ids_out, uint32_t* targets_out) {
    return tb_sample_batch_range(tokens, num_tokens, T, 0, B, seed_base, ids_out, targets_out);
}

int tb_pcg_uniform_fill(uint64_t seed, uint64_t seq, uint64_t n, double* out) {
    TB_CHECK(out || n == 0, "tb_pcg_uniform_fill: null pointer");
    Pcg32 rng(seed, seq);
    for (uint64_t i = 0; i < n; ++i) out[i] = rng.uniform();
    return 0;
}

float tb_lr_warmup_cosine(uint64_t step, uint64_t warmup_steps, uint64_t total_steps, float peak_lr, float min_lr) {
    if (warmup_steps > 0 && step < warmup_steps) return peak_lr * (float)(step + 1) / (float)warmup_steps;
    if (total_steps <= warmup_steps) return min_lr;
    double p = (double)(step - warmup_steps) / (double)(total_steps - warmup_steps);
    if (p > 1.0) p = 1.0;
    const double c = 0.5 * (1.0 + std::cos(3.14159265358979323846 * p));
    return (float)((double)min_lr + ((double)peak_lr - (double)min_lr) * c);
}

int tb_checkpoint_save(const char* path, TbTrainer* g, int with_optimizer, uint64_t adam_t) {
    TB_CHECK(path && g, "tb_checkpoint_save: null argument");
    Dims d;
    TB_TRY(get_dims(g, &d));
    const int np = tb_trainer_num_params(g);
    const int64_t total = tb_trainer_total_scalars(g);
    std::vector<int64_t> off(np), num(np);
    TB_TRY(tb_trainer_param_layout(g, off.data(), num.data()));
    std::vector<float> p((size_t)total), m, v;
    TB_TRY(tb_trainer_download(g, 0, p.data()));
    if (with_optimizer) {
        m.resize((size_t)total);
        v.resize((size_t)total);
        TB_TRY(tb_trainer_download(g, 2, m.data()));
        TB_TRY(tb_trainer_download(g, 3, v.data()));
    }
    // written to <path>.tmp and renamed once complete, so that an interrupted save leaves the
    // previous checkpoint intact (training/checkpoint.c:24-74)
    const std::string tmp = std::string(path) + ".tmp";
    bool ok = true;
    {
        File out;
        out.f = fopen(tmp.c_str(), "wb");
        TB_CHECK(out.f, "tb_checkpoint_save: cannot open %s", tmp.c_str());
        auto put = [&](const void* data, size_t bytes) { if (ok && fwrite(data, 1, bytes, out.f) != bytes) ok = false; };
        const uint32_t version = 1, n = (uint32_t)np, has_opt = with_optimizer ? 1u : 0u;
        put("TRLM", 4);
        put(&version, 4);
        put(&n, 4);
        put(&has_opt, 4);
        for (int i = 0; i < np; ++i) {
            uint64_t shape[2];
            const uint32_t ndim = (uint32_t)param_shape(d, i, shape);
            put(&ndim, 4);
            put(shape, 8 * ndim);
            put(p.data() + off[i], (size_t)num[i] * 4);
        }
        if (with_optimizer) {
            for (int i = 0; i < np; ++i) {
                put(m.data() + off[i], (size_t)num[i] * 4);
                put(v.data() + off[i], (size_t)num[i] * 4);
            }
            put(&adam_t, 8);
        }
        if (ok && fflush(out.f) != 0) ok = false;
    }
    if (ok && std::rename(tmp.c_str(), path) != 0) ok = false;
    if (!ok) std::remove(tmp.c_str());
    TB_CHECK(ok, "tb_checkpoint_save: writing %s failed", path);
    return 0;
}

int tb_checkpoint_load(const char* path, TbTrainer* g, int with_optimizer, uint64_t* adam_t_out) {
    TB_CHECK(path && g, "tb_checkpoint_load: null argument");
    Dims d;
    TB_TRY(get_dims(g, &d));
    const int np = tb_trainer_num_params(g);
    const int64_t total = tb_trainer_total_scalars(g);
    std::vector<int64_t> off(np), num(np);
    TB_TRY(tb_trainer_param_layout(g, off.data(), num.data()));
    std::vector<unsigned char> buf;
    {
        File in;
        in.f = fopen(path, "rb");
        TB_CHECK(in.f, "tb_checkpoint_load: cannot open %s", path);
        fseek(in.f, 0, SEEK_END);
        const long size = ftell(in.f);
        fseek(in.f, 0, SEEK_SET);
        TB_CHECK(size >= 16, "tb_checkpoint_load: %s is not a TRLM checkpoint", path);
        buf.resize((size_t)size);
        TB_CHECK(fread(buf.data(), 1, buf.size(), in.f) == buf.size(), "tb_checkpoint_load: short read of %s", path);
    }
    // first pass validates the whole file against the model, the second copies: a rejected file
    // leaves the trainer untouched (training/checkpoint.c:76-135)
    const size_t size = buf.size();
    TB_CHECK(std::memcmp(buf.data(), "TRLM", 4) == 0, "tb_checkpoint_load: %s is not a TRLM checkpoint", path);
    uint32_t version, n, has_opt;
    std::memcpy(&version, buf.data() + 4, 4);
    std::memcpy(&n, buf.data() + 8, 4);
    std::memcpy(&has_opt, buf.data() + 12, 4);
    TB_CHECK(version == 1, "tb_checkpoint_load: version %u, expected 1", version);
    TB_CHECK((int)n == np, "tb_checkpoint_load: %u parameter tensors in the file, the model has %d", n, np);
    TB_CHECK(!with_optimizer || has_opt, "tb_checkpoint_load: %s holds no optimiser state", path);
    size_t pos = 16;
    std::vector<size_t> where(np);
    for (int i = 0; i < np; ++i) {
        uint64_t shape[2];
        const uint32_t ndim = (uint32_t)param_shape(d, i, shape);
        uint32_t file_ndim;
        TB_CHECK(pos + 4 <= size, "tb_checkpoint_load: %s is truncated", path);
        std::memcpy(&file_ndim, buf.data() + pos, 4);
        pos += 4;
        TB_CHECK(file_ndim == ndim, "tb_checkpoint_load: tensor %d has %u dimensions, expected %u", i, file_ndim, ndim);
        for (uint32_t k = 0; k < ndim; ++k) {
            uint64_t dim;
            TB_CHECK(pos + 8 <= size, "tb_checkpoint_load: %s is truncated", path);
            std::memcpy(&dim, buf.data() + pos, 8);
            pos += 8;
            TB_CHECK(dim == shape[k], "tb_checkpoint_load: tensor %d dimension %u is %llu, expected %llu", i, k,
                     (unsigned long long)dim, (unsigned long long)shape[k]);
        }
        const size_t bytes = (size_t)num[i] * 4;
        TB_CHECK(pos + bytes <= size, "tb_checkpoint_load: %s is truncated", path);
        where[i] = pos;
        pos += bytes;
    }
    const size_t opt_pos = pos;
    if (has_opt) pos += 2 * (size_t)total * 4 + 8;
    TB_CHECK(pos == size, "tb_checkpoint_load: %s has %zu bytes, the model needs %zu", path, size, pos);

    std::vector<float> flat((size_t)total);
    for (int i = 0; i < np; ++i) std::memcpy(flat.data() + off[i], buf.data() + where[i], (size_t)num[i] * 4);
    TB_TRY(tb_trainer_upload(g, 0, flat.data()));
    if (with_optimizer) {
        std::vector<float> v((size_t)total);
        pos = opt_pos;
        for (int i = 0; i < np; ++i) {
            const size_t bytes = (size_t)num[i] * 4;
            std::memcpy(flat.data() + off[i], buf.data() + pos, bytes);
            pos += bytes;
            std::memcpy(v.data() + off[i], buf.data() + pos, bytes);
            pos += bytes;
        }
        TB_TRY(tb_trainer_upload(g, 2, flat.data()));
        TB_TRY(tb_trainer_upload(g, 3, v.data()));
        if (adam_t_out) std::memcpy(adam_t_out, buf.data() + pos, 8);
    }
    return 0;
}

int tb_trainer_run(TbTrainer* g, const uint32_t* tokens, uint64_t num_tokens, uint32_t start_step, uint32_t num_steps,
                   uint32_t warmup_steps, uint32_t total_steps, float peak_lr, float min_lr, float max_norm,
                   float beta1, float beta2, float eps, uint64_t* adam_t, float* losses_out, double* norms_out) {
    TB_CHECK(g && tokens && adam_t, "tb_trainer_run: null argument");
    Dims d;
    TB_TRY(get_dims(g, &d));
    const size_t n = (size_t)d.B * d.T;
    std::vector<uint32_t> ids[2], tgt[2];
    for (int i = 0; i < 2; ++i) { ids[i].resize(n); tgt[i].resize(n); }
    if (num_steps == 0) return 0;
    TB_TRY(tb_sample_batch(tokens, num_tokens, d.T, d.B, 2026ull + start_step, ids[0].data(), tgt[0].data()));
    for (uint32_t s = 0; s < num_steps; ++s) {
        const uint32_t step = start_step + s;
        const int cur = s & 1;
        const float lr = tb_lr_warmup_cosine(step, warmup_steps, total_steps, peak_lr, min_lr);
        *adam_t += 1;
        TB_TRY(tb_trainer_zero_grads(g));
        TB_TRY(tb_trainer_forward(g, ids[cur].data(), tgt[cur].data(), 1));
        TB_TRY(tb_trainer_backward_head(g));
        for (int l = d.L - 1; l >= 0; --l) TB_TRY(tb_trainer_backward_layer(g, l));
        TB_TRY(tb_trainer_backward_embed(g));
        TB_TRY(tb_trainer_clip_adam_async(g, *adam_t, lr, beta1, beta2, eps, max_norm, 1.0f));
        // the device is busy with this step: draw the next step's windows now
        if (s + 1 < num_steps)
            TB_TRY(tb_sample_batch(tokens, num_tokens, d.T, d.B, 2026ull + step + 1, ids[cur ^ 1].data(),
                                   tgt[cur ^ 1].data()));
        float loss = 0.f;
        TB_TRY(tb_trainer_read_loss(g, &loss));         // the step's only host synchronisation
        if (losses_out) losses_out[s] = loss;
        if (norms_out) TB_TRY(tb_trainer_last_norm(g, &norms_out[s]));
    }
    return 0;
}

}  // extern "C"
