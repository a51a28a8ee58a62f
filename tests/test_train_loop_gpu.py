"""The training loop around the trainer on the GPU: checkpoints in the reference's TRLM format
(training/checkpoint.c), the loop of training/train_lm_gpu.c:212-223, and bit-identical resume
(the property tests/test_resume.c:114-120 checks on the reference)."""
import hashlib
import json

import numpy as np
import pytest

from conftest import golden_path

pytestmark = pytest.mark.gpu

SCHED = dict(warmup_steps=4, total_steps=40, peak_lr=1e-3, min_lr=1e-4)


def small_trainer():
    from turkce_llm_b200.gpu_train import GpuTrainer
    g = np.load(golden_path("model_step_small.npz"))
    V, D, H, L, F, T, B = [int(x) for x in g["dims"]]
    return GpuTrainer(V, D, H, L, F, T, B, 1e-5), g, (V, D, H, L, F, T, B)


def test_checkpoint_file_is_the_references_byte_for_byte(tb, tmp_path):
    """State of the reference's small end-to-end model after one Adam step: the file written here has the
    SHA-256 of the file the reference's checkpoint_save wrote from the same state."""
    from turkce_llm_b200.gpu_train import ADAM_M, ADAM_V, PARAMS, AdamState
    want = json.load(open(golden_path("train_loop.json")))["checkpoint_of_model_step_small"]
    t, g, _ = small_trainer()
    t.upload(g["params1"], PARAMS); t.upload(g["adam_m"], ADAM_M); t.upload(g["adam_v"], ADAM_V)
    opt = AdamState(); opt.t = 1
    for with_opt in (0, 1):
        path = tmp_path / ("c%d.bin" % with_opt)
        t.save_checkpoint(path, opt if with_opt else None)
        data = open(path, "rb").read()
        assert len(data) == want["with_opt_%d" % with_opt]["bytes"]
        assert hashlib.sha256(data).hexdigest() == want["with_opt_%d" % with_opt]["sha256"]
        assert not (tmp_path / ("c%d.bin.tmp" % with_opt)).exists()
    t.destroy()


def test_checkpoint_crosses_to_the_reference_and_back(tb, ref, tmp_path):
    from oracle import pyoracle
    from turkce_llm_b200.gpu_train import ADAM_M, ADAM_V, PARAMS, AdamState
    t, g, (V, D, H, L, F, T, B) = small_trainer()
    rng = np.random.default_rng(3)
    p, m, v = [rng.standard_normal(t.total).astype(np.float32) for _ in range(3)]
    t.upload(p, PARAMS); t.upload(m, ADAM_M); t.upload(np.abs(v), ADAM_V)
    opt = AdamState(); opt.t = 77
    t.save_checkpoint(tmp_path / "ours.bin", opt)
    lm = pyoracle.RefLM(ref, V, D, H, L, F, 1e-5, 1, 1)
    assert lm.checkpoint_load(tmp_path / "ours.bin", True)
    assert np.array_equal(lm.get(0), p) and np.array_equal(lm.get(2), m) and np.array_equal(lm.get(3), np.abs(v))
    assert lm.adam_t() == 77
    # the other way: the reference writes, the trainer loads
    lm.set(0, p[::-1].copy()); lm.set_adam_t(123)
    assert lm.checkpoint_save(tmp_path / "theirs.bin", True)
    opt2 = AdamState()
    t.load_checkpoint(tmp_path / "theirs.bin", opt2)
    assert opt2.t == 123
    assert np.array_equal(t.download(PARAMS), p[::-1]) and np.array_equal(t.download(ADAM_M), m)
    # parameters only, from a file that has optimiser state, is allowed; the reverse is not
    t.load_checkpoint(tmp_path / "ours.bin", None)
    assert np.array_equal(t.download(PARAMS), p)
    assert lm.checkpoint_save(tmp_path / "noopt.bin", False)
    with pytest.raises(tb.TbError):
        t.load_checkpoint(tmp_path / "noopt.bin", AdamState())
    lm.close()
    t.destroy()


def test_checkpoint_load_rejects_bad_files_and_leaves_the_trainer_untouched(tb, tmp_path):
    from turkce_llm_b200.gpu_train import PARAMS, AdamState, GpuTrainer
    t, g, (V, D, H, L, F, T, B) = small_trainer()
    t.upload(g["params0"], PARAMS)
    opt = AdamState(); opt.t = 5
    t.save_checkpoint(tmp_path / "good.bin", opt)
    data = open(tmp_path / "good.bin", "rb").read()
    t.upload(g["params1"], PARAMS)
    bad = {
        "truncated": data[:-9],
        "trailing": data + b"\0",
        "magic": b"TRLX" + data[4:],
        "version": data[:4] + (2).to_bytes(4, "little") + data[8:],
        "count": data[:8] + (7).to_bytes(4, "little") + data[12:],
        "shape": data[:20] + (V + 1).to_bytes(8, "little") + data[28:],
        "empty": b"",
    }
    for name, blob in bad.items():
        open(tmp_path / (name + ".bin"), "wb").write(blob)
        with pytest.raises(tb.TbError):
            t.load_checkpoint(tmp_path / (name + ".bin"), AdamState())
        assert np.array_equal(t.download(PARAMS), g["params1"]), name
    with pytest.raises(tb.TbError):
        t.load_checkpoint(tmp_path / "does_not_exist.bin", None)
    other = GpuTrainer(V, D, H, L + 1, F, T, B, 1e-5)        # another architecture
    with pytest.raises(tb.TbError):
        other.load_checkpoint(tmp_path / "good.bin", None)
    other.destroy()
    t.destroy()


def test_run_equals_the_loop_written_out(tb):
    """tb_trainer_run against the same loop made of sample_batch + lr_warmup_cosine + train_step: bitwise."""
    from turkce_llm_b200.gpu_train import PARAMS, AdamState, lr_warmup_cosine, sample_batch
    a, g, (V, D, H, L, F, T, B) = small_trainer()
    b, _, _ = small_trainer()
    tokens = (np.random.default_rng(9).zipf(1.1, 5000) % V).astype(np.uint32)
    a.upload(g["params0"]); b.upload(g["params0"])
    oa, ob = AdamState(), AdamState()
    losses, norms = a.run(tokens, 0, 12, oa, max_norm=1.0, **SCHED)
    for step in range(12):
        ob.lr = lr_warmup_cosine(step, SCHED["warmup_steps"], SCHED["total_steps"], SCHED["peak_lr"], SCHED["min_lr"])
        ids, tgt = sample_batch(tokens, T, B, 2026 + step)
        loss, norm = b.train_step(ids, tgt, ob, max_norm=1.0)
        assert loss == losses[step] and norm == norms[step], step
    assert oa.t == ob.t == 12
    assert np.array_equal(a.download(PARAMS).view(np.uint32), b.download(PARAMS).view(np.uint32))
    assert losses[-1] < losses[0]
    a.destroy(); b.destroy()


def test_resume_from_checkpoint_is_bit_identical(tb, tmp_path):
    from turkce_llm_b200.gpu_train import ADAM_M, ADAM_V, PARAMS, AdamState
    a, g, (V, D, H, L, F, T, B) = small_trainer()
    tokens = (np.random.default_rng(10).zipf(1.1, 5000) % V).astype(np.uint32)
    a.upload(g["params0"])
    oa = AdamState()
    straight, _ = a.run(tokens, 0, 10, oa, max_norm=1.0, **SCHED)
    want = [a.download(w) for w in (PARAMS, ADAM_M, ADAM_V)]
    a.destroy()

    b, _, _ = small_trainer()
    b.upload(g["params0"])
    ob = AdamState()
    first, _ = b.run(tokens, 0, 6, ob, max_norm=1.0, **SCHED)
    b.save_checkpoint(tmp_path / "mid.bin", ob)
    b.destroy()
    c, _, _ = small_trainer()
    oc = AdamState()
    c.load_checkpoint(tmp_path / "mid.bin", oc)
    assert oc.t == 6
    rest, _ = c.run(tokens, 6, 4, oc, max_norm=1.0, **SCHED)
    assert np.array_equal(np.concatenate([first, rest]).view(np.uint32), straight.view(np.uint32))
    for w, x in zip((PARAMS, ADAM_M, ADAM_V), want):
        assert np.array_equal(c.download(w).view(np.uint32), x.view(np.uint32))
    c.destroy()


def test_micro_batch_accumulation_equals_one_large_batch(tb):
    """Two micro-batches of 4 sequences accumulated into one optimiser step against one batch of 8 sequences
    (the fixed-global-batch mode of the data-parallel step): same mean loss and mean gradients up to the
    summation order; a second run is bit-identical."""
    from conftest import rel_to_maxabs
    from turkce_llm_b200.data_parallel import DataParallelStep, layer_buckets, micro_batches, shard_sequences
    from turkce_llm_b200.gpu_train import GRADS, PARAMS, AdamState, GpuTrainer, sample_batch
    V, D, H, L, F, T = 500, 64, 2, 2, 128, 64
    tokens = (np.random.default_rng(4).zipf(1.1, 20000) % V).astype(np.uint32)
    big = GpuTrainer(V, D, H, L, F, T, 8, 1e-5)
    p = (np.random.default_rng(5).standard_normal(big.total) * 0.05).astype(np.float32)
    big.upload(p)
    ids, tgt = sample_batch(tokens, T, 8, 2026)
    loss_big = big.forward_backward(ids, tgt)
    norm_big = big.grad_norm()
    g_big = big.download(GRADS)
    big.destroy()

    results = []
    for _ in range(2):
        small = GpuTrainer(V, D, H, L, F, T, 4, 1e-5)
        small.upload(p)
        step = DataParallelStep(small, None, layer_buckets(*small.param_layout()), 1, None)
        batches = [sample_batch(tokens, T, c, 2026, first_sequence=f)
                   for f, c in micro_batches(*shard_sequences(8, 1, 0), 4)]
        assert np.array_equal(np.concatenate([b[0] for b in batches]), ids)
        opt = AdamState(lr=1e-3)
        loss, norm = step.host_accumulate(batches, opt, max_norm=0.0)
        results.append((loss, norm, small.download(GRADS), small.download(PARAMS)))
        small.destroy()
    loss, norm, g_sum, _ = results[0]
    assert abs(loss - loss_big) <= 1e-5 * abs(loss_big)
    assert rel_to_maxabs(g_sum * np.float32(0.5), g_big) <= 2e-3
    assert abs(norm - np.sqrt(np.sum((g_sum.astype(np.float64) * 0.5) ** 2))) <= 1e-4 * norm
    assert abs(norm - norm_big) <= 2e-3 * norm_big          # the clipped norm is that of the MEAN gradients
    assert results[1][0] == loss and results[1][1] == norm
    assert np.array_equal(results[0][3].view(np.uint32), results[1][3].view(np.uint32))
