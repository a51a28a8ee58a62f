"""The library's data-parallel step (tb_dp_step) on one GPU, through the C ABI: with one rank it must equal
the single-GPU training step bit for bit, and micro-batch accumulation must give the mean gradient and the
mean loss of the micro-batches (the reference's data_parallel_step averages its workers' gradients and
losses the same way: training/data_parallel.c:102-117,150-162).  More than one rank needs more than one
GPU: the benchmark's `repro` record covers that; the sharding arithmetic is covered on CPU."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

CFG = (211, 64, 2, 2, 128, 96, 3)       # V, D, H, L, F, T, B


def start(g, seed):
    rng = np.random.default_rng(seed)
    p = (rng.standard_normal(g.total) * 0.05).astype(np.float32)
    off, num = g.param_layout()
    for i, (o, n) in enumerate(zip(off, num)):
        k = (i - 1) % 10 if 0 < i < len(off) - 1 else -1
        if i == len(off) - 1 or k in (0, 5):
            p[o:o + n] = 1.0
    return p


def batch(rng, V, n):
    s = rng.integers(0, V, n + 1).astype(np.uint32)
    return s[:-1].copy(), s[1:].copy()


@pytest.mark.parametrize("mode", [0, 1], ids=["allreduce", "sharded"])
def test_one_rank_equals_the_single_gpu_step_bit_for_bit(tb, mode):
    from turkce_llm_b200.data_parallel import DataParallel
    from turkce_llm_b200.gpu_train import ADAM_M, ADAM_V, PARAMS, AdamState, GpuTrainer
    V, D, H, L, F, T, B = CFG
    rng = np.random.default_rng(1)
    batches = [batch(rng, V, B * T) for _ in range(3)]
    results = []
    for use_dp in (False, True):
        g = GpuTrainer(V, D, H, L, F, T, B, 1e-5)
        g.upload(start(g, 2))
        opt = AdamState(lr=1e-3)
        dp = DataParallel(g, 0, 1, None, mode=mode) if use_dp else None
        out = []
        for ids, tgt in batches:
            out.append(dp.step_host(ids, tgt, opt, 1.0) if use_dp else g.train_step(ids, tgt, opt, 1.0))
        state = [g.download(w) for w in (PARAMS, ADAM_M, ADAM_V)]
        if dp:
            assert dp.describe()["combine"].startswith("one rank")
            dp.destroy()
        g.destroy()
        results.append((out, state))
    (out_a, st_a), (out_b, st_b) = results
    for (la, na), (lb, nb) in zip(out_a, out_b):
        assert np.float32(la).tobytes() == np.float32(lb).tobytes()
        assert np.float64(na).tobytes() == np.float64(nb).tobytes()
    for a, b in zip(st_a, st_b):
        assert np.array_equal(a, b)


def test_micro_batches_accumulate_to_the_mean(tb):
    from turkce_llm_b200.data_parallel import DataParallel
    from turkce_llm_b200.gpu_train import GRADS, AdamState, GpuTrainer
    V, D, H, L, F, T, B = CFG
    rng = np.random.default_rng(3)
    micro = [batch(rng, V, B * T) for _ in range(3)]
    g = GpuTrainer(V, D, H, L, F, T, B, 1e-5)
    p = start(g, 4)
    g.upload(p)
    losses, grads = [], []
    for ids, tgt in micro:
        losses.append(g.forward_backward(ids, tgt))
        grads.append(g.download(GRADS).astype(np.float64))
    want_sum = sum(grads)
    want_norm = float(np.sqrt(((want_sum / 3) ** 2).sum()))
    dp = DataParallel(g, 0, 1, None)
    opt = AdamState(lr=0.0)                       # lr 0: the weights stay, so the gradient buffer can be compared
    loss, norm = dp.step_host_accumulate(micro, opt, 0.0)
    got = g.download(GRADS).astype(np.float64)
    assert np.array_equal(g.download(0), p)
    assert abs(loss - np.mean(losses)) <= 1e-6 * abs(np.mean(losses))
    assert np.abs(got - want_sum).max() <= 1e-5 * np.abs(want_sum).max()
    assert abs(norm - want_norm) <= 1e-5 * want_norm
    # the resident form of the step: same inputs, same result as the host form, and asynchronous until asked
    g.set_inputs(*micro[0])
    dp.step_resident(opt, 0.0)
    loss_r, norm_r = dp.last_result()
    loss_h, norm_h = dp.step_host(micro[0][0], micro[0][1], opt, 0.0)
    assert np.float32(loss_r).tobytes() == np.float32(loss_h).tobytes() and norm_r == norm_h
    dp.destroy()
    g.destroy()
