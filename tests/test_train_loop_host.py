"""Host code of the training loop against the reference: window sampling (model/gpu_train.c:296-307,
training/data_parallel.c:73-77) and the learning-rate schedule (training/lr_schedule.c:6-15).  No GPU."""
import json

import numpy as np
import pytest

from conftest import golden_path


@pytest.fixture(scope="module")
def golden():
    return json.load(open(golden_path("train_loop.json")))


def test_sample_batch_golden_windows(golden):
    from turkce_llm_b200.gpu_train import sample_batch
    for c in golden["windows"]:
        tokens = np.arange(c["num_tokens"], dtype=np.uint32)
        ids, tgt = sample_batch(tokens, c["T"], c["B"], c["seed_base"])
        assert [int(x) for x in ids[::c["T"]]] == c["starts"], c
        assert np.array_equal(tgt, ids + 1)
        assert np.array_equal(ids.reshape(c["B"], c["T"]), np.asarray(c["starts"])[:, None] + np.arange(c["T"])[None])


def test_sample_batch_matches_reference_live(ref):
    from turkce_llm_b200.gpu_train import sample_batch
    rng = np.random.default_rng(5)
    for num_tokens, T, B in [(67, 64, 2), (1000, 7, 64), (50000, 128, 28), (3_000_000, 1024, 16)]:
        tokens = rng.integers(0, 31769, num_tokens).astype(np.uint32)
        for seed_base in (0, 1, 2026, 2026 + 69999, 2**40 + 3):
            got = sample_batch(tokens, T, B, seed_base)
            want = ref.sample_batch(tokens, T, B, seed_base)
            assert np.array_equal(got[0], want[0]) and np.array_equal(got[1], want[1])


def test_sample_batch_rejects_short_corpus():
    from turkce_llm_b200 import lib
    from turkce_llm_b200.gpu_train import sample_batch
    with pytest.raises(lib.TbError):
        sample_batch(np.zeros(65, dtype=np.uint32), 64, 2, 1)


def test_lr_schedule_golden(golden):
    from turkce_llm_b200.gpu_train import lr_warmup_cosine
    for c in golden["schedule"]:
        if "warmup" in c:
            got = lr_warmup_cosine(c["step"], c["warmup"], c["total"], 1e-3, 1e-4)
        else:
            got = lr_warmup_cosine(c["step"], 1000, 70000, 6e-4, 6e-5)
        # cos comes from libm here and from the reference's own series there: allow one float32 ulp
        assert abs(int(np.float32(got).view(np.uint32)) - c["lr_bits"]) <= 1, c


def test_lr_schedule_matches_reference_live(ref):
    from turkce_llm_b200.gpu_train import lr_warmup_cosine
    exact = 0
    steps = list(range(0, 1200)) + list(range(1200, 72000, 97))
    for step in steps:
        got = np.float32(lr_warmup_cosine(step, 1000, 70000, 6e-4, 6e-5))
        want = np.float32(ref.lr_warmup_cosine(step, 1000, 70000, 6e-4, 6e-5))
        assert abs(int(got.view(np.uint32)) - int(want.view(np.uint32))) <= 1, step
        exact += int(got == want)
    assert exact >= 0.99 * len(steps)


def test_pcg_uniform_matches_reference(ref):
    from turkce_llm_b200.decode import pcg_uniform
    for seed, seq in ((4242, 7), (0, 0), (2**63 + 5, 2**40)):
        assert np.array_equal(pcg_uniform(seed, seq, 1000), ref.uniform(1000, seed, seq))


def test_pcg_uniform_known_values():
    """The first draws of the reference generator's stream pcg_seed(4242, 7) (training/generate.c:181)."""
    from turkce_llm_b200.decode import pcg_uniform
    got = pcg_uniform(4242, 7, 4)
    assert [int(x * 2**32) for x in got] == [1341512397, 1709436583, 702394695, 2554193518]
