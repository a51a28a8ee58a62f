"""Greedy decoding with a KV cache against the CPU oracle's full-recompute forward: the reference
generates by running its whole forward on the growing window and reading the last logits row
(training/generate.c:186-212); the cached path must give the same logits at every step."""
import numpy as np
import pytest

from conftest import rel_to_maxabs

pytestmark = pytest.mark.gpu


def make_params(oracle, cfg, seed):
    V, D, H, L, F, T, B, eps = cfg
    total = oracle.model_total_scalars(cfg)
    rng = np.random.default_rng(seed)
    p = (rng.standard_normal(total) * 0.05).astype(np.float32)
    # layout: embedding, per layer 10 tensors, final norm
    sizes = [V * D]
    for _ in range(L):
        sizes += [D, D * 3 * D, 3 * D, D * D, D, D, D * 2 * F, 2 * F, F * D, D]
    sizes.append(D)
    off = 0
    for i, n in enumerate(sizes):
        k = (i - 1) % 10 if 0 < i < len(sizes) - 1 else -1
        if i == len(sizes) - 1 or k in (0, 5):
            p[off:off + n] = 1.0 + 0.05 * rng.standard_normal(n)
        off += n
    return p


@pytest.mark.parametrize("dims", [(97, 32, 2, 2, 48, 3, 5, 6), (300, 64, 2, 2, 128, 4, 140, 20)])
def test_cached_decode_matches_full_recompute(tb, oracle, dims):
    from turkce_llm_b200.decode import Decoder
    V, D, H, L, F, S, prompt_len, n_new = dims
    cap = prompt_len + n_new + 2
    p = make_params(oracle, (V, D, H, L, F, 1, 1, 1e-5), 5)
    dec = Decoder(V, D, H, L, F, S, cap)
    dec.upload(p)
    rng = np.random.default_rng(6)
    prompts = rng.integers(0, V, (S, prompt_len)).astype(np.uint32)
    dec.prefill(prompts)
    window = prompts.copy()
    worst = 0.0
    for step in range(n_new):
        if step > 0:
            dec.generate(1)
        got_logits = dec.logits()
        got_tok = dec.tokens(step + 1)[:, step]
        T = window.shape[1]
        _, _, logits = oracle.model_forward_backward((V, D, H, L, F, T, S, 1e-5), p, window.reshape(-1),
                                                     np.zeros(S * T, np.uint32), want_grads=False, want_logits=True)
        want = logits.reshape(S, T, V)[:, -1, :]
        worst = max(worst, rel_to_maxabs(got_logits, want))
        assert rel_to_maxabs(got_logits, want) <= 2e-2, step          # the BF16-mode bound
        # the chosen token is the argmax of the engine's own logits, and equals the oracle's choice
        # wherever the oracle's top-2 margin is larger than the bf16 noise
        assert np.array_equal(got_tok, got_logits.argmax(1))
        srt = np.sort(want, axis=1)
        clear = (srt[:, -1] - srt[:, -2]) > 4e-2 * np.abs(want).max()
        assert np.array_equal(got_tok[clear], want.argmax(1)[clear])
        window = np.concatenate([window, got_tok[:, None].astype(np.uint32)], axis=1)
    dec.destroy()


def test_generate_in_one_call_equals_stepwise(tb, oracle):
    """n graph-replayed steps in one call give the tokens of n single-step calls, bit for bit."""
    from turkce_llm_b200.decode import Decoder
    V, D, H, L, F, S, prompt_len, n_new = 211, 64, 2, 3, 128, 8, 33, 24
    p = make_params(oracle, (V, D, H, L, F, 1, 1, 1e-5), 9)
    prompts = np.random.default_rng(10).integers(0, V, (S, prompt_len)).astype(np.uint32)
    outs = []
    for chunk in (1, n_new - 1):
        dec = Decoder(V, D, H, L, F, S, prompt_len + n_new + 1)
        dec.upload(p)
        dec.prefill(prompts)
        done = 1
        while done < n_new:
            k = min(chunk, n_new - done)
            dec.generate(k)
            done += k
        outs.append(dec.tokens(n_new))
        dec.destroy()
    assert np.array_equal(outs[0], outs[1])


@pytest.mark.parametrize("shape", [(64, 31769, 384), (5, 300, 64), (64, 1000, 128), (17, 40000, 384), (64, 2049, 1024)])
def test_fused_lmhead_argmax_matches_oracle(tb, oracle, shape):
    """tb_lmhead_argmax_bf16 against the oracle's BF16-mode product (operands rounded to bf16, float32
    accumulation): the optional logits within the BF16 bound, the token equal to the argmax of those
    logits, and equal to the oracle's choice wherever its top-2 margin is clear of the rounding noise."""
    import torch
    from turkce_llm_b200 import lib
    S, V, K = shape
    rng = np.random.default_rng(11)
    X = rng.standard_normal((S, K)).astype(np.float32)
    E = (rng.standard_normal((V, K)) * 0.05).astype(np.float32)
    from oracle import pyoracle
    want = oracle.gemm(0, 1, X, E, S, V, K, mode=pyoracle.BF16).reshape(S, V)      # X . E^T, operands rounded to bf16
    x16 = torch.from_numpy(X).cuda().to(torch.bfloat16)
    e16 = torch.from_numpy(E).cuda().to(torch.bfloat16)
    tok = torch.full((S,), -1, device="cuda", dtype=torch.int32)
    ld = V + 3
    logits = torch.zeros(S, ld, device="cuda")
    lib.lmhead_argmax_bf16(x16, e16, tok, logits, ld)
    tok2 = torch.full((S,), -1, device="cuda", dtype=torch.int32)
    lib.lmhead_argmax_bf16(x16, e16, tok2)                 # the product path: no logits written
    lib.sync_check()
    got = logits[:, :V].cpu().numpy()
    assert np.all(logits[:, V:].cpu().numpy() == 0.0)       # nothing written past column V
    assert rel_to_maxabs(got, want) <= 2e-2
    t = tok.cpu().numpy()
    assert np.array_equal(t, tok2.cpu().numpy())
    assert np.array_equal(t, got.argmax(1))                 # lowest index on ties, like numpy
    srt = np.sort(want, axis=1)
    clear = (srt[:, -1] - srt[:, -2]) > 4e-2 * np.abs(want).max()
    assert clear.sum() > 0
    assert np.array_equal(t[clear], want.argmax(1)[clear])
