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


@pytest.mark.parametrize("dims", [(97, 32, 2, 2, 48, 3, 5, 6), (300, 64, 2, 2, 128, 4, 140, 20),
                                  (300, 128, 2, 2, 256, 5, 20, 12), (500, 256, 4, 3, 1024, 64, 9, 5)])
def test_cached_decode_matches_full_recompute(tb, oracle, dims):
    """(The last two shapes are also those the optional decode-step linear kernel supports, see
    test_lean_decode_step_matches_general_step.)"""
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


def test_full_size_cached_decode_matches_full_recompute(tb, oracle):
    """The decode configuration of the benchmark at full size: the 33,490,176-parameter decoder (12 layers,
    d_model 384, 6 heads, d_ff 1024, 31,769 tokens), 64 sequences with 128-token Zipf(1.1) prompts, 128 greedy
    tokens, cache length up to 256.  The logits each token was chosen from are compared with the oracle's
    full-recompute forward over the window (training/generate.c:186-212) after the prefill and at decode steps
    1, 64 and 127, on eight of the 64 sequences (sequences are independent; the oracle's forward over all 64
    windows would hold 2 GB of logits)."""
    import os
    from turkce_llm_b200.decode import Decoder
    V, D, H, L, F, S, prompt_len, n_new = 31769, 384, 6, 12, 1024, 64, 128, 128
    oracle.set_threads(min(os.cpu_count() or 8, 64))
    rng = np.random.default_rng(3)
    p = make_params(oracle, (V, D, H, L, F, 1, 1, 1e-5), 3)
    w = 1.0 / np.arange(1, V + 1, dtype=np.float64) ** 1.1
    cdf = np.cumsum(w / w.sum())
    prompts = np.minimum(np.searchsorted(cdf, rng.random((S, prompt_len))), V - 1).astype(np.uint32)
    dec = Decoder(V, D, H, L, F, S, prompt_len + n_new + 1)
    dec.upload(p)
    dec.prefill(prompts)
    rows = [0, 9, 18, 27, 36, 45, 54, 63]
    checks = {}
    for step in (0, 1, 64, n_new - 1):
        have = 1 if not checks else max(checks) + 1
        if step + 1 > have:
            dec.generate(step + 1 - have)
        checks[step] = (dec.logits()[rows], dec.tokens(step + 1))
    all_tokens = dec.tokens(n_new)
    assert all_tokens.max() < V
    dec.destroy()
    for step, (got_logits, toks) in checks.items():
        assert np.array_equal(toks, all_tokens[:, :step + 1])          # earlier tokens do not change later
        window = np.concatenate([prompts[rows], toks[rows][:, :step]], axis=1)
        T = window.shape[1]
        assert T == prompt_len + step
        _, _, logits = oracle.model_forward_backward((V, D, H, L, F, T, len(rows), 1e-5), p, window.reshape(-1),
                                                     np.zeros(len(rows) * T, np.uint32), want_grads=False,
                                                     want_logits=True)
        want = logits.reshape(len(rows), T, V)[:, -1, :]
        assert rel_to_maxabs(got_logits, want) <= 2e-2, step           # the BF16-mode bound
        got_tok = toks[rows][:, step]
        assert np.array_equal(got_tok, got_logits.argmax(1))
        srt = np.sort(want, axis=1)
        clear = (srt[:, -1] - srt[:, -2]) > 4e-2 * np.abs(want).max()
        assert np.array_equal(got_tok[clear], want.argmax(1)[clear])


def test_greedy_choice_stays_in_vocabulary_for_nan_and_inf_rows(tb):
    """A row of logits that is all NaN or all -inf (diverged weights) must still give a token inside [0, V):
    the token is fed back into the embedding lookup.  Both greedy paths: the fused LM head (NaN hidden states
    make every product NaN) and the decoder's general path."""
    import torch
    from turkce_llm_b200 import lib
    from turkce_llm_b200.decode import Decoder
    S, V, K = 8, 3000, 128
    x = torch.randn(S, K, device="cuda")
    x[1] = float("nan")
    x[3] = float("-inf")              # products of mixed sign: -inf and +inf sum to NaN
    x[5] = 0.0
    e16 = (torch.randn(V, K, device="cuda") * 0.05).to(torch.bfloat16)
    tok = torch.full((S,), -1, device="cuda", dtype=torch.int32)
    lib.lmhead_argmax_bf16(x.to(torch.bfloat16), e16, tok)
    lib.sync_check()
    t = tok.cpu().numpy()
    assert ((t >= 0) & (t < V)).all(), t
    assert t[5] == 0                   # all-equal row: lowest index
    # a decoder whose weights are NaN: every step's token must stay a valid row of the embedding table
    # (d_model 32 is below the fused head's smallest K, so this decoder takes the general argmax kernel)
    V, D, H, L, F, S = 211, 32, 2, 2, 128, 4
    dec = Decoder(V, D, H, L, F, S, 16)
    p = np.full(dec.total, np.nan, np.float32)
    dec.upload(p)
    dec.prefill(np.zeros((S, 4), np.uint32))
    dec.generate(6)
    toks = dec.tokens(7)
    assert toks.max() < V
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


def sample_next(logits, temperature, u):
    """sample_next of the reference's generator (training/generate.c:57-73), restated: float32 exponentials of
    (z - max) / temperature, float64 running sum in ascending token order, first index whose sum reaches u * total."""
    z = logits.astype(np.float32)
    e = np.exp((z - z.max()) / np.float32(temperature)).astype(np.float32)
    c = np.cumsum(e.astype(np.float64))
    j = int(np.searchsorted(c, u * c[-1], side="left"))
    return min(j, z.size - 1), c


@pytest.mark.parametrize("dims", [(97, 32, 2, 2, 48, 3, 5, 12), (31769, 64, 2, 1, 128, 4, 6, 10)])
def test_temperature_sampling_follows_the_references_sampler(tb, oracle, dims):
    """Every sampled token is the reference sampler's choice on the engine's own logits with the reference's
    uniform draws (PCG32 stream (4242, 7 + s)); the logits themselves still match the oracle's full recompute."""
    from turkce_llm_b200.decode import Decoder, pcg_uniform
    V, D, H, L, F, S, prompt_len, n_new = dims
    cap = prompt_len + n_new + 2
    p = make_params(oracle, (V, D, H, L, F, 1, 1, 1e-5), 7)
    dec = Decoder(V, D, H, L, F, S, cap)
    dec.upload(p)
    temperature = 0.85                                       # training/generate.c:52
    dec.set_sampling(temperature, 4242, 7)
    prompts = np.random.default_rng(8).integers(0, V, (S, prompt_len)).astype(np.uint32)
    dec.prefill(prompts)
    u = np.stack([pcg_uniform(4242, 7 + s, cap) for s in range(S)])
    window = prompts.copy()
    distinct = set()
    for step in range(n_new):
        if step > 0:
            dec.generate(1)
        logits = dec.logits()
        tok = dec.tokens(step + 1)[:, step]
        for s in range(S):
            want, c = sample_next(logits[s], temperature, u[s, step])
            if tok[s] != want:
                # only a draw that lands within rounding of a boundary of the running sum may differ, by one
                r = u[s, step] * c[-1]
                assert abs(int(tok[s]) - want) == 1 and abs(c[min(tok[s], want)] - r) <= 1e-6 * c[-1], (step, s)
            distinct.add(int(tok[s]))
        if step == 0 and V < 1000:
            T = window.shape[1]
            _, _, full = oracle.model_forward_backward((V, D, H, L, F, T, S, 1e-5), p, window.reshape(-1),
                                                       np.zeros(S * T, np.uint32), want_grads=False, want_logits=True)
            assert rel_to_maxabs(logits, full.reshape(S, T, V)[:, -1, :]) <= 2e-2
        window = np.concatenate([window, tok[:, None].astype(np.uint32)], axis=1)
    assert len(distinct) > S                                  # it sampled, it did not collapse to one token
    dec.destroy()


def test_sampling_limits_and_reproducibility(tb, oracle):
    """A vanishing temperature gives the greedy tokens; the same seed gives the same tokens, another seed does
    not; switching back to temperature 0 restores the greedy engine."""
    from turkce_llm_b200.decode import Decoder
    V, D, H, L, F, S, prompt_len, n_new = 300, 64, 2, 2, 128, 4, 9, 16
    p = make_params(oracle, (V, D, H, L, F, 1, 1, 1e-5), 9)
    prompts = np.random.default_rng(10).integers(0, V, (S, prompt_len)).astype(np.uint32)
    dec = Decoder(V, D, H, L, F, S, prompt_len + n_new + 2)
    dec.upload(p)

    def run(temperature, seed):
        dec.set_sampling(temperature, seed, 7)
        dec.prefill(prompts)
        dec.generate(n_new - 1)
        return dec.tokens(n_new)

    greedy = run(0.0, 1)
    assert np.array_equal(run(1e-4, 1), greedy)
    a, b, c = run(0.85, 4242), run(0.85, 4242), run(0.85, 4243)
    assert np.array_equal(a, b) and not np.array_equal(a, c) and not np.array_equal(a, greedy)
    assert np.array_equal(run(0.0, 1), greedy)
    dec.destroy()


@pytest.mark.parametrize("mode", ["norm_qkv", "out_residual", "norm_swiglu", "down_residual"])
def test_decode_linear_entry_matches_oracle(tb, oracle, mode):
    """tb_decode_linear -- the decode step's own linear kernel with the RMSNorm, the SwiGLU and the residual add fused
    (model/model_ops.c's rmsnorm, model/feedforward.c:9-14, model/transformer_block.c:7-15) -- against the oracle's
    separate steps on bf16-rounded operands, at the layer shapes of the 33.49M model and a ragged sequence count."""
    import torch
    from oracle.pyoracle import BF16
    rng = np.random.default_rng(21)
    D, F = 384, 1024
    for S in (64, 37):
        if mode == "norm_qkv":
            K, N = D, 3 * D
        elif mode == "out_residual":
            K, N = D, D
        elif mode == "norm_swiglu":
            K, N = D, 2 * F
        else:
            K, N = F, D
        x = rng.standard_normal((S, K)).astype(np.float32)
        W = oracle.round((rng.standard_normal((K, N)) * 0.05).astype(np.float32), BF16)
        bias = rng.standard_normal(N).astype(np.float32)
        res = rng.standard_normal((S, N)).astype(np.float32)
        w16 = torch.from_numpy(W).cuda().to(torch.bfloat16)
        if mode.startswith("norm"):
            nw = (1.0 + 0.1 * rng.standard_normal(K)).astype(np.float32)
            xn, _ = oracle.rmsnorm_fwd(x, nw, 1e-5)
            want = oracle.gemm_bias(oracle.round(xn, BF16), W, bias, None)
            x_in = dict(x32=torch.from_numpy(x).cuda(), norm_w=torch.from_numpy(nw).cuda())
        else:
            xb = oracle.round(x, BF16)
            want = oracle.gemm_bias(xb, W, bias, res)
            x_in = dict(x16=torch.from_numpy(xb).cuda().to(torch.bfloat16), residual=torch.from_numpy(res).cuda())
        if mode == "norm_swiglu":
            h = torch.full((S, F), float("nan"), device="cuda", dtype=torch.bfloat16)
            tb.decode_linear(w16, S, N, K, bias=torch.from_numpy(bias).cuda(), h16=h, **x_in)
            tb.sync_check()
            got = h.float().cpu().numpy()
            want = oracle.swiglu_fwd(want)
            assert rel_to_maxabs(got, want) <= 6e-3, (mode, S)          # one bf16 rounding of the output
        else:
            y = torch.full((S, N), float("nan"), device="cuda")
            tb.decode_linear(w16, S, N, K, bias=torch.from_numpy(bias).cuda(), y32=y, **x_in)
            tb.sync_check()
            # a normalised value that sits on a bf16 rounding boundary may round the other way than the oracle's
            assert rel_to_maxabs(y.cpu().numpy(), want) <= (2e-3 if mode.startswith("norm") else 2e-5), (mode, S)


def test_lean_decode_step_matches_general_step(tb, oracle, monkeypatch):
    """TB_DECODE_LEAN=1 routes the decode step through tb_decode_linear's kernel: same tokens as the default step
    wherever the logits' top-2 margin is clear, logits within the BF16-mode bound of each other."""
    from turkce_llm_b200.decode import Decoder
    V, D, H, L, F, S, prompt_len, n_new = 500, 256, 4, 3, 1024, 64, 9, 6
    p = make_params(oracle, (V, D, H, L, F, 1, 1, 1e-5), 5)
    prompts = np.random.default_rng(6).integers(0, V, (S, prompt_len)).astype(np.uint32)
    outs = []
    for lean in (False, True):
        if lean:
            monkeypatch.setenv("TB_DECODE_LEAN", "1")
        dec = Decoder(V, D, H, L, F, S, prompt_len + n_new + 2)
        dec.upload(p)
        dec.prefill(prompts)
        dec.generate(1)
        outs.append(dec.logits())
        dec.destroy()
    assert rel_to_maxabs(outs[1], outs[0]) <= 2e-2


@pytest.mark.parametrize("dims", [(500, 256, 4, 3, 1024, 64, 9, 6), (300, 128, 2, 2, 256, 5, 20, 6),
                                  (31769, 384, 6, 12, 1024, 64, 16, 4)])
def test_one_kernel_decode_step_matches_launch_per_kernel_step(tb, oracle, monkeypatch, dims):
    """The default decode step runs every layer in one cooperative kernel (three launches per token with the final
    norm and the head); TB_DECODE_NO_MEGA=1 selects the launch-per-kernel step.  Same bf16 operands and the same
    RMSNorm summation order, so the logits differ only by the accumulation order of the products."""
    from turkce_llm_b200 import lib
    from turkce_llm_b200.decode import Decoder
    V, D, H, L, F, S, prompt_len, n_new = dims
    p = make_params(oracle, (V, D, H, L, F, 1, 1, 1e-5), 5)
    prompts = np.random.default_rng(6).integers(0, V, (S, prompt_len)).astype(np.uint32)
    outs, toks, launches = [], [], []
    for mega in (True, False):
        if not mega:
            monkeypatch.setenv("TB_DECODE_NO_MEGA", "1")
        dec = Decoder(V, D, H, L, F, S, prompt_len + n_new + 2)
        dec.upload(p)
        dec.prefill(prompts)
        dec.generate(1)                      # (the first step of a decoder runs outside a graph)
        before = lib.launch_count()
        dec.generate(n_new - 1)
        launches.append((lib.launch_count() - before) // (n_new - 1))
        outs.append(dec.logits())
        toks.append(dec.tokens(n_new + 1))
        dec.destroy()
    assert launches[0] <= 4 and launches[1] > 5 * L, launches
    # a sequence whose greedy choice fell the other way at a near-tie sees other inputs from then on: compare the rest
    same_so_far = (toks[0][:, :-1] == toks[1][:, :-1]).all(axis=1)
    assert same_so_far.mean() >= 0.8, same_so_far.mean()
    assert rel_to_maxabs(outs[0][same_so_far], outs[1][same_so_far]) <= 1e-2
    srt = np.sort(outs[1], axis=1)
    clear = (srt[:, -1] - srt[:, -2]) > 2e-2 * np.abs(outs[1]).max()
    assert np.array_equal(toks[0][same_so_far & clear, -1], toks[1][same_so_far & clear, -1])
