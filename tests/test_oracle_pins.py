"""Pins the CPU oracle (oracle/oracle.c) to the reference: the reference's own known-answer
tests, fixtures generated from the reference's unmodified CPU sources (tests/golden/), and --
where oracle/_ref/libref.so exists -- the reference itself, live."""
import hashlib
import json

import numpy as np
import pytest

from conftest import golden_path, rel_to_maxabs
from oracle.pyoracle import BF16, FP32

import os
import sys
sys.path.insert(0, os.path.join(os.path.dirname(__file__), "golden"))
from make_golden import gemm_inputs  # noqa: E402  (the committed input generator)


def sha(a):
    return hashlib.sha256(np.ascontiguousarray(a, dtype=np.float32).tobytes()).hexdigest()


def test_known_answers(oracle):
    ka = json.load(open(golden_path("matmul_known_answers.json")))
    c = ka["test_tensor_2x2"]
    got = oracle.gemm(0, 0, np.array(c["A"], np.float32), np.array(c["B"], np.float32), 2, 2, 2).reshape(2, 2)
    assert got.tolist() == [[19.0, 22.0], [43.0, 50.0]] == c["C"]
    c = ka["test_tensor_2x2_transposed_view"]
    got = oracle.gemm(1, 0, np.array(c["A_stored"], np.float32), np.array(c["B"], np.float32), 2, 2, 2).reshape(2, 2)
    assert got.tolist() == c["C"]
    c = ka["test_cuda_4x3x5"]
    got = oracle.gemm(0, 0, np.array(c["A"], np.float32), np.array(c["B"], np.float32), 4, 5, 3).reshape(4, 5)
    assert got.tolist() == c["C"]


def test_small_gemms_bit_exact(oracle):
    g = np.load(golden_path("gemm_small.npz"))
    for name in ("s0", "s1", "s2"):
        M, K, N = (int(v) for v in g[name + "_shape"])
        X, W, dY = gemm_inputs(int(g[name + "_seed"][0]), M, K, N)
        C = oracle.gemm(0, 0, X, W, M, N, K).reshape(M, N)
        dX = oracle.gemm(0, 1, dY, W, M, K, N).reshape(M, K)     # dX = dY @ W^T
        dW = oracle.gemm(1, 0, X, dY, K, N, M).reshape(K, N)     # dW = X^T @ dY
        assert np.array_equal(C.view(np.uint32), g[name + "_C"].view(np.uint32))
        assert np.array_equal(dX.view(np.uint32), g[name + "_dX"].view(np.uint32))
        assert np.array_equal(dW.view(np.uint32), g[name + "_dW"].view(np.uint32))


@pytest.mark.parametrize("name", ["qkv", "out", "gate_up", "down"])
def test_layer_gemms_digest(oracle, name):
    d = json.load(open(golden_path("gemm_layer_digests.json")))[name]
    M, K, N = d["M"], d["K"], d["N"]
    X, W, dY = gemm_inputs(d["seed"], M, K, N)
    assert sha(oracle.gemm(0, 0, X, W, M, N, K)) == d["C_sha256"]
    assert sha(oracle.gemm(0, 1, dY, W, M, K, N)) == d["dX_sha256"]
    assert sha(oracle.gemm(1, 0, X, dY, K, N, M)) == d["dW_sha256"]


def test_bf16_rounding(oracle):
    # round-to-nearest-even on the upper 16 bits (cuda/train_kernels.cu:207-212)
    cases = {0x3F800000: 0x3F800000, 0x3F808000: 0x3F800000, 0x3F818000: 0x3F820000, 0x3F808001: 0x3F810000,
             0x3F80FFFF: 0x3F810000, 0xBF808000: 0xBF800000, 0x00000000: 0x00000000}
    for src, want in cases.items():
        x = np.array([src], dtype=np.uint32).view(np.float32)
        got = oracle.round(x, BF16).view(np.uint32)[0]
        assert got == want, (hex(src), hex(got), hex(want))
    import torch
    v = np.random.default_rng(0).standard_normal(4096).astype(np.float32)
    t = torch.from_numpy(v).to(torch.bfloat16).to(torch.float32).numpy()
    assert np.array_equal(oracle.round(v, BF16).view(np.uint32), t.view(np.uint32))


def test_attention_block_golden(oracle):
    g = np.load(golden_path("attention_block.npz"))
    B, T, H, D = (int(v) for v in g["dims"])
    hd = D // H
    x, w_qkv, b_qkv, wo, bo, dout = (g[k] for k in ("x", "w_qkv", "b_qkv", "wo", "bo", "dout"))
    qkv = oracle.gemm_bias(x, w_qkv, b_qkv, None)
    Q, K, V = oracle.qkv_rope_split(qkv, B, T, H, hd)
    scale = 1.0 / np.sqrt(np.float32(hd))
    O = oracle.attention_fwd(Q, K, V, scale)
    att = oracle.heads_merge(O, B, T, H, hd)
    out = oracle.gemm_bias(att, wo, bo, None)
    assert rel_to_maxabs(out, g["out"]) < 2e-6
    # backward
    dbo = dout.sum(0)
    dwo = oracle.gemm(1, 0, att, dout, D, D, B * T).reshape(D, D)
    datt = oracle.gemm(0, 1, dout, wo, B * T, D, D).reshape(B * T, D)
    dO = oracle.heads_split(datt, B, T, H, hd)
    dQ, dK, dV = oracle.attention_bwd(Q, K, V, dO, scale)
    dqkv = oracle.qkv_rope_merge_bwd(dQ, dK, dV, B, T, H, hd)
    dw = oracle.gemm(1, 0, x, dqkv, D, 3 * D, B * T).reshape(D, 3 * D)
    dx = oracle.gemm(0, 1, dqkv, w_qkv, B * T, D, 3 * D).reshape(B * T, D)
    for got, key in ((dx, "dx"), (dw, "dw_qkv"), (dqkv.sum(0), "db_qkv"), (dwo, "dwo"), (dbo, "dbo")):
        assert rel_to_maxabs(got, g[key]) < 5e-6, key


def test_ffn_block_golden(oracle):
    g = np.load(golden_path("ffn_block.npz"))
    N, D, F = (int(v) for v in g["dims"])
    x, w_gu, b_gu, w_down, b_down, dout = (g[k] for k in ("x", "w_gu", "b_gu", "w_down", "b_down", "dout"))
    gu = oracle.gemm_bias(x, w_gu, b_gu, None)
    h = oracle.swiglu_fwd(gu)
    out = oracle.gemm_bias(h, w_down, b_down, None)
    assert rel_to_maxabs(out, g["out"]) < 2e-6
    dh = oracle.gemm(0, 1, dout, w_down, N, F, D).reshape(N, F)
    dgu = oracle.swiglu_bwd(gu, dh)
    assert rel_to_maxabs(oracle.gemm(1, 0, h, dout, F, D, N), g["dw_down"].reshape(-1)) < 5e-6
    assert rel_to_maxabs(oracle.gemm(1, 0, x, dgu, D, 2 * F, N), g["dw_gu"].reshape(-1)) < 5e-6
    assert rel_to_maxabs(oracle.gemm(0, 1, dgu, w_gu, N, D, 2 * F), g["dx"].reshape(-1)) < 5e-6
    assert rel_to_maxabs(oracle.colsum_acc(dgu), g["db_gu"]) < 5e-6
    assert rel_to_maxabs(oracle.colsum_acc(dout), g["db_down"]) < 5e-6


def test_model_step_golden(oracle):
    """The reference's small end-to-end case (tests/test_gpu_train.c:261-263) through its CPU
    production path: loss, every gradient tensor, and the weights after one Adam step."""
    g = np.load(golden_path("model_step_small.npz"))
    V, D, H, L, F, T, B = (int(v) for v in g["dims"])
    cfg = (V, D, H, L, F, T, B, 1e-5)
    assert oracle.model_total_scalars(cfg) == g["params0"].size == int(g["numels"].sum())
    loss, grads, _ = oracle.model_forward_backward(cfg, g["params0"], g["ids"], g["targets"])
    assert abs(loss - float(g["loss"])) <= 2e-6 * abs(float(g["loss"]))
    off = 0
    for n in g["numels"]:
        n = int(n)
        assert rel_to_maxabs(grads[off:off + n], g["grads"][off:off + n]) < 1e-5
        off += n
    bc1, bc2 = 1.0 - 0.9, 1.0 - 0.999
    p1, m1, v1 = oracle.adam(g["params0"], g["grads"], np.zeros_like(grads), np.zeros_like(grads), 3e-4, 0.9, 0.999,
                             1e-8, np.float32(bc1), np.float32(bc2))
    assert np.abs(p1 - g["params1"]).max() <= 1e-3 * 3e-4      # the reference's own Adam bound (test_gpu_train.c:199)
    assert rel_to_maxabs(m1, g["adam_m"]) < 1e-6 and rel_to_maxabs(v1, g["adam_v"]) < 1e-6


def test_rope_tables_golden(oracle):
    g = np.load(golden_path("rope_tables.npz"))
    c, s = oracle.rope_tables(32, 16)
    assert np.abs(c - g["cos"]).max() < 2e-6 and np.abs(s - g["sin"]).max() < 2e-6


def test_bf16_mode_close_to_fp32(oracle):
    X, W, dY = gemm_inputs(7, 96, 384, 80)
    c32 = oracle.gemm(0, 0, X, W, 96, 80, 384)
    c16 = oracle.gemm(0, 0, X, W, 96, 80, 384, mode=BF16)
    assert 0 < rel_to_maxabs(c16, c32) < 2e-2
    truth = oracle.gemm_f64(0, 0, X, W, 96, 80, 384).reshape(-1)
    assert rel_to_maxabs(c32, truth) < 1e-5


# ---- live against the reference's compiled CPU code (skipped where it was not built) ----

def test_live_matmul_bit_exact(oracle, ref):
    rng = np.random.default_rng(5)
    for (M, K, N) in ((17, 9, 23), (64, 48, 32), (130, 70, 65)):
        A = rng.standard_normal((M, K)).astype(np.float32)
        B = rng.standard_normal((K, N)).astype(np.float32)
        dC = rng.standard_normal((M, N)).astype(np.float32)
        C, dA, dB = ref.matmul2d_fwd_bwd(A, B, dC)
        assert np.array_equal(C.view(np.uint32), oracle.gemm(0, 0, A, B, M, N, K).reshape(M, N).view(np.uint32))
        assert np.array_equal(dA.view(np.uint32), oracle.gemm(0, 1, dC, B, M, K, N).reshape(M, K).view(np.uint32))
        assert np.array_equal(dB.view(np.uint32), oracle.gemm(1, 0, A, dC, K, N, M).reshape(K, N).view(np.uint32))
        # transposed views, as backward_matmul2d passes them (autograd/node.c:116-127)
        assert np.array_equal(ref.matmul2d(dC, B.T).view(np.uint32), dA.view(np.uint32))


def test_live_model_step(oracle, ref):
    from oracle.pyoracle import RefLM
    V, D, H, L, F, T, B = 61, 16, 2, 1, 24, 9, 3
    lm = RefLM(ref, V, D, H, L, F, 1e-5, 11, 3, arena=1 << 30)
    tokens = ref.range_u32(700, 5, 2, 0, V - 1)
    loss = lm.dp_step(tokens, T, B, 77, step_arena=256 << 20)
    ids, tgt = ref.sample_batch(tokens, T, B, 77)
    lo, grads, _ = oracle.model_forward_backward((V, D, H, L, F, T, B, 1e-5), lm.params(), ids, tgt)
    assert abs(lo - loss) <= 2e-6 * abs(loss)
    assert rel_to_maxabs(grads, lm.grads()) < 1e-5
    lm.close()
