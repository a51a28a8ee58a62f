"""Generates the golden fixtures in this folder from the REFERENCE's own CPU code.

Run where the reference checkout is available (it builds oracle/_ref/libref.so from the
reference's unmodified sources, see oracle/Makefile):

    python tests/golden/make_golden.py /path/to/reference [train_loop]

Inputs come from numpy's seeded generator (reproducible anywhere), outputs from the reference:
tensor_matmul2d / backward_matmul2d, causal_self_attention, swiglu_feedforward,
lm_init + data_parallel_step + adam_step.  Small cases store the full outputs; cases at the
benchmark's shapes store a SHA-256 of the output bytes plus a few sampled values, which is
enough because the oracle's float32 GEMM is bit-identical to the reference's.
"""
import hashlib
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import pyoracle  # noqa: E402


def digest(a):
    return hashlib.sha256(np.ascontiguousarray(a, dtype=np.float32).tobytes()).hexdigest()


def gemm_inputs(seed, M, K, N):
    """X, dY ~ N(0,1); W ~ N(0,0.02) -- the value distributions of the benchmark's GEMMs."""
    rng = np.random.default_rng(seed)
    X = rng.standard_normal((M, K)).astype(np.float32)
    W = (rng.standard_normal((K, N)) * 0.02).astype(np.float32)
    dY = rng.standard_normal((M, N)).astype(np.float32)
    return X, W, dY


def train_loop_fixtures(ref):
    """Window sampling (model/gpu_train.c:296-307), learning-rate schedule (training/lr_schedule.c:6-15) and
    the checkpoint file (training/checkpoint.c:24-74) of the reference's small end-to-end model."""
    cases = []
    for num_tokens, T, B, seed_base in [(4000, 12, 5, 2026), (100000, 128, 8, 2027), (2_000_000, 1024, 8, 2226),
                                        (70, 64, 3, 5), (1 << 20, 256, 64, 123456789)]:
        tokens = np.arange(num_tokens, dtype=np.uint32)          # ids[w*T] is then the window's start
        ids, tgt = ref.sample_batch(tokens, T, B, seed_base)
        assert np.array_equal(tgt, ids + 1)
        cases.append({"num_tokens": num_tokens, "T": T, "B": B, "seed_base": seed_base,
                      "starts": [int(x) for x in ids[::T]]})
    sched = []
    for step in [0, 1, 10, 999, 1000, 1001, 5000, 35000, 69999, 70000, 90000]:
        sched.append({"step": step, "lr_bits": int(np.float32(ref.lr_warmup_cosine(step, 1000, 70000, 6e-4, 6e-5))
                                                   .view(np.uint32))})
    sched.append({"step": 3, "warmup": 0, "total": 10, "lr_bits": int(np.float32(
        ref.lr_warmup_cosine(3, 0, 10, 1e-3, 1e-4)).view(np.uint32))})
    g = np.load(os.path.join(HERE, "model_step_small.npz"))
    V, D, H, L, F, T, Bn = [int(x) for x in g["dims"]]
    lm = pyoracle.RefLM(ref, V, D, H, L, F, 1e-5, 1337, 1)
    lm.set(0, g["params1"]); lm.set(2, g["adam_m"]); lm.set(3, g["adam_v"]); lm.set_adam_t(1)
    digests = {}
    for with_opt in (0, 1):
        path = "/tmp/_golden_ckpt_%d.bin" % with_opt
        assert lm.checkpoint_save(path, with_opt)
        data = open(path, "rb").read()
        digests["with_opt_%d" % with_opt] = {"bytes": len(data), "sha256": hashlib.sha256(data).hexdigest()}
        os.remove(path)
    lm.close()
    json.dump({"windows": cases, "schedule": sched, "checkpoint_of_model_step_small": digests},
              open(os.path.join(HERE, "train_loop.json"), "w"), indent=1)


def main():
    if len(sys.argv) > 2 and sys.argv[2] == "train_loop":
        pyoracle.build_ref(sys.argv[1])
        train_loop_fixtures(pyoracle.Ref())
        return
    if len(sys.argv) < 2:
        raise SystemExit("usage: make_golden.py <reference checkout> [train_loop]")
    ref_root = sys.argv[1]
    pyoracle.build_ref(ref_root)
    ref = pyoracle.Ref()

    # ---- known-answer vectors the reference's own tests hold --------------------------
    ka = {}
    A = np.array([[1, 2], [3, 4]], np.float32)
    B = np.array([[5, 6], [7, 8]], np.float32)
    ka["test_tensor_2x2"] = {"A": A.tolist(), "B": B.tolist(), "C": ref.matmul2d(A, B).tolist(),
                             "source": "tests/test_tensor.c:118-141 expects [[19,22],[43,50]]"}
    At = np.ascontiguousarray(A.T)
    ka["test_tensor_2x2_transposed_view"] = {"A_stored": At.tolist(), "B": B.tolist(),
                                             "C": ref.matmul2d(At.T, B).tolist(),
                                             "source": "tests/test_tensor.c:118-141 (transposed-view input)"}
    A2 = np.array([(i % 7) - 3 for i in range(12)], np.float32).reshape(4, 3)
    B2 = np.array([(i % 5) * 0.5 for i in range(15)], np.float32).reshape(3, 5)
    ka["test_cuda_4x3x5"] = {"A": A2.tolist(), "B": B2.tolist(), "C": ref.matmul2d(A2, B2).tolist(),
                             "source": "tests/test_cuda.c:55-94 (A[i]=(i%7)-3, B[i]=(i%5)*0.5)"}
    with open(os.path.join(HERE, "matmul_known_answers.json"), "w") as f:
        json.dump(ka, f, indent=1)

    # ---- small GEMM triples with full outputs (fwd, dX, dW as backward_matmul2d forms them)
    small = {}
    for i, (name, (M, K, N)) in enumerate({"s0": (64, 48, 32), "s1": (33, 20, 17), "s2": (128, 96, 72)}.items()):
        X, W, dY = gemm_inputs(100 + i, M, K, N)
        C, dX, dW = ref.matmul2d_fwd_bwd(X, W, dY)
        small[name + "_shape"] = np.array([M, K, N])
        small[name + "_seed"] = np.array([100 + i])
        small[name + "_C"], small[name + "_dX"], small[name + "_dW"] = C, dX, dW
    np.savez_compressed(os.path.join(HERE, "gemm_small.npz"), **small)

    # ---- layer GEMMs at the CPU-reference configuration's shapes (M = 4*256 tokens): digests only
    big = {}
    shapes = {"qkv": (1024, 384, 1152), "out": (1024, 384, 384), "gate_up": (1024, 384, 2048),
              "down": (1024, 1024, 384)}
    for i, (name, (M, K, N)) in enumerate(shapes.items()):
        X, W, dY = gemm_inputs(200 + i, M, K, N)
        C, dX, dW = ref.matmul2d_fwd_bwd(X, W, dY)
        big[name] = {"M": M, "K": K, "N": N, "seed": 200 + i,
                     "C_sha256": digest(C), "dX_sha256": digest(dX), "dW_sha256": digest(dW),
                     "C_sample": C.reshape(-1)[::max(1, C.size // 16)][:16].tolist(),
                     "dX_sample": dX.reshape(-1)[::max(1, dX.size // 16)][:16].tolist(),
                     "dW_sample": dW.reshape(-1)[::max(1, dW.size // 16)][:16].tolist()}
        print("layer GEMM", name, "done", flush=True)
    with open(os.path.join(HERE, "gemm_layer_digests.json"), "w") as f:
        json.dump(big, f, indent=1)

    # ---- attention block and feed-forward block, forward + backward
    rng = np.random.default_rng(300)
    Bn, T, H, D = 2, 24, 2, 32
    x = rng.standard_normal((Bn * T, D)).astype(np.float32)
    w_qkv = (rng.standard_normal((D, 3 * D)) * 0.2).astype(np.float32)
    b_qkv = (rng.standard_normal(3 * D) * 0.1).astype(np.float32)
    wo = (rng.standard_normal((D, D)) * 0.2).astype(np.float32)
    bo = (rng.standard_normal(D) * 0.1).astype(np.float32)
    dout = rng.standard_normal((Bn * T, D)).astype(np.float32)
    out, dx, dw, db, dwo, dbo = ref.attention_fwd_bwd(x, w_qkv, b_qkv, wo, bo, dout, Bn, T, H)
    np.savez_compressed(os.path.join(HERE, "attention_block.npz"), dims=np.array([Bn, T, H, D]), x=x, w_qkv=w_qkv,
                        b_qkv=b_qkv, wo=wo, bo=bo, dout=dout, out=out, dx=dx, dw_qkv=dw, db_qkv=db, dwo=dwo, dbo=dbo)

    F = 40
    N = 36
    x = rng.standard_normal((N, D)).astype(np.float32)
    w_gu = (rng.standard_normal((D, 2 * F)) * 0.2).astype(np.float32)
    b_gu = (rng.standard_normal(2 * F) * 0.1).astype(np.float32)
    w_down = (rng.standard_normal((F, D)) * 0.2).astype(np.float32)
    b_down = (rng.standard_normal(D) * 0.1).astype(np.float32)
    dout = rng.standard_normal((N, D)).astype(np.float32)
    out, dx, dwg, dbg, dwd, dbd = ref.ffn_fwd_bwd(x, w_gu, b_gu, w_down, b_down, dout)
    np.savez_compressed(os.path.join(HERE, "ffn_block.npz"), dims=np.array([N, D, F]), x=x, w_gu=w_gu, b_gu=b_gu,
                        w_down=w_down, b_down=b_down, dout=dout, out=out, dx=dx, dw_gu=dwg, db_gu=dbg, dw_down=dwd,
                        db_down=dbd)

    # ---- whole-model step: the reference's own small end-to-end case
    # (tests/test_gpu_train.c:261-263: V=50 D=32 H=2 L=2 F=48 T=12 B=5, model seed (1337,1),
    #  tokens from pcg_seed(4242,7), data seed 2026), then one adam_step with lr 3e-4.
    V, D, H, L, F, T, Bn = 50, 32, 2, 2, 48, 12, 5
    lm = pyoracle.RefLM(ref, V, D, H, L, F, 1e-5, 1337, 1)
    tokens = ref.range_u32(4000, 4242, 7, 0, V - 1)
    params0 = lm.params()
    loss = lm.dp_step(tokens, T, Bn, 2026)
    grads = lm.grads()
    ids, tgt = ref.sample_batch(tokens, T, Bn, 2026)
    lm.adam_step(3e-4)
    params1 = lm.params()
    np.savez_compressed(os.path.join(HERE, "model_step_small.npz"), dims=np.array([V, D, H, L, F, T, Bn]),
                        params0=params0, ids=ids, targets=tgt, loss=np.float32(loss), grads=grads, params1=params1,
                        adam_m=lm.get(2), adam_v=lm.get(3), numels=np.array(lm.param_numels()))
    lm.close()

    # ---- rope tables and host scalars
    c, s = ref.rope_tables(32, 16)
    np.savez_compressed(os.path.join(HERE, "rope_tables.npz"), cos=c, sin=s)
    train_loop_fixtures(ref)
    print("golden fixtures written to", HERE)


if __name__ == "__main__":
    main()
