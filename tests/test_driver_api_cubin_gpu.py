"""The Driver-API route: this library's GEMM kernels as an sm_100a module image under the reference's kernel names,
loaded and launched by the reference's own UNMODIFIED loader (cuda/cuda_backend.c: cuModuleLoadData,
cuModuleGetFunction, cuLaunchKernel with void** parameters on the NULL stream, a context of the reference's own),
with the launch geometry of the reference's host helpers (model/gpu_train.c:45-118, cuda/cuda_backend.c:141-148).

 * every GEMM entry of turkce_llm_b200/turkce_b200_gemm.cubin against the CPU oracle on seeded inputs (off-tile,
   strided, batched, alpha/beta, bias/residual cases), and the reference's known-answer vectors;
 * the reference's whole GPU trainer (model/gpu_train.c unmodified) running on a module in which exactly the GEMM
   entries are this library's: one training step against the CPU oracle with the bounds of the reference's own
   trainer test (tests/test_gpu_train.c:119,128).

The reference's loader makes a CUDA context of its own current, so each launch runs in a child process."""
import json
import os

import numpy as np
import pytest

from conftest import ROOT, compare_tensor_bad, golden_path, rel_to_maxabs
from oracle.pyoracle import BF16, FP32, TF32

pytestmark = pytest.mark.gpu

CUBIN = os.path.join(ROOT, "turkce_llm_b200", "turkce_b200_gemm.cubin")


@pytest.fixture(scope="module")
def refgpu():
    from oracle import ref_gpu
    if not ref_gpu.available():
        pytest.skip("oracle/_ref/librefgpu.so (the reference's loader) is not built on this machine")
    assert os.path.exists(CUBIN), "turkce_b200_gemm.cubin is missing: run python -m turkce_llm_b200.build"
    return ref_gpu


def launch(refgpu, tmp_path, entry, form, A, B, C0, M, N, K, lda=0, ldb=0, ldc=0, batch=1, sA=0, sB=0, sC=0, alpha=1.0,
           beta=0.0, bias=None, residual=None, module=CUBIN, tag="g"):
    """Grid and block as the reference's helpers compute them: 64 x 64 output blocks (16 x 16 threads for k_gemm_*,
    256 for k_bf16_*), 16 x 16 output blocks for k_matmul."""
    if form == 2:
        gx, gy, gz, bx, by = (N + 15) // 16, (M + 15) // 16, 1, 16, 16          # cuda_launch_2d
    else:
        gx, gy, gz = (N + 63) // 64, (M + 63) // 64, batch
        bx, by = (16, 16) if entry.startswith("k_gemm_") else (256, 1)
    extra = {}
    if bias is not None:
        extra["bias"] = bias
    if residual is not None:
        extra["residual"] = residual
    inp, out = tmp_path / (tag + ".npz"), tmp_path / (tag + ".npy")
    np.savez(inp, entry=entry, form=form, A=A, B=B, C=C0, M=M, N=N, K=K, lda=lda, ldb=ldb, ldc=ldc, sA=sA, sB=sB, sC=sC,
             alpha=alpha, beta=beta, gx=gx, gy=gy, gz=gz, bx=bx, by=by, iters=1, **extra)
    r = refgpu.run_child(["gemm", "--module", module, "--tokens", inp, "--out", out])
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    return np.load(out)


@pytest.mark.parametrize("family", ["k_bf16_gemm", "k_gemm"])
@pytest.mark.parametrize("kind", ["nn", "nt", "tn"])
def test_gemm_entries_match_oracle(refgpu, oracle, tmp_path, family, kind):
    """k_bf16_gemm_* (bf16 operands) and k_gemm_* (float32 operands as tf32): contiguous layer shape, an off-tile
    shape, and a strided batched case with alpha and beta."""
    ta, tb_ = (1 if kind == "tn" else 0), (1 if kind == "nt" else 0)
    mode, tol = (BF16, 2e-2) if family == "k_bf16_gemm" else (TF32, 5e-3)
    rng = np.random.default_rng(hash((family, kind)) % (1 << 31))
    for case, (M, N, K) in enumerate(((256, 384, 384), (130, 70, 100), (1, 1, 1))):
        a_shape = (K, M) if ta else (M, K)
        b_shape = (N, K) if tb_ else (K, N)
        A = rng.standard_normal(a_shape).astype(np.float32)
        B = (rng.standard_normal(b_shape) * 0.05).astype(np.float32)
        got = launch(refgpu, tmp_path, "%s_%s" % (family, kind), 0, A, B, np.full((M, N), np.nan, np.float32), M, N, K,
                     a_shape[1], b_shape[1], N, tag="c%d" % case).reshape(M, N)
        same = oracle.gemm(ta, tb_, A, B, M, N, K, mode=mode).reshape(M, N)
        want = oracle.gemm(ta, tb_, A, B, M, N, K, mode=FP32).reshape(M, N)
        assert np.isfinite(got).all()
        assert rel_to_maxabs(got, same) <= 2e-5, (case, rel_to_maxabs(got, same))
        assert rel_to_maxabs(got, want) <= tol
    # strided, batched, alpha / beta
    M, N, K, batch = 70, 52, 40, 3
    lda = (M if ta else K) + 4
    ldb = (K if tb_ else N) + 8
    ldc = N + 4
    sA, sB, sC = (K if ta else M) * lda + 4, (N if tb_ else K) * ldb + 8, M * ldc + 4
    A = rng.standard_normal(batch * sA).astype(np.float32)
    B = rng.standard_normal(batch * sB).astype(np.float32)
    C0 = rng.standard_normal(batch * sC).astype(np.float32)
    got = launch(refgpu, tmp_path, "%s_%s" % (family, kind), 0, A, B, C0, M, N, K, lda, ldb, ldc, batch, sA, sB, sC, 0.5, 2.0,
                 tag="strided")
    want = oracle.gemm(ta, tb_, A, B, M, N, K, lda, ldb, ldc, batch, sA, sB, sC, alpha=0.5, beta=2.0, C_in=C0, mode=mode)
    assert rel_to_maxabs(got, want) <= 2e-5
    # elements between the rows and between the matrices are not touched
    mask = np.ones(batch * sC, bool)
    for z in range(batch):
        for m in range(M):
            mask[z * sC + m * ldc: z * sC + m * ldc + N] = False
    assert np.array_equal(got[mask], C0[mask])


def test_gemm_bias_entry_and_matmul_entry(refgpu, oracle, tmp_path):
    rng = np.random.default_rng(5)
    M, N, K = 260, 200, 96
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = (rng.standard_normal((K, N)) * 0.05).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    res = rng.standard_normal((M, N)).astype(np.float32)
    for b, r, tag in ((bias, res, "br"), (bias, None, "b"), (None, None, "n")):
        got = launch(refgpu, tmp_path, "k_bf16_gemm_nn_bias", 1, A, B, np.zeros((M, N), np.float32), M, N, K, bias=b, residual=r,
                     tag=tag).reshape(M, N)
        assert rel_to_maxabs(got, oracle.gemm_bias(A, B, b, r, mode=BF16)) <= 2e-5, tag
    # k_matmul: the reference's own known-answer vectors (tests/test_tensor.c:118-141, tests/test_cuda.c:55-94), exact
    ka = json.load(open(golden_path("matmul_known_answers.json")))
    for name in ("test_tensor_2x2", "test_cuda_4x3x5"):
        c = ka[name]
        A, B = np.array(c["A"], np.float32), np.array(c["B"], np.float32)
        M, K = A.shape
        N = B.shape[1]
        got = launch(refgpu, tmp_path, "k_matmul", 2, A, B, np.zeros((M, N), np.float32), M, N, K, tag=name)
        assert got.reshape(M, N).tolist() == c["C"], name
    M, K, N = 100, 130, 90
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = rng.standard_normal((K, N)).astype(np.float32)
    got = launch(refgpu, tmp_path, "k_matmul", 2, A, B, np.zeros((M, N), np.float32), M, N, K, tag="mm").reshape(M, N)
    assert rel_to_maxabs(got, oracle.gemm(0, 0, A, B, M, N, K, mode=TF32).reshape(M, N)) <= 2e-5
    assert rel_to_maxabs(got, oracle.gemm(0, 0, A, B, M, N, K).reshape(M, N)) <= 5e-3


@pytest.mark.parametrize("case", ["off_tile", "real_width"])
def test_reference_trainer_runs_on_the_drop_in_gemm_kernels(refgpu, oracle, tmp_path, case):
    """model/gpu_train.c, unmodified, loading a module whose GEMM entries are this library's (the other 17 kernels
    are the reference's own): one forward + backward against the float32 CPU oracle."""
    if not os.path.exists(refgpu.REFGPU_TB_CUBIN):
        pytest.skip("oracle/_ref/train_kernels_tb_gemm.cubin is not built on this machine")
    V, D, H, L, F, T, B = {"off_tile": (50, 32, 2, 2, 48, 12, 5), "real_width": (31769, 384, 6, 2, 1024, 128, 4)}[case]
    cfg = (V, D, H, L, F, T, B, 1e-5)
    total = oracle.model_total_scalars(cfg)
    rng = np.random.default_rng(1)
    p = (rng.standard_normal(total) * 0.02).astype(np.float32)
    sizes = [V * D] + [D, D * 3 * D, 3 * D, D * D, D, D, D * 2 * F, 2 * F, F * D, D] * L + [D]
    off = np.concatenate([[0], np.cumsum(sizes)[:-1]])
    for i, (o, n) in enumerate(zip(off, sizes)):
        k = (i - 1) % 10 if 0 < i < len(sizes) - 1 else -1
        if i == len(sizes) - 1 or k in (0, 5):
            p[o:o + n] = 1.0 + 0.05 * rng.standard_normal(n)
    ids = rng.integers(0, V, B * T).astype(np.uint32)
    tgt = rng.integers(0, V, B * T).astype(np.uint32)
    np.save(tmp_path / "p.npy", p)
    np.savez(tmp_path / "batch.npz", ids=ids, tgt=tgt)
    r = refgpu.run_child(["step", "--module", refgpu.REFGPU_TB_CUBIN, "--cfg", V, D, H, L, F, T, B, "--params", tmp_path / "p.npy",
                          "--tokens", tmp_path / "batch.npz", "--grads-out", tmp_path / "g.npy", "--out", tmp_path / "s.json"])
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    got = json.load(open(tmp_path / "s.json"))
    grads = np.load(tmp_path / "g.npy")
    want_loss, want_grads, _ = oracle.model_forward_backward(cfg, p, ids, tgt, mode=FP32)
    assert abs(got["loss"] - want_loss) <= 2e-2 * abs(want_loss)
    for i, (o, n) in enumerate(zip(off, sizes)):
        assert compare_tensor_bad(grads[o:o + n], want_grads[o:o + n], 8e-2) == 0, "parameter %d" % i
    assert abs(got["grad_norm"] - oracle.grad_norm(want_grads)) <= 2e-2 * oracle.grad_norm(want_grads)


def test_c_abi_works_inside_the_references_own_context(refgpu, oracle, tmp_path):
    """The other route of the boundary: the C ABI called from the reference's process.  The reference creates a
    context of its own with cuCtxCreate and keeps it current (cuda/cuda_backend.c:56-107, cuda/cuda_backend.h:36-40);
    the library (CUDA runtime API) must work in that context on the reference's CUdeviceptr buffers, as the binding
    of bf16_gemm_bias (model/gpu_train.c:103-107) needs."""
    rng = np.random.default_rng(9)
    M, N, K = 300, 200, 384
    A = rng.standard_normal((M, K)).astype(np.float32)
    B = (rng.standard_normal((K, N)) * 0.05).astype(np.float32)
    bias = rng.standard_normal(N).astype(np.float32)
    res = rng.standard_normal((M, N)).astype(np.float32)
    np.savez(tmp_path / "in.npz", A=A, B=B, bias=bias, residual=res)
    lib_path = os.path.join(ROOT, "turkce_llm_b200", "libturkce_b200.so")
    r = refgpu.run_child(["abi_in_context", "--tokens", tmp_path / "in.npz", "--params", lib_path, "--out", tmp_path / "c.npy"])
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    info = json.load(open(str(tmp_path / "c.npy") + ".json"))
    assert info["rc"] == 0, info
    got = np.load(tmp_path / "c.npy")
    assert rel_to_maxabs(got, oracle.gemm_bias(A, B, bias, res, mode=BF16)) <= 2e-5
