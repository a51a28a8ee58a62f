"""The allocation-free split-K GEMM (tb_gemm_bf16_splitk_static) against the regular entry point.

This file is collected last, so a run that stops at the first failure has already run every other
test.  The static entry point is called twice in a row on different problems: the scratch array keeps
the first call's partial sums, and the second result must not see them.  When this file runs alone in
a fresh process the static calls are also the first use of the library on the device (hosts that cannot
allocate device memory will not have called tb_init either); after the other tests the library is
already initialised, and the results must be the same.
"""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

TOL = 2e-5      # the bound the other GEMM tests use for equal operands


def _operands(kind, M, N, K, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    a_shape = (K, M) if kind == 2 else (M, K)
    b_shape = (N, K) if kind == 1 else (K, N)
    A = torch.randn(a_shape, device="cuda", generator=g).to(torch.bfloat16)
    B = (torch.randn(b_shape, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    return A, B, a_shape[1], b_shape[1]


def test_static_scratch_entry_matches_regular_entry():
    from turkce_llm_b200 import lib
    assert torch.cuda.is_available(), "a test marked gpu ran without a CUDA device"
    torch.cuda.set_device(0)
    lib.load()
    cases = [(2, 384, 1152, 8192, 4), (0, 256, 200, 4096, 6)]     # weight-gradient shape (TN), then a ragged NN
    statics = []
    for i, (kind, M, N, K, splits) in enumerate(cases):
        A, B, lda, ldb = _operands(kind, M, N, K, 40 + i)
        bias = torch.randn(N, device="cuda")
        C0 = torch.randn(M, N, device="cuda")
        C = C0.clone()
        lib.gemm_bf16_splitk_static(kind, A, B, M, N, K, lda, ldb, C, N, bias=bias, alpha=0.5, beta=1.0,
                                    splits=splits, wait=True)
        statics.append((kind, M, N, K, splits, A, B, lda, ldb, bias, C0, C))
    # the asynchronous form: the caller reads the status word itself, without allocating
    kind, M, N, K, splits, A, B, lda, ldb, bias, C0, C = statics[0]
    C_async = C0.clone()
    lib.gemm_bf16_splitk_static(kind, A, B, M, N, K, lda, ldb, C_async, N, bias=bias, alpha=0.5, beta=1.0,
                                splits=splits, wait=False)
    lib.gemm_bf16_splitk_static_status()
    assert torch.equal(C_async, C)
    # only now the regular path (this initialises the library's own state and scratch on the device)
    lib.init(0)
    for kind, M, N, K, splits, A, B, lda, ldb, bias, C0, C in statics:
        R = C0.clone()
        lib.gemm_bf16(kind, A, B, M, N, K, lda, ldb, C32=R, ldc32=N, bias=bias, alpha=0.5, beta=1.0, splits=splits)
        lib.sync_check()
        err = ((C - R).abs().max() / R.abs().max()).item()
        assert err <= TOL, (kind, M, N, K, err)
        assert torch.equal(C, R)      # same kernels, same split order: in fact bit-identical
        opA = A.float().T if kind == 2 else A.float()
        opB = B.float().T if kind == 1 else B.float()
        want = 0.5 * (opA.double() @ opB.double()).float() + bias + C0
        assert ((C - want).abs().max() / want.abs().max()).item() <= TOL


def test_static_scratch_entry_rejects_oversize():
    from turkce_llm_b200 import lib
    torch.cuda.set_device(0)
    lib.load()
    M, N, K = 2048, 2048, 1024
    A = torch.zeros(M, K, device="cuda", dtype=torch.bfloat16)
    B = torch.zeros(K, N, device="cuda", dtype=torch.bfloat16)
    C = torch.zeros(M, N, device="cuda")
    with pytest.raises(lib.TbError, match="exceeds the built-in scratch"):
        lib.gemm_bf16_splitk_static(0, A, B, M, N, K, K, N, C, N, splits=2)      # 8.4M floats > 4,194,304
    lib.gemm_bf16_splitk_static(0, A, B, M, N, K, K, N, C, N, splits=1)           # no partials needed: accepted
