"""Single-kernel micro-benchmarks through the C ABI (also the programs the ncu captures run).

    python -m turkce_llm_b200.microbench gemm M N K kind [iters] [out=f32|bf16] [tile_n] [splits]
    python -m turkce_llm_b200.microbench attention B H T hd [iters]

kind: 0 = NN, 1 = NT, 2 = TN.  Prints the mean device time per launch (CUDA events) and the
algorithmic throughput.
"""
import sys

import torch

from . import lib


def gemm(M, N, K, kind, iters=20, out="f32", tile_n=0, splits=1):
    lib.init(0)
    a_shape = (K, M) if kind == 2 else (M, K)
    b_shape = (N, K) if kind == 1 else (K, N)
    A = torch.randn(a_shape, device="cuda").to(torch.bfloat16)
    B = (torch.randn(b_shape, device="cuda") * 0.02).to(torch.bfloat16)
    C32 = torch.empty(M, N, device="cuda") if out == "f32" else None
    C16 = torch.empty(M, N, device="cuda", dtype=torch.bfloat16) if out == "bf16" else None

    def run():
        lib.gemm_bf16(kind, A, B, M, N, K, a_shape[1], b_shape[1], C32=C32, ldc32=N, C16=C16, ldc16=N,
                      splits=splits, tile_n=tile_n)
    for _ in range(3):
        run()
    lib.sync_check()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        run()
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / iters
    print("gemm kind=%d %dx%dx%d out=%s tile_n=%d splits=%d: %.2f us  %.1f TFLOP/s"
          % (kind, M, N, K, out, tile_n, splits, us, 2.0 * M * N * K / us / 1e6), flush=True)
    return us


def attention(B, H, T, hd, iters=10):
    lib.init(0)
    g = torch.Generator(device="cuda").manual_seed(0)
    Q, K, V = (torch.randn(B * H, T, hd, device="cuda", generator=g).to(torch.bfloat16) for _ in range(3))
    att = torch.zeros(B * T, H * hd, device="cuda", dtype=torch.bfloat16)
    datt = torch.randn(B * T, H * hd, device="cuda", generator=g).to(torch.bfloat16)
    lse = torch.zeros(B * H, T, device="cuda")
    delta = torch.zeros(B * H, T, device="cuda")
    dQ, dK, dV = (torch.zeros(B * H, T, hd, device="cuda") for _ in range(3))
    scale = float(hd) ** -0.5
    for _ in range(2):
        lib.attention_fwd(Q, K, V, att, lse, B, H, T, hd, scale)
        lib.attention_bwd(Q, K, V, att, datt, lse, delta, dQ, dK, dV, B, H, T, hd, scale)
    lib.sync_check()
    e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    e[0].record()
    for _ in range(iters):
        lib.attention_fwd(Q, K, V, att, lse, B, H, T, hd, scale)
    e[1].record()
    for _ in range(iters):
        lib.attention_bwd(Q, K, V, att, datt, lse, delta, dQ, dK, dV, B, H, T, hd, scale)
    e[2].record()
    torch.cuda.synchronize()
    tri = B * H * T * T * hd            # flops of one lower-triangular product
    f_us = e[0].elapsed_time(e[1]) * 1e3 / iters
    b_us = e[1].elapsed_time(e[2]) * 1e3 / iters
    print("attention B=%d H=%d T=%d hd=%d: fwd %.1f us (%.1f TFLOP/s)  bwd %.1f us (%.1f TFLOP/s)"
          % (B, H, T, hd, f_us, 2 * tri / f_us / 1e6, b_us, 7 * tri / b_us / 1e6), flush=True)
    return f_us, b_us


def main(argv):
    if len(argv) >= 5 and argv[0] == "gemm":
        M, N, K, kind = (int(x) for x in argv[1:5])
        iters = int(argv[5]) if len(argv) > 5 else 20
        out = argv[6] if len(argv) > 6 else "f32"
        tile_n = int(argv[7]) if len(argv) > 7 else 0
        splits = int(argv[8]) if len(argv) > 8 else 1
        gemm(M, N, K, kind, iters, out, tile_n, splits)
    elif len(argv) >= 5 and argv[0] == "attention":
        B, H, T, hd = (int(x) for x in argv[1:5])
        attention(B, H, T, hd, int(argv[5]) if len(argv) > 5 else 10)
    else:
        print(__doc__)
        return 2
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
