"""Single-kernel micro-benchmarks through the C ABI (also the programs the ncu captures run).

    python -m turkce_llm_b200.microbench gemm M N K kind [iters] [out=f32|bf16] [tile_n] [splits]
    python -m turkce_llm_b200.microbench attention B H T hd [iters]
    python -m turkce_llm_b200.microbench decode S prompt_len new_tokens      (33.49M-parameter model)
    python -m turkce_llm_b200.microbench lmhead S [V] [K] [iters] [copies]   (decode LM head, fused argmax)

kind: 0 = NN, 1 = NT, 2 = TN.  Prints the mean device time per launch (CUDA events) and the
algorithmic throughput.
"""
import sys

import torch

from . import lib


def graph_time_us(run, iters, replays=5):
    """Device time per call with the host out of the picture: `iters` calls captured into one CUDA
    graph on a side stream, the graph replayed and timed with events (mean over the replays)."""
    st = torch.cuda.Stream()
    st.wait_stream(torch.cuda.current_stream())
    g = torch.cuda.CUDAGraph()
    with torch.cuda.stream(st):
        run(0)                                   # everything lazily set up before the capture
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=st):
            for i in range(iters):
                run(i)
        g.replay()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(replays):
            g.replay()
        e1.record()
        torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (iters * replays)


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
    # the kernel's own time: events directly around each launch (not stretched by host launch cost)
    lib.profile_begin()
    for _ in range(iters):
        run()
    prof = lib.profile_end(torch.cuda.current_stream().cuda_stream)
    kus = sum(v["ms"] for k, v in prof.items() if k.startswith("gemm_")) * 1e3 / iters
    gus = graph_time_us(lambda i: run(), iters)
    print("  in a CUDA graph (no host launch cost): %.2f us per call = %.1f TFLOP/s" % (gus, 2.0 * M * N * K / gus / 1e6))
    a_bytes, b_bytes = 2.0 * M * K, 2.0 * K * N
    c_bytes = M * N * (4.0 if out == "f32" else 2.0)
    print("gemm kind=%d %dx%dx%d out=%s tile_n=%d splits=%d: %.2f us per call, kernel %.2f us = %.1f TFLOP/s, "
          "%.0f GB/s of operand+result bytes"
          % (kind, M, N, K, out, tile_n, splits, us, kus, 2.0 * M * N * K / kus / 1e6,
             (a_bytes + b_bytes + c_bytes) / kus / 1e3), flush=True)
    return kus


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


def decode(S, prompt_len, n_new):
    """Batched greedy decoding of the 33.49M-parameter decoder with a KV cache (random bf16 weights)."""
    import numpy as np
    from .decode import Decoder
    V, D, H, L, F = 31769, 384, 6, 12, 1024
    dec = Decoder(V, D, H, L, F, S, prompt_len + n_new + 1)
    rng = np.random.default_rng(3)
    dec.upload((rng.standard_normal(dec.total) * 0.02).astype(np.float32))
    w = 1.0 / np.arange(1, V + 1, dtype=np.float64) ** 1.1
    cdf = np.cumsum(w / w.sum())
    prompts = np.minimum(np.searchsorted(cdf, rng.random((S, prompt_len))), V - 1).astype(np.uint32)
    st = torch.cuda.ExternalStream(dec.stream_ptr())
    dec.prefill(prompts)
    dec.generate(3)                      # eager step, capture, first replay
    dec.tokens(4)
    e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    with torch.cuda.stream(st):
        e[0].record()
        dec.prefill(prompts)
        e[1].record()
        dec.generate(n_new - 1)
        e[2].record()
    toks = dec.tokens(n_new)
    pre_ms = e[0].elapsed_time(e[1])
    gen_ms = e[1].elapsed_time(e[2])
    step_us = gen_ms * 1e3 / (n_new - 1)
    weight_mb = 2.0 * (12 * 1769472 + 12199296) / 1e6
    print("decode S=%d prompt=%d new=%d: prefill %.2f ms (%.0f tokens/s), %.1f us per step = %.0f tokens/s, "
          "weights streamed at %.0f GB/s; first tokens %s"
          % (S, prompt_len, n_new, pre_ms, S * prompt_len / pre_ms * 1e3, step_us, S / step_us * 1e6,
             weight_mb / step_us * 1e3, toks[0, :4].tolist()), flush=True)
    dec.destroy()
    return pre_ms, step_us


def lmhead(S, V=31769, K=384, iters=40, copies=8):
    """Decode-time LM head [S, K] x [V, K]^T with fused argmax.  `copies` tables are used in turn so
    that every launch streams its table from HBM (8 x 24.4 MB is larger than the 126 MB L2)."""
    lib.init(0)
    X = torch.randn(S, K, device="cuda").to(torch.bfloat16)
    Es = [(torch.randn(V, K, device="cuda") * 0.02).to(torch.bfloat16) for _ in range(copies)]
    tok = torch.zeros(S, device="cuda", dtype=torch.int32)
    for i in range(copies):
        lib.lmhead_argmax_bf16(X, Es[i], tok)
    lib.sync_check()
    want = (X.float() @ Es[copies - 1].float().t()).argmax(1).to(torch.int32)
    agree = int((want == tok).sum())
    # back to back on one stream: the next launch's prologue overlaps this launch's tail, as in a decode step
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(iters):
        lib.lmhead_argmax_bf16(X, Es[i % copies], tok)
    e1.record()
    torch.cuda.synchronize()
    us = e0.elapsed_time(e1) * 1e3 / iters
    lib.profile_begin()
    for i in range(iters):
        lib.lmhead_argmax_bf16(X, Es[i % copies], tok)
    prof = lib.profile_end(torch.cuda.current_stream().cuda_stream)
    kus = prof["lmhead_argmax"]["ms"] * 1e3 / iters
    nbytes = 2.0 * V * K + 2.0 * S * K
    gus = graph_time_us(lambda i: lib.lmhead_argmax_bf16(X, Es[i % copies], tok), iters)
    sus = graph_time_us(lambda i: lib.lmhead_argmax_bf16(X, Es[i % copies], tok, table_is_stable=True), iters)
    print("lmhead S=%d V=%d K=%d: in a CUDA graph %.2f us per call = %.0f GB/s of table+input bytes "
          "(%.2f us = %.0f GB/s when the table may be read before the previous kernel ends); eager %.2f us per call, "
          "events around each launch %.2f us; tokens agree with torch on %d of %d"
          % (S, V, K, gus, nbytes / gus / 1e3, sus, nbytes / sus / 1e3, us, kus, agree, S), flush=True)
    return gus


def main(argv):
    if len(argv) >= 5 and argv[0] == "gemm":
        M, N, K, kind = (int(x) for x in argv[1:5])
        iters = int(argv[5]) if len(argv) > 5 else 20
        out = argv[6] if len(argv) > 6 else "f32"
        tile_n = int(argv[7]) if len(argv) > 7 else 0
        splits = int(argv[8]) if len(argv) > 8 else 1
        gemm(M, N, K, kind, iters, out, tile_n, splits)
    elif len(argv) >= 2 and argv[0] == "lmhead":
        lmhead(*(int(x) for x in argv[1:6]))
    elif len(argv) >= 4 and argv[0] == "decode":
        decode(int(argv[1]), int(argv[2]), int(argv[3]))
    elif len(argv) >= 5 and argv[0] == "attention":
        B, H, T, hd = (int(x) for x in argv[1:5])
        attention(B, H, T, hd, int(argv[5]) if len(argv) > 5 else 10)
    else:
        print(__doc__)
        return 2
    return 0


if __name__ == "__main__":
    sys.exit(main(sys.argv[1:]))
