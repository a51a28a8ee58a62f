"""TEST INFRASTRUCTURE ONLY -- the reference's own GPU-resident trainer as a checker.

ctypes binding of oracle/_ref/librefgpu.so (the reference's unmodified model/gpu_train.c,
cuda/cuda_backend.c and CPU sources, built by `make -C oracle refgpu`) together with
oracle/_ref/train_kernels.cubin (the reference's cuda/train_kernels.cu compiled for sm_100a).

The reference creates and switches to a CUDA context of its own on every call, so this module is
run as a CHILD PROCESS (`python -m oracle.ref_gpu <command> ...`) that touches no other CUDA state;
`run_child` is the helper the tests use.  Commands:

  trajectory  the training loop of training/train_lm_gpu.c:212-223 from given start weights over a
              given token stream; writes losses, gradient norms and seconds per step
  step        one forward+backward from given weights on a given batch; writes loss, norm, gradients
  gemms       times the reference's GEMM kernels alone on the layer shapes of one training step
  abi_in_context  the product library's tb_gemm_bias_f32 called inside the reference's own CUDA context
  gemm        one GEMM launch of a named kernel of any module image through the reference's loader
              (cuda_init / cuda_get_kernel / cuda_launch): inputs from an .npz, output to an .npy

--module selects the module image the reference's loader reads (default: the reference's own kernels; the
drop-in tests pass oracle/_ref/train_kernels_tb_gemm.cubin or turkce_llm_b200/turkce_b200_gemm.cubin).
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
REFGPU_SO = os.path.join(HERE, "_ref", "librefgpu.so")
REFGPU_CUBIN = os.path.join(HERE, "_ref", "train_kernels.cubin")
# the reference's non-GEMM kernels + this library's GEMM entries under the reference's names, in one module
REFGPU_TB_CUBIN = os.path.join(HERE, "_ref", "train_kernels_tb_gemm.cubin")


def available():
    return os.path.exists(REFGPU_SO) and os.path.exists(REFGPU_CUBIN)


def _ptr(a, t):
    return a.ctypes.data_as(C.POINTER(t))


class RefGpu:
    """gpu_trainer_* of the reference (model/gpu_train.h:86-125) behind oracle/ref_gpu_shim.c."""

    def __init__(self, V, D, H, L, F, T, B, eps=1e-5, seed=1337, seq=1, arena_bytes=None, module=None):
        self.lib = lib = C.CDLL(REFGPU_SO)
        lib.refgpu_create.restype = C.c_void_p
        lib.refgpu_create.argtypes = [C.c_uint32] * 5 + [C.c_float, C.c_uint64, C.c_uint64, C.c_uint32, C.c_uint32,
                                                         C.c_char_p, C.c_uint64]
        lib.refgpu_total_scalars.restype = C.c_uint64
        lib.refgpu_total_scalars.argtypes = [C.c_void_p]
        lib.refgpu_set.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_float)]
        lib.refgpu_get.argtypes = [C.c_void_p, C.c_int, C.POINTER(C.c_float)]
        lib.refgpu_forward_backward.restype = C.c_float
        lib.refgpu_forward_backward.argtypes = [C.c_void_p, C.POINTER(C.c_uint32), C.POINTER(C.c_uint32)]
        lib.refgpu_grad_norm.restype = C.c_double
        lib.refgpu_grad_norm.argtypes = [C.c_void_p]
        lib.refgpu_adam_scaled.argtypes = [C.c_void_p, C.c_float, C.c_float]
        lib.refgpu_train_loop.restype = C.c_double
        lib.refgpu_train_loop.argtypes = [C.c_void_p, C.POINTER(C.c_uint32), C.c_uint64, C.c_uint32, C.c_uint32,
                                          C.c_uint32, C.c_uint32, C.c_float, C.c_float, C.c_float,
                                          C.POINTER(C.c_float), C.POINTER(C.c_double)]
        lib.refgpu_time_gemm_bias.restype = C.c_double
        lib.refgpu_time_gemm_bias.argtypes = [C.c_void_p, C.c_int32, C.c_int32, C.c_int32, C.c_int, C.c_int]
        lib.refgpu_time_gemm.restype = C.c_double
        lib.refgpu_time_gemm.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int32, C.c_int32, C.c_int32, C.c_uint32,
                                         C.c_int]
        lib.refgpu_destroy.argtypes = [C.c_void_p]
        total = V * D + L * (D + D * 3 * D + 3 * D + D * D + D + D + D * 2 * F + 2 * F + F * D + D) + D
        if arena_bytes is None:
            # values + grads + adam m, v on the host mirror, loss rows, tables, slack
            arena_bytes = 4 * 4 * total + 64 * B * T + (64 << 20)
        self.h = lib.refgpu_create(V, D, H, L, F, eps, seed, seq, B, T, (module or REFGPU_CUBIN).encode(), arena_bytes)
        self.total = int(lib.refgpu_total_scalars(self.h))
        assert self.total == total
        self.B, self.T = B, T

    def set(self, which, flat):
        flat = np.ascontiguousarray(flat, dtype=np.float32)
        assert flat.size == self.total
        self.lib.refgpu_set(self.h, which, _ptr(flat, C.c_float))

    def get(self, which):
        out = np.empty(self.total, dtype=np.float32)
        self.lib.refgpu_get(self.h, which, _ptr(out, C.c_float))
        return out

    def forward_backward(self, ids, tgt):
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        tgt = np.ascontiguousarray(tgt, dtype=np.uint32)
        return float(self.lib.refgpu_forward_backward(self.h, _ptr(ids, C.c_uint32), _ptr(tgt, C.c_uint32)))

    def grad_norm(self):
        return float(self.lib.refgpu_grad_norm(self.h))

    def train_loop(self, tokens, step0, steps, warmup, total_steps, peak_lr, min_lr, clip):
        tokens = np.ascontiguousarray(tokens, dtype=np.uint32)
        losses = np.empty(steps, dtype=np.float32)
        norms = np.empty(steps, dtype=np.float64)
        sec = self.lib.refgpu_train_loop(self.h, _ptr(tokens, C.c_uint32), tokens.size, step0, steps, warmup,
                                         total_steps, peak_lr, min_lr, clip, _ptr(losses, C.c_float),
                                         _ptr(norms, C.c_double))
        return losses, norms, float(sec)

    def time_gemm_bias(self, M, N, K, residual, iters):
        return float(self.lib.refgpu_time_gemm_bias(self.h, M, N, K, int(residual), iters))

    def time_gemm(self, kind, fp32_kernel, M, N, K, batch, iters):
        return float(self.lib.refgpu_time_gemm(self.h, kind, int(fp32_kernel), M, N, K, batch, iters))

    def destroy(self):
        if self.h:
            self.lib.refgpu_destroy(self.h)
            self.h = None


def cmd_trajectory(a):
    V, D, H, L, F, T, B = a.cfg
    r = RefGpu(V, D, H, L, F, T, B, a.eps, module=a.module)
    if a.params:
        r.set(0, np.load(a.params))
    tokens = np.load(a.tokens)
    losses, norms, sec = r.train_loop(tokens, 0, a.steps, a.warmup, a.total_steps, a.peak_lr, a.min_lr, a.clip)
    out = {"losses": [float(x) for x in losses], "norms": [float(x) for x in norms], "seconds": sec,
           "seconds_per_step": sec / a.steps, "tokens_per_s": a.steps * B * T / sec}
    r.destroy()
    with open(a.out, "w") as f:
        json.dump(out, f)


def cmd_step(a):
    """One gpu_trainer_forward_backward from given weights on given ids/targets (an .npz with `ids`, `tgt`);
    writes the loss and gradient norm to --out and the flat gradients to --grads-out (.npy)."""
    V, D, H, L, F, T, B = a.cfg
    r = RefGpu(V, D, H, L, F, T, B, a.eps, module=a.module)
    r.set(0, np.load(a.params))
    batch = np.load(a.tokens)
    loss = r.forward_backward(batch["ids"], batch["tgt"])
    norm = r.grad_norm()
    np.save(a.grads_out, r.get(1))
    r.destroy()
    with open(a.out, "w") as f:
        json.dump({"loss": loss, "grad_norm": norm}, f)


def cmd_gemms(a):
    """The reference's GEMM kernels alone on the shapes of one training step at B*T = a.tokens."""
    V, D, H, L, F, T, B = a.cfg
    N = B * T
    r = RefGpu(V, D, H, 1, F, T, B, a.eps, module=a.module)   # one layer: the shapes do not depend on depth
    rows = []

    def add(name, sec, M, Nn, K, batch=1):
        rows.append({"kernel": name, "M": M, "N": Nn, "K": K, "batch": batch, "us": sec * 1e6,
                     "tflops": 2.0 * M * Nn * K * batch / sec / 1e12})

    it = a.iters
    # forward projections: bf16_gemm_bias call sites model/gpu_train.c:338,361,364,370
    add("k_bf16_gemm_nn_bias qkv", r.time_gemm_bias(N, 3 * D, D, 0, it), N, 3 * D, D)
    add("k_bf16_gemm_nn_bias out+res", r.time_gemm_bias(N, D, D, 1, it), N, D, D)
    add("k_bf16_gemm_nn_bias gate|up", r.time_gemm_bias(N, 2 * F, D, 0, it), N, 2 * F, D)
    add("k_bf16_gemm_nn_bias down+res", r.time_gemm_bias(N, D, F, 1, it), N, D, F)
    # input gradients dX = dY . W^T (NT), model/gpu_train.c:419
    add("k_bf16_gemm_nt dX qkv", r.time_gemm(1, 0, N, D, 3 * D, 1, it), N, D, 3 * D)
    add("k_bf16_gemm_nt dX gate|up", r.time_gemm(1, 0, N, D, 2 * F, 1, it), N, D, 2 * F)
    add("k_bf16_gemm_nt dX down", r.time_gemm(1, 0, N, F, D, 1, it), N, F, D)
    # weight gradients dW = X^T . dY (TN, float32 SIMT kernel in the reference), model/gpu_train.c:417
    add("k_gemm_tn dW qkv", r.time_gemm(2, 1, D, 3 * D, N, 1, it), D, 3 * D, N)
    add("k_gemm_tn dW gate|up", r.time_gemm(2, 1, D, 2 * F, N, 1, it), D, 2 * F, N)
    add("k_gemm_tn dW down", r.time_gemm(2, 1, F, D, N, 1, it), F, D, N)
    # LM head logits = nf . E^T (NT), model/gpu_train.c:378
    add("k_bf16_gemm_nt lm head", r.time_gemm(1, 0, N, V, D, 1, max(2, it // 4)), N, V, D)
    # attention scores, one launch over B*H heads: Q . K^T, model/gpu_train.c:343-347
    add("k_bf16_gemm_nt QK^T batched", r.time_gemm(1, 0, T, T, D // H, B * H, it), T, T, D // H, B * H)
    add("k_bf16_gemm_nn P.V batched", r.time_gemm(0, 0, T, D // H, T, B * H, it), T, D // H, T, B * H)
    r.destroy()
    with open(a.out, "w") as f:
        json.dump({"tokens": N, "rows": rows}, f)


def cmd_gemm(a):
    """--tokens: an .npz with entry (str), form, A, B, C, optional bias / residual, and the integers M, N, K, lda,
    ldb, ldc, sA, sB, sC, gx, gy, gz, bx, by, iters and floats alpha, beta.  Writes the result matrix to --out (.npy)
    and, next to it, <out>.json with the seconds per launch."""
    z = np.load(a.tokens, allow_pickle=False)
    lib = C.CDLL(REFGPU_SO)
    f32p = C.POINTER(C.c_float)
    lib.refcuda_gemm.restype = C.c_double
    lib.refcuda_gemm.argtypes = [C.c_char_p, C.c_char_p, C.c_int, f32p, C.c_uint64, f32p, C.c_uint64, f32p, f32p, f32p,
                                 C.c_uint64] + [C.c_int32] * 6 + [C.c_int64] * 3 + [C.c_float] * 2 + [C.c_uint32] * 5 + [C.c_int]
    A = np.ascontiguousarray(z["A"], dtype=np.float32).reshape(-1)
    B = np.ascontiguousarray(z["B"], dtype=np.float32).reshape(-1)
    Cm = np.ascontiguousarray(z["C"], dtype=np.float32).reshape(-1).copy()
    bias = np.ascontiguousarray(z["bias"], dtype=np.float32) if "bias" in z else None
    res = np.ascontiguousarray(z["residual"], dtype=np.float32).reshape(-1) if "residual" in z else None
    i = lambda k: int(z[k])
    sec = lib.refcuda_gemm((a.module or REFGPU_CUBIN).encode(), str(z["entry"]).encode(), i("form"),
                           _ptr(A, C.c_float), A.size, _ptr(B, C.c_float), B.size,
                           _ptr(bias, C.c_float) if bias is not None else None,
                           _ptr(res, C.c_float) if res is not None else None, _ptr(Cm, C.c_float), Cm.size,
                           i("M"), i("N"), i("K"), i("lda"), i("ldb"), i("ldc"), i("sA"), i("sB"), i("sC"),
                           float(z["alpha"]), float(z["beta"]), i("gx"), i("gy"), i("gz"), i("bx"), i("by"), i("iters"))
    np.save(a.out, Cm)
    with open(a.out + ".json", "w") as f:
        json.dump({"seconds_per_launch": float(sec)}, f)


def cmd_abi_in_context(a):
    """tb_gemm_bias_f32 of the product library called inside the context the reference's cuda_init created, on
    buffers from the reference's cuda_alloc.  --tokens: an .npz with A, B, bias, residual; --params: path of
    libturkce_b200.so.  Writes C to --out (.npy) and {"rc", "error"} to <out>.json."""
    z = np.load(a.tokens)
    lib = C.CDLL(REFGPU_SO)
    f32p = C.POINTER(C.c_float)
    lib.refcuda_call_tb_gemm_bias.restype = C.c_int
    lib.refcuda_call_tb_gemm_bias.argtypes = [C.c_char_p, C.c_char_p, f32p, f32p, f32p, f32p, f32p, C.c_int32, C.c_int32,
                                              C.c_int32, C.c_char_p, C.c_int]
    A, B = (np.ascontiguousarray(z[k], dtype=np.float32) for k in ("A", "B"))
    bias, res = (np.ascontiguousarray(z[k], dtype=np.float32) for k in ("bias", "residual"))
    M, K = A.shape
    N = B.shape[1]
    out = np.zeros((M, N), dtype=np.float32)
    err = C.create_string_buffer(1024)
    rc = lib.refcuda_call_tb_gemm_bias((a.module or REFGPU_CUBIN).encode(), a.params.encode(), _ptr(A, C.c_float),
                                       _ptr(B, C.c_float), _ptr(bias, C.c_float), _ptr(res, C.c_float), _ptr(out, C.c_float),
                                       M, N, K, err, len(err))
    np.save(a.out, out)
    with open(a.out + ".json", "w") as f:
        json.dump({"rc": int(rc), "error": err.value.decode("utf-8", "replace")}, f)


def run_child(args, timeout=1200):
    """Runs `python -m oracle.ref_gpu <args>` from the repository root; returns the completed process."""
    root = os.path.dirname(HERE)
    return subprocess.run([sys.executable, "-m", "oracle.ref_gpu"] + [str(x) for x in args], cwd=root,
                          capture_output=True, text=True, timeout=timeout)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("command", choices=["trajectory", "step", "gemms", "gemm", "abi_in_context"])
    ap.add_argument("--module", default=None, help="module image for the reference's loader (default: its own kernels)")
    ap.add_argument("--cfg", type=int, nargs=7, metavar=("V", "D", "H", "L", "F", "T", "B"),
                    default=[31769, 384, 6, 12, 1024, 1024, 8])
    ap.add_argument("--eps", type=float, default=1e-5)
    ap.add_argument("--params", default=None, help=".npy of the flat float32 start weights")
    ap.add_argument("--tokens", default=None, help=".npy of the uint32 token stream")
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=1000)
    ap.add_argument("--total-steps", type=int, default=70000)
    ap.add_argument("--peak-lr", type=float, default=6e-4)
    ap.add_argument("--min-lr", type=float, default=6e-5)
    ap.add_argument("--clip", type=float, default=1.0)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--grads-out", default=None, help=".npy to receive the flat gradients (step)")
    ap.add_argument("--out", required=True)
    a = ap.parse_args()
    if not available():
        raise SystemExit("oracle/_ref/librefgpu.so or train_kernels.cubin is not built (make -C oracle refgpu)")
    {"trajectory": cmd_trajectory, "step": cmd_step, "gemms": cmd_gemms, "gemm": cmd_gemm,
     "abi_in_context": cmd_abi_in_context}[a.command](a)


if __name__ == "__main__":
    main()
