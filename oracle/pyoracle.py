"""TEST INFRASTRUCTURE ONLY: ctypes bindings for the two CPU checkers.

* ``Oracle``  -> oracle/liboracle.so, this repository's plain-C restatement (oracle.c).
* ``Ref``     -> oracle/_ref/libref.so, the reference's own CPU sources compiled
  unmodified plus the forwarding shim ref_shim.c (present only where it was built;
  the built library travels to the GPU machine, the reference sources do not).

Only tests/, the smoke check and bench.py's CPU legs import this module.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(HERE, "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "libref.so")

FP32, BF16, TF32 = 0, 1, 2

_f32p = C.POINTER(C.c_float)
_u32p = C.POINTER(C.c_uint32)
_f64p = C.POINTER(C.c_double)


def _fp(a):
    return None if a is None else a.ctypes.data_as(_f32p)


def _up(a):
    return a.ctypes.data_as(_u32p)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def build_oracle(force=False):
    """Compile liboracle.so (gcc, a second or two)."""
    src = os.path.join(HERE, "oracle.c")
    if force or not os.path.exists(ORACLE_SO) or os.path.getmtime(ORACLE_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", HERE, "oracle"], stdout=subprocess.DEVNULL)
    return ORACLE_SO


def build_ref(ref_root):
    """Compile the reference's CPU sources where they lie into oracle/_ref/libref.so."""
    subprocess.check_call(["make", "-C", HERE, "ref", "REF=" + ref_root], stdout=subprocess.DEVNULL,
                          stderr=subprocess.DEVNULL)
    return REF_SO


def build_ref_gpu(ref_root):
    """Compile the reference's GPU-resident trainer where it lies into oracle/_ref/librefgpu.so, and its
    cuda/train_kernels.cu into oracle/_ref/train_kernels.cubin (sm_100a); used on a GPU box only."""
    subprocess.check_call(["make", "-C", HERE, "refgpu", "refgpu_tb", "REF=" + ref_root], stdout=subprocess.DEVNULL,
                          stderr=subprocess.DEVNULL)


class ModelCfg(C.Structure):
    _fields_ = [("V", C.c_int), ("D", C.c_int), ("H", C.c_int), ("L", C.c_int),
                ("F", C.c_int), ("T", C.c_int), ("B", C.c_int), ("eps", C.c_float)]


class Oracle:
    def __init__(self):
        build_oracle()
        L = self.lib = C.CDLL(ORACLE_SO)
        L.orc_bf16_round.restype = C.c_float
        L.orc_bf16_round.argtypes = [C.c_float]
        L.orc_tf32_trunc.restype = C.c_float
        L.orc_tf32_trunc.argtypes = [C.c_float]
        L.orc_round_array.argtypes = [_f32p, _f32p, C.c_int64, C.c_int]
        L.orc_gemm.argtypes = [C.c_int, C.c_int, _f32p, _f32p, _f32p] + [C.c_int] * 6 + \
            [C.c_int, C.c_int64, C.c_int64, C.c_int64, C.c_float, C.c_float, C.c_int]
        L.orc_gemm_f64.argtypes = [C.c_int, C.c_int, _f32p, _f32p, _f64p] + [C.c_int] * 6
        L.orc_gemm_bias.argtypes = [_f32p] * 5 + [C.c_int] * 4
        L.orc_colsum_acc.argtypes = [_f32p, _f32p, C.c_int, C.c_int]
        L.orc_rmsnorm_fwd.argtypes = [_f32p] * 4 + [C.c_int, C.c_int, C.c_float]
        L.orc_rmsnorm_bwd.argtypes = [_f32p] * 6 + [C.c_int, C.c_int]
        L.orc_rope_tables.argtypes = [C.c_int, C.c_int, C.c_float, _f32p, _f32p]
        L.orc_qkv_rope_split.argtypes = [_f32p] * 6 + [C.c_int] * 4
        L.orc_qkv_rope_merge_bwd.argtypes = [_f32p] * 6 + [C.c_int] * 4
        L.orc_attention_fwd.argtypes = [_f32p] * 5 + [C.c_int] * 3 + [C.c_float, C.c_int]
        L.orc_attention_bwd.argtypes = [_f32p] * 7 + [C.c_int] * 3 + [C.c_float, C.c_int]
        L.orc_heads_merge.argtypes = [_f32p, _f32p] + [C.c_int] * 4
        L.orc_heads_split.argtypes = [_f32p, _f32p] + [C.c_int] * 4
        L.orc_swiglu_fwd.argtypes = [_f32p, _f32p, C.c_int, C.c_int]
        L.orc_swiglu_bwd.argtypes = [_f32p, _f32p, _f32p, C.c_int, C.c_int]
        L.orc_embed_fwd.argtypes = [_f32p, _u32p, _f32p, C.c_int, C.c_int]
        L.orc_embed_bwd.argtypes = [_f32p, _u32p, _f32p, C.c_int, C.c_int]
        L.orc_cross_entropy.argtypes = [_f32p, _u32p, _f32p, C.c_int, C.c_int, C.c_int, C.c_float]
        L.orc_adam.argtypes = [_f32p] * 4 + [C.c_int64] + [C.c_float] * 7
        L.orc_grad_norm.restype = C.c_double
        L.orc_grad_norm.argtypes = [_f32p, C.c_int64]
        L.orc_model_total_scalars.restype = C.c_int64
        L.orc_model_total_scalars.argtypes = [C.POINTER(ModelCfg)]
        L.orc_model_forward_backward.restype = C.c_float
        L.orc_model_forward_backward.argtypes = [C.POINTER(ModelCfg), _f32p, _u32p, _u32p, _f32p, _f32p,
                                                 C.c_int, C.c_int]
        L.orc_set_num_threads.argtypes = [C.c_int]
        L.orc_num_threads.restype = C.c_int

    def set_threads(self, n):
        self.lib.orc_set_num_threads(int(n))

    def round(self, a, mode):
        a = _f32(a)
        out = np.empty_like(a)
        self.lib.orc_round_array(_fp(a), _fp(out), a.size, mode)
        return out

    def gemm(self, ta, tb, A, B, M, N, K, lda=None, ldb=None, ldc=None, batch=1, sA=0, sB=0, sC=0,
             alpha=1.0, beta=0.0, C_in=None, mode=FP32):
        """A, B: flat float32 buffers holding the stored matrices (any leading dims)."""
        A = _f32(A)
        B = _f32(B)
        lda = lda if lda is not None else (M if ta else K)
        ldb = ldb if ldb is not None else (K if tb else N)
        ldc = ldc if ldc is not None else N
        if C_in is None:
            size = (batch - 1) * sC + M * ldc if batch > 1 else M * ldc
            Cb = np.zeros(size, dtype=np.float32)
        else:
            Cb = _f32(C_in).copy().reshape(-1)
        self.lib.orc_gemm(ta, tb, _fp(A), _fp(B), _fp(Cb), M, N, K, lda, ldb, ldc, batch, sA, sB, sC,
                          alpha, beta, mode)
        return Cb

    def gemm_f64(self, ta, tb, A, B, M, N, K):
        A = _f32(A)
        B = _f32(B)
        out = np.zeros((M, N), dtype=np.float64)
        self.lib.orc_gemm_f64(ta, tb, _fp(A), _fp(B), out.ctypes.data_as(_f64p), M, N, K,
                              M if ta else K, K if tb else N, N)
        return out

    def gemm_bias(self, A, B, bias, residual, mode=FP32):
        A = _f32(A)
        B = _f32(B)
        M, K = A.shape
        N = B.shape[1]
        out = np.zeros((M, N), dtype=np.float32)
        bias = None if bias is None else _f32(bias)
        residual = None if residual is None else _f32(residual)
        self.lib.orc_gemm_bias(_fp(A), _fp(B), _fp(bias), _fp(residual), _fp(out), M, N, K, mode)
        return out

    def rope_tables(self, T, hd, base=10000.0):
        c = np.zeros((T, hd // 2), dtype=np.float32)
        s = np.zeros((T, hd // 2), dtype=np.float32)
        self.lib.orc_rope_tables(T, hd, base, _fp(c), _fp(s))
        return c, s

    def qkv_rope_split(self, qkv, B, T, H, hd):
        qkv = _f32(qkv)
        c, s = self.rope_tables(T, hd)
        Q, K, V = (np.zeros((B * H, T, hd), dtype=np.float32) for _ in range(3))
        self.lib.orc_qkv_rope_split(_fp(qkv), _fp(c), _fp(s), _fp(Q), _fp(K), _fp(V), B, T, H, hd)
        return Q, K, V

    def qkv_rope_merge_bwd(self, dQ, dK, dV, B, T, H, hd):
        c, s = self.rope_tables(T, hd)
        out = np.zeros((B * T, 3 * H * hd), dtype=np.float32)
        self.lib.orc_qkv_rope_merge_bwd(_fp(_f32(dQ)), _fp(_f32(dK)), _fp(_f32(dV)), _fp(c), _fp(s), _fp(out),
                                        B, T, H, hd)
        return out

    def attention_fwd(self, Q, K, V, scale, mode=FP32, want_P=False):
        Q, K, V = _f32(Q), _f32(K), _f32(V)
        BH, T, hd = Q.shape
        O = np.zeros_like(Q)
        P = np.zeros((BH, T, T), dtype=np.float32) if want_P else None
        self.lib.orc_attention_fwd(_fp(Q), _fp(K), _fp(V), _fp(O), _fp(P), BH, T, hd, scale, mode)
        return (O, P) if want_P else O

    def attention_bwd(self, Q, K, V, dO, scale, mode=FP32):
        Q, K, V, dO = _f32(Q), _f32(K), _f32(V), _f32(dO)
        BH, T, hd = Q.shape
        dQ, dK, dV = np.zeros_like(Q), np.zeros_like(Q), np.zeros_like(Q)
        self.lib.orc_attention_bwd(_fp(Q), _fp(K), _fp(V), _fp(dO), _fp(dQ), _fp(dK), _fp(dV), BH, T, hd, scale, mode)
        return dQ, dK, dV

    def heads_merge(self, O, B, T, H, hd):
        O = _f32(O)
        out = np.zeros((B * T, H * hd), dtype=np.float32)
        self.lib.orc_heads_merge(_fp(O), _fp(out), B, T, H, hd)
        return out

    def heads_split(self, dout, B, T, H, hd):
        dout = _f32(dout)
        out = np.zeros((B * H, T, hd), dtype=np.float32)
        self.lib.orc_heads_split(_fp(dout), _fp(out), B, T, H, hd)
        return out

    def rmsnorm_fwd(self, x, w, eps):
        x, w = _f32(x), _f32(w)
        rows, cols = x.shape
        out = np.zeros_like(x)
        rinv = np.zeros(rows, dtype=np.float32)
        self.lib.orc_rmsnorm_fwd(_fp(x), _fp(w), _fp(out), _fp(rinv), rows, cols, eps)
        return out, rinv

    def rmsnorm_bwd(self, x, w, rinv, dy, dx_in=None, dw_in=None):
        x, w, rinv, dy = _f32(x), _f32(w), _f32(rinv), _f32(dy)
        rows, cols = x.shape
        dx = np.zeros_like(x) if dx_in is None else _f32(dx_in).copy()
        dw = np.zeros(cols, dtype=np.float32) if dw_in is None else _f32(dw_in).copy()
        self.lib.orc_rmsnorm_bwd(_fp(x), _fp(w), _fp(rinv), _fp(dy), _fp(dx), _fp(dw), rows, cols)
        return dx, dw

    def swiglu_fwd(self, gu):
        gu = _f32(gu)
        rows, F2 = gu.shape
        h = np.zeros((rows, F2 // 2), dtype=np.float32)
        self.lib.orc_swiglu_fwd(_fp(gu), _fp(h), rows, F2 // 2)
        return h

    def swiglu_bwd(self, gu, dh):
        gu, dh = _f32(gu), _f32(dh)
        rows, F2 = gu.shape
        dgu = np.zeros_like(gu)
        self.lib.orc_swiglu_bwd(_fp(gu), _fp(dh), _fp(dgu), rows, F2 // 2)
        return dgu

    def colsum_acc(self, x, out_in=None):
        x = _f32(x)
        out = np.zeros(x.shape[1], dtype=np.float32) if out_in is None else _f32(out_in).copy()
        self.lib.orc_colsum_acc(_fp(x), _fp(out), x.shape[0], x.shape[1])
        return out

    def cross_entropy(self, logits, targets, grad_scale):
        z = _f32(logits).copy()
        rows, V = z.shape
        t = np.ascontiguousarray(targets, dtype=np.uint32)
        loss = np.zeros(rows, dtype=np.float32)
        self.lib.orc_cross_entropy(_fp(z), _up(t), _fp(loss), rows, V, V, grad_scale)
        return loss, z

    def adam(self, p, g, m, v, lr, b1, b2, eps, bc1, bc2, grad_scale=1.0):
        p, m, v = _f32(p).copy(), _f32(m).copy(), _f32(v).copy()
        g = _f32(g)
        self.lib.orc_adam(_fp(p), _fp(g), _fp(m), _fp(v), p.size, lr, b1, b2, eps, bc1, bc2, grad_scale)
        return p, m, v

    def grad_norm(self, g):
        g = _f32(g)
        return float(self.lib.orc_grad_norm(_fp(g), g.size))

    def model_total_scalars(self, cfg):
        c = ModelCfg(*cfg)
        return int(self.lib.orc_model_total_scalars(C.byref(c)))

    def model_forward_backward(self, cfg, params, ids, targets, want_grads=True, want_logits=False,
                               mode=FP32, mode_dw=FP32):
        """cfg = (V, D, H, L, F, T, B, eps). Returns (loss, grads or None, logits or None)."""
        c = ModelCfg(*cfg)
        params = _f32(params)
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        targets = np.ascontiguousarray(targets, dtype=np.uint32)
        grads = np.zeros_like(params) if want_grads else None
        logits = np.zeros((c.B * c.T, c.V), dtype=np.float32) if want_logits else None
        loss = self.lib.orc_model_forward_backward(C.byref(c), _fp(params), _up(ids), _up(targets),
                                                   _fp(grads), _fp(logits), mode, mode_dw)
        return float(loss), grads, logits


class Ref:
    """The reference's own CPU code (unmodified sources), through ref_shim.c."""

    def __init__(self):
        if not os.path.exists(REF_SO):
            raise FileNotFoundError(REF_SO + " not built (make -C oracle ref REF=<reference checkout>)")
        L = self.lib = C.CDLL(REF_SO)
        u64, i64 = C.c_uint64, C.c_int64
        L.ref_gaussian_fill.argtypes = [_f32p, u64, u64, u64, C.c_double, C.c_double]
        L.ref_uniform_fill.argtypes = [_f64p, u64, u64, u64]
        L.ref_range_fill.argtypes = [_u32p, u64, u64, u64, i64, i64]
        L.ref_matmul2d.argtypes = [_f32p, u64, u64, i64, i64, _f32p, u64, i64, i64, _f32p]
        L.ref_matmul2d_fwd_bwd.argtypes = [_f32p, _f32p, _f32p, u64, u64, u64, _f32p, _f32p, _f32p]
        L.ref_rope_tables.argtypes = [u64, u64, C.c_float, _f32p, _f32p]
        for n in ("ref_sqrtf", "ref_expf"):
            getattr(L, n).restype = C.c_float
            getattr(L, n).argtypes = [C.c_float]
        L.ref_powf.restype = C.c_float
        L.ref_powf.argtypes = [C.c_float, C.c_float]
        L.ref_sqrt.restype = C.c_double
        L.ref_sqrt.argtypes = [C.c_double]
        L.ref_lm_create.restype = C.c_void_p
        L.ref_lm_create.argtypes = [C.c_uint32] * 5 + [C.c_float, u64, u64, u64]
        L.ref_lm_destroy.argtypes = [C.c_void_p]
        L.ref_lm_num_params.restype = C.c_uint32
        L.ref_lm_num_params.argtypes = [C.c_void_p]
        L.ref_lm_param_numel.restype = u64
        L.ref_lm_param_numel.argtypes = [C.c_void_p, C.c_uint32]
        L.ref_lm_total_scalars.restype = u64
        L.ref_lm_total_scalars.argtypes = [C.c_void_p]
        L.ref_lm_get.argtypes = [C.c_void_p, C.c_int, _f32p]
        L.ref_lm_set.argtypes = [C.c_void_p, C.c_int, _f32p]
        L.ref_lm_dp_step.restype = C.c_float
        L.ref_lm_dp_step.argtypes = [C.c_void_p, _u32p, u64, u64, C.c_uint32, u64, u64]
        L.ref_sample_batch.argtypes = [_u32p, u64, C.c_uint32, C.c_uint32, u64, _u32p, _u32p]
        L.ref_lm_adam_step.argtypes = [C.c_void_p, C.c_float]
        L.ref_lm_adam_t.restype = u64
        L.ref_lm_adam_t.argtypes = [C.c_void_p]
        L.ref_lm_set_adam_t.argtypes = [C.c_void_p, u64]
        L.ref_lm_checkpoint_save.restype = C.c_int
        L.ref_lm_checkpoint_save.argtypes = [C.c_void_p, C.c_char_p, C.c_int]
        L.ref_lm_checkpoint_load.restype = C.c_int
        L.ref_lm_checkpoint_load.argtypes = [C.c_void_p, C.c_char_p, C.c_int]
        L.ref_lr_warmup_cosine.restype = C.c_float
        L.ref_lr_warmup_cosine.argtypes = [u64, u64, u64, C.c_float, C.c_float]
        L.ref_lm_forward_logits.argtypes = [C.c_void_p, _u32p, C.c_uint32, u64, _f32p, u64]
        L.ref_attention_fwd_bwd.argtypes = [_f32p] * 6 + [C.c_uint32, u64, C.c_uint32, C.c_uint32] + [_f32p] * 6 + [u64]
        L.ref_ffn_fwd_bwd.argtypes = [_f32p] * 6 + [u64, C.c_uint32, C.c_uint32] + [_f32p] * 6 + [u64]

    def gaussian(self, n, seed, seq=1, mean=0.0, std=1.0):
        out = np.zeros(n, dtype=np.float32)
        self.lib.ref_gaussian_fill(_fp(out), n, seed, seq, mean, std)
        return out

    def uniform(self, n, seed, seq=1):
        out = np.zeros(n, dtype=np.float64)
        self.lib.ref_uniform_fill(out.ctypes.data_as(_f64p), n, seed, seq)
        return out

    def range_u32(self, n, seed, seq, lo, hi):
        out = np.zeros(n, dtype=np.uint32)
        self.lib.ref_range_fill(_up(out), n, seed, seq, lo, hi)
        return out

    def matmul2d(self, A, B):
        """A, B: 2-D float32 numpy arrays, possibly transposed views (strides honoured)."""
        assert A.dtype == np.float32 and B.dtype == np.float32
        M, K = A.shape
        N = B.shape[1]
        out = np.zeros((M, N), dtype=np.float32)
        sa = [s // 4 for s in A.strides]
        sb = [s // 4 for s in B.strides]
        self.lib.ref_matmul2d(A.ctypes.data_as(_f32p), M, K, sa[0], sa[1],
                              B.ctypes.data_as(_f32p), N, sb[0], sb[1], _fp(out))
        return out

    def matmul2d_fwd_bwd(self, A, B, dC):
        A, B, dC = _f32(A), _f32(B), _f32(dC)
        M, K = A.shape
        N = B.shape[1]
        Cc, dA, dB = np.zeros((M, N), np.float32), np.zeros((M, K), np.float32), np.zeros((K, N), np.float32)
        self.lib.ref_matmul2d_fwd_bwd(_fp(A), _fp(B), _fp(dC), M, K, N, _fp(Cc), _fp(dA), _fp(dB))
        return Cc, dA, dB

    def rope_tables(self, T, hd, base=10000.0):
        c = np.zeros((T, hd // 2), dtype=np.float32)
        s = np.zeros((T, hd // 2), dtype=np.float32)
        self.lib.ref_rope_tables(T, hd, base, _fp(c), _fp(s))
        return c, s

    def attention_fwd_bwd(self, x, w_qkv, b_qkv, wo, bo, dout, B, T, H, arena=2 << 30):
        x, w_qkv, b_qkv, wo, bo, dout = map(_f32, (x, w_qkv, b_qkv, wo, bo, dout))
        D = x.shape[1]
        out, dx = np.zeros_like(x), np.zeros_like(x)
        dw, db, dwo, dbo = np.zeros_like(w_qkv), np.zeros_like(b_qkv), np.zeros_like(wo), np.zeros_like(bo)
        self.lib.ref_attention_fwd_bwd(_fp(x), _fp(w_qkv), _fp(b_qkv), _fp(wo), _fp(bo), _fp(dout), B, T, H, D,
                                       _fp(out), _fp(dx), _fp(dw), _fp(db), _fp(dwo), _fp(dbo), arena)
        return out, dx, dw, db, dwo, dbo

    def ffn_fwd_bwd(self, x, w_gu, b_gu, w_down, b_down, dout, arena=2 << 30):
        x, w_gu, b_gu, w_down, b_down, dout = map(_f32, (x, w_gu, b_gu, w_down, b_down, dout))
        N, D = x.shape
        F = w_down.shape[0]
        out, dx = np.zeros_like(x), np.zeros_like(x)
        dwg, dbg, dwd, dbd = np.zeros_like(w_gu), np.zeros_like(b_gu), np.zeros_like(w_down), np.zeros_like(b_down)
        self.lib.ref_ffn_fwd_bwd(_fp(x), _fp(w_gu), _fp(b_gu), _fp(w_down), _fp(b_down), _fp(dout), N, D, F,
                                 _fp(out), _fp(dx), _fp(dwg), _fp(dbg), _fp(dwd), _fp(dbd), arena)
        return out, dx, dwg, dbg, dwd, dbd

    def lr_warmup_cosine(self, step, warmup, total, peak, min_lr):
        return float(self.lib.ref_lr_warmup_cosine(step, warmup, total, peak, min_lr))

    def sample_batch(self, tokens, T, B, seed_base):
        tokens = np.ascontiguousarray(tokens, dtype=np.uint32)
        ids = np.zeros(B * T, dtype=np.uint32)
        tgt = np.zeros(B * T, dtype=np.uint32)
        self.lib.ref_sample_batch(_up(tokens), tokens.size, T, B, seed_base, _up(ids), _up(tgt))
        return ids, tgt


class RefLM:
    """lm_init + data_parallel_step + adam_step of the reference, CPU only."""

    def __init__(self, ref, V, D, H, L, F, eps=1e-5, seed=1337, seq=1, arena=4 << 30):
        self.ref = ref
        self.h = ref.lib.ref_lm_create(V, D, H, L, F, eps, seed, seq, arena)
        self.cfg = (V, D, H, L, F)
        self.total = int(ref.lib.ref_lm_total_scalars(self.h))

    def close(self):
        if self.h:
            self.ref.lib.ref_lm_destroy(self.h)
            self.h = None

    def get(self, which):
        out = np.zeros(self.total, dtype=np.float32)
        self.ref.lib.ref_lm_get(self.h, which, _fp(out))
        return out

    def set(self, which, flat):
        flat = _f32(flat)
        assert flat.size == self.total
        self.ref.lib.ref_lm_set(self.h, which, _fp(flat))

    def params(self):
        return self.get(0)

    def grads(self):
        return self.get(1)

    def param_numels(self):
        n = self.ref.lib.ref_lm_num_params(self.h)
        return [int(self.ref.lib.ref_lm_param_numel(self.h, i)) for i in range(n)]

    def dp_step(self, tokens, T, workers, seed_base, step_arena=1536 << 20):
        tokens = np.ascontiguousarray(tokens, dtype=np.uint32)
        return float(self.ref.lib.ref_lm_dp_step(self.h, _up(tokens), tokens.size, T, workers, seed_base, step_arena))

    def adam_step(self, lr):
        self.ref.lib.ref_lm_adam_step(self.h, lr)

    def adam_t(self):
        return int(self.ref.lib.ref_lm_adam_t(self.h))

    def set_adam_t(self, t):
        self.ref.lib.ref_lm_set_adam_t(self.h, t)

    def checkpoint_save(self, path, with_opt):
        return bool(self.ref.lib.ref_lm_checkpoint_save(self.h, str(path).encode(), int(with_opt)))

    def checkpoint_load(self, path, with_opt):
        return bool(self.ref.lib.ref_lm_checkpoint_load(self.h, str(path).encode(), int(with_opt)))

    def forward_logits(self, ids, B, T, arena=4 << 30):
        ids = np.ascontiguousarray(ids, dtype=np.uint32)
        V = self.cfg[0]
        out = np.zeros((B * T, V), dtype=np.float32)
        self.ref.lib.ref_lm_forward_logits(self.h, _up(ids), B, T, _fp(out), arena)
        return out
