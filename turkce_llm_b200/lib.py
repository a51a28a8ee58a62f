"""ctypes binding of the C ABI in include/turkce_b200.h.

There is no fallback: if libturkce_b200.so is missing or a call fails, an exception is raised.
"""
import ctypes as C
import os

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libturkce_b200.so")

NN, NT, TN = 0, 1, 2
PREC_BF16, PREC_TF32, PREC_FP32 = 0, 1, 2
CAUSAL_NONE, CAUSAL_SKIP_UPPER, CAUSAL_K_PREFIX, CAUSAL_K_SUFFIX = 0, 1, 2, 3

_vp, _i, _i64, _f = C.c_void_p, C.c_int, C.c_int64, C.c_float

# name -> (restype, argtypes); every symbol include/turkce_b200.h declares is listed here
SIGNATURES = {
    "tb_init": (_i, [_i]),
    "tb_device_count": (_i, []),
    "tb_last_error": (C.c_char_p, []),
    "tb_launch_count": (C.c_longlong, []),
    "tb_check": (_i, [_vp]),
    "tb_shutdown": (_i, []),
    "tb_profile_begin": (_i, []),
    "tb_profile_end": (_i, [_vp, C.c_char_p, _i]),
    "tb_alloc": (_i, [C.POINTER(_vp), C.c_uint64]),
    "tb_free": (_i, [_vp]),
    "tb_h2d": (_i, [_vp, _vp, C.c_uint64]),
    "tb_d2h": (_i, [_vp, _vp, C.c_uint64]),
    "tb_memset_zero": (_i, [_vp, C.c_uint64]),
    "tb_sync": (_i, []),
    "tb_gemm_f32": (_i, [_i, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i64, _i64, _i64, _f, _f, _i, _vp]),
    "tb_gemm_bias_f32": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp]),
    "tb_matmul_host": (_i, [_vp, _vp, _vp, _i, _i, _i, _i]),
    "tb_gemm_bf16": (_i, [_i, _vp, _vp, _i, _i, _i, _i64, _i64, _i, _i64, _i64,
                          _vp, _i64, _i64, _vp, _i64, _i64, _vp, _vp, _i64, _i64,
                          _f, _f, _i, _i, _i, _vp]),
    "tb_gemm_bf16_splitk_static": (_i, [_i, _vp, _vp, _i, _i, _i, _i64, _i64, _vp, _i64, _vp, _f, _f, _i, _i, _vp]),
    "tb_gemm_bf16_splitk_static_status": (_i, [_vp]),
    "tb_attention_fwd": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _vp]),
    "tb_attention_bwd": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _f, _vp]),
    "tb_pack_bf16": (_i, [_vp, _vp, _i, _i, _i64, _i64, _i, _i64, _i64, _vp]),
    "tb_gemm_swiglu_bf16": (_i, [_vp, _vp, _vp, _i, _i, _i, _vp, _vp, _vp]),
    "tb_gemm_qkv_rope_bf16": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp, _vp]),
    "tb_decode_linear": (_i, [_vp, _vp, _vp, _f, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp]),
    "tb_lmhead_argmax_bf16": (_i, [_vp, _vp, _i, _i, _i, _vp, _vp, _i64, _i, _vp]),
    "tb_decoder_create": (_i, [C.POINTER(_vp), _i, _i, _i, _i, _i, _i, _i, _f, _vp]),
    "tb_decoder_destroy": (_i, [_vp]),
    "tb_decoder_total_scalars": (_i64, [_vp]),
    "tb_decoder_upload": (_i, [_vp, _vp]),
    "tb_decoder_set_sampling": (_i, [_vp, _f, C.c_uint64, C.c_uint64]),
    "tb_decoder_prefill": (_i, [_vp, _vp, _i]),
    "tb_decoder_generate": (_i, [_vp, _i]),
    "tb_decoder_read_tokens": (_i, [_vp, _vp, _i]),
    "tb_decoder_read_logits": (_i, [_vp, _vp]),
    "tb_decoder_stream": (_vp, [_vp]),
    "tb_trainer_create": (_i, [C.POINTER(_vp), _i, _i, _i, _i, _i, _i, _i, _f, _vp]),
    "tb_trainer_create_prec": (_i, [C.POINTER(_vp), _i, _i, _i, _i, _i, _i, _i, _f, _i, _vp]),
    "tb_trainer_destroy": (_i, [_vp]),
    "tb_trainer_total_scalars": (_i64, [_vp]),
    "tb_trainer_num_params": (_i, [_vp]),
    "tb_trainer_param_layout": (_i, [_vp, _vp, _vp]),
    "tb_trainer_upload": (_i, [_vp, _i, _vp]),
    "tb_trainer_download": (_i, [_vp, _i, _vp]),
    "tb_trainer_device_ptr": (_vp, [_vp, _i]),
    "tb_trainer_stream": (_vp, [_vp]),
    "tb_trainer_forward_backward": (_i, [_vp, _vp, _vp, C.POINTER(_f)]),
    "tb_trainer_eval_loss": (_i, [_vp, _vp, _vp, C.POINTER(_f)]),
    "tb_trainer_grad_norm": (_i, [_vp, C.POINTER(C.c_double)]),
    "tb_trainer_adam_step_scaled": (_i, [_vp, C.c_uint64, _f, _f, _f, _f, _f]),
    "tb_trainer_train_step": (_i, [_vp, _vp, _vp, C.c_uint64, _f, _f, _f, _f, _f, C.POINTER(_f),
                                   C.POINTER(C.c_double)]),
    "tb_trainer_zero_grads": (_i, [_vp]),
    "tb_trainer_forward": (_i, [_vp, _vp, _vp, _i]),
    "tb_trainer_backward_head": (_i, [_vp]),
    "tb_trainer_backward_layer": (_i, [_vp, _i]),
    "tb_trainer_backward_embed": (_i, [_vp]),
    "tb_trainer_clip_adam_async": (_i, [_vp, C.c_uint64, _f, _f, _f, _f, _f, _f]),
    "tb_trainer_read_loss": (_i, [_vp, C.POINTER(_f)]),
    "tb_trainer_set_inputs": (_i, [_vp, _vp, _vp]),
    "tb_trainer_step_resident": (_i, [_vp, C.c_uint64, _f, _f, _f, _f, _f]),
    "tb_trainer_forward_resident": (_i, [_vp, _i]),
    "tb_trainer_last_norm": (_i, [_vp, C.POINTER(C.c_double)]),
    "tb_trainer_dims": (_i, [_vp] + [C.POINTER(_i)] * 7),
    "tb_sample_batch": (_i, [_vp, C.c_uint64, _i, _i, C.c_uint64, _vp, _vp]),
    "tb_sample_batch_range": (_i, [_vp, C.c_uint64, _i, _i, _i, C.c_uint64, _vp, _vp]),
    "tb_pcg_uniform_fill": (_i, [C.c_uint64, C.c_uint64, C.c_uint64, _vp]),
    "tb_lr_warmup_cosine": (_f, [C.c_uint64, C.c_uint64, C.c_uint64, _f, _f]),
    "tb_checkpoint_save": (_i, [C.c_char_p, _vp, _i, C.c_uint64]),
    "tb_checkpoint_load": (_i, [C.c_char_p, _vp, _i, C.POINTER(C.c_uint64)]),
    "tb_dp_unique_id": (_i, [_vp]),
    "tb_dp_create": (_i, [C.POINTER(_vp), _vp, _vp, _i, _i, _i]),
    "tb_dp_destroy": (_i, [_vp]),
    "tb_dp_slice": (_i, [_i64, _i, _i, C.POINTER(_i64), C.POINTER(_i64), C.POINTER(_i64)]),
    "tb_dp_info": (_i, [_vp] + [C.POINTER(_i)] * 4),
    "tb_dp_step": (_i, [_vp, _vp, _vp, _i, C.c_uint64, _f, _f, _f, _f, _f, C.POINTER(_f), C.POINTER(C.c_double)]),
    "tb_dp_step_resident": (_i, [_vp, C.c_uint64, _f, _f, _f, _f, _f]),
    "tb_dp_last_result": (_i, [_vp, C.POINTER(_f), C.POINTER(C.c_double)]),
    "tb_trainer_run": (_i, [_vp, _vp, C.c_uint64, C.c_uint32, C.c_uint32, C.c_uint32, C.c_uint32, _f, _f, _f,
                            _f, _f, _f, C.POINTER(C.c_uint64), _vp, _vp]),
}

_lib = None


class TbError(RuntimeError):
    pass


def load():
    """Loads the shared library (once) and declares every entry point."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise TbError("%s is missing: run `python -m turkce_llm_b200.build` (there is no CPU fallback)" % LIB_PATH)
        lib = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = res
            fn.argtypes = args
        _lib = lib
    return _lib


def check(rc):
    if rc != 0:
        raise TbError(load().tb_last_error().decode("utf-8", "replace"))


def _ptr(t):
    """Device/host pointer of a torch tensor or numpy array, or None."""
    if t is None:
        return None
    if hasattr(t, "data_ptr"):
        return t.data_ptr()
    return t.ctypes.data


def _stream():
    import torch
    return torch.cuda.current_stream().cuda_stream


def init(device=0):
    check(load().tb_init(int(device)))


def sync_check():
    """Waits for the current stream and raises if a kernel reported a failed bounded wait."""
    check(load().tb_check(_stream()))


def profile_begin():
    check(load().tb_profile_begin())


def profile_end(stream=None):
    """Returns {kernel name: {"launches", "ms", "flops", "bytes"}} for the launches since profile_begin()."""
    buf = C.create_string_buffer(1 << 16)
    check(load().tb_profile_end(stream, buf, len(buf)))
    out = {}
    for line in buf.value.decode().splitlines():
        name, n, ms, fl, by = line.split()
        out[name] = {"launches": int(n), "ms": float(ms), "flops": float(fl), "bytes": float(by)}
    return out


def launch_count():
    return int(load().tb_launch_count())


def gemm_f32(kind, A, B, C_out, M, N, K, lda, ldb, ldc, batch=1, sA=0, sB=0, sC=0, alpha=1.0, beta=0.0,
             precision=PREC_BF16):
    check(load().tb_gemm_f32(kind, _ptr(A), _ptr(B), _ptr(C_out), M, N, K, lda, ldb, ldc, batch, sA, sB, sC,
                             alpha, beta, precision, _stream()))


def gemm_bias_f32(A, B, bias, residual, C_out, M, N, K, precision=PREC_BF16):
    check(load().tb_gemm_bias_f32(_ptr(A), _ptr(B), _ptr(bias), _ptr(residual), _ptr(C_out), M, N, K, precision,
                                  _stream()))


def matmul_host(hA, hB, hC, M, K, N, precision=PREC_BF16):
    check(load().tb_matmul_host(_ptr(hA), _ptr(hB), _ptr(hC), M, K, N, precision))


def gemm_bf16(kind, A, B, M, N, K, lda, ldb, batch=1, sA=0, sB=0, C32=None, ldc32=0, sC32=0, C16=None, ldc16=0,
              sC16=0, bias=None, residual=None, ldr=0, sR=0, alpha=1.0, beta=0.0, causal=CAUSAL_NONE, splits=0,
              tile_n=0):
    check(load().tb_gemm_bf16(kind, _ptr(A), _ptr(B), M, N, K, lda, ldb, batch, sA, sB,
                              _ptr(C32), ldc32, sC32, _ptr(C16), ldc16, sC16, _ptr(bias), _ptr(residual), ldr, sR,
                              alpha, beta, causal, splits, tile_n, _stream()))


def gemm_bf16_splitk_static(kind, A, B, M, N, K, lda, ldb, C32, ldc32, bias=None, alpha=1.0, beta=0.0, splits=0,
                            wait=True):
    """Split-K GEMM whose scratch is built into the library image: allocates nothing (see the header)."""
    check(load().tb_gemm_bf16_splitk_static(kind, _ptr(A), _ptr(B), M, N, K, lda, ldb, _ptr(C32), ldc32, _ptr(bias),
                                            alpha, beta, splits, 1 if wait else 0, _stream()))


def gemm_bf16_splitk_static_status():
    """Waits for the current stream and raises if a static split-K call gave up on a bounded wait."""
    check(load().tb_gemm_bf16_splitk_static_status(_stream()))


def attention_fwd(Q, K, V, att, lse, B, H, T, hd, scale):
    check(load().tb_attention_fwd(_ptr(Q), _ptr(K), _ptr(V), _ptr(att), _ptr(lse), B, H, T, hd, scale, _stream()))


def attention_bwd(Q, K, V, att, datt, lse, delta, dQ, dK, dV, B, H, T, hd, scale):
    check(load().tb_attention_bwd(_ptr(Q), _ptr(K), _ptr(V), _ptr(att), _ptr(datt), _ptr(lse), _ptr(delta),
                                  _ptr(dQ), _ptr(dK), _ptr(dV), B, H, T, hd, scale, _stream()))


def gemm_swiglu_bf16(x16, w16, bias, h16, gu16=None):
    """h16[M,F] = silu(g) * u with [g | u] = x16[M,K] @ w16[K,2F] + bias[2F]; gu16 (optional bf16 [M,2F]) keeps g, u."""
    M, K = x16.shape
    F = w16.shape[1] // 2
    check(load().tb_gemm_swiglu_bf16(_ptr(x16), _ptr(w16), _ptr(bias), M, F, K, _ptr(h16), _ptr(gu16), _stream()))


def gemm_qkv_rope_bf16(x16, w16, bias, cos_t, sin_t, B, T, H, hd, qkv16):
    """qkv16 [3, B, H, T, hd] bf16 = head-split, rotated (q, k) projection x16[B*T, D] @ w16[D, 3D] + bias."""
    check(load().tb_gemm_qkv_rope_bf16(_ptr(x16), _ptr(w16), _ptr(bias), _ptr(cos_t), _ptr(sin_t), B, T, H, hd,
                                       _ptr(qkv16), _stream()))


def decode_linear(w16, S, N, K, x16=None, x32=None, norm_w=None, eps=1e-5, bias=None, residual=None, y32=None, h16=None):
    """One decode-step linear layer (see tb_decode_linear): bf16 or float32-to-normalise input, float32 or SwiGLU output."""
    check(load().tb_decode_linear(_ptr(x16), _ptr(x32), _ptr(norm_w), eps, _ptr(w16), _ptr(bias), _ptr(residual), _ptr(y32),
                                  _ptr(h16), S, N, K, _stream()))


def lmhead_argmax_bf16(x16, e16, tok, logits=None, ld_logits=0, table_is_stable=False):
    """tok[s] = argmax_v <x16[s], e16[v]> (bf16 device tensors [S, K], [V, K]; tok int32/uint32 [S]);
    logits: optional float32 [S, ld_logits] that receives the products; table_is_stable: e16 is not
    being written by earlier work of the stream (the kernel may then start reading it early)."""
    S, K = x16.shape
    V = e16.shape[0]
    check(load().tb_lmhead_argmax_bf16(_ptr(x16), _ptr(e16), S, V, K, _ptr(tok), _ptr(logits), ld_logits,
                                       1 if table_is_stable else 0, _stream()))


def pack_bf16(src, dst, rows, cols, ld_src, ld_dst, batch=1, s_src=0, s_dst=0):
    check(load().tb_pack_bf16(_ptr(src), _ptr(dst), rows, cols, ld_src, ld_dst, batch, s_src, s_dst, _stream()))
