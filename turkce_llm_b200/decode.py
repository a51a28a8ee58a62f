"""Greedy or temperature-sampled decoding with a KV cache (host-side wrapper of the tb_decoder_* entry points).

The reference generates by re-running its full forward per token (training/generate.c:186-212);
this wrapper keeps that calling shape -- prompts in, tokens out -- over the incremental engine."""
import ctypes as C

import numpy as np

from . import lib


class Decoder:
    def __init__(self, V, D, H, L, F, max_seqs, max_len, eps=1e-5, device=0):
        self._lib = lib.load()
        lib.init(device)
        h = C.c_void_p()
        lib.check(self._lib.tb_decoder_create(C.byref(h), V, D, H, L, F, max_seqs, max_len, eps, None))
        self.h = h
        self.V, self.S, self.cap = V, max_seqs, max_len
        self.total = int(self._lib.tb_decoder_total_scalars(self.h))

    def destroy(self):
        if self.h:
            self._lib.tb_decoder_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass

    def upload(self, flat):
        flat = np.ascontiguousarray(flat, dtype=np.float32)
        if flat.size != self.total:
            raise ValueError("expected %d scalars, got %d" % (self.total, flat.size))
        lib.check(self._lib.tb_decoder_upload(self.h, flat.ctypes.data))

    def set_sampling(self, temperature, seed=4242, seq=7):
        """sample_next of training/generate.c:57-73 with the reference generator's PCG32 stream per sequence
        (seed, seq + s); temperature <= 0 selects the greedy choice again.  Call before prefill."""
        lib.check(self._lib.tb_decoder_set_sampling(self.h, temperature, seed, seq))

    def prefill(self, prompts):
        prompts = np.ascontiguousarray(prompts, dtype=np.uint32)
        assert prompts.shape[0] == self.S
        lib.check(self._lib.tb_decoder_prefill(self.h, prompts.ctypes.data, prompts.shape[1]))

    def generate(self, n):
        lib.check(self._lib.tb_decoder_generate(self.h, n))

    def tokens(self, count):
        out = np.zeros((self.S, count), dtype=np.uint32)
        lib.check(self._lib.tb_decoder_read_tokens(self.h, out.ctypes.data, count))
        return out

    def logits(self):
        out = np.zeros((self.S, self.V), dtype=np.float32)
        lib.check(self._lib.tb_decoder_read_logits(self.h, out.ctypes.data))
        return out

    def stream_ptr(self):
        return int(self._lib.tb_decoder_stream(self.h) or 0)


def pcg_uniform(seed, seq, n):
    """n draws of the reference's pcg_uniform (runtime/prng.c:34-37) from the stream (seed, seq)."""
    out = np.empty(n, dtype=np.float64)
    lib.check(lib.load().tb_pcg_uniform_fill(seed, seq, n, out.ctypes.data))
    return out
