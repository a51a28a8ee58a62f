"""Host-side mirror of the reference's GPU-resident trainer API (model/gpu_train.h:86-125),
a thin layer over the C ABI (include/turkce_b200.h).  Method names follow the reference's
gpu_trainer_* functions; parameters are flat float32 numpy arrays in lm_collect_params order.
"""
import ctypes as C

import numpy as np

from . import lib

PARAMS, GRADS, ADAM_M, ADAM_V = 0, 1, 2, 3


class AdamState:
    """The scalars of the reference's AdamOptimizer (training/adam.h): step counter and hyper-parameters."""

    def __init__(self, lr=3e-4, beta1=0.9, beta2=0.999, eps=1e-8):
        self.t = 0
        self.lr, self.beta1, self.beta2, self.eps = lr, beta1, beta2, eps


def _u32(a):
    a = np.ascontiguousarray(a, dtype=np.uint32)
    return a, a.ctypes.data


class GpuTrainer:
    def __init__(self, V, D, H, L, F, T, B, eps=1e-5, device=0, stream=None, precision=lib.PREC_BF16):
        """precision: lib.PREC_BF16 or lib.PREC_TF32, the operand format of the linear-layer GEMMs."""
        self._lib = lib.load()
        lib.init(device)
        h = C.c_void_p()
        lib.check(self._lib.tb_trainer_create_prec(C.byref(h), V, D, H, L, F, T, B, eps, precision, stream))
        self.precision = precision
        self.h = h
        self.cfg = (V, D, H, L, F, T, B, eps)
        self.total = int(self._lib.tb_trainer_total_scalars(self.h))
        self.num_params = int(self._lib.tb_trainer_num_params(self.h))

    # gpu_trainer_destroy
    def destroy(self):
        if self.h:
            self._lib.tb_trainer_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass

    def param_layout(self):
        off = np.zeros(self.num_params, dtype=np.int64)
        num = np.zeros(self.num_params, dtype=np.int64)
        lib.check(self._lib.tb_trainer_param_layout(self.h, off.ctypes.data, num.ctypes.data))
        return off, num

    # gpu_trainer_upload / gpu_trainer_upload_grads
    def upload(self, flat, which=PARAMS):
        flat = np.ascontiguousarray(flat, dtype=np.float32)
        if flat.size != self.total:
            raise ValueError("expected %d scalars, got %d" % (self.total, flat.size))
        lib.check(self._lib.tb_trainer_upload(self.h, which, flat.ctypes.data))

    # gpu_trainer_download / gpu_trainer_download_grads
    def download(self, which=PARAMS):
        out = np.empty(self.total, dtype=np.float32)
        lib.check(self._lib.tb_trainer_download(self.h, which, out.ctypes.data))
        return out

    def device_ptr(self, which):
        return int(self._lib.tb_trainer_device_ptr(self.h, which))

    def stream_ptr(self):
        """cudaStream_t (as an integer) all of this trainer's work is issued on."""
        return int(self._lib.tb_trainer_stream(self.h) or 0)

    # gpu_trainer_forward_backward
    def forward_backward(self, ids, targets):
        ids, pi = _u32(ids)
        targets, pt = _u32(targets)
        loss = C.c_float()
        lib.check(self._lib.tb_trainer_forward_backward(self.h, pi, pt, C.byref(loss)))
        return loss.value

    # gpu_trainer_eval_loss
    def eval_loss(self, ids, targets):
        ids, pi = _u32(ids)
        targets, pt = _u32(targets)
        loss = C.c_float()
        lib.check(self._lib.tb_trainer_eval_loss(self.h, pi, pt, C.byref(loss)))
        return loss.value

    # gpu_trainer_grad_norm
    def grad_norm(self):
        n = C.c_double()
        lib.check(self._lib.tb_trainer_grad_norm(self.h, C.byref(n)))
        return n.value

    # gpu_trainer_adam_step / gpu_trainer_adam_step_scaled
    def adam_step(self, opt, grad_scale=1.0):
        opt.t += 1
        lib.check(self._lib.tb_trainer_adam_step_scaled(self.h, opt.t, opt.lr, opt.beta1, opt.beta2, opt.eps,
                                                        grad_scale))

    def train_step(self, ids, targets, opt, max_norm=1.0):
        """forward + backward + clip + Adam (one iteration of training/train_lm_gpu.c:212-223)."""
        ids, pi = _u32(ids)
        targets, pt = _u32(targets)
        opt.t += 1
        loss, norm = C.c_float(), C.c_double()
        lib.check(self._lib.tb_trainer_train_step(self.h, pi, pt, opt.t, opt.lr, opt.beta1, opt.beta2, opt.eps,
                                                  max_norm, C.byref(loss), C.byref(norm)))
        return loss.value, norm.value

    # ---- device-resident inputs: steps with no host transfer or synchronisation
    def set_inputs(self, ids, targets):
        ids, pi = _u32(ids)
        targets, pt = _u32(targets)
        lib.check(self._lib.tb_trainer_set_inputs(self.h, pi, pt))

    def step_resident(self, opt, max_norm=1.0):
        opt.t += 1
        lib.check(self._lib.tb_trainer_step_resident(self.h, opt.t, opt.lr, opt.beta1, opt.beta2, opt.eps, max_norm))

    def forward_resident(self, want_grad=True):
        lib.check(self._lib.tb_trainer_forward_resident(self.h, 1 if want_grad else 0))

    def last_norm(self):
        n = C.c_double()
        lib.check(self._lib.tb_trainer_last_norm(self.h, C.byref(n)))
        return n.value

    # ---- staged step for data parallelism
    def zero_grads(self):
        lib.check(self._lib.tb_trainer_zero_grads(self.h))

    def forward(self, ids, targets, want_grad=True):
        ids, pi = _u32(ids)
        targets, pt = _u32(targets)
        lib.check(self._lib.tb_trainer_forward(self.h, pi, pt, 1 if want_grad else 0))

    def backward_head(self):
        lib.check(self._lib.tb_trainer_backward_head(self.h))

    def backward_layer(self, layer):
        lib.check(self._lib.tb_trainer_backward_layer(self.h, layer))

    def backward_embed(self):
        lib.check(self._lib.tb_trainer_backward_embed(self.h))

    def clip_adam_async(self, opt, max_norm=1.0, grad_scale=1.0):
        opt.t += 1
        lib.check(self._lib.tb_trainer_clip_adam_async(self.h, opt.t, opt.lr, opt.beta1, opt.beta2, opt.eps,
                                                       max_norm, grad_scale))

    def read_loss(self):
        loss = C.c_float()
        lib.check(self._lib.tb_trainer_read_loss(self.h, C.byref(loss)))
        return loss.value

    # ---- the loop around the trainer (training/train_lm_gpu.c:195-260)
    def run(self, tokens, start_step, num_steps, opt, warmup_steps, total_steps, peak_lr, min_lr, max_norm=1.0):
        """Steps [start_step, start_step + num_steps) of the reference's training loop; returns (losses, norms).
        opt.t advances by num_steps."""
        tokens, pt = _u32(tokens)
        losses = np.empty(num_steps, dtype=np.float32)
        norms = np.empty(num_steps, dtype=np.float64)
        t = C.c_uint64(opt.t)
        lib.check(self._lib.tb_trainer_run(self.h, pt, tokens.size, start_step, num_steps, warmup_steps, total_steps,
                                           peak_lr, min_lr, max_norm, opt.beta1, opt.beta2, opt.eps, C.byref(t),
                                           losses.ctypes.data, norms.ctypes.data))
        opt.t = t.value
        return losses, norms

    def save_checkpoint(self, path, opt=None):
        """checkpoint_save (training/checkpoint.h:30): the reference's TRLM file; opt adds Adam m, v and t."""
        lib.check(self._lib.tb_checkpoint_save(str(path).encode(), self.h, int(opt is not None),
                                               opt.t if opt is not None else 0))

    def load_checkpoint(self, path, opt=None):
        """checkpoint_load (training/checkpoint.h:41): raises and leaves the trainer untouched on any mismatch."""
        t = C.c_uint64(0)
        lib.check(self._lib.tb_checkpoint_load(str(path).encode(), self.h, int(opt is not None), C.byref(t)))
        if opt is not None:
            opt.t = t.value


def sample_batch(tokens, T, B, seed_base, first_sequence=0):
    """gpu_trainer_sample_batch (model/gpu_train.c:296-307): B windows of one step and their targets, starting at
    sequence `first_sequence` of the global batch (a data-parallel rank draws its own slice)."""
    tokens, pt = _u32(tokens)
    ids = np.empty(B * T, dtype=np.uint32)
    tgt = np.empty(B * T, dtype=np.uint32)
    lib.check(lib.load().tb_sample_batch_range(pt, tokens.size, T, first_sequence, B, seed_base, ids.ctypes.data,
                                               tgt.ctypes.data))
    return ids, tgt


def lr_warmup_cosine(step, warmup_steps, total_steps, peak_lr, min_lr):
    """lr_warmup_cosine (training/lr_schedule.c:6-15)."""
    return float(lib.load().tb_lr_warmup_cosine(step, warmup_steps, total_steps, peak_lr, min_lr))
