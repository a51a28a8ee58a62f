"""Data parallelism over GPUs: the multi-GPU extension of the reference's data_parallel_step
(training/data_parallel.c:119-163).

The reference runs one sequence per CPU thread on a shadow model and then adds the workers'
gradients in a fixed order and divides by the worker count (dp_reduce_run, :102-117).  Here every
rank holds a full replica on its own GPU and processes its own sequences; the flat float32 gradient
buffer is summed over the ranks and the division by the number of ranks is folded into Adam's
gradient scale.

`DataParallel` binds the library's own step (tb_dp_* in include/turkce_b200.h: NCCL called from the
library).  `DataParallelStep` is the same sequence written over torch.distributed on the staged
tb_trainer_* calls, with the choice of where the collectives go (TB_DP_MODE: one all-reduce after the
backward pass, one per layer bucket as soon as the layer's backward has been issued, or two halves);
a bucket is one layer's ten tensors (contiguous in the flat layout); the tied embedding receives
gradient both first (LM head) and last (token lookup), so its bucket goes last.
"""
import ctypes as C
import os

import numpy as np

from . import lib


def layer_buckets(offsets, numels):
    """Buckets (name, lo, hi) over the flat parameter layout, in the order backward finishes them."""
    n = len(offsets)
    L = (n - 2) // 10
    total = int(offsets[-1] + numels[-1])
    buckets = [("final_norm", int(offsets[-1]), total)]
    for l in range(L - 1, -1, -1):
        lo = int(offsets[1 + 10 * l])
        hi = int(offsets[1 + 10 * (l + 1)]) if l + 1 < L else int(offsets[-1])
        buckets.append(("layer%d" % l, lo, hi))
    buckets.append(("embedding", 0, int(offsets[1]) if n > 1 else total))
    return buckets


def check_buckets(buckets, total):
    """The buckets tile [0, total) exactly once."""
    spans = sorted((lo, hi) for _, lo, hi in buckets)
    pos = 0
    for lo, hi in spans:
        if lo != pos or hi <= lo:
            return False
        pos = hi
    return pos == total


def shard_sequences(global_batch, world, rank):
    """(first sequence, count) of the global batch that `rank` processes: contiguous slices, as the reference
    hands sequence w to worker w (training/data_parallel.c:126-135)."""
    if global_batch % world != 0:
        raise ValueError("a global batch of %d sequences does not divide over %d ranks" % (global_batch, world))
    per = global_batch // world
    return rank * per, per


def micro_batches(first, count, micro):
    """Cuts a rank's slice into micro-batches of `micro` sequences: [(first sequence, count), ...]."""
    if count % micro != 0:
        raise ValueError("%d sequences per rank do not divide into micro-batches of %d" % (count, micro))
    return [(first + i, micro) for i in range(0, count, micro)]


def all_reduce_bucket(dist, flat, lo, hi, async_op=True):
    """Sum of flat[lo:hi] over all ranks, in place."""
    return dist.all_reduce(flat[lo:hi], op=dist.ReduceOp.SUM, async_op=async_op)


class DataParallelStep:
    """One training step of a replica, with bucketed gradient all-reduce when world > 1."""

    def __init__(self, trainer, grads_view, buckets, world, dist):
        self.g = trainer
        self.grads = grads_view
        self.buckets = {name: (lo, hi) for name, lo, hi in buckets}
        self.world = world
        self.dist = dist
        self.L = trainer.cfg[3]
        if not check_buckets(buckets, trainer.total):
            raise ValueError("gradient buckets do not tile the flat buffer")
        # TB_DP_MODE: "end" (default: one all-reduce of the flat buffer after the backward pass), "overlap"
        # (one all-reduce per layer bucket as soon as the layer's backward has been issued), "halves" (two
        # collectives), or for diagnosis "none" (no all-reduce: wrong results, timing only).
        self.mode = os.environ.get("TB_DP_MODE", "end")
        self.stream = None
        self.loss_device = "cuda"      # where the ranks' losses are averaged (the host tests set "cpu")
        if world > 1 and trainer.stream_ptr():
            # collectives must be ordered against the trainer's own stream: make it torch's current one
            import torch
            self.stream = torch.cuda.ExternalStream(trainer.stream_ptr())

    def _reduce(self, name, handles):
        if self.world > 1 and self.mode == "overlap":
            lo, hi = self.buckets[name]
            handles.append(all_reduce_bucket(self.dist, self.grads, lo, hi))

    def _backward(self, reduce=True):
        g, handles = self.g, []
        if not reduce:        # a micro-batch that is not the step's last: accumulate locally, no collective
            g.backward_head()
            for l in range(self.L - 1, -1, -1):
                g.backward_layer(l)
            g.backward_embed()
            return
        g.backward_head()
        self._reduce("final_norm", handles)
        mid = self.L // 2
        for l in range(self.L - 1, -1, -1):
            g.backward_layer(l)
            self._reduce("layer%d" % l, handles)
            if self.world > 1 and self.mode == "halves" and l == mid and mid > 0:
                # layers mid..L-1 and the final norm are final: one collective for the upper part of the buffer
                handles.append(all_reduce_bucket(self.dist, self.grads, self.buckets["layer%d" % mid][0], self.g.total))
        g.backward_embed()
        self._reduce("embedding", handles)
        if self.world > 1 and self.mode == "end":       # one collective after the whole backward
            handles.append(all_reduce_bucket(self.dist, self.grads, 0, self.g.total))
        if self.world > 1 and self.mode == "halves":
            hi = self.buckets["layer%d" % mid][0] if mid > 0 else self.g.total
            handles.append(all_reduce_bucket(self.dist, self.grads, 0, hi))
        for h in handles:
            h.wait()          # orders the optimiser after the collectives on the compute stream

    def _on_stream(self):
        import contextlib
        if self.stream is None:
            return contextlib.nullcontext()
        import torch
        return torch.cuda.stream(self.stream)

    def resident(self, opt, max_norm):
        """Step on the inputs already on the device (set_inputs); nothing crosses PCIe."""
        with self._on_stream():
            self._resident(opt, max_norm)

    def host(self, ids, targets, opt, max_norm):
        """Step on host token buffers; returns (mean loss over ranks, gradient norm)."""
        with self._on_stream():
            return self._host(ids, targets, opt, max_norm)

    def _resident(self, opt, max_norm):
        g = self.g
        g.zero_grads()
        g.forward_resident(True)
        self._backward()
        g.clip_adam_async(opt, max_norm, 1.0 / self.world)

    def _host(self, ids, targets, opt, max_norm):
        g = self.g
        g.zero_grads()
        g.forward(ids, targets, True)
        self._backward()
        g.clip_adam_async(opt, max_norm, 1.0 / self.world)
        loss = g.read_loss()
        if self.world > 1:
            import torch
            t = torch.tensor([loss], device="cuda", dtype=torch.float32)
            self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
            loss = float(t.item()) / self.world
        return loss, g.last_norm()

    def host_accumulate(self, batches, opt, max_norm):
        """One optimiser step over several micro-batches [(ids, targets), ...] of this rank: the gradients of
        the micro-batches add up in the flat buffer (every backward kernel accumulates, as the reference's do),
        the ranks' sums are all-reduced once after the last micro-batch, and 1 / (world * micro-batches) is
        folded into Adam's gradient scale -- the mean over the global batch, as data_parallel_step defines it
        (training/data_parallel.c:102-117,150-162).  Returns (mean loss, gradient norm)."""
        with self._on_stream():
            g = self.g
            g.zero_grads()
            loss = 0.0
            for i, (ids, targets) in enumerate(batches):
                g.forward(ids, targets, True)
                last = i + 1 == len(batches)
                self._backward(reduce=last)
                if not last:
                    loss += g.read_loss()          # before the next forward overwrites the loss rows
            g.clip_adam_async(opt, max_norm, 1.0 / (self.world * len(batches)))
            loss = (loss + g.read_loss()) / len(batches)
            if self.world > 1:
                import torch
                t = torch.tensor([loss], device=self.loss_device, dtype=torch.float32)
                self.dist.all_reduce(t, op=self.dist.ReduceOp.SUM)
                loss = float(t.item()) / self.world
            return loss, g.last_norm()


ALLREDUCE, SHARDED, OVERLAP = 0, 1, 2


class DataParallel:
    """The library's data-parallel step (tb_dp_*): one instance per rank, over that rank's GpuTrainer.

    `dist` (torch.distributed, any backend) is used once, to hand rank 0's NCCL id to the other ranks;
    every collective of a step is issued by the library itself on the trainer's stream."""

    def __init__(self, trainer, rank=0, world=1, dist=None, mode=None):
        self.g = trainer
        self._lib = lib.load()
        if mode is None:
            # TB_DP_MODE = allreduce | sharded | overlap.  Unset: the sharded optimiser from four ranks on (measured at 8
            # GPUs: 5.78 ms per step against 5.86 with the all-reduce; the two are equal at 2 GPUs), else one all-reduce.
            name = os.environ.get("TB_DP_MODE", "sharded" if world >= 4 else "allreduce")
            mode = {"sharded": SHARDED, "overlap": OVERLAP}.get(name, ALLREDUCE)
        uid = None
        if world > 1:
            buf = (C.c_ubyte * 128)()
            if rank == 0:
                lib.check(self._lib.tb_dp_unique_id(buf))
            box = [bytes(buf)]
            dist.broadcast_object_list(box, src=0)
            uid = (C.c_ubyte * 128).from_buffer_copy(box[0])
        h = C.c_void_p()
        lib.check(self._lib.tb_dp_create(C.byref(h), trainer.h, uid, rank, world, mode))
        self.h = h
        self.rank, self.world, self.mode = rank, world, mode

    def destroy(self):
        if self.h:
            self._lib.tb_dp_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.destroy()
        except Exception:
            pass

    def describe(self):
        r, w, m, v = C.c_int(), C.c_int(), C.c_int(), C.c_int()
        lib.check(self._lib.tb_dp_info(self.h, C.byref(r), C.byref(w), C.byref(m), C.byref(v)))
        how = "one rank: no collective" if w.value == 1 else (
            "reduce-scatter + Adam on the rank's slice + all-gather of the float32 weights" if m.value == SHARDED
            else "all-reduce in per-layer buckets on a side stream under the backward pass" if m.value == OVERLAP
            else "one all-reduce of the flat float32 gradient buffer after the backward pass")
        return {"entry": "tb_dp_step (C, NCCL called by the library)", "combine": how, "nccl_version": v.value}

    def step_host(self, ids, targets, opt, max_norm):
        """One optimiser step on this rank's host token buffers; returns (mean loss over ranks, gradient norm)."""
        return self.step_host_accumulate([(ids, targets)], opt, max_norm)

    def step_host_accumulate(self, batches, opt, max_norm):
        """One optimiser step over several micro-batches [(ids, targets), ...] of this rank."""
        ids = np.ascontiguousarray(np.concatenate([np.asarray(b[0], dtype=np.uint32).reshape(-1) for b in batches]))
        tgt = np.ascontiguousarray(np.concatenate([np.asarray(b[1], dtype=np.uint32).reshape(-1) for b in batches]))
        opt.t += 1
        loss, norm = C.c_float(), C.c_double()
        lib.check(self._lib.tb_dp_step(self.h, ids.ctypes.data, tgt.ctypes.data, len(batches), opt.t, opt.lr,
                                       opt.beta1, opt.beta2, opt.eps, max_norm, C.byref(loss), C.byref(norm)))
        return loss.value, norm.value

    def step_resident(self, opt, max_norm):
        """One optimiser step on the inputs already on the device (GpuTrainer.set_inputs); asynchronous."""
        opt.t += 1
        lib.check(self._lib.tb_dp_step_resident(self.h, opt.t, opt.lr, opt.beta1, opt.beta2, opt.eps, max_norm))

    def last_result(self):
        loss, norm = C.c_float(), C.c_double()
        lib.check(self._lib.tb_dp_last_result(self.h, C.byref(loss), C.byref(norm)))
        return loss.value, norm.value
