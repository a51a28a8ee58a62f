"""Data parallelism over GPUs: the multi-GPU extension of the reference's data_parallel_step
(training/data_parallel.c:119-163).

The reference runs one sequence per CPU thread on a shadow model and then adds the workers'
gradients in a fixed order and divides by the worker count (dp_reduce_run, :102-117).  Here every
rank holds a full replica on its own GPU, processes its own sequences, and the flat float32
gradient buffer is summed over ranks with one all-reduce per bucket; the division by the number of
ranks is folded into Adam's gradient scale.  A bucket is one layer's ten tensors (contiguous in the
flat layout); it is reduced as soon as that layer's backward has been issued, so the transfer
overlaps the backward of the layers below.  The tied embedding receives gradient both first (LM
head) and last (token lookup), so its bucket goes last.
"""
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
        self.stream = None
        if world > 1:
            # collectives must be ordered against the trainer's own stream: make it torch's current one
            import torch
            self.stream = torch.cuda.ExternalStream(trainer.stream_ptr())

    def _reduce(self, name, handles):
        if self.world > 1:
            lo, hi = self.buckets[name]
            handles.append(all_reduce_bucket(self.dist, self.grads, lo, hi))

    def _backward(self):
        g, handles = self.g, []
        g.backward_head()
        self._reduce("final_norm", handles)
        for l in range(self.L - 1, -1, -1):
            g.backward_layer(l)
            self._reduce("layer%d" % l, handles)
        g.backward_embed()
        self._reduce("embedding", handles)
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
