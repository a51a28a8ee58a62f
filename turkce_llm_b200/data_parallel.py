"""Data parallelism over GPUs: the multi-GPU extension of the reference's data_parallel_step
(training/data_parallel.c:119-163).

The reference runs one sequence per CPU thread on a shadow model and then adds the workers'
gradients in a fixed order and divides by the worker count (dp_reduce_run, :102-117).  Here every
rank holds a full replica on its own GPU, processes its own sequences, and the flat float32
gradient buffer is summed over ranks with one all-reduce per bucket; the division by the number of
ranks is folded into Adam's gradient scale.  By default the whole flat buffer is reduced by one
collective after the backward pass (0.4 ms for 134 MB on 8 GPUs).  The bucketed variant -- a bucket is one
layer's ten tensors (contiguous in the flat layout), reduced as soon as that layer's backward has been
issued; the tied embedding receives gradient both first (LM head) and last (token lookup), so its bucket
goes last -- is kept (TB_DP_MODE=overlap): it measures slower with the current GEMM kernels, see below.
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
        # Measured on 8 B200 (6.10 / 6.40 / 6.16 ms per step against 5.70 ms without any all-reduce): the
        # persistent GEMM kernels hand out their tiles statically, one CTA per SM, so a communication CTA that
        # occupies an SM while a GEMM runs holds up that whole GEMM -- the collectives under the backward pass
        # cost more than the 0.4 ms they hide.
        import os
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
