"""Host-side logic of the multi-GPU step, on CPU: the gradient buckets tile the flat buffer, and a
2-rank gloo all-reduce over the buckets followed by the 1/world scale gives the mean of the ranks'
gradients -- the result of the reference's fixed-order reduction (training/data_parallel.c:102-117)."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from turkce_llm_b200.data_parallel import all_reduce_bucket, check_buckets, layer_buckets


def layout(V, D, L, F):
    numels = [V * D]
    for _ in range(L):
        numels += [D, D * 3 * D, 3 * D, D * D, D, D, D * 2 * F, 2 * F, F * D, D]
    numels.append(D)
    off = np.concatenate([[0], np.cumsum(numels)[:-1]])
    return off.astype(np.int64), np.array(numels, dtype=np.int64)


def test_buckets_tile_the_flat_buffer():
    for (V, D, L, F) in ((50, 32, 2, 48), (31769, 384, 12, 1024), (7, 8, 0, 8), (9, 8, 1, 16)):
        off, num = layout(V, D, L, F)
        b = layer_buckets(off, num)
        total = int(off[-1] + num[-1])
        assert check_buckets(b, total)
        assert b[0][0] == "final_norm" and b[-1][0] == "embedding"
        assert [n for n, _, _ in b[1:-1]] == ["layer%d" % l for l in range(L - 1, -1, -1)]
    assert int(layout(31769, 384, 12, 1024)[1].sum()) == 33490176
    assert not check_buckets([("a", 0, 4), ("b", 5, 9)], 9)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    off, num = layout(50, 32, 2, 48)
    total = int(off[-1] + num[-1])
    g = torch.from_numpy(np.random.default_rng(100 + rank).standard_normal(total).astype(np.float32))
    handles = [all_reduce_bucket(dist, g, lo, hi) for _, lo, hi in layer_buckets(off, num)]
    for h in handles:
        h.wait()
    g *= 1.0 / world
    if rank == 0:
        np.save(out, g.numpy())
    dist.destroy_process_group()


def test_bucketed_all_reduce_is_the_mean_of_ranks(tmp_path):
    world = 2
    out = str(tmp_path / "g.npy")
    mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    off, num = layout(50, 32, 2, 48)
    total = int(off[-1] + num[-1])
    g0 = np.random.default_rng(100).standard_normal(total).astype(np.float32)
    g1 = np.random.default_rng(101).standard_normal(total).astype(np.float32)
    want = (g0 + g1) * np.float32(0.5)
    assert np.array_equal(np.load(out), want)


def test_shards_and_micro_batches_cover_the_global_batch():
    from turkce_llm_b200.data_parallel import micro_batches, shard_sequences
    import pytest
    for G, world, micro in ((128, 8, 16), (128, 1, 16), (128, 4, 16), (28, 4, 7), (8, 2, 4)):
        seen = []
        for r in range(world):
            first, count = shard_sequences(G, world, r)
            for f, c in micro_batches(first, count, micro):
                seen += list(range(f, f + c))
        assert seen == list(range(G))
    with pytest.raises(ValueError):
        shard_sequences(10, 4, 0)
    with pytest.raises(ValueError):
        micro_batches(0, 10, 4)


def test_windows_of_a_step_do_not_depend_on_the_number_of_ranks():
    """Each rank draws its slice of the global batch; together they are the windows one worker would draw."""
    from turkce_llm_b200.data_parallel import micro_batches, shard_sequences
    from turkce_llm_b200.gpu_train import sample_batch
    tokens = np.arange(300000, dtype=np.uint32)
    T, G = 64, 32
    whole = sample_batch(tokens, T, G, 2030)[0].reshape(G, T)
    for world in (1, 2, 4, 8):
        rows = []
        for r in range(world):
            for f, c in micro_batches(*shard_sequences(G, world, r), 4):
                rows.append(sample_batch(tokens, T, c, 2030, first_sequence=f)[0].reshape(c, T))
        assert np.array_equal(np.concatenate(rows), whole)


class _FakeTrainer:
    """Stands in for GpuTrainer on CPU: the 'gradient' of a micro-batch is a fixed function of its ids, added
    into the flat buffer as the device kernels do; Adam is replaced by recording the scaled gradient."""

    def __init__(self, total, L):
        self.total, self.cfg = total, (0, 0, 0, L)
        self.grads = torch.zeros(total)
        self.applied = None
        self._loss = 0.0

    def stream_ptr(self):
        return 0

    def zero_grads(self):
        self.grads.zero_()

    def forward(self, ids, targets, want_grad):
        self._ids = ids
        self._loss = float(np.mean(ids))

    def backward_head(self):
        rng = np.random.default_rng(int(self._ids.sum()))
        self.grads += torch.from_numpy(rng.standard_normal(self.total).astype(np.float32))

    def backward_layer(self, l):
        pass

    def backward_embed(self):
        pass

    def clip_adam_async(self, opt, max_norm, grad_scale):
        self.applied = self.grads * grad_scale

    def read_loss(self):
        return self._loss

    def last_norm(self):
        return float(self.applied.norm())


def _micro(seq):
    ids = np.full(8, seq, dtype=np.uint32)
    return ids, ids


def _accumulate_worker(rank, world, port, out):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from turkce_llm_b200 import data_parallel as dp
    off, num = layout(50, 32, 2, 48)
    total = int(off[-1] + num[-1])
    g = _FakeTrainer(total, 2)

    step = dp.DataParallelStep(g, g.grads, dp.layer_buckets(off, num), world, dist)
    step.loss_device = "cpu"
    first, count = dp.shard_sequences(8, world, rank)
    batches = [_micro(f) for f, _ in dp.micro_batches(first, count, 1)]
    loss, _ = step.host_accumulate(batches, None, 1.0)
    if rank == 0:
        np.save(out, np.concatenate([g.applied.numpy(), [loss]]))
    dist.destroy_process_group()


def test_accumulated_micro_batches_over_two_ranks_give_the_global_mean(tmp_path):
    world = 2
    out = str(tmp_path / "acc.npy")
    mp.spawn(_accumulate_worker, args=(world, _free_port(), out), nprocs=world, join=True)
    got = np.load(out)
    off, num = layout(50, 32, 2, 48)
    total = int(off[-1] + num[-1])
    want = np.zeros(total, dtype=np.float64)
    for seq in range(8):
        want += np.random.default_rng(8 * seq).standard_normal(total).astype(np.float32)
    assert np.allclose(got[:-1], want / 8, rtol=0, atol=2e-6)
    assert abs(got[-1] - np.mean(np.arange(8))) < 1e-6


def test_sharded_optimiser_slices_tile_the_flat_buffer():
    """tb_dp_slice (host arithmetic of the sharded mode, no GPU involved): the ranks' slices tile [0, total) in rank
    order, every slice starts on a multiple of 8 scalars, and world * chunk stays inside the padded flat buffers
    (1024 spare scalars behind the last parameter)."""
    import ctypes as C
    from turkce_llm_b200 import lib
    L = lib.load()
    for total in (33490176, 1000, 7, 8, 123457):
        for world in (1, 2, 3, 4, 8, 16):
            pos = 0
            chunks = set()
            for rank in range(world):
                chunk, first, count = C.c_int64(), C.c_int64(), C.c_int64()
                assert L.tb_dp_slice(total, world, rank, C.byref(chunk), C.byref(first), C.byref(count)) == 0
                chunks.add(chunk.value)
                assert first.value % 8 == 0 and chunk.value % 8 == 0
                assert first.value == rank * chunk.value
                if count.value:
                    assert first.value == pos
                    pos += count.value
                assert count.value <= chunk.value
            assert pos == total
            assert len(chunks) == 1
            assert world * chunks.pop() <= total + 1024
    assert L.tb_dp_slice(100, 4, 4, None, None, None) != 0          # rank out of range
