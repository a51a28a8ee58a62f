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
