"""Multi-rank host logic on CPU: shard arithmetic, and the cross-rank finish of a reduction over the sharded axis
with two gloo ranks (the local reduction is a stand-in computed by the oracle; on GPUs it is the compiled group)."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cinn_b200 import sharding


def test_shard_ranges_cover_the_axis_without_overlap():
    for extent in (0, 1, 7, 64, 128, 1000):
        for world in (1, 2, 3, 4, 8):
            pos = 0
            for rank in range(world):
                start, count = sharding.shard_range(extent, world, rank)
                assert start == pos and count >= 0
                pos += count
            assert pos == extent
            counts = [sharding.shard_range(extent, world, r)[1] for r in range(world)]
            assert max(counts) - min(counts) <= 1
    assert sharding.sharded_shape((128, 1024, 1024), 8, 3) == (16, 1024, 1024)
    assert sharding.sharded_shape((64, 1024, 1024), 8, 7) == (8, 1024, 1024)
    with pytest.raises(ValueError):
        sharding.shard_range(10, 2, 2)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, kind, shape, seed, result_dir):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from oracle import x86_oracle as orc
        x = np.random.default_rng(seed).standard_normal(shape).astype(np.float32)
        start, count = sharding.shard_range(shape[0], world, rank)
        inner = int(np.prod(shape[1:]))

        def local_reduce(xs, out):
            out.copy_(torch.from_numpy(orc.reduce(kind, xs.numpy(), 1, xs.shape[0], inner)).view(out.shape))

        op = sharding.ShardedReduceAxis0(kind, shape, world, rank, local_reduce)
        out = torch.empty(shape[1:], dtype=torch.float32)
        op(torch.from_numpy(np.ascontiguousarray(x[start:start + count])), out)
        np.save(os.path.join(result_dir, "rank%d.npy" % rank), out.numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("kind,shape", [("max", (9, 5, 7)), ("sum", (8, 33)), ("min", (1, 6))])
def test_reduce_over_sharded_axis_two_gloo_ranks(tmp_path, oracle, kind, shape):
    world, seed = 2, 5
    mp.spawn(_worker, args=(world, _free_port(), kind, shape, seed, str(tmp_path)), nprocs=world, join=True)
    x = np.random.default_rng(seed).standard_normal(shape).astype(np.float32)
    want = oracle.reduce(kind, x, 1, shape[0], int(np.prod(shape[1:]))).reshape(shape[1:])
    for rank in range(world):
        got = np.load(tmp_path / ("rank%d.npy" % rank))
        if kind in ("max", "min"):
            assert np.array_equal(got, want), rank  # order-independent: bit-exact on every rank
        else:
            assert np.allclose(got, want, rtol=1e-5, atol=1e-5), rank
