"""Two-GPU checks (skipped on a single-GPU box): outer-axis sharding of an elementwise group with no communication,
and a reduction over the sharded axis finished by one NCCL all-reduce.  Each rank is its own process on its own GPU;
ranks leave only between steps, with nothing in flight."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


# calls per context of the fused reduction: more than the three exchange areas it rotates through
N_FUSED_CALLS = 7


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        import cinn_b200
        from cinn_b200 import sharding
        from cinn_b200 import workloads as W
        dev = torch.device("cuda", rank)
        # (1) reduce_max over the sharded axis 0
        full = (64, 96, 128)
        x = W.reduce_input(full, seed=31)
        start, count = sharding.shard_range(full[0], world, rank)
        op = sharding.ShardedReduceAxis0.from_library("max", full, world, rank)
        out = torch.empty(full[1:], device=dev)
        op(torch.from_numpy(np.ascontiguousarray(x[start:start + count])).to(dev), out)
        torch.cuda.synchronize()
        np.save(os.path.join(out_dir, "max_rank%d.npy" % rank), out.cpu().numpy())
        # (2) an elementwise group on this rank's slice of axis 0: no communication at all
        shape = (32, 64, 1024)
        w = W.bias_scale_tanh_cast(shape)
        xs, bias = w.inputs
        s0, c0 = sharding.shard_range(shape[0], world, rank)
        wl = W.bias_scale_tanh_cast((c0,) + shape[1:], name="fn_c2_rank%d" % rank)
        g = cinn_b200.FusedGroup(wl.desc)
        y = torch.empty((c0,) + shape[1:], dtype=torch.float16, device=dev)
        g.run([torch.from_numpy(np.ascontiguousarray(xs[s0:s0 + c0])).to(dev), torch.from_numpy(bias).to(dev), y])
        torch.cuda.synchronize()
        np.save(os.path.join(out_dir, "c2_rank%d.npy" % rank), y.cpu().numpy())
        # (3) the fused reduction + exchange over NVLink peer memory: full result and owned band, several calls in a row
        import ctypes
        full2 = (48, 64, 256)
        inner = 64 * 256
        st, cnt = sharding.shard_range(full2[0], world, rank)
        for kind in ("max", "sum"):
            for gather in (True, False):
                fused = sharding.FusedShardedReduceAxis0(kind, full2, world, rank, all_gather=gather)
                for call in range(N_FUSED_CALLS):
                    xf = W.reduce_input(full2, seed=40 + call)
                    xl = torch.from_numpy(np.ascontiguousarray(xf[st:st + cnt])).to(dev)
                    o = torch.full(fused.out_shape, float("nan"), device=dev)
                    fused(xl, o)
                    torch.cuda.synchronize()
                    np.save(os.path.join(out_dir, "fused_%s_%d_%d_rank%d.npy" % (kind, int(gather), call, rank)),
                            o.cpu().numpy())
                if kind == "max" and gather:
                    # the same context replayed from a CUDA graph (the call counter lives on the device)
                    xf = W.reduce_input(full2, seed=77)
                    xl = torch.from_numpy(np.ascontiguousarray(xf[st:st + cnt])).to(dev)
                    o = torch.full(fused.out_shape, float("nan"), device=dev)
                    side = torch.cuda.Stream()
                    graph = torch.cuda.CUDAGraph()
                    with torch.cuda.stream(side):
                        with torch.cuda.graph(graph, stream=side):
                            for _ in range(4):
                                fused(xl, o)
                    for _ in range(2):
                        graph.replay()
                    torch.cuda.synchronize()
                    np.save(os.path.join(out_dir, "fused_graph_rank%d.npy" % rank), o.cpu().numpy())
                assert fused.status() == 0
                dist.barrier()
                fused.close()  # unmaps the peers' buffers on every rank before any rank frees its own
        n = ctypes.c_uint(0)
        assert cinn_b200.lib().cinn_b200_device_status(ctypes.byref(n)) == 0 and n.value == 0, n.value
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_two_ranks_sharded_groups(tmp_path, oracle):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    from cinn_b200 import sharding
    from cinn_b200 import workloads as W
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    full = (64, 96, 128)
    x = W.reduce_input(full, seed=31)
    want = oracle.reduce("max", x, 1, 64, 96 * 128).reshape(96, 128)
    for r in range(world):
        assert np.array_equal(np.load(tmp_path / ("max_rank%d.npy" % r)), want)
    shape = (32, 64, 1024)
    w = W.bias_scale_tanh_cast(shape)
    ref = oracle.bias_scale_tanh_f16(w.inputs[0], w.inputs[1], 0.5, 0.0)
    got = np.concatenate([np.load(tmp_path / ("c2_rank%d.npy" % r)) for r in range(world)], axis=0)
    bad, worst = oracle.count_not_close(got, ref, 1e-2, 1.2e-7)
    assert bad == 0, (bad, worst)
    # fused reduce + exchange
    full2, inner = (48, 64, 256), 64 * 256
    want = oracle.reduce("max", W.reduce_input(full2, seed=77), 1, 48, inner)
    for r in range(world):
        assert np.array_equal(np.load(tmp_path / ("fused_graph_rank%d.npy" % r)).reshape(-1), want), r
    for kind in ("max", "sum"):
        for call in range(N_FUSED_CALLS):
            xf = W.reduce_input(full2, seed=40 + call)
            want = oracle.reduce(kind, xf, 1, 48, inner)
            for r in range(world):
                full_res = np.load(tmp_path / ("fused_%s_1_%d_rank%d.npy" % (kind, call, r))).reshape(-1)
                band_res = np.load(tmp_path / ("fused_%s_0_%d_rank%d.npy" % (kind, call, r))).reshape(-1)
                band = inner // world
                if kind == "max":
                    assert np.array_equal(full_res, want), (kind, call, r)
                    assert np.array_equal(band_res, want[r * band:(r + 1) * band]), (kind, call, r)
                else:
                    assert np.allclose(full_res, want, rtol=1e-5, atol=1e-4), (kind, call, r)
                    assert np.allclose(band_res, want[r * band:(r + 1) * band], rtol=1e-5, atol=1e-4), (kind, call, r)
