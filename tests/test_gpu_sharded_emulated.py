"""The fused reduce + exchange kernel (cinn_b200_col_reduce_sharded_f32) with all ranks of a world on ONE GPU.

The library's emulated form runs the ranks of a 2-, 4- or 8-rank world as one launch (one grid row per rank, every
rank's exchange buffer in this GPU's memory), so the whole protocol is exercised where only one GPU is present:
partials stored into the owner's receive area, arrival by sentinel, combination in rank order, the all-gather step,
and the rotation of the three exchange areas over many calls in a row.  The expected result is the CPU oracle's
serial reduction of the unsharded tensor (bit-exact for max / min; sums within the reduction tolerance, and equal
bit for bit on every rank because partials are combined in rank order)."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

N_CALLS = 7  # more than the three areas the exchange rotates through


@pytest.mark.parametrize("world", [1, 2, 4, 8])
@pytest.mark.parametrize("kind", ["max", "sum"])
@pytest.mark.parametrize("gather", [True, False])
def test_emulated_world_matches_oracle(world, kind, gather, oracle):
    from cinn_b200 import sharding
    from cinn_b200 import workloads as W
    full = (48, 40, 352)  # inner = 14080 = 4 * 8 * 440: bands whose last tile is ragged (440 % 256 != 0)
    inner = full[1] * full[2]
    rows = full[0] // world
    op = sharding.EmulatedFusedShardedReduceAxis0(kind, full, world, all_gather=gather)
    dev = torch.device("cuda:0")
    band = inner // world
    try:
        for call in range(N_CALLS):
            x = W.reduce_input(full, seed=100 + call)
            xs = [torch.from_numpy(np.ascontiguousarray(x[r * rows:(r + 1) * rows])).to(dev) for r in range(world)]
            outs = [torch.full(op.out_shape, float("nan"), device=dev) for _ in range(world)]
            op(xs, outs)
            torch.cuda.synchronize()
            want = oracle.reduce(kind, x, 1, full[0], inner)
            for r in range(world):
                got = outs[r].cpu().numpy().reshape(-1)
                ref = want if gather else want[r * band:(r + 1) * band]
                if kind == "max":
                    assert np.array_equal(got, ref), (world, call, r)
                else:
                    assert np.allclose(got, ref, rtol=1e-5, atol=1e-4), (world, call, r)
                    if gather:
                        assert np.array_equal(got, outs[0].cpu().numpy().reshape(-1)), "ranks disagree"
        assert op.status() == 0
    finally:
        op.close()


def test_emulated_world_replayed_from_a_cuda_graph(oracle):
    """The call counter lives on the device, so the same launch replays from a CUDA graph."""
    from cinn_b200 import sharding
    from cinn_b200 import workloads as W
    world, full = 4, (32, 64, 256)
    inner, rows = 64 * 256, 8
    dev = torch.device("cuda:0")
    op = sharding.EmulatedFusedShardedReduceAxis0("max", full, world, all_gather=True)
    try:
        x = W.reduce_input(full, seed=77)
        xs = [torch.from_numpy(np.ascontiguousarray(x[r * rows:(r + 1) * rows])).to(dev) for r in range(world)]
        outs = [torch.full(op.out_shape, float("nan"), device=dev) for _ in range(world)]
        side = torch.cuda.Stream()
        with torch.cuda.stream(side):
            op(xs, outs)  # first call outside the capture
            side.synchronize()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph, stream=side):
                for _ in range(4):
                    op(xs, outs)
        for _ in range(3):
            for o in outs:
                o.fill_(float("nan"))
            graph.replay()
        torch.cuda.synchronize()
        want = oracle.reduce("max", x, 1, full[0], inner)
        for r in range(world):
            assert np.array_equal(outs[r].cpu().numpy().reshape(-1), want), r
        assert op.status() == 0
    finally:
        op.close()


def test_sentinel_valued_result_is_delivered_as_default_nan():
    """A partial whose bits equal the "not arrived" pattern is sent as the default NaN instead of stalling the wait."""
    from cinn_b200 import sharding
    world, full = 2, (4, 8, 64)
    dev = torch.device("cuda:0")
    op = sharding.EmulatedFusedShardedReduceAxis0("max", full, world, all_gather=True)
    try:
        x = torch.zeros(full, device=dev)
        x.view(torch.int32)[:, 3, 5] = -1  # 0xFFFFFFFF in every row of one column: max of NaNs keeps the pattern
        xs = [x[:2].contiguous(), x[2:].contiguous()]
        outs = [torch.zeros(op.out_shape, device=dev) for _ in range(world)]
        op(xs, outs)
        torch.cuda.synchronize()
        assert op.status() == 0
        for o in outs:
            bits = o.view(torch.int32).cpu().numpy().reshape(full[1:])
            assert bits[3, 5] != -1  # never the sentinel
            bits[3, 5] = 0
            assert not bits.any()
    finally:
        op.close()


def test_missing_rank_runs_the_waits_out_and_the_context_turns_failed():
    """Three of four ranks launched: the partials of the fourth never arrive, every wait gives up within its budget
    (no fault, no hang), the give-up is counted, the context reports failed and a later call leaves its outputs
    alone."""
    import ctypes
    import cinn_b200
    from cinn_b200 import sharding
    world, full = 4, (8, 16, 64)
    dev = torch.device("cuda:0")
    L = cinn_b200.lib()
    cleared = ctypes.c_uint(0)
    L.cinn_b200_device_status(ctypes.byref(cleared))  # start from a clean counter
    op = sharding.EmulatedFusedShardedReduceAxis0("sum", full, world, all_gather=True)
    try:
        xs = [torch.ones((2,) + full[1:], device=dev) for _ in range(world)]
        outs = [torch.full(op.out_shape, -5.0, device=dev) for _ in range(world)]
        op(xs, outs, ranks=(0, 3))
        torch.cuda.synchronize()
        gave_up = ctypes.c_uint(0)
        assert L.cinn_b200_device_status(ctypes.byref(gave_up)) == 0 and gave_up.value >= 1
        assert op.status() == 1
        # the context stays answerable; in a complete launch the ranks that failed return at once without writing
        # results (the fourth rank, which never ran, finds the old partials, but then waits in vain for the others)
        outs2 = [torch.full(op.out_shape, -7.0, device=dev) for _ in range(world)]
        op(xs, outs2)
        torch.cuda.synchronize()
        assert all(bool((o == -7.0).all()) for o in outs2[:3])
        assert op.status() == 1
    finally:
        op.close()
        L.cinn_b200_device_status(ctypes.byref(cleared))  # leave the device counter clean for the other tests
    # a fresh context on the same device works
    op = sharding.EmulatedFusedShardedReduceAxis0("sum", full, world, all_gather=True)
    try:
        outs = [torch.zeros(op.out_shape, device=dev) for _ in range(world)]
        op(xs, outs)
        torch.cuda.synchronize()
        assert op.status() == 0 and all(bool((o == 8.0).all()) for o in outs)
    finally:
        op.close()


@pytest.mark.parametrize("reducers_per_sm", [1, 2])
def test_emulated_world_with_fewer_reducers(reducers_per_sm, oracle):
    """The `peer_reducers_per_sm` option caps the reducer CTAs (their items then take more rounds): same results."""
    import cinn_b200
    from cinn_b200 import sharding
    from cinn_b200 import workloads as W
    world, full = 4, (32, 64, 1024)  # inner = 65536: 16 tiles per band, 64 items per rank
    inner, rows = full[1] * full[2], full[0] // 4
    L = cinn_b200.lib()
    L.cinn_b200_set_option(b"peer_reducers_per_sm", reducers_per_sm)
    op = sharding.EmulatedFusedShardedReduceAxis0("max", full, world, all_gather=True)
    dev = torch.device("cuda:0")
    try:
        for call in range(4):
            x = W.reduce_input(full, seed=300 + call)
            xs = [torch.from_numpy(np.ascontiguousarray(x[r * rows:(r + 1) * rows])).to(dev) for r in range(world)]
            outs = [torch.full(op.out_shape, float("nan"), device=dev) for _ in range(world)]
            op(xs, outs)
            torch.cuda.synchronize()
            want = oracle.reduce("max", x, 1, full[0], inner)
            for r in range(world):
                assert np.array_equal(outs[r].cpu().numpy().reshape(-1), want), (call, r)
        assert op.status() == 0
    finally:
        L.cinn_b200_set_option(b"peer_reducers_per_sm", 0)
        op.close()
