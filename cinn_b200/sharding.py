"""Outer-axis sharding of fused groups over the GPUs of one node (one process per GPU, torch.distributed).

Every group of this library is independent along its outermost axis, so a rank simply compiles the group for its
own slice of that axis and runs it on its own buffers: no communication.  The one exception is a reduction over
the sharded axis itself (reduce over axis 0 of a tensor sharded on axis 0): each rank reduces its slice to a
full-size partial in its own HBM and a single all-reduce with the matching operator combines the partials
(NCCL over NVLink on GPUs, gloo in the CPU tests) -- or, in the fused form, the reduction kernel itself stores its
partials into the owner ranks' memory over NVLink and no collective library is called (FusedShardedReduceAxis0).

The reference has no multi-GPU execution at all (its only per-device state is one CUmodule per card,
cinn/runtime/cuda/cuda_module.h:67); this module is new functionality behind the same group interface.
"""
import torch
import torch.distributed as dist

_REDUCE_OPS = {"sum": dist.ReduceOp.SUM, "prod": dist.ReduceOp.PRODUCT, "max": dist.ReduceOp.MAX,
               "min": dist.ReduceOp.MIN}


def shard_range(extent, world, rank):
    """(start, count) of rank's contiguous slice of an axis of `extent` elements; earlier ranks take the remainder."""
    if not 0 <= rank < world:
        raise ValueError("rank %d outside world of %d" % (rank, world))
    base, rem = divmod(extent, world)
    start = rank * base + min(rank, rem)
    return start, base + (1 if rank < rem else 0)


def sharded_shape(shape, world, rank):
    """Shape of rank's slice when axis 0 is sharded."""
    _, count = shard_range(shape[0], world, rank)
    return (count,) + tuple(shape[1:])


def finish_reduce_over_sharded_axis(partial, kind, group=None):
    """All-reduce the per-rank partial of a reduction over the sharded axis, in place, on the current stream.

    `partial` holds this rank's reduce_<kind> over its slice (identity elements if the slice is empty)."""
    if kind not in _REDUCE_OPS:
        raise ValueError("unknown reduce kind %r" % (kind,))
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(partial, op=_REDUCE_OPS[kind], group=group)
    return partial


def identity_of(kind):
    """Initial value of the reduction (cinn/lang/builtin.cc:123-143: lowest()/max(), not infinities)."""
    return {"sum": 0.0, "prod": 1.0, "max": -3.4028234663852886e38, "min": 3.4028234663852886e38}[kind]


class ShardedReduceAxis0:
    """reduce_<kind> over axis 0 of a [R, ...] fp32 tensor whose axis 0 is sharded over the ranks.

    `local_reduce(x_slice, out)` computes the reduction of this rank's slice into `out`; on GPUs it is the
    compiled group's entry point (see `from_library`), in CPU tests a stand-in."""

    def __init__(self, kind, full_shape, world, rank, local_reduce, group=None):
        self.kind, self.full_shape, self.world, self.rank = kind, tuple(full_shape), world, rank
        self.local_shape = sharded_shape(full_shape, world, rank)
        self.out_shape = tuple(full_shape[1:])
        self.local_reduce = local_reduce
        self.group = group

    @classmethod
    def from_library(cls, kind, full_shape, world, rank, group=None):
        import cinn_b200
        local = sharded_shape(full_shape, world, rank)
        fused = None
        if local[0] > 0:
            s_in = ",".join(str(d) for d in local)
            s_out = ",".join(str(d) for d in full_shape[1:])
            fused = cinn_b200.FusedGroup(
                "group fn_reduce_%s_axis0_rank%d\ninput X float32 %s\nop reduce_%s var_0 = X ; dim=0 keep_dim=false\n"
                "output var_0 float32 %s\n" % (kind, rank, s_in, kind, s_out))

        def local_reduce(x, out):
            stream = torch.cuda.current_stream().cuda_stream
            import ctypes
            fused.run([x, out], ctypes.c_void_p(stream))

        obj = cls(kind, full_shape, world, rank, local_reduce, group)
        obj.fused = fused
        return obj

    def __call__(self, x_slice, out):
        if tuple(x_slice.shape) != self.local_shape:
            raise ValueError("rank %d expects a slice of shape %s, got %s" % (self.rank, self.local_shape,
                                                                           tuple(x_slice.shape)))
        if self.local_shape[0] > 0:
            self.local_reduce(x_slice, out)
        else:
            out.fill_(identity_of(self.kind))
        return finish_reduce_over_sharded_axis(out, self.kind, self.group)


class FusedShardedReduceAxis0:
    """reduce_<kind> over axis 0 of a [R, inner...] fp32 tensor sharded on axis 0, local reduction and cross-GPU
    exchange in ONE kernel per rank over NVLink peer memory (see cinn_b200_col_reduce_sharded_f32).

    `all_gather=True` leaves the full result on every rank (what an all-reduce gives); `False` leaves on each rank
    the band of columns it owns (what a reduce-scatter gives).  Needs an initialised process group with one rank per
    GPU of the node; the exchange buffers are mapped across processes with CUDA IPC at construction."""

    KINDS = {"sum": 0, "prod": 1, "max": 2, "min": 3}

    def __init__(self, kind, full_shape, world, rank, all_gather=True, group=None):
        import ctypes
        from . import _lib
        self.kind, self.full_shape, self.world, self.rank = kind, tuple(full_shape), world, rank
        self.all_gather = all_gather
        self.local_shape = sharded_shape(full_shape, world, rank)
        self.inner = 1
        for d in full_shape[1:]:
            self.inner *= int(d)
        if self.inner % (4 * world):
            raise ValueError("the reduced tensor's inner size must be a multiple of 4 * world")
        self.out_shape = tuple(full_shape[1:]) if all_gather else (self.inner // world,)
        L = _lib.lib()
        handle = ctypes.create_string_buffer(64)
        ctx = ctypes.c_void_p()
        _lib.check(L.cinn_b200_peer_create(rank, world, self.inner, handle, ctypes.byref(ctx)))
        self._ctx = ctx
        self._group = group
        handles = [None] * world
        if world > 1:
            dist.all_gather_object(handles, handle.raw, group=group)
        else:
            handles[0] = handle.raw
        _lib.check(L.cinn_b200_peer_connect(ctx, b"".join(handles)))
        if world > 1:
            dist.barrier(group=group)  # every rank has mapped every buffer before anyone stores into them

    def __call__(self, x_slice, out):
        import ctypes
        from . import _lib
        if tuple(x_slice.shape) != self.local_shape or self.local_shape[0] == 0:
            raise ValueError("rank %d expects a non-empty slice of shape %s" % (self.rank, self.local_shape))
        if out.numel() != (self.inner if self.all_gather else self.inner // self.world):
            raise ValueError("output has the wrong number of elements")
        stream = torch.cuda.current_stream().cuda_stream
        _lib.check(_lib.lib().cinn_b200_col_reduce_sharded_f32(
            self._ctx, self.KINDS[self.kind], ctypes.c_void_p(x_slice.data_ptr()), self.local_shape[0], self.inner,
            ctypes.c_void_p(out.data_ptr()), 1 if self.all_gather else 0, ctypes.c_void_p(stream)))
        return out

    def status(self):
        """1 if a bounded wait of an earlier call gave up (the context is then unusable), else 0.  Synchronises."""
        import ctypes
        from . import _lib
        failed = ctypes.c_int(0)
        _lib.check(_lib.lib().cinn_b200_peer_status(self._ctx, ctypes.byref(failed)))
        return failed.value

    def close(self):
        """Every rank must call this, with none of its calls in flight.  The peers' buffers are unmapped on every
        rank before any rank frees its own (freeing an allocation that another process still has open is undefined)."""
        from . import _lib
        if self._ctx is not None:
            _lib.lib().cinn_b200_peer_close_imports(self._ctx)
            if self.world > 1:
                dist.barrier(group=self._group)
            _lib.lib().cinn_b200_peer_destroy(self._ctx)
            self._ctx = None


class EmulatedFusedShardedReduceAxis0:
    """FusedShardedReduceAxis0 with all `world` ranks on ONE GPU and in one launch (the library's emulated form):
    the exchange protocol without NVLink, for machines with a single GPU.  Called with the list of every rank's
    slice and the list of every rank's output tensor."""

    def __init__(self, kind, full_shape, world, all_gather=True):
        import ctypes
        from . import _lib
        self.kind, self.full_shape, self.world, self.all_gather = kind, tuple(full_shape), world, all_gather
        if full_shape[0] % world:
            raise ValueError("the emulated form needs equal slices")
        self.rows_local = full_shape[0] // world
        self.inner = 1
        for d in full_shape[1:]:
            self.inner *= int(d)
        self.out_shape = tuple(full_shape[1:]) if all_gather else (self.inner // world,)
        ctx = ctypes.c_void_p()
        _lib.check(_lib.lib().cinn_b200_peer_create_emulated(world, self.inner, ctypes.byref(ctx)))
        self._ctx = ctx

    def __call__(self, x_slices, outs, ranks=None):
        """ranks = (first, count) launches only those ranks: with fewer than the world their bounded waits run out
        (about a quarter of a second) and the context turns failed -- the give-up path, exercised without a peer."""
        import ctypes
        from . import _lib
        xs = (ctypes.c_void_p * self.world)(*[x.data_ptr() for x in x_slices])
        os_ = (ctypes.c_void_p * self.world)(*[o.data_ptr() for o in outs])
        stream = torch.cuda.current_stream().cuda_stream
        first, count = ranks if ranks is not None else (0, self.world)
        _lib.check(_lib.lib().cinn_b200_col_reduce_sharded_f32_emulated_ranks(
            self._ctx, FusedShardedReduceAxis0.KINDS[self.kind], xs, self.rows_local, self.inner, os_,
            1 if self.all_gather else 0, first, count, ctypes.c_void_p(stream)))
        return outs

    def status(self):
        import ctypes
        from . import _lib
        failed = ctypes.c_int(0)
        _lib.check(_lib.lib().cinn_b200_peer_status(self._ctx, ctypes.byref(failed)))
        return failed.value

    def close(self):
        from . import _lib
        if self._ctx is not None:
            _lib.lib().cinn_b200_peer_destroy(self._ctx)
            self._ctx = None
