"""GPU: transpose / slice / concat / squeeze / expand_dims through NetBuilder against numpy (bit-exact: data movement)."""
import numpy as np
import pytest

from cinn_b200 import common
from cinn_b200.frontend import Computation, NetBuilder

pytestmark = pytest.mark.gpu
TARGET = common.DefaultNVGPUTarget()
TYPES = {"float32": (common.Float(32), np.float32), "float16": (common.Float(16), np.float16),
         "int64": (common.Int(64), np.int64), "bool": (common.Bool(), np.bool_)}


def draw(rng, shape, npt):
    if npt == np.bool_:
        return rng.random(shape) > 0.5
    if np.issubdtype(npt, np.integer):
        return rng.integers(-2 ** 40, 2 ** 40, shape).astype(npt)
    return rng.standard_normal(shape).astype(npt)


def run(b, feeds, fetch):
    comp = Computation.build_and_compile(TARGET, b)
    for k, v in feeds.items():
        comp.get_tensor(k).from_numpy(v, TARGET)
    comp.execute()
    return comp, [comp.get_tensor(str(f)).numpy(TARGET) for f in fetch]


TRANSPOSES = [((37, 53), (1, 0), "transpose_tiled"), ((4, 16, 9, 11), (0, 2, 3, 1), "transpose_tiled"),
              ((4, 9, 11, 16), (0, 3, 1, 2), "transpose_tiled"), ((3, 1, 130, 70), (0, 1, 3, 2), "transpose_tiled"),
              ((5, 6, 7), (2, 0, 1), "transpose_tiled"), ((5, 6, 7), (1, 0, 2), "transpose_gather"),
              ((2, 3, 4, 5, 6), (4, 2, 0, 3, 1), "transpose_gather"), ((8, 1, 32), (1, 0, 2), None),
              ((1024, 2048), (1, 0), "transpose_tiled")]


@pytest.mark.parametrize("shape,perm,pattern", TRANSPOSES)
@pytest.mark.parametrize("dtype", list(TYPES))
def test_transpose(shape, perm, pattern, dtype):
    t, npt = TYPES[dtype]
    b = NetBuilder("tr")
    y = b.transpose(b.create_input(t, shape, "X"), perm)
    X = draw(np.random.default_rng(90), shape, npt)
    comp, (got,) = run(b, {"X": X}, [y])
    if pattern:
        assert comp.groups()[0][1].split()[0] == pattern, comp.groups()
    assert got.dtype == X.dtype and np.array_equal(got, np.transpose(X, perm))


SLICES = [((10, 20), [0, 1], [2, 3], [9, 17], [], []), ((10, 20), [1], [-5], [100], [], []),
          ((6, 8, 10), [0, 2], [1, 0], [6, 10], [2, 3], []), ((6, 8, 10), [1], [3], [4], [], [1]),
          ((9, 33), [1], [30], [2], [-3], []), ((4, 5, 6, 7), [0, 1, 2, 3], [1, 1, 1, 1], [3, 4, 5, 6], [], [])]


@pytest.mark.parametrize("shape,axes,starts,ends,strides,decrease", SLICES)
@pytest.mark.parametrize("dtype", ["float32", "float16", "bool"])
def test_slice(oracle, shape, axes, starts, ends, strides, decrease, dtype):
    from oracle import x86_graph_eval as ge
    t, npt = TYPES[dtype]
    b = NetBuilder("sl")
    y = b.slice(b.create_input(t, shape, "X"), axes, starts, ends, strides=strides, decrease_axis=decrease)
    X = draw(np.random.default_rng(91), shape, npt)
    comp, (got,) = run(b, {"X": X}, [y])
    desc = [d for d, p in comp.groups() if p.startswith("slice_gather")][0]
    assert np.array_equal(got.reshape(-1), ge.run(desc, [X]).reshape(-1))
    if not strides and not decrease:   # and against plain numpy indexing
        sl = [slice(None)] * len(shape)
        for a, s0, e0 in zip(axes, starts, ends):
            sl[a] = slice(s0, e0)
        assert np.array_equal(got, X[tuple(sl)])


@pytest.mark.parametrize("dtype", list(TYPES))
@pytest.mark.parametrize("axis,shapes", [(0, [(3, 8), (5, 8)]), (1, [(6, 4), (6, 16), (6, 3)]), (-1, [(2, 3, 5), (2, 3, 7)]),
                                         (1, [(4, 64, 16), (4, 32, 16)]), (0, [(1000, 512), (24, 512)])])
def test_concat(axis, shapes, dtype):
    t, npt = TYPES[dtype]
    rng = np.random.default_rng(92)
    b = NetBuilder("cc")
    ins = [b.create_input(t, s, "X%d" % i) for i, s in enumerate(shapes)]
    y = b.concat(ins, axis)
    feeds = {"X%d" % i: draw(rng, s, npt) for i, s in enumerate(shapes)}
    comp, (got,) = run(b, feeds, [y])
    assert comp.groups()[0][1].split()[0] == "concat_rows"
    assert np.array_equal(got, np.concatenate([feeds["X%d" % i] for i in range(len(shapes))], axis=axis))


def test_squeeze_and_expand_dims_are_aliases():
    b = NetBuilder("sq")
    x = b.create_input(common.Float(32), (4, 1, 6, 1), "X")
    y = b.relu(b.expand_dims(b.squeeze(x, [1, 3]), [0, 3]))
    assert y._info()[1] == (1, 4, 6, 1)
    X = np.random.default_rng(93).standard_normal((4, 1, 6, 1)).astype(np.float32)
    comp, (got,) = run(b, {"X": X}, [y])
    assert [p.split()[0] for _, p in comp.groups()].count("reshape_alias") == 2
    assert np.array_equal(got, np.maximum(X, 0).reshape(1, 4, 6, 1))


def test_transforms_between_fused_groups(oracle):
    """NCHW -> NHWC transpose feeding an elementwise group, then a slice and a concat of the results."""
    rng = np.random.default_rng(94)
    X = rng.standard_normal((2, 8, 5, 6)).astype(np.float32)
    bias = rng.standard_normal(8).astype(np.float32)
    b = NetBuilder("mix")
    x = b.create_input(common.Float(32), X.shape, "X")
    bb = b.create_input(common.Float(32), (8,), "bias")
    nhwc = b.transpose(x, [0, 2, 3, 1])
    act = b.relu(b.add(nhwc, bb))
    left = b.slice(act, [3], [0], [3])
    out = b.concat([left, act], 3)
    comp, (got,) = run(b, {"X": X, "bias": bias}, [out])
    want_act = np.maximum(np.transpose(X, (0, 2, 3, 1)) + bias, 0)
    assert np.array_equal(got, np.concatenate([want_act[..., :3], want_act], axis=3))


def test_transpose_collapsing_keeps_the_values():
    """A chain of transposes before and after the TransposeCollapsing pass: same bits, one kernel instead of three."""
    from cinn_b200 import common
    from cinn_b200.frontend import Computation, NetBuilder
    target = common.DefaultNVGPUTarget()
    rng = np.random.default_rng(55)
    X = rng.standard_normal((48, 40, 36)).astype(np.float32)

    def build():
        b = NetBuilder("net")
        x = b.create_input(common.Float(32), X.shape, "X")
        t = b.transpose(b.transpose(b.transpose(x, [0, 2, 1]), [2, 1, 0]), [1, 2, 0])
        return b, x, b.relu(t)
    want = np.maximum(X.transpose(0, 2, 1).transpose(2, 1, 0).transpose(1, 2, 0), 0)
    b, x, out = build()
    comp = Computation.build_and_compile(target, b, fetch=[str(out)])
    n_plain = len(comp.groups())
    b, x, out = build()
    got, = b.build_and_get_output(target, [x], [X], [out], passes=["TransposeCollapsing"])
    comp = Computation.build_and_compile(target, b, fetch=[str(out)])
    assert len(comp.groups()) < n_plain
    assert np.array_equal(got, want)
