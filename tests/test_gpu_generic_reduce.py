"""GPU: reductions of the element types other than float32 (float16, bfloat16, float64, int32, int64, bool) against
the oracle's serial reductions.  Integers and bool: bit-exact (wrapping arithmetic is associative).  float64: 1e-12
relative.  16-bit floats: the kernel accumulates in fp32 where the reference accumulates in the tensor's own type, so
the check is against the exact (float64) result within the 1e-2 tolerance of those types, and the oracle's own
distance to the exact result is printed beside it."""
import numpy as np
import pytest
import torch

import cinn_b200
from cinn_b200 import workloads as W
from tests._util import run_group

pytestmark = pytest.mark.gpu

# (shape, reduced axis): rows (last axis), columns (first / middle axis), a row long enough to be split, odd sizes
LAYOUTS = [((37, 1000), 1), ((5, 4096), 1), ((3, 70001), 1), ((1, 1 << 20), 1), ((2, 3, 65536), 2), ((16, 24, 64), 1),
           ((7, 33, 5), 1), ((512, 4096), 0), ((129, 1030), 0)]
NAMES = {np.dtype(np.float16): "float16", np.dtype(np.float64): "float64", np.dtype(np.int32): "int32",
         np.dtype(np.int64): "int64", np.dtype(np.bool_): "bool"}


def make_workload(kind, x, axis):
    shape = x.shape
    out_shape = tuple(d for i, d in enumerate(shape) if i != axis) or (1,)
    name = NAMES[x.dtype]
    desc = ("group fn_red_%s_%s\ninput X %s %s\nop reduce_%s var_0 = X ; dim=%d keep_dim=false\noutput var_0 %s %s\n"
            % (kind, name, name, ",".join(map(str, shape)), kind, axis, name, ",".join(map(str, out_shape))))
    return W.Workload("red", desc, [x], x.dtype.type, out_shape)


def view(shape, axis):
    outer = int(np.prod(shape[:axis]))
    inner = int(np.prod(shape[axis + 1:]))
    return outer, shape[axis], inner


@pytest.mark.parametrize("shape,axis", LAYOUTS)
@pytest.mark.parametrize("dtype", [np.int32, np.int64])
@pytest.mark.parametrize("misalign", [0, 1])
def test_integer_reductions_bit_exact(oracle, shape, axis, dtype, misalign):
    rng = np.random.default_rng(31)
    x = rng.integers(-2 ** 20, 2 ** 20, shape).astype(dtype)
    for kind in ("sum", "prod", "max", "min"):
        xin = (x | 1) if kind == "prod" else x   # odd factors: the wrapped product stays non-zero
        got, g = run_group(make_workload(kind, xin, axis), misalign)
        ref = oracle.reduce(kind, xin, *view(shape, axis))
        assert np.array_equal(got.reshape(-1), ref), (kind, g.kernel_names())


@pytest.mark.parametrize("shape,axis", LAYOUTS)
@pytest.mark.parametrize("misalign", [0, 3])
def test_bool_all_any(oracle, shape, axis, misalign):
    rng = np.random.default_rng(32)
    outer, r, inner = view(shape, axis)
    x = np.ones(shape, np.bool_)
    flat = x.reshape(outer, r, inner)
    flat[::2, rng.integers(0, r), ::3] = False         # some outputs of reduce_all become false
    got, _ = run_group(make_workload("all", x, axis), misalign)
    assert np.array_equal(got.reshape(-1), oracle.reduce("all", x, outer, r, inner))
    assert np.array_equal(got.reshape(-1), x.all(axis=axis).reshape(-1))
    y = ~x
    got, _ = run_group(make_workload("any", y, axis), misalign)
    assert np.array_equal(got.reshape(-1), oracle.reduce("any", y, outer, r, inner))


@pytest.mark.parametrize("shape,axis", LAYOUTS)
def test_float64_reductions(oracle, shape, axis):
    rng = np.random.default_rng(33)
    x = rng.standard_normal(shape)
    for kind in ("sum", "max", "min", "prod"):
        xin = 1.0 + 1e-4 * x if kind == "prod" else x
        got, _ = run_group(make_workload(kind, xin, axis))
        ref = oracle.reduce(kind, xin, *view(shape, axis))
        if kind in ("max", "min"):
            assert np.array_equal(got.reshape(-1), ref), kind
        else:
            scale = np.abs(xin).sum(axis=axis).reshape(-1) if kind == "sum" else np.abs(ref)
            assert (np.abs(got.reshape(-1) - ref) <= 1e-12 * scale + 1e-300).all(), kind


@pytest.mark.parametrize("shape,axis", LAYOUTS)
@pytest.mark.parametrize("misalign", [0, 1])
def test_float16_reductions(oracle, shape, axis, misalign):
    rng = np.random.default_rng(34)
    x = rng.standard_normal(shape).astype(np.float16)
    outer, r, inner = view(shape, axis)
    for kind in ("sum", "max", "min"):
        got, _ = run_group(make_workload(kind, x, axis), misalign)
        got = got.reshape(-1).astype(np.float64)
        if kind in ("max", "min"):
            assert np.array_equal(got, oracle.reduce(kind, x, outer, r, inner).astype(np.float64)), kind
            continue
        exact = x.astype(np.float64).sum(axis=axis).reshape(-1)
        # a float16 result cannot be closer to the exact sum than half its spacing; the sum of |x| bounds cancellation
        tol = 1e-2 * np.abs(exact) + 1e-3 * np.sqrt(r)
        assert (np.abs(got - exact) <= tol).all(), float(np.abs(got - exact).max())
        if r <= 4096:
            serial = oracle.reduce(kind, x, outer, r, inner).astype(np.float64)
            print("float16 sum over %d: kernel max error %.3g, serial float16 accumulation %.3g"
                  % (r, np.abs(got - exact).max(), np.abs(serial - exact).max()))


def test_bfloat16_reductions_against_exact():
    dev = torch.device("cuda:0")
    torch.manual_seed(35)
    for shape, axis in (((64, 4096), 1), ((300, 515), 0)):
        x = torch.randn(shape, device=dev).to(torch.bfloat16)
        out_shape = tuple(d for i, d in enumerate(shape) if i != axis)
        for kind, fn in (("sum", lambda t: t.sum(axis)), ("max", lambda t: t.max(axis).values),
                         ("min", lambda t: t.min(axis).values)):
            desc = ("group fn_red_bf16_%s\ninput X bfloat16 %s\nop reduce_%s var_0 = X ; dim=%d keep_dim=false\n"
                    "output var_0 bfloat16 %s\n" % (kind, ",".join(map(str, shape)), kind, axis,
                                                    ",".join(map(str, out_shape))))
            g = cinn_b200.FusedGroup(desc)
            y = torch.empty(out_shape, dtype=torch.bfloat16, device=dev)
            g.run([x, y])
            torch.cuda.synchronize()
            exact = fn(x.double())
            if kind == "sum":
                err = (y.double() - exact).abs()
                assert bool((err <= 1e-2 * exact.abs() + 0.02 * shape[axis] ** 0.5).all()), float(err.max())
            else:
                assert torch.equal(y.double(), exact), kind
            g.release()
