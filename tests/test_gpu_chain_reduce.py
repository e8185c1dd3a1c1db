"""GPU: reductions whose operand is an elementwise chain, run as ONE kernel (chain_reduce.cu), against an exact
(float64) evaluation of the same expression on the same inputs.

Tolerance.  Every term f_i is computed in fp32 within 2 ulp (the chain kernel's bar), so a sum of n terms differs from
the exact sum by at most ~2.4e-7 * sum|f_i| from the terms plus the fp32 accumulation error of a tree, which is far below
1e-6 * sum|f_i|: sums are checked with |gpu - exact| <= 1e-5 * |exact| + 1e-6 * sum|f_i|.  max / min pick one term:
|gpu - exact| <= 1e-6 * |exact| + 1e-30.  16-bit results: 1e-2 relative.
"""
import numpy as np
import pytest

from cinn_b200 import common
from cinn_b200.frontend import Computation, NetBuilder

pytestmark = pytest.mark.gpu

TARGET = common.DefaultNVGPUTarget()


def run(builder, feeds, out):
    comp = Computation.build_and_compile(TARGET, builder, fetch=[str(out)])
    for name, arr in feeds.items():
        comp.get_tensor(name).from_numpy(arr, TARGET)
    comp.execute()
    return comp.get_tensor(str(out)).numpy(TARGET), [p for _, p in comp.groups()]


def check_sum(got, terms, axis, rtol=1e-5):
    exact = terms.sum(axis=axis)
    slack = 1e-6 * np.abs(terms).sum(axis=axis)
    assert got.shape == exact.shape
    assert np.all(np.abs(got.astype(np.float64) - exact) <= rtol * np.abs(exact) + slack), \
        float(np.max(np.abs(got - exact) / (np.abs(exact) + slack)))


def sigmoid(v):
    return 1.0 / (1.0 + np.exp(-v))


# (shape, reduced axis): rows short / long / cut into segments / odd, columns wide / tall and narrow / odd, middle axis
LAYOUTS = [((8, 16, 1024), 2), ((64, 8192), 1), ((2, 1 << 20), 1), ((33, 1001), 1), ((4096, 2048), 0), ((65536, 64), 0),
           ((1001, 33), 0), ((16, 64, 256), 1)]


@pytest.mark.parametrize("shape,axis", LAYOUTS)
def test_sum_of_a_chain_with_a_broadcast_operand(shape, axis):
    rng = np.random.default_rng(41)
    X = rng.standard_normal(shape).astype(np.float32)
    Bv = rng.standard_normal(shape[-1]).astype(np.float32)
    b = NetBuilder("net")
    x = b.create_input(common.Float(32), shape, "X")
    bias = b.create_input(common.Float(32), (shape[-1],), "B")
    out = b.reduce_sum(b.sigmoid(b.multiply(b.add(x, bias), bias)), [axis])
    got, patterns = run(b, {"X": X, "B": Bv}, out)
    assert len(patterns) == 1 and patterns[0].startswith("chain_row_reduce" if axis == len(shape) - 1 else "chain_col_reduce"), patterns
    x64, b64 = X.astype(np.float64), Bv.astype(np.float64)
    check_sum(got, sigmoid((x64 + b64) * b64), axis)


@pytest.mark.parametrize("shape,axis", LAYOUTS)
def test_sum_of_absolute_differences_of_two_tensors(shape, axis):
    rng = np.random.default_rng(42)
    X = rng.standard_normal(shape).astype(np.float32)
    Y = rng.standard_normal(shape).astype(np.float32)
    b = NetBuilder("net")
    x = b.create_input(common.Float(32), shape, "X")
    y = b.create_input(common.Float(32), shape, "Y")
    out = b.reduce_sum(b.abs(b.subtract(x, y)), [axis])
    got, patterns = run(b, {"X": X, "Y": Y}, out)
    assert len(patterns) == 1 and "chain_reduce" in patterns[0], patterns
    # |x - y| is exact up to one rounding of the difference: the only slack needed is the accumulation's
    check_sum(got, np.abs((X - Y).astype(np.float64)), axis)


@pytest.mark.parametrize("shape,axis", [((64, 8192), 1), ((4096, 2048), 0), ((33, 1001), 1), ((16, 64, 256), 1)])
@pytest.mark.parametrize("kind", ["max", "min", "prod"])
def test_max_min_prod_of_a_chain(shape, axis, kind):
    rng = np.random.default_rng(43)
    X = rng.uniform(-2, 2, shape).astype(np.float32)
    W_ = rng.uniform(0.5, 1.5, shape[-1]).astype(np.float32)
    b = NetBuilder("net")
    x = b.create_input(common.Float(32), shape, "X")
    w = b.create_input(common.Float(32), (shape[-1],), "W")
    if kind == "prod":
        # factors close to 1 so that the product of thousands of them stays finite
        val = b.scale(b.tanh(b.multiply(x, w)), 1e-3, 1.0, True)
        terms = 1e-3 * np.tanh(X.astype(np.float64) * W_) + 1.0
    else:
        val = b.multiply(b.exp(x), w)
        terms = np.exp(X.astype(np.float64)) * W_
    out = getattr(b, "reduce_" + kind)(val, [axis])
    got, patterns = run(b, {"X": X, "W": W_}, out)
    assert len(patterns) == 1 and "chain_reduce" in patterns[0], patterns
    exact = getattr(np, kind)(terms, axis=axis)
    rtol = 1e-6 if kind != "prod" else 3e-7 * shape[axis] + 1e-6   # a product accumulates one rounding per factor
    assert np.all(np.abs(got.astype(np.float64) - exact) <= rtol * np.abs(exact) + 1e-30)


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("shape,axis", [((256, 2048), 1), ((2048, 512), 0)])
def test_sixteen_bit_program_after_the_default_passes(dtype, shape, axis):
    """exp then reduce_sum on 16-bit storage: AutoCast widens both, CastCollapsing drops the pair of casts between
    them, and the whole program is one kernel reading 16-bit values and writing 16-bit sums."""
    import torch
    torch.manual_seed(5)
    tdt = torch.float16 if dtype == "float16" else torch.bfloat16
    xt = (torch.randn(shape) * 0.5).to(tdt)
    b = NetBuilder("net")
    x = b.create_input(common.Type(dtype), shape, "X")
    out = b.reduce_sum(b.exp(x), [axis])
    b.apply_pass([out])
    comp = Computation.build_and_compile(TARGET, b, fetch=[str(out)])
    patterns = [p for _, p in comp.groups()]
    assert len(patterns) == 1 and "chain_reduce" in patterns[0], patterns
    xd = xt.cuda()
    yd = torch.empty([d for i, d in enumerate(shape) if i != axis], dtype=tdt, device="cuda:0")
    comp.get_tensor("X").bind(xd.data_ptr())
    comp.get_tensor(str(out)).bind(yd.data_ptr())
    comp.execute()
    torch.cuda.synchronize()
    exact = torch.exp(xt.double()).sum(dim=axis)
    assert bool(((yd.cpu().double() - exact).abs() <= 1e-2 * exact.abs()).all())


def test_reduce_to_a_scalar_uses_the_whole_gpu():
    rng = np.random.default_rng(44)
    X = rng.standard_normal((4096, 4096)).astype(np.float32)
    Y = rng.standard_normal((4096, 4096)).astype(np.float32)
    b = NetBuilder("net")
    x = b.create_input(common.Float(32), X.shape, "X")
    y = b.create_input(common.Float(32), Y.shape, "Y")
    d = b.subtract(x, y)
    out = b.reduce_sum(b.multiply(d, d), [0, 1])
    got, patterns = run(b, {"X": X, "Y": Y}, out)
    # the interpreting kernel, or the kernel specialised at build time for sum((x - y)^2); then the fold of the segments
    assert patterns in (["chain_row_reduce chain_reduce_row_s1 reduce_generic_row_sum_f32"],
                        ["chain_row_reduce chain_reduce_static_sum_sq_diff_rows reduce_generic_row_sum_f32"]), patterns
    d = (X - Y).astype(np.float64)
    check_sum(got.reshape(()), d * d, None)
