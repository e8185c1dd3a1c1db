"""GPU: seeded random elementwise / broadcast / reduce programs through NetBuilder -> fusion -> kernels, against the
op-by-op oracle evaluation of the very groups the fusion pass produced.  The point is the plumbing (operand order,
broadcast addressing, constants, fusion boundaries, multi-group ordering), so ops are chosen to be well conditioned
and results are compared at a few ulp (reductions: reduction tolerance)."""
import numpy as np
import pytest

from cinn_b200 import common
from cinn_b200.frontend import Computation, NetBuilder
from oracle import x86_graph_eval as ge

pytestmark = pytest.mark.gpu
TARGET = common.DefaultNVGPUTarget()

UNARY = ["abs", "negative", "relu", "sigmoid", "tanh", "floor", "ceil", "sign", "identity", "sqrt_abs", "exp_small"]
BINARY = ["add", "subtract", "multiply", "max", "min", "divide_safe"]


def build_random_program(rng, b, shape, half=False):
    """Returns (feeds, fetch list).  Values: full-shape tensors, last-axis vectors, axis-1 vectors, constants."""
    feeds = {}
    F = common.Float(16 if half else 32)
    npt = np.float16 if half else np.float32
    dt = "float16" if half else "float32"

    def new_input(shp, name):
        feeds[name] = rng.uniform(-2, 2, shp).astype(npt)
        return b.create_input(F, shp, name)

    full = [new_input(shape, "A"), new_input(shape, "B")]
    last = new_input((shape[-1],), "v_last")
    mid = new_input((shape[1],), "v_mid") if len(shape) >= 3 else None
    fetch = []
    for step in range(int(rng.integers(4, 12))):
        kind = rng.choice(["unary", "binary_full", "binary_vec", "binary_const", "reduce", "select"],
                          p=[0.3, 0.2, 0.2, 0.15, 0.1, 0.05])
        x = full[int(rng.integers(0, len(full)))]
        if kind == "unary":
            op = str(rng.choice(UNARY))
            if op == "sqrt_abs":
                y = b.sqrt(b.abs(x))
            elif op == "exp_small":
                y = b.exp(b.scale(x, 0.25))
            else:
                y = getattr(b, op)(x)
        elif kind in ("binary_full", "binary_vec", "binary_const"):
            op = str(rng.choice(BINARY))
            if kind == "binary_full":
                other, axis = full[int(rng.integers(0, len(full)))], -1
            elif kind == "binary_vec":
                if mid is not None and rng.random() < 0.5:
                    other, axis = mid, 1
                else:
                    other, axis = last, -1
            else:
                other, axis = b.fill_constant(list(shape), float(rng.uniform(-1.5, 1.5)), dtype=dt), -1
            lhs, rhs = (x, other) if rng.random() < 0.5 or kind == "binary_vec" else (other, x)
            if op == "divide_safe":
                rhs = b.add(b.abs(rhs), b.fill_constant(list(shape) if kind != "binary_vec" else
                                                         [int(d) for d in rhs._info()[1]], 0.5, dtype=dt), axis=-1)
                y = b.divide(lhs, rhs, axis=axis)
            else:
                y = getattr(b, op)(lhs, rhs, axis=axis)
        elif kind == "reduce":
            if half:
                continue   # 16-bit reductions accumulate differently by design (fp32 tree vs fp16 serial)
            # one axis, or (half of the time, from rank 3) any subset of axes, non-adjacent ones included
            if len(shape) >= 3 and rng.random() < 0.5:
                axes = sorted(int(a) for a in rng.choice(len(shape), size=int(rng.integers(2, len(shape))), replace=False))
            else:
                axes = [int(rng.integers(0, len(shape)))]
            r = getattr(b, str(rng.choice(["reduce_sum", "reduce_max", "reduce_min"])))(x, axes)
            fetch.append(r)
            continue
        else:
            cond = b.greater_than(x, full[int(rng.integers(0, len(full)))])
            y = b.select(cond, x, full[int(rng.integers(0, len(full)))])
        if tuple(y._info()[1]) == tuple(shape):
            full.append(y)
    fetch.append(full[-1])
    if len(full) > 3:
        fetch.append(full[len(full) // 2])
    return feeds, fetch


@pytest.mark.parametrize("half", [False, True])
@pytest.mark.parametrize("seed", range(100))
def test_random_program_matches_the_oracle(oracle, seed, half):
    _random_program_case(seed, half, passes=False)


@pytest.mark.parametrize("half", [False, True])
@pytest.mark.parametrize("seed", range(0, 100, 3))
def test_random_program_after_the_default_passes(oracle, seed, half):
    """The same programs rewritten by the default program passes first (AutoCast, the collapsing passes,
    AutoBroadcast, the constant passes, RemoveIdentity, DeadCodeEliminate): whatever groups come out are checked
    against the oracle's evaluation of those groups."""
    _random_program_case(seed, half, passes=True)


def _random_program_case(seed, half, passes):
    rng = np.random.default_rng(1000 + seed)
    shape = [(6, 40), (3, 5, 16), (2, 7, 3, 12), (33,), (4, 9, 28)][seed % 5]
    b = NetBuilder("rand%d" % seed)
    feeds, fetch = build_random_program(rng, b, shape, half)
    if passes:
        b.apply_pass([str(f) for f in fetch])
    comp = Computation.build_and_compile(TARGET, b, fetch=[str(f) for f in fetch])
    for k, v in feeds.items():
        if k in comp.get_all_tensor_names():
            comp.get_tensor(k).from_numpy(v, TARGET)
    comp.execute()
    vals = dict(feeds)
    for desc, pattern in comp.groups():
        g = ge.parse(desc)
        if pattern.startswith("reshape_alias"):
            continue
        vals.update(ge.run_all(desc, [vals[name] for name, _, _ in g["inputs"]]))
    for f in fetch:
        got, ref = comp.get_tensor(str(f)).numpy(TARGET), vals[str(f)]
        assert got.shape == ref.shape and got.dtype == ref.dtype, (str(f), got.shape, ref.shape)
        both_nan = np.isnan(got) & np.isnan(ref)
        err = np.abs(np.where(both_nan, 0, got).astype(np.float64) - np.where(both_nan, 0, ref))
        # a few ulp, accumulated along a chain of up to a dozen ops (relative to the magnitudes involved)
        # (16-bit: a differently rounded transcendental may move a result by one float16 step per op)
        tol = (1e-2 if half else 1e-5) * np.maximum(np.abs(ref.astype(np.float64)), 1.0)
        assert (err <= tol).all(), (seed, str(f), float(err.max()), [p for _, p in comp.groups()])


def build_random_int_program(rng, b, shape, bits, extended=False):
    """extended: also draws integer pow (small bases, exponents from -2 to 6) and fetches a value cast to a 16-bit
    float."""
    unsigned = bits == 8  # uint8: the unsigned instructions, everything modulo 256
    T = common.UInt(8) if unsigned else common.Int(bits)
    npt = {8: np.uint8, 32: np.int32, 64: np.int64}[bits]
    feeds = {}

    def new_input(shp, name, lo=-2 ** 20, hi=2 ** 20):
        if unsigned:
            lo, hi = max(lo, 0), min(hi, 256)
        feeds[name] = rng.integers(lo, hi, shp).astype(npt)
        return b.create_input(T, shp, name)

    full = [new_input(shape, "A"), new_input(shape, "B", -2 ** (bits - 2), 2 ** (bits - 2))]
    div = new_input(shape, "D", 1, 97)            # strictly positive divisors
    last = new_input((shape[-1],), "v_last")
    const = lambda v: b.fill_constant(list(shape), float(v), dtype=T.name)  # noqa: E731
    fetch = []
    for step in range(int(rng.integers(4, 10))):
        x = full[int(rng.integers(0, len(full)))]
        kinds = ["unary", "binary", "vec", "const", "shift", "divmod", "select"] + ([] if unsigned else ["reduce"])
        kinds += ["pow", "pow"] if extended and not unsigned else []
        kind = str(rng.choice(kinds))
        if kind == "unary":
            y = getattr(b, str(rng.choice(["abs", "negative", "bitwise_not", "identity", "relu"])))(x)
        elif kind == "pow":
            o = full[int(rng.integers(0, len(full)))]
            base = b.subtract(b.mod(x, const(int(rng.integers(5, 40)))), const(int(rng.integers(0, 6))))
            y = b.pow(base, b.subtract(b.mod(o, const(9)), const(2)))
        elif kind == "binary":
            op = str(rng.choice(["add", "subtract", "multiply", "max", "min", "bitwise_and", "bitwise_or", "bitwise_xor"]))
            o = full[int(rng.integers(0, len(full)))]
            y = getattr(b, op)(x, o) if rng.random() < 0.5 else getattr(b, op)(o, x)
        elif kind == "vec":
            y = getattr(b, str(rng.choice(["add", "subtract", "max", "bitwise_xor"])))(x, last)
        elif kind == "const":
            y = getattr(b, str(rng.choice(["add", "multiply", "min", "bitwise_and"])))(
                x, const(int(rng.integers(0, 256) if unsigned else rng.integers(-1000, 1000))))
        elif kind == "shift":
            y = getattr(b, str(rng.choice(["left_shift", "right_shift", "logical_right_shift"])))(x, const(int(rng.integers(0, bits))))
        elif kind == "divmod":
            y = getattr(b, str(rng.choice(["floor_divide", "mod", "divide"])))(x, div)
        elif kind == "select":
            y = b.select(b.less_than(x, full[int(rng.integers(0, len(full)))]), x, full[int(rng.integers(0, len(full)))])
        else:
            fetch.append(getattr(b, str(rng.choice(["reduce_sum", "reduce_max", "reduce_min"])))(x, [int(rng.integers(0, len(shape)))]))
            continue
        full.append(y)
    fetch.append(full[-1])
    if rng.random() < 0.5:
        fetch.append(b.cast(full[len(full) // 2], "float32"))
    if extended:
        fetch.append(b.cast(full[int(rng.integers(0, len(full)))], "float16"))
    return feeds, fetch


@pytest.mark.parametrize("bits", [32, 64, 8])
@pytest.mark.parametrize("seed", range(60))
def test_random_integer_program_is_bit_exact(oracle, seed, bits):
    rng = np.random.default_rng(5000 + seed)
    shape = [(6, 40), (3, 5, 16), (33,), (4, 9, 28)][seed % 4]
    b = NetBuilder("randint%d" % seed)
    feeds, fetch = build_random_int_program(rng, b, shape, bits, extended=seed >= 40)
    comp = Computation.build_and_compile(TARGET, b, fetch=[str(f) for f in fetch])
    for k, v in feeds.items():
        if k in comp.get_all_tensor_names():
            comp.get_tensor(k).from_numpy(v, TARGET)
    comp.execute()
    vals = dict(feeds)
    for desc, pattern in comp.groups():
        g = ge.parse(desc)
        vals.update(ge.run_all(desc, [vals[name] for name, _, _ in g["inputs"]]))
    for f in fetch:
        got, ref = comp.get_tensor(str(f)).numpy(TARGET), vals[str(f)]
        assert got.dtype == ref.dtype and np.array_equal(got, ref), (seed, str(f), [p for _, p in comp.groups()])
