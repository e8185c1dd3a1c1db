"""GPU: programs built with NetBuilder, fused, compiled and executed through Computation, against the oracle.

Elementwise chains are checked op-graph by op-graph with oracle/x86_graph_eval.py (the x86 arithmetic incl. the
Mul+Add contraction).  fp32 results: <= 2 ulp, except where the formula itself cancels (tanh near 0), where the
bound is 2 ulp of the cancelling operand (documented per case)."""
import ctypes

import numpy as np
import pytest

import cinn_b200
from cinn_b200 import common
from cinn_b200.frontend import Computation, NetBuilder
from oracle import x86_graph_eval as ge

pytestmark = pytest.mark.gpu
TARGET = common.DefaultNVGPUTarget()


def is_chain_kernel(kernel, interpreted):
    """`kernel` is the interpreting chain kernel variant `interpreted`, or a kernel specialised at build time for the
    same program (those take the interpreter's place whenever the program is in the library's table)."""
    return kernel == interpreted or kernel.startswith("ew_static_")


def one_chain_group(comp, interpreted):
    groups = comp.groups()
    if len(groups) != 1:
        return False
    pattern, kernel = groups[0][1].split()[:2]
    return pattern == "ew_chain" and is_chain_kernel(kernel, interpreted)


def run_program(builder, feeds, fetch):
    comp = Computation.build_and_compile(TARGET, builder)
    for name, arr in feeds.items():
        comp.get_tensor(name).from_numpy(arr, TARGET)
    comp.execute()
    return comp, {str(f): comp.get_tensor(str(f)).numpy(TARGET) for f in fetch}


def run_program_fetch(builder, feeds, fetch):
    comp = Computation.build_and_compile(TARGET, builder, fetch=[str(f) for f in fetch])
    for name, arr in feeds.items():
        comp.get_tensor(name).from_numpy(arr, TARGET)
    comp.execute()
    return comp, {str(f): comp.get_tensor(str(f)).numpy(TARGET) for f in fetch}


def oracle_program(comp, feeds):
    """Evaluate the computation's groups in order with the oracle, feeding each group from the values so far."""
    vals = dict(feeds)
    for desc, pattern in comp.groups():
        if pattern.startswith("reshape_alias"):
            g = ge.parse(desc)
            vals[g["ops"][0]["out"]] = vals[g["ops"][0]["ins"][0]].reshape(
                [int(d) for d in g["ops"][0]["attrs"]["shape"].split(",")])
            continue
        g = ge.parse(desc)
        vals.update(ge.run_all(desc, [vals[name] for name, _, _ in g["inputs"]]))
    return vals


def test_readme_example_end_to_end(oracle):
    builder = NetBuilder(name="network")
    a = builder.create_input(type=common.Float(32), shape=(1, 3, 224, 224), id_hint="A")
    b = builder.create_input(type=common.Float(32), shape=(1, 3, 224, 224), id_hint="B")
    res = builder.relu(builder.add(a, b))
    rng = np.random.default_rng(0)
    A = rng.uniform(-1, 1, (1, 3, 224, 224)).astype(np.float32)
    B = rng.uniform(-1, 1, (1, 3, 224, 224)).astype(np.float32)
    computation = Computation.build_and_compile(TARGET, builder)
    computation.get_tensor("A").from_numpy(A, TARGET)
    computation.get_tensor("B").from_numpy(B, TARGET)
    computation.execute()
    out = computation.get_tensor(str(res)).numpy(TARGET)
    assert oracle.max_ulp(out, oracle.add_relu(A, B)) == 0


UNARY_CASES = [("exp", (-10, 10), 2), ("log", (1e-3, 50), 2), ("sqrt", (0, 100), 0), ("rsqrt", (1e-3, 100), 0),
               ("sigmoid", (-15, 15), 2), ("relu", (-3, 3), 0), ("abs", (-3, 3), 0), ("negative", (-3, 3), 0),
               ("floor", (-9, 9), 0), ("ceil", (-9, 9), 0), ("trunc", (-9, 9), 0), ("round", (-9, 9), 0),
               ("sign", (-3, 3), 0), ("reciprocal", (0.01, 9), 0), ("erf", (-3, 3), 2), ("sin", (-6, 6), 2),
               ("cos", (-6, 6), 2), ("log2", (1e-3, 50), 2), ("log10", (1e-3, 50), 2), ("identity", (-3, 3), 0)]


@pytest.mark.parametrize("op,rng_range,ulps", UNARY_CASES)
def test_single_unary_op_groups(oracle, op, rng_range, ulps):
    b = NetBuilder("u_" + op)
    x = b.create_input(common.Float(32), (257, 129), "X")
    y = getattr(b, op)(x)
    X = np.random.default_rng(7).uniform(rng_range[0], rng_range[1], (257, 129)).astype(np.float32)
    comp, out = run_program(b, {"X": X}, [y])
    ref = oracle.unary(op, X)
    got = out[str(y)]
    d = oracle.max_ulp(got, ref)
    print("%s: max ulp distance to the x86 oracle %d" % (op, d))
    assert d <= ulps, (op, d)


def test_tanh_fp32_within_two_ulp_of_the_cancelling_term(oracle):
    """tanh = (1 - e)/(1 + e) with e = exp(-2|x|): an ulp of e (<= 2^-24) moves the result by up to 2^-25, so the
    bound is absolute near zero and relative (2 ulp) elsewhere."""
    b = NetBuilder("tanh32")
    x = b.create_input(common.Float(32), (513, 127), "X")
    y = b.tanh(x)
    X = np.random.default_rng(8).standard_normal((513, 127)).astype(np.float32) * 2
    comp, out = run_program(b, {"X": X}, [y])
    ref = oracle.unary("tanh", X)
    err = np.abs(out[str(y)].astype(np.float64) - ref)
    assert (err <= 2 * 2.0 ** -24 + 2 * np.spacing(np.abs(ref))).all(), float(err.max())


def chain_programs():
    def per_channel(b):
        x = b.create_input(common.Float(32), (4, 8, 15, 17), "X")
        ch = b.create_input(common.Float(32), (8,), "ch")
        y = b.relu(b.add(b.multiply(x, ch, axis=1), ch, axis=1))  # Mul+Add -> fma, per-channel side operand
        return {"X": (4, 8, 15, 17), "ch": (8,)}, b.sigmoid(b.subtract(b.fill_constant([4, 8, 15, 17], 1.0), y))

    def last_axis(b):
        x = b.create_input(common.Float(32), (6, 5, 64), "X")
        v = b.create_input(common.Float(32), (64,), "v")
        y = b.divide(b.add(x, v), b.fill_constant([1], 3.0))
        return {"X": (6, 5, 64), "v": (64,)}, b.scale(b.max(y, v), 1.5, -0.25, bias_after_scale=False)

    def odd_sizes(b):
        x = b.create_input(common.Float(32), (3, 5, 7), "X")
        v = b.create_input(common.Float(32), (7,), "v")
        w = b.create_input(common.Float(32), (3, 5, 7), "W")
        return {"X": (3, 5, 7), "v": (7,), "W": (3, 5, 7)}, b.sqrt(b.abs(b.subtract(b.multiply(x, v), w)))

    def square_fma(b):
        x = b.create_input(common.Float(32), (33, 65), "X")
        c = b.create_input(common.Float(32), (33, 65), "C")
        return {"X": (33, 65), "C": (33, 65)}, b.add(b.multiply(x, b.identity(x)), c)  # fma(x, x, c)

    def scale_chain(b):
        x = b.create_input(common.Float(32), (1000,), "X")
        return {"X": (1000,)}, b.exp(b.scale(b.negative(b.abs(x)), 0.3333333, 0.1))

    def middle_axis(b):
        x = b.create_input(common.Float(32), (4, 6, 10), "X")
        m = b.create_input(common.Float(32), (6, 1), "m")
        return {"X": (4, 6, 10), "m": (6, 1)}, b.min(b.pow(b.abs(x), b.fill_constant([1], 1.5)), b.abs(m))

    return [per_channel, last_axis, odd_sizes, square_fma, scale_chain, middle_axis]


@pytest.mark.parametrize("make", chain_programs(), ids=lambda f: f.__name__)
def test_generic_chains_match_the_oracle(oracle, make):
    b = NetBuilder(make.__name__)
    shapes, y = make(b)
    rng = np.random.default_rng(11)
    feeds = {k: rng.standard_normal(s).astype(np.float32) for k, s in shapes.items()}
    comp, out = run_program(b, feeds, [y])
    # chains, or (an operand computed from a small input: abs(m) of shape [6, 1]) one register program
    assert all(p.split()[0] in ("ew_chain", "ew_dag") for _, p in comp.groups()), comp.groups()
    ref = oracle_program(comp, feeds)[str(y)]
    d = oracle.max_ulp(out[str(y)], ref)
    print("%s: %d group(s), max ulp %d" % (make.__name__, len(comp.groups()), d))
    assert d <= 2, d


def test_fp16_chain_rounds_after_every_op(oracle):
    b = NetBuilder("h")
    x = b.create_input(common.Float(16), (40, 72), "X")
    y = b.create_input(common.Float(16), (40, 72), "Y")
    z = b.relu(b.multiply(b.add(x, y), y))
    rng = np.random.default_rng(12)
    feeds = {"X": rng.standard_normal((40, 72)).astype(np.float16), "Y": rng.standard_normal((40, 72)).astype(np.float16)}
    comp, out = run_program(b, feeds, [z])
    ref = oracle_program(comp, feeds)[str(z)]
    assert np.array_equal(out[str(z)].view(np.uint16), ref.view(np.uint16))


def test_comparison_gives_bool_bit_exact(oracle):
    b = NetBuilder("cmp")
    x = b.create_input(common.Float(32), (37, 41), "X")
    y = b.create_input(common.Float(32), (41,), "Y")
    z = b._op("greater_than", [x, y], axis=-1)
    rng = np.random.default_rng(13)
    X, Y = rng.standard_normal((37, 41)).astype(np.float32), rng.standard_normal(41).astype(np.float32)
    comp, out = run_program(b, {"X": X, "Y": Y}, [z])
    assert out[str(z)].dtype == np.bool_ and np.array_equal(out[str(z)], X > Y)


def test_tree_shaped_expression_is_one_kernel_and_correct(oracle):
    b = NetBuilder("tree")
    x = b.create_input(common.Float(32), (64, 96), "X")
    y = b.add(b.sqrt(b.abs(x)), b.exp(b.negative(x)))
    X = np.random.default_rng(14).standard_normal((64, 96)).astype(np.float32)
    comp, out = run_program(b, {"X": X}, [y])
    assert one_chain_group(comp, "ew_chain_f32_s3t"), comp.groups()  # one branch stashed in a temporary
    ref = oracle_program(comp, {"X": X})[str(y)]
    assert oracle.max_ulp(out[str(y)], ref) <= 2


TREE_SHAPES = [(64, 1024), (33, 1001), (2048, 4096)]


def _four_inputs(b, shape, dtype=32):
    return [b.create_input(common.Float(dtype), shape, n) for n in "ABCD"]


def _tree_cases():
    def product_of_sum_and_difference(b, A, B, C, D):
        return b.multiply(b.add(A, B), b.subtract(C, D))

    def sum_of_products(b, A, B, C, D):       # fma(C, D, A * B): the right product is the contracted one
        return b.add(b.multiply(A, B), b.multiply(C, D))

    def product_plus_chain(b, A, B, C, D):    # fma(A, B, relu(C) - D): the only product is on the left
        return b.add(b.multiply(A, B), b.subtract(b.relu(C), D))

    def shared_product_is_not_contracted(b, A, B, C, D):
        m = b.multiply(A, B)                  # two users: materialised by the reference, hence a plain add
        return b.multiply(b.add(m, C), b.max(m, C))

    def nested(b, A, B, C, D):
        return b.subtract(b.multiply(b.add(A, B), b.min(A, C)), b.sqrt(b.abs(B)))   # two joins, two temporaries
    return [product_of_sum_and_difference, sum_of_products, product_plus_chain, shared_product_is_not_contracted, nested]


@pytest.mark.parametrize("shape", TREE_SHAPES)
@pytest.mark.parametrize("case", _tree_cases(), ids=lambda f: f.__name__)
def test_arithmetic_trees_are_one_kernel_and_bit_exact(oracle, shape, case):
    rng = np.random.default_rng(16)
    feeds = {n: rng.standard_normal(shape).astype(np.float32) for n in "ABCD"}
    b = NetBuilder("tree")
    out = case(b, *_four_inputs(b, shape))
    if case.__name__ in ("nested", "shared_product_is_not_contracted"):
        del feeds["D"]  # not used by this expression, hence not a tensor of the computation
    comp, got = run_program(b, feeds, [out])
    assert one_chain_group(comp, "ew_chain_f32_s3t"), comp.groups()
    ref = oracle_program(comp, feeds)[str(out)]
    assert oracle.max_ulp(got[str(out)], ref) == 0


def test_tree_with_broadcast_operands_and_a_reused_input(oracle):
    rng = np.random.default_rng(17)
    shape = (257, 1024)
    feeds = {"X": rng.standard_normal(shape).astype(np.float32), "bias": rng.standard_normal(1024).astype(np.float32),
             "mean": rng.standard_normal(1024).astype(np.float32)}
    b = NetBuilder("tree")
    x = b.create_input(common.Float(32), shape, "X")
    bias = b.create_input(common.Float(32), (1024,), "bias")
    mean = b.create_input(common.Float(32), (1024,), "mean")
    out = b.multiply(b.add(x, bias), b.subtract(x, mean))   # X feeds both branches
    comp, got = run_program(b, feeds, [out])
    assert one_chain_group(comp, "ew_chain_f32_s3t"), comp.groups()
    ref = oracle_program(comp, feeds)[str(out)]
    assert oracle.max_ulp(got[str(out)], ref) == 0


def test_float16_tree_rounds_after_every_op(oracle):
    rng = np.random.default_rng(18)
    shape = (128, 1000)
    feeds = {n: rng.standard_normal(shape).astype(np.float16) for n in "ABCD"}
    b = NetBuilder("tree")
    A, B, C, D = _four_inputs(b, shape, 16)
    out = b.multiply(b.add(A, B), b.subtract(C, D))
    comp, got = run_program(b, feeds, [out])
    assert one_chain_group(comp, "ew_chain_f16_s3t"), comp.groups()
    ref = oracle_program(comp, feeds)[str(out)]
    assert np.array_equal(got[str(out)].view(np.uint16), ref.view(np.uint16))


def test_sum_of_a_tree_is_one_reduction_kernel():
    rng = np.random.default_rng(19)
    shape = (512, 4096)
    feeds = {n: rng.standard_normal(shape).astype(np.float32) for n in "ABCD"}
    b = NetBuilder("tree")
    A, B, C, D = _four_inputs(b, shape)
    out = b.reduce_sum(b.multiply(b.add(A, B), b.subtract(C, D)), [1])
    comp, got = run_program(b, feeds, [out])
    assert [p for _, p in comp.groups()] == ["chain_row_reduce chain_reduce_row_s3t"], comp.groups()
    f = {k: v.astype(np.float64) for k, v in feeds.items()}
    terms = (f["A"] + f["B"]) * (f["C"] - f["D"])
    exact = terms.sum(axis=1)
    assert np.all(np.abs(got[str(out)] - exact) <= 1e-5 * np.abs(exact) + 1e-6 * np.abs(terms).sum(axis=1))


def test_mixed_program_chain_reduce_chain(oracle):
    b = NetBuilder("mixed")
    x = b.create_input(common.Float(32), (8, 16, 1024), "X")
    bias = b.create_input(common.Float(32), (1024,), "bias")
    y = b.sigmoid(b.multiply(b.add(x, bias), bias))
    z = b.reduce_sum(y, [2])
    w = b.sqrt(b.abs(z))
    rng = np.random.default_rng(15)
    feeds = {"X": rng.standard_normal((8, 16, 1024)).astype(np.float32),
             "bias": rng.standard_normal(1024).astype(np.float32)}
    comp, out = run_program(b, feeds, [w])
    assert [p.split()[0] for _, p in comp.groups()] == ["chain_row_reduce", "ew_chain"]
    ref = oracle_program(comp, feeds)[str(w)]
    bad, worst = oracle.count_not_close(out[str(w)], ref, 1e-5, 1e-5)
    assert bad == 0, (bad, worst)


def test_reshape_aliases_and_layer_norm_on_3d(oracle):
    b = NetBuilder("ln3d")
    x = b.create_input(common.Float(32), (4, 8, 256), "X")
    g = b.create_input(common.Float(32), (256,), "gamma")
    be = b.create_input(common.Float(32), (256,), "beta")
    y = b.reshape(b.layer_norm(b.reshape(x, [32, 256]), g, be), [4, 8, 256])
    rng = np.random.default_rng(16)
    feeds = {"X": rng.standard_normal((4, 8, 256)).astype(np.float32),
             "gamma": (1 + 0.02 * rng.standard_normal(256)).astype(np.float32),
             "beta": (0.02 * rng.standard_normal(256)).astype(np.float32)}
    comp, out = run_program(b, feeds, [y])
    ref = oracle.layernorm(feeds["X"].reshape(32, 256), feeds["gamma"], feeds["beta"], 1e-5).reshape(4, 8, 256)
    bad, worst = oracle.count_not_close(out[str(y)], ref, 1e-5, 1e-6)
    assert bad == 0, (bad, worst)


def test_bind_caller_memory_and_run_on_a_stream(oracle):
    import torch
    b = NetBuilder("bind")
    x = b.create_input(common.Float(32), (128, 256), "X")
    y = b.tanh(b.scale(x, 0.5))
    comp = Computation.build_and_compile(TARGET, b)
    X = torch.randn(128, 256, device="cuda")
    out = torch.empty(128, 256, device="cuda")
    comp.get_tensor("X").bind(X.data_ptr())
    comp.get_tensor(str(y)).bind(out.data_ptr())
    s = torch.cuda.Stream()
    torch.cuda.synchronize()
    with torch.cuda.stream(s):
        comp.execute(ctypes.c_void_p(s.cuda_stream))
    s.synchronize()
    ref = oracle.unary("tanh", oracle.scale(X.cpu().numpy(), 0.5, 0.0, True))
    err = np.abs(out.cpu().numpy().astype(np.float64) - ref)
    assert (err <= 2 * 2.0 ** -24 + 2 * np.spacing(np.abs(ref))).all()


def test_no_bounded_wait_gave_up():
    L = cinn_b200.lib()
    n = ctypes.c_uint(99)
    assert L.cinn_b200_device_status(ctypes.byref(n)) == 0
    assert n.value == 0


@pytest.mark.parametrize("shape,axis", [((64, 4096), 1), ((300, 1000), 1), ((128, 64, 32), 0), ((5, 70000), 1)])
def test_reductions_with_a_folded_producer(oracle, shape, axis):
    """reduce_sum(x*x), reduce_sum(|x|), reduce_sum(exp(x)), reduce_max(|x|): one kernel each, no materialised
    intermediate; against the oracle's materialise-then-reduce evaluation."""
    b = NetBuilder("fold")
    x = b.create_input(common.Float(32), shape, "X")
    outs = {"sumsq": b.reduce_sum(b.multiply(x, b.identity(x)), [axis]), "sumabs": b.reduce_sum(b.abs(x), [axis]),
            "sumexp": b.reduce_sum(b.exp(x), [axis]), "maxabs": b.reduce_max(b.abs(x), [axis])}
    X = np.random.default_rng(17).standard_normal(shape).astype(np.float32)
    comp, got = run_program(b, {"X": X}, list(outs.values()))
    kernels = " ".join(p for _, p in comp.groups())
    assert len(comp.groups()) == 4 and all(k in kernels for k in ("sumsq", "sumabs", "sumexp", "maxabs")), kernels
    ref = oracle_program(comp, {"X": X})
    r = shape[axis]
    for name, var in outs.items():
        g, w = got[str(var)], ref[str(var)]
        if name == "maxabs":
            assert np.array_equal(g, w)
        else:
            scale = float(np.abs(w).max())
            assert np.allclose(g, w, rtol=1e-5, atol=2e-7 * r * scale / max(np.sqrt(r), 1)), name


# ---- the remaining elementwise ops of the registry: trigonometric / hyperbolic, predicates, logical, select, casts ----

MORE_UNARY_CASES = [("tan", (-1.4, 1.4), 2), ("sinh", (1.0, 8.0), 2), ("cosh", (-8.0, 8.0), 2), ("asin", (-1, 1), 2),
                    ("acos", (-1, 1), 2), ("atan", (-20, 20), 2), ("asinh", (-50, 50), 2), ("acosh", (1, 50), 2),
                    ("atanh", (-0.99, 0.99), 2), ("cbrt", (-50, 50), 1)]


@pytest.mark.parametrize("op,rng_range,ulps", MORE_UNARY_CASES)
def test_more_unary_op_groups(oracle, op, rng_range, ulps):
    b = NetBuilder("u_" + op)
    x = b.create_input(common.Float(32), (257, 129), "X")
    y = getattr(b, op)(x)
    X = np.random.default_rng(21).uniform(rng_range[0], rng_range[1], (257, 129)).astype(np.float32)
    comp, out = run_program(b, {"X": X}, [y])
    d = oracle.max_ulp(out[str(y)], oracle.unary(op, X))
    print("%s: max ulp distance to the x86 oracle %d" % (op, d))
    assert d <= ulps, (op, d)


def test_predicates_on_special_values(oracle):
    X = np.random.default_rng(22).standard_normal((33, 64)).astype(np.float32)
    X[::3, 1] = np.nan
    X[1::5, 2] = np.inf
    X[2::7, 3] = -np.inf
    for op, want in (("isnan", np.isnan(X)), ("isinf", np.isinf(X)), ("isfinite", np.isfinite(X))):
        b = NetBuilder("p_" + op)
        x = b.create_input(common.Float(32), X.shape, "X")
        y = getattr(b, op)(x)
        comp, out = run_program(b, {"X": X}, [y])
        assert out[str(y)].dtype == np.bool_ and np.array_equal(out[str(y)], want), op
        assert np.array_equal(oracle_program(comp, {"X": X})[str(y)], want), op


@pytest.mark.parametrize("op", ["mod", "remainder", "floor_divide", "atan2"])
def test_more_binary_ops(oracle, op):
    b = NetBuilder("b_" + op)
    x = b.create_input(common.Float(32), (65, 48), "X")
    y = b.create_input(common.Float(32), (48,), "Y")
    z = getattr(b, op)(x, y)
    rng = np.random.default_rng(23)
    X = (rng.standard_normal((65, 48)) * 5).astype(np.float32)
    Y = (rng.standard_normal(48) * 2).astype(np.float32)
    Y[3] = 0.0
    X[:, 5] = 0.0
    comp, out = run_program(b, {"X": X, "Y": Y}, [z])
    ref = oracle_program(comp, {"X": X, "Y": Y})[str(z)]
    got = out[str(z)]
    both_nan = np.isnan(got) & np.isnan(ref)
    d = oracle.max_ulp(np.where(both_nan, 0, got).astype(np.float32), np.where(both_nan, 0, ref).astype(np.float32))
    print("%s: max ulp %d" % (op, d))
    assert d <= (2 if op == "atan2" else 0), (op, d)


def test_logical_ops_and_not(oracle):
    rng = np.random.default_rng(24)
    P, Q = rng.random((40, 36)) > 0.5, rng.random((40, 36)) > 0.5
    for op, want in (("logical_and", P & Q), ("logical_or", P | Q), ("logical_xor", P ^ Q)):
        b = NetBuilder(op)
        p = b.create_input(common.Bool(), P.shape, "P")
        q = b.create_input(common.Bool(), Q.shape, "Q")
        y = b.logical_not(getattr(b, op)(p, q))
        comp, out = run_program(b, {"P": P, "Q": Q}, [y])
        assert out[str(y)].dtype == np.bool_ and np.array_equal(out[str(y)], ~want), op


def test_select_with_mask_input_and_with_computed_condition(oracle):
    rng = np.random.default_rng(25)
    X = rng.standard_normal((31, 100)).astype(np.float32)
    Y = rng.standard_normal((31, 100)).astype(np.float32)
    M = rng.random((31, 100)) > 0.3
    # (1) mask as an input, both values computed from inputs: where(M, exp(X), Y)
    b = NetBuilder("sel1")
    x = b.create_input(common.Float(32), X.shape, "X")
    y = b.create_input(common.Float(32), Y.shape, "Y")
    m = b.create_input(common.Bool(), M.shape, "M")
    z = b.select(m, b.exp(x), y)
    comp, out = run_program(b, {"X": X, "Y": Y, "M": M}, [z])
    assert len(comp.groups()) == 1, comp.groups()
    ref = oracle_program(comp, {"X": X, "Y": Y, "M": M})[str(z)]
    assert oracle.max_ulp(out[str(z)], ref) <= 2
    # (2) leaky relu written with a comparison: where(X > 0, X, 0.1 * X) (a tree: cut into groups, same values)
    b = NetBuilder("sel2")
    x = b.create_input(common.Float(32), X.shape, "X")
    z = b.select(b.greater_than(x, b.fill_constant(list(X.shape), 0.0)), x, b.scale(x, 0.1))
    comp, out = run_program(b, {"X": X}, [z])
    ref = oracle_program(comp, {"X": X})[str(z)]
    assert np.array_equal(out[str(z)], ref)
    assert np.array_equal(ref, np.where(X > 0, X, np.float32(0.1) * X))
    # (3) the comparison feeds arithmetic: relu as x * cast(x > 0)
    b = NetBuilder("sel3")
    x = b.create_input(common.Float(32), X.shape, "X")
    z = b.multiply(b.cast(b.greater_than(x, b.fill_constant(list(X.shape), 0.0)), "float32"), x)
    comp, out = run_program(b, {"X": X}, [z])
    assert np.array_equal(out[str(z)], np.where(X > 0, X, X * 0).astype(np.float32))


def test_casts_to_and_from_integers_and_bool(oracle):
    rng = np.random.default_rng(26)
    X = (rng.standard_normal((29, 52)) * 1000).astype(np.float32)
    X[0, :6] = [np.nan, np.inf, -np.inf, 3e9, -3e9, 2147483520.0]
    for to, npt in (("int32", np.int32), ("int64", np.int64)):
        b = NetBuilder("f2" + to)
        x = b.create_input(common.Float(32), X.shape, "X")
        y = b.cast(b.scale(x, 1.5, 0.25), to)
        comp, out = run_program(b, {"X": X}, [y])
        ref = oracle_program(comp, {"X": X})[str(y)]
        assert out[str(y)].dtype == npt and np.array_equal(out[str(y)], ref), to
    I = rng.integers(-2 ** 31, 2 ** 31 - 1, (29, 52), dtype=np.int64)
    for frm, arr in (("int32", I.astype(np.int32)), ("int64", I * 1025)):
        b = NetBuilder(frm + "2f")
        x = b.create_input(common.Int(int(frm[3:])), arr.shape, "X")
        y = b.abs(b.cast(x, "float32"))
        comp, out = run_program(b, {"X": arr}, [y])
        assert np.array_equal(out[str(y)], np.abs(arr.astype(np.float32))), frm
    b = NetBuilder("f2b")
    x = b.create_input(common.Float(32), X.shape, "X")
    y = b.cast(b.relu(x), "bool")
    comp, out = run_program(b, {"X": X}, [y])
    assert out[str(y)].dtype == np.bool_ and np.array_equal(out[str(y)], np.where(X > 0, X, 0) != 0)


# ---- integer chains (int32 / int64 arithmetic, bit operations, comparisons, select, casts at the ends) -------------

def int_programs(bits):
    T = common.Int(bits)
    shape = (37, 52)

    def arith(b):
        x, y = b.create_input(T, shape, "X"), b.create_input(T, (52,), "Y")
        return b.subtract(b.multiply(b.add(x, y), b.fill_constant([1], 3, dtype=T.name)), b.fill_constant([1], -7, dtype=T.name))

    def divisions(b):
        x, y = b.create_input(T, shape, "X"), b.create_input(T, shape, "Y")
        return b.mod(b.floor_divide(b.divide(x, b.fill_constant([1], 3, dtype=T.name)), y), y)

    def bit_ops(b):
        x, y = b.create_input(T, shape, "X"), b.create_input(T, shape, "Y")
        z = b.bitwise_xor(b.bitwise_not(b.bitwise_or(b.bitwise_and(x, y), b.fill_constant([1], 0x0f0f, dtype=T.name))), y)
        return b.right_shift(b.logical_right_shift(b.left_shift(z, b.fill_constant([1], 3, dtype=T.name)),
                                                   b.fill_constant([1], 5, dtype=T.name)),
                             b.fill_constant([1], 1, dtype=T.name))

    def counts(b):
        x = b.create_input(T, shape, "X")
        return b.add(b.popc(x), b.clz(b.abs(x)))

    def compare(b):
        x, y = b.create_input(T, shape, "X"), b.create_input(T, (52,), "Y")
        return b.logical_not(b.greater_equal(b.max(b.negative(x), y), b.fill_constant([1], 100, dtype=T.name)))

    def choose(b):
        x, y = b.create_input(T, shape, "X"), b.create_input(T, shape, "Y")
        m = b.create_input(common.Bool(), shape, "M")
        return b.select(m, b.min(x, y), b.relu(y))

    def to_float(b):
        x, y = b.create_input(T, shape, "X"), b.create_input(T, shape, "Y")
        return b.cast(b.add(x, y), "float32")

    def other_width(b):
        x, y = b.create_input(T, shape, "X"), b.create_input(T, shape, "Y")
        other = "int64" if bits == 32 else "int32"
        return b.cast(b.multiply(x, y), other)

    return [arith, divisions, bit_ops, counts, compare, choose, to_float, other_width]


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("index", range(8))
def test_integer_chains_bit_exact(oracle, bits, index):
    make = int_programs(bits)[index]
    b = NetBuilder("int_%s_%d" % (make.__name__, bits))
    y = make(b)
    rng = np.random.default_rng(40 + index)
    npt = np.int32 if bits == 32 else np.int64
    lo, hi = (-2 ** 31, 2 ** 31 - 1) if bits == 32 else (-2 ** 63, 2 ** 63 - 1)
    X = rng.integers(lo, hi, (37, 52), dtype=npt)
    Y = rng.integers(-50, 50, (37, 52), dtype=npt) if make.__name__ == "divisions" else rng.integers(lo, hi, (37, 52), dtype=npt)
    X[0, :4] = [lo, hi, 0, -1]
    feeds = {"X": X, "Y": Y, "M": rng.random((37, 52)) > 0.5}
    names = {n for d, _ in Computation.build_and_compile(TARGET, b, plan_only=True).groups() for n in
             [l.split()[1] for l in d.splitlines() if l.startswith("input")]}
    if make.__name__ in ("arith", "compare"):
        feeds["Y"] = Y[0].copy()
    feeds = {k: v for k, v in feeds.items() if k in names}
    comp, out = run_program(b, feeds, [y])
    assert all(p.split()[1].startswith("ew_chain_int_") for _, p in comp.groups()), comp.groups()
    ref = oracle_program(comp, feeds)[str(y)]
    got = out[str(y)]
    assert got.dtype == ref.dtype and np.array_equal(got, ref), (make.__name__, comp.groups())


@pytest.mark.parametrize("bits", [32, 64])
def test_integer_pow_bit_exact(oracle, bits):
    """pow on integers follows the host intrinsic (cinn/runtime/cpu/host_intrinsics.cc:234-239, 255): through double
    pow and the truncating conversion -- zero to a negative power, negative exponents, overflow and results beyond
    2^53 included."""
    T = common.Int(bits)
    npt = np.int32 if bits == 32 else np.int64
    lo, hi = (-2 ** 31, 2 ** 31 - 1) if bits == 32 else (-2 ** 63, 2 ** 63 - 1)
    rng = np.random.default_rng(77 + bits)
    shape = (41, 64)
    X = rng.integers(-12, 13, shape).astype(npt)
    Y = rng.integers(-3, 24, shape).astype(npt)
    X[0, :12] = [lo, hi, 0, 0, 1, -1, -1, 2, -2, 46341, -46341, 3]
    Y[0, :12] = [1, 1, -1, 0, hi, hi, lo, 62, 63, 2, 2, 39]
    X[1, :8] = [2, 2, -2, 3037000500, -3037000499 if bits == 64 else -3, 7, lo, hi][:8] if bits == 64 else [2, 2, -2, 1290, -1291, 7, lo, hi]
    Y[1, :8] = [31, 30, 31, 2, 2, 22 if bits == 64 else 11, 2, 2]
    X[2] = rng.integers(lo, hi, shape[1], dtype=npt)   # any base, exponent 0..2
    Y[2] = rng.integers(0, 3, shape[1]).astype(npt)
    X[3] = rng.integers(-3, 4, shape[1]).astype(npt)   # small bases, any exponent
    Y[3] = rng.integers(lo, hi, shape[1], dtype=npt)
    b = NetBuilder("int_pow_%d" % bits)
    x, y = b.create_input(T, shape, "X"), b.create_input(T, shape, "Y")
    z = b.pow(x, y)
    comp, out = run_program(b, {"X": X, "Y": Y}, [z])
    assert all(p.split()[1].startswith("ew_chain_int_") for _, p in comp.groups()), comp.groups()
    ref = oracle_program(comp, {"X": X, "Y": Y})[str(z)]
    got = out[str(z)]
    assert got.dtype == ref.dtype
    # Beyond 2^53 the host function returns whatever double pow returns for a power that no double holds exactly;
    # glibc's pow is within one ulp of it but not always the nearest double (9^17 sits exactly between two doubles and
    # glibc returns the upper one), while the kernel rounds the exact integer power to nearest-even.  There the two
    # may differ by one step of the double grid; everything a double holds exactly must be equal.
    mag = np.abs(ref.astype(np.float64))
    step = np.where(mag > 2.0 ** 53, 2.0 ** (np.floor(np.log2(np.maximum(mag, 1.0))) - 52), 0.0)
    diff = np.abs(got.astype(np.float64) - ref.astype(np.float64))
    lowest = np.iinfo(npt).min
    bad = np.argwhere((diff > step) | ((got == lowest) != (ref == lowest)))
    assert bad.size == 0, [(int(X[i, j]), int(Y[i, j]), int(got[i, j]), int(ref[i, j])) for i, j in bad[:8]]
    if bits == 32:
        assert np.array_equal(got, ref)


# ---- uint8 chains: the unsigned instructions of cinn/backends/llvm/codegen_llvm.cc:205-216, 280-340, 1449-1457 -------

def uint8_programs():
    T = common.UInt(8)
    shape = (37, 52)
    c = lambda b, v: b.fill_constant([1], v, dtype="uint8")  # noqa: E731

    def wrap(b):
        x, y = b.create_input(T, shape, "X"), b.create_input(T, (52,), "Y")
        return b.subtract(b.multiply(b.add(x, y), c(b, 3)), c(b, 7))

    def divisions(b):
        x, y = b.create_input(T, shape, "X"), b.create_input(T, shape, "Y")
        return b.mod(b.floor_divide(b.divide(b.add(x, c(b, 100)), c(b, 3)), y), b.max(y, c(b, 2)))

    def bit_ops(b):
        x, y = b.create_input(T, shape, "X"), b.create_input(T, shape, "Y")
        z = b.bitwise_xor(b.bitwise_not(b.bitwise_or(b.bitwise_and(x, y), c(b, 0x0f))), y)
        return b.right_shift(b.logical_right_shift(b.left_shift(z, c(b, 3)), c(b, 2)), c(b, 1))

    def compare(b):
        x, y = b.create_input(T, shape, "X"), b.create_input(T, (52,), "Y")
        return b.logical_not(b.greater_equal(b.max(b.negative(x), y), c(b, 100)))

    def choose(b):
        x, y = b.create_input(T, shape, "X"), b.create_input(T, shape, "Y")
        m = b.create_input(common.Bool(), shape, "M")
        return b.select(m, b.min(x, y), b.abs(y))

    def to_float(b):
        x, y = b.create_input(T, shape, "X"), b.create_input(T, shape, "Y")
        return b.cast(b.add(x, y), "float32")

    def to_int32(b):
        x, y = b.create_input(T, shape, "X"), b.create_input(T, shape, "Y")
        return b.cast(b.multiply(x, y), "int32")

    def image_normalise(b):  # uint8 pixels -> float: the cast runs in the load of the float chain
        x = b.create_input(T, shape, "X")
        return b.scale(b.cast(x, "float32"), 1.0 / 255.0, -0.5)

    return [wrap, divisions, bit_ops, compare, choose, to_float, to_int32, image_normalise]


@pytest.mark.parametrize("index", range(8))
def test_uint8_chains_bit_exact(oracle, index):
    make = uint8_programs()[index]
    b = NetBuilder("u8_%s" % make.__name__)
    y = make(b)
    rng = np.random.default_rng(60 + index)
    X = rng.integers(0, 256, (37, 52)).astype(np.uint8)
    Y = rng.integers(0, 256, (37, 52)).astype(np.uint8)
    X[0, :4] = [0, 255, 1, 128]
    Y[0, :4] = [0, 255, 0, 1]
    feeds = {"X": X, "Y": Y, "M": rng.random((37, 52)) > 0.5}
    names = {n for d, _ in Computation.build_and_compile(TARGET, b, plan_only=True).groups() for n in
             [l.split()[1] for l in d.splitlines() if l.startswith("input")]}
    if make.__name__ in ("wrap", "compare"):
        feeds["Y"] = Y[0].copy()
    feeds = {k: v for k, v in feeds.items() if k in names}
    comp, out = run_program(b, feeds, [y])
    ref = oracle_program(comp, feeds)[str(y)]
    got = out[str(y)]
    assert got.dtype == ref.dtype and np.array_equal(got, ref), (make.__name__, comp.groups())


def test_uint8_pow_and_clz_are_refused_with_a_message():
    for op in ("pow", "clz"):
        b = NetBuilder("u8_" + op)
        x = b.create_input(common.UInt(8), (8, 16), "X")
        y = b.pow(x, x) if op == "pow" else b.clz(x)
        with pytest.raises(Exception) as e:
            Computation.build_and_compile(TARGET, b, fetch=[str(y)], plan_only=True)
        assert "is not offered for uint8" in str(e.value)


# ---- float64 chains ---------------------------------------------------------------------------------------------

def f64_programs():
    T = common.Float(64)
    shape = (33, 76)

    def affine(b):
        x, v = b.create_input(T, shape, "X"), b.create_input(T, (76,), "V")
        return b.add(b.multiply(b.scale(x, 0.1, 1e-5), v), v)       # fma(scale(x), v, v), constants not exact in fp32

    def transcendental(b):
        x = b.create_input(T, shape, "X")
        return b.tanh(b.log(b.add(b.exp(b.negative(b.abs(x))), b.fill_constant([1], 1.0, dtype="float64"))))

    def trig(b):
        x, y = b.create_input(T, shape, "X"), b.create_input(T, shape, "Y")
        return b.atan2(b.sin(x), b.cosh(y))

    def compare_select(b):
        x, y = b.create_input(T, shape, "X"), b.create_input(T, shape, "Y")
        m = b.create_input(common.Bool(), shape, "M")
        return b.select(m, b.sqrt(b.abs(x)), b.floor_divide(y, b.fill_constant([1], 0.3, dtype="float64")))

    def to_float32(b):
        x = b.create_input(T, shape, "X")
        return b.cast(b.sigmoid(x), "float32")

    def from_float32(b):
        x = b.create_input(common.Float(32), shape, "X32")
        y = b.create_input(T, shape, "Y")
        return b.divide(b.cast(x, "float64"), b.relu6(y))

    def predicate(b):
        x, y = b.create_input(T, shape, "X"), b.create_input(T, shape, "Y")
        return b.logical_not(b.less_equal(b.rsqrt(b.abs(x)), y))

    return [affine, transcendental, trig, compare_select, to_float32, from_float32, predicate]


@pytest.mark.parametrize("index", range(7))
def test_float64_chains(oracle, index):
    make = f64_programs()[index]
    b = NetBuilder("f64_" + make.__name__)
    y = make(b)
    rng = np.random.default_rng(60 + index)
    feeds = {"X": rng.standard_normal((33, 76)), "Y": rng.standard_normal((33, 76)) * 3, "V": rng.standard_normal(76),
             "M": rng.random((33, 76)) > 0.5, "X32": rng.standard_normal((33, 76)).astype(np.float32)}
    names = {n for d, _ in Computation.build_and_compile(TARGET, b, plan_only=True).groups() for n in
             [l.split()[1] for l in d.splitlines() if l.startswith("input")]}
    feeds = {k: v for k, v in feeds.items() if k in names}
    comp, out = run_program(b, feeds, [y])
    assert all(p.split()[1].startswith("ew_chain_f64_") for _, p in comp.groups()), comp.groups()
    ref = oracle_program(comp, feeds)[str(y)]
    got = out[str(y)]
    assert got.dtype == ref.dtype
    if got.dtype == np.bool_:
        assert np.array_equal(got, ref)
    else:
        fin = np.isfinite(ref)
        assert np.array_equal(np.isfinite(got), fin)
        # 4 ulp, plus 4 ulp of 1.0 where the x86 tanh formula (1 - e) / (1 + e) cancels (as in the fp32 test above)
        eps = 2.0 ** -52 if got.dtype == np.float64 else 2.0 ** -23
        err = np.abs(got[fin].astype(np.float64) - ref[fin])
        ulp = err / np.spacing(np.abs(ref[fin]).astype(got.dtype)).astype(np.float64)
        print("%s: max distance %.2f ulp" % (make.__name__, ulp.max()))
        slack = 4 * eps if make.__name__ == "transcendental" else 0.0
        assert (err <= 4 * np.spacing(np.abs(ref[fin]).astype(got.dtype)).astype(np.float64) + slack).all(), float(ulp.max())


# ---- batch_norm_train (decomposed): fused channel statistics + normalisation kernel ---------------------------------

@pytest.mark.parametrize("shape", [(8, 16, 12, 12), (3, 5, 7, 9), (32, 64, 56, 56), (2, 3, 1, 5)])
def test_batch_norm_train_decomposed(oracle, shape):
    n, c, h, w = shape
    b = NetBuilder("bn_train")
    x = b.create_input(common.Float(32), shape, "x")
    ps = [b.create_input(common.Float(32), (c,), nm) for nm in ("scale", "bias", "moving_mean", "moving_variance")]
    outs = b.batchnorm(x, *ps, epsilon=1e-5, momentum=0.9, is_test=False)
    rng = np.random.default_rng(70)
    feeds = {"x": (rng.standard_normal(shape) * 2 + 0.5).astype(np.float32),
             "scale": (1 + 0.1 * rng.standard_normal(c)).astype(np.float32),
             "bias": (0.1 * rng.standard_normal(c)).astype(np.float32),
             "moving_mean": (0.1 * rng.standard_normal(c)).astype(np.float32),
             "moving_variance": rng.uniform(0.5, 1.5, c).astype(np.float32)}
    comp, out = run_program(b, feeds, outs)
    pats = [p.split()[0] for _, p in comp.groups()]
    assert pats.count("channel_stats") == 1 and pats.count("ew_bn_train_apply_nchw") == 1, pats
    ref = oracle_program(comp, feeds)
    y, mean, var, new_mean, new_var = (str(o) for o in outs)
    # statistics: reduction class (tree order on the GPU, serial in the oracle), checked against float64 as well
    x64 = feeds["x"].astype(np.float64)
    m64 = x64.mean(axis=(0, 2, 3))
    v64 = (x64 * x64).mean(axis=(0, 2, 3)) - m64 * m64
    cnt = n * h * w
    assert np.allclose(out[mean], m64, rtol=1e-5, atol=1e-6)
    assert (np.abs(out[mean] - ref[mean]) <= np.abs(ref[mean] - m64) + 1e-5 * np.abs(m64) + 1e-6).all()
    assert np.allclose(out[var], v64, rtol=1e-4, atol=1e-5), np.abs(out[var] - v64).max()
    assert np.allclose(out[new_mean], ref[new_mean], rtol=1e-5, atol=1e-6)
    assert np.allclose(out[new_var], ref[new_var], rtol=1e-4, atol=1e-5)
    # normalisation: the kernel given the oracle's statistics would be exact; with its own statistics the difference
    # is that of the statistics, amplified by |x - mean| / std <= a few units
    assert np.allclose(out[y], ref[y], rtol=1e-4, atol=1e-4), np.abs(out[y] - ref[y]).max()


def test_bn_train_apply_kernel_is_bit_exact_given_the_statistics(oracle):
    """The normalisation group alone (statistics as inputs): same bits as the x86 arithmetic (1 / sqrt, one fma)."""
    shape, c = (6, 10, 9, 11), 10
    b = NetBuilder("bn_apply")
    F = common.Float(32)
    x = b.create_input(F, shape, "x")
    mean, var, scale, bias = [b.create_input(F, (c,), nm) for nm in ("mean", "var", "scale", "bias")]
    full = list(shape)
    std = b.rsqrt(b.add(b.broadcast_to(var, full, [1]), b.fill_constant(full, 1e-5)))
    norm = b.multiply(b.subtract(x, b.broadcast_to(mean, full, [1])), std)
    y = b.relu(b.add(b.multiply(norm, b.broadcast_to(scale, full, [1])), b.broadcast_to(bias, full, [1])))
    rng = np.random.default_rng(71)
    feeds = {"x": rng.standard_normal(shape).astype(np.float32), "mean": (0.1 * rng.standard_normal(c)).astype(np.float32),
             "var": rng.uniform(0.5, 1.5, c).astype(np.float32), "scale": (1 + 0.1 * rng.standard_normal(c)).astype(np.float32),
             "bias": (0.1 * rng.standard_normal(c)).astype(np.float32)}
    comp, out = run_program(b, feeds, [y])
    assert [p.split()[0] for _, p in comp.groups()] == ["ew_bn_train_apply_relu_nchw"], comp.groups()
    m, v, s_, b_ = (feeds[k].reshape(1, c, 1, 1) for k in ("mean", "var", "scale", "bias"))
    inv = oracle.unary("rsqrt", (v + np.float32(1e-5)).astype(np.float32))
    normalized = ((feeds["x"] - m).astype(np.float32) * inv).astype(np.float32)
    want = np.maximum(oracle.fma(normalized, np.broadcast_to(s_, shape).copy(), np.broadcast_to(b_, shape).copy(), shape), 0)
    assert oracle.max_ulp(out[str(y)], want.astype(np.float32)) == 0


@pytest.mark.parametrize("kind", ["sum", "max", "min"])
@pytest.mark.parametrize("shape", [(8, 16, 12, 12), (5, 3, 7), (64, 32, 50, 20), (2, 7, 1, 1030)])
def test_reduce_over_leading_and_trailing_axes(oracle, kind, shape):
    b = NetBuilder("midkeep")
    x = b.create_input(common.Float(32), shape, "X")
    dims = [0] + list(range(2, len(shape)))
    y = getattr(b, "reduce_" + kind)(x, dims)
    X = np.random.default_rng(72).standard_normal(shape).astype(np.float32)
    comp, out = run_program(b, {"X": X}, [y])
    assert [p.split()[0] for _, p in comp.groups()] == ["mid_keep_reduce"], comp.groups()
    ref = oracle_program(comp, {"X": X})[str(y)]
    if kind == "sum":
        cnt = X.size // shape[1]
        # the serial fp32 sum of the oracle is itself off by up to ~sqrt(cnt) * 2^-24 * |partial sums|; the float64
        # sum arbitrates: the kernel (tree order) must be at least as close to it as the tolerance, and no farther
        # from the oracle than the oracle is from the exact sum plus that tolerance
        exact = X.astype(np.float64).sum(axis=tuple(dims))
        tol = 1e-5 * np.abs(exact) + 1e-6 * np.sqrt(cnt)
        assert (np.abs(out[str(y)] - exact) <= tol).all()
        assert (np.abs(out[str(y)] - ref) <= np.abs(ref - exact) + tol).all()
    else:
        assert np.array_equal(out[str(y)], ref)


def test_gelu_relu_grad_and_safe_softmax_compositions(oracle):
    rng = np.random.default_rng(80)
    X = (rng.standard_normal((48, 200)) * 2).astype(np.float32)
    D = rng.standard_normal((48, 200)).astype(np.float32)
    b = NetBuilder("gelu")
    y = b.gelu(b.create_input(common.Float(32), X.shape, "X"))
    comp, out = run_program(b, {"X": X}, [y])
    assert len(comp.groups()) == 1
    # 0.5 + 0.5 * erf(..) cancels for negative x: an ulp of erf (2^-24 near -1) is an absolute error of the factor
    ref = oracle_program(comp, {"X": X})[str(y)]
    err = np.abs(out[str(y)].astype(np.float64) - ref)
    assert (err <= 2 * np.spacing(np.abs(ref)) + 2.0 ** -23 * np.abs(X)).all(), float(err.max())
    b = NetBuilder("relu_grad")
    o, d = b.create_input(common.Float(32), X.shape, "O"), b.create_input(common.Float(32), X.shape, "D")
    y = b.relu_grad(d, o)
    comp, out = run_program(b, {"O": X, "D": D}, [y])
    assert np.array_equal(out[str(y)], np.where(X > 0, D, np.float32(0)))
    b = NetBuilder("softmax_safe")
    y = b.softmax(b.create_input(common.Float(32), X.shape, "X"), mode="safe")
    comp, out = run_program(b, {"X": X * 30}, [y])
    assert [p.split()[0] for _, p in comp.groups()] == ["softmax_safe_row"]
    ref = oracle_program(comp, {"X": X * 30})[str(y)]
    assert oracle.count_not_close(out[str(y)], ref, 1e-5, 1e-30)[0] == 0


def test_chain_that_starts_from_a_broadcast_operand(oracle):
    """No operand has the output's size: broadcast_to alone, and a broadcast followed by arithmetic."""
    rng = np.random.default_rng(81)
    V = rng.standard_normal(24).astype(np.float32)
    b = NetBuilder("bc")
    v = b.create_input(common.Float(32), (24,), "V")
    y = b.broadcast_to(v, [5, 24, 7], [1])
    z = b.exp(b.scale(b.broadcast_to(v, [3, 24], [1]), 0.5, 1.0))
    comp, out = run_program(b, {"V": V}, [y, z])
    assert all(p.split()[0] == "ew_chain" for _, p in comp.groups())
    assert np.array_equal(out[str(y)], np.broadcast_to(V.reshape(1, 24, 1), (5, 24, 7)))
    ref = oracle_program(comp, {"V": V})[str(z)]
    assert oracle.max_ulp(out[str(z)], ref) <= 2
    I = rng.integers(-100, 100, (6,), dtype=np.int32)
    b = NetBuilder("bci")
    i = b.create_input(common.Int(32), (6,), "I")
    y = b.negative(b.broadcast_to(i, [6, 10], [0]))
    comp, out = run_program(b, {"I": I}, [y])
    assert np.array_equal(out[str(y)], -np.broadcast_to(I.reshape(6, 1), (6, 10)))


def test_exported_program_runs_the_same_bits(oracle, tmp_path):
    """Export -> load (no builder, no fusion pass) -> execute: same results as the computation it came from."""
    rng = np.random.default_rng(95)
    b = NetBuilder("exp")
    x = b.create_input(common.Float(32), (4, 8, 6, 10), "x")
    ps = [b.create_input(common.Float(32), (8,), nm) for nm in ("scale", "bias", "mm", "mv")]
    outs = b.batchnorm(x, *ps, is_test=False)
    t = b.transpose(b.relu(outs[0]), [0, 2, 3, 1])
    final = b.reshape(b.softmax(b.reshape(t, [4 * 6 * 10, 8]), mode="safe"), [4, 6, 10, 8])
    feeds = {"x": rng.standard_normal((4, 8, 6, 10)).astype(np.float32), "scale": np.ones(8, np.float32),
             "bias": np.zeros(8, np.float32), "mm": np.zeros(8, np.float32), "mv": np.ones(8, np.float32)}
    fetch = [final, outs[3], outs[4]]
    comp, out = run_program(b, feeds, fetch)
    path = str(tmp_path / "program.txt")
    comp.export(path)
    loaded = Computation.load(path, TARGET)
    for k, v in feeds.items():
        loaded.get_tensor(k).from_numpy(v, TARGET)
    loaded.execute()
    for f in fetch:
        assert np.array_equal(loaded.get_tensor(str(f)).numpy(TARGET), out[str(f)]), str(f)
    assert np.allclose(out[str(final)].sum(axis=-1), 1.0, atol=1e-5)


@pytest.mark.parametrize("shape", [(8, 16, 12, 12), (3, 5, 7, 9), (16, 32, 28, 28)])
def test_batch_norm_grad_decomposed(oracle, shape):
    n, c, h, w = shape
    rng = np.random.default_rng(96)
    b = NetBuilder("bn_grad")
    F = common.Float(32)
    dy, x = b.create_input(F, shape, "dy"), b.create_input(F, shape, "x")
    scale, mean, var = (b.create_input(F, (c,), nm) for nm in ("scale", "mean", "var"))
    outs = b.batch_norm_grad(dy, x, scale, mean, var, epsilon=1e-5)
    X = (rng.standard_normal(shape) * 1.5 + 0.3).astype(np.float32)
    feeds = {"dy": rng.standard_normal(shape).astype(np.float32), "x": X,
             "scale": (1 + 0.1 * rng.standard_normal(c)).astype(np.float32),
             "mean": X.mean(axis=(0, 2, 3)).astype(np.float32), "var": X.var(axis=(0, 2, 3)).astype(np.float32)}
    comp, out = run_program(b, feeds, outs)
    pats = [p.split()[0] for _, p in comp.groups()]
    assert pats.count("bn_grad_stats") == 1 and pats.count("ew_bn_grad_apply_nchw") == 1 and len(pats) == 3, pats
    ref = oracle_program(comp, feeds)
    x_grad, scale_grad, bias_grad = (str(o) for o in outs)
    # float64 evaluation of the same formulas
    d64 = {k: v.astype(np.float64) for k, v in feeds.items()}
    m, v, s = (d64[k].reshape(1, c, 1, 1) for k in ("mean", "var", "scale"))
    cnt = n * h * w
    db = d64["dy"].sum(axis=(0, 2, 3))
    S = (d64["dy"] * (d64["x"] - m)).sum(axis=(0, 2, 3))
    inv = 1 / np.sqrt(v + 1e-5)
    dx = (s * inv / cnt) * ((d64["dy"] * cnt - db.reshape(1, c, 1, 1)) - (d64["x"] - m) * S.reshape(1, c, 1, 1) / (v + 1e-5))
    tol_sum = 1e-5 * np.abs(d64["dy"]).sum(axis=(0, 2, 3)) + 1e-6
    assert (np.abs(out[bias_grad] - db) <= tol_sum).all()
    assert (np.abs(out[scale_grad] - S * inv.reshape(-1)) <= 3e-5 * (np.abs(d64["dy"] * (d64["x"] - m)).sum(axis=(0, 2, 3)) * inv.reshape(-1)) + 1e-6).all()
    scale_dx = np.abs(dx).max()
    assert np.abs(out[x_grad] - dx).max() <= 2e-4 * scale_dx, np.abs(out[x_grad] - dx).max() / scale_dx
    # and no farther from the oracle than the oracle is from the float64 result (+ the same tolerance)
    assert np.abs(out[x_grad] - ref[x_grad]).max() <= np.abs(ref[x_grad] - dx).max() + 2e-4 * scale_dx


def test_bn_grad_apply_kernel_is_bit_exact_given_the_statistics(oracle):
    """The x_grad group alone with every per-channel operand as an input: the oracle's bits."""
    shape, c = (4, 6, 5, 12), 6
    rng = np.random.default_rng(97)
    b = NetBuilder("bn_grad_apply")
    F = common.Float(32)
    dy, x = b.create_input(F, shape, "dy"), b.create_input(F, shape, "x")
    t0, db, mean, S, vae = (b.create_input(F, (c,), nm) for nm in ("t0", "db", "mean", "S", "vae"))
    full, cnt = list(shape), float(4 * 5 * 12)
    tmp1 = b.multiply(dy, b.fill_constant(full, cnt))
    tmp3 = b.divide(b.multiply(b.subtract(x, b.broadcast_to(mean, full, [1])), b.broadcast_to(S, full, [1])),
                    b.broadcast_to(vae, full, [1]))
    y = b.multiply(b.broadcast_to(t0, full, [1]), b.subtract(b.subtract(tmp1, b.broadcast_to(db, full, [1])), tmp3))
    feeds = {"dy": rng.standard_normal(shape).astype(np.float32), "x": rng.standard_normal(shape).astype(np.float32),
             "t0": rng.uniform(0.001, 0.01, c).astype(np.float32), "db": rng.standard_normal(c).astype(np.float32),
             "mean": (0.1 * rng.standard_normal(c)).astype(np.float32), "S": rng.standard_normal(c).astype(np.float32),
             "vae": rng.uniform(0.5, 1.5, c).astype(np.float32)}
    comp, out = run_program(b, feeds, [y])
    assert [p.split()[0] for _, p in comp.groups()] == ["ew_bn_grad_apply_nchw"], comp.groups()
    r = lambda k: feeds[k].reshape(1, c, 1, 1)  # noqa: E731
    f32 = np.float32
    want = (r("t0") * (((feeds["dy"] * f32(cnt)).astype(f32) - r("db")).astype(f32)
                        - (((feeds["x"] - r("mean")).astype(f32) * r("S")).astype(f32) / r("vae")).astype(f32)).astype(f32)).astype(f32)
    assert oracle.max_ulp(out[str(y)], want) == 0


def test_program_replayed_as_one_cuda_graph(oracle):
    """batch_norm_train at a small shape is nine launches, seven of them on [C]-sized vectors: replayed from one CUDA
    graph it gives the same bits, and costs less host time than nine launches."""
    import torch
    rng = np.random.default_rng(98)
    shape, c = (4, 16, 14, 14), 16
    b = NetBuilder("graph")
    x = b.create_input(common.Float(32), shape, "x")
    ps = [b.create_input(common.Float(32), (c,), nm) for nm in ("scale", "bias", "mm", "mv")]
    outs = b.batchnorm(x, *ps, is_test=False)
    feeds = {"x": rng.standard_normal(shape).astype(np.float32), "scale": np.ones(c, np.float32),
             "bias": np.zeros(c, np.float32), "mm": np.zeros(c, np.float32), "mv": np.ones(c, np.float32)}
    comp, want = run_program(b, feeds, outs)
    stream = torch.cuda.Stream()
    for _ in range(3):   # capture, then two replays
        comp.get_tensor("x").from_numpy(feeds["x"] * 0 + 7, TARGET)   # clobber, then restore: results must be recomputed
        comp.execute_graph(stream.cuda_stream)
        stream.synchronize()
        comp.get_tensor("x").from_numpy(feeds["x"], TARGET)
        comp.execute_graph(stream.cuda_stream)
        stream.synchronize()
        for o in outs:
            assert np.array_equal(comp.get_tensor(str(o)).numpy(TARGET), want[str(o)]), str(o)
    plain, graph = comp.execute_test(300), comp.execute_test(300, use_graph=True)
    print("batch_norm_train %s: %.1f us per run launch by launch, %.1f us replayed from one CUDA graph" % (shape, plain * 1e3, graph * 1e3))
    assert graph < plain


# ---- program passes, run ---------------------------------------------------------------------------------------------
def test_default_passes_on_a_float16_program(oracle):
    """Default pass list on a 16-bit program: exp and reduce_sum computed in float32 (AutoCast), the bias
    broadcast explicitly (AutoBroadcast), the dead branch gone; the result equals the oracle's evaluation of the
    rewritten program and stays within 1e-2 of an exact evaluation."""
    rng = np.random.default_rng(11)
    X = rng.standard_normal((256, 2048)).astype(np.float16)
    Bv = (0.1 * rng.standard_normal(2048)).astype(np.float16)
    b = NetBuilder("net")
    x = b.create_input(common.Float(16), X.shape, "X")
    bias = b.create_input(common.Float(16), Bv.shape, "B")
    out = b.reduce_sum(b.exp(b.identity(b.add(x, bias))), [1], False)
    b.tanh(x)  # dead
    got, = b.build_and_get_output(TARGET, [x, bias], [X, Bv], [out])
    ops = [ln.split()[0] for ln in b.program_text().splitlines()]
    # the float32 -> float16 -> float32 pair between exp and reduce_sum is collapsed away (CastCollapsing)
    assert ops == ["broadcast_to", "elementwise_add", "cast", "exp", "reduce_sum", "cast"]
    comp = Computation.build_and_compile(TARGET, b, fetch=[str(out)])
    ref = oracle_program(comp, {"X": X, "B": Bv})[str(out)]
    assert got.dtype == np.float16 and got.shape == (256,)
    np.testing.assert_allclose(got.astype(np.float64), ref.astype(np.float64), rtol=1e-2)
    exact = np.exp((X + Bv).astype(np.float64)).sum(axis=1)
    np.testing.assert_allclose(got.astype(np.float64), exact, rtol=1e-2)


def test_cast_collapsing_changes_the_result_like_the_reference():
    """cast(cast(x, int32), float32) is x itself after CastCollapsing (cast_collapsing_test.cc:90-109): the truncation
    disappears, exactly as in the reference."""
    rng = np.random.default_rng(12)
    X = rng.uniform(-9, 9, (64, 333)).astype(np.float32)

    def build():
        b = NetBuilder("net")
        x = b.create_input(common.Float(32), X.shape, "X")
        t = b.cast(b.cast(x, "int32"), "float32")
        return b, x, b.add(t, t)
    b, x, out = build()
    plain = run_program(b, {"X": X}, [out])[1][str(out)]
    assert np.array_equal(plain, 2 * np.trunc(X))
    b, x, out = build()
    got, = b.build_and_get_output(TARGET, [x], [X], [out], passes=["CastCollapsing"])
    assert np.array_equal(got, X + X)


def test_auto_broadcast_keeps_the_dedicated_kernel_and_its_bits(oracle):
    from cinn_b200 import workloads as W
    w = W.bias_scale_tanh_cast((6, 1000))
    X, Bv = w.inputs

    def build():
        b = NetBuilder("net")
        x = b.create_input(common.Float(32), X.shape, "X")
        bias = b.create_input(common.Float(32), Bv.shape, "bias")
        return b, x, bias, b.cast(b.tanh(b.scale(b.add(x, bias), 0.5, 0.0, True)), "float16")
    b, x, bias, out = build()
    plain = run_program(b, {"X": X, "bias": Bv}, [out])[1][str(out)]
    b, x, bias, out = build()
    got, = b.build_and_get_output(TARGET, [x, bias], [X, Bv], [out], passes=["AutoBroadcast"])
    comp = Computation.build_and_compile(TARGET, b, fetch=[str(out)])
    assert "ew_bias_scale_tanh_cast" in comp.groups()[0][1]
    assert np.array_equal(got.view(np.uint16), plain.view(np.uint16))


# ---- 16-bit batch_norm_train / batch_norm_grad: float32 arithmetic between casts, 16-bit storage -----------------------
def _bind_run(comp, tensors):
    import torch
    for name, t in tensors.items():
        comp.get_tensor(name).bind(t.data_ptr())
    comp.execute()
    torch.cuda.synchronize()


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("shape", [(8, 16, 12, 12), (3, 5, 7, 9), (32, 64, 56, 56)])
def test_sixteen_bit_batch_norm_train(dtype, shape):
    import torch
    torch.manual_seed(71)
    tdt = torch.float16 if dtype == "float16" else torch.bfloat16
    n, c, h, w = shape
    b = NetBuilder("bn_train16")
    x = b.create_input(common.Type(dtype), shape, "x")
    ps = [b.create_input(common.Float(32), (c,), nm) for nm in ("scale", "bias", "moving_mean", "moving_variance")]
    outs = b.batch_norm_train(x, *ps, epsilon=1e-5, momentum=0.9)
    comp = Computation.build_and_compile(TARGET, b, fetch=[str(o) for o in outs])
    pats = [p for _, p in comp.groups()]
    short = "f16" if dtype == "float16" else "bf16"
    assert "channel_stats mid_keep_reduce_sum_sumsq_" + short in pats and "ew_bn_train_apply_nchw ew_bn_train_apply_nchw_" + short in pats, pats
    dev = "cuda:0"
    t = {"x": (torch.randn(shape, device=dev) * 2 + 0.5).to(tdt),
         "scale": 1 + 0.1 * torch.randn(c, device=dev), "bias": 0.1 * torch.randn(c, device=dev),
         "moving_mean": 0.1 * torch.randn(c, device=dev), "moving_variance": torch.rand(c, device=dev) + 0.5}
    y = torch.empty(shape, dtype=tdt, device=dev)
    stats = [torch.empty(c, dtype=torch.float32, device=dev) for _ in range(4)]
    _bind_run(comp, {**t, str(outs[0]): y, **{str(o): s for o, s in zip(outs[1:], stats)}})
    x64 = t["x"].double()
    m = x64.mean(dim=(0, 2, 3))
    v = (x64 * x64).mean(dim=(0, 2, 3)) - m * m
    r = lambda a: a.double().reshape(1, c, 1, 1)  # noqa: E731
    want = (x64 - r(m)) / torch.sqrt(r(v) + 1e-5) * r(t["scale"]) + r(t["bias"])
    assert torch.allclose(stats[0].double(), m, rtol=1e-5, atol=1e-6)
    assert torch.allclose(stats[1].double(), v, rtol=1e-4, atol=1e-5)
    assert torch.allclose(stats[2].double(), 0.9 * t["moving_mean"].double() + 0.1 * m, rtol=1e-5, atol=1e-6)
    assert torch.allclose(stats[3].double(), 0.9 * t["moving_variance"].double() + 0.1 * v, rtol=1e-4, atol=1e-5)
    assert bool(((y.double() - want).abs() <= 1e-2 * want.abs() + 1e-2).all()), float((y.double() - want).abs().max())


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("shape", [(8, 16, 12, 12), (3, 5, 7, 9), (32, 64, 56, 56)])
def test_sixteen_bit_batch_norm_grad(dtype, shape):
    import torch
    torch.manual_seed(72)
    tdt = torch.float16 if dtype == "float16" else torch.bfloat16
    n, c, h, w = shape
    b = NetBuilder("bn_grad16")
    dy, x = b.create_input(common.Type(dtype), shape, "dy"), b.create_input(common.Type(dtype), shape, "x")
    scale, mean, var = (b.create_input(common.Float(32), (c,), nm) for nm in ("scale", "mean", "var"))
    outs = b.batch_norm_grad(dy, x, scale, mean, var, epsilon=1e-5)
    comp = Computation.build_and_compile(TARGET, b, fetch=[str(o) for o in outs])
    pats = [p for _, p in comp.groups()]
    short = "f16" if dtype == "float16" else "bf16"
    assert len(pats) == 3 and pats[0] == "bn_grad_stats bn_grad_stats_" + short, pats
    assert is_chain_kernel(pats[1].split()[1], "ew_chain_f32_s1"), pats
    assert pats[2] == "ew_bn_grad_apply_nchw ew_bn_grad_apply_nchw_" + short, pats
    dev = "cuda:0"
    X = (torch.randn(shape, device=dev) * 1.5 + 0.3).to(tdt)
    t = {"dy": torch.randn(shape, device=dev).to(tdt), "x": X, "scale": 1 + 0.1 * torch.randn(c, device=dev),
         "mean": X.float().mean(dim=(0, 2, 3)), "var": X.float().var(dim=(0, 2, 3), unbiased=False)}
    dx = torch.empty(shape, dtype=tdt, device=dev)
    dscale, dbias = (torch.empty(c, dtype=torch.float32, device=dev) for _ in range(2))
    _bind_run(comp, {**t, str(outs[0]): dx, str(outs[1]): dscale, str(outs[2]): dbias})
    d = {k: v_.double() for k, v_ in t.items()}
    m, v, s = (d[k].reshape(1, c, 1, 1) for k in ("mean", "var", "scale"))
    cnt = n * h * w
    db = d["dy"].sum(dim=(0, 2, 3))
    S = (d["dy"] * (d["x"] - m)).sum(dim=(0, 2, 3))
    inv = 1 / torch.sqrt(v + 1e-5)
    want = (s * inv / cnt) * ((d["dy"] * cnt - db.reshape(1, c, 1, 1)) - (d["x"] - m) * S.reshape(1, c, 1, 1) / (v + 1e-5))
    assert bool(((dbias.double() - db).abs() <= 1e-5 * d["dy"].abs().sum(dim=(0, 2, 3)) + 1e-6).all())
    assert bool(((dscale.double() - S * inv.reshape(-1)).abs()
                 <= 3e-5 * (d["dy"] * (d["x"] - m)).abs().sum(dim=(0, 2, 3)) * inv.reshape(-1) + 1e-6).all())
    assert bool(((dx.double() - want).abs() <= 1e-2 * want.abs() + 1e-2 * want.abs().max()).all())


# ---- elementwise groups with two outputs: a value on the way is stored as well ------------------------------------
@pytest.mark.parametrize("shape", [(64, 1024), (33, 1001), (1024, 4096)])
def test_pre_activation_and_activation_from_one_kernel(oracle, shape):
    rng = np.random.default_rng(81)
    feeds = {"X": rng.standard_normal(shape).astype(np.float32), "B": rng.standard_normal(shape[-1]).astype(np.float32)}
    b = NetBuilder("two_out")
    x = b.create_input(common.Float(32), shape, "X")
    bias = b.create_input(common.Float(32), (shape[-1],), "B")
    pre = b.add(x, bias)
    act = b.sigmoid(b.relu(pre))
    comp = Computation.build_and_compile(TARGET, b, fetch=[str(pre), str(act)])
    assert one_chain_group(comp, "ew_chain_f32_s1o"), comp.groups()
    for name, arr in feeds.items():
        comp.get_tensor(name).from_numpy(arr, TARGET)
    comp.execute()
    ref = oracle_program(comp, feeds)
    assert oracle.max_ulp(comp.get_tensor(str(pre)).numpy(TARGET), ref[str(pre)]) == 0
    assert oracle.max_ulp(comp.get_tensor(str(act)).numpy(TARGET), ref[str(act)]) <= 2


def test_second_output_of_another_type_and_no_contraction_across_it(oracle):
    """A stored product is read back by the add in the reference (an output node is not inlined), so no fused
    multiply-add there; the second output may be a bool or a 16-bit value."""
    rng = np.random.default_rng(82)
    shape = (128, 1000)
    feeds = {n: rng.standard_normal(shape).astype(np.float32) for n in "ABC"}
    b = NetBuilder("two_out")
    A, B, C = (b.create_input(common.Float(32), shape, n) for n in "ABC")
    prod = b.multiply(A, B)
    total = b.add(prod, C)
    comp, got = run_program_fetch(b, feeds, [prod, total])
    assert one_chain_group(comp, "ew_chain_f32_s3o"), comp.groups()
    assert np.array_equal(got[str(prod)], feeds["A"] * feeds["B"])
    assert np.array_equal(got[str(total)], feeds["A"] * feeds["B"] + feeds["C"])  # rounded product, then the add
    b = NetBuilder("two_out")
    A, B, C = (b.create_input(common.Float(32), shape, n) for n in "ABC")
    mask = b.greater_than(A, B)
    half = b.cast(b.select(mask, A, C), "float16")
    comp, got = run_program_fetch(b, feeds, [mask, half])
    assert len(comp.groups()) == 1 and "s3o" in comp.groups()[0][1], comp.groups()
    assert np.array_equal(got[str(mask)], feeds["A"] > feeds["B"])
    want = np.where(feeds["A"] > feeds["B"], feeds["A"], feeds["C"]).astype(np.float16)
    assert np.array_equal(got[str(half)].view(np.uint16), want.view(np.uint16))


def test_value_with_two_consumers_is_computed_once(oracle):
    rng = np.random.default_rng(83)
    X = rng.standard_normal((256, 2048)).astype(np.float32)
    b = NetBuilder("fanout")
    x = b.create_input(common.Float(32), X.shape, "X")
    e = b.exp(x)
    s = b.reduce_sum(e, [1])
    y = b.sqrt(b.scale(e, 2.0, 0.0, True))
    comp, got = run_program_fetch(b, {"X": X}, [s, y])
    assert len(comp.groups()) == 2, comp.groups()
    ref = oracle_program(comp, {"X": X})
    assert oracle.max_ulp(got[str(y)], ref[str(y)]) <= 2
    exact = np.exp(X.astype(np.float64)).sum(axis=1)
    assert np.allclose(got[str(s)], exact, rtol=1e-5)


@pytest.mark.parametrize("shape", [(64, 1024), (33, 1001), (1024, 4096)])
def test_sibling_expressions_share_one_kernel(oracle, shape):
    """Two expressions over the same inputs, neither on the way to the other: horizontal fusion."""
    rng = np.random.default_rng(84)
    feeds = {"X": rng.standard_normal(shape).astype(np.float32), "B": rng.standard_normal(shape[-1]).astype(np.float32)}
    b = NetBuilder("siblings")
    x = b.create_input(common.Float(32), shape, "X")
    bias = b.create_input(common.Float(32), (shape[-1],), "B")
    y1 = b.relu(b.add(x, bias))
    y2 = b.multiply(b.subtract(x, bias), bias)
    comp, got = run_program_fetch(b, feeds, [y1, y2])
    assert len(comp.groups()) == 1 and ("ew_chain_f32_s" in comp.groups()[0][1] or "ew_static_" in comp.groups()[0][1]), comp.groups()
    ref = oracle_program(comp, feeds)
    assert oracle.max_ulp(got[str(y1)], ref[str(y1)]) == 0 and oracle.max_ulp(got[str(y2)], ref[str(y2)]) == 0
    # a shared prefix is evaluated for each output; the results are the same bits
    b = NetBuilder("siblings_prefix")
    x = b.create_input(common.Float(32), shape, "X")
    t = b.sqrt(b.abs(x))
    z1, z2 = b.relu(b.negative(t)), b.scale(t, 3.0, 1.0, True)
    comp, got = run_program_fetch(b, {"X": feeds["X"]}, [z1, z2])
    assert len(comp.groups()) == 1, comp.groups()
    ref = oracle_program(comp, {"X": feeds["X"]})
    assert oracle.max_ulp(got[str(z1)], ref[str(z1)]) == 0 and oracle.max_ulp(got[str(z2)], ref[str(z2)]) == 0


@pytest.mark.parametrize("dtype", ["float16", "bfloat16", "float32"])
def test_batch_norm_relu_after_the_default_passes(dtype):
    """relu(batch_norm(x)) rewritten by AutoCast + Decomposer (+ the rest of the default list): the decomposed
    arithmetic ((x - mean) * rsqrt(var + eps)) * scale + bias between casts, relu after the narrowing cast; still one
    dedicated kernel."""
    import torch
    torch.manual_seed(73)
    tdt = {"float16": torch.float16, "bfloat16": torch.bfloat16, "float32": torch.float32}[dtype]
    shape, c = (8, 16, 28, 28), 16
    b = NetBuilder("bn_relu_passes")
    x = b.create_input(common.Type(dtype), shape, "x")
    ps = [b.create_input(common.Float(32), (c,), nm) for nm in ("scale", "bias", "mean", "variance")]
    y = b.relu(b.batch_norm(x, *ps, epsilon=1e-5, is_test=True))
    assert b.apply_pass([y]) == 1
    comp = Computation.build_and_compile(TARGET, b, fetch=[str(y)])
    short = {"float16": "f16", "bfloat16": "bf16", "float32": "f32"}[dtype]
    assert [p for _, p in comp.groups()] == ["ew_bn_train_apply_relu_nchw ew_bn_train_apply_relu_nchw_" + short]
    dev = "cuda:0"
    t = {"x": torch.randn(shape, device=dev).to(tdt), "scale": 1 + 0.1 * torch.randn(c, device=dev),
         "bias": 0.1 * torch.randn(c, device=dev), "mean": 0.1 * torch.randn(c, device=dev),
         "variance": torch.rand(c, device=dev) + 0.5}
    out = torch.empty(shape, dtype=tdt, device=dev)
    _bind_run(comp, {**t, str(y): out})
    r = lambda a: a.double().reshape(1, c, 1, 1)  # noqa: E731
    want = torch.relu((t["x"].double() - r(t["mean"])) / torch.sqrt(r(t["variance"]) + 1e-5) * r(t["scale"]) + r(t["bias"]))
    tol = 1e-5 if dtype == "float32" else 1e-2
    assert bool(((out.double() - want).abs() <= tol * want.abs() + tol).all())


def test_compositions_between_other_ops(oracle):
    """op -> layer_norm -> op and gelu -> max-subtracted softmax -> relu: three kernels each, results as the oracle's
    evaluation of those groups."""
    rng = np.random.default_rng(85)
    X = rng.standard_normal((128, 2048)).astype(np.float32)
    G = (1 + 0.02 * rng.standard_normal(2048)).astype(np.float32)
    Bt = (0.02 * rng.standard_normal(2048)).astype(np.float32)
    b = NetBuilder("mid")
    x = b.create_input(common.Float(32), X.shape, "X")
    g, be = b.create_input(common.Float(32), (2048,), "G"), b.create_input(common.Float(32), (2048,), "Bt")
    y = b.tanh(b.layer_norm(b.relu(b.scale(x, 2.0, 1.0)), g, be))
    feeds = {"X": X, "G": G, "Bt": Bt}
    comp, out = run_program(b, feeds, [y])
    assert [p.split()[0] for _, p in comp.groups()] == ["ew_chain", "layernorm_row", "ew_chain"]
    ref = oracle_program(comp, feeds)[str(y)]
    bad, worst = oracle.count_not_close(out[str(y)], ref, 1e-4, 1e-5)
    assert bad == 0, (bad, worst)
    b = NetBuilder("mid2")
    x = b.create_input(common.Float(32), X.shape, "X")
    y = b.relu(b.softmax(b.gelu(x), (-1,), "safe"))
    comp, out = run_program(b, {"X": X}, [y])
    assert [p.split()[0] for _, p in comp.groups()] == ["ew_chain", "softmax_safe_row", "ew_chain"]
    ref = oracle_program(comp, {"X": X})[str(y)]
    bad, worst = oracle.count_not_close(out[str(y)], ref, 1e-5, 1e-9)
    assert bad == 0, (bad, worst)
    assert np.allclose(out[str(y)].sum(axis=1), 1.0, rtol=1e-5)


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_sixteen_bit_gelu_and_max_subtracted_softmax(dtype):
    """The builder's gelu and softmax(mode != "fast") on 16-bit tensors: float32 arithmetic between casts."""
    import torch
    torch.manual_seed(74)
    tdt = torch.float16 if dtype == "float16" else torch.bfloat16
    shape = (96, 2048)
    b = NetBuilder("half_acts")
    x = b.create_input(common.Type(dtype), shape, "X")
    y, z = b.gelu(x), b.softmax(x, (-1,), "safe")
    comp = Computation.build_and_compile(TARGET, b, fetch=[str(y), str(z)])
    short = "f16" if dtype == "float16" else "bf16"
    kernels = sorted(p.split()[1] for _, p in comp.groups())
    assert len(kernels) == 2 and kernels[1].startswith("softmax_safe_" + short), kernels
    assert kernels[0].startswith("ew_chain_" + short) or kernels[0].startswith("ew_static_"), kernels
    xt = (torch.randn(shape, device="cuda:0") * 1.5).to(tdt)
    yt, zt = (torch.empty(shape, dtype=tdt, device="cuda:0") for _ in range(2))
    _bind_run(comp, {"X": xt, str(y): yt, str(z): zt})
    x64 = xt.double()
    want_y = x64 * 0.5 * (1 + torch.erf(x64 * (0.5 ** 0.5)))
    want_z = torch.softmax(x64, dim=1)
    assert bool(((yt.double() - want_y).abs() <= 1e-2 * want_y.abs() + 1e-3).all())
    assert bool(((zt.double() - want_z).abs() <= 1e-2 * want_z + 1e-7).all())


@pytest.mark.parametrize("bits", [32, 64])
def test_integer_trees_are_one_kernel_and_bit_exact(bits):
    rng = np.random.default_rng(86)
    npt = np.int32 if bits == 32 else np.int64
    shape = (129, 1000)
    feeds = {n: rng.integers(-1000, 1000, shape).astype(npt) for n in "ABC"}
    b = NetBuilder("int_tree")
    A, B, C = (b.create_input(common.Int(bits), shape, n) for n in "ABC")
    out = b.subtract(b.multiply(b.add(A, B), b.max(A, C)), b.bitwise_and(B, C))   # two joins, three tensors
    comp, got = run_program_fetch(b, feeds, [out])
    assert [p for _, p in comp.groups()] == ["ew_chain ew_chain_int_i%d_i%d_s3t" % (bits, bits)], comp.groups()
    f = feeds
    want = ((f["A"] + f["B"]) * np.maximum(f["A"], f["C"]) - (f["B"] & f["C"])).astype(npt)
    assert np.array_equal(got[str(out)], want)


def test_float64_trees_are_one_kernel(oracle):
    rng = np.random.default_rng(87)
    shape = (129, 1000)
    feeds = {n: rng.standard_normal(shape) for n in "ABCD"}
    b = NetBuilder("f64_tree")
    A, B, C, D = (b.create_input(common.Float(64), shape, n) for n in "ABCD")
    out = b.add(b.multiply(A, B), b.multiply(C, D))        # fma(C, D, A * B) in double
    comp, got = run_program_fetch(b, feeds, [out])
    assert [p for _, p in comp.groups()] == ["ew_chain ew_chain_f64_f64_s3t"], comp.groups()
    ref = oracle_program(comp, feeds)[str(out)]
    assert np.array_equal(got[str(out)], ref)
    b = NetBuilder("f64_tree2")
    A, B, C, D = (b.create_input(common.Float(64), shape, n) for n in "ABCD")
    out = b.divide(b.subtract(A, B), b.add(b.abs(C), b.abs(D)))
    comp, got = run_program_fetch(b, feeds, [out])
    assert len(comp.groups()) == 1 and "s3t" in comp.groups()[0][1], comp.groups()
    f = feeds
    assert np.array_equal(got[str(out)], (f["A"] - f["B"]) / (np.abs(f["C"]) + np.abs(f["D"])))


def test_cast_and_squeeze_relations_of_the_reference_api_tests():
    """cinn/frontend/net_builder_test.cc:441-491 (cast int32 -> float32: out == (float)in) and :493-783 (squeeze over
    {1}, {-3}, {1, 3}, {1, -1}, {}: out == in with the extent-1 axes dropped), run on the GPU."""
    rng = np.random.default_rng(10)
    b = NetBuilder("net_builder")
    x = b.create_input(common.Int(32), (4, 7), "In")
    y = b.cast(x, "float32")
    X = rng.integers(-2**31, 2**31 - 1, (4, 7), dtype=np.int64).astype(np.int32)
    comp, got = run_program(b, {"In": X}, [y])
    assert got[str(y)].dtype == np.float32 and np.array_equal(got[str(y)], X.astype(np.float32))
    X = rng.standard_normal((4, 1, 7, 1)).astype(np.float32)
    for axes, want in (([1], (4, 7, 1)), ([-3], (4, 7, 1)), ([1, 3], (4, 7)), ([1, -1], (4, 7)), ([], (4, 7))):
        b = NetBuilder("net_builder")
        out = b.squeeze(b.create_input(common.Float(32), (4, 1, 7, 1), "In"), axes)
        comp, got = run_program_fetch(b, {"In": X}, [out])
        assert got[str(out)].shape == want and np.array_equal(got[str(out)].reshape(-1), X.reshape(-1)), axes
