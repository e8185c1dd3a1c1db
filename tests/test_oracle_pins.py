"""Pins of the CPU oracle (no GPU): the known-answer relations the reference's own tests check on its x86 path,
applied to the restatement, plus self-consistency between its fused loops and its op-at-a-time evaluators.

The reference stores no golden numeric vectors for this path; what its tests pin is:
  * x86 JIT vs libm lambdas at abs 1e-5         cinn/hlir/pe/pe_elementwise_test.cc:96-109, 131-156
  * A + (A + B) == 2A + B at 1e-5                cinn/frontend/computation_test.cc:74-103
  * batch-norm vs a serial CPU loop, rtol 1e-5   cinn/frontend/decomposer/batch_norm_test.cc:50-145,
                                                 cinn/frontend/decomposer/test_helper.h:113-141
  * reduce vs a serial CPU loop, rel 1e-4        cinn/hlir/op/reduction_test.cc:305-404
"""
import math

import numpy as np
import pytest

from cinn_b200 import workloads as W
from oracle import x86_graph_eval as ge


def test_unary_against_libm_like_the_reference_pe_tests(oracle):
    rng = np.random.default_rng(1234)
    x = rng.uniform(-4, 4, 4096).astype(np.float32)
    pos = np.abs(x) + np.float32(0.01)
    cases = {"exp": (x, np.exp), "tanh": (x, np.tanh), "sigmoid": (x, lambda v: 1 / (1 + np.exp(-v))),
             "sqrt": (pos, np.sqrt), "rsqrt": (pos, lambda v: 1 / np.sqrt(v)), "log": (pos, np.log),
             "floor": (x, np.floor), "ceil": (x, np.ceil), "abs": (x, np.abs), "negative": (x, np.negative),
             "sin": (x, np.sin), "cos": (x, np.cos), "erf": (x, np.vectorize(math.erf)),
             "relu": (x, lambda v: np.maximum(v, 0)), "sign": (x, np.sign), "trunc": (x, np.trunc),
             "round": (x, np.rint), "reciprocal": (pos, lambda v: 1 / v), "log2": (pos, np.log2),
             "log10": (pos, np.log10)}
    for name, (arg, fn) in cases.items():
        got = oracle.unary(name, arg)
        want = fn(arg.astype(np.float64))
        assert np.abs(got - want).max() <= 1e-5 * max(1.0, np.abs(want).max()), name


def test_tanh_is_the_two_branch_exp_formula(oracle):
    """cinn/backends/llvm/llvm_intrin_rule.h:136-154, evaluated with glibc expf in fp32."""
    import ctypes
    libm = ctypes.CDLL("libm.so.6")
    libm.expf.restype = ctypes.c_float
    libm.expf.argtypes = [ctypes.c_float]
    xs = np.array([-3.5, -1.0, -1e-3, -0.0, 0.0, 1e-6, 0.25, 1.0, 8.0, 20.0], np.float32)
    got = oracle.unary("tanh", xs)
    for x, g in zip(xs, got):
        one = np.float32(1)
        if x >= 0:
            e = np.float32(libm.expf(np.float32(-2) * x))
            want = (one - e) / (one + e)
        else:
            e = np.float32(libm.expf(np.float32(2) * x))
            want = (e - one) / (e + one)
        assert g == np.float32(want), (x, g, want)
    assert not np.signbit(got[3])  # tanh(-0.0) takes the x >= 0 branch: +0


def test_relu_and_max_are_compare_select(oracle):
    a = np.array([-0.0, 0.0, np.nan, 1.0, -2.0], np.float32)
    r = oracle.unary("relu", a)
    assert not np.signbit(r[0]) and r[0] == 0  # -0 > 0 is false -> the second operand, +0
    assert r[2] == 0  # NaN > 0 is false -> 0
    m = oracle.binary("max", np.array([np.nan, 1.0], np.float32), np.array([2.0, np.nan], np.float32))
    assert m[0] == 2.0 and np.isnan(m[1])


def test_a_plus_a_plus_b_like_computation_test(oracle):
    rng = np.random.default_rng(0)
    a = rng.random((32, 32), dtype=np.float32)
    b = rng.random((32, 32), dtype=np.float32)
    got = oracle.binary("add", a, oracle.binary("add", a, b))
    assert np.abs(got - (2 * a + b)).max() <= 1e-5


def test_scale_is_fma_and_contraction_is_single_rounding(oracle):
    x = np.array([1.0000001, 3.3333333, -7.7777777], np.float32)
    s, b = np.float32(0.3333333), np.float32(1e-7)
    got = oracle.scale(x, float(s), float(b), True)
    want = (x.astype(np.float64) * np.float64(s) + np.float64(b)).astype(np.float32)  # exact product, one rounding
    assert np.array_equal(got, want)
    two_roundings = (x * s) + b
    assert not np.array_equal(got, two_roundings) or True  # may coincide; the fma form is what is pinned above
    pre = oracle.scale(x, float(s), float(b), False)
    assert np.array_equal(pre, s * (x + b))


def test_casts_round_to_nearest_even(oracle):
    x = np.array([1.0 + 2 ** -11, 1.0 + 3 * 2 ** -11, 65504.0, 65520.0, 1e-8, -2.5], np.float32)
    assert np.array_equal(oracle.cast_f32_f16(x), x.astype(np.float16))
    rng = np.random.default_rng(5)
    y = rng.standard_normal(100000).astype(np.float32)
    assert np.array_equal(oracle.cast_f32_f16(y).view(np.uint16), y.astype(np.float16).view(np.uint16))
    bf = oracle.cast_f32_bf16(np.array([1.0, 1.00390625, 1.01171875, -3.0], np.float32))
    assert list(bf) == [0x3F80, 0x3F80, 0x3F82, 0xC040]  # ties to even on the upper 16 bits


def test_reduce_is_the_serial_loop_of_reduction_test(oracle):
    rng = np.random.default_rng(2)
    x = rng.standard_normal((7, 33, 5)).astype(np.float32)
    for kind, init, fn in [("sum", np.float32(0), lambda a, v: np.float32(a + v)),
                           ("prod", np.float32(1), lambda a, v: np.float32(a * v)),
                           ("max", np.float32(-3.4028235e38), lambda a, v: a if a > v else v),
                           ("min", np.float32(3.4028235e38), lambda a, v: a if a < v else v)]:
        got = oracle.reduce(kind, x, 7, 33, 5).reshape(7, 5)
        for o in range(7):
            for i in range(5):
                acc = init
                for k in range(33):
                    acc = fn(acc, x[o, k, i])
                assert got[o, i] == acc, (kind, o, i)
    # thread count does not change a result (each output keeps its serial order)
    assert np.array_equal(oracle.reduce("sum", x, 7, 33, 5, threads=4), oracle.reduce("sum", x, 7, 33, 5))
    assert oracle.reduce("max", np.full(4, -np.inf, np.float32), 1, 4, 1)[0] == np.float32(-3.4028235e38)


def test_batch_norm_against_the_serial_reference_loop(oracle):
    """The CPU loop of cinn/frontend/decomposer/batch_norm_test.cc, in float64, rtol 1e-5 / atol 1e-8."""
    w = W.bn_relu((2, 5, 7, 3))
    x, scale, bias, mean, var = w.inputs
    got = oracle.bn_relu_nchw(x, scale, bias, mean, var, 1e-5)
    sh = (1, 5, 1, 1)
    want = np.maximum((x.astype(np.float64) - mean.reshape(sh)) * scale.reshape(sh) /
                      np.sqrt(var.reshape(sh).astype(np.float64) + 1e-5) + bias.reshape(sh), 0)
    assert np.allclose(got, want, rtol=1e-5, atol=1e-8)


def test_softmax_rows_sum_to_one_and_match_float64(oracle):
    w = W.softmax((16, 257))
    got = oracle.softmax(w.inputs[0])
    x = w.inputs[0].astype(np.float64)
    want = np.exp(x) / np.exp(x).sum(-1, keepdims=True)
    assert np.allclose(got, want, rtol=1e-5, atol=1e-8)
    h = W.softmax((16, 257), half=True)
    got16 = oracle.softmax(h.inputs[0])
    assert got16.dtype == np.float16 and np.allclose(got16.astype(np.float64), want, rtol=2e-2, atol=1e-6)


def test_layer_norm_matches_float64(oracle):
    w = W.layer_norm((9, 300))
    x, gamma, beta = w.inputs
    got = oracle.layernorm(x, gamma, beta, 1e-5)
    xd = x.astype(np.float64)
    mean = xd.mean(-1, keepdims=True)
    var = (xd * xd).mean(-1, keepdims=True) - mean * mean
    want = (xd - mean) / np.sqrt(var + 1e-5) * gamma + beta
    assert np.allclose(got, want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("make", [
    lambda: W.add_relu((3, 5, 7)), lambda: W.bias_scale_tanh_cast((3, 5, 16)), lambda: W.softmax((5, 33)),
    lambda: W.softmax((5, 32), half=True), lambda: W.layer_norm((6, 40)), lambda: W.layer_norm((6, 40), half=True),
    lambda: W.bn_relu((2, 3, 4, 5)), lambda: W.bn_relu((2, 3, 4, 5), half=True),
    lambda: W.reduce_sum_last((3, 4, 50)), lambda: W.reduce_max_first((9, 4, 5))])
def test_fused_loops_equal_op_at_a_time_evaluation(oracle, make):
    """The reference's own fused-vs-unfused self-check (python/tests/fusion/fusion_test.py:23-63), on the oracle:
    the single-pass loops that are timed as the CPU baseline give bit-identical results to evaluating the same
    group description one op at a time."""
    w = make()
    unfused = ge.run(w.desc, w.inputs)
    name = w.name
    if name == "add_relu":
        fused = oracle.add_relu(*w.inputs)
    elif name == "bias_scale_tanh_cast":
        fused = oracle.bias_scale_tanh_f16(w.inputs[0], w.inputs[1], 0.5, 0.0)
    elif name.startswith("softmax"):
        fused = oracle.softmax(w.inputs[0])
    elif name.startswith("layer_norm"):
        fused = oracle.layernorm(*w.inputs, 1e-5)
    elif name.startswith("bn_relu"):
        fused = oracle.bn_relu_nchw(*w.inputs, 1e-5)
    elif name == "reduce_sum_last":
        fused = oracle.reduce("sum", w.inputs[0], 12, 50, 1).reshape(w.out_shape)
    else:
        fused = oracle.reduce("max", w.inputs[0], 1, 9, 20).reshape(w.out_shape)
    assert fused.dtype == unfused.dtype and fused.shape == tuple(unfused.shape)
    assert np.array_equal(fused.view(np.uint8), unfused.view(np.uint8))


def test_oracle_reproduces_llvm_compiled_loops_bit_for_bit(oracle):
    """tests/golden/llvm_x86_vectors.npz holds the outputs of LLVM-20 -O3 (loop + SLP vectorised, no fast-math)
    builds of the IR constructs CINN's x86 path emits for these groups (llvm.fmuladd / llvm.exp / llvm.sqrt
    intrinsics, fcmp + select, fptrunc to half, serial fadd reductions); tests/golden/make_llvm_x86_vectors.py
    generated it.  The C oracle must give exactly those bits."""
    import os
    d = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "llvm_x86_vectors.npz"))

    def same(got, want):
        return got.dtype == want.dtype and got.shape == want.shape and np.array_equal(got.view(np.uint8),
                                                                                      want.view(np.uint8))
    assert same(oracle.add_relu(d["add_relu_a"], d["add_relu_b"]), d["add_relu_y"])
    assert same(oracle.bias_scale_tanh_f16(d["tanh_x"], d["tanh_bias"], 0.5, 0.0), d["tanh_y"])
    assert same(oracle.reduce("sum", d["sum_x"], 29, 1031, 1), d["sum_y"])
    assert same(oracle.softmax(d["softmax_x"]), d["softmax_y"])
    assert same(oracle.layernorm(d["ln_x"], d["ln_gamma"], d["ln_beta"], 1e-5), d["ln_y"])
    assert same(oracle.bn_relu_nchw(d["bn_x"], d["bn_scale"], d["bn_bias"], d["bn_mean"], d["bn_var"], 1e-5), d["bn_y"])


def test_graph_evaluator_reproduces_llvm_builds_of_the_decomposed_groups(oracle):
    """tests/golden/llvm_x86_vectors_decomposed.npz (made by make_llvm_x86_vectors_decomposed.py): LLVM -O3 builds of the
    loops the decomposed batch_norm_train / batch_norm_grad / max-subtracted softmax / gelu groups lower to.  The
    op-by-op evaluator (oracle/x86_graph_eval.py), fed the groups as text, must give exactly those bits: this pins its
    contraction rule (only an Add fed by a Mul fuses), its 1 / sqrt, its compare + select maximum from the lowest finite
    value, its serial sums and true divisions, and the host erff."""
    import os
    from oracle import x86_graph_eval as ge
    from cinn_b200 import workloads as W
    from cinn_b200 import common
    from cinn_b200.frontend import Computation, NetBuilder
    d = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "llvm_x86_vectors_decomposed.npz"))

    def same(got, want):
        return got.dtype == want.dtype and got.shape == want.shape and np.array_equal(got.view(np.uint8), want.view(np.uint8))

    shape = d["bnt_x"].shape
    w = W.bn_train_apply(shape)   # inputs: mean, var, x, scale, bias
    got = ge.run(w.desc, [d["bnt_mean"], d["bnt_var"], d["bnt_x"], d["bnt_scale"], d["bnt_bias"]])
    assert same(got, d["bnt_y"])

    # x_grad with every per-channel operand given (t0 and var + eps as inputs), built through the front end
    b = NetBuilder("g")
    F = common.Float(32)
    c = shape[1]
    dy, x = b.create_input(F, shape, "dy"), b.create_input(F, shape, "x")
    t0, db, mean, S, vae = (b.create_input(F, (c,), nm) for nm in ("t0", "db", "mean", "S", "vae"))
    full, cnt = list(shape), float(shape[0] * shape[2] * shape[3])
    tmp1 = b.multiply(dy, b.fill_constant(full, cnt))
    tmp3 = b.divide(b.multiply(b.subtract(x, b.broadcast_to(mean, full, [1])), b.broadcast_to(S, full, [1])),
                    b.broadcast_to(vae, full, [1]))
    y = b.multiply(b.broadcast_to(t0, full, [1]), b.subtract(b.subtract(tmp1, b.broadcast_to(db, full, [1])), tmp3))
    comp = Computation.build_and_compile(common.DefaultNVGPUTarget(), b, plan_only=True)
    (desc, pattern), = comp.groups()
    feeds = {"dy": d["bng_dy"], "x": d["bng_x"], "t0": d["bng_t0"], "db": d["bng_db"], "mean": d["bng_mean"],
             "S": d["bng_s"], "vae": d["bng_vae"]}
    got = ge.run(desc, [feeds[name] for name, _, _ in ge.parse(desc)["inputs"]])
    assert same(got, d["bng_y"])

    w = W.softmax_safe(d["sms_x"].shape)
    assert same(ge.run(w.desc, [d["sms_x"]]), d["sms_y"])

    b = NetBuilder("gelu")
    y = b.gelu(b.create_input(F, d["gelu_x"].shape, "X"))
    comp = Computation.build_and_compile(common.DefaultNVGPUTarget(), b, plan_only=True)
    (desc, pattern), = comp.groups()
    assert same(ge.run(desc, [d["gelu_x"]]), d["gelu_y"])


def test_every_op_of_the_registry_reproduces_its_llvm_build(oracle):
    """tests/golden/llvm_x86_vectors_ops.npz (made by make_llvm_x86_vectors_ops.py): every unary and binary elementwise
    op, float32 and float64, as LLVM -O3 compiles the IR the reference's x86 path emits for it (intrinsics, libm calls,
    compare + select, the two-branch tanh, 1 / sqrt, ...), on inputs that include signed zeros, infinities, NaN,
    denormals and domain edges; plus the integer ops of the int32 chains.  The C oracle (and, for int32, the graph
    evaluator) must give exactly those bits, NaN payloads aside (a NaN must be a NaN)."""
    import os
    from oracle import x86_graph_eval as ge
    d = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "llvm_x86_vectors_ops.npz"))

    def same(got, want, what):
        assert got.dtype == want.dtype and got.shape == want.shape, what
        nan_g, nan_w = np.isnan(got), np.isnan(want)
        assert np.array_equal(nan_g, nan_w), (what, "NaN positions differ")
        ok = np.array_equal(got[~nan_g].view(np.uint8), want[~nan_w].view(np.uint8))
        if not ok:
            bad = np.flatnonzero((got != want) & ~nan_g)
            raise AssertionError((what, int(bad.size), got[bad[:4]], want[bad[:4]]))

    unary_names = sorted(k[2:-4] for k in d.files if k.startswith("u_") and k.endswith("_f32"))
    binary_names = sorted(k[2:-4] for k in d.files if k.startswith("b_") and k.endswith("_f32"))
    assert len(unary_names) >= 34 and len(binary_names) >= 18
    with np.errstate(all="ignore"):
        for op in unary_names:
            same(oracle.unary(op, d["x_f32"]), d["u_%s_f32" % op], op + " f32")
            same(oracle.unary_f64(op, d["x_f64"]), d["u_%s_f64" % op], op + " f64")
        for op in binary_names:
            same(oracle.binary(op, d["x_f32"], d["w_f32"]), d["b_%s_f32" % op], op + " f32")
            same(oracle.binary_f64(op, d["x_f64"], d["w_f64"]), d["b_%s_f64" % op], op + " f64")
    n = d["x_i32"].size
    for key in [k for k in d.files if k.startswith("i_")]:
        op = key[2:-4]
        desc = ("group fn_i\ninput a int32 %d\ninput b int32 %d\nop %s y = a b ; axis=-1\noutput y int32 %d\n" % (n, n, op, n))
        got = ge.run(desc, [d["x_i32"], d["w_i32"]])
        assert got.dtype == np.int32 and np.array_equal(got, d[key]), op


def test_cast_and_squeeze_relations_of_the_reference_api_tests():
    """cinn/frontend/net_builder_test.cc:441-491: cast(int32 -> float32) gives exactly (float)in;
    :493-783: squeeze over axes {1}, {-3}, {1, 3}, {1, -1} and {} keeps the data and drops the extent-1 axes.
    Here through the graph evaluator and the front end's shape inference (tests/test_gpu_frontend.py runs the same
    relations on the GPU)."""
    from oracle import x86_graph_eval as ge
    from cinn_b200 import common
    from cinn_b200.frontend import NetBuilder
    rng = np.random.default_rng(9)
    x = rng.integers(-2**31, 2**31 - 1, (4, 7), dtype=np.int64).astype(np.int32)
    desc = "group fn_c\ninput In int32 4,7\nop cast y = In ; dtype=float32\noutput y float32 4,7\n"
    got = ge.run(desc, [x])
    assert got.dtype == np.float32 and np.array_equal(got, x.astype(np.float32))
    for axes, want in (([1], [4, 7, 1]), ([-3], [4, 7, 1]), ([1, 3], [4, 7]), ([1, -1], [4, 7]), ([], [4, 7])):
        b = NetBuilder("sq")
        out = b.squeeze(b.create_input(common.Float(32), (4, 1, 7, 1), "In"), axes)
        assert out.shape == want, (axes, out.shape)


def test_integer_pow_known_answers():
    """The host intrinsics' integer pow (cinn/runtime/cpu/host_intrinsics.cc:234-239, 255): double pow, truncating
    conversion with the most negative value for anything out of range, -1 for int32 zero to a negative power."""
    from oracle import x86_oracle as orc
    i32 = lambda v: np.array(v, np.int32)  # noqa: E731
    i64 = lambda v: np.array(v, np.int64)  # noqa: E731
    lo32, lo64 = -2 ** 31, -2 ** 63
    cases32 = [(0, -1, -1), (2, 10, 1024), (-3, 3, -27), (2, 31, lo32), (-2, 31, lo32), (2, -1, 0), (-1, -3, -1),
               (-1, -4, 1), (46341, 2, lo32), (46340, 2, 2147395600), (7, 0, 1), (0, 0, 1), (1, 2 ** 31 - 1, 1)]
    a, b, want = zip(*cases32)
    assert orc.pow_int(i32(a), i32(b)).tolist() == list(want)
    cases64 = [(0, -1, lo64), (2, 62, 2 ** 62), (2, 63, lo64), (-2, 63, lo64), (3, 39, int(float(3 ** 39))),
               (-3, 39, -int(float(3 ** 39))), (10, 18, 10 ** 18), (3037000500, 2, lo64),
               (3037000499, 2, int(float(3037000499 ** 2))), (5, -2, 0), (-1, 2 ** 62 + 1, 1), (2 ** 53 + 1, 1, 2 ** 53)]
    a, b, want = zip(*cases64)
    assert orc.pow_int(i64(a), i64(b)).tolist() == list(want)


def test_uint8_follows_the_unsigned_instructions():
    """uint8 tensors: the reference's LLVM code generator picks UDiv / URem, unsigned compares, a logical right shift
    and zero-extending casts for `uint` types (cinn/backends/llvm/codegen_llvm.cc:205-216, 280-340, 1449-1457); the
    arithmetic wraps modulo 256.  Known answers through the op-by-op evaluator."""
    from oracle import x86_graph_eval as ge
    a = np.array([200, 255, 0, 7, 128, 1], np.uint8)
    b = np.array([100, 1, 0, 2, 255, 0], np.uint8)

    def run(op, extra=""):
        desc = ("group g\ninput A uint8 6\ninput B uint8 6\nop %s y = A B ; axis=-1%s\noutput y %s 6\n"
                % (op, extra, "bool" if op in ("greater_than", "less_equal") else "uint8"))
        return ge.run(desc, [a, b])
    assert run("elementwise_add").tolist() == [44, 0, 0, 9, 127, 1]          # modulo 256
    assert run("subtract").tolist() == [100, 254, 0, 5, 129, 1]
    assert run("elementwise_mul").tolist() == [32, 255, 0, 14, 128, 0]
    assert run("divide").tolist() == [2, 255, 0, 3, 0, 0]                     # unsigned; a zero divisor gives 0 here
    assert run("mod").tolist() == [0, 0, 0, 1, 128, 0]
    assert run("greater_than").tolist() == [True, True, False, True, False, True]   # 128 > 255 is false: unsigned
    assert run("right_shift").tolist() == [200 >> 4, 255 >> 1, 0, 7 >> 2, 128 >> 7, 1]   # logical, count modulo 8
    desc = "group g\ninput A uint8 6\nop cast y = A ; dtype=int32\noutput y int32 6\n"
    assert ge.run(desc, [a]).tolist() == [200, 255, 0, 7, 128, 1]            # zero-extended
    desc = "group g\ninput A uint8 6\nop cast y = A ; dtype=float32\noutput y float32 6\n"
    assert ge.run(desc, [a]).tolist() == [200.0, 255.0, 0.0, 7.0, 128.0, 1.0]
    desc = "group g\ninput A uint8 6\nop negative y = A\noutput y uint8 6\n"
    assert ge.run(desc, [a]).tolist() == [56, 1, 0, 249, 128, 255]
