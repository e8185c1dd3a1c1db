"""Program passes (AutoCast, Decomposer, AutoBroadcast, CastCollapsing, TransposeCollapsing, FillConstantRewriter,
FillConstantFolding, RemoveIdentity, DeadCodeEliminate) on CPU.

The expected instruction-count changes are the ones the reference's own pass tests assert
(cinn/frontend/pass/cast_collapsing_test.cc:28-233, transpose_collapsing_test.cc:77-450, auto_cast_test.cc:29-71,
fill_constant_rewriter_test.cc:20-145, fill_constant_folding_test.cc:40-205: `size before - size after`).
"""
import pytest

from cinn_b200 import frontend as F


def _count(b):
    return len([ln for ln in b.program_text().splitlines() if ln.strip()])


def _ops(b):
    return [ln.split()[0] for ln in b.program_text().splitlines() if ln.strip()]


def _x(b, dtype="float32", shape=(4, 5, 3)):
    return b.create_input(F.Type(dtype), list(shape), "X")


# ---- CastCollapsing: the reference's seven cases --------------------------------------------------------------------
def test_cast_collapsing_two_casts():
    b = F.NetBuilder("net")
    out = b.cast(b.cast(_x(b), "float16"), "float32")
    n = _count(b)
    b.apply_pass([out], None, ["Decomposer", "CastCollapsing"])
    assert n - _count(b) == 1
    assert _ops(b) == ["identity"]  # x -> float32 is useless but fetched


def test_cast_collapsing_three_casts():
    b = F.NetBuilder("net")
    out = b.cast(b.cast(b.cast(_x(b), "int32"), "int64"), "float32")
    n = _count(b)
    b.apply_pass([out], None, ["CastCollapsing"])
    assert n - _count(b) == 2


def test_cast_collapsing_single_useless_cast_is_left_alone():
    b = F.NetBuilder("net")
    out = b.cast(_x(b), "float32")
    b.apply_pass([out], None, ["CastCollapsing"])
    assert _ops(b) == ["cast"]


def test_cast_collapsing_chain_becomes_useless():
    b = F.NetBuilder("net")
    t = b.cast(b.cast(b.cast(_x(b), "int32"), "int64"), "float32")
    out = b.add(t, t)
    n = _count(b)
    b.apply_pass([out], None, ["CastCollapsing"])
    assert n - _count(b) == 3
    assert b.program_text().strip().startswith("elementwise_add") and "= X, X" in b.program_text()


def test_cast_collapsing_with_other_users():
    b = F.NetBuilder("net")
    x = _x(b)
    t1 = b.cast(x, "int32")
    t2 = b.cast(t1, "float32")
    t3 = b.cast(t2, "int32")
    outs = [b.transpose(t, [0, 2, 1]) for t in (t1, t2, t3)]
    n = _count(b)
    b.apply_pass(outs, None, ["CastCollapsing"])
    assert n - _count(b) == 1


def test_cast_collapsing_two_chains():
    b = F.NetBuilder("net")
    x = _x(b)
    t2 = b.cast(b.cast(x, "int32"), "float32")
    out1 = b.reshape(t2, [5, 3, 4])
    b.cast(b.cast(out1, "int32"), "float32")
    out2 = b.transpose(t2, [0, 2, 1])
    n = _count(b)
    b.apply_pass([out1, out2], None, ["CastCollapsing"])
    assert n - _count(b) == 4
    assert sorted(_ops(b)) == ["reshape", "transpose"]


def test_cast_collapsing_parallel_casts_stay():
    b = F.NetBuilder("net")
    x = _x(b)
    out = b.add(b.cast(x, "int32"), b.cast(x, "int32"))
    n = _count(b)
    b.apply_pass([out], None, ["CastCollapsing"])
    assert n - _count(b) == 0


def test_cast_collapsing_vertical_and_parallel():
    b = F.NetBuilder("net")
    x = _x(b)
    out = b.add(b.cast(b.cast(x, "int32"), "float32"), b.cast(x, "float32"))
    n = _count(b)
    b.apply_pass([out], None, ["CastCollapsing"])
    assert n - _count(b) == 3


# ---- AutoCast --------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_auto_cast_exp(dtype):
    b = F.NetBuilder("net")
    out = b.exp(_x(b, dtype))
    n = _count(b)
    b.apply_pass([out], None, ["AutoCast", "Decomposer"])
    assert n - _count(b) == -2
    assert _ops(b) == ["cast", "exp", "cast"]
    assert out.type.name == dtype
    lines = b.program_text().splitlines()
    assert "dtype=float32" in lines[0] and ("dtype=" + dtype) in lines[2] and lines[2].split()[1] == str(out)


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
def test_auto_cast_batch_norm_casts_x_only(dtype):
    b = F.NetBuilder("net")
    x = _x(b, dtype, (8, 16, 14, 14))
    params = [b.create_input(F.Type("float32"), [16], n) for n in ("scale", "bias", "mean", "variance")]
    out = b.batch_norm(x, *params, epsilon=1e-5, is_test=True)
    n = _count(b)
    b.apply_pass([out], None, ["AutoCast"])
    assert n - _count(b) == -2
    assert _ops(b).count("cast") == 2
    b.apply_pass([out], None, ["Decomposer"])   # then the float32 batch_norm goes into primitives between the casts
    assert "batch_norm" not in _ops(b) and _ops(b)[0] == "cast" and _ops(b)[-1] == "cast"
    comp = F.Computation.build_and_compile(None, b, fetch=[str(out)], plan_only=True)
    short = "f16" if dtype == "float16" else "bf16"
    assert [p for _, p in comp.groups()] == ["ew_bn_train_apply_nchw ew_bn_train_apply_nchw_" + short]


def test_auto_cast_leaves_float32_and_unlisted_ops():
    b = F.NetBuilder("net")
    out = b.exp(_x(b))
    h = b.relu(b.create_input(F.Type("float16"), [4, 4], "H"))
    before = b.program_text()
    b.apply_pass([out, h], None, ["AutoCast"])
    assert b.program_text() == before


def test_auto_cast_then_fusion_picks_the_half_storage_reduction():
    b = F.NetBuilder("net")
    x = b.create_input(F.Type("float16"), [64, 4096], "X")
    out = b.reduce_sum(x, [1], False)
    assert b.apply_pass([out], None, ["AutoCast"]) == 1  # cast + reduce_sum + cast: one group


# ---- AutoBroadcast ---------------------------------------------------------------------------------------------------
def test_auto_broadcast_inserts_broadcast_to():
    b = F.NetBuilder("net")
    x = b.create_input(F.Type("float32"), [2, 8, 1024], "X")
    bias = b.create_input(F.Type("float32"), [1024], "B")
    out = b.cast(b.tanh(b.scale(b.add(x, bias), 0.5, 0.0, True)), "float16")
    groups = b.apply_pass([out], None, ["AutoBroadcast"])
    lines = b.program_text().splitlines()
    assert lines[0].startswith("broadcast_to") and "broadcast_axes=2" in lines[0] and "out_shape=2,8,1024" in lines[0]
    assert "axis=-1" in lines[1]
    assert groups == 1
    comp = F.Computation.build_and_compile(None, b, fetch=[str(out)], plan_only=True)
    assert "ew_bias_scale_tanh_cast" in comp.groups()[0][1]  # still the dedicated kernel


def test_auto_broadcast_with_axis_and_same_rank():
    b = F.NetBuilder("net")
    x = b.create_input(F.Type("float32"), [4, 6, 5], "X")
    m = b.create_input(F.Type("float32"), [6], "M")
    k = b.create_input(F.Type("float32"), [1, 1, 5], "K")
    out = b.multiply(b.add(x, m, axis=1), k)
    b.apply_pass([out], None, ["AutoBroadcast"])
    lines = b.program_text().splitlines()
    assert "broadcast_axes=1" in lines[0] and "broadcast_axes=0,1,2" in lines[2]
    same = F.NetBuilder("net")
    a = same.create_input(F.Type("float32"), [4, 4], "A")
    c = same.create_input(F.Type("float32"), [4, 4], "C")
    o = same.add(a, c)
    before = same.program_text()
    same.apply_pass([o], None, ["AutoBroadcast"])
    assert same.program_text() == before


# ---- RemoveIdentity / DeadCodeEliminate / the default list -----------------------------------------------------------
def test_remove_identity():
    b = F.NetBuilder("net")
    x = _x(b)
    t = b.identity(b.scale(b.exp(x), 1.0, 0.0, True))
    out = b.relu(t)
    kept = b.identity(b.tanh(x))  # fetched: its producer writes the fetched variable directly
    same_in = b.identity(x)       # input and fetched: both ends survive
    b.apply_pass([out, kept, same_in], None, ["RemoveIdentity"])
    assert sorted(_ops(b)) == ["exp", "identity", "relu", "tanh"]
    text = b.program_text()
    assert ("tanh %s = X" % kept) in text and ("identity %s = X" % same_in) in text


def test_dead_code_eliminate():
    b = F.NetBuilder("net")
    x = _x(b)
    out = b.relu(x)
    b.exp(b.tanh(x))
    b.apply_pass([out], None, ["DeadCodeEliminate"])
    assert _ops(b) == ["relu"]


def test_default_pass_list_and_unknown_pass():
    b = F.NetBuilder("net")
    x = b.create_input(F.Type("float16"), [64, 1024], "X")
    bias = b.create_input(F.Type("float16"), [1024], "B")
    out = b.exp(b.identity(b.add(x, bias)))
    b.tanh(x)  # dead
    assert b.apply_pass([out]) == 1
    assert _ops(b) == ["broadcast_to", "elementwise_add", "cast", "exp", "cast"]
    with pytest.raises(Exception, match="no program pass named"):
        b.apply_pass([out], None, ["NoSuchPass"])


# ---- TransposeCollapsing: the reference's cases (transpose_collapsing_test.cc:77-450) ---------------------------------
def _tc(build, fetch_of, expected_removed, expected_text=None):
    b = F.NetBuilder("net")
    x = b.create_input(F.Type("float32"), [4, 5, 3], "X")
    outs = build(b, x)
    n = _count(b)
    b.apply_pass(fetch_of(outs), None, ["TransposeCollapsing"])
    assert n - _count(b) == expected_removed, b.program_text()
    if expected_text:
        assert expected_text in b.program_text(), b.program_text()
    return b


def test_transpose_collapsing_chains():
    # two transposes become one with the composed permutation [1,2,0]
    _tc(lambda b, x: [b.transpose(b.transpose(x, [0, 2, 1]), [2, 1, 0])], lambda o: o, 1, "axis=1,2,0")
    # three: [0,2,1] then [2,1,0] then [1,2,0]
    _tc(lambda b, x: [b.transpose(b.transpose(b.transpose(x, [0, 2, 1]), [2, 1, 0]), [1, 2, 0])], lambda o: o, 2)
    # a single useless transpose is left alone when fetched ...
    _tc(lambda b, x: [b.transpose(x, [0, 1, 2])], lambda o: o, 0)
    # ... three [0,2,1] in a row collapse into one
    def three(b, x):
        t = b.transpose(b.transpose(b.transpose(x, [0, 2, 1]), [0, 2, 1]), [0, 2, 1])
        return [b.add(t, t)]
    _tc(three, lambda o: o, 2, "axis=0,2,1")


def test_transpose_collapsing_with_other_users_and_two_chains():
    def multi(b, x):
        t1 = b.transpose(x, [0, 2, 1])
        t2 = b.transpose(t1, [2, 0, 1])
        t3 = b.transpose(t2, [2, 1, 0])
        return [b.sqrt(t1), b.sqrt(t2), b.sqrt(t3)]
    b = _tc(multi, lambda o: o, 0)
    # every transpose now reads X directly
    assert all("= X" in ln for ln in b.program_text().splitlines() if ln.startswith("transpose"))

    def two_sections(b, x):
        out1 = b.reshape(b.transpose(b.transpose(x, [0, 2, 1]), [2, 1, 0]), [5, 3, 4])
        out2 = b.sqrt(b.transpose(b.transpose(out1, [0, 2, 1]), [2, 1, 0]))
        return [out1, out2]
    _tc(two_sections, lambda o: o, 2)
    # parallel transposes of one input are not merged (the horizontal step is off in the reference too)
    _tc(lambda b, x: [b.add(b.transpose(x, [0, 2, 1]), b.transpose(x, [0, 2, 1]))], lambda o: o, 0)
    # a chain that composes to what a parallel transpose already computes: the chain still folds
    def ver_and_hor(b, x):
        return [b.add(b.transpose(b.transpose(x, [0, 2, 1]), [2, 1, 0]), b.transpose(x, [1, 2, 0]))]
    _tc(ver_and_hor, lambda o: o, 1)


def test_transpose_collapsing_shapes_stay_consistent():
    """The composed permutation applied to X gives the shape the last transpose of the chain had."""
    b = F.NetBuilder("net")
    x = b.create_input(F.Type("float32"), [4, 5, 3], "X")
    out = b.transpose(b.transpose(x, [0, 2, 1]), [2, 1, 0])   # [4,3,5] -> [5,3,4]
    b.apply_pass([out], None, ["TransposeCollapsing"])
    comp = F.Computation.build_and_compile(None, b, fetch=[str(out)], plan_only=True)
    assert len(comp.groups()) == 1 and out.shape == [5, 3, 4]


# ---- FillConstantRewriter / FillConstantFolding (fill_constant_rewriter_test.cc, fill_constant_folding_test.cc) -----
def test_fill_constant_rewriter_cases_of_the_reference():
    # reshape of a constant becomes a constant; the reshape of x to its own shape goes with RemoveIdentity: 2 removed
    b = F.NetBuilder("net")
    x = b.create_input(F.Type("float32"), [32, 16], "x")
    c1 = b.fill_constant([16, 32], 1.0, "constant_1")
    out = b.add(b.reshape(c1, [32, 16]), b.reshape(x, [32, 16]))
    n = _count(b)
    b.apply_pass([out], None, ["FillConstantRewriter", "RemoveIdentity"])
    assert n - _count(b) == 2
    assert "fill_constant" in b.program_text() and "shape=32,16" in b.program_text() and "reshape" not in b.program_text()
    # scale(128, -1) = -128
    b = F.NetBuilder("net")
    x = b.create_input(F.Type("float32"), [32, 16], "x")
    out = b.add(b.scale(b.fill_constant([32, 16], 128.0, "c"), -1.0), b.scale(x, 1.0))
    n = _count(b)
    b.apply_pass([out], None, ["FillConstantRewriter", "RemoveIdentity"])
    assert n - _count(b) == 2 and "value=-128" in b.program_text()
    # three scales in a row: ((128 * -1) * 2 + 10 + 1) * 3 = -735
    b = F.NetBuilder("net")
    x = b.create_input(F.Type("float32"), [32, 16], "x")
    s3 = b.scale(b.scale(b.scale(b.fill_constant([32, 16], 128.0, "c"), -1.0), 2.0, 10.0), 3.0, 1.0, False)
    out = b.add(s3, b.scale(x, 1.0))
    n = _count(b)
    b.apply_pass([out], None, ["FillConstantRewriter", "RemoveIdentity"])
    assert n - _count(b) == 4 and "value=-735" in b.program_text()
    # cast and the math functions; a constant with another kind of user stays
    b = F.NetBuilder("net")
    x = b.create_input(F.Type("float32"), [4, 4], "x")
    c = b.fill_constant([4, 4], -2.5, "c")
    out = b.add(b.add(x, b.abs(c)), b.cast(b.cast(c, "int32"), "float32"))
    keep = b.multiply(x, c)
    b.apply_pass([out, keep], None, ["FillConstantRewriter"])
    assert set(_ops(b)) == {"fill_constant", "elementwise_add", "elementwise_mul"}
    values = sorted(ln.split("value=")[1].split()[0] for ln in b.program_text().splitlines() if "value=" in ln)
    assert values == ["-2", "-2.5", "2.5"]  # float32(int32(c)) (the int32 constant in between is gone), c itself, |c|


def test_fill_constant_folding_cases_of_the_reference():
    def build(values, use):
        b = F.NetBuilder("net")
        cs = [b.fill_constant([32, 32], v, "") for v in values]
        outs = use(b, cs)
        n = _count(b)
        b.apply_pass(outs, None, ["FillConstantFolding"])
        return n - _count(b), b
    # (the reference's cases put a transpose on the constants; a transposed constant has no kernel here, relu stands in)
    assert build([1.0, 1.0], lambda b, c: [b.add(b.relu(c[0]), b.relu(c[1]))])[0] == 1
    assert build([1.0, 1.0], lambda b, c: [b.relu(c[0]), b.add(c[1], c[1])])[0] == 1
    assert build([1.0, 1.0, 1.0], lambda b, c: [b.relu(c[0]), b.add(c[1], c[2])])[0] == 2
    removed, b = build([1.0, 1.0, 0.0], lambda b, c: [b.relu(c[0]), b.add(c[1], c[2])])
    assert removed == 1 and b.program_text().count("fill_constant") == 2


def test_default_pass_list_is_fully_built():
    b = F.NetBuilder("net")
    x = b.create_input(F.Type("float16"), [64, 1024], "X")
    c = b.scale(b.fill_constant([64, 1024], 2.0, "", "float16"), 0.5, 0.25)
    t = b.transpose(b.transpose(b.add(x, c), [1, 0]), [1, 0])
    out = b.exp(t)
    assert b.apply_pass([out]) == 1
    assert _ops(b) == ["fill_constant", "elementwise_add", "cast", "exp", "cast"]
    assert "value=1.25" in b.program_text()


# ---- Decomposer --------------------------------------------------------------------------------------------------------
def _group_text_without_names(comp):
    import re
    out = []
    for desc, pattern in comp.groups():
        out.append((re.sub(r"var_[0-9]+|fn_[^ \n]+", "_", desc), pattern))
    return out


def test_decomposer_emits_what_the_builder_methods_compose():
    """gelu, the max-subtracted softmax and inference batch_norm as instructions, decomposed by the pass: the same
    groups (up to variable names), hence the same kernels and arguments, as the builder's own compositions."""
    def plan(b, out):
        return F.Computation.build_and_compile(None, b, fetch=[str(out)], plan_only=True)
    # gelu
    b1 = F.NetBuilder("net")
    y1 = b1.gelu(b1.create_input(F.Type("float32"), [64, 4096], "X"))
    b2 = F.NetBuilder("net")
    y2 = b2._op("gelu", [b2.create_input(F.Type("float32"), [64, 4096], "X")])
    b2.apply_pass([y2], None, ["Decomposer"])
    assert "gelu" not in b2.program_text()
    assert _group_text_without_names(plan(b1, y1)) == _group_text_without_names(plan(b2, y2))
    # softmax, any mode but "fast"
    b1 = F.NetBuilder("net")
    y1 = b1.softmax(b1.create_input(F.Type("float32"), [64, 4096], "X"), (-1,), "safe")
    b2 = F.NetBuilder("net")
    y2 = b2._op("softmax", [b2.create_input(F.Type("float32"), [64, 4096], "X")], axis=-1, mode="safe")
    b2.apply_pass([y2], None, ["Decomposer"])
    g1, g2 = _group_text_without_names(plan(b1, y1)), _group_text_without_names(plan(b2, y2))
    assert g1 == g2 and g2[0][1].startswith("softmax_safe_row")
    # the fast mode stays the op
    b3 = F.NetBuilder("net")
    y3 = b3._op("softmax", [b3.create_input(F.Type("float32"), [64, 4096], "X")], axis=-1, mode="fast")
    b3.apply_pass([y3], None, ["Decomposer"])
    assert _ops(b3) == ["softmax"]
    # inference batch_norm: the decomposed arithmetic ((x - mean) * rsqrt(var + eps)) * scale + bias
    b4 = F.NetBuilder("net")
    x = b4.create_input(F.Type("float32"), [8, 16, 14, 14], "x")
    ps = [b4.create_input(F.Type("float32"), [16], n) for n in ("scale", "bias", "mean", "variance")]
    y4 = b4.batch_norm(x, *ps, epsilon=1e-5, is_test=True)
    b4.apply_pass([y4], None, ["Decomposer"])
    assert "batch_norm" not in b4.program_text() and "rsqrt" in b4.program_text()
    comp = plan(b4, y4)
    assert [p for _, p in comp.groups()] == ["ew_bn_train_apply_nchw ew_bn_train_apply_nchw_f32"]


def test_default_passes_decompose_a_sixteen_bit_gelu():
    b = F.NetBuilder("net")
    y = b._op("gelu", [b.create_input(F.Type("float16"), [64, 4096], "X")])
    assert b.apply_pass([y]) == 1           # cast, the float32 gelu primitives, cast: one chain kernel
    assert "gelu" not in b.program_text() and _ops(b).count("cast") == 2


def test_default_passes_are_idempotent_and_keep_the_fetched_variables():
    """Seeded random programs (the generator of the GPU tests): the default pass list applied twice changes nothing
    the second time, the fetched variables keep their shapes and types, and the rewritten program still plans."""
    import importlib
    import numpy as np
    gen = importlib.import_module("tests.test_gpu_random_programs")
    for half in (False, True):
        for seed in range(0, 100, 4):
            rng = np.random.default_rng(1000 + seed)
            shape = [(6, 40), (3, 5, 16), (2, 7, 3, 12), (33,), (4, 9, 28)][seed % 5]
            b = F.NetBuilder("rand%d" % seed)
            _, fetch = gen.build_random_program(rng, b, shape, half)
            ids = [str(f) for f in fetch]
            before = [(f.shape, f.type.name) for f in fetch]
            groups = b.apply_pass(ids)
            text = b.program_text()
            assert b.apply_pass(ids) == groups and b.program_text() == text, (seed, half)
            assert [(f.shape, f.type.name) for f in fetch] == before
