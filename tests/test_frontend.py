"""NetBuilder shape inference, the fusion pass and the matcher, planned without a GPU.

Group-count assertions follow the style of the reference's fusion tests
(cinn/hlir/pass/op_fusion_pass_test.cc:22-253, fusion_merge_pass_test.cc:22-462)."""
import ctypes

import pytest

import cinn_b200
from cinn_b200 import common
from cinn_b200 import workloads as W
from cinn_b200.frontend import Computation, NetBuilder

TARGET = common.DefaultNVGPUTarget()


@pytest.fixture(autouse=True, scope="module")
def interpreted_chain_kernels():
    """The kernel names asserted in this file are the interpreting chain kernel's variants (which one a program
    needs: side operands, temporaries, a second output); programs that also have a kernel specialised at build time
    would show that kernel's name instead, so the substitution is switched off for this module."""
    L = cinn_b200.lib()
    L.cinn_b200_set_option(b"enable_static_chains", 0)
    yield
    L.cinn_b200_set_option(b"enable_static_chains", 1)


def plan(builder, **kw):
    return Computation.build_and_compile(TARGET, builder, plan_only=True, **kw)


def patterns(comp):
    return [p.split()[0] for _, p in comp.groups()]


def test_readme_example_is_one_group():
    b = NetBuilder(name="network")
    a = b.create_input(type=common.Float(32), shape=(1, 3, 224, 224), id_hint="A")
    bb = b.create_input(type=common.Float(32), shape=(1, 3, 224, 224), id_hint="B")
    res = b.relu(b.add(a, bb))
    c = plan(b)
    assert patterns(c) == ["ew_add_relu"]
    desc, _ = c.groups()[0]
    assert desc.splitlines()[1].split()[:2] == ["input", "A"] and desc.splitlines()[2].split()[:2] == ["input", "B"]
    assert res.shape == [1, 3, 224, 224] and str(res.type) == "float32"
    assert set(c.get_all_tensor_names()) == {"A", "B", str(res)}


def test_shape_and_dtype_inference():
    b = NetBuilder("infer")
    x = b.create_input(common.Float(32), (4, 8, 16), "x")
    v = b.create_input(common.Float(32), (8,), "v")
    assert b.add(x, v, axis=1).shape == [4, 8, 16]
    assert b.reduce_sum(x, [1]).shape == [4, 16]
    assert b.reduce_max(x, [0, 1], keep_dim=True).shape == [1, 1, 16]
    assert b.reduce_sum(x).shape == [1]
    assert b.reduce_sum(x, [-1]).shape == [4, 8]
    assert str(b.cast(x, "float16").type) == "float16"
    assert b.broadcast_to(v, [4, 8, 16], [1]).shape == [4, 8, 16]
    assert b.reshape(x, [32, -1]).shape == [32, 16]
    with pytest.raises(cinn_b200.CinnB200Error):
        b.add(x, b.create_input(common.Float(32), (7,), "bad"))
    with pytest.raises(cinn_b200.CinnB200Error):
        b.add(x, b.cast(x, "float16"))
    with pytest.raises(cinn_b200.CinnB200Error):
        b.reduce_sum(x, [3])
    with pytest.raises(cinn_b200.CinnB200Error):
        b._op("conv2d", [x, x])


def test_broadcast_chain_is_one_group():
    b = NetBuilder("c2")
    x = b.create_input(common.Float(32), (64, 1024, 1024), "X")
    bias = b.create_input(common.Float(32), (1024,), "bias")
    y = b.cast(b.tanh(b.scale(b.add(x, bias), 0.5, 0.0)), "float16")
    c = plan(b)
    assert patterns(c) == ["ew_bias_scale_tanh_cast"]
    assert y.shape == [64, 1024, 1024]


def test_reductions_are_their_own_groups():
    b = NetBuilder("c3")
    x = b.create_input(common.Float(32), (128, 1024, 1024), "X")
    b.reduce_sum(x, [2])
    b.reduce_max(x, [0])
    c = plan(b)
    assert sorted(patterns(c)) == ["col_reduce", "row_reduce"]


def test_softmax_op_and_decomposed_form_and_fp16_wrappers():
    for half in (False, True):
        b = NetBuilder("sm")
        x = b.create_input(common.Float(16 if half else 32), (16384, 4096), "X")
        xin = b.cast(x, "float32") if half else x
        y = b.softmax(xin)
        if half:
            y = b.cast(y, "float16")
        assert patterns(plan(b)) == ["softmax_row"]
    # decomposed "fast" form: exp -> reduce_sum -> broadcast -> divide, rows far longer than the reference's 1024
    # limit for fusing a reduce with its broadcast consumer: still ONE group here
    b = NetBuilder("smd")
    x = b.create_input(common.Float(32), (64, 4096), "X")
    e = b.exp(x)
    s = b.reduce_sum(e, [1])
    b.divide(e, b.broadcast_to(s, [64, 4096], [0]))
    assert patterns(plan(b)) == ["softmax_row"]


def test_layer_norm_composition_is_one_group():
    for half in (False, True):
        b = NetBuilder("ln")
        x = b.create_input(common.Float(16 if half else 32), (16384, 4096), "X")
        g = b.create_input(common.Float(32), (4096,), "gamma")
        be = b.create_input(common.Float(32), (4096,), "beta")
        b.layer_norm(x, g, be, 1e-5)
        c = plan(b)
        assert patterns(c) == ["layernorm_row"]
        desc, _ = c.groups()[0]
        assert [l.split()[1] for l in desc.splitlines() if l.startswith("input")] == ["X", "gamma", "beta"]


def test_batch_norm_relu_group_and_argument_order():
    b = NetBuilder("bn")
    x = b.create_input(common.Float(32), (256, 64, 112, 112), "x")
    names = ["scale", "bias", "mean", "variance"]
    params = [b.create_input(common.Float(32), (64,), n) for n in names]
    b.relu(b.batchnorm(x, *params, epsilon=1e-5, is_test=True)[0])
    c = plan(b)
    assert patterns(c) == ["ew_bn_relu_nchw"]
    desc, _ = c.groups()[0]
    assert [l.split()[1] for l in desc.splitlines() if l.startswith("input")] == ["x"] + names


def test_mixed_graph_partitions_into_fused_chain_reduce_and_chain():
    b = NetBuilder("mixed")
    x = b.create_input(common.Float(32), (8, 16, 1024), "X")
    bias = b.create_input(common.Float(32), (1024,), "bias")
    y = b.sigmoid(b.multiply(b.add(x, bias), bias))
    z = b.reduce_sum(y, [2])
    b.sqrt(b.abs(z))
    c = plan(b)
    # the chain in front of the reduction runs inside the reduction kernel: no intermediate tensor
    assert [p for _, p in c.groups()] == ["chain_row_reduce chain_reduce_row_s1", "ew_chain ew_chain_f32_s0"]


def test_elementwise_producer_folds_into_reduction():
    b = NetBuilder("fold")
    x = b.create_input(common.Float(32), (64, 4096), "X")
    b.sqrt(b.divide(b.reduce_sum(b.multiply(x, b.identity(x)), [1]), b.fill_constant([64], 4096.0)))
    c = plan(b)
    assert [p for _, p in c.groups()] == ["row_reduce row_reduce_cta_sumsq_f32", "ew_chain ew_chain_f32_s0"]


def test_value_used_twice_feeds_two_outputs_of_one_kernel():
    """Two elementwise consumers of one value are fused horizontally (fusion_merge_pass.cc:85-460)."""
    b = NetBuilder("fanout")
    x = b.create_input(common.Float(32), (64, 64), "X")
    t = b.exp(x)
    b.relu(t)
    b.tanh(t)
    c = plan(b)
    # the two consumers are siblings over one input: one kernel with two outputs, exp never reaches memory
    assert [p for _, p in c.groups()] == ["ew_chain ew_chain_f32_s1o"]
    assert str(t) not in c.get_all_tensor_names()


def test_fetch_keeps_an_intermediate():
    b = NetBuilder("fetch")
    x = b.create_input(common.Float(32), (64, 64), "X")
    t = b.exp(x)
    y = b.relu(t)
    assert len(plan(b).groups()) == 1
    c = plan(b, fetch=[t, y])
    # one kernel with two outputs: the fetched intermediate is stored on the way
    assert [p for _, p in c.groups()] == ["ew_chain ew_chain_f32_s1o"] and str(t) in c.get_all_tensor_names()


def test_unmatched_group_is_an_error_not_a_fallback():
    L = cinn_b200.lib()
    fn = ctypes.c_void_p()
    rc = L.cinn_b200_compile_group(b"group g\ninput x float32 4,4\nop conv2d y = x x\noutput y float32 4,4\n",
                                   ctypes.byref(fn))
    assert rc == -2 and b"no prebuilt sm_100a kernel" in L.cinn_b200_last_error()
    rc = L.cinn_b200_compile_group(b"group g\ninput x uint8 4,4\nop exp y = x\noutput y uint8 4,4\n", ctypes.byref(fn))
    assert rc == -2
    rc = L.cinn_b200_compile_group(b"nonsense", ctypes.byref(fn))
    assert rc == -1
    # a float32 reduce over non-adjacent axes is planned as one launch per run of adjacent axes ...
    rc = L.cinn_b200_compile_group(
        b"group g_multi\ninput x float32 4,5,6,7\nop reduce_sum y = x ; dim=1,3\noutput y float32 4,6\n", ctypes.byref(fn))
    assert rc == 0
    assert L.cinn_b200_release_group(b"g_multi") == 0
    # ... and so are the other element types
    rc = L.cinn_b200_compile_group(
        b"group g_multi_i\ninput x int32 4,5,6,7\nop reduce_sum y = x ; dim=1,3\noutput y int32 4,6\n", ctypes.byref(fn))
    assert rc == 0
    assert L.cinn_b200_release_group(b"g_multi_i") == 0
    # a reduction of a type without reduction kernels stays an error
    rc = L.cinn_b200_compile_group(
        b"group g\ninput x uint8 4,5,6,7\nop reduce_sum y = x ; dim=1,3\noutput y uint8 4,6\n", ctypes.byref(fn))
    assert rc == -2
    assert L.cinn_b200_lookup(b"g") is None


def test_canonical_expression_and_plans_of_the_workloads():
    L = cinn_b200.lib()
    buf = ctypes.create_string_buffer(4096)
    w = W.bias_scale_tanh_cast((2, 4, 8))
    assert L.cinn_b200_canonical_expr(w.desc.encode(), buf, 4096) == 0
    assert buf.value == b"cast(tanh(scale(elementwise_add(%0,%1))))"
    expect = {
        "add_relu": (W.add_relu((1, 3, 224, 224)), ["ew_add_relu_f32"]),
        "c2": (W.bias_scale_tanh_cast((64, 1024, 1024)), ["ew_bias_scale_tanh_cast_stream_f32_f16"]),
        "c3a": (W.reduce_sum_last((128, 1024, 1024)), ["row_reduce_warp8_sum_f32"]),
        "c3b": (W.reduce_max_first((128, 1024, 1024)), ["col_reduce_max_f32"]),
        "c4a": (W.softmax((16384, 4096)), ["softmax_row_f32_g256_v4_r1"]),
        "c4b16": (W.layer_norm((16384, 4096), half=True), ["layernorm_tma_f16_g256_v2"]),
        "c5": (W.bn_relu((256, 64, 112, 112)), ["ew_bn_relu_nchw_f32"]),
        "long_row": (W.reduce_sum_last((1, 3000001)), ["row_reduce_cta_sum_f32", "row_reduce_warp4_sum_f32"]),
        "cluster_row": (W.reduce_sum_last((40, 70000)), ["row_reduce_cluster_sum_f32"]),
        "cluster_softmax": (W.softmax((2, 100000)), ["rownorm_cluster_f32"]),
    }
    for key, (w, kernels) in expect.items():
        g = cinn_b200.FusedGroup(w.desc)
        assert g.kernel_names() == kernels, key
        assert g.algorithmic_bytes == w.algorithmic_bytes(), key
        g.release()


def test_byte_counts_of_the_benchmark_groups():
    sizes = {"c1": (W.add_relu(), 1806336), "c2": (None, 402657280), "c3a": (None, 537395200),
             "c3b": (None, 541065216)}
    assert W.add_relu().algorithmic_bytes() == sizes["c1"][1]


def test_host_x86_target_is_refused():
    b = NetBuilder("x86")
    x = b.create_input(common.Float(32), (4, 4), "X")
    b.relu(x)
    with pytest.raises(RuntimeError):
        Computation.build_and_compile(common.DefaultHostTarget(), b)


def test_other_dtypes_pick_their_kernel_families():
    """float64 / integer / bool groups are planned onto the double, integer and typed-reduction kernels."""
    def one(make):
        b = NetBuilder("p")
        make(b)
        return [p for _, p in plan(b).groups()]

    i32, i64, f64, f16 = common.Int(32), common.Int(64), common.Float(64), common.Float(16)
    assert one(lambda b: b.abs(b.add(b.create_input(i32, (8, 64), "X"), b.create_input(i32, (64,), "Y")))) == \
        ["ew_chain ew_chain_int_i32_i32_s1"]
    assert one(lambda b: b.cast(b.bitwise_and(b.create_input(i64, (8, 64), "X"), b.create_input(i64, (8, 64), "Y")),
                                "int32")) == ["ew_chain ew_chain_int_i64_i32_s1"]
    assert one(lambda b: b.less_than(b.create_input(i32, (8, 64), "X"), b.create_input(i32, (8, 64), "Y"))) == \
        ["ew_chain ew_chain_int_i32_bool_s1"]
    assert one(lambda b: b.tanh(b.create_input(f64, (8, 64), "X"))) == ["ew_chain ew_chain_f64_f64_s0"]
    assert one(lambda b: b.cast(b.floor(b.create_input(common.Float(32), (8, 64), "X")), "int64")) == \
        ["ew_chain ew_chain_i64_s0"]
    assert one(lambda b: b.select(b.create_input(common.Bool(), (8, 64), "M"), b.create_input(f16, (8, 64), "X"),
                                  b.create_input(f16, (8, 64), "Y"))) == ["ew_chain ew_chain_f16_s3"]
    assert one(lambda b: b.reduce_sum(b.create_input(i32, (8, 64), "X"), [1])) == \
        ["row_reduce reduce_generic_row_sum_i32"]
    assert one(lambda b: b.reduce_max(b.create_input(f16, (8, 64, 32), "X"), [1])) == \
        ["col_reduce reduce_generic_col_max_f16"]
    assert one(lambda b: b.reduce_all(b.create_input(common.Bool(), (8, 64), "X"), [1])) == \
        ["row_reduce reduce_generic_row_all_bool"]
    assert one(lambda b: b.reduce_any(b.create_input(common.Bool(), (8, 64), "X"), [0])) == \
        ["col_reduce reduce_generic_col_any_bool"]


def test_operand_type_rules_of_the_new_ops():
    b = NetBuilder("bad")
    x = b.create_input(common.Float(32), (4, 4), "X")
    m = b.create_input(common.Bool(), (4, 4), "M")
    for make in (lambda: b.logical_and(x, x), lambda: b.logical_not(x), lambda: b.reduce_all(x, [0]),
                 lambda: b.popc(x), lambda: b.select(x, x, x)):
        with pytest.raises(Exception):
            make()
    assert b.isnan(x)._info()[0] == "bool" and b.logical_xor(m, m)._info()[0] == "bool"


def test_batch_norm_train_plans_one_statistics_pass_and_one_normalisation_pass():
    b = NetBuilder("bnt")
    x = b.create_input(common.Float(32), (256, 64, 112, 112), "x")
    ps = [b.create_input(common.Float(32), (64,), n) for n in ["scale", "bias", "mm", "mv"]]
    b.batchnorm(x, *ps, is_test=False)
    c = plan(b)
    pats = patterns(c)
    assert pats.count("channel_stats") == 1 and pats.count("ew_bn_train_apply_nchw") == 1
    # everything else works on [64]-element vectors
    for desc, p in c.groups():
        if p.split()[0] == "ew_chain":
            assert all(l.split()[3] == "64" for l in desc.splitlines() if l.startswith(("input", "output"))), desc
    stats = [d for d, p in c.groups() if p.startswith("channel_stats")][0]
    assert len([l for l in stats.splitlines() if l.startswith("output")]) == 2


def test_exported_program_loads_without_builder_and_plans_the_same_kernels(tmp_path):
    b = NetBuilder("exp")
    x = b.create_input(common.Float(32), (8, 16, 1024), "X")
    bias = b.create_input(common.Float(32), (1024,), "bias")
    y = b.sigmoid(b.multiply(b.add(x, bias), bias))
    z = b.reduce_sum(y, [2])
    b.sqrt(b.abs(b.reshape(z, [128])))
    c = plan(b)
    text = c.export(str(tmp_path / "prog.txt"))
    assert text.startswith("cinn_b200_program 1\n") and "begin_group" in text and "alias " in text
    c2 = Computation.load(str(tmp_path / "prog.txt"), plan_only=True)
    kernels = lambda comp: [p.split()[1:] for _, p in comp.groups() if not p.startswith("reshape_alias")]  # noqa: E731
    assert kernels(c2) == kernels(c)
    assert sorted(c2.get_all_tensor_names()) == sorted(c.get_all_tensor_names())
    with pytest.raises(Exception):
        Computation.load("not a program", plan_only=True)
    with pytest.raises(Exception):
        Computation.load(text.replace("op sigmoid", "op conv2d"), plan_only=True)


def test_bfloat16_storage_picks_bf16_kernels():
    """The dedicated batch_norm / softmax / layer_norm kernels exist for bfloat16 storage as for float16."""
    from cinn_b200 import workloads as W
    import cinn_b200
    for w, want in ((W.softmax((64, 4096), half=True), "bf16"), (W.softmax_safe((64, 4096), half=True), "softmax_safe_bf16"),
                    (W.layer_norm((64, 4096), half=True), "bf16"), (W.bn_relu((2, 8, 14, 14), half=True), "ew_bn_relu_nchw_bf16")):
        g = cinn_b200.FusedGroup(w.desc.replace("float16", "bfloat16"))
        assert want in g.kernel_names()[0], g.kernel_names()
        g.release()


def test_expression_trees_compile_into_one_kernel_with_temporaries():
    """A binary op whose operands are both computed in the group: one branch runs first and is stashed in a temporary
    (two temporaries at most, three side operands at most); beyond that the fusion pass splits the group."""
    def build(n_inputs=4):
        b = NetBuilder("tree")
        return b, [b.create_input(common.Float(32), (64, 1024), n) for n in "ABCD"[:n_inputs]]
    b, (A, B, C, D) = build()
    b.multiply(b.add(A, B), b.subtract(C, D))
    assert [p for _, p in plan(b).groups()] == ["ew_chain ew_chain_f32_s3t"]
    b, (A, B, C, D) = build()
    b.reduce_max(b.add(b.multiply(A, B), b.multiply(C, D)), [0])
    assert [p for _, p in plan(b).groups()] == ["chain_col_reduce chain_reduce_col_s3t"]
    # the integer and float64 forms have the same variant
    b = NetBuilder("tree")
    I = [b.create_input(common.Int(32), (64, 1024), n) for n in "ABCD"]
    b.multiply(b.add(I[0], I[1]), b.subtract(I[2], I[3]))
    assert [p for _, p in plan(b).groups()] == ["ew_chain ew_chain_int_i32_i32_s3t"]
    b = NetBuilder("tree")
    D = [b.create_input(common.Float(64), (64, 1024), n) for n in "ABCD"]
    b.multiply(b.add(D[0], D[1]), b.subtract(D[2], D[3]))
    assert [p for _, p in plan(b).groups()] == ["ew_chain ew_chain_f64_f64_s3t"]
    # three joins need three temporaries: no chain any more.  The fusion pass splits the region (only the
    # interpreting register-program kernel would take it whole); asked to, it keeps it as one register program
    b, (A, B, C, D) = build()
    b.add(b.multiply(b.exp(A), b.tanh(B)), b.multiply(b.sqrt(b.abs(C)), b.sigmoid(D)))
    assert len(plan(b).groups()) > 1
    cinn_b200.lib().cinn_b200_set_option(b"fuse_interpreted_programs", 1)
    try:
        assert [p for _, p in plan(b).groups()] == ["ew_dag ew_dag"]
    finally:
        cinn_b200.lib().cinn_b200_set_option(b"fuse_interpreted_programs", 0)
    # what no elementwise kernel takes is still split: nine tensors read at once
    b = NetBuilder("wide")
    xs = [b.create_input(common.Float(32), (64, 1024), "X%d" % i) for i in range(9)]
    acc = xs[0]
    for x in xs[1:]:
        acc = b.add(acc, x)
    assert len(plan(b).groups()) > 1


def _assert_topological(c, program_inputs):
    """Every group reads program inputs or results of earlier groups."""
    known = set(program_inputs)
    for desc, _ in c.groups():
        lines = desc.splitlines()
        for ln in lines:
            if ln.startswith("input "):
                assert ln.split()[1] in known, (ln, [p for _, p in c.groups()])
        for ln in lines:
            if ln.startswith("output "):
                known.add(ln.split()[1])
            if ln.startswith("op reshape"):
                known.add(ln.split()[2])


def test_two_output_groups_and_no_group_cycles():
    # a fetched intermediate is stored on the way: one kernel
    b = NetBuilder("two_out")
    x = b.create_input(common.Float(32), (64, 1024), "X")
    bias = b.create_input(common.Float(32), (1024,), "B")
    pre = b.add(x, bias)
    act = b.tanh(b.relu(pre))
    c = plan(b, fetch=[pre, act])
    assert [p for _, p in c.groups()] == ["ew_chain ew_chain_f32_s1o"]
    # siblings (neither is on the way to the other): one kernel that evaluates one, stores it and restarts
    b = NetBuilder("siblings")
    x = b.create_input(common.Float(32), (64, 1024), "X")
    t = b.exp(x)
    c = plan(b, fetch=[b.relu(t), b.tanh(t)])
    assert [p for _, p in c.groups()] == ["ew_chain ew_chain_f32_s1o"]
    # three siblings: two in one kernel, the third on its own
    b = NetBuilder("siblings3")
    x = b.create_input(common.Float(32), (64, 1024), "X")
    c = plan(b, fetch=[b.relu(x), b.tanh(x), b.exp(x)])
    assert len(c.groups()) == 2
    _assert_topological(c, ["X"])
    # exp may not join the subtract: its other user (the reduction) feeds the subtract as well, and the two groups
    # would wait for each other
    b = NetBuilder("no_cycle")
    x = b.create_input(common.Float(32), (64, 1024), "X")
    e = b.exp(x)
    m = b.reduce_max(e, [1])
    b.subtract(e, b.broadcast_to(m, [64, 1024], [0]))
    c = plan(b)
    _assert_topological(c, ["X"])
    assert len(c.groups()) >= 2
    # ... unless the three instructions are one group: a row program (exp is evaluated again in the pass after the
    # maximum), which the fusion pass forms when asked to use the interpreting kernel
    cinn_b200.lib().cinn_b200_set_option(b"fuse_interpreted_programs", 1)
    try:
        assert [p for _, p in plan(b).groups()] == ["row_program row_program"]
    finally:
        cinn_b200.lib().cinn_b200_set_option(b"fuse_interpreted_programs", 0)


def test_export_and_load_keep_two_output_and_tree_groups():
    b = NetBuilder("aot")
    x = b.create_input(common.Float(32), (64, 1024), "X")
    y = b.create_input(common.Float(32), (64, 1024), "Y")
    bias = b.create_input(common.Float(32), (1024,), "B")
    pre = b.add(x, bias)
    act = b.relu(pre)                                             # two outputs, one on the way to the other
    tree = b.multiply(b.add(x, y), b.subtract(x, bias))           # a tree
    norm = b.reduce_sum(b.abs(b.subtract(x, y)), [1])             # chain + reduce
    c = plan(b, fetch=[pre, act, tree, norm])
    text = c.export()
    loaded = Computation.load(text, plan_only=True)
    assert [p for _, p in loaded.groups()] == [p for _, p in c.groups()]
    assert sorted(loaded.get_all_tensor_names()) == sorted(c.get_all_tensor_names())
    kinds = " ".join(p for _, p in c.groups())
    assert "chain_row_reduce" in kinds and "_s1o" in kinds and "_s3t" in kinds


def test_compositions_between_other_ops_are_still_one_kernel():
    """A decomposed softmax / layer_norm whose operand is computed in the program and whose result feeds more ops: the
    part of the region between the fork and the point where its branches meet again is a group of its own."""
    b = NetBuilder("mid")
    x = b.create_input(common.Float(32), (64, 4096), "X")
    g, be = b.create_input(common.Float(32), (4096,), "G"), b.create_input(common.Float(32), (4096,), "Bt")
    b.tanh(b.layer_norm(b.relu(b.scale(x, 2.0, 1.0)), g, be))
    assert patterns(plan(b)) == ["ew_chain", "layernorm_row", "ew_chain"]
    b = NetBuilder("mid2")
    x = b.create_input(common.Float(32), (64, 4096), "X")
    b.relu(b.softmax(b.gelu(x), (-1,), "safe"))
    assert patterns(plan(b)) == ["ew_chain", "softmax_safe_row", "ew_chain"]
    b = NetBuilder("mid3")
    x = b.create_input(common.Float(32), (64, 4096), "X")
    b.softmax(b.softmax(x, (-1,), "safe"), (-1,), "safe")
    assert patterns(plan(b)) == ["softmax_safe_row", "softmax_safe_row"]


def test_compile_options_use_decomposer_and_passes():
    """CinnComputation::CompileOptions (cinn/frontend/computation.h:30-44): the Decomposer first, then named passes."""
    b = NetBuilder("opts")
    x = b.create_input(common.Float(32), (64, 4096), "X")
    y = b._op("softmax", [b._op("gelu", [x])], axis=-1, mode="safe")
    with pytest.raises(Exception, match="no prebuilt"):
        Computation.build_and_compile(None, b, fetch=[str(y)], plan_only=True)   # gelu as such has no kernel
    opts = Computation.default_compile_options()
    opts.use_decomposer = True
    opts.passes = ["RemoveIdentity"]
    c = Computation.build_and_compile(None, b, options=opts, fetch=[str(y)], plan_only=True)
    assert patterns(c) == ["ew_chain", "softmax_safe_row"]
