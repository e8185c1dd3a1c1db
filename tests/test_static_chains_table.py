"""The table of chain programs compiled into kernels at build time (cinn_b200/csrc/ew_static_table.inc) is what the
generator beside it produces from today's matcher, and the library holds one kernel per line (no GPU needed)."""
import importlib.util
import os
import re

import cinn_b200

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GEN = os.path.join(ROOT, "cinn_b200", "csrc", "gen_static_chains.py")


def load_generator():
    spec = importlib.util.spec_from_file_location("gen_static_chains", GEN)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_committed_table_is_up_to_date_and_registered():
    gen = load_generator()
    L = cinn_b200.lib()
    total = 0
    for fname, text, _, count in gen.tables():
        committed = open(os.path.join(ROOT, "cinn_b200", "csrc", fname)).read()
        assert committed == text, "run python cinn_b200/csrc/gen_static_chains.py and rebuild the library"
        total += count
        for m in re.finditer(r"^STATIC_(CHAIN_REDUCE_ROW|CHAIN_REDUCE_COL|CHAIN|DAG|ROW_PROGRAM|INT_CHAIN|F64_CHAIN)\((\w+),", text, flags=re.M):
            prefix = {"CHAIN": "ew_static_", "DAG": "ew_dag_static_", "ROW_PROGRAM": "row_program_static_", "INT_CHAIN": "ew_int_static_", "F64_CHAIN": "ew_f64_static_"}.get(m.group(1), "chain_reduce_static_")
            assert L.cinn_b200_get_kernel((prefix + m.group(2)).encode()), prefix + m.group(2)
    # (a row program has 19 kernels -- a CTA per row, and a warp, half a CTA or a CTA with eight vectors per thread for
    # any row and for rows of exactly 2 / 4 / 6 / 8, 2 ... 8 and 5 ... 8 vectors per thread: 19 registry entries per
    # table line)
    rows = len(re.findall(r"^STATIC_ROW_PROGRAM\(", open(os.path.join(ROOT, "cinn_b200", "csrc", "row_prog_static_table.inc")).read(), flags=re.M))
    assert L.cinn_b200_num_static_chains() == total + 18 * rows and total >= 60


def test_listed_groups_plan_to_their_static_kernel_and_others_to_the_interpreter():
    gen = load_generator()
    by_name = dict(gen.GROUPS)
    g = cinn_b200.FusedGroup(by_name["abs_add_f32"])
    assert g.kernel_names() == ["ew_static_abs_add_f32"]
    interpreted_plan = None
    L = cinn_b200.lib()
    L.cinn_b200_set_option(b"enable_static_chains", 0)
    try:
        g2 = cinn_b200.FusedGroup(by_name["abs_add_f32"].replace("fn_static_abs_add_f32", "fn_interp_abs_add_f32"))
        assert g2.kernel_names() == ["ew_chain_f32_s1"]
        interpreted_plan = g2.launch_text()
        g2.release()
    finally:
        L.cinn_b200_set_option(b"enable_static_chains", 1)
    # same launch shape and the same parameters: only the kernel differs
    strip = lambda t: re.sub(r"^launch 0 \S+", "launch 0 K", t)  # noqa: E731
    assert strip(g.launch_text()) == strip(interpreted_plan)
    g.release()
    # a different constant is the same program (immediates are parameters) ...
    d = by_name["scale_relu_f32"].replace("scale=2.0 bias=1.0", "scale=-0.75 bias=3.5").replace("fn_static", "fn_other")
    g = cinn_b200.FusedGroup(d)
    assert g.kernel_names() == ["ew_static_scale_relu_f32"]
    g.release()
    # ... another shape with the same addressing modes too, but another op sequence is not
    d = by_name["abs_add_f32"].replace("64,1024", "7,12,20").replace("fn_static", "fn_shape")
    g = cinn_b200.FusedGroup(d)
    assert g.kernel_names() == ["ew_static_abs_add_f32"]
    g.release()
    d = by_name["abs_add_f32"].replace("op abs t1 = t0", "op ceil t1 = t0").replace("fn_static", "fn_ceil")
    g = cinn_b200.FusedGroup(d)
    assert g.kernel_names() == ["ew_chain_f32_s1"]
    g.release()
    # a reduction whose operand is a listed chain: its own specialised kernel, at any size
    red = dict(gen.REDUCE_GROUPS)
    g = cinn_b200.FusedGroup(red["sum_abs_diff_rows"].replace("64,1024", "8192,8192").replace("float32 64\n", "float32 8192\n"))
    assert g.kernel_names()[0] == "chain_reduce_static_sum_abs_diff_rows", g.kernel_names()
    g.release()


def test_builder_row_compositions_fuse_into_one_specialised_kernel():
    """The row compositions the table lists as NetBuilder programs (rms_norm, standardise, log_softmax, l1_normalise,
    moments, min_max_normalise): with the default options the fusion pass forms ONE group for each and the matcher
    gives it its specialised row-program kernel, at the table's shape and at others (the shape and the constants are
    kernel parameters); min_max_normalise folds the same operand twice in one pass."""
    from cinn_b200.frontend import Computation, NetBuilder
    gen = load_generator()
    for shape in [(64, 4096), (16384, 4096), (70, 1024), (5, 2052)]:
        for make in gen.builder_row_programs(*shape):
            b = NetBuilder(make.__name__)
            fetch = make(b)
            comp = Computation.build_and_compile(None, b, fetch=[str(f) for f in fetch], plan_only=True)
            kernels = [p.split()[1] for _, p in comp.groups()]
            # (suffix _w: the warp-per-row form, taken for short rows and for single-pass programs)
            # (suffix _h: half a CTA per row, taken for programs of several passes over rows of 1025 to 4096 elements)
            # (a digit after the suffix: the kernel for rows of exactly that many vectors per thread)
            assert len(kernels) == 1 and re.fullmatch("row_program_static_" + make.__name__ + r"(|_w[2-8]?|_h[2-8]?|_c8[5-8]?)", kernels[0]), \
                (shape, make.__name__, kernels)
            if shape[1] <= 1024:
                assert "_w" in kernels[0][len("row_program_static_" + make.__name__):]
            if shape[1] == 4096:
                single_pass = kernels[0].endswith("_w")  # programs of one pass do not keep the row: a warp per row
                assert single_pass or kernels[0].endswith("_h8"), kernels


def test_passes_that_repeat_steps_with_other_constants_keep_the_interpreter():
    """A specialised row program evaluates the steps its passes share once per row, which is only the same arithmetic
    when those steps carry the same constants: softmax of x * 0.125 is the listed program; with the maximum taken
    of x * 0.125 but the exponent of x * 0.25 the step words are the same and the constants are not, so the matcher
    leaves the program to the interpreting kernel."""
    gen = load_generator()
    desc = dict(gen.ROW_GROUPS)["scaled_softmax"]
    g = cinn_b200.FusedGroup(desc.replace("64,4096", "16,2048"))
    assert g.kernel_names() == ["row_program_static_scaled_softmax_h4"], g.kernel_names()
    g.release()
    other = desc.replace("op subtract z = d mb", "op scale d2 = X ; bias=0.0 bias_after_scale=true scale=0.25\nop subtract z = d2 mb")
    assert other != desc
    g = cinn_b200.FusedGroup(other.replace("fn_static_scaled_softmax", "fn_two_scales"))
    assert g.pattern == "row_program" and g.kernel_names() == ["row_program"], g.kernel_names()
    g.release()
