"""Row programs (row_prog.cu): reductions over the trailing axes with elementwise ops before, between and after them,
one kernel per group, against the op-by-op CPU oracle.  Sums are compared at the reduction tolerance (the kernel folds
per-thread partials in a tree, the oracle serially); values computed from them inherit it."""
import numpy as np
import pytest

import cinn_b200
from cinn_b200 import common
from cinn_b200.frontend import Computation, NetBuilder
from oracle import x86_graph_eval as ge
from tests.test_gpu_frontend import oracle_program

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True, scope="module")
def fuse_interpreted_programs():
    """These tests are about the register-program and row-program kernels themselves, interpreting forms included, so
    the fusion pass is asked to form their groups even where only the interpreting kernel takes them."""
    import cinn_b200
    L = cinn_b200.lib()
    L.cinn_b200_set_option(b"fuse_interpreted_programs", 1)
    yield
    L.cinn_b200_set_option(b"fuse_interpreted_programs", 0)
TARGET = common.DefaultNVGPUTarget()
F32 = common.Float(32)


def l2_normalise(b, rows, r):
    x = b.create_input(F32, (rows, r), "X")
    s = b.reduce_sum(b.multiply(x, b.identity(x)), [1], keep_dim=True)
    return [b.divide(x, b.broadcast_to(b.sqrt(s), [rows, r], [0, 1]))]


def centre(b, rows, r):
    x = b.create_input(F32, (rows, r), "X")
    m = b.divide(b.reduce_sum(x, [1]), b.fill_constant([rows], float(r)))
    return [b.subtract(x, b.broadcast_to(m, [rows, r], [0]))]


def shifted_exponentials_with_bias(b, rows, r):
    # three passes: the maximum, the sum of exp(x - max), the result
    x = b.create_input(F32, (rows, r), "X")
    g = b.create_input(F32, (r,), "G")
    mx = b.broadcast_to(b.reduce_max(x, [1]), [rows, r], [0])
    e = b.exp(b.scale(b.subtract(x, mx), 0.5, 0.0))  # (not the softmax composition, which has its own kernel)
    s = b.broadcast_to(b.reduce_sum(e, [1]), [rows, r], [0])
    return [b.add(b.divide(e, s), g)]


def three_sums(b, rows, r):
    a, c = b.create_input(F32, (rows, r), "A"), b.create_input(F32, (rows, r), "B")
    return [b.reduce_sum(a, [1]), b.reduce_sum(c, [1]), b.reduce_sum(b.add(a, c), [1])]


def centred_and_its_variance(b, rows, r):
    x = b.create_input(F32, (rows, r), "X")
    n = b.fill_constant([rows], float(r))
    m = b.divide(b.reduce_sum(x, [1]), n)
    xc = b.subtract(x, b.broadcast_to(m, [rows, r], [0]))
    var = b.divide(b.reduce_sum(b.multiply(xc, b.identity(xc)), [1]), n)
    return [xc, var]


def exp_minus_its_maximum(b, rows, r):
    x = b.create_input(F32, (rows, r), "X")
    e = b.exp(x)
    return [b.subtract(e, b.broadcast_to(b.reduce_max(e, [1]), [rows, r], [0]))]


def _tabled(index):
    """The builder programs of the specialised-kernel table (cinn_b200/csrc/gen_static_chains.py), at any shape."""
    import importlib.util
    import os
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "cinn_b200", "csrc", "gen_static_chains.py")
    spec = importlib.util.spec_from_file_location("gen_static_chains", path)
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    name = gen.builder_row_programs()[index].__name__

    def make(b, rows, r):
        return gen.builder_row_programs(rows, r)[index](b)
    make.__name__ = name
    return make


def scaled_softmax(b, rows, r):
    # attention scores: the scaling joins the max-subtracted softmax in one kernel
    x = b.create_input(F32, (rows, r), "X")
    d = b.scale(x, 0.125, 0.0)
    e = b.exp(b.subtract(d, b.broadcast_to(b.reduce_max(d, [1]), [rows, r], [0])))
    return [b.divide(e, b.broadcast_to(b.reduce_sum(e, [1]), [rows, r], [0]))]


def masked_softmax(b, rows, r):
    x, m = b.create_input(F32, (rows, r), "X"), b.create_input(F32, (rows, r), "M")
    d = b.add(b.scale(x, 0.125, 0.0), m)
    e = b.exp(b.subtract(d, b.broadcast_to(b.reduce_max(d, [1]), [rows, r], [0])))
    return [b.divide(e, b.broadcast_to(b.reduce_sum(e, [1]), [rows, r], [0]))]


PROGRAMS = [l2_normalise, centre, shifted_exponentials_with_bias, three_sums, centred_and_its_variance,
            exp_minus_its_maximum, scaled_softmax, masked_softmax] + [_tabled(i) for i in range(10)]
SHAPES = [(70, 1024), (9, 4096), (33, 1001), (5, 2050), (128, 64), (7, 8192), (6, 6144), (11, 2048), (13, 512), (21, 256), (10, 3072), (9, 768), (7, 1536), (6, 2560), (5, 3584), (12, 384), (11, 640), (10, 896), (4, 5120), (3, 7168)]  # warp / half CTA / CTA per row, ragged, short and long rows


@pytest.mark.parametrize("make", PROGRAMS, ids=lambda f: f.__name__)
@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "%dx%d" % s)
def test_row_program_matches_the_oracle(make, shape):
    rows, r = shape
    b = NetBuilder(make.__name__)
    fetch = make(b, rows, r)
    comp = Computation.build_and_compile(TARGET, b, fetch=[str(f) for f in fetch])
    assert [p.split()[0] for _, p in comp.groups()] == ["row_program"], [p for _, p in comp.groups()]
    rng = np.random.default_rng(rows * 7 + r)
    feeds = {}
    for t in comp.get_input_tensors():
        _, shp, _ = t._info()
        feeds[t.name] = rng.standard_normal(shp).astype(np.float32)
        t.from_numpy(feeds[t.name], TARGET)
    comp.execute()
    want = oracle_program(comp, feeds)
    for f in fetch:
        got, ref = comp.get_tensor(str(f)).numpy(TARGET), np.asarray(want[str(f)])
        assert got.shape == ref.shape
        scale = max(1.0, float(np.abs(ref).max()))
        assert np.allclose(got, ref, rtol=2e-5, atol=2e-6 * np.sqrt(r) * scale), \
            (str(f), float(np.abs(got - ref).max()), [p for _, p in comp.groups()])


def test_reduction_with_a_per_row_epilogue_as_one_group():
    """relu(reduce_sum(x) * a + c): given as ONE group it is one row-program launch (the fusion pass itself leaves such
    a group to the dedicated reduction kernels unless a specialised row program exists)."""
    import torch
    rows, r = 300, 1536
    desc = ("group fn_row_affine_relu\ninput X float32 %d,%d\ninput a float32 %d\ninput c float32 %d\n"
            "op reduce_sum s = X ; dim=1 keep_dim=false\nop elementwise_mul t = s a ; axis=-1\n"
            "op elementwise_add u = t c ; axis=-1\nop relu y = u\noutput y float32 %d\n" % (rows, r, rows, rows, rows))
    g = cinn_b200.FusedGroup(desc)
    assert g.pattern == "row_program" and g.launches == 1
    rng = np.random.default_rng(5)
    ins = [rng.standard_normal((rows, r)).astype(np.float32), rng.standard_normal(rows).astype(np.float32),
           rng.standard_normal(rows).astype(np.float32)]
    out = torch.empty(rows, device="cuda")
    g.run([torch.from_numpy(a).cuda() for a in ins] + [out])
    torch.cuda.synchronize()
    g.release()
    want = ge.run_all(desc, ins)["y"]
    assert np.allclose(out.cpu().numpy(), want, rtol=2e-5, atol=1e-4)


def test_softmax_with_other_constants_in_the_later_passes():
    """max(x * 0.125) but exp(x * 0.25 - max): the passes repeat the same step words with other constants, so the
    value a specialised kernel would keep from the first pass is not the one the later passes need; the matcher
    gives the program to the interpreting kernel, and the result is the oracle's."""
    import torch
    rows, r = 37, 4096
    desc = ("group fn_two_scales\ninput X float32 %d,%d\n"
            "op scale d = X ; bias=0.0 bias_after_scale=true scale=0.125\n"
            "op reduce_max mx = d ; dim=1 keep_dim=false\nop broadcast_to mb = mx ; broadcast_axes=0 out_shape=%d,%d\n"
            "op scale d2 = X ; bias=0.0 bias_after_scale=true scale=0.25\nop subtract z = d2 mb ; axis=-1\nop exp e = z\n"
            "op reduce_sum s = e ; dim=1 keep_dim=false\nop broadcast_to sb = s ; broadcast_axes=0 out_shape=%d,%d\n"
            "op divide y = e sb ; axis=-1\noutput y float32 %d,%d\n" % ((rows, r) * 4))
    g = cinn_b200.FusedGroup(desc)
    assert g.pattern == "row_program" and g.kernel_names() == ["row_program"], g.kernel_names()
    x = np.random.default_rng(3).standard_normal((rows, r)).astype(np.float32)
    out = torch.empty((rows, r), device="cuda")
    g.run([torch.from_numpy(x).cuda(), out])
    torch.cuda.synchronize()
    g.release()
    want = ge.run_all(desc, [x])["y"]
    assert np.allclose(out.cpu().numpy(), want, rtol=2e-5, atol=1e-6)


@pytest.mark.parametrize("form", [32, 128, 256])
@pytest.mark.parametrize("index", [0, 1, 2, 5])  # rms_norm, standardise, log_softmax, min_max_normalise
@pytest.mark.parametrize("shape", [(37, 4096), (19, 2052), (41, 1024)], ids=lambda s: "%dx%d" % s)
def test_specialised_row_program_in_every_form(form, index, shape):
    """The three forms of a specialised row program -- a warp, half a CTA (two rows per CTA, a named barrier per half)
    or a CTA per row -- forced through the `rowp_form` option, against the oracle."""
    rows, r = shape
    make = _tabled(index)
    L = cinn_b200.lib()
    L.cinn_b200_set_option(b"rowp_form", form)
    try:
        b = NetBuilder("%s_form%d" % (make.__name__, form))
        fetch = make(b, rows, r)
        comp = Computation.build_and_compile(TARGET, b, fetch=[str(f) for f in fetch])
    finally:
        L.cinn_b200_set_option(b"rowp_form", 0)
    kernels = [p.split()[1] for _, p in comp.groups()]
    want_suffix = {32: "_w", 128: "_h", 256: ""}[form]
    # (a digit after the suffix: the kernel for rows of exactly that many vectors per thread of the row's group)
    exact = {(32, 1024): "8", (128, 4096): "8", (128, 1024): "2"}.get((form, r), "")
    assert kernels == ["row_program_static_" + make.__name__ + want_suffix + exact], kernels
    rng = np.random.default_rng(rows * 11 + r + form)
    feeds = {}
    for t in comp.get_input_tensors():
        _, shp, _ = t._info()
        feeds[t.name] = rng.standard_normal(shp).astype(np.float32)
        t.from_numpy(feeds[t.name], TARGET)
    comp.execute()
    want = oracle_program(comp, feeds)
    for f in fetch:
        got, ref = comp.get_tensor(str(f)).numpy(TARGET), np.asarray(want[str(f)])
        scale = max(1.0, float(np.abs(ref).max()))
        assert np.allclose(got, ref, rtol=2e-5, atol=2e-6 * np.sqrt(r) * scale), \
            (str(f), float(np.abs(got - ref).max()), kernels)


@pytest.mark.parametrize("dtype", ["float16", "bfloat16"])
@pytest.mark.parametrize("shape", [(64, 4096), (37, 1024), (5, 8192)], ids=lambda s: "%dx%d" % s)
def test_rms_norm_with_16_bit_storage_is_one_specialised_kernel(dtype, shape):
    """x, the weight and the result stored as 16-bit floats, fp32 arithmetic between the casts: one row-program kernel
    from the table; against a float64 evaluation at the 16-bit tolerance."""
    import torch
    rows, r = shape
    T = common.Float16() if dtype == "float16" else common.BFloat16()
    b = NetBuilder("rms_norm_" + dtype)
    x, g = b.create_input(T, (rows, r), "X"), b.create_input(T, (r,), "G")
    xf, gf = b.cast(x, "float32"), b.cast(g, "float32")
    inv = b.rsqrt(b.scale(b.reduce_sum(b.multiply(xf, xf), [1]), 1.0 / r, 1e-6))
    y = b.cast(b.multiply(b.multiply(xf, b.broadcast_to(inv, [rows, r], [0])), gf), dtype)
    comp = Computation.build_and_compile(TARGET, b, fetch=[str(y)], plan_only=True)
    groups = comp.groups()
    assert len(groups) == 1 and groups[0][1].split()[1].startswith("row_program_static_rms_norm_"), groups
    tt = torch.float16 if dtype == "float16" else torch.bfloat16
    gen = torch.Generator(device="cuda").manual_seed(rows + r)
    X = torch.randn((rows, r), device="cuda", generator=gen).to(tt)
    G = (1.0 + 0.1 * torch.randn((r,), device="cuda", generator=gen)).to(tt)
    out = torch.empty((rows, r), device="cuda", dtype=tt)
    fg = cinn_b200.FusedGroup(groups[0][0].replace(groups[0][0].splitlines()[0], "group fn_rms16_%s_%d_%d" % (dtype, rows, r)))
    fg.run([X, G, out])
    torch.cuda.synchronize()
    fg.release()
    xd = X.double()
    want = xd * torch.rsqrt((xd * xd).sum(1, keepdim=True) / r + 1e-6) * G.double()
    assert bool(((out.double() - want).abs() <= 1e-2 * want.abs() + 1e-3).all())
