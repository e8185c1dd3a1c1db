"""Every chain kernel specialised at build time against the interpreting kernel it replaces: the same group, the
same inputs, once with the substitution on and once with it off, bit for bit -- both run chain_step(), so any
difference would be a miscompiled specialisation.  Sizes that leave a ragged tail, and a misaligned case that takes
the scalar path, are included; a few entries are also checked against the CPU oracle through the usual parity
helpers elsewhere (abs_add, select, trees, bias + relu with a second output)."""
import importlib.util
import os

import numpy as np
import pytest
import torch

import cinn_b200

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_spec = importlib.util.spec_from_file_location(
    "gen_static_chains", os.path.join(ROOT, "cinn_b200", "csrc", "gen_static_chains.py"))
GEN = importlib.util.module_from_spec(_spec)
_spec.loader.exec_module(GEN)

TORCH_T = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16, "bool": torch.bool,
           "int32": torch.int32, "int64": torch.int64, "float64": torch.float64}


def _tensors(desc, seed, misalign):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    ins, outs = [], []
    for line in desc.splitlines():
        w = line.split()
        if not w or w[0] not in ("input", "output"):
            continue
        shape = tuple(int(d) for d in w[3].split(","))
        n = int(np.prod(shape))
        dt = TORCH_T[w[2]]
        raw = torch.empty(n + misalign, dtype=dt, device="cuda")
        view = raw[misalign:].view(shape)
        if w[0] == "input":
            if dt == torch.bool:
                view.copy_(torch.rand(shape, device="cuda", generator=gen) > 0.5)
            elif dt in (torch.int32, torch.int64):
                view.copy_(torch.randint(-40000, 40000, shape, device="cuda", generator=gen, dtype=dt))
            else:
                # positive and negative values, magnitudes around one, a few exact zeros
                v = torch.randn(shape, device="cuda", generator=gen) * 1.5
                v[torch.rand(shape, device="cuda", generator=gen) < 0.01] = 0.0
                view.copy_(v.to(dt))
            ins.append(view)
        else:
            outs.append(view)
    return ins, outs


def _run(desc, name, static, seed, misalign):
    L = cinn_b200.lib()
    L.cinn_b200_set_option(b"enable_static_chains", 1 if static else 0)
    try:
        g = cinn_b200.FusedGroup(desc.replace("fn_static_", "fn_%s_" % name))
    finally:
        L.cinn_b200_set_option(b"enable_static_chains", 1)
    ins, outs = _tensors(desc, seed, misalign)
    for o in outs:
        o.view(torch.uint8).fill_(0x5A)
    g.run(ins + outs)
    torch.cuda.synchronize()
    kernels = g.kernel_names()
    g.release()
    return [o.view(torch.uint8).cpu().numpy().copy() for o in outs], kernels


ALL_CHAINS = GEN.GROUPS + GEN.INT_GROUPS + GEN.F64_GROUPS


@pytest.mark.parametrize("name,desc", ALL_CHAINS, ids=[n for n, _ in ALL_CHAINS])
@pytest.mark.parametrize("variant", ["table_shape", "ragged", "misaligned"])
def test_static_kernel_equals_interpreter(name, desc, variant):
    if variant == "ragged":
        # 61 x 1028 / 3 x 16 x 9 x 28: vector path plus a tail, a last extent that keeps the addressing modes
        desc = desc.replace("64,1024", "61,1028").replace(" 1024\n", " 1028\n").replace("8,16,32,32", "3,16,9,28")
    misalign = 1 if variant == "misaligned" else 0
    got_s, k_s = _run(desc, "s_" + variant, True, seed=11, misalign=misalign)
    got_i, k_i = _run(desc, "i_" + variant, False, seed=11, misalign=misalign)
    assert all(k.startswith("ew_chain_") for k in k_i), k_i
    if "_static_" not in k_s[0]:
        pytest.skip("no specialised kernel for this entry (%s)" % k_s[0])
    # A specialised ROW program may run in another form than the interpreter (half a CTA or a warp per row: another
    # summation tree) and evaluates exp / tanh / sigmoid through the approximate exponential and reciprocal; its
    # results are of the reduction class.  Register programs are the interpreter's bit for bit.
    approximate = k_i[0] == "row_program"
    for a, b in zip(got_s, got_i):
        if approximate:
            fa, fb = a.view(np.float32), b.view(np.float32)
            assert np.allclose(fa, fb, rtol=2e-5, atol=4e-6 * float(np.abs(fb).max())), (name, variant, k_s)
        else:
            assert np.array_equal(a, b), (name, variant, k_s, int((a != b).sum()))


@pytest.mark.parametrize("name,desc", GEN.REDUCE_GROUPS, ids=[n for n, _ in GEN.REDUCE_GROUPS])
@pytest.mark.parametrize("shape", ["64,1024", "61,1028", "4,65536", "4096,8"])
def test_static_chain_reduction_equals_interpreter(name, desc, shape):
    """The reductions with a chain as operand: the specialised kernel folds the same values in the same order."""
    rows, cols = (int(d) for d in shape.split(","))
    axis = 1 if name.endswith("_rows") else 0
    out = str(rows if axis == 1 else cols)
    lines = []
    for l in desc.splitlines():
        w = l.split()
        if w[0] in ("input", "output") and w[3] == "64,1024":
            l = " ".join(w[:3] + [shape])
        elif w[0] == "input" and w[3] == "1024":
            l = " ".join(w[:3] + [str(cols)])
        elif w[0] == "output":
            l = " ".join(w[:3] + [out])
        lines.append(l)
    desc = "\n".join(lines) + "\n"
    got_s, k_s = _run(desc, "rs", True, seed=5, misalign=0)
    got_i, k_i = _run(desc, "ri", False, seed=5, misalign=0)
    assert k_i[0].startswith("chain_reduce_"), k_i
    if not k_s[0].startswith("chain_reduce_static_"):
        pytest.skip("no specialised kernel at this shape (%s)" % k_s[0])
    for a, b in zip(got_s, got_i):
        if "sigmoid" in name:
            # the specialised reductions use the approximate exponential and reciprocal: reduction tolerance
            fa, fb = a.view(np.float32), b.view(np.float32)
            assert np.allclose(fa, fb, rtol=1e-5, atol=1e-5 * np.abs(fb).max()), (name, shape, k_s)
        else:
            assert np.array_equal(a, b), (name, shape, k_s, int((a != b).sum()))


@pytest.mark.parametrize("name,desc", GEN.DAG_GROUPS + GEN.ROW_GROUPS, ids=[n for n, _ in GEN.DAG_GROUPS + GEN.ROW_GROUPS])
@pytest.mark.parametrize("variant", ["table_shape", "other_size"])
def test_static_register_and_row_programs_equal_their_interpreters(name, desc, variant):
    """Register programs (several outputs, shared values) and row programs (reductions with elementwise ops around
    them): the kernel with the program as template arguments against the interpreting kernel -- bit for bit for the
    register programs (same steps), at the reduction tolerance for the row programs."""
    if variant == "other_size":
        desc = (desc.replace("64,4096", "37,1028").replace("shape=64 ", "shape=37 ").replace(" 64\n", " 37\n")
                .replace("value=4096.0", "value=1028.0").replace("64,1024", "61,1028").replace(" 1024\n", " 1028\n"))
    got_s, k_s = _run(desc, "ps_" + variant, True, seed=17, misalign=0)
    got_i, k_i = _run(desc, "pi_" + variant, False, seed=17, misalign=0)
    if k_i[0] not in ("ew_dag", "row_program"):
        pytest.skip("this entry is a chain (%s): covered by the chain table" % k_i[0])
    if "_static_" not in k_s[0]:
        pytest.skip("no specialised kernel for this entry (%s)" % k_s[0])
    # A specialised ROW program may run in another form than the interpreter (half a CTA or a warp per row: another
    # summation tree) and evaluates exp / tanh / sigmoid through the approximate exponential and reciprocal; its
    # results are of the reduction class.  Register programs are the interpreter's bit for bit.
    approximate = k_i[0] == "row_program"
    for a, b in zip(got_s, got_i):
        if approximate:
            fa, fb = a.view(np.float32), b.view(np.float32)
            assert np.allclose(fa, fb, rtol=2e-5, atol=4e-6 * float(np.abs(fb).max())), (name, variant, k_s)
        else:
            assert np.array_equal(a, b), (name, variant, k_s, int((a != b).sum()))
