"""The programs of the reference's fusion-pass tests (tests/test_fusion_reference_cases.py) run on the GPU and
checked against the op-by-op CPU oracle: every fetched value of every case, whatever groups the fusion pass made of
it.  Elementwise results are bit-exact (the oracle contracts the same Mul + Add pairs); sums are compared at the
reduction tolerance.  A second set of programs exercises what the register-program kernel adds on top of the chain
kernels: values used several times, three and four outputs, 16-bit storage, constants, selects."""
import numpy as np
import pytest

from cinn_b200 import common
from cinn_b200.frontend import Computation, NetBuilder
from tests.test_fusion_reference_cases import CASES, build, inputs
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


def run_and_check(b, fetch, seed, exact=True, rtol=1e-5, atol=1e-4):
    comp = Computation.build_and_compile(TARGET, b, fetch=[str(f) for f in fetch])
    rng = np.random.default_rng(seed)
    feeds = {}
    for t in comp.get_input_tensors():
        dtype, shape, _ = t._info()
        dt = {"float32": np.float32, "float16": np.float16, "bool": np.bool_}[dtype]
        arr = (rng.random(shape) > 0.5) if dt is np.bool_ else rng.standard_normal(shape).astype(dt)
        feeds[t.name] = arr
        t.from_numpy(arr, TARGET)
    comp.execute()
    want = oracle_program(comp, feeds)
    for f in fetch:
        got, ref = comp.get_tensor(str(f)).numpy(TARGET), want[str(f)]
        assert got.shape == tuple(ref.shape), (str(f), got.shape, ref.shape)
        if exact:
            assert np.array_equal(got.view(np.uint8), np.ascontiguousarray(ref).view(np.uint8)), \
                (str(f), [p for _, p in comp.groups()], float(np.abs(got.astype(np.float64) - ref).max()))
        else:
            assert np.allclose(got, ref, rtol=rtol, atol=atol), (str(f), [p for _, p in comp.groups()])
    return comp


@pytest.mark.parametrize("name", sorted(CASES))
def test_reference_fusion_case_on_the_gpu(name):
    b, fetch, _, _, _ = build(name)
    run_and_check(b, fetch, seed=sum(map(ord, name)), exact="reduce" not in name)


def _dag_programs():
    F32, F16 = common.Float(32), common.Float(16)

    def shared_value_four_outputs(b):
        v = inputs(b, A=(33, 260), B=(33, 260), C=(33, 260), D=(260,))
        g = b.multiply(v["A"], v["B"])
        return [b.add(g, v["C"]), b.subtract(g, v["D"]), b.relu(g), b.add(b.sigmoid(g), g)]

    def fma_contraction_choice(b):
        # add(mul, mul): the right product is contracted, the left one is rounded (cinn/optim/lower_intrin.cc:45-50)
        v = inputs(b, A=(64, 128), B=(64, 128), C=(64, 128), D=(64, 128))
        s = b.add(b.multiply(v["A"], v["B"]), b.multiply(v["C"], v["D"]))
        return [s, b.multiply(s, s)]

    def half_storage(b):
        x = b.create_input(F16, (48, 256), "X")
        y = b.create_input(F16, (48, 256), "Y")
        s = b.add(x, y)
        return [b.multiply(s, x), b.subtract(s, y), b.relu(s)]

    def constants_and_select(b):
        v = inputs(b, A=(40, 96), B=(40, 96))
        m = b.greater_than(v["A"], v["B"])
        lo = b.fill_constant([40, 96], -0.5, "lo")
        t = b.select(m, v["A"], lo)
        return [t, b.scale(t, 2.0, 1.0), b.max(t, v["B"])]

    def odd_size_takes_the_scalar_tail(b):
        v = inputs(b, A=(7, 13), B=(7, 13), C=(13,))
        e = b.add(v["A"], v["B"])
        return [b.add(e, v["C"]), b.multiply(e, e), b.tanh(e)]

    def adam_step(b):
        # both moments and the parameter of an Adam step from one read of the gradient (the second moment enters
        # squared here, so that random test data never puts a negative number under the root)
        v = inputs(b, P=(96, 512), G=(96, 512), M=(96, 512), V=(96, 512))
        vv = b.multiply(v["V"], v["V"])
        m2 = b.add(b.scale(v["M"], 0.9, 0.0), b.scale(v["G"], 0.1, 0.0))
        v2 = b.add(b.scale(vv, 0.999, 0.0), b.scale(b.multiply(v["G"], v["G"]), 0.001, 0.0))
        upd = b.divide(m2, b.scale(b.sqrt(v2), 1.0, 1e-8))
        return [m2, v2, b.add(v["P"], b.scale(upd, -0.001, 0.0))]

    return [shared_value_four_outputs, fma_contraction_choice, half_storage, constants_and_select,
            odd_size_takes_the_scalar_tail, adam_step]


@pytest.mark.parametrize("make", _dag_programs(), ids=lambda f: f.__name__)
def test_register_programs_match_the_oracle(make):
    b = NetBuilder(make.__name__)
    fetch = make(b)
    # sigmoid / tanh go through the device's expf, within 2 ulp of the host library's: those programs are compared
    # at a few ulp, everything else bit for bit
    approx = make.__name__ in ("shared_value_four_outputs", "odd_size_takes_the_scalar_tail")
    comp = run_and_check(b, fetch, seed=3, exact=not approx, rtol=5e-7, atol=2e-7)
    # one kernel either way: a register program, or (add of two products, squared) a chain with temporaries
    assert [p.split()[0] for _, p in comp.groups()] in (["ew_dag"], ["ew_chain"]), [p for _, p in comp.groups()]
