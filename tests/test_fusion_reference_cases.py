"""The graphs of the reference's own fusion-pass tests, with the group counts those tests assert.

cinn/hlir/pass/op_fusion_pass_test.cc:22-274 asserts the number of groups after OpFusionPass alone;
cinn/hlir/pass/fusion_merge_pass_test.cc:22-485 asserts it after OpFusionPass and again after FusionMergePass (a few of
its final assertions are commented out in the reference; those cases carry the OpFusionPass count only).  The fusion
pass of this library is one pass with a different algorithm (propose a region, keep it when a prebuilt kernel covers
it), so each case states the reference's final count and this library's, and where they differ, why.  Every case is
planned without a GPU here; tests/test_gpu_fusion_reference_cases.py runs the same programs on the GPU against the
op-by-op oracle."""
import pytest

from cinn_b200 import common
from cinn_b200.frontend import Computation, NetBuilder

TARGET = common.DefaultNVGPUTarget()
F32 = common.Float(32)


def inputs(b, **shapes):
    return {k: b.create_input(F32, v, k) for k, v in shapes.items()}


# name -> (builder function returning the fetched variables, reference count, this library's count, reason if different)
CASES = {}


def case(ref, ours=None, why=""):
    def deco(fn):
        CASES[fn.__name__] = (fn, ref, ref if ours is None else ours, why)
        return fn
    return deco


H, W = 32, 32

# ---- op_fusion_pass_test.cc ------------------------------------------------------------------------------------------


@case(1)
def op_elementwise_fusion_0(b):  # :22-44
    v = inputs(b, A=(H, W), B=(H, W), C=(H, W), D=(H, W))
    return [b.add(b.add(v["A"], v["B"]), b.add(v["C"], v["D"]))]


@case(1)
def op_elementwise_fusion_1(b):  # :46-69
    v = inputs(b, A=(H, W), B=(H, W), C=(H, W), D=(H, W))
    e = b.add(v["A"], v["B"])
    return [b.add(b.add(e, v["C"]), b.add(e, v["D"]))]


@case(1)
def op_broadcast_0(b):  # :71-93
    v = inputs(b, A=(W,), B=(W,), C=(H, W), D=(H, W))
    return [b.add(b.add(v["C"], v["A"], axis=0), b.add(v["D"], v["B"], axis=0))]


@case(1)
def op_broadcast_1(b):  # :95-119
    v = inputs(b, A=(W,), B=(W,), C=(H, W), D=(H, W))
    e, f = b.add(v["A"], v["B"]), b.add(v["C"], v["D"])
    g = b.add(f, e, axis=0)
    return [b.add(b.add(g, v["C"]), v["D"])]


@case(1)
def op_broadcast_2(b):  # :121-141
    v = inputs(b, A=(16,), B=(2, 16, 32, 32))
    return [b.multiply(v["B"], b.reshape(v["A"], [16, 1, 1]))]


@case(2)
def op_reduce_0(b):  # :143-166
    v = inputs(b, A=(W,), B=(W,), C=(H, W), D=(H, W))
    e, f = b.add(v["A"], v["B"]), b.add(v["C"], v["D"])
    return [b.add(e, b.reduce_sum(f, [0]))]


@case(1, 3, "two column reductions of different tensors plus their elementwise consumers: reductions of different inputs are not merged horizontally and the epilogue is a kernel of its own")
def op_reduce_1(b):  # :168-192
    v = inputs(b, A=(W,), B=(W,), C=(H, W), D=(H, W))
    e = b.add(v["A"], v["B"])
    f, g = b.reduce_sum(v["C"], [0]), b.reduce_sum(v["D"], [0])
    return [b.add(g, b.add(e, f))]


@case(2, 3, "the two reductions run over different axes; each keeps its one elementwise consumer outside (a single reduction with a per-row epilogue stays with the dedicated reduction kernels)")
def op_reduce_2(b):  # :194-218
    v = inputs(b, A=(W,), B=(W,), C=(H, W), D=(H, W))
    e, f = b.reduce_sum(v["C"], [0]), b.reduce_sum(v["D"], [1])
    return [b.add(b.add(v["A"], e), b.add(v["B"], f))]


@case(1, 3, "concat is a data-movement kernel of its own (copy_rows), not an operand of the elementwise kernels")
def op_injective_0(b):  # :220-243
    v = inputs(b, A=(H, W), B=(H, W), C=(H, W), D=(2 * H, W))
    return [b.add(v["D"], b.concat([v["C"], b.add(v["A"], v["B"])], 0))]


@case(1, 2, "transpose is a tiled data-movement kernel of its own; expand_dims / broadcast_to fold into the add")
def op_injective_1(b):  # :245-262
    v = inputs(b, A=(1, 19), B=(1, 19, 204))
    d = b.broadcast_to(b.expand_dims(v["A"], [1]), [1, 204, 19], [0, 1, 2])
    return [b.add(d, b.transpose(v["B"], [0, 2, 1]))]


@case(1)
def op_insert_broadcast_to(b):  # :264-282
    v = inputs(b, A=(W,), B=(W,), C=(H, W))
    return [b.add(b.add(v["C"], v["A"], axis=-1), v["B"], axis=-1)]


# ---- fusion_merge_pass_test.cc ---------------------------------------------------------------------------------------


@case(1)
def merge_elementwise_0(b):  # :22-45
    v = inputs(b, A=(H, W), B=(H, W), C=(H, W), D=(H, W))
    e = b.add(v["A"], v["B"])
    return [b.add(e, v["C"]), b.add(e, v["D"])]


@case(1)
def merge_elementwise_1(b):  # :47-71
    v = inputs(b, A=(H, W), B=(H, W), C=(H, W), D=(H, W))
    e, f = b.add(v["A"], v["B"]), b.add(v["C"], v["D"])
    return [b.add(e, f), b.add(e, f)]


@case(1)
def merge_elementwise_2(b):  # :73-100
    v = inputs(b, A=(H, W), B=(H, W), C=(H, W), D=(H, W), E=(H, W), F=(H, W))
    g, h = b.add(v["A"], v["B"]), b.add(v["C"], v["D"])
    return [b.add(v["E"], g), b.add(g, h), b.add(h, v["F"])]


@case(1)
def merge_elementwise_3(b):  # :102-129
    v = inputs(b, A=(H, W), B=(H, W), C=(H, W), D=(H, W), E=(H, W), F=(H, W))
    g = b.add(v["A"], v["B"])
    return [b.add(g, v[k]) for k in "CDEF"]


@case(1)
def merge_elementwise_4(b):  # :131-158
    v = inputs(b, A=(H, W), B=(H, W), C=(H, W), D=(H, W), E=(H, W), F=(H, W))
    g = b.add(v["A"], v["B"])
    i = b.add(g, v["D"])
    return [b.add(g, v["C"]), b.add(i, v["E"]), b.add(i, v["F"])]


@case(1)
def merge_elementwise_5(b):  # :160-180
    v = inputs(b, A=(H, W), B=(H, W))
    return [b.add(v["A"], v["B"]), b.add(v["A"], v["B"])]


@case(1)
def merge_broadcast_0(b):  # :182-205
    v = inputs(b, A=(W,), B=(W,), C=(H, W), D=(H, W))
    return [b.add(b.add(v["C"], v["D"]), b.add(v["A"], v["B"]))]


@case(1)
def merge_broadcast_1(b):  # :207-230
    v = inputs(b, A=(W,), B=(W,), C=(H, W), D=(H, W))
    e = b.add(v["A"], v["B"])
    return [b.add(v["C"], e), b.add(v["D"], e)]


@case(2)
def merge_broadcast_2(b):  # :232-255
    v = inputs(b, A=(W,), B=(W,), C=(W,), D=(H, W))
    e = b.add(v["A"], v["B"])
    return [b.add(v["C"], e), b.add(v["D"], e)]


@case(2)
def merge_broadcast_3(b):  # :257-280
    v = inputs(b, A=(W,), B=(W,), C=(H * W, W), D=(H, W))
    e = b.add(v["A"], v["B"])
    return [b.add(v["C"], e), b.add(v["D"], e)]


@case(2)
def merge_broadcast_4(b):  # :282-307
    v = inputs(b, A=(W,), B=(W,), C=(W,), D=(H, W), E=(H, W))
    f = b.add(v["A"], v["B"])
    return [b.add(v["C"], f), b.add(v["D"], f), b.add(v["E"], f)]


@case(3)
def merge_broadcast_5(b):  # :309-334
    v = inputs(b, A=(W,), B=(W,), C=(W,), D=(H, W), E=(H * W, W))
    f = b.add(v["A"], v["B"])
    return [b.add(v["C"], f), b.add(v["D"], f), b.add(v["E"], f)]


@case(4, 3, "fewer: the shared sum is recomputed inside each of the three reductions instead of being written once (the reference leaves its final count for this case commented out)")
def merge_reduce_0(b):  # :336-358 (final count commented out in the reference: the OpFusionPass count stands)
    v = inputs(b, A=(H, W), B=(H, W))
    c = b.add(v["A"], v["B"])
    return [b.reduce_sum(c, [0]) for _ in range(3)]


@case(2)
def merge_reduce_1(b):  # :360-381
    v = inputs(b, A=(H, W), B=(H, W))
    c = b.add(v["A"], v["B"])
    return [b.reduce_sum(c, [0]), b.reduce_sum(c, [1])]


@case(2, 3, "the shared sum is recomputed inside both reductions (as in the reference), but the two elementwise consumers of the reduced vectors run as one more, two-output kernel instead of inside the reduction kernels")
def merge_reduce_2(b):  # :383-407
    v = inputs(b, A=(H, W), B=(H, W), C=(W,))
    d = b.add(v["A"], v["B"])
    return [b.add(v["C"], b.reduce_sum(d, [0])), b.add(v["C"], b.reduce_sum(d, [1]))]


@case(4, 3, "fewer: the sum runs inside the reduction kernel")
def merge_reduce_3(b):  # :409-433 (final count commented out in the reference)
    v = inputs(b, A=(H, W), B=(H, W), C=(W,), D=(H, W))
    f = b.reduce_sum(b.add(v["A"], v["B"]), [0])
    return [b.add(v["C"], f), b.add(v["D"], f)]


@case(5, 3, "fewer: the sum runs inside the reduction kernel and the two identical consumers share a two-output kernel")
def merge_reduce_4(b):  # :435-460 (final count commented out in the reference)
    v = inputs(b, A=(H, W), B=(H, W), C=(W,), D=(H, W))
    f = b.reduce_sum(b.add(v["A"], v["B"]), [0])
    return [b.add(v["C"], f), b.add(v["D"], f), b.add(v["D"], f)]


@case(1)
def merge_reduce_5(b):  # :462-485
    v = inputs(b, A=(128, 128), B=(128, 128))
    c = b.add(v["A"], v["B"])
    return [b.reduce_sum(v["A"], [1]), b.reduce_sum(v["B"], [1]), b.reduce_sum(c, [1])]


def build(name):
    fn, ref, ours, why = CASES[name]
    b = NetBuilder(name)
    fetch = fn(b)
    return b, fetch, ref, ours, why


@pytest.mark.parametrize("name", sorted(CASES))
def test_group_count(name):
    b, fetch, ref, ours, why = build(name)
    comp = Computation.build_and_compile(TARGET, b, plan_only=True, fetch=[str(f) for f in fetch])
    got = len([1 for _, p in comp.groups() if not p.startswith("reshape_alias")])
    assert got == ours, (name, got, [p for _, p in comp.groups()])
    if ours != ref:
        assert why, "a count that differs from the reference's needs its reason stated"


def test_every_reference_case_is_here():
    assert len([n for n in CASES if n.startswith("op_")]) == 11
    assert len([n for n in CASES if n.startswith("merge_")]) == 18
