"""The allocation-free column reduction (cinn_b200_col_reduce_f32_static_scratch), collected last.

It serves callers that may not let the library allocate device memory (a framework that owns the device pool, or
a loop where cudaMalloc's device-wide synchronisation is unacceptable): its partial results live in a fixed array
inside the library.  The test calls it through the C ABI twice in a row on different data and compares each
result with the regular compiled-group entry point (which allocates its scratch), using the tolerances of the
other reduction tests: bit-exact for max/min, rtol 1e-5 plus the summation-order allowance for sums."""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _group_result(kind, x, shape):
    import torch
    import cinn_b200
    r, inner = shape
    desc = ("group fn_noalloc_ref_%s\ninput X float32 %d,%d\nop reduce_%s var_0 = X ; dim=0 keep_dim=false\n"
            "output var_0 float32 %d\n" % (kind, r, inner, kind, inner))
    g = cinn_b200.FusedGroup(desc)
    out = torch.empty(inner, device="cuda")
    g.run([x, out])
    torch.cuda.synchronize()
    assert g.scratch_bytes > 0, "the comparison path is expected to be the split (scratch-using) plan"
    g.release()
    return out.cpu().numpy()


@pytest.mark.parametrize("kind,code", [("max", 2), ("sum", 0), ("min", 3)])
def test_static_scratch_matches_compiled_group_twice_in_a_row(kind, code):
    import torch
    import cinn_b200
    L = cinn_b200.lib()
    shape = (8192, 96)  # few columns, many rows: the planner splits the rows and needs scratch
    gen = torch.Generator(device="cuda").manual_seed(21)
    for call in range(2):
        x = torch.randn(shape, device="cuda", generator=gen)
        y = torch.full((shape[1],), float("nan"), device="cuda")
        rc = L.cinn_b200_col_reduce_f32_static_scratch(code, ctypes.c_void_p(x.data_ptr()),
                                                       ctypes.c_void_p(y.data_ptr()), 1, shape[0], shape[1], None)
        assert rc == 0, L.cinn_b200_last_error()
        torch.cuda.synchronize()
        got = y.cpu().numpy()
        want = _group_result(kind, x, shape)
        if kind in ("max", "min"):
            assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), (kind, call)
        else:
            rms = float(x.float().pow(2).mean().sqrt())
            atol = 2e-6 * np.sqrt(shape[0]) * rms  # two different summation trees of r terms each
            assert (np.abs(got - want) <= 1e-5 * np.abs(want) + atol).all(), (kind, call)
            ref64 = x.double().sum(0).cpu().numpy()
            assert (np.abs(got - ref64) <= 1e-5 * np.abs(ref64) + atol).all(), (kind, call)


def test_static_scratch_middle_axis_and_unaligned():
    import torch
    import cinn_b200
    L = cinn_b200.lib()
    x = torch.randn(3, 4096, 10, device="cuda")  # inner = 10: scalar path
    y = torch.empty(3, 10, device="cuda")
    rc = L.cinn_b200_col_reduce_f32_static_scratch(2, ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(y.data_ptr()),
                                                   3, 4096, 10, None)
    assert rc == 0, L.cinn_b200_last_error()
    torch.cuda.synchronize()
    assert torch.equal(y, x.max(dim=1).values)


def test_static_scratch_rejects_what_does_not_fit():
    import torch
    import cinn_b200
    L = cinn_b200.lib()
    # 600000 output columns: two partials of the output (1.2 M floats) exceed the 1 Mi-float array, so the call is
    # refused whatever plan the shape would get.  The buffers are real and large enough for the shape all the same:
    # an entry point that may launch is never handed pointers it could overrun.
    r, inner = 64, 600000
    x = torch.zeros(r, inner, device="cuda")
    y = torch.full((inner,), 7.0, device="cuda")
    rc = L.cinn_b200_col_reduce_f32_static_scratch(0, ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(y.data_ptr()),
                                                   1, r, inner, None)
    assert rc == -6 and b"static scratch holds" in L.cinn_b200_last_error()
    torch.cuda.synchronize()
    assert bool((y == 7.0).all()), "a refused call must not launch anything"
    # the largest output that is accepted: exactly half the array
    inner = 524288
    x = torch.randn(64, inner, device="cuda")
    y = torch.empty(inner, device="cuda")
    rc = L.cinn_b200_col_reduce_f32_static_scratch(2, ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(y.data_ptr()),
                                                   1, 64, inner, None)
    assert rc == 0, L.cinn_b200_last_error()
    torch.cuda.synchronize()
    assert torch.equal(y, x.max(dim=0).values)
    # an unknown reduce kind is refused too (real buffers again: no call that could launch gets a pointer it may not use)
    assert L.cinn_b200_col_reduce_f32_static_scratch(7, ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(y.data_ptr()),
                                                     1, 64, inner, None) == -1
    torch.cuda.synchronize()
