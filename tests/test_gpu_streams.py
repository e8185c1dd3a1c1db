"""A group's first run allocates and zeroes its scratch memory; a run on ANOTHER stream right after it must see the
zeroed ticket counters / partials too (the zeroing is complete before the first call returns)."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_first_run_on_one_stream_then_another_stream(oracle):
    import cinn_b200
    from cinn_b200 import workloads as W
    # channel statistics keep one ticket counter per channel in scratch memory (must start at zero)
    w = W.bn_train_stats((16, 32, 28, 28))
    g = cinn_b200.FusedGroup(w.desc)
    assert g.scratch_bytes > 0
    dev = torch.device("cuda:0")
    ins = [torch.from_numpy(a).to(dev) for a in w.inputs]
    c = w.inputs[0].shape[1]

    def outs():
        return [torch.full((c,), float("nan"), device=dev), torch.full((c,), float("nan"), device=dev)]
    a_out, b_out = outs(), outs()
    sa, sb = torch.cuda.Stream(), torch.cuda.Stream()
    torch.cuda.synchronize()
    g.run(ins + a_out, ctypes.c_void_p(sa.cuda_stream))   # first run: allocates + zeroes the scratch
    sa.synchronize()
    g.run(ins + b_out, ctypes.c_void_p(sb.cuda_stream))   # another stream, no ordering with `sa` needed
    torch.cuda.synchronize()
    x = w.inputs[0].astype(np.float64)
    s1, s2 = x.sum(axis=(0, 2, 3)), (x * x).sum(axis=(0, 2, 3))
    for o in (a_out, b_out):
        assert np.allclose(o[0].cpu().numpy(), s1, rtol=1e-5, atol=1e-3)
        assert np.allclose(o[1].cpu().numpy(), s2, rtol=1e-5, atol=1e-3)
    g.release()


def test_first_run_inside_capture_is_refused_with_a_message():
    import cinn_b200
    from cinn_b200 import workloads as W
    w = W.bn_train_stats((8, 16, 14, 14))
    desc = w.desc.replace(w.group_name, w.group_name + "_cap")
    g = cinn_b200.FusedGroup(desc)
    dev = torch.device("cuda:0")
    ins = [torch.from_numpy(a).to(dev) for a in w.inputs]
    outs = [torch.empty(16, device=dev), torch.empty(16, device=dev)]
    side = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        with torch.cuda.graph(graph, stream=side, capture_error_mode="relaxed"):
            with pytest.raises(cinn_b200._lib.CinnB200Error) as e:
                g.run(ins + outs, ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
            assert "outside stream capture" in str(e.value)
    torch.cuda.synchronize()
    g.run(ins + outs)  # the ordinary first run still works afterwards
    torch.cuda.synchronize()
    g.release()
