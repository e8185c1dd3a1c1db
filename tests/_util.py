"""Helpers shared by the GPU parity tests: run a workload's group through the C ABI on cuda:0."""
import numpy as np
import torch

import cinn_b200

NP2TORCH = {np.dtype(np.float32): torch.float32, np.dtype(np.float16): torch.float16,
            np.dtype(np.float64): torch.float64, np.dtype(np.int32): torch.int32, np.dtype(np.int64): torch.int64,
            np.dtype(np.bool_): torch.bool}


def run_group(workload, misalign=0, check_canary=True):
    """Compile the workload's group, run it on device copies of its inputs, return the output as numpy.

    misalign > 0 offsets every device buffer by that many elements from its allocation, to exercise the
    unaligned code paths.  The output buffer is surrounded by canary elements that must survive the launch.
    """
    g = cinn_b200.FusedGroup(workload.desc)
    dev = torch.device("cuda:0")
    ins = []
    for a in workload.inputs:
        t = torch.empty(a.size + misalign, dtype=NP2TORCH[a.dtype], device=dev)
        view = t[misalign:].view(a.shape)
        view.copy_(torch.from_numpy(a))
        ins.append(view)
    n_out = int(np.prod(workload.out_shape))
    pad = 64
    out_t = NP2TORCH[np.dtype(workload.out_dtype)]
    canary = True if out_t == torch.bool else 77
    raw = torch.full((n_out + 2 * pad + misalign,), canary, dtype=out_t, device=dev)
    out = raw[pad + misalign: pad + misalign + n_out].view(workload.out_shape)
    g.run(ins + [out])
    torch.cuda.synchronize()
    if check_canary:
        head = raw[: pad + misalign].float().cpu().numpy()
        tail = raw[pad + misalign + n_out:].float().cpu().numpy()
        assert (head == float(canary)).all() and (tail == float(canary)).all(), "kernel wrote outside its output buffer"
    res = out.cpu().numpy()
    g.release()
    return res, g
