#!/usr/bin/env python
"""Benchmark of the fused-group kernels on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl b200|reference]

A step is one launch of the headline fused group, cast_fp16(tanh((X + bias) * 0.5)) with X fp32 [64,1024,1024]
and bias [1024] broadcast on the last axis, through the group's C-ABI entry point.  With N > 1 (one process per
GPU under torch.distributed.run) every rank runs the same group on its own shard-sized copy (weak scaling, the
group shards on axis 0 with no communication); the reported value is the whole-job GB/s over the slowest rank.
One JSON line is printed by rank 0.  `--impl reference` times the CPU restatement of the reference's x86 path on
the host cores instead (rank 0 only).
"""
import argparse
import ctypes
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

HEADLINE_SHAPE = (64, 1024, 1024)
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the headline kernel at full size, from the ncu
# capture summarised in profiles/ncu_bias_scale_tanh_cast.md (268.5 MB read + 95.0 MB written; the write-back L2
# still holds part of the 134 MB output when the kernel ends).
HEADLINE_DRAM_TRAFFIC_BYTES = 363450000
METRIC = "fused-group HBM throughput"
UNIT = "GB/s"


def measured_peak_gbs():
    """(HBM GB/s used as the roofline denominator, where it came from)."""
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons of one GPU through NVML while the timed region runs."""

    def __init__(self, index, period_s=0.02):
        super().__init__(daemon=True)
        self.index, self.period = index, period_s
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop_evt = threading.Event()
        self.ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            self.nv = None

    def _sample(self):
        nv = self.nv
        self.samples.append(int(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM)))
        try:
            mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
        except Exception:
            mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h))
        names = {
            0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
            0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting", 0x10: "sync_boost",
        }
        for bit, name in names.items():
            if mask & bit:
                self.reasons.add(name)

    def run(self):
        if not self.ok:
            return
        while not self._stop_evt.is_set():
            try:
                self._sample()
            except Exception:
                break
            time.sleep(self.period)

    def stop(self):
        self._stop_evt.set()
        self.join(timeout=2)
        med = int(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


def cpu_reference_run(steps, warmup):
    """Times the CPU restatement of the reference's x86 path on the headline group, all host threads."""
    from oracle import x86_oracle
    from cinn_b200 import workloads as W
    # torchrun exports OMP_NUM_THREADS=1; the CPU arm uses every core this process may run on instead.
    threads = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else x86_oracle.num_threads()
    w = W.bias_scale_tanh_cast(HEADLINE_SHAPE)
    x, bias = w.inputs
    for _ in range(max(warmup, 1)):
        x86_oracle.bias_scale_tanh_f16(x, bias, 0.5, 0.0, threads=threads)
    t0 = time.perf_counter()
    for _ in range(steps):
        x86_oracle.bias_scale_tanh_f16(x, bias, 0.5, 0.0, threads=threads)
    dt = (time.perf_counter() - t0) / steps
    return w.algorithmic_bytes() / dt / 1e9, dt * 1e3, threads


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    steps = min(args.steps, 10)
    warm = min(args.warmup, 2)
    gbs, ms, threads = cpu_reference_run(steps, warm)
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warm, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "bias_scale_tanh_cast X f32[64,1024,1024] + bias[1024] -> f16", "elements": 67108864},
        "cpu_baseline": {"value": gbs, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": "full headline group per step, OpenMP over rows, %d threads" % threads},
        "e2e": {"value": gbs, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "elements_per_s": 67108864 / (ms * 1e-3),
    }
    print(json.dumps(line))
    return 0


def time_group(group, tensors_sets, iters, warmup, torch):
    """Average device time (ms) of one launch of `group`, rotating through the given argument sets."""
    stream = torch.cuda.current_stream()
    sp = ctypes.c_void_p(stream.cuda_stream)
    bound = [group.bind(ts) for ts in tensors_sets]
    for i in range(warmup):
        pods, _ = bound[i % len(bound)]
        group.run_entry(pods, len(tensors_sets[0]), sp)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for i in range(iters):
        pods, _ = bound[i % len(bound)]
        group.run_entry(pods, len(tensors_sets[0]), sp)
    e1.record(stream)
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / iters


def graph_launch_us(group, tensors, torch, launches=100, replays=20):
    """Device time per launch (us) of `launches` launches of the group captured into one CUDA graph."""
    pods, keep = group.bind(tensors)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        sp = ctypes.c_void_p(side.cuda_stream)
        group.run_entry(pods, len(tensors), sp)  # warm-up outside the capture
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(launches):
                group.run_entry(pods, len(tensors), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    graph.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(replays):
        graph.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) * 1e3 / (launches * replays)


def TORCH_OF_NUMPY(torch):
    return {np.dtype(np.float32): torch.float32, np.dtype(np.float16): torch.float16,
            np.dtype(np.float64): torch.float64, np.dtype(np.int32): torch.int32, np.dtype(np.int64): torch.int64,
            np.dtype(np.bool_): torch.bool}


def side_groups(torch, dev, peak, only=None):
    """Per-group throughput of the other fused groups (device-resident inputs, kernel time only)."""
    import cinn_b200
    from cinn_b200 import workloads as W
    out = {}

    def dev_inputs(w, reps):
        sets = []
        for _ in range(reps):
            ins = [torch.from_numpy(a).to(dev) for a in w.inputs]
            o = torch.empty(w.out_shape, dtype=TORCH_OF_NUMPY(torch)[np.dtype(w.out_dtype)], device=dev)
            more = [torch.empty(sh, dtype=TORCH_OF_NUMPY(torch)[np.dtype(dt)], device=dev) for dt, sh in w.more_outputs]
            sets.append(ins + [o] + more)
        return sets

    plan = [
        ("add_relu_1x3x224x224", lambda: W.add_relu((1, 3, 224, 224)), 4, "L2-resident (1.8 MB): launch-latency-bound"),
        ("add_relu_stacked_256x3x224x224", lambda: W.add_relu((256, 3, 224, 224), name="fn_add_relu_stacked"), 2,
         "256 stacked copies so that the working set exceeds L2"),
        ("reduce_sum_axis2_128x1024x1024", lambda: W.reduce_sum_last((128, 1024, 1024)), 1, ""),
        ("reduce_max_axis0_128x1024x1024", lambda: W.reduce_max_first((128, 1024, 1024)), 1, ""),
        ("softmax_f32_16384x4096", lambda: W.softmax((16384, 4096)), 2, ""),
        ("softmax_f16_16384x4096", lambda: W.softmax((16384, 4096), half=True), 2, ""),
        ("layer_norm_f32_16384x4096", lambda: W.layer_norm((16384, 4096)), 2, ""),
        ("layer_norm_f16_16384x4096", lambda: W.layer_norm((16384, 4096), half=True), 2, ""),
        ("bn_relu_f32_256x64x112x112", lambda: W.bn_relu((256, 64, 112, 112)), 1, ""),
        ("bn_relu_f16_256x64x112x112", lambda: W.bn_relu((256, 64, 112, 112), half=True), 1, ""),
        ("softmax_max_subtracted_f32_16384x4096", lambda: W.softmax_safe((16384, 4096)), 2, "decomposed softmax, mode != fast"),
        ("softmax_max_subtracted_f16_16384x4096", lambda: W.softmax_safe((16384, 4096), half=True), 2, ""),
        # data movement either side of the groups
        ("transpose_nchw_to_nhwc_f32_256x64x112x112", lambda: W.transpose((256, 64, 112, 112), (0, 2, 3, 1)), 1, ""),
        ("transpose_nhwc_to_nchw_f16_256x112x112x64", lambda: W.transpose((256, 112, 112, 64), (0, 3, 1, 2), "float16"), 1, ""),
        ("transpose_matrix_f32_8192x8192", lambda: W.transpose((8192, 8192), (1, 0)), 1, ""),
        ("concat_axis1_f32_2x(4096x8192)", lambda: W.concat([(4096, 8192), (4096, 8192)], 1), 1, ""),
        # batch_norm_train as the reference decomposes it: one statistics pass (two outputs) + one normalisation pass
        ("bn_train_stats_256x64x112x112", lambda: W.bn_train_stats((256, 64, 112, 112)), 1,
         "sum and sum of squares per channel in one read of x"),
        ("bn_train_apply_256x64x112x112", lambda: W.bn_train_apply((256, 64, 112, 112)), 1, ""),
        ("bn_grad_stats_256x64x112x112", lambda: W.bn_grad_stats((256, 64, 112, 112)), 1,
         "sum(dy) and sum(dy * (x - mean)) per channel in one read of dy and x"),
        ("bn_grad_apply_256x64x112x112", lambda: W.bn_grad_apply((256, 64, 112, 112)), 1, ""),
        # the generic families: any other elementwise chain / element type (interpreted program, not a dedicated kernel)
        ("generic_chain_abs_add_f32_8192x8192", lambda: W.generic_chain("abs_add_f32"), 1, "generic chain kernel"),
        ("generic_chain_select_f32_8192x8192", lambda: W.generic_chain("select_f32"), 1, "generic chain kernel"),
        ("generic_chain_greater_than_f32_8192x8192", lambda: W.generic_chain("greater_than_f32"), 1, "generic chain kernel"),
        ("generic_chain_abs_add_i32_8192x8192", lambda: W.generic_chain("abs_add_i32"), 1, "generic integer chain kernel"),
        ("generic_chain_affine_f64_8192x8192", lambda: W.generic_chain("affine_f64"), 1, "generic float64 chain kernel"),
        ("generic_reduce_sum_f16_rows_16384x8192", lambda: W.generic_reduce("sum", "float16", axis=1), 2, ""),
        ("generic_reduce_sum_f16_cols_16384x8192", lambda: W.generic_reduce("sum", "float16", axis=0), 2, ""),
        ("generic_reduce_max_i32_rows_16384x8192", lambda: W.generic_reduce("max", "int32", axis=1), 1, ""),
        ("generic_reduce_sum_i32_cols_16384x8192", lambda: W.generic_reduce("sum", "int32", axis=0), 1, ""),
        ("generic_reduce_all_bool_rows_16384x8192", lambda: W.generic_reduce("all", "bool", axis=1), 4, ""),
        ("generic_tree_f32_8192x8192", lambda: W.chain_tree(), 1, "(A+B)*(C-D): chain kernel with temporaries"),
        ("generic_two_outputs_f32_8192x8192", lambda: W.chain_two_outputs(), 1,
         "pre = X + bias and relu(pre) from one kernel: one read, two writes"),
        ("bn_train_stats_f16_256x64x112x112", lambda: W.bn_train_stats((256, 64, 112, 112), half=True), 1,
         "fp16 x widened in the load; sum and sum of squares per channel"),
        ("bn_train_apply_f16_256x64x112x112", lambda: W.bn_train_apply((256, 64, 112, 112), half=True), 1, "fp16 storage"),
        # a reduction with an elementwise chain as its operand: the chain runs inside the reduction kernel
        ("chain_reduce_sum_abs_diff_rows_8192x8192", lambda: W.chain_reduce("sum_abs_diff", axis=1), 1, "chain + reduce, one kernel"),
        ("chain_reduce_sum_abs_diff_cols_8192x8192", lambda: W.chain_reduce("sum_abs_diff", axis=0), 1, "chain + reduce, one kernel"),
        ("chain_reduce_sum_sigmoid_affine_rows_8192x8192", lambda: W.chain_reduce("sum_sigmoid_affine", axis=1), 1,
         "chain + reduce, one kernel"),
    ]
    if not only or any(o in "add_relu_1x3x224x224" for o in only):
        # config 1 through NetBuilder / Computation, timed by the library's own ExecuteTest loop (no Python per launch)
        from cinn_b200 import common
        from cinn_b200.frontend import Computation, NetBuilder
        b = NetBuilder("c1")
        a_ = b.create_input(common.Float(32), (1, 3, 224, 224), "A")
        b_ = b.create_input(common.Float(32), (1, 3, 224, 224), "B")
        b.relu(b.add(a_, b_))
        comp = Computation.build_and_compile(common.DefaultNVGPUTarget(), b)
        out["add_relu_1x3x224x224_execute_test"] = {
            "us_per_run": round(comp.execute_test(5000) * 1e3, 3),
            "note": "Program::ExecuteTest of the one-group program: host clock over 5000 back-to-back runs"}
        del comp
    for name, make, reps, note in plan:
        if only and not any(o in name for o in only):
            continue
        w = make()
        g = cinn_b200.FusedGroup(w.desc)
        sets = dev_inputs(w, reps)
        ms = time_group(g, sets, iters=50, warmup=10, torch=torch)
        gbs = g.algorithmic_bytes / (ms * 1e-3) / 1e9
        out[name] = {"ms": round(ms, 5), "GB/s": round(gbs, 1), "frac_of_peak": round(gbs / peak, 4),
                     "elements_per_s": g.elements / (ms * 1e-3), "kernels": g.kernel_names(),
                     "bytes": g.algorithmic_bytes}
        if note:
            out[name]["note"] = note
        if name == "add_relu_1x3x224x224":
            # The 1.8 MB group is launch-bound: 100 launches captured in a CUDA graph remove the host launch cost.
            out[name]["us_per_launch_in_cuda_graph"] = round(graph_launch_us(g, sets[0], torch), 3)
        g.release()
        del sets
        torch.cuda.empty_cache()
    return out


PROFILE_GROUPS = {
    "bias_scale_tanh_cast": lambda W: W.bias_scale_tanh_cast(HEADLINE_SHAPE),
    "add_relu": lambda W: W.add_relu((256, 3, 224, 224), name="fn_add_relu_stacked"),
    "reduce_sum": lambda W: W.reduce_sum_last((128, 1024, 1024)),
    "reduce_max": lambda W: W.reduce_max_first((128, 1024, 1024)),
    "softmax_f32": lambda W: W.softmax((16384, 4096)),
    "softmax_f16": lambda W: W.softmax((16384, 4096), half=True),
    "layer_norm_f32": lambda W: W.layer_norm((16384, 4096)),
    "layer_norm_f16": lambda W: W.layer_norm((16384, 4096), half=True),
    "bn_relu_f32": lambda W: W.bn_relu((256, 64, 112, 112)),
    "bn_relu_f16": lambda W: W.bn_relu((256, 64, 112, 112), half=True),
    "transpose_nchw_to_nhwc": lambda W: W.transpose((256, 64, 112, 112), (0, 2, 3, 1)),
    "softmax_safe_f32": lambda W: W.softmax_safe((16384, 4096)),
    "bn_train_stats": lambda W: W.bn_train_stats((256, 64, 112, 112)),
    "bn_train_apply": lambda W: W.bn_train_apply((256, 64, 112, 112)),
    "bn_grad_stats": lambda W: W.bn_grad_stats((256, 64, 112, 112)),
    "bn_grad_apply": lambda W: W.bn_grad_apply((256, 64, 112, 112)),
    "chain_abs_add_f32": lambda W: W.generic_chain("abs_add_f32"),
    "chain_select_f32": lambda W: W.generic_chain("select_f32"),
    "chain_abs_add_i32": lambda W: W.generic_chain("abs_add_i32"),
    "reduce_sum_f16_rows": lambda W: W.generic_reduce("sum", "float16", axis=1),
    "reduce_sum_i32_cols": lambda W: W.generic_reduce("sum", "int32", axis=0),
    "chain_reduce_rows": lambda W: W.chain_reduce("sum_abs_diff", axis=1),
    "chain_tree": lambda W: W.chain_tree(),
    "bn_train_stats_f16": lambda W: W.bn_train_stats((256, 64, 112, 112), half=True),
}


def run_profile_case(args):
    """One group alone, a handful of launches: the command that is run under ncu (and once without it)."""
    import torch
    import cinn_b200
    from cinn_b200 import workloads as W
    for kv in args.option or []:
        k, v = kv.split("=")
        cinn_b200._lib.check(cinn_b200.lib().cinn_b200_set_option(k.encode(), int(v)))
    dev = torch.device("cuda", 0)
    w = PROFILE_GROUPS[args.profile](W)
    g = cinn_b200.FusedGroup(w.desc)
    ins = [torch.from_numpy(a).to(dev) for a in w.inputs]
    out = [torch.empty(w.out_shape, dtype=TORCH_OF_NUMPY(torch)[np.dtype(w.out_dtype)], device=dev)]
    out += [torch.empty(sh, dtype=TORCH_OF_NUMPY(torch)[np.dtype(dt)], device=dev) for dt, sh in w.more_outputs]
    g.run(ins + out)  # status-checked first launch
    ms = time_group(g, [ins + out], iters=max(args.steps, 1), warmup=max(args.warmup, 1), torch=torch)
    print(json.dumps({"profile": args.profile, "kernels": g.kernel_names(), "ms": ms,
                      "bytes_per_launch": g.algorithmic_bytes,
                      "GB/s": g.algorithmic_bytes / (ms * 1e-3) / 1e9}))
    return 0


def strong_scaling_headline(torch, dist, dev, world, rank):
    """The headline group with its TOTAL size fixed and axis 0 split over the ranks (no communication): every rank
    runs its [64 / world, 1024, 1024] slice; argument sets rotate through more than 2 x L2 so that inputs come from
    HBM.  Reported beside the weak-scaling headline; the speed-up over one GPU is total bytes / max-over-ranks time."""
    import cinn_b200
    from cinn_b200 import sharding
    from cinn_b200 import workloads as W
    start, count = sharding.shard_range(HEADLINE_SHAPE[0], world, rank)
    if count == 0:
        return None
    shape = (count,) + tuple(HEADLINE_SHAPE[1:])
    w = W.bias_scale_tanh_cast(shape, name="fn_bias_scale_tanh_cast_shard%d" % rank)
    g = cinn_b200.FusedGroup(w.desc)
    per_set = 6 * count * HEADLINE_SHAPE[1] * HEADLINE_SHAPE[2]
    nsets = max(2, int(300e6 // per_set) + 1)
    bias = torch.randn(HEADLINE_SHAPE[-1], device=dev) * 0.1
    sets = [[torch.randn(shape, device=dev), bias, torch.empty(shape, dtype=torch.float16, device=dev)]
            for _ in range(nsets)]
    torch.cuda.synchronize()
    dist.barrier()
    ms = time_group(g, sets, iters=100, warmup=10, torch=torch)
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    total = 6 * HEADLINE_SHAPE[0] * HEADLINE_SHAPE[1] * HEADLINE_SHAPE[2] + 4 * HEADLINE_SHAPE[2]
    g.release()
    return {"ms_per_step_max_over_ranks": round(ms, 5), "GB/s_whole_job": round(total / (ms * 1e-3) / 1e9, 1),
            "slice_per_rank": list(shape), "argument_sets_rotated": nsets, "scaling": "strong",
            "note": "no communication; speed-up over one GPU = this GB/s / the N=1 value"}


def sharded_reduce_max(torch, dist, dev, world, rank, peak):
    """reduce_max over axis 0 of [128,1024,1024] with axis 0 sharded over the ranks (strong scaling): the local
    column reduction alone, and with the NCCL all-reduce(MAX) of the 4 MiB partials that finishes it."""
    from cinn_b200 import sharding
    full = (128, 1024, 1024)
    op = sharding.ShardedReduceAxis0.from_library("max", full, world, rank)
    x = torch.randn(op.local_shape, device=dev)
    out = torch.empty(op.out_shape, device=dev)
    stream = torch.cuda.current_stream()

    def timed(fn, iters=30, warm=5):
        for _ in range(warm):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(iters):
            fn()
        e1.record(stream)
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / iters], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed_in_graph(fn, iters=20, replays=5):
        """The same calls replayed from one CUDA graph: no per-launch host work, so the device time shows even where
        a launch from Python (some 15-20 us) is longer than the kernel."""
        try:
            fn()
            torch.cuda.synchronize()
            side = torch.cuda.Stream()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, stream=side):
                    for _ in range(iters):
                        fn()
            graph.replay()
            torch.cuda.synchronize()
            dist.barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(stream)
            for _ in range(replays):
                graph.replay()
            e1.record(stream)
            torch.cuda.synchronize()
            t = torch.tensor([e0.elapsed_time(e1) / (iters * replays)], device=dev, dtype=torch.float64)
        except Exception as exc:  # reported, not hidden: the eager numbers stand on their own
            sys.stderr.write("graph timing failed on rank %d: %r\n" % (rank, exc))
            t = torch.tensor([float("nan")], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        v = float(t.item())
        return None if v != v else round(v, 5)

    ms_local = timed(lambda: op.local_reduce(x, out))
    ms_total = timed(lambda: op(x, out))
    g_local = timed_in_graph(lambda: op.local_reduce(x, out))
    g_total = timed_in_graph(lambda: op(x, out))
    # The same reduction with the exchange fused into the kernel (peer stores over NVLink, no NCCL call).
    fused_full = sharding.FusedShardedReduceAxis0("max", full, world, rank, all_gather=True)
    ms_fused_full = timed(lambda: fused_full(x, out))
    g_fused_full = timed_in_graph(lambda: fused_full(x, out))
    check = out.clone()
    op(x, out)
    torch.cuda.synchronize()
    same = bool(torch.equal(check, out))
    fused_band = sharding.FusedShardedReduceAxis0("max", full, world, rank, all_gather=False)
    band_out = torch.empty(fused_band.out_shape, device=dev)
    ms_fused_band = timed(lambda: fused_band(x, band_out))
    g_fused_band = timed_in_graph(lambda: fused_band(x, band_out))
    dist.barrier()
    fused_full.close()
    fused_band.close()
    total_bytes = 4 * (full[0] * full[1] * full[2]) + 4 * full[1] * full[2]
    gbs = lambda ms: round(total_bytes / (ms * 1e-3) / 1e9, 1)  # noqa: E731
    return {"ms_local_kernel": round(ms_local, 5), "ms_with_nccl_allreduce": round(ms_total, 5),
            "ms_fused_kernel_full_result": round(ms_fused_full, 5),
            "ms_fused_kernel_owned_band": round(ms_fused_band, 5),
            "fused_equals_nccl_result": same,
            "ms_in_cuda_graph": {"local_kernel": g_local, "with_nccl_allreduce": g_total,
                                 "fused_kernel_full_result": g_fused_full, "fused_kernel_owned_band": g_fused_band},
            "GB/s_whole_job_local": gbs(ms_local), "GB/s_whole_job_with_nccl_allreduce": gbs(ms_total),
            "GB/s_whole_job_fused_full_result": gbs(ms_fused_full),
            "GB/s_whole_job_fused_owned_band": gbs(ms_fused_band),
            "frac_of_peak_per_gpu_fused_full_result": round(total_bytes / (ms_fused_full * 1e-3) / 1e9 / world / peak, 4),
            "scaling": "strong",
            "collective": "nccl all_reduce(MAX) of 4 MiB per rank, vs one kernel per rank exchanging over NVLink peer memory"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-side-groups", action="store_true", help="skip the per-group table of the other configs")
    ap.add_argument("--only", nargs="*", default=None, help="side groups whose name contains one of these")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--profile", choices=sorted(PROFILE_GROUPS), default=None,
                    help="run only this group for --warmup + --steps launches (the small case captured by ncu)")
    ap.add_argument("--option", nargs="*", default=None, help="planner options key=value (see cinn_b200_set_option)")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference_arm(args)
    if args.profile:
        return run_profile_case(args)

    import torch
    import torch.distributed as dist
    import cinn_b200
    from cinn_b200 import workloads as W

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the fused-group kernels have no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    warmup = max(args.warmup, 3)
    peak, peak_src = measured_peak_gbs()

    # Headline group.  Two argument sets (2 x 403 MB) so that consecutive launches never touch the same lines;
    # each set is itself larger than the 126 MB L2.
    w = W.bias_scale_tanh_cast(HEADLINE_SHAPE)
    g = cinn_b200.FusedGroup(w.desc)
    x_host = torch.from_numpy(w.inputs[0]).pin_memory()
    bias_host = torch.from_numpy(w.inputs[1]).pin_memory()
    out_host = torch.empty(w.out_shape, dtype=torch.float16).pin_memory()
    sets = []
    for _ in range(2):
        sets.append([x_host.to(dev, non_blocking=True), bias_host.to(dev, non_blocking=True),
                     torch.empty(w.out_shape, dtype=torch.float16, device=dev)])
    torch.cuda.synchronize()

    stream = torch.cuda.current_stream()
    sp = ctypes.c_void_p(stream.cuda_stream)
    bound = [g.bind(ts) for ts in sets]
    for i in range(warmup):
        g.run_entry(bound[i % 2][0], 3, sp)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    sampler = ClockSampler(local_rank)
    sampler.start()
    launches0 = cinn_b200.lib().cinn_b200_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    e0.record(stream)
    for i in range(args.steps):
        g.run_entry(bound[i % 2][0], 3, sp)
    e1.record(stream)
    torch.cuda.synchronize()
    launches = cinn_b200.lib().cinn_b200_launch_count() - launches0
    clocks = sampler.stop()
    total_ms = e0.elapsed_time(e1)
    if world > 1:
        t = torch.tensor([total_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        dist.barrier()
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    bytes_per_launch = g.algorithmic_bytes
    value = bytes_per_launch * world / (ms_per_step * 1e-3) / 1e9
    per_gpu = value / world

    # End to end through the host-buffer entry point: pinned host inputs -> device -> kernel -> pinned host output.
    e2e_steps = max(3, min(args.steps, 20))
    host_arrays = [x_host, bias_host, out_host]
    for _ in range(3):
        g.run_host(host_arrays, device=local_rank)
    if world > 1:
        dist.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        g.run_host(host_arrays, device=local_rank)
    e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    if world > 1:
        t = torch.tensor([e2e_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = bytes_per_launch * world / (e2e_ms * 1e-3) / 1e9

    line = {
        "metric": METRIC, "value": round(value, 2), "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "bias_scale_tanh_cast X f32[64,1024,1024] + bias[1024] -> f16 (per GPU)",
                   "elements": g.elements, "bytes_per_launch": bytes_per_launch,
                   "l2": "inputs (268 MB) larger than L2; two argument sets alternated",
                   "sharding": "axis 0, no collective; each rank runs the full-size group (weak scaling)"},
        "elements_per_s": g.elements * world / (ms_per_step * 1e-3),
        "roofline": {"bound": "hbm", "achieved": round(per_gpu, 2), "peak": peak, "unit": "GB/s",
                     "frac": round(per_gpu / peak, 4), "traffic": HEADLINE_DRAM_TRAFFIC_BYTES,
                     "traffic_unit": "bytes per launch (dram read + write, one ncu --set full capture)",
                     "algorithmic_bytes": bytes_per_launch, "peak_source": peak_src,
                     "kernel": g.kernel_names()[0]},
        "e2e": {"value": round(e2e_value, 3), "unit": UNIT, "ms_per_step": e2e_ms,
                "h2d_bytes_per_step": int(x_host.numel() * 4 + bias_host.numel() * 4),
                "d2h_bytes_per_step": int(out_host.numel() * 2), "steps": e2e_steps},
        "gpu_launches": int(launches),
        "clocks": clocks,
    }
    g.release()
    del sets, bound
    torch.cuda.empty_cache()

    if rank == 0 and not args.no_cpu_baseline:
        gbs, ms, threads = cpu_reference_run(steps=20, warmup=2)
        line["cpu_baseline"] = {"value": round(gbs, 3), "unit": UNIT, "cores": threads, "kind": "port", "ms": ms,
                                "sample": "full headline group, 20 passes after 2 warm-up passes, OpenMP over rows, %d threads" % threads}
    if rank == 0 and world == 1 and not args.no_side_groups:
        line["groups"] = side_groups(torch, dev, peak, args.only)
    if world > 1 and not args.no_side_groups:
        sharded = sharded_reduce_max(torch, dist, dev, world, rank, peak)
        strong = strong_scaling_headline(torch, dist, dev, world, rank)
        if rank == 0:
            line["groups"] = {"reduce_max_axis0_128x1024x1024_sharded_on_axis0": sharded,
                              "headline_group_total_size_fixed_sharded_on_axis0": strong}
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
