"""Offline build of libcinn_b200.so for sm_100a (replaces the reference's run-time NVRTC step).

`python -m cinn_b200.build` compiles every file under csrc/ with nvcc and links one shared library next to
this file.  The CUDA runtime is linked statically, so the library loads on a machine without a GPU driver
(planning and description parsing work there; launching does not).
"""
import concurrent.futures
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
OBJ_DIR = os.path.join(HERE, "build")
LIB_PATH = os.path.join(HERE, "libcinn_b200.so")

SOURCES = [
    "ew_kernels.cu",
    "reduce_kernels.cu",
    "reduce_generic.cu",
    "channel_reduce.cu",
    "transform_kernels.cu",
    "rownorm_kernels.cu",
    "rownorm_tma.cu",
    "softmax_safe.cu",
    "ew_chain.cu", "chain_reduce.cu", "ew_static.cu", "ew_dag.cu", "row_prog.cu", "row_prog_half.cu", "row_prog_half_b.cu",
    "ew_chain_int.cu",
    "ew_chain_f64.cu",
    "ew_stream.cu",
    "reduce_static_scratch.cu",
    "peer_reduce.cu",
    "group_desc.cc",
    "group_match.cc",
    "chain_match.cc",
    "runtime.cc",
    "frontend.cc", "program_pass.cc",
    "capi_frontend.cc",
]

# -fmad=false: a*b+c is fused only where fmaf() is written (the x86 path's contraction rule);
# division and sqrt keep their IEEE-rounded defaults, no fast-math, no flush-to-zero.
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-std=c++17", "-O3", "-fmad=false", "-lineinfo",
    "-Xcompiler", "-fPIC,-Wall,-Wno-unused-function",
    "-x", "cu",
]


def _nvcc():
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(nvcc):
        raise RuntimeError("nvcc not found; the kernel library can only be built with the CUDA toolkit")
    return nvcc


def _stale(target, deps):
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def build_library(force=False, verbose=False):
    """Compile csrc/ into libcinn_b200.so; returns the library path.  Up-to-date objects are reused."""
    nvcc = _nvcc()
    os.makedirs(OBJ_DIR, exist_ok=True)
    headers = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".h", ".cuh", ".inc"))]
    headers += [os.path.join(HERE, "..", "include", f) for f in os.listdir(os.path.join(HERE, "..", "include"))]
    headers.append(os.path.abspath(__file__))
    jobs = []
    objs = []
    for src in SOURCES:
        src_path = os.path.join(CSRC, src)
        obj = os.path.join(OBJ_DIR, src + ".o")
        objs.append(obj)
        if force or _stale(obj, [src_path] + headers):
            cmd = [nvcc] + NVCC_FLAGS + ["-c", src_path, "-o", obj]
            if verbose:
                cmd.insert(1, "-Xptxas=-v")
            jobs.append(cmd)

    def run(cmd):
        r = subprocess.run(cmd, capture_output=True, text=True)
        return cmd, r

    if jobs:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(len(jobs), os.cpu_count() or 4)) as ex:
            for cmd, r in ex.map(run, jobs):
                if verbose or r.returncode != 0:
                    sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
                if r.returncode != 0:
                    raise RuntimeError("nvcc failed for " + cmd[-3])
    if jobs or force or _stale(LIB_PATH, objs):
        cmd = [nvcc, "-shared", "-cudart", "static", "-gencode", "arch=compute_100a,code=sm_100a",
               "-o", LIB_PATH] + objs + ["-Xlinker", "--no-undefined"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
            raise RuntimeError("link of libcinn_b200.so failed")
    return LIB_PATH


if __name__ == "__main__":
    print(build_library(force="--force" in sys.argv, verbose="-v" in sys.argv))
