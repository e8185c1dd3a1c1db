"""Host-side re-entrancy of the group registry (no GPU needed).

Compile time in the reference is multi-threaded (ParallelCompiler runs its tasks on std::threads,
cinn/hlir/framework/parallel_compiler.cc:99-111, 219-226) and launch entry points must be re-entrant across
Computation objects.  Here one thread keeps recompiling and releasing a group name while others query and run it:
a run holds its own reference to the plan, so neither may free it under a running call."""
import ctypes
import threading

import pytest

import cinn_b200
from cinn_b200 import runtime as rt

DESC = ("group fn_thread_race\ninput A float32 64,256\ninput B float32 64,256\n"
        "op elementwise_add t0 = A B ; axis=-1\nop relu t1 = t0\noutput t1 float32 64,256\n")


def _has_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def test_recompile_and_release_while_other_threads_use_the_group():
    L = cinn_b200.lib()
    stop = threading.Event()
    errors = []
    fn = ctypes.c_void_p()
    assert L.cinn_b200_compile_group(DESC.encode(), ctypes.byref(fn)) == 0
    host = (ctypes.c_float * (64 * 256))()
    bufs = [rt.make_buffer(ctypes.addressof(host), "float32", (64, 256)) for _ in range(3)]
    pods = rt.make_pods(bufs)
    run_it = not _has_gpu()  # with a GPU present the launch would really run on these host pointers: query only

    def churn():
        f = ctypes.c_void_p()
        while not stop.is_set():
            rc = L.cinn_b200_compile_group(DESC.encode(), ctypes.byref(f))
            if rc != 0:
                errors.append(("compile", rc))
            L.cinn_b200_release_group(b"fn_thread_race")

    def use():
        pat = ctypes.create_string_buffer(128)
        ab = ctypes.c_longlong()
        while not stop.is_set():
            rc = L.cinn_b200_group_info(b"fn_thread_race", pat, 128, ctypes.byref(ab), None, None, None)
            if rc == 0 and ab.value != 3 * 64 * 256 * 4:
                errors.append(("info", ab.value))
            elif rc not in (0, -3):
                errors.append(("info rc", rc))
            if run_it:
                # no device here: the call validates the arguments against the plan and fails at the launch
                # (CUDA error) or finds the name gone; it must never crash
                rc = L.cinn_b200_group_run(b"fn_thread_race", pods, 3, None)
                if rc not in (-3, -4):
                    errors.append(("run rc", rc))

    threads = [threading.Thread(target=churn)] + [threading.Thread(target=use) for _ in range(3)]
    for t in threads:
        t.start()
    stop.wait(1.5)
    stop.set()
    for t in threads:
        t.join()
    assert not errors, errors[:5]
    L.cinn_b200_release_group(b"fn_thread_race")


def test_many_threads_compile_distinct_groups():
    L = cinn_b200.lib()
    errors = []

    def work(i):
        name = "fn_thread_many_%d" % i
        desc = DESC.replace("fn_thread_race", name)
        f = ctypes.c_void_p()
        for _ in range(20):
            if L.cinn_b200_compile_group(desc.encode(), ctypes.byref(f)) != 0:
                errors.append(i)
            if not L.cinn_b200_lookup(name.encode()):
                errors.append(("lookup", i))
            if L.cinn_b200_release_group(name.encode()) != 0:
                errors.append(("release", i))

    threads = [threading.Thread(target=work, args=(i,)) for i in range(8)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors[:5]
