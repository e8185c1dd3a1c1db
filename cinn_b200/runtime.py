"""Host-side mirror of the reference runtime's argument model, over ctypes.

`cinn_buffer_t` / `cinn_pod_value_t` are laid out exactly as in cinn/runtime/cinn_runtime.h:186-292, 390-460
(the C declarations this module mirrors are in include/cinn_runtime_abi.h).  `FusedGroup` is the analogue of
the reference's `hlir::framework::Instruction` (cinn/hlir/framework/instruction.cc:77-165): it holds the
entry point of one compiled group and calls it with a pod array of inputs followed by outputs.
"""
import ctypes

import numpy as np

from . import _lib

CINN_BUFFER_MAX_DIMS = 8

# cinn_type_code_t (cinn_runtime.h:51-58)
TYPE_INT, TYPE_UINT, TYPE_FLOAT, TYPE_HANDLE, TYPE_BFLOAT = 0, 1, 2, 3, 4
# cinn_type_code<T>() (cinn_runtime.h:467-488)
POD_INT32, POD_INT64, POD_FLOAT, POD_DOUBLE, POD_VOIDP, POD_BUFFERP = 0, 1, 2, 3, 4, 7
BUFFER_ON_DEVICE = 1 << 1


class cinn_type_t(ctypes.Structure):
    _fields_ = [("code", ctypes.c_int), ("bits", ctypes.c_uint8), ("lanes", ctypes.c_uint16),
                ("num_asterisks", ctypes.c_uint8)]


class cinn_buffer_t(ctypes.Structure):
    _fields_ = [
        ("device", ctypes.c_int),
        ("device_interface", ctypes.c_void_p),
        ("memory", ctypes.c_void_p),
        ("flag", ctypes.c_uint64),
        ("type", cinn_type_t),
        ("dimensions", ctypes.c_int32),
        ("dims", ctypes.c_int * CINN_BUFFER_MAX_DIMS),
        ("lazy", ctypes.c_char),
        ("memory_size", ctypes.c_uint64),
        ("align", ctypes.c_uint16),
        ("external_malloc", ctypes.c_void_p),
        ("external_free", ctypes.c_void_p),
    ]


class cinn_value_t(ctypes.Union):
    _fields_ = [("v_int64", ctypes.c_int64), ("v_float64", ctypes.c_double), ("v_handle", ctypes.c_void_p)]


class cinn_pod_value_t(ctypes.Structure):
    _fields_ = [("type_code_", ctypes.c_int), ("value_", cinn_value_t)]


assert ctypes.sizeof(cinn_type_t) == 12
assert ctypes.sizeof(cinn_buffer_t) == 120
assert ctypes.sizeof(cinn_pod_value_t) == 16

# dtype name -> (type code, bits, numpy dtype or None)
DTYPES = {
    "float32": (TYPE_FLOAT, 32, np.float32),
    "float16": (TYPE_FLOAT, 16, np.float16),
    "bfloat16": (TYPE_BFLOAT, 16, None),
    "float64": (TYPE_FLOAT, 64, np.float64),
    "int32": (TYPE_INT, 32, np.int32),
    "int64": (TYPE_INT, 64, np.int64),
    "bool": (TYPE_INT, 1, np.bool_),
    "uint8": (TYPE_UINT, 8, np.uint8),
}


def dtype_bytes(name):
    return (DTYPES[name][1] + 7) // 8


def make_buffer(ptr, dtype, shape, on_device=True):
    """A cinn_buffer_t describing `shape` elements of `dtype` at address `ptr` (device or host memory)."""
    if len(shape) > CINN_BUFFER_MAX_DIMS:
        raise ValueError("cinn_buffer_t holds at most %d dimensions" % CINN_BUFFER_MAX_DIMS)
    code, bits, _ = DTYPES[dtype]
    b = cinn_buffer_t()
    b.device = 0
    b.memory = ptr
    b.flag = BUFFER_ON_DEVICE if on_device else 0
    b.type = cinn_type_t(code, bits, 1, 0)
    b.dimensions = len(shape)
    n = 1
    for i, d in enumerate(shape):
        b.dims[i] = int(d)
        n *= int(d)
    b.lazy = b"\x00"
    b.memory_size = n * ((bits + 7) // 8)
    b.align = 0
    return b


def make_pods(buffers):
    """cinn_pod_value_t[len(buffers)], each holding a cinn_buffer_t* (type code 7)."""
    pods = (cinn_pod_value_t * len(buffers))()
    for i, b in enumerate(buffers):
        pods[i].type_code_ = POD_BUFFERP
        pods[i].value_.v_handle = ctypes.addressof(b)
    return pods


def torch_dtype_name(t):
    import torch
    return {torch.float32: "float32", torch.float16: "float16", torch.bfloat16: "bfloat16",
            torch.float64: "float64", torch.int32: "int32", torch.int64: "int64", torch.bool: "bool",
            torch.uint8: "uint8"}[t.dtype]


class FusedGroup:
    """One compiled fused group: entry point + facts, callable with device tensors or host arrays."""

    def __init__(self, desc_text):
        L = _lib.lib()
        fn = ctypes.c_void_p()
        _lib.check(L.cinn_b200_compile_group(desc_text.encode(), ctypes.byref(fn)))
        self.desc = desc_text
        self.name = next(l.split()[1] for l in desc_text.splitlines() if l.strip().startswith("group"))
        self._fn_addr = fn.value
        self.fn = _lib.LOWER_FUNC_PTR_G(fn.value)
        pat = ctypes.create_string_buffer(128)
        ab, el, ls, sc = ctypes.c_longlong(), ctypes.c_longlong(), ctypes.c_int(), ctypes.c_longlong()
        _lib.check(L.cinn_b200_group_info(self.name.encode(), pat, 128, ctypes.byref(ab), ctypes.byref(el),
                                          ctypes.byref(ls), ctypes.byref(sc)))
        self.pattern = pat.value.decode()
        self.algorithmic_bytes = ab.value
        self.elements = el.value
        self.launches = ls.value
        self.scratch_bytes = sc.value

    def kernel_names(self):
        L = _lib.lib()
        out = []
        for i in range(self.launches):
            buf = ctypes.create_string_buffer(128)
            _lib.check(L.cinn_b200_group_kernel(self.name.encode(), i, buf, 128))
            out.append(buf.value.decode())
        return out

    def launch_text(self):
        """The launch plan as text (kernel, grid, block and every kernel parameter of each launch)."""
        L = _lib.lib()
        need = L.cinn_b200_group_launch_text(self.name.encode(), None, 0)
        if need < 0:
            _lib.check(int(need))
        buf = ctypes.create_string_buffer(int(need))
        L.cinn_b200_group_launch_text(self.name.encode(), buf, int(need))
        return buf.value.decode()

    def bind(self, tensors):
        """Pod array for device tensors (inputs then outputs).  Keep the returned tuple alive while it is used."""
        bufs = [make_buffer(t.data_ptr(), torch_dtype_name(t), tuple(t.shape)) for t in tensors]
        return make_pods(bufs), bufs

    def run(self, tensors, stream=None):
        """Launch on torch device tensors through the status-returning entry point."""
        pods, keep = self.bind(tensors)
        _lib.check(_lib.lib().cinn_b200_group_run(self.name.encode(), pods, len(tensors), stream))

    def run_entry(self, pods, num_args, stream=None):
        """Call the lower_func_ptr_g entry point exactly as the reference's Instruction::Run does."""
        self.fn(ctypes.cast(pods, ctypes.c_void_p), num_args, stream)

    def run_host(self, arrays, device=0):
        """Run on host numpy arrays / pinned host torch tensors: copies in, launches, copies out."""
        bufs = []
        for a in arrays:
            if isinstance(a, np.ndarray):
                name = {np.dtype(np.float32): "float32", np.dtype(np.float16): "float16",
                        np.dtype(np.float64): "float64", np.dtype(np.int32): "int32",
                        np.dtype(np.int64): "int64", np.dtype(np.bool_): "bool",
                        np.dtype(np.uint8): "uint8"}[a.dtype]
                if not a.flags["C_CONTIGUOUS"]:
                    raise ValueError("host arrays must be C-contiguous")
                bufs.append(make_buffer(a.ctypes.data, name, a.shape, on_device=False))
            else:
                bufs.append(make_buffer(a.data_ptr(), torch_dtype_name(a), tuple(a.shape), on_device=False))
        pods = make_pods(bufs)
        _lib.check(_lib.lib().cinn_b200_group_run_host(self.name.encode(), pods, len(bufs), device))

    def release(self):
        _lib.lib().cinn_b200_release_group(self.name.encode())
