"""ctypes wrapper of libcinn_x86_oracle.so, the CPU restatement of CINN's x86-path arithmetic.

TEST INFRASTRUCTURE: imported only by tests/, by `__graft_entry__.smoke()` and by the CPU-baseline legs of
bench.py.  See the header of cinn_x86_oracle.c for the rules it follows and their reference citations.
"""
import ctypes
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libcinn_x86_oracle.so")

UNARY = {name: i for i, name in enumerate(
    ["exp", "tanh", "sigmoid", "rsqrt", "sqrt", "relu", "negative", "abs", "identity", "log", "floor", "ceil",
     "erf", "sin", "cos", "reciprocal", "round", "trunc", "log2", "log10", "sign", "tan", "sinh", "cosh", "asin",
     "acos", "atan", "asinh", "acosh", "atanh", "cbrt", "isnan", "isinf", "isfinite", "logical_not"])}
BINARY = {name: i for i, name in enumerate(
    ["add", "subtract", "multiply", "divide", "max", "min", "pow", "equal", "not_equal", "greater_than", "less_than",
     "greater_equal", "less_equal", "mod", "floor_divide", "atan2", "logical_and", "logical_or", "logical_xor"])}
REDUCE = {"sum": 0, "prod": 1, "max": 2, "min": 3}

_lib = None


def build():
    """Compile the oracle with the Makefile next to this file (gcc, a second or two)."""
    subprocess.run(["make", "-C", HERE, "libcinn_x86_oracle.so"], check=True, capture_output=True)
    return LIB_PATH


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            build()
        L = ctypes.CDLL(LIB_PATH)
        L.orc_max_ulp_f32.restype = ctypes.c_int64
        L.orc_count_not_close_f32.restype = ctypes.c_int64
        L.orc_count_not_close_f16.restype = ctypes.c_int64
        _lib = L
    return _lib


def num_threads():
    return int(lib().orc_num_threads())


def _p(a):
    return ctypes.c_void_p(a.ctypes.data)


def _f32(a):
    a = np.ascontiguousarray(a)
    assert a.dtype == np.float32, a.dtype
    return a


def _i64(v):
    return ctypes.c_int64(int(v))


def _spec(a, out_shape):
    """(mid, inner) such that operand[(i // inner) % mid] is the broadcast of `a` to `out_shape` (flat index i).

    Covers: same shape; scalar; a vector aligned to one axis of the output (CINN's `axis` rule,
    cinn/hlir/pe/broadcast.cc:35-239) given here already reshaped to ndim-compatible form.
    """
    n = int(np.prod(out_shape))
    if a.size == n:
        return n, 1
    if a.size == 1:
        return 1, 1
    shape = [1] * (len(out_shape) - a.ndim) + list(a.shape)
    nz = [i for i, d in enumerate(shape) if d != 1]
    lo, hi = nz[0], nz[-1]
    if any(shape[i] != out_shape[i] for i in range(lo, hi + 1)):
        raise ValueError("unsupported broadcast %s -> %s" % (a.shape, out_shape))
    mid = int(np.prod(out_shape[lo:hi + 1]))
    inner = int(np.prod(out_shape[hi + 1:]))
    return mid, inner


def _f64(a):
    a = np.ascontiguousarray(a)
    assert a.dtype == np.float64, a.dtype
    return a


def unary_f64(op, x):
    x = _f64(x)
    y = np.empty_like(x)
    lib().orc_unary_f64(UNARY[op], _p(x), _p(y), _i64(x.size))
    return y


def binary_f64(op, a, b, out_shape=None):
    a, b = _f64(a), _f64(b)
    if out_shape is None:
        out_shape = np.broadcast_shapes(a.shape, b.shape)
    y = np.empty(out_shape, np.float64)
    am, ai = _spec(a, out_shape)
    bm, bi = _spec(b, out_shape)
    lib().orc_binary_f64(BINARY[op], _p(a), _i64(am), _i64(ai), _p(b), _i64(bm), _i64(bi), _p(y), _i64(y.size))
    return y


def fma_f64(a, b, c, out_shape=None):
    a, b, c = _f64(a), _f64(b), _f64(c)
    if out_shape is None:
        out_shape = np.broadcast_shapes(a.shape, b.shape, c.shape)
    y = np.empty(out_shape, np.float64)
    sp = [_spec(t, out_shape) for t in (a, b, c)]
    lib().orc_fma_f64(_p(a), _i64(sp[0][0]), _i64(sp[0][1]), _p(b), _i64(sp[1][0]), _i64(sp[1][1]), _p(c),
                      _i64(sp[2][0]), _i64(sp[2][1]), _p(y), _i64(y.size))
    return y


def unary(op, x):
    if np.asarray(x).dtype == np.float64:
        return unary_f64(op, x)
    x = _f32(x)
    y = np.empty_like(x)
    lib().orc_unary_f32(UNARY[op], _p(x), _p(y), _i64(x.size))
    return y


def binary(op, a, b, out_shape=None):
    a, b = _f32(a), _f32(b)
    if out_shape is None:
        out_shape = np.broadcast_shapes(a.shape, b.shape)
    y = np.empty(out_shape, np.float32)
    am, ai = _spec(a, out_shape)
    bm, bi = _spec(b, out_shape)
    lib().orc_binary_f32(BINARY[op], _p(a), _i64(am), _i64(ai), _p(b), _i64(bm), _i64(bi), _p(y), _i64(y.size))
    return y


def fma(a, b, c, out_shape=None):
    a, b, c = _f32(a), _f32(b), _f32(c)
    if out_shape is None:
        out_shape = np.broadcast_shapes(a.shape, b.shape, c.shape)
    y = np.empty(out_shape, np.float32)
    sp = [_spec(t, out_shape) for t in (a, b, c)]
    lib().orc_fma_f32(_p(a), _i64(sp[0][0]), _i64(sp[0][1]), _p(b), _i64(sp[1][0]), _i64(sp[1][1]), _p(c),
                      _i64(sp[2][0]), _i64(sp[2][1]), _p(y), _i64(y.size))
    return y


def scale(x, s, b, bias_after_scale=True):
    x = _f32(x)
    y = np.empty_like(x)
    lib().orc_scale_f32(_p(x), ctypes.c_float(s), ctypes.c_float(b), ctypes.c_int(int(bias_after_scale)), _p(y),
                        _i64(x.size))
    return y


def cast_f32_int(x, dtype):
    """float32 -> int32 / int64 the way the x86 conversion instruction does it (toward zero)."""
    x = _f32(x)
    y = np.empty(x.shape, dtype)
    fn = lib().orc_cast_f32_i32 if np.dtype(dtype) == np.int32 else lib().orc_cast_f32_i64
    fn(_p(x), _p(y), _i64(x.size))
    return y


def pow_int(a, b):
    """Integer pow (int32 or int64 arrays of one shape) as the host intrinsic computes it."""
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    assert a.dtype == b.dtype and a.dtype in (np.int32, np.int64) and a.shape == b.shape
    y = np.empty(a.shape, a.dtype)
    fn = lib().orc_pow_i32 if a.dtype == np.int32 else lib().orc_pow_i64
    fn(_p(a), _p(b), _p(y), _i64(a.size))
    return y


def cast_f32_f16(x):
    x = _f32(x)
    y = np.empty(x.shape, np.float16)
    lib().orc_cast_f32_f16(_p(x), _p(y), _i64(x.size))
    return y


def cast_f16_f32(x):
    x = np.ascontiguousarray(x)
    assert x.dtype == np.float16
    y = np.empty(x.shape, np.float32)
    lib().orc_cast_f16_f32(_p(x), _p(y), _i64(x.size))
    return y


def cast_f32_bf16(x):
    """Returns the bfloat16 bit patterns as uint16."""
    x = _f32(x)
    y = np.empty(x.shape, np.uint16)
    lib().orc_cast_f32_bf16(_p(x), _p(y), _i64(x.size))
    return y


_TYPED = {np.dtype(np.float16): 1, np.dtype(np.float64): 3, np.dtype(np.int32): 4, np.dtype(np.int64): 5,
          np.dtype(np.bool_): 6}


def reduce_typed(kind, x, outer, r, inner):
    """Serial reduction with the accumulator in the tensor's own type (float16, float64, int32, int64, bool)."""
    x = np.ascontiguousarray(x)
    assert x.size == outer * r * inner
    y = np.empty(outer * inner, x.dtype)
    code = {"sum": 0, "prod": 1, "max": 2, "min": 3, "all": 4, "any": 5}[kind]
    rc = lib().orc_reduce_typed(code, _TYPED[x.dtype], _p(x), _i64(outer), _i64(r), _i64(inner), _p(y))
    assert rc == 0, (kind, x.dtype)
    return y


def reduce(kind, x, outer, r, inner, threads=1):
    if np.asarray(x).dtype != np.float32:
        return reduce_typed(kind, x, outer, r, inner)
    x = _f32(x)
    assert x.size == outer * r * inner
    y = np.empty(outer * inner, np.float32)
    rc = lib().orc_reduce_f32(REDUCE[kind], _p(x), _i64(outer), _i64(r), _i64(inner), _p(y), ctypes.c_int(threads))
    assert rc == 0
    return y


def reduce_sum_f64(x, outer, r, inner, threads=1):
    x = _f32(x)
    y = np.empty(outer * inner, np.float64)
    lib().orc_reduce_sum_f64acc(_p(x), _i64(outer), _i64(r), _i64(inner), _p(y), ctypes.c_int(threads))
    return y


def add_relu(a, b, threads=1):
    a, b = _f32(a), _f32(b)
    y = np.empty_like(a)
    lib().orc_add_relu_f32(_p(a), _p(b), _p(y), _i64(a.size), ctypes.c_int(threads))
    return y


def bias_scale_tanh_f16(x, bias, scale_v, shift_v, threads=1):
    x, bias = _f32(x), _f32(bias)
    cols = x.shape[-1]
    y = np.empty(x.shape, np.float16)
    lib().orc_bias_scale_tanh_f16(_p(x), _p(bias), _i64(x.size // cols), _i64(cols), ctypes.c_float(scale_v),
                                  ctypes.c_float(shift_v), _p(y), ctypes.c_int(threads))
    return y


def softmax(x, threads=1):
    x = np.ascontiguousarray(x)
    cols = x.shape[-1]
    y = np.empty_like(x)
    fn = lib().orc_softmax_f32 if x.dtype == np.float32 else lib().orc_softmax_f16
    fn(_p(x), _i64(x.size // cols), _i64(cols), _p(y), ctypes.c_int(threads))
    return y


def layernorm(x, gamma, beta, eps, threads=1):
    x, gamma, beta = np.ascontiguousarray(x), _f32(gamma), _f32(beta)
    cols = x.shape[-1]
    rows = x.size // cols
    y = np.empty_like(x)
    if x.dtype == np.float32:
        lib().orc_layernorm_f32(_p(x), _p(gamma), _p(beta), _i64(rows), _i64(cols), ctypes.c_float(eps), _p(y),
                                ctypes.c_int(threads))
    else:
        scratch = np.empty(max(threads, 1) * cols, np.float32)
        lib().orc_layernorm_f16(_p(x), _p(gamma), _p(beta), _i64(rows), _i64(cols), ctypes.c_float(eps), _p(y),
                                _p(scratch), ctypes.c_int(threads))
    return y


def bn_relu_nchw(x, scale_v, bias, mean, var, eps, threads=1):
    x = np.ascontiguousarray(x)
    n, c, h, w = x.shape
    y = np.empty_like(x)
    fn = lib().orc_bn_relu_nchw_f32 if x.dtype == np.float32 else lib().orc_bn_relu_nchw_f16
    fn(_p(x), _p(_f32(scale_v)), _p(_f32(bias)), _p(_f32(mean)), _p(_f32(var)), _i64(n), _i64(c), _i64(h * w),
       ctypes.c_float(eps), _p(y), ctypes.c_int(threads))
    return y


def max_ulp(a, b):
    a, b = _f32(a), _f32(b)
    assert a.shape == b.shape
    return int(lib().orc_max_ulp_f32(_p(a), _p(b), _i64(a.size)))


def count_not_close(a, b, rtol, atol):
    """(number of elements with |a-b| > atol + rtol*|b|, worst |a-b| / limit)."""
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    assert a.shape == b.shape and a.dtype == b.dtype
    worst = ctypes.c_double()
    fn = lib().orc_count_not_close_f32 if a.dtype == np.float32 else lib().orc_count_not_close_f16
    bad = fn(_p(a), _p(b), _i64(a.size), ctypes.c_double(rtol), ctypes.c_double(atol), ctypes.byref(worst))
    return int(bad), worst.value
