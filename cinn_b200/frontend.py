"""NetBuilder / Computation with the method names of the reference's Python API.

Mirrors `cinn.frontend` as exposed by cinn/pybind/frontend.cc:156-761 for the ops that form elementwise,
broadcast and reduction fused groups: `NetBuilder.create_input / add / relu / scale / cast / reduce_sum / ...`,
`Computation.build_and_compile(target, builder)`, `.get_tensor(name).from_numpy(a, target)`, `.numpy(target)`,
`.execute()`.  All work happens in libcinn_b200.so (C++): graph building, shape inference, the fusion pass,
group compilation and execution.
"""
import ctypes

import numpy as np

from . import _lib
from .common import Target, Type

_NP = {"float32": np.float32, "float16": np.float16, "float64": np.float64, "int32": np.int32, "int64": np.int64,
       "bool": np.bool_, "uint8": np.uint8}


def _attrs(**kw):
    parts = []
    for k, v in kw.items():
        if v is None:
            continue
        if isinstance(v, bool):
            v = "true" if v else "false"
        elif isinstance(v, (list, tuple)):
            v = ",".join(str(int(i)) for i in v)
        elif isinstance(v, float):
            v = repr(v)
        elif isinstance(v, Type):
            v = v.name
        parts.append("%s=%s" % (k, v))
    return " ".join(parts)


class Variable:
    """A value of the program; `str(v)` is its id, as with the reference's frontend.Variable."""

    def __init__(self, builder, vid):
        self._builder = builder
        self.id = vid

    def __str__(self):
        return self.id

    __repr__ = __str__

    def _info(self):
        L = _lib.lib()
        dt = ctypes.create_string_buffer(32)
        shape = (ctypes.c_longlong * 8)()
        nd = ctypes.c_int()
        _lib.check(L.cinn_b200_builder_var_info(self._builder._h, self.id.encode(), dt, 32, shape, ctypes.byref(nd)))
        return dt.value.decode(), tuple(shape[i] for i in range(nd.value))

    @property
    def shape(self):
        return list(self._info()[1])

    @property
    def type(self):
        return Type(self._info()[0])


class NetBuilder:
    def __init__(self, name="net"):
        L = _lib.lib()
        self._h = ctypes.c_void_p(L.cinn_b200_builder_create(name.encode()))
        self.name = name

    def __del__(self):
        try:
            _lib.lib().cinn_b200_builder_destroy(self._h)
        except Exception:
            pass

    # ---- plumbing ------------------------------------------------------------------------------
    def _op(self, op_type, inputs, **attrs):
        L = _lib.lib()
        ids = (ctypes.c_char_p * max(len(inputs), 1))(*[str(v).encode() for v in inputs])
        out = ctypes.create_string_buffer(128)
        _lib.check(L.cinn_b200_builder_add_op(self._h, op_type.encode(), ids, len(inputs), _attrs(**attrs).encode(),
                                              out, 128))
        return Variable(self, out.value.decode())

    # ---- program passes (Program.apply_pass / build_and_get_output, cinn/pybind/frontend.cc:157-242) ----------
    def apply_pass(self, fetch_ids=(), target=None, passes=()):
        """Rewrites the program by the named program passes, in order; an empty list applies the reference's
        default list (cinn/frontend/optimize.cc:44-82).  `fetch_ids` are the variables that must survive.  Returns
        the number of fused groups the rewritten program compiles into, as the reference's apply_pass does."""
        L = _lib.lib()
        fetch = [str(f).encode() for f in fetch_ids]
        names = [str(p).encode() for p in passes]
        f_arr = (ctypes.c_char_p * max(len(fetch), 1))(*fetch)
        p_arr = (ctypes.c_char_p * max(len(names), 1))(*names)
        _lib.check(L.cinn_b200_builder_apply_passes(self._h, p_arr, len(names), f_arr, len(fetch)))
        comp = Computation.build_and_compile(None, self, fetch=[str(f) for f in fetch_ids], plan_only=True)
        return len(comp.groups())

    def program_text(self):
        """One line per instruction, `op out = in, in ; attr=value ...`."""
        L = _lib.lib()
        L.cinn_b200_builder_program_text.restype = ctypes.c_longlong
        L.cinn_b200_builder_program_text.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
        need = L.cinn_b200_builder_program_text(self._h, None, 0)
        buf = ctypes.create_string_buffer(int(need))
        L.cinn_b200_builder_program_text(self._h, buf, len(buf))
        return buf.value.decode()

    def build_and_get_output(self, target, tensor_inputs, input_data, tensor_outputs, passes=()):
        """Applies the program passes (default list when empty), compiles, feeds `input_data` (numpy arrays, in the
        order of `tensor_inputs`), runs once and returns the outputs as numpy arrays."""
        self.apply_pass([str(v) for v in tensor_outputs], target, passes)
        comp = Computation.build_and_compile(target, self, fetch=[str(v) for v in tensor_outputs])
        for var, data in zip(tensor_inputs, input_data):
            comp.get_tensor(str(var)).from_numpy(data, target)
        comp.execute()
        return [comp.get_tensor(str(v)).numpy(target) for v in tensor_outputs]

    def create_input(self, type, shape, id_hint=""):
        L = _lib.lib()
        sh = (ctypes.c_longlong * max(len(shape), 1))(*[int(d) for d in shape])
        out = ctypes.create_string_buffer(128)
        name = type.name if isinstance(type, Type) else str(type)
        _lib.check(L.cinn_b200_builder_create_input(self._h, name.encode(), sh, len(shape), id_hint.encode(), out, 128))
        return Variable(self, out.value.decode())

    # ---- unary (cinn/frontend/net_builder.cc:130-180) -------------------------------------------
    def _unary(name):  # noqa: N805
        def f(self, x):
            return self._op(name, [x])
        f.__name__ = name
        return f

    for _n in ["sqrt", "tanh", "sigmoid", "identity", "exp", "erf", "rsqrt", "log", "log2", "log10", "floor", "ceil",
               "round", "trunc", "sin", "cos", "negative", "sign", "abs", "reciprocal", "tan", "sinh", "cosh", "asin",
               "acos", "atan", "asinh", "acosh", "atanh", "cbrt", "isnan", "isinf", "isfinite", "logical_not",
               "bitwise_not", "clz", "popc"]:
        locals()[_n] = _unary(_n)
    del _n, _unary

    def relu(self, x):
        return self._op("relu", [x])

    def relu6(self, x, threshold=6.0):
        return self._op("relu6", [x], threshold=float(threshold))

    # ---- binary with the `axis` broadcast rule (net_builder.cc:182-227) -------------------------
    def add(self, x, y, axis=-1):
        return self._op("elementwise_add", [x, y], axis=axis)

    elementwise_add = add

    def multiply(self, x, y, axis=-1):
        return self._op("elementwise_mul", [x, y], axis=axis)

    elementwise_mul = multiply

    def subtract(self, x, y, axis=-1):
        return self._op("subtract", [x, y], axis=axis)

    def divide(self, x, y, axis=-1):
        return self._op("divide", [x, y], axis=axis)

    def max(self, x, y, axis=-1):
        return self._op("max", [x, y], axis=axis)

    def min(self, x, y, axis=-1):
        return self._op("min", [x, y], axis=axis)

    def pow(self, x, y, axis=-1):
        return self._op("pow", [x, y], axis=axis)

    def _binary(name):  # noqa: N805
        def f(self, x, y, axis=-1):
            return self._op(name, [x, y], axis=axis)
        f.__name__ = name
        return f

    for _n in ["mod", "remainder", "floor_divide", "atan2", "logical_and", "logical_or", "logical_xor", "bitwise_and",
               "bitwise_or", "bitwise_xor", "left_shift", "right_shift", "logical_right_shift", "equal", "not_equal",
               "greater_than", "less_than", "greater_equal", "less_equal"]:
        locals()[_n] = _binary(_n)
    del _n, _binary

    # ---- others ------------------------------------------------------------------------------------
    def scale(self, x, scale=1.0, bias=0.0, bias_after_scale=True):
        return self._op("scale", [x], scale=float(scale), bias=float(bias), bias_after_scale=bool(bias_after_scale))

    def cast(self, x, dtype):
        return self._op("cast", [x], dtype=dtype.name if isinstance(dtype, Type) else dtype)

    def select(self, condition, true_value, false_value):
        return self._op("select", [condition, true_value, false_value])

    def broadcast_to(self, x, out_shape, broadcast_axes=None):
        return self._op("broadcast_to", [x], out_shape=list(out_shape), broadcast_axes=broadcast_axes)

    def fill_constant(self, shape, value, name="", dtype="float32", force_cpu=False):
        return self._op("fill_constant", [], shape=list(shape), value=float(value), dtype=dtype)

    def reshape(self, x, shape):
        return self._op("reshape", [x], shape=list(shape))

    def squeeze(self, x, axes=()):
        return self._op("squeeze", [x], axes=list(axes) or None)

    def expand_dims(self, x, axes):
        return self._op("expand_dims", [x], axes=list(axes))

    def transpose(self, x, axis):
        return self._op("transpose", [x], axis=list(axis))

    def concat(self, inputs, axis=0):
        return self._op("concat", list(inputs), axis=int(axis))

    def slice(self, x, axes, starts, ends, infer_flags=(), strides=(), decrease_axis=()):
        return self._op("slice", [x], axes=list(axes), starts=list(starts), ends=list(ends),
                        strides=list(strides) or None, decrease_axis=list(decrease_axis) or None)

    def reduce_sum(self, x, dim=(), keep_dim=False):
        return self._op("reduce_sum", [x], dim=list(dim) or None, keep_dim=keep_dim)

    def reduce_prod(self, x, dim=(), keep_dim=False):
        return self._op("reduce_prod", [x], dim=list(dim) or None, keep_dim=keep_dim)

    def reduce_max(self, x, dim=(), keep_dim=False):
        return self._op("reduce_max", [x], dim=list(dim) or None, keep_dim=keep_dim)

    def reduce_min(self, x, dim=(), keep_dim=False):
        return self._op("reduce_min", [x], dim=list(dim) or None, keep_dim=keep_dim)

    def reduce_all(self, x, dim=(), keep_dim=False):
        return self._op("reduce_all", [x], dim=list(dim) or None, keep_dim=keep_dim)

    def reduce_any(self, x, dim=(), keep_dim=False):
        return self._op("reduce_any", [x], dim=list(dim) or None, keep_dim=keep_dim)

    def softmax(self, x, axes=(-1,), mode="fast", data_format="AnyLayout"):
        """mode "fast": exp(x) / sum(exp(x)) (the op's own definition, cinn/hlir/pe/nn.cc:755-796); any other mode
        subtracts the row maximum first and is composed from primitives as the reference's decomposer does
        (cinn/frontend/decomposer/activation.cc:104-116)."""
        if len(axes) != 1:
            raise ValueError("softmax over several axes has no prebuilt kernel")
        if mode == "fast":
            return self._op("softmax", [x], axis=int(axes[0]))
        dt, shape = x._info()
        half_dt = dt if dt in ("float16", "bfloat16") else None
        if half_dt:  # computed in float32 between casts, as AutoCast arranges it around the op (auto_cast.cc:100-104)
            x = self.cast(x, "float32")
        nd = len(shape)
        axis = int(axes[0]) % nd
        b_axes = [i for i in range(nd) if i != axis] or [-1]
        x_max = self.broadcast_to(self.reduce_max(x, [axis]), list(shape), b_axes)
        x_exp = self.exp(self.subtract(x, x_max))
        x_sum = self.broadcast_to(self.reduce_sum(x_exp, [axis]), list(shape), b_axes)
        y = self.divide(self.exp(self.subtract(x, x_max)), x_sum)
        return self.cast(y, half_dt) if half_dt else y

    def gelu(self, x):
        """x * (0.5 + 0.5 * erf(sqrt(0.5) * x)), cinn/frontend/decomposer/activation.cc:54-69."""
        dt, shape = x._info()
        half_dt = dt if dt in ("float16", "bfloat16") else None
        if half_dt:  # computed in float32 between casts, as AutoCast arranges it around the op (auto_cast.cc:100-104)
            x, dt = self.cast(x, "float32"), "float32"
        p_5 = self.fill_constant(list(shape), 0.5, dtype=dt)
        p_7 = self.fill_constant(list(shape), float(np.sqrt(0.5)), dtype=dt)
        cdf = self.add(p_5, self.multiply(p_5, self.erf(self.multiply(x, p_7))))
        y = self.multiply(x, cdf)
        return self.cast(y, half_dt) if half_dt else y

    def relu_grad(self, dout, out):
        """select(out > 0, dout, 0), cinn/frontend/decomposer/activation.cc:36-51."""
        dt, shape = out._info()
        zero = self.fill_constant(list(shape), 0.0, dtype=dt)
        return self.select(self.greater_than(out, zero), dout, zero)

    def batchnorm(self, x, scale, bias, mean, variance, epsilon=1e-5, momentum=0.9, data_layout="NCHW", is_test=True):
        if not is_test:
            return self.batch_norm_train(x, scale, bias, mean, variance, epsilon, momentum, data_layout)
        return [self._op("batch_norm", [x, scale, bias, mean, variance], epsilon=float(epsilon),
                         momentum=float(momentum), data_layout=data_layout)]

    def batch_norm(self, *a, **kw):
        return self.batchnorm(*a, **kw)[0]

    def batch_norm_train(self, x, scale, bias, moving_mean, moving_variance, epsilon=1e-5, momentum=0.9,
                         data_layout="NCHW"):
        """Training-mode batch norm, composed from primitives exactly as the reference's decomposer does
        (cinn/frontend/decomposer/batch_norm.cc:60-177).  Returns [y, saved_mean, saved_variance, new_moving_mean,
        new_moving_variance]."""
        if data_layout != "NCHW":
            raise NotImplementedError("batch_norm_train: only NCHW has prebuilt kernels")
        dt, shape = x._info()
        n, c, h, w = shape
        count = float(n * h * w)
        red = [0, 2, 3]
        full = list(shape)
        # 16-bit x: computed in float32 between casts, as the AutoCast pass arranges it around the op
        # (cinn/frontend/pass/auto_cast.cc:138-172); statistics and moving averages stay float32.  The statistics and
        # the normalisation each widen x themselves, so that neither needs a float32 copy of it in memory.
        half_dt = dt if dt in ("float16", "bfloat16") else None
        x_in = x
        if half_dt:
            dt = "float32"
            x = self.cast(x_in, "float32")
        # mean = reduce_sum(x) / nhw ; variance = reduce_sum(x * x) / nhw - mean * mean
        mean = self.divide(self.reduce_sum(x, red), self.fill_constant([c], count, dtype=dt))
        sq_mean = self.divide(self.reduce_sum(self.multiply(x, self.identity(x)), red),
                              self.fill_constant([c], count, dtype=dt))
        if half_dt:
            x = self.cast(x_in, "float32")
        variance = self.subtract(sq_mean, self.multiply(mean, self.identity(mean)))
        mean_4d = self.broadcast_to(mean, full, [1])
        var_4d = self.broadcast_to(variance, full, [1])
        std_inv_4d = self.rsqrt(self.add(var_4d, self.fill_constant(full, float(epsilon), dtype=dt)))
        # y = scale * (x - mean) * std_variance_inv + bias
        normalized = self.multiply(self.subtract(x, mean_4d), std_inv_4d)
        y = self.add(self.multiply(normalized, self.broadcast_to(scale, full, [1])), self.broadcast_to(bias, full, [1]))
        if half_dt:
            y = self.cast(y, half_dt)

        def update(moving, saved):
            return self.add(self.multiply(moving, self.fill_constant([c], float(momentum), dtype=dt)),
                            self.multiply(saved, self.fill_constant([c], 1.0 - float(momentum), dtype=dt)))
        return [y, mean, variance, update(moving_mean, mean), update(moving_variance, variance)]

    def batch_norm_grad(self, y_grad, x, scale, save_mean, save_variance, epsilon=1e-5, data_layout="NCHW"):
        """Gradient of training-mode batch norm, composed as the reference's decomposer does
        (cinn/frontend/decomposer/batch_norm.cc:179-243).  Returns [x_grad, scale_grad, bias_grad]."""
        if data_layout != "NCHW":
            raise NotImplementedError("batch_norm_grad: only NCHW has prebuilt kernels")
        dt, shape = x._info()
        n, c, h, w = shape
        count = float(n * h * w)
        red, full = [0, 2, 3], list(shape)
        # 16-bit y_grad and x: computed in float32 between casts (cinn/frontend/pass/auto_cast.cc:173-214); x_grad goes
        # back to the 16-bit type, scale_grad and bias_grad stay float32.  The statistics and the x_grad expression
        # each widen their operands themselves, so that no float32 copy of them is written to memory.
        half_dt = dt if dt in ("float16", "bfloat16") else None
        y_grad_in, x_in = y_grad, x
        if half_dt:
            dt = "float32"
            y_grad, x = self.cast(y_grad_in, "float32"), self.cast(x_in, "float32")

        def std_inv_1d():
            return self.rsqrt(self.add(save_variance, self.fill_constant([c], float(epsilon), dtype=dt)))
        x_mean_diff = self.subtract(x, self.broadcast_to(save_mean, full, [1]))
        bias_grad = self.reduce_sum(y_grad, red)
        sum_dy_xmu = self.reduce_sum(self.multiply(y_grad, x_mean_diff), red)
        scale_grad = self.multiply(sum_dy_xmu, std_inv_1d())
        scaled_std_inv = self.multiply(scale, std_inv_1d())
        tmp0 = self.broadcast_to(self.divide(scaled_std_inv, self.fill_constant([c], count, dtype=dt)), full, [1])
        if half_dt:
            y_grad, x = self.cast(y_grad_in, "float32"), self.cast(x_in, "float32")
        tmp1 = self.multiply(y_grad, self.fill_constant(full, count, dtype=dt))
        tmp2 = self.broadcast_to(bias_grad, full, [1])
        x_mean_diff2 = self.subtract(x, self.broadcast_to(save_mean, full, [1]))
        tmp3_0 = self.multiply(x_mean_diff2, self.broadcast_to(sum_dy_xmu, full, [1]))
        var_eps_4d = self.broadcast_to(self.add(save_variance, self.fill_constant([c], float(epsilon), dtype=dt)), full, [1])
        tmp3 = self.divide(tmp3_0, var_eps_4d)
        x_grad = self.multiply(tmp0, self.subtract(self.subtract(tmp1, tmp2), tmp3))
        if half_dt:
            x_grad = self.cast(x_grad, half_dt)
        return [x_grad, scale_grad, bias_grad]

    def layer_norm(self, x, gamma, beta, epsilon=1e-5):
        """layer_norm over the last axis of a 2-D `x`, composed from primitives the way the reference's Paddle
        op mapper does (cinn/frontend/op_mappers/paddle/layer_norm.cc:84-139) with rsqrt + multiply."""
        dt, (rows, cols) = x._info()
        half = dt in ("float16", "bfloat16")
        x32 = self.cast(x, "float32") if half else x
        s1 = self.reduce_sum(x32, [1])
        n = self.fill_constant([rows], float(cols))
        mean = self.divide(s1, n)
        xx = self.multiply(x32, self.identity(x32))
        s2 = self.reduce_sum(xx, [1])
        m2 = self.divide(s2, n)
        mm = self.multiply(mean, self.identity(mean))
        var = self.max(self.subtract(m2, mm), self.fill_constant([rows], 0.0))
        rstd = self.rsqrt(self.add(var, self.fill_constant([rows], float(epsilon))))
        xc = self.subtract(x32, self.broadcast_to(mean, [rows, cols], [0]))
        xn = self.multiply(xc, self.broadcast_to(rstd, [rows, cols], [0]))
        y = self.add(self.multiply(xn, self.broadcast_to(gamma, [rows, cols], [1])),
                     self.broadcast_to(beta, [rows, cols], [1]))
        return self.cast(y, dt) if half else y


class Tensor:
    """A tensor of a computation's scope (hlir::framework::Tensor as exposed by cinn/pybind/framework.cc:116-172)."""

    def __init__(self, comp, name):
        self._comp = comp
        self.name = name

    def _info(self):
        L = _lib.lib()
        dt = ctypes.create_string_buffer(32)
        shape = (ctypes.c_longlong * 8)()
        nd = ctypes.c_int()
        ptr = ctypes.c_void_p()
        _lib.check(L.cinn_b200_computation_tensor_info(self._comp._h, self.name.encode(), dt, 32, shape,
                                                       ctypes.byref(nd), ctypes.byref(ptr)))
        return dt.value.decode(), tuple(shape[i] for i in range(nd.value)), ptr.value

    def shape(self):
        return list(self._info()[1])

    def data_ptr(self):
        return self._info()[2]

    def from_numpy(self, array, target=None):
        dt, shape, _ = self._info()
        a = np.ascontiguousarray(array)
        if a.dtype != _NP[dt] or tuple(a.shape) != shape:
            raise ValueError("tensor %s is %s%s, got %s%s" % (self.name, dt, shape, a.dtype, a.shape))
        _lib.check(_lib.lib().cinn_b200_computation_set_tensor_data(self._comp._h, self.name.encode(),
                                                                   a.ctypes.data_as(ctypes.c_void_p), a.nbytes))

    def numpy(self, target=None):
        dt, shape, _ = self._info()
        a = np.empty(shape, _NP[dt])
        _lib.check(_lib.lib().cinn_b200_computation_get_tensor_data(self._comp._h, self.name.encode(),
                                                                   a.ctypes.data_as(ctypes.c_void_p), a.nbytes))
        return a

    def bind(self, device_ptr):
        """Use caller-owned device memory for this tensor (the reference's external-buffer mode)."""
        _lib.check(_lib.lib().cinn_b200_computation_bind_tensor(self._comp._h, self.name.encode(),
                                                               ctypes.c_void_p(device_ptr)))


class Computation:
    class CompileOptions:
        def __init__(self):
            self.use_decomposer = False
            self.do_prerun = True
            self.use_default_passes = True
            self.passes = []

    def __init__(self, handle, builder):
        self._h = handle
        self._builder = builder  # keeps the builder alive

    def __del__(self):
        try:
            _lib.lib().cinn_b200_computation_destroy(self._h)
        except Exception:
            pass

    @staticmethod
    def default_compile_options():
        return Computation.CompileOptions()

    @staticmethod
    def build_and_compile(target, builder, options=None, fetch=None, plan_only=False):
        """Fuse, compile and allocate.  `plan_only=True` (or no GPU needed) plans without a device."""
        if isinstance(target, Target) and target.arch != "nvgpu":
            raise RuntimeError("the fused-group kernel library runs on NVIDIA B200 only; there is no x86 path")
        device = -1 if plan_only else (target.device if isinstance(target, Target) else 0)
        L = _lib.lib()
        L.cinn_b200_computation_build_and_compile.restype = ctypes.c_void_p
        fetch = [str(f) for f in (fetch or [])]
        if options is not None and (options.use_decomposer or options.passes):
            # CinnComputation::CompileOptions (cinn/frontend/computation.h:30-44): the Decomposer first when asked
            # for (computation.cc:53-55), then the named passes (there graph passes; here program passes by name)
            names = (["Decomposer"] if options.use_decomposer else []) + [str(p) for p in options.passes]
            f_arr = (ctypes.c_char_p * max(len(fetch), 1))(*[f.encode() for f in fetch])
            p_arr = (ctypes.c_char_p * len(names))(*[n.encode() for n in names])
            _lib.check(L.cinn_b200_builder_apply_passes(builder._h, p_arr, len(names), f_arr, len(fetch)))
        ids = (ctypes.c_char_p * max(len(fetch), 1))(*[f.encode() for f in fetch])
        h = L.cinn_b200_computation_build_and_compile(builder._h, device, ids, len(fetch))
        if not h:
            raise _lib.CinnB200Error(-2, L.cinn_b200_last_error().decode())
        return Computation(ctypes.c_void_p(h), builder)

    def export(self, path=None):
        """The compiled program as text (tensors, group descriptions in execution order, aliases): the ahead-of-time
        format that `Computation.load` runs without a builder or a fusion pass (what Program::Export and the tiny
        runtime are in the reference).  Written to `path` when given; returned either way."""
        L = _lib.lib()
        L.cinn_b200_computation_export.restype = ctypes.c_longlong
        L.cinn_b200_computation_export.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_size_t]
        need = L.cinn_b200_computation_export(self._h, None, 0)
        if need < 0:
            raise _lib.CinnB200Error(int(need), L.cinn_b200_last_error().decode())
        buf = ctypes.create_string_buffer(int(need))
        L.cinn_b200_computation_export(self._h, buf, len(buf))
        text = buf.value.decode()
        if path is not None:
            with open(path, "w") as f:
                f.write(text)
        return text

    @staticmethod
    def load(program, target=None, plan_only=False):
        """A computation from an exported program (its text, or the path of a file holding it)."""
        import os
        text = open(program).read() if os.path.exists(program) else program
        device = -1 if plan_only else (target.device if isinstance(target, Target) else 0)
        L = _lib.lib()
        L.cinn_b200_program_load.restype = ctypes.c_void_p
        L.cinn_b200_program_load.argtypes = [ctypes.c_char_p, ctypes.c_int]
        h = L.cinn_b200_program_load(text.encode(), device)
        if not h:
            raise _lib.CinnB200Error(-2, L.cinn_b200_last_error().decode())
        return Computation(ctypes.c_void_p(h), None)

    def get_all_tensor_names(self):
        L = _lib.lib()
        n = L.cinn_b200_computation_num_tensors(self._h)
        return [L.cinn_b200_computation_tensor_name(self._h, i).decode() for i in range(n)]

    def get_tensor(self, name):
        return Tensor(self, str(name))

    def _tensors_of_role(self, role):
        L = _lib.lib()
        return [Tensor(self, n) for n in self.get_all_tensor_names()
                if L.cinn_b200_computation_tensor_role(self._h, n.encode()) == role]

    def get_input_tensors(self):
        return self._tensors_of_role(0)

    def get_output_tensors(self):
        return self._tensors_of_role(2)

    def execute(self, stream=None):
        _lib.check(_lib.lib().cinn_b200_computation_execute(self._h, stream))

    def execute_graph(self, stream):
        """The whole program replayed as one CUDA graph (captured at the first call); `stream` is a raw stream handle."""
        L = _lib.lib()
        L.cinn_b200_computation_execute_graph.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
        _lib.check(L.cinn_b200_computation_execute_graph(self._h, ctypes.c_void_p(stream)))

    def execute_test(self, repeat=1000, use_graph=False):
        """Program::ExecuteTest: 100 untimed runs, then `repeat` timed ones; average milliseconds per run (the whole
        loop runs inside the library, so no Python call overhead is in the figure).  use_graph=True replays the
        program's CUDA graph instead of issuing the launches one by one."""
        ms = ctypes.c_double(0.0)
        L = _lib.lib()
        L.cinn_b200_computation_execute_test.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_double)]
        _lib.check(L.cinn_b200_computation_execute_test(self._h, -int(repeat) if use_graph else int(repeat), ctypes.byref(ms)))
        return ms.value

    def groups(self):
        """[(group description text, 'pattern kernel kernel ...')] after fusion, for inspection and tests."""
        L = _lib.lib()
        out = []
        for i in range(L.cinn_b200_computation_num_groups(self._h)):
            d = ctypes.create_string_buffer(1 << 16)
            p = ctypes.create_string_buffer(1 << 12)
            _lib.check(L.cinn_b200_computation_group_desc(self._h, i, d, len(d)))
            _lib.check(L.cinn_b200_computation_group_pattern(self._h, i, p, len(p)))
            out.append((d.value.decode(), p.value.decode()))
        return out
