"""Evaluates a fused-group description op by op with the x86-path arithmetic of cinn_x86_oracle.c.

TEST INFRASTRUCTURE (see the header of cinn_x86_oracle.c).  Given the text description of a group (the same
text the product compiles) and numpy inputs, it computes every value of the group the way the reference's x86
path would after inlining: one C loop per op, except that an Add whose operand is an inlined Mul (same group,
fp32, single use) is evaluated as a fused multiply-add (cinn/optim/lower_intrin.cc:41-59), and a `scale` is
fma(scale, x, bias) (cinn/hlir/op/elementwise.cc:149-163).  Values of float16 type are rounded after every op.
"""
import numpy as np

from . import x86_oracle as orc

UNARY = {"exp", "tanh", "sigmoid", "rsqrt", "sqrt", "relu", "negative", "abs", "identity", "log", "floor", "ceil",
         "erf", "sin", "cos", "reciprocal", "round", "trunc", "log2", "log10", "sign", "tan", "sinh", "cosh", "asin",
         "acos", "atan", "asinh", "acosh", "atanh", "cbrt", "isnan", "isinf", "isfinite", "logical_not"}
PREDICATES = {"isnan", "isinf", "isfinite", "logical_not"}
BINARY = {"elementwise_add": "add", "subtract": "subtract", "elementwise_mul": "multiply", "divide": "divide",
          "max": "max", "min": "min", "pow": "pow", "equal": "equal", "not_equal": "not_equal",
          "greater_than": "greater_than", "less_than": "less_than", "greater_equal": "greater_equal",
          "less_equal": "less_equal", "mod": "mod", "remainder": "mod", "floor_divide": "floor_divide",
          "atan2": "atan2", "logical_and": "logical_and", "logical_or": "logical_or", "logical_xor": "logical_xor"}
BOOL_RESULT = {"equal", "not_equal", "greater_than", "less_than", "greater_equal", "less_equal", "logical_and",
               "logical_or", "logical_xor"}
REDUCE = {"reduce_sum": "sum", "reduce_prod": "prod", "reduce_max": "max", "reduce_min": "min", "reduce_all": "all",
          "reduce_any": "any"}
NP = {"float32": np.float32, "float16": np.float16, "bool": np.bool_, "int32": np.int32, "int64": np.int64,
      "float64": np.float64, "uint8": np.uint8}
UNSIGNED_OF = {8: np.uint8, 32: np.uint32, 64: np.uint64}


def parse(desc):
    g = {"inputs": [], "outputs": [], "ops": []}
    for line in desc.splitlines():
        line = line.split("#")[0]
        attrs = {}
        if ";" in line:
            line, a = line.split(";", 1)
            for kv in a.split():
                k, v = kv.split("=", 1)
                attrs[k] = v
        w = line.split()
        if not w:
            continue
        if w[0] == "group":
            g["name"] = w[1]
        elif w[0] in ("input", "output"):
            shape = tuple(int(d) for d in w[3].split(",")) if w[3] != "scalar" else ()
            g[w[0] + "s"].append((w[1], w[2], shape))
        elif w[0] == "op":
            g["ops"].append({"type": w[1], "out": w[2], "ins": w[4:], "attrs": attrs})
    return g


def _aligned(a, out_shape, axis):
    """Reshape operand `a` so that numpy-style right-aligned broadcasting places it at `axis` of out_shape."""
    if a.ndim == len(out_shape) or axis < 0:
        return a
    return a.reshape(a.shape + (1,) * (len(out_shape) - axis - a.ndim))


def _f32(v):
    """The value as the fp32 numbers the arithmetic sees: float16 widened, bool as 0/1, integers converted the way
    the cast op does (round to nearest even)."""
    if v.dtype == np.float16:
        return orc.cast_f16_f32(v)
    if v.dtype == np.float32:
        return v
    return np.ascontiguousarray(v.astype(np.float32))


def _store(v32, dtype):
    dtype = np.dtype(dtype)
    if dtype == np.float16:
        return orc.cast_f32_f16(v32)
    if dtype == np.bool_:
        return v32 != 0
    if dtype in (np.dtype(np.int32), np.dtype(np.int64)):
        return orc.cast_f32_int(v32, dtype)
    return v32


INT_UNARY = {"negative", "abs", "identity", "relu", "logical_not", "bitwise_not", "clz", "popc"}


def _int_unary(t, x):
    """Integer tensors: plain two's-complement arithmetic (numpy wraps like the C operators)."""
    bits = x.dtype.itemsize * 8
    u = x.view(UNSIGNED_OF[bits])
    with np.errstate(over="ignore"):
        if t == "negative":
            return (np.zeros((), x.dtype) - x).astype(x.dtype)
        if t == "abs":
            return np.where(x > 0, x, (np.zeros((), x.dtype) - x).astype(x.dtype)).astype(x.dtype)
        if t == "relu":
            return np.maximum(x, 0).astype(x.dtype)
        if t == "logical_not":
            return x == 0
        if t == "bitwise_not":
            return ~x
        if t in ("clz", "popc"):
            ones = np.zeros(x.shape, np.int64)
            lead = np.full(x.shape, bits, np.int64)
            for b in range(bits):
                bit = ((u >> np.array(b, u.dtype)) & np.array(1, u.dtype)).astype(np.int64)
                ones += bit
                lead = np.where(bit == 1, bits - 1 - b, lead)
            return (ones if t == "popc" else lead).astype(x.dtype)
    return x


def _int_binary(t, a, b):
    """a, b broadcast-compatible integer arrays of one dtype (or bool for the logical ops)."""
    dt = a.dtype
    bits = dt.itemsize * 8
    with np.errstate(over="ignore", divide="ignore"):
        if t == "elementwise_add":
            return (a + b).astype(dt)
        if t == "subtract":
            return (a - b).astype(dt)
        if t == "elementwise_mul":
            return (a * b).astype(dt)
        if t in ("divide", "floor_divide", "mod", "remainder"):
            m1 = (b == -1) if dt.kind == "i" else np.zeros(np.shape(b), bool)   # unsigned: UDiv / URem, no -1
            safe = np.where((b == 0) | m1, 1, b).astype(dt)
            fl = np.floor_divide(a, safe)
            md = (a - fl * safe).astype(dt)                       # sign of the divisor
            tr = np.where((md != 0) & ((a < 0) != (safe < 0)), fl + 1, fl).astype(dt)   # toward zero
            neg = (np.zeros((), dt) - a).astype(dt)
            if t == "divide":
                return np.where(b == 0, 0, np.where(m1, neg, tr)).astype(dt)
            if t == "floor_divide":
                return np.where(b == 0, 0, np.where(m1, neg, fl)).astype(dt)
            return np.where((b == 0) | m1, 0, md).astype(dt)
        if t == "pow":
            shape = np.broadcast_shapes(a.shape, b.shape)
            return orc.pow_int(np.broadcast_to(a, shape), np.broadcast_to(b, shape))
        if t == "max":
            return np.where(a > b, a, b).astype(dt)
        if t == "min":
            return np.where(a < b, a, b).astype(dt)
        if t in ("equal", "not_equal", "greater_than", "less_than", "greater_equal", "less_equal"):
            return {"equal": a == b, "not_equal": a != b, "greater_than": a > b, "less_than": a < b,
                    "greater_equal": a >= b, "less_equal": a <= b}[t]
        if t in ("logical_and", "logical_or", "logical_xor"):
            p, q = a != 0, b != 0
            return {"logical_and": p & q, "logical_or": p | q, "logical_xor": p ^ q}[t]
        if t == "bitwise_and":
            return a & b
        if t == "bitwise_or":
            return a | b
        if t == "bitwise_xor":
            return a ^ b
        cnt = (b & (bits - 1)).astype(dt)
        if t == "left_shift":
            ut = UNSIGNED_OF[bits]
            return (a.astype(dt).view(ut) << cnt.view(ut)).view(dt)
        if t == "right_shift":
            return (a >> cnt).astype(dt)
        if t == "logical_right_shift":
            ut = UNSIGNED_OF[bits]
            return (np.ascontiguousarray(np.broadcast_to(a, np.broadcast_shapes(a.shape, b.shape))).view(ut)
                    >> np.ascontiguousarray(np.broadcast_to(cnt, np.broadcast_shapes(a.shape, b.shape))).view(ut)).view(dt)
    raise NotImplementedError(t)


INT_BINARY = {"elementwise_add", "subtract", "elementwise_mul", "divide", "max", "min", "pow", "equal", "not_equal",
              "greater_than", "less_than", "greater_equal", "less_equal", "mod", "remainder", "floor_divide",
              "logical_and", "logical_or", "logical_xor", "bitwise_and", "bitwise_or", "bitwise_xor", "left_shift",
              "right_shift", "logical_right_shift"}


def evaluate(desc, inputs):
    """inputs: list of numpy arrays in the group's input order.  Returns {value name: array}."""
    g = parse(desc)
    vals = {}
    for (name, dt, shape), a in zip(g["inputs"], inputs):
        assert a.dtype == NP[dt] and tuple(a.shape) == shape, (name, a.dtype, a.shape)
        vals[name] = np.ascontiguousarray(a)
    uses = {}
    producer = {}
    for op in g["ops"]:
        producer[op["out"]] = op
        for i in op["ins"]:
            uses[i] = uses.get(i, 0) + 1
    outputs = {o[0] for o in g["outputs"]}
    feeds_reduce = {i for op in g["ops"] if op["type"] in REDUCE for i in op["ins"]}

    def inlined_mul(name):
        """The Mul op producing `name` if it is inlined into its single consumer (then it can be contracted)."""
        p = producer.get(name)
        if p is None or name in outputs or name in feeds_reduce or uses.get(name, 0) != 1:
            return None
        if p["type"] == "elementwise_mul" and vals[name].dtype in (np.float32, np.float64):
            return p
        return None

    for op in g["ops"]:
        t, ins, at = op["type"], op["ins"], op["attrs"]
        if t == "fill_constant":
            shape = tuple(int(d) for d in at["shape"].split(","))
            out = np.full(shape, float(at["value"]), NP[at.get("dtype", "float32")])
        elif t == "cast":
            x = vals[ins[0]]
            to = NP[at["dtype"]]
            if x.dtype == to:
                out = x
            elif x.dtype == np.float64 or to == np.float64:
                # float64 <-> float32 / integers / bool: one IEEE conversion (numpy rounds to nearest even)
                out = (x != 0) if to == np.bool_ else x.astype(to)
            elif x.dtype.kind in "iub" and np.dtype(to).kind in "iub":
                out = (x != 0) if to == np.bool_ else x.astype(to)   # widen / truncate / 0-1
            else:
                out = _store(_f32(x), to)
        elif t in INT_UNARY and vals[ins[0]].dtype.kind in "iu":
            out = _int_unary(t, vals[ins[0]])
        elif t in INT_BINARY and vals[ins[0]].dtype.kind in "iu":
            a, b = vals[ins[0]], vals[ins[1]]
            axis = int(at.get("axis", -1))
            big, small = (a, b) if a.ndim >= b.ndim else (b, a)
            shape = np.broadcast_shapes(big.shape, _aligned(small, big.shape, axis).shape)
            aa = a if a is big else _aligned(a, shape, axis)
            bb = b if b is big else _aligned(b, shape, axis)
            out = np.broadcast_to(_int_binary(t, aa, bb), shape)
        elif t == "broadcast_to":
            x = vals[ins[0]]
            shape = tuple(int(d) for d in at["out_shape"].split(","))
            axes = [int(d) for d in at["broadcast_axes"].split(",")]
            view = [1] * len(shape)
            for i, ax in enumerate(axes):
                view[ax] = x.shape[i]
            out = np.ascontiguousarray(np.broadcast_to(x.reshape(view), shape))
        elif t == "scale" and vals[ins[0]].dtype == np.float64:
            x = vals[ins[0]]
            after = at.get("bias_after_scale", "true") in ("true", "1", "True")
            sc, bi = np.full(1, float(at.get("scale", 1))), np.full(1, float(at.get("bias", 0)))
            out = orc.fma_f64(sc, x, bi, x.shape) if after else orc.binary_f64("multiply", sc, orc.binary_f64("add", x, bi, x.shape), x.shape)
        elif t == "scale":
            x = vals[ins[0]]
            after = at.get("bias_after_scale", "true") in ("true", "1", "True")
            out = _store(orc.scale(_f32(x), float(at.get("scale", 1)), float(at.get("bias", 0)), after), x.dtype)
        elif t in UNARY and vals[ins[0]].dtype == np.float64:
            out = orc.unary_f64(t, vals[ins[0]])
            out = (out != 0) if t in PREDICATES else out
        elif t == "relu6" and vals[ins[0]].dtype == np.float64:
            x = vals[ins[0]]
            out = orc.binary_f64("min", orc.unary_f64("relu", x), np.full(1, float(at.get("threshold", 6))), x.shape)
        elif t in UNARY:
            x = vals[ins[0]]
            out = _store(orc.unary(t, _f32(x)), np.bool_ if t in PREDICATES else x.dtype)
        elif t == "select":
            c, tv, fv = (vals[i] for i in ins)
            out = np.where(c, tv, fv)
        elif t == "relu6":
            x = vals[ins[0]]
            thr = np.float32(float(at.get("threshold", 6)))
            out = _store(orc.binary("min", orc.unary("relu", _f32(x)), np.full(1, thr, np.float32), x.shape), x.dtype)
        elif t in BINARY:
            a, b = vals[ins[0]], vals[ins[1]]
            axis = int(at.get("axis", -1))
            big, small = (a, b) if a.ndim >= b.ndim else (b, a)
            shape = np.broadcast_shapes(big.shape, _aligned(small, big.shape, axis).shape)
            aa = a if a is big else _aligned(a, shape, axis)
            bb = b if b is big else _aligned(b, shape, axis)
            dt = np.dtype(np.bool_) if t in BOOL_RESULT else a.dtype
            done = False
            dbl = a.dtype == np.float64 or b.dtype == np.float64
            if dbl:
                aa, bb = np.ascontiguousarray(aa.astype(np.float64)), np.ascontiguousarray(bb.astype(np.float64))
            if t == "elementwise_add" and dt in (np.float32, np.float64):
                # lower_intrin.cc:45-50: the right operand is tried first
                for mul_name, other in ((ins[1], aa), (ins[0], bb)):
                    m = inlined_mul(mul_name)
                    if m is not None:
                        ma, mb = vals[m["ins"][0]], vals[m["ins"][1]]
                        maxis = int(m["attrs"].get("axis", -1))
                        mbig = ma if ma.ndim >= mb.ndim else mb
                        ma2 = ma if ma is mbig else _aligned(ma, mbig.shape, maxis)
                        mb2 = mb if mb is mbig else _aligned(mb, mbig.shape, maxis)
                        out = orc.fma_f64(ma2, mb2, other, shape) if dbl else orc.fma(ma2, mb2, other, shape)
                        done = True
                        break
            if not done and dbl:
                out = orc.binary_f64(BINARY[t], aa, bb, shape)
                out = (out != 0) if t in BOOL_RESULT else out
            elif not done:
                out = _store(orc.binary(BINARY[t], _f32(aa), _f32(bb), shape), dt)
        elif t in REDUCE:
            x = vals[ins[0]]
            dims = sorted(int(d) % x.ndim for d in at["dim"].split(",")) if at.get("dim") else list(range(x.ndim))
            keep = at.get("keep_dim", "false") in ("true", "1", "True")
            lo, hi = dims[0], dims[-1]
            if dims == list(range(lo, hi + 1)):
                outer = int(np.prod(x.shape[:lo]))
                r = int(np.prod(x.shape[lo:hi + 1]))
                inner = int(np.prod(x.shape[hi + 1:]))
                res = orc.reduce(REDUCE[t], x, outer, r, inner)
            else:
                # non-adjacent axes: the serial loop nest visits the reduced axes in increasing order, innermost
                # fastest (cinn/hlir/pe/reduction.cc:139-227) -- the same as reducing a copy with the kept axes first
                kept = [i for i in range(x.ndim) if i not in dims]
                xt = np.ascontiguousarray(np.transpose(x, kept + dims))
                res = orc.reduce(REDUCE[t], xt, int(np.prod([x.shape[i] for i in kept])),
                                 int(np.prod([x.shape[i] for i in dims])), 1)
            oshape = [d for i, d in enumerate(x.shape) if i not in dims or keep]
            if keep:
                oshape = [1 if i in dims else d for i, d in enumerate(x.shape)]
            out = res.reshape(oshape if oshape else (1,))
        elif t == "transpose":
            out = np.transpose(vals[ins[0]], [int(d) for d in at["axis"].split(",")])
        elif t == "concat":
            out = np.concatenate([vals[i] for i in ins], axis=int(at.get("axis", 0)))
        elif t == "reshape":
            out = vals[ins[0]].reshape([int(d) for d in at["shape"].split(",")])
        elif t == "slice":
            x = vals[ins[0]]
            ints = lambda k: [int(d) for d in at[k].split(",")] if at.get(k) else []  # noqa: E731
            sl = [slice(None)] * x.ndim
            strides = ints("strides")
            for k, a in enumerate(ints("axes")):
                a %= x.ndim
                st = strides[k] if k < len(strides) else 1
                b, e = ints("starts")[k], ints("ends")[k]
                dim = x.shape[a]
                b = b + dim if b < 0 else b
                e = e + dim if e < 0 else e
                if st > 0:
                    sl[a] = slice(min(max(b, 0), dim), min(max(e, 0), dim), st)
                else:   # positions clamped to [-1, dim - 1]; -1 means "before the first element"
                    b, e = min(max(b, -1), dim - 1), min(max(e, -1), dim - 1)
                    sl[a] = slice(b, e if e >= 0 else None, st)
            out = x[tuple(sl)]
            drop = [d % x.ndim for d in ints("decrease_axis")]
            if drop:
                out = out.reshape([d for i, d in enumerate(out.shape) if i not in drop] or [1])
        elif t == "softmax":
            out = orc.softmax(vals[ins[0]])
        elif t == "batch_norm":
            x, scale, bias, mean, var = (vals[i] for i in ins)
            eps = np.float32(float(at.get("epsilon", 1e-5)))
            c = x.shape[1]
            sh = (1, c, 1, 1)
            d = orc.unary("sqrt", orc.binary("add", var, np.full(1, eps, np.float32), var.shape))
            t1 = orc.binary("subtract", x, mean.reshape(sh), x.shape)
            t2 = orc.binary("multiply", t1, scale.reshape(sh), x.shape)
            t3 = orc.binary("divide", t2, d.reshape(sh), x.shape)
            out = orc.binary("add", t3, bias.reshape(sh), x.shape)
        else:
            raise NotImplementedError("oracle evaluator: op " + t)
        vals[op["out"]] = np.ascontiguousarray(out)
    return vals


def run(desc, inputs):
    """The group's single output."""
    g = parse(desc)
    return evaluate(desc, inputs)[g["outputs"][0][0]]


def run_all(desc, inputs):
    """{name: array} of all outputs of the group."""
    g = parse(desc)
    vals = evaluate(desc, inputs)
    return {o[0]: vals[o[0]] for o in g["outputs"]}
