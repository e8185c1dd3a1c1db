"""The fused groups the library is measured on, as group descriptions plus seeded synthetic inputs.

Each workload is one fused group of the kind the reference's OpFusionPass / FusionMergePass produce
(cinn/hlir/pass/op_fusion_pass.cc:123-331) for a small NetBuilder program; shapes are parameters so that tests
can run the same group at small sizes.  Inputs are drawn with numpy's default_rng(seed) in the listed order as
float32; 16-bit variants are `.astype(float16)` of the same draw.
"""
import numpy as np


def _shape(s):
    return ",".join(str(int(d)) for d in s)


class Workload:
    """name, group description text, input arrays (host numpy, generated on first use), output dtype/shape."""

    def __init__(self, name, desc, inputs, out_dtype, out_shape, more_outputs=()):
        self.name = name
        self.desc = desc
        self._inputs = inputs  # a list of arrays, or a function returning one
        self.out_dtype = out_dtype
        self.out_shape = tuple(int(d) for d in out_shape)
        self.more_outputs = tuple(more_outputs)  # (dtype, shape) of the outputs after the first

    @property
    def inputs(self):
        if callable(self._inputs):
            self._inputs = self._inputs()
        return self._inputs

    @property
    def group_name(self):
        return self.desc.split()[1]

    def input_bytes(self):
        """From the description's input lines, so that it does not materialise the arrays."""
        total = 0
        for line in self.desc.splitlines():
            w = line.split()
            if w and w[0] == "input":
                n = 1
                for d in w[3].split(","):
                    n *= int(d)
                total += n * {"float32": 4, "float16": 2, "bfloat16": 2, "float64": 8}[w[2]]
        return total

    def output_bytes(self):
        return int(np.prod(self.out_shape)) * np.dtype(self.out_dtype).itemsize

    def algorithmic_bytes(self):
        return self.input_bytes() + self.output_bytes()


def add_relu(shape=(1, 3, 224, 224), seed=0, name="fn_elementwise_add_relu"):
    """relu(A + B), fp32: the README example (one elementwise group)."""
    def gen():
        rng = np.random.default_rng(seed)
        a = rng.uniform(-1, 1, shape).astype(np.float32)
        b = rng.uniform(-1, 1, shape).astype(np.float32)
        return [a, b]
    s = _shape(shape)
    desc = (f"group {name}\ninput A float32 {s}\ninput B float32 {s}\n"
            f"op elementwise_add var_0 = A B ; axis=-1\nop relu var_1 = var_0\noutput var_1 float32 {s}\n")
    return Workload("add_relu", desc, gen, np.float32, shape)


def bias_scale_tanh_cast(shape=(64, 1024, 1024), seed=1, name="fn_bias_scale_tanh_cast"):
    """cast_fp16(tanh((X + bias) * 0.5)), bias broadcast on the last axis."""
    def gen():
        rng = np.random.default_rng(seed)
        x = rng.standard_normal(shape, dtype=np.float32)
        bias = (0.1 * rng.standard_normal(shape[-1])).astype(np.float32)
        return [x, bias]
    s = _shape(shape)
    desc = (f"group {name}\ninput X float32 {s}\ninput bias float32 {shape[-1]}\n"
            f"op elementwise_add var_0 = X bias ; axis=-1\n"
            f"op scale var_1 = var_0 ; scale=0.5 bias=0.0 bias_after_scale=true\n"
            f"op tanh var_2 = var_1\nop cast var_3 = var_2 ; dtype=float16\noutput var_3 float16 {s}\n")
    return Workload("bias_scale_tanh_cast", desc, gen, np.float16, shape)


def reduce_input(shape=(128, 1024, 1024), seed=2):
    return np.random.default_rng(seed).standard_normal(shape, dtype=np.float32)


def reduce_sum_last(shape=(128, 1024, 1024), seed=2, x=None, name="fn_reduce_sum_last"):
    """reduce_sum over the last axis (row reduction)."""
    out_shape = shape[:-1]
    desc = (f"group {name}\ninput X float32 {_shape(shape)}\n"
            f"op reduce_sum var_0 = X ; dim={len(shape) - 1} keep_dim=false\n"
            f"output var_0 float32 {_shape(out_shape)}\n")
    return Workload("reduce_sum_last", desc, (lambda: [reduce_input(shape, seed)]) if x is None else [x], np.float32,
                    out_shape)


def reduce_max_first(shape=(128, 1024, 1024), seed=2, x=None, name="fn_reduce_max_first"):
    """reduce_max over axis 0 (column reduction)."""
    out_shape = shape[1:]
    desc = (f"group {name}\ninput X float32 {_shape(shape)}\n"
            f"op reduce_max var_0 = X ; dim=0 keep_dim=false\n"
            f"output var_0 float32 {_shape(out_shape)}\n")
    return Workload("reduce_max_first", desc, (lambda: [reduce_input(shape, seed)]) if x is None else [x], np.float32,
                    out_shape)


def rownorm_inputs(shape=(16384, 4096), seed=3):
    rng = np.random.default_rng(seed)
    x = rng.standard_normal(shape, dtype=np.float32)
    gamma = (1 + 0.02 * rng.standard_normal(shape[-1])).astype(np.float32)
    beta = (0.02 * rng.standard_normal(shape[-1])).astype(np.float32)
    return x, gamma, beta


def softmax(shape=(16384, 4096), seed=3, half=False, name=None):
    """softmax along the last axis; half=True stores x and out as fp16 and computes in fp32."""
    s = _shape(shape)
    name = name or ("fn_softmax_f16" if half else "fn_softmax_f32")
    if half:
        desc = (f"group {name}\ninput X float16 {s}\nop cast var_0 = X ; dtype=float32\n"
                f"op softmax var_1 = var_0 ; axis=-1\nop cast var_2 = var_1 ; dtype=float16\n"
                f"output var_2 float16 {s}\n")
        return Workload("softmax_f16", desc, lambda: [rownorm_inputs(shape, seed)[0].astype(np.float16)], np.float16,
                        shape)
    desc = f"group {name}\ninput X float32 {s}\nop softmax var_0 = X ; axis=-1\noutput var_0 float32 {s}\n"
    return Workload("softmax_f32", desc, lambda: [rownorm_inputs(shape, seed)[0]], np.float32, shape)


def layer_norm_ops(rows, cols, eps, half):
    """The op sequence of the layer_norm composition (reduce_sum / divide / multiply / rsqrt ...), as lines."""
    x = "X"
    lines = []
    if half:
        lines.append("op cast x32 = X ; dtype=float32")
        x = "x32"
    sh, r = f"{rows},{cols}", f"{rows}"
    lines += [
        f"op reduce_sum s1 = {x} ; dim=1 keep_dim=false",
        f"op fill_constant n = ; shape={r} value={float(cols)} dtype=float32",
        "op divide mean = s1 n",
        f"op identity x_id = {x}",
        f"op elementwise_mul xx = {x} x_id",
        "op reduce_sum s2 = xx ; dim=1 keep_dim=false",
        "op divide m2 = s2 n",
        "op identity mean_id = mean",
        "op elementwise_mul mm = mean mean_id",
        "op subtract dv = m2 mm",
        f"op fill_constant zero = ; shape={r} value=0.0 dtype=float32",
        "op max var = dv zero",
        f"op fill_constant eps = ; shape={r} value={eps!r} dtype=float32",
        "op elementwise_add ve = var eps",
        "op rsqrt rstd = ve",
        f"op broadcast_to mean_b = mean ; out_shape={sh} broadcast_axes=0",
        f"op subtract xc = {x} mean_b",
        f"op broadcast_to rstd_b = rstd ; out_shape={sh} broadcast_axes=0",
        "op elementwise_mul xn = xc rstd_b",
        f"op broadcast_to gamma_b = gamma ; out_shape={sh} broadcast_axes=1",
        "op elementwise_mul xg = xn gamma_b",
        f"op broadcast_to beta_b = beta ; out_shape={sh} broadcast_axes=1",
        "op elementwise_add y = xg beta_b",
    ]
    out = "y"
    if half:
        lines.append("op cast y16 = y ; dtype=float16")
        out = "y16"
    return lines, out


def layer_norm(shape=(16384, 4096), seed=3, half=False, eps=1e-5, name=None):
    """layer_norm along the last axis of a 2-D tensor, composed from NetBuilder primitives."""
    rows, cols = shape
    name = name or ("fn_layer_norm_f16" if half else "fn_layer_norm_f32")
    dt = "float16" if half else "float32"
    lines, out = layer_norm_ops(rows, cols, eps, half)
    desc = (f"group {name}\ninput X {dt} {rows},{cols}\ninput gamma float32 {cols}\ninput beta float32 {cols}\n" +
            "\n".join(lines) + f"\noutput {out} {dt} {rows},{cols}\n")
    def gen():
        x, gamma, beta = rownorm_inputs(shape, seed)
        return [x.astype(np.float16) if half else x, gamma, beta]
    return Workload("layer_norm_f16" if half else "layer_norm_f32", desc, gen, np.float16 if half else np.float32,
                    shape)


def bn_relu(shape=(256, 64, 112, 112), seed=4, half=False, eps=1e-5, name=None):
    """relu(batch_norm_infer(X)) on NCHW; argument order x, scale, bias, mean, variance."""
    c = shape[1]

    def gen():
        rng = np.random.default_rng(seed)
        x = rng.standard_normal(shape, dtype=np.float32)
        mean = (0.1 * rng.standard_normal(c)).astype(np.float32)
        var = rng.uniform(0.5, 1.5, c).astype(np.float32)
        scale = (1 + 0.1 * rng.standard_normal(c)).astype(np.float32)
        bias = (0.1 * rng.standard_normal(c)).astype(np.float32)
        return [x.astype(np.float16) if half else x, scale, bias, mean, var]
    s = _shape(shape)
    name = name or ("fn_batch_norm_relu_f16" if half else "fn_batch_norm_relu_f32")
    params = f"input scale float32 {c}\ninput bias float32 {c}\ninput mean float32 {c}\ninput variance float32 {c}\n"
    attrs = f"epsilon={eps!r} momentum=0.9 data_layout=NCHW"
    if half:
        desc = (f"group {name}\ninput X float16 {s}\n" + params +
                "op cast x32 = X ; dtype=float32\n"
                f"op batch_norm var_0 = x32 scale bias mean variance ; {attrs}\n"
                "op relu var_1 = var_0\nop cast var_2 = var_1 ; dtype=float16\n"
                f"output var_2 float16 {s}\n")
        return Workload("bn_relu_f16", desc, gen, np.float16, shape)
    desc = (f"group {name}\ninput X float32 {s}\n" + params +
            f"op batch_norm var_0 = X scale bias mean variance ; {attrs}\n"
            f"op relu var_1 = var_0\noutput var_1 float32 {s}\n")
    return Workload("bn_relu_f32", desc, gen, np.float32, shape)


# ---- groups of the generic kernel families (elementwise chains of any op / type, typed reductions) ----------------

_NP = {"float32": np.float32, "float16": np.float16, "float64": np.float64, "int32": np.int32, "int64": np.int64,
       "bool": np.bool_}


def _draw(rng, shape, dtype):
    if dtype in ("int32", "int64"):
        return rng.integers(-1000, 1000, shape).astype(_NP[dtype])
    if dtype == "bool":
        return rng.random(shape) > 0.5
    return rng.standard_normal(shape, dtype=np.float32).astype(_NP[dtype])


def generic_chain(kind, shape=(8192, 8192), seed=5):
    """Elementwise groups that only the generic chain kernels cover.  kind: leaky_relu_f32 (select on a mask
    input), abs_add_f32, greater_than_f32 (bool output), abs_add_i32, abs_add_f64, affine_f64."""
    s = _shape(shape)
    table = {
        "abs_add_f32": (["A float32", "B float32"], ["op elementwise_add t0 = A B", "op abs t1 = t0"], "t1", "float32"),
        "select_f32": (["M bool", "A float32", "B float32"], ["op select t0 = M A B"], "t0", "float32"),
        "greater_than_f32": (["A float32", "B float32"], ["op greater_than t0 = A B"], "t0", "bool"),
        "abs_add_i32": (["A int32", "B int32"], ["op elementwise_add t0 = A B", "op abs t1 = t0"], "t1", "int32"),
        "abs_add_f64": (["A float64", "B float64"], ["op elementwise_add t0 = A B", "op abs t1 = t0"], "t1", "float64"),
        "gelu_f32": (["x float32"], ["op fill_constant h = ; dtype=float32 shape=%s value=0.5" % s,
                                    "op fill_constant r = ; dtype=float32 shape=%s value=0.7071067811865476" % s,
                                    "op elementwise_mul u = x r ; axis=-1", "op erf e = u", "op elementwise_mul v = h e ; axis=-1",
                                    "op elementwise_add w = h v ; axis=-1", "op elementwise_mul y = x w ; axis=-1"], "y", "float32"),
        "sigmoid_grad_f32": (["y float32", "dy float32"], ["op scale c = y ; bias=1.0 bias_after_scale=true scale=-1.0",
                                                           "op elementwise_mul t = y c ; axis=-1",
                                                           "op elementwise_mul g = dy t ; axis=-1"], "g", "float32"),
        "affine_f64": (["A float64"], ["op scale t0 = A ; scale=0.1 bias=1e-05", "op abs t1 = t0"], "t1", "float64"),
    }
    ins, ops, out, out_dtype = table[kind]
    desc = "group fn_chain_%s\n%s\n%s\noutput %s %s %s\n" % (
        kind, "\n".join("input %s %s" % (i, s) for i in ins), "\n".join(ops), out, out_dtype, s)

    def gen():
        rng = np.random.default_rng(seed)
        return [_draw(rng, shape, i.split()[1]) for i in ins]
    return Workload("chain_" + kind, desc, gen, _NP[out_dtype], shape)


def generic_reduce(kind, dtype, shape=(16384, 8192), axis=1, seed=6):
    """reduce_<kind> of a tensor of one of the other element types over one axis of a 2-D shape."""
    out_shape = tuple(d for i, d in enumerate(shape) if i != axis)
    desc = ("group fn_reduce_%s_%s_axis%d\ninput X %s %s\nop reduce_%s var_0 = X ; dim=%d keep_dim=false\n"
            "output var_0 %s %s\n" % (kind, dtype, axis, dtype, _shape(shape), kind, axis, dtype, _shape(out_shape)))
    return Workload("reduce_%s_%s" % (kind, dtype), desc, lambda: [_draw(np.random.default_rng(seed), shape, dtype)],
                    _NP[dtype], out_shape)


def chain_tree(shape=(8192, 8192), seed=9):
    """(A + B) * (C - D): an expression tree, one kernel (one branch stashed in a temporary)."""
    s = _shape(shape)
    desc = (f"group fn_tree\ninput A float32 {s}\ninput B float32 {s}\ninput C float32 {s}\ninput D float32 {s}\n"
            f"op elementwise_add t = A B ; axis=-1\nop subtract u = C D ; axis=-1\nop elementwise_mul y = t u ; axis=-1\n"
            f"output y float32 {s}\n")
    return Workload("chain_tree", desc, lambda: [_draw(np.random.default_rng(seed + k), shape, "float32") for k in range(4)],
                    np.float32, shape)


def chain_two_outputs(shape=(8192, 8192), seed=10):
    """pre = X + bias (kept for the backward pass) and act = relu(pre): one kernel, two outputs."""
    s = _shape(shape)
    desc = (f"group fn_pre_act\ninput X float32 {s}\ninput B float32 {shape[-1]}\n"
            f"op elementwise_add pre = X B ; axis=-1\nop relu act = pre\noutput pre float32 {s}\noutput act float32 {s}\n")
    return Workload("chain_two_outputs", desc,
                    lambda: [_draw(np.random.default_rng(seed), shape, "float32"),
                             _draw(np.random.default_rng(seed + 1), (shape[-1],), "float32")],
                    np.float32, shape, more_outputs=[(np.float32, shape)])


def chain_reduce(kind="sum_abs_diff", shape=(8192, 8192), axis=1, seed=8):
    """A reduction whose operand is an elementwise chain, one kernel: `sum_abs_diff` = reduce_sum(|x - y|) of two
    tensors, `sum_sigmoid_affine` = reduce_sum(sigmoid((x + b) * b)) with a row vector b."""
    out_shape = tuple(d for i, d in enumerate(shape) if i != axis)
    s, o = _shape(shape), _shape(out_shape)
    if kind == "sum_abs_diff":
        desc = (f"group fn_sum_abs_diff_axis{axis}\ninput X float32 {s}\ninput Y float32 {s}\n"
                f"op subtract d = X Y ; axis=-1\nop abs a = d\nop reduce_sum r = a ; dim={axis} keep_dim=false\n"
                f"output r float32 {o}\n")
        gen = lambda: [_draw(np.random.default_rng(seed), shape, "float32"),  # noqa: E731
                       _draw(np.random.default_rng(seed + 1), shape, "float32")]
    else:
        desc = (f"group fn_sum_sigmoid_affine_axis{axis}\ninput X float32 {s}\ninput B float32 {shape[-1]}\n"
                f"op elementwise_add t = X B ; axis=-1\nop elementwise_mul u = t B ; axis=-1\nop sigmoid v = u\n"
                f"op reduce_sum r = v ; dim={axis} keep_dim=false\noutput r float32 {o}\n")
        gen = lambda: [_draw(np.random.default_rng(seed), shape, "float32"),  # noqa: E731
                       _draw(np.random.default_rng(seed + 1), (shape[-1],), "float32")]
    return Workload("chain_reduce_" + kind, desc, gen, np.float32, out_shape)


def bn_train_inputs(shape=(256, 64, 112, 112), seed=4):
    rng = np.random.default_rng(seed)
    c = shape[1]
    x = rng.standard_normal(shape, dtype=np.float32)
    mean = (0.1 * rng.standard_normal(c)).astype(np.float32)
    var = rng.uniform(0.5, 1.5, c).astype(np.float32)
    scale = (1 + 0.1 * rng.standard_normal(c)).astype(np.float32)
    bias = (0.1 * rng.standard_normal(c)).astype(np.float32)
    return x, mean, var, scale, bias


def bn_train_stats(shape=(256, 64, 112, 112), seed=4, half=False):
    """The statistics pass of the decomposed batch_norm_train: {reduce_sum(x), reduce_sum(x * x)} over N, H, W.
    half=True: x is stored as fp16 and widened by a cast inside the group."""
    s, c = _shape(shape), shape[1]
    if half:
        desc = (f"group fn_bn_train_stats_f16\ninput x16 float16 {s}\nop cast x = x16 ; dtype=float32\n"
                f"op reduce_sum s1 = x ; dim=0,2,3 keep_dim=false\n"
                f"op identity xi = x\nop elementwise_mul xx = x xi ; axis=-1\n"
                f"op reduce_sum s2 = xx ; dim=0,2,3 keep_dim=false\noutput s1 float32 {c}\noutput s2 float32 {c}\n")
        return Workload("bn_train_stats_f16", desc, lambda: [bn_train_inputs(shape, seed)[0].astype(np.float16)],
                        np.float32, (c,), more_outputs=[(np.float32, (c,))])
    desc = (f"group fn_bn_train_stats\ninput x float32 {s}\nop reduce_sum s1 = x ; dim=0,2,3 keep_dim=false\n"
            f"op identity xi = x\nop elementwise_mul xx = x xi ; axis=-1\n"
            f"op reduce_sum s2 = xx ; dim=0,2,3 keep_dim=false\noutput s1 float32 {c}\noutput s2 float32 {c}\n")
    return Workload("bn_train_stats", desc, lambda: [bn_train_inputs(shape, seed)[0]], np.float32, (c,),
                    more_outputs=[(np.float32, (c,))])


def bn_train_apply(shape=(256, 64, 112, 112), seed=4, half=False):
    """The normalisation pass: ((x - mean) * rsqrt(var + eps)) * scale + bias with per-channel operands."""
    s, c = _shape(shape), shape[1]
    bc = f"broadcast_axes=1 out_shape={s}"
    desc = (f"group fn_bn_train_apply\ninput mean float32 {c}\ninput var float32 {c}\ninput x float32 {s}\n"
            f"input scale float32 {c}\ninput bias float32 {c}\n"
            f"op broadcast_to m4 = mean ; {bc}\nop broadcast_to v4 = var ; {bc}\n"
            f"op fill_constant e = ; shape={s} value=1e-05 dtype=float32\nop elementwise_add ve = v4 e ; axis=-1\n"
            f"op rsqrt r = ve\nop subtract d = x m4 ; axis=-1\nop elementwise_mul n = d r ; axis=-1\n"
            f"op broadcast_to s4 = scale ; {bc}\nop elementwise_mul sn = n s4 ; axis=-1\n"
            f"op broadcast_to b4 = bias ; {bc}\nop elementwise_add y = sn b4 ; axis=-1\noutput y float32 {s}\n")

    if half:
        desc = desc.replace("fn_bn_train_apply", "fn_bn_train_apply_f16").replace(f"input x float32 {s}", f"input x16 float16 {s}")
        desc = desc.replace("op broadcast_to m4", "op cast x = x16 ; dtype=float32\nop broadcast_to m4", 1)
        desc = desc.replace(f"output y float32 {s}", f"op cast y16 = y ; dtype=float16\noutput y16 float16 {s}")

    def gen():
        x, mean, var, scale, bias = bn_train_inputs(shape, seed)
        return [mean, var, x.astype(np.float16) if half else x, scale, bias]
    return Workload("bn_train_apply_f16" if half else "bn_train_apply", desc, gen, np.float16 if half else np.float32, shape)


def softmax_safe(shape=(16384, 4096), seed=3, half=False):
    """softmax along the last axis of a 2-D tensor with the row maximum subtracted (the decomposed form of every
    softmax mode but "fast"); half=True stores x and out as fp16 and computes in fp32."""
    rows, cols = shape
    s, r = _shape(shape), str(rows)
    x = "x32" if half else "X"
    lines = ["op cast x32 = X ; dtype=float32"] if half else []
    lines += [
        f"op reduce_max m = {x} ; dim=1 keep_dim=false",
        f"op broadcast_to m2 = m ; broadcast_axes=0 out_shape={s}",
        f"op subtract d = {x} m2 ; axis=-1", "op exp e = d",
        "op reduce_sum sm = e ; dim=1 keep_dim=false",
        f"op broadcast_to s2 = sm ; broadcast_axes=0 out_shape={s}",
        f"op subtract d2 = {x} m2 ; axis=-1", "op exp e2 = d2", "op divide y = e2 s2 ; axis=-1"]
    out = "y"
    if half:
        lines.append("op cast y16 = y ; dtype=float16")
        out = "y16"
    dt = "float16" if half else "float32"
    desc = "group fn_softmax_safe_%s\ninput X %s %s\n%s\noutput %s %s %s\n" % (dt, dt, s, "\n".join(lines), out, dt, s)
    npdt = np.float16 if half else np.float32
    return Workload("softmax_safe_" + dt, desc, lambda: [(3 * rownorm_inputs(shape, seed)[0]).astype(npdt)], npdt, shape)


def transpose(shape, perm, dtype="float32", seed=7):
    out_shape = tuple(shape[p] for p in perm)
    desc = ("group fn_transpose\ninput X %s %s\nop transpose y = X ; axis=%s\noutput y %s %s\n"
            % (dtype, _shape(shape), ",".join(map(str, perm)), dtype, _shape(out_shape)))
    return Workload("transpose", desc, lambda: [_draw(np.random.default_rng(seed), shape, dtype)], _NP[dtype], out_shape)


def concat(shapes, axis, dtype="float32", seed=8):
    out_shape = list(shapes[0])
    out_shape[axis] = sum(s[axis] for s in shapes)
    ins = "\n".join("input X%d %s %s" % (i, dtype, _shape(s)) for i, s in enumerate(shapes))
    desc = ("group fn_concat\n%s\nop concat y = %s ; axis=%d\noutput y %s %s\n"
            % (ins, " ".join("X%d" % i for i in range(len(shapes))), axis, dtype, _shape(out_shape)))

    def gen():
        rng = np.random.default_rng(seed)
        return [_draw(rng, s, dtype) for s in shapes]
    return Workload("concat", desc, gen, _NP[dtype], out_shape)


def bn_grad_stats(shape=(256, 64, 112, 112), seed=4):
    """Statistics pass of the decomposed batch_norm_grad: {sum(dy), sum(dy * (x - mean))} over N, H, W."""
    s, c = _shape(shape), shape[1]
    desc = (f"group fn_bn_grad_stats\ninput mean float32 {c}\ninput x float32 {s}\ninput dy float32 {s}\n"
            f"op broadcast_to m4 = mean ; broadcast_axes=1 out_shape={s}\nop subtract d = x m4 ; axis=-1\n"
            f"op reduce_sum db = dy ; dim=0,2,3 keep_dim=false\nop elementwise_mul p = dy d ; axis=-1\n"
            f"op reduce_sum sd = p ; dim=0,2,3 keep_dim=false\noutput db float32 {c}\noutput sd float32 {c}\n")

    def gen():
        x, mean, var, scale, bias = bn_train_inputs(shape, seed)
        return [mean, x, np.random.default_rng(seed + 100).standard_normal(shape, dtype=np.float32)]
    return Workload("bn_grad_stats", desc, gen, np.float32, (c,), more_outputs=[(np.float32, (c,))])


def bn_grad_apply(shape=(256, 64, 112, 112), seed=4):
    """x_grad of the decomposed batch_norm_grad with its per-channel prologue fused in."""
    s, c = _shape(shape), shape[1]
    cnt = float(shape[0] * shape[2] * shape[3])
    bc = f"broadcast_axes=1 out_shape={s}"
    desc = (f"group fn_bn_grad_apply\ninput scale float32 {c}\ninput var float32 {c}\ninput dy float32 {s}\n"
            f"input db float32 {c}\ninput x float32 {s}\ninput mean float32 {c}\ninput sd float32 {c}\n"
            f"op fill_constant e1 = ; shape={c} value=1e-05 dtype=float32\nop elementwise_add ve1 = var e1 ; axis=-1\n"
            f"op rsqrt r = ve1\nop elementwise_mul sr = scale r ; axis=-1\n"
            f"op fill_constant n1 = ; shape={c} value={cnt} dtype=float32\nop divide t0 = sr n1 ; axis=-1\n"
            f"op broadcast_to t04 = t0 ; {bc}\nop fill_constant n4 = ; shape={s} value={cnt} dtype=float32\n"
            f"op elementwise_mul t1 = dy n4 ; axis=-1\nop broadcast_to t2 = db ; {bc}\n"
            f"op broadcast_to m4 = mean ; {bc}\nop subtract d = x m4 ; axis=-1\nop broadcast_to s4 = sd ; {bc}\n"
            f"op elementwise_mul t30 = d s4 ; axis=-1\nop fill_constant e2 = ; shape={c} value=1e-05 dtype=float32\n"
            f"op elementwise_add ve2 = var e2 ; axis=-1\nop broadcast_to v4 = ve2 ; {bc}\nop divide t3 = t30 v4 ; axis=-1\n"
            f"op subtract a = t1 t2 ; axis=-1\nop subtract b = a t3 ; axis=-1\nop elementwise_mul y = t04 b ; axis=-1\n"
            f"output y float32 {s}\n")

    def gen():
        x, mean, var, scale, bias = bn_train_inputs(shape, seed)
        rng = np.random.default_rng(seed + 100)
        dy = rng.standard_normal(shape, dtype=np.float32)
        return [scale, var, dy, rng.standard_normal(c).astype(np.float32), x, mean, rng.standard_normal(c).astype(np.float32)]
    return Workload("bn_grad_apply", desc, gen, np.float32, shape)


# ---- groups that are neither a chain nor a single reduction ---------------------------------------------------------

def row_program(kind, shape=(16384, 4096), seed=12):
    """Reductions over the last axis with elementwise ops around them, one group (row_prog.cu).  kind: l2_normalise
    (x / sqrt(sum(x^2))), centre (x - mean(x)), affine_relu (relu(sum(x) * a + c), one value per row), three_sums
    (sum(A), sum(B), sum(A + B))."""
    rows, r = shape
    s = _shape(shape)
    if kind == "l2_normalise":
        ins, outs = [f"X float32 {s}"], [("y", "float32", shape)]
        ops = ["identity xi = X", "elementwise_mul xx = X xi ; axis=-1", "reduce_sum s = xx ; dim=1 keep_dim=true",
               "sqrt n = s", f"broadcast_to nb = n ; out_shape={s} broadcast_axes=0,1", "divide y = X nb ; axis=-1"]
    elif kind == "centre":
        ins, outs = [f"X float32 {s}"], [("y", "float32", shape)]
        ops = ["reduce_sum s = X ; dim=1 keep_dim=false", f"fill_constant c = ; shape={rows} value={float(r)} dtype=float32",
               "divide m = s c ; axis=-1", f"broadcast_to mb = m ; out_shape={s} broadcast_axes=0", "subtract y = X mb ; axis=-1"]
    elif kind == "affine_relu":
        ins, outs = [f"X float32 {s}", f"a float32 {rows}", f"c float32 {rows}"], [("y", "float32", (rows,))]
        ops = ["reduce_sum s = X ; dim=1 keep_dim=false", "elementwise_mul t = s a ; axis=-1",
               "elementwise_add u = t c ; axis=-1", "relu y = u"]
    elif kind in ("scaled_softmax", "masked_softmax"):
        ins = [f"X float32 {s}"] + ([f"M float32 {s}"] if kind == "masked_softmax" else [])
        outs = [("y", "float32", shape)]
        ops = ["scale d0 = X ; bias=0.0 bias_after_scale=true scale=0.125"]
        ops += ["elementwise_add d = d0 M ; axis=-1"] if kind == "masked_softmax" else ["identity d = d0"]
        ops += ["reduce_max mx = d ; dim=1 keep_dim=false", f"broadcast_to mb = mx ; broadcast_axes=0 out_shape={s}",
                "subtract z = d mb ; axis=-1", "exp e = z", "reduce_sum sm = e ; dim=1 keep_dim=false",
                f"broadcast_to sb = sm ; broadcast_axes=0 out_shape={s}", "divide y = e sb ; axis=-1"]
    elif kind == "three_sums":
        ins = [f"A float32 {s}", f"B float32 {s}"]
        outs = [("sa", "float32", (rows,)), ("sb", "float32", (rows,)), ("sc", "float32", (rows,))]
        ops = ["elementwise_add c = A B ; axis=-1", "reduce_sum sa = A ; dim=1 keep_dim=false",
               "reduce_sum sb = B ; dim=1 keep_dim=false", "reduce_sum sc = c ; dim=1 keep_dim=false"]
    elif kind in ("rms_norm", "standardise", "log_softmax", "l1_normalise", "moments", "min_max_normalise",
                  "rms_norm_plain", "l2_normalise_eps", "cosine_similarity", "log_sum_exp", "rms_norm_f16"):
        return _row_program_from_builder(kind, shape, seed)
    else:
        raise ValueError(kind)
    desc = (f"group fn_row_{kind}\n" + "".join(f"input {i}\n" for i in ins) + "".join(f"op {o}\n" for o in ops) +
            "".join(f"output {n} {d} {_shape(sh)}\n" for n, d, sh in outs))

    def gen():
        rng = np.random.default_rng(seed)
        return [rng.standard_normal([int(d) for d in i.split()[2].split(",")], dtype=np.float32) for i in ins]
    return Workload("row_" + kind, desc, gen, np.float32, outs[0][2],
                    more_outputs=[(np.float32, sh) for _, _, sh in outs[1:]])


def _row_program_from_builder(kind, shape, seed):
    """The row compositions that the table of specialised kernels lists as NetBuilder programs
    (csrc/gen_static_chains.py: rms_norm, standardise, log_softmax, l1_normalise, moments), at `shape`: the group is
    the one the fusion pass forms from the program."""
    import importlib.util
    import os
    from .frontend import Computation, NetBuilder
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "csrc", "gen_static_chains.py")
    spec = importlib.util.spec_from_file_location("cinn_b200_gen_static_chains", path)
    gen = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(gen)
    make = [m for m in gen.builder_row_programs(*shape) if m.__name__ == kind][0]
    b = NetBuilder("row_" + kind)
    fetch = make(b)
    comp = Computation.build_and_compile(None, b, fetch=[str(f) for f in fetch], plan_only=True)
    groups = comp.groups()
    if len(groups) != 1:
        raise RuntimeError("%s at %s is not one group: %s" % (kind, shape, [p for _, p in groups]))
    desc = groups[0][0]
    ins = [l.split() for l in desc.splitlines() if l.startswith("input ")]
    outs = [l.split() for l in desc.splitlines() if l.startswith("output ")]
    dims = lambda w: tuple(int(d) for d in w[3].split(","))  # noqa: E731

    def gen_inputs():
        rng = np.random.default_rng(seed)
        return [rng.standard_normal(dims(w), dtype=np.float32).astype(_NP[w[2]]) for w in ins]
    return Workload("row_" + kind, desc, gen_inputs, _NP[outs[0][2]], dims(outs[0]),
                    more_outputs=[(_NP[w[2]], dims(w)) for w in outs[1:]])


def dag_program(kind="shared_sum_4out", shape=(8192, 8192), seed=13):
    """Elementwise groups that are not chains (ew_dag.cu).  shared_sum_4out: g = A + B feeding four sums with C..F (six
    reads, four writes); bias_relu_mask_3out: x + bias, its relu and the mask of its positive part; adam_update: both
    moments and the parameter of an Adam step (four reads, three writes; V is made non-negative by the generator)."""
    s = _shape(shape)
    if kind == "shared_sum_4out":
        ins = [f"{n} float32 {s}" for n in "ABCDEF"]
        ops = ["elementwise_add g = A B ; axis=-1"] + [f"elementwise_add {o} = g {i} ; axis=-1" for o, i in zip("hijk", "CDEF")]
        outs = list("hijk")
    elif kind == "bias_relu_mask_3out":
        ins = [f"x float32 {s}", f"b float32 {shape[-1]}"]
        ops = ["elementwise_add pre = x b ; axis=-1", "relu act = pre", f"fill_constant z = ; shape={s} value=0.0 dtype=float32",
               "greater_than m = pre z ; axis=-1", "cast mf = m ; dtype=float32"]
        outs = ["pre", "act", "mf"]
    elif kind == "adam_update":
        ins = [f"{n} float32 {s}" for n in "PGMV"]
        ops = ["scale m1 = M ; scale=0.9 bias=0.0 bias_after_scale=true", "scale g1 = G ; scale=0.1 bias=0.0 bias_after_scale=true",
               "elementwise_add m2 = m1 g1 ; axis=-1", "elementwise_mul gg = G G ; axis=-1",
               "scale v1 = V ; scale=0.999 bias=0.0 bias_after_scale=true", "scale g2 = gg ; scale=0.001 bias=0.0 bias_after_scale=true",
               "elementwise_add v2 = v1 g2 ; axis=-1", "sqrt sv = v2", "scale den = sv ; scale=1.0 bias=1e-08 bias_after_scale=true",
               "divide upd = m2 den ; axis=-1", "scale st = upd ; scale=-0.001 bias=0.0 bias_after_scale=true",
               "elementwise_add p2 = P st ; axis=-1"]
        outs = ["m2", "v2", "p2"]
    else:
        raise ValueError(kind)
    desc = (f"group fn_dag_{kind}\n" + "".join(f"input {i}\n" for i in ins) + "".join(f"op {o}\n" for o in ops) +
            "".join(f"output {o} float32 {s}\n" for o in outs))

    def gen():
        rng = np.random.default_rng(seed)
        arrays = [rng.standard_normal([int(d) for d in i.split()[2].split(",")], dtype=np.float32) for i in ins]
        if kind == "adam_update":
            arrays[3] = np.abs(arrays[3])  # the second moment is a running mean of squares
        return arrays
    return Workload("dag_" + kind, desc, gen, np.float32, shape, more_outputs=[(np.float32, shape)] * (len(outs) - 1))
