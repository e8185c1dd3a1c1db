"""Generates ew_static_table.inc: one STATIC_CHAIN line per elementwise program that gets a kernel specialised at
build time (see ew_static.cu).

    python cinn_b200/csrc/gen_static_chains.py            # rewrite the table, then rebuild the library
    python cinn_b200/csrc/gen_static_chains.py --check    # exit 1 if the committed table is out of date

Each entry of GROUPS is a fused group as the fusion pass would emit it.  The script compiles it with the library's
own matcher (interpreter forced, no GPU needed), reads the plan back as text and turns the interpreted kernel's name,
its `meta` word (operand types and addressing modes) and the low halves of its step words into the template
arguments of one kernel.  Shapes only matter through the addressing mode they give each operand: a full-size operand,
a vector along the last axis, a per-channel vector of NCHW, a single element.  Sizes and immediates stay run-time
parameters of the generated kernel, so an entry serves every shape with the same modes and every constant.

The list holds what elementwise groups of real networks mostly are (bias + activation, residual add, affine,
clamp, masks and compares, casts, gelu / swish) and the groups the benchmark times.
"""
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

FULL = "64,1024"        # a full-size operand
ROWVEC = "1024"         # broadcast along the last axis
NCHW = "8,16,32,32"     # with a per-channel operand [16] on axis 1
CHAN = "16"


def group(name, inputs, ops, out, out_dtype, shape=FULL):
    lines = ["group fn_static_" + name]
    lines += ["input %s" % i for i in inputs]
    lines += ["op %s" % o for o in ops]
    lines.append("output %s %s %s" % (out, out_dtype, shape))
    return name, "\n".join(lines) + "\n"


def unary(op, dt="float32"):
    return group("%s_%s" % (op, dt), ["x %s %s" % (dt, FULL)], ["%s y = x" % op], "y", dt)


def binary(op, dt="float32", out_dt=None, tag=None):
    return group("%s_%s" % (tag or op, dt), ["a %s %s" % (dt, FULL), "b %s %s" % (dt, FULL)],
                 ["%s y = a b ; axis=-1" % op], "y", out_dt or dt)


def bias_act(act, dt="float32"):
    """act(x + bias) with bias along the last axis; 16-bit storage widened by casts as AutoCast leaves it."""
    if dt == "float32":
        ops = ["elementwise_add t = x b ; axis=-1"] + (["%s y = t" % act] if act else [])
        return group("bias_%s_f32" % (act or "add"), ["x float32 " + FULL, "b float32 " + ROWVEC], ops,
                     "y" if act else "t", "float32")
    ops = ["cast x32 = x ; dtype=float32", "elementwise_add t = x32 b ; axis=-1"]
    ops += ["%s u = t" % act] if act else ["identity u = t"]
    ops += ["cast y = u ; dtype=%s" % dt]
    return group("bias_%s_%s" % (act or "add", dt), ["x %s %s" % (dt, FULL), "b float32 " + ROWVEC], ops, "y", dt)


GROUPS = []
# unary math
for op in ("relu", "sigmoid", "tanh", "exp", "log", "sqrt", "rsqrt", "abs", "negative", "reciprocal", "erf"):
    GROUPS.append(unary(op))
for op in ("relu", "sigmoid", "tanh", "exp"):
    GROUPS.append(group("%s_f16" % op, ["x float16 " + FULL], ["cast a = x ; dtype=float32", "%s b = a" % op,
                                                                  "cast y = b ; dtype=float16"], "y", "float16"))
# binary, both operands full size
for op, tag in (("elementwise_add", "add"), ("subtract", "sub"), ("elementwise_mul", "mul"), ("divide", "div"),
                ("max", "max"), ("min", "min")):
    GROUPS.append(binary(op, tag=tag))
for op in ("greater_than", "less_than", "equal", "greater_equal"):
    GROUPS.append(binary(op, out_dt="bool"))
GROUPS.append(binary("logical_and", dt="bool"))
GROUPS.append(binary("logical_or", dt="bool"))
for op, tag in (("elementwise_add", "add"), ("elementwise_mul", "mul")):
    GROUPS.append(group("%s_f16" % tag, ["a float16 " + FULL, "b float16 " + FULL],
                        ["cast a32 = a ; dtype=float32", "cast b32 = b ; dtype=float32",
                         "%s t = a32 b32 ; axis=-1" % op, "cast y = t ; dtype=float16"], "y", "float16"))
# the benchmark's generic groups
GROUPS.append(group("abs_add_f32", ["A float32 " + FULL, "B float32 " + FULL],
                    ["elementwise_add t0 = A B", "abs t1 = t0"], "t1", "float32"))
GROUPS.append(group("select_f32", ["M bool " + FULL, "A float32 " + FULL, "B float32 " + FULL],
                    ["select t0 = M A B"], "t0", "float32"))
GROUPS.append(group("tree_add_mul_sub_f32", ["A float32 " + FULL, "B float32 " + FULL, "C float32 " + FULL,
                                             "D float32 " + FULL],
                    ["elementwise_add s = A B ; axis=-1", "subtract d = C D ; axis=-1",
                     "elementwise_mul y = s d ; axis=-1"], "y", "float32"))
# bias (last axis) + activation
for act in (None, "relu", "sigmoid", "tanh", "gelu"):
    if act == "gelu":
        continue
    GROUPS.append(bias_act(act))
for act in (None, "relu", "sigmoid"):
    GROUPS.append(bias_act(act, "float16"))
# residual: relu(a + b) exists as a dedicated kernel; three-operand sum and add + activation variants
GROUPS.append(group("add3_f32", ["a float32 " + FULL, "b float32 " + FULL, "c float32 " + FULL],
                    ["elementwise_add t = a b ; axis=-1", "elementwise_add y = t c ; axis=-1"], "y", "float32"))
GROUPS.append(group("add_sigmoid_f32", ["a float32 " + FULL, "b float32 " + FULL],
                    ["elementwise_add t = a b ; axis=-1", "sigmoid y = t"], "y", "float32"))
GROUPS.append(group("add_tanh_f32", ["a float32 " + FULL, "b float32 " + FULL],
                    ["elementwise_add t = a b ; axis=-1", "tanh y = t"], "y", "float32"))
# affine forms
GROUPS.append(group("scale_f32", ["x float32 " + FULL], ["scale y = x ; scale=2.0 bias=1.0 bias_after_scale=true"],
                    "y", "float32"))
GROUPS.append(group("scale_relu_f32", ["x float32 " + FULL],
                    ["scale t = x ; scale=2.0 bias=1.0 bias_after_scale=true", "relu y = t"], "y", "float32"))
GROUPS.append(group("mul_add_f32", ["x float32 " + FULL, "a float32 " + FULL, "b float32 " + FULL],
                    ["elementwise_mul t = x a ; axis=-1", "elementwise_add y = t b ; axis=-1"], "y", "float32"))
GROUPS.append(group("rowvec_mul_add_f32", ["x float32 " + FULL, "g float32 " + ROWVEC, "b float32 " + ROWVEC],
                    ["elementwise_mul t = x g ; axis=-1", "elementwise_add y = t b ; axis=-1"], "y", "float32"))
GROUPS.append(group("channel_mul_add_f32", ["x float32 " + NCHW, "g float32 " + CHAN, "b float32 " + CHAN],
                    ["elementwise_mul t = x g ; axis=1", "elementwise_add y = t b ; axis=1"], "y", "float32", NCHW))
GROUPS.append(group("channel_mul_add_relu_f32", ["x float32 " + NCHW, "g float32 " + CHAN, "b float32 " + CHAN],
                    ["elementwise_mul t = x g ; axis=1", "elementwise_add u = t b ; axis=1", "relu y = u"], "y",
                    "float32", NCHW))
# clamp, masks, casts
GROUPS.append(group("clip_f32", ["x float32 " + FULL],
                    ["fill_constant lo = ; shape=%s value=-1.0 dtype=float32" % FULL, "max t = x lo ; axis=-1",
                     "fill_constant hi = ; shape=%s value=1.0 dtype=float32" % FULL, "min y = t hi ; axis=-1"],
                    "y", "float32"))
GROUPS.append(unary("relu6"))
GROUPS.append(group("dropout_apply_f32", ["x float32 " + FULL, "m float32 " + FULL],
                    ["elementwise_mul t = x m ; axis=-1", "scale y = t ; scale=1.25 bias=0.0 bias_after_scale=true"],
                    "y", "float32"))
GROUPS.append(group("cast_f32_f16", ["x float32 " + FULL], ["cast y = x ; dtype=float16"], "y", "float16"))
GROUPS.append(group("cast_f16_f32", ["x float16 " + FULL], ["cast y = x ; dtype=float32"], "y", "float32"))
GROUPS.append(group("cast_f32_bf16", ["x float32 " + FULL], ["cast y = x ; dtype=bfloat16"], "y", "bfloat16"))
# squared difference, swish, gelu (as the decomposer writes it)
GROUPS.append(group("sq_diff_f32", ["a float32 " + FULL, "b float32 " + FULL],
                    ["subtract d = a b ; axis=-1", "identity di = d", "elementwise_mul y = d di ; axis=-1"], "y",
                    "float32"))
GROUPS.append(group("swish_f32", ["x float32 " + FULL], ["sigmoid s = x", "elementwise_mul y = x s ; axis=-1"], "y",
                    "float32"))
# two outputs: the pre-activation kept beside the activation
GROUPS.append(("bias_pre_and_relu_f32",
               "group fn_static_bias_pre_and_relu_f32\ninput X float32 %s\ninput bias float32 %s\n"
               "op elementwise_add pre = X bias ; axis=-1\nop relu act = pre\n"
               "output pre float32 %s\noutput act float32 %s\n" % (FULL, ROWVEC, FULL, FULL)))
# swish with its sigmoid kept, a momentum step (velocity and parameter), gelu's tanh form with the tanh kept: chains
# that store one value on the way
GROUPS.append(("swish_and_sigmoid_f32",
               "group fn_static_swish_and_sigmoid_f32\ninput x float32 %s\nop sigmoid s = x\n"
               "op elementwise_mul y = x s ; axis=-1\noutput s float32 %s\noutput y float32 %s\n" % (FULL, FULL, FULL)))
GROUPS.append(("momentum_update_f32",
               "group fn_static_momentum_update_f32\ninput W float32 %s\ninput G float32 %s\ninput V float32 %s\n"
               "op scale v1 = V ; scale=0.9 bias=0.0 bias_after_scale=true\nop elementwise_add v2 = v1 G ; axis=-1\n"
               "op scale st = v2 ; scale=-0.01 bias=0.0 bias_after_scale=true\nop elementwise_add w2 = W st ; axis=-1\n"
               "output v2 float32 %s\noutput w2 float32 %s\n" % (FULL, FULL, FULL, FULL, FULL)))
GROUPS.append(("gelu_tanh_kept_f32",
               "group fn_static_gelu_tanh_kept_f32\ninput x float32 %s\nop elementwise_mul x2 = x x ; axis=-1\n"
               "op elementwise_mul x3 = x2 x ; axis=-1\nop scale c = x3 ; scale=0.044715 bias=0.0 bias_after_scale=true\n"
               "op elementwise_add u = x c ; axis=-1\nop scale w = u ; scale=0.7978845608 bias=0.0 bias_after_scale=true\n"
               "op tanh t = w\nop scale h = t ; scale=0.5 bias=0.5 bias_after_scale=true\n"
               "op elementwise_mul y = x h ; axis=-1\noutput y float32 %s\noutput t float32 %s\n" % (FULL, FULL, FULL)))


# What the NetBuilder emits for the activation and backward forms below (the decomposed gelu of
# cinn/frontend/decomposer/activation.cc, relu_grad, the sigmoid / tanh derivatives written with the primitive ops,
# softplus, a scaled residual): group texts as the fusion pass prints them, so that users' programs meet the entries.
def _raw(name, body):
    return name, "group fn_static_%s\n%s" % (name, body)


_GELU = ("op fill_constant h = ; dtype=float32 shape={s} value=0.5\n"
         "op fill_constant r = ; dtype=float32 shape={s} value=0.7071067811865476\n"
         "op elementwise_mul u = {x} r ; axis=-1\nop erf e = u\nop elementwise_mul v = h e ; axis=-1\n"
         "op elementwise_add w = h v ; axis=-1\nop elementwise_mul y = {x} w ; axis=-1\n")
GROUPS += [
    _raw("gelu_f32", "input x float32 %s\n" % FULL + _GELU.format(s=FULL, x="x") + "output y float32 %s\n" % FULL),
    _raw("bias_gelu_f32", "input x float32 %s\ninput b float32 %s\nop elementwise_add t = x b ; axis=-1\n" % (FULL, ROWVEC) +
         _GELU.format(s=FULL, x="t") + "output y float32 %s\n" % FULL),
    _raw("gelu_f16", "input x float16 %s\nop cast xf = x ; dtype=float32\n" % FULL + _GELU.format(s=FULL, x="xf") +
         "op cast z = y ; dtype=float16\noutput z float16 %s\n" % FULL),
    _raw("relu_grad_f32", "input y float32 {s}\ninput dy float32 {s}\nop fill_constant z = ; dtype=float32 shape={s} value=0.0\n"
         "op greater_than m = y z ; axis=-1\nop select g = m dy z\noutput g float32 {s}\n".format(s=FULL)),
    _raw("sigmoid_grad_f32", "input y float32 {s}\ninput dy float32 {s}\n"
         "op scale c = y ; bias=1.0 bias_after_scale=true scale=-1.0\nop elementwise_mul t = y c ; axis=-1\n"
         "op elementwise_mul g = dy t ; axis=-1\noutput g float32 {s}\n".format(s=FULL)),
    _raw("tanh_grad_f32", "input y float32 {s}\ninput dy float32 {s}\nop elementwise_mul q = y y ; axis=-1\n"
         "op scale c = q ; bias=1.0 bias_after_scale=true scale=-1.0\nop elementwise_mul g = dy c ; axis=-1\n"
         "output g float32 {s}\n".format(s=FULL)),
    _raw("softplus_f32", "input x float32 {s}\nop exp e = x\nop scale p = e ; bias=1.0 bias_after_scale=true scale=1.0\n"
         "op log y = p\noutput y float32 {s}\n".format(s=FULL)),
    _raw("residual_scale_f32", "input f float32 {s}\ninput x float32 {s}\n"
         "op scale t = f ; bias=0.0 bias_after_scale=true scale=0.5\nop elementwise_add y = x t ; axis=-1\n"
         "output y float32 {s}\n".format(s=FULL)),
]


def reduce_group(name, inputs, ops, red, operand, axis, shape=FULL):
    """reduce_<red>(chain) over one axis of a 2-D shape: rows (axis 1) or columns (axis 0)."""
    dims = [int(d) for d in shape.split(",")]
    out_shape = ",".join(str(d) for i, d in enumerate(dims) if i != axis)
    lines = ["group fn_static_" + name] + ["input %s" % i for i in inputs] + ["op %s" % o for o in ops]
    lines.append("op reduce_%s y = %s ; dim=%d keep_dim=false" % (red, operand, axis))
    lines.append("output y float32 " + out_shape)
    return name, "\n".join(lines) + "\n"


REDUCE_GROUPS = []
for axis, tag in ((1, "rows"), (0, "cols")):
    two = ["x float32 " + FULL, "y0 float32 " + FULL]
    REDUCE_GROUPS.append(reduce_group("sum_abs_diff_" + tag, two, ["subtract d = x y0 ; axis=-1", "abs a = d"], "sum",
                                      "a", axis))
    REDUCE_GROUPS.append(reduce_group("sum_sq_diff_" + tag, two, ["subtract d = x y0 ; axis=-1", "identity di = d",
                                                                   "elementwise_mul a = d di ; axis=-1"], "sum", "a",
                                      axis))
    REDUCE_GROUPS.append(reduce_group("sum_mul_" + tag, two, ["elementwise_mul a = x y0 ; axis=-1"], "sum", "a", axis))
    REDUCE_GROUPS.append(reduce_group("max_abs_diff_" + tag, two, ["subtract d = x y0 ; axis=-1", "abs a = d"], "max",
                                      "a", axis))
    REDUCE_GROUPS.append(reduce_group("sum_sigmoid_affine_" + tag, ["x float32 " + FULL, "b float32 " + ROWVEC],
                                      ["elementwise_add t = x b ; axis=-1", "elementwise_mul u = t b ; axis=-1",
                                       "sigmoid a = u"], "sum", "a", axis))
    REDUCE_GROUPS.append(reduce_group("sum_log_" + tag, ["x float32 " + FULL], ["log a = x"], "sum", "a", axis))
    REDUCE_GROUPS.append(reduce_group("sum_relu_bias_" + tag, ["x float32 " + FULL, "b float32 " + ROWVEC],
                                      ["elementwise_add t = x b ; axis=-1", "relu a = t"], "sum", "a", axis))
    REDUCE_GROUPS.append(reduce_group("max_scale_" + tag, ["x float32 " + FULL],
                                      ["scale a = x ; scale=0.5 bias=1.0 bias_after_scale=true"], "max", "a", axis))

def multi(name, inputs, ops, outputs, shape=FULL, dt="float32"):
    lines = ["group fn_static_" + name] + ["input %s" % i for i in inputs] + ["op %s" % o for o in ops]
    lines += ["output %s %s %s" % (o, dt, shape) for o in outputs]
    return name, "\n".join(lines) + "\n"


def _f(names, shape=FULL):
    return ["%s float32 %s" % (n, shape) for n in names]


# Elementwise groups that are not chains (register programs, ew_dag.cu): a value used several times, several outputs.
DAG_GROUPS = [
    # a shared sum feeding two, three and four consumers (the shapes of the reference's merge-pass tests)
    multi("shared_sum_2out", _f("ABCD"), ["elementwise_add e = A B ; axis=-1", "elementwise_add f = e C ; axis=-1",
                                          "elementwise_add g = e D ; axis=-1"], ["f", "g"]),
    multi("shared_sum_joined", _f("ABCD"), ["elementwise_add e = A B ; axis=-1", "elementwise_add f = e C ; axis=-1",
                                            "elementwise_add g = e D ; axis=-1", "elementwise_add h = f g ; axis=-1"],
          ["h"]),
    multi("two_sums_3out", _f("ABCDEF"), ["elementwise_add g = A B ; axis=-1", "elementwise_add h = C D ; axis=-1",
                                          "elementwise_add i = E g ; axis=-1", "elementwise_add j = g h ; axis=-1",
                                          "elementwise_add k = h F ; axis=-1"], ["i", "j", "k"]),
    multi("shared_sum_4out", _f("ABCDEF"), ["elementwise_add g = A B ; axis=-1", "elementwise_add h = g C ; axis=-1",
                                            "elementwise_add i = g D ; axis=-1", "elementwise_add j = g E ; axis=-1",
                                            "elementwise_add k = g F ; axis=-1"], ["h", "i", "j", "k"]),
    # bias vectors summed first, then broadcast into two full-size sums
    multi("bias_sum_2out", _f("AB", ROWVEC) + _f("CD"), ["elementwise_add e = A B ; axis=-1",
                                                        "elementwise_add f = C e ; axis=-1",
                                                        "elementwise_add g = D e ; axis=-1"], ["f", "g"]),
    # what training graphs keep: the pre-activation, the activation and its mask
    multi("bias_relu_mask_3out", ["x float32 " + FULL, "b float32 " + ROWVEC],
          ["elementwise_add pre = x b ; axis=-1", "relu act = pre",
           "fill_constant z = ; shape=%s value=0.0 dtype=float32" % FULL, "greater_than m = pre z ; axis=-1",
           "cast mf = m ; dtype=float32"], ["pre", "act", "mf"]),
    # Adam: both moments and the parameter from one read of the gradient (three outputs)
    multi("adam_update", _f("PGMV"),
          ["scale m1 = M ; scale=0.9 bias=0.0 bias_after_scale=true",
           "scale g1 = G ; scale=0.1 bias=0.0 bias_after_scale=true",
           "elementwise_add m2 = m1 g1 ; axis=-1",
           "elementwise_mul gg = G G ; axis=-1",
           "scale v1 = V ; scale=0.999 bias=0.0 bias_after_scale=true",
           "scale g2 = gg ; scale=0.001 bias=0.0 bias_after_scale=true",
           "elementwise_add v2 = v1 g2 ; axis=-1",
           "sqrt sv = v2",
           "scale den = sv ; scale=1.0 bias=1e-08 bias_after_scale=true",
           "divide upd = m2 den ; axis=-1",
           "scale st = upd ; scale=-0.001 bias=0.0 bias_after_scale=true",
           "elementwise_add p2 = P st ; axis=-1"], ["m2", "v2", "p2"]),
]

# Row programs (row_prog.cu): reductions over the last axis with elementwise ops around them.  Two row lengths per
# program: one that a warp takes (1024) and one that a CTA takes (4096) plan to the same program, so one entry each.
ROWS = "64,4096"


def row_group(name, inputs, ops, outputs):
    lines = ["group fn_static_" + name] + ["input %s" % i for i in inputs] + ["op %s" % o for o in ops]
    lines += ["output %s" % o for o in outputs]
    return name, "\n".join(lines) + "\n"


ROW_GROUPS = [
    row_group("l2_normalise", ["X float32 " + ROWS],
              ["identity xi = X", "elementwise_mul xx = X xi ; axis=-1", "reduce_sum s = xx ; dim=1 keep_dim=true",
               "sqrt n = s", "broadcast_to nb = n ; out_shape=%s broadcast_axes=0,1" % ROWS, "divide y = X nb ; axis=-1"],
              ["y float32 " + ROWS]),
    row_group("centre", ["X float32 " + ROWS],
              ["reduce_sum s = X ; dim=1 keep_dim=false", "fill_constant c = ; shape=64 value=4096.0 dtype=float32",
               "divide m = s c ; axis=-1", "broadcast_to mb = m ; out_shape=%s broadcast_axes=0" % ROWS,
               "subtract y = X mb ; axis=-1"], ["y float32 " + ROWS]),
    row_group("row_affine_relu", ["X float32 " + ROWS, "a float32 64", "c float32 64"],
              ["reduce_sum s = X ; dim=1 keep_dim=false", "elementwise_mul t = s a ; axis=-1",
               "elementwise_add u = t c ; axis=-1", "relu y = u"], ["y float32 64"]),
    row_group("shifted_exp_normalised", ["X float32 " + ROWS],
              ["reduce_max mx = X ; dim=1 keep_dim=false", "broadcast_to mb = mx ; out_shape=%s broadcast_axes=0" % ROWS,
               "subtract d = X mb ; axis=-1", "exp e = d", "reduce_sum s = e ; dim=1 keep_dim=false",
               "broadcast_to sb = s ; out_shape=%s broadcast_axes=0" % ROWS, "divide p = e sb ; axis=-1",
               "scale y = p ; scale=2.0 bias=0.0 bias_after_scale=true"], ["y float32 " + ROWS]),
    # attention scores: softmax of the scaled (and masked) scores, maximum subtracted -- the scaling and the mask join
    # the softmax in one kernel instead of running as a chain kernel in front of the dedicated softmax kernel
    row_group("scaled_softmax", ["X float32 " + ROWS],
              ["scale d = X ; bias=0.0 bias_after_scale=true scale=0.125",
               "reduce_max mx = d ; dim=1 keep_dim=false", "broadcast_to mb = mx ; broadcast_axes=0 out_shape=%s" % ROWS,
               "subtract z = d mb ; axis=-1", "exp e = z", "reduce_sum s = e ; dim=1 keep_dim=false",
               "broadcast_to sb = s ; broadcast_axes=0 out_shape=%s" % ROWS, "divide y = e sb ; axis=-1"],
              ["y float32 " + ROWS]),
    row_group("masked_softmax", ["X float32 " + ROWS, "M float32 " + ROWS],
              ["scale d0 = X ; bias=0.0 bias_after_scale=true scale=0.125", "elementwise_add d = d0 M ; axis=-1",
               "reduce_max mx = d ; dim=1 keep_dim=false", "broadcast_to mb = mx ; broadcast_axes=0 out_shape=%s" % ROWS,
               "subtract z = d mb ; axis=-1", "exp e = z", "reduce_sum s = e ; dim=1 keep_dim=false",
               "broadcast_to sb = s ; broadcast_axes=0 out_shape=%s" % ROWS, "divide y = e sb ; axis=-1"],
              ["y float32 " + ROWS]),
    row_group("three_sums", ["A float32 " + ROWS, "B float32 " + ROWS],
              ["elementwise_add c = A B ; axis=-1", "reduce_sum sa = A ; dim=1 keep_dim=false",
               "reduce_sum sb = B ; dim=1 keep_dim=false", "reduce_sum sc = c ; dim=1 keep_dim=false"],
              ["sa float32 64", "sb float32 64", "sc float32 64"]),
]

# Integer chains (ew_chain_int.cu): index arithmetic, masks and counters.
def _i(names, dt="int32"):
    return ["%s %s %s" % (n, dt, FULL) for n in names]


INT_GROUPS = [
    group("abs_add_i32", _i("AB"), ["elementwise_add t0 = A B", "abs t1 = t0"], "t1", "int32"),
    group("add_i32", _i("AB"), ["elementwise_add y = A B ; axis=-1"], "y", "int32"),
    group("sub_i32", _i("AB"), ["subtract y = A B ; axis=-1"], "y", "int32"),
    group("mul_i32", _i("AB"), ["elementwise_mul y = A B ; axis=-1"], "y", "int32"),
    group("max_i32", _i("AB"), ["max y = A B ; axis=-1"], "y", "int32"),
    group("equal_i32", _i("AB"), ["equal y = A B ; axis=-1"], "y", "bool"),
    group("less_than_i32", _i("AB"), ["less_than y = A B ; axis=-1"], "y", "bool"),
    group("bitwise_and_i32", _i("AB"), ["bitwise_and y = A B ; axis=-1"], "y", "int32"),
    group("add_i64", _i("AB", "int64"), ["elementwise_add y = A B ; axis=-1"], "y", "int64"),
    group("mul_add_i32", _i("ABC"), ["elementwise_mul t = A B ; axis=-1", "elementwise_add y = t C ; axis=-1"], "y", "int32"),
]
INT_T = {"i32": "int32_t", "i64": "long long", "bool": "uint8_t", "f32": "float"}


F64_GROUPS = [
    group("affine_abs_f64", _i("A", "float64"), ["scale t0 = A ; scale=0.1 bias=1e-05", "abs t1 = t0"], "t1", "float64"),
    group("abs_add_f64", _i("AB", "float64"), ["elementwise_add t0 = A B", "abs t1 = t0"], "t1", "float64"),
    group("add_f64", _i("AB", "float64"), ["elementwise_add y = A B ; axis=-1"], "y", "float64"),
    group("sub_f64", _i("AB", "float64"), ["subtract y = A B ; axis=-1"], "y", "float64"),
    group("mul_f64", _i("AB", "float64"), ["elementwise_mul y = A B ; axis=-1"], "y", "float64"),
    group("div_f64", _i("AB", "float64"), ["divide y = A B ; axis=-1"], "y", "float64"),
    group("max_f64", _i("AB", "float64"), ["max y = A B ; axis=-1"], "y", "float64"),
    group("less_than_f64", _i("AB", "float64"), ["less_than y = A B ; axis=-1"], "y", "bool"),
    group("mul_add_f64", _i("ABC", "float64"), ["elementwise_mul t = A B ; axis=-1", "elementwise_add y = t C ; axis=-1"], "y", "float64"),
    group("scale_f64", _i("A", "float64"), ["scale y = A ; scale=2.0 bias=1.0"], "y", "float64"),
    group("relu_f64", _i("A", "float64"), ["relu y = A"], "y", "float64"),
    group("cast_f64_f32", _i("A", "float64"), ["cast y = A ; dtype=float32"], "y", "float32"),
]
F64_T = {"f64": "double", "f32": "float", "bool": "uint8_t"}


def typed_table_lines(groups, kernel_re, line_of):
    """One table line per distinct program among `groups` whose interpreted kernel's name matches `kernel_re`;
    line_of(name, kernel, match, ns, nt, meta, sig) formats it."""
    import cinn_b200
    L = cinn_b200.lib()
    cinn_b200._lib.check(L.cinn_b200_set_option(b"enable_static_chains", 0))
    try:
        seen, lines, skipped = {}, [], []
        for name, desc in groups:
            try:
                g = cinn_b200.FusedGroup(desc)
            except cinn_b200.CinnB200Error as e:
                skipped.append("%s: %s" % (name, e))
                continue
            text = g.launch_text()
            g.release()
            kernel = [l for l in text.splitlines() if l.startswith("launch ")][0].split()[2]
            m = re.match(kernel_re, kernel)
            if not m:
                skipped.append("%s: not a chain of this form (%s)" % (name, kernel))
                continue
            args = {int(l.split()[1]): int(l.split()[3]) for l in text.splitlines() if l.startswith("arg ") and l.split()[2] == "int"}
            meta, nsteps = args[7], args[14]
            sig = tuple(args[15 + k] & 0xffffffff for k in range(nsteps))
            ns, nt, _ = VARIANT[m.groups()[-1]]
            if nsteps == 0 or (kernel, meta, sig) in seen:
                skipped.append("%s: empty or repeated program" % name)
                continue
            seen[(kernel, meta, sig)] = name
            lines.append(line_of(name, kernel, m, ns, nt, meta, ", ".join("0x%08xu" % w for w in sig)))
        return lines, skipped
    finally:
        L.cinn_b200_set_option(b"enable_static_chains", 1)


def int_table_lines():
    return typed_table_lines(
        INT_GROUPS, r"ew_chain_int_(i32|i64)_(i32|i64|bool|f32)(_s\w+)$",
        lambda name, kernel, m, ns, nt, meta, sig: 'STATIC_INT_CHAIN(%s, "%s", %s, %s, %d, %d, %d, %s);' % (
            name, kernel, INT_T[m.group(1)], INT_T[m.group(2)], ns, nt, meta, sig))


def f64_table_lines():
    return typed_table_lines(
        F64_GROUPS, r"ew_chain_f64_(f64|f32|bool)(_s\w+)$",
        lambda name, kernel, m, ns, nt, meta, sig: 'STATIC_F64_CHAIN(%s, "%s", %s, %d, %d, %d, %s);' % (
            name, kernel, F64_T[m.group(1)], ns, nt, meta, sig))


def builder_programs():
    """Small NetBuilder programs whose register-program groups get kernels too: the shared-value graphs of the
    reference's fusion tests (cinn/hlir/pass/fusion_merge_pass_test.cc:47-71, 131-158, 182-205;
    op_fusion_pass_test.cc:95-119) that no entry above already equals.  The group descriptions are the fusion pass's
    own, so the programs match what a user's graph of that form compiles to."""
    from cinn_b200 import common
    from cinn_b200.frontend import NetBuilder

    def ins(b, **shapes):
        return {k: b.create_input(common.Float(32), v, k) for k, v in shapes.items()}
    H, W = 32, 32

    def twice_the_same_sum(b):
        v = ins(b, A=(H, W), B=(H, W), C=(H, W), D=(H, W))
        e, f = b.add(v["A"], v["B"]), b.add(v["C"], v["D"])
        return [b.add(e, f), b.add(e, f)]

    def two_levels_of_sharing(b):
        v = ins(b, A=(H, W), B=(H, W), C=(H, W), D=(H, W), E=(H, W), F=(H, W))
        g = b.add(v["A"], v["B"])
        i = b.add(g, v["D"])
        return [b.add(g, v["C"]), b.add(i, v["E"]), b.add(i, v["F"])]

    def vector_sum_into_matrix_sum(b):
        v = ins(b, A=(W,), B=(W,), C=(H, W), D=(H, W))
        return [b.add(b.add(v["C"], v["D"]), b.add(v["A"], v["B"]))]

    def column_vector_sum_then_two_more(b):
        v = ins(b, A=(W,), B=(W,), C=(H, W), D=(H, W))
        e, f = b.add(v["A"], v["B"]), b.add(v["C"], v["D"])
        return [b.add(b.add(b.add(f, e, axis=0), v["C"]), v["D"])]

    def vector_sum_recomputed_in_two_shapes(b):  # fusion_merge_pass_test.cc:257-280: E = A + B joins both consumers
        v = ins(b, A=(W,), B=(W,), C=(H * W, W), D=(H, W))
        e = b.add(v["A"], v["B"])
        return [b.add(v["C"], e), b.add(v["D"], e)]

    return [twice_the_same_sum, two_levels_of_sharing, vector_sum_into_matrix_sum, column_vector_sum_then_two_more,
            vector_sum_recomputed_in_two_shapes]


def builder_row_programs(R=64, C=4096):
    """Row compositions written with the NetBuilder, as a user's program would: the fusion pass's own description of
    their row-program group goes into the table, so that such programs run as ONE specialised kernel (the constants
    and the shape are parameters of that kernel, not part of its key)."""
    from cinn_b200 import common
    F32 = common.Float(32)

    def rms_norm(b):  # x * rsqrt(mean(x^2) + eps) * gamma
        x, g = b.create_input(F32, (R, C), "X"), b.create_input(F32, (C,), "G")
        inv = b.rsqrt(b.scale(b.reduce_sum(b.multiply(x, x), [1]), 1.0 / C, 1e-6))
        return [b.multiply(b.multiply(x, b.broadcast_to(inv, [R, C], [0])), g)]

    def standardise(b):  # (x - mean) * rsqrt(var + eps): three passes over a row held in registers
        x = b.create_input(F32, (R, C), "X")
        n = b.fill_constant([R], float(C))
        xc = b.subtract(x, b.broadcast_to(b.divide(b.reduce_sum(x, [1]), n), [R, C], [0]))
        var = b.divide(b.reduce_sum(b.multiply(xc, xc), [1]), n)
        return [b.multiply(xc, b.broadcast_to(b.rsqrt(b.scale(var, 1.0, 1e-5)), [R, C], [0]))]

    def log_softmax(b):
        x = b.create_input(F32, (R, C), "X")
        d = b.subtract(x, b.broadcast_to(b.reduce_max(x, [1]), [R, C], [0]))
        return [b.subtract(d, b.broadcast_to(b.log(b.reduce_sum(b.exp(d), [1])), [R, C], [0]))]

    def l1_normalise(b):
        x = b.create_input(F32, (R, C), "X")
        return [b.divide(x, b.broadcast_to(b.reduce_sum(b.abs(x), [1]), [R, C], [0]))]

    def moments(b):  # mean and variance per row from one read
        x = b.create_input(F32, (R, C), "X")
        n = b.fill_constant([R], float(C))
        m = b.divide(b.reduce_sum(x, [1]), n)
        return [m, b.subtract(b.divide(b.reduce_sum(b.multiply(x, x), [1]), n), b.multiply(m, m))]

    def min_max_normalise(b):  # (x - min) / (max - min): two reductions of the same operand in one pass
        x = b.create_input(F32, (R, C), "X")
        mn, mx = b.reduce_min(x, [1]), b.reduce_max(x, [1])
        return [b.divide(b.subtract(x, b.broadcast_to(mn, [R, C], [0])), b.broadcast_to(b.subtract(mx, mn), [R, C], [0]))]

    def rms_norm_plain(b):  # without the weight vector
        x = b.create_input(F32, (R, C), "X")
        inv = b.rsqrt(b.scale(b.reduce_sum(b.multiply(x, x), [1]), 1.0 / C, 1e-6))
        return [b.multiply(x, b.broadcast_to(inv, [R, C], [0]))]

    def l2_normalise_eps(b):  # x / max(||x||, eps)
        x = b.create_input(F32, (R, C), "X")
        n = b.sqrt(b.reduce_sum(b.multiply(x, x), [1]))
        return [b.divide(x, b.broadcast_to(b.max(n, b.fill_constant([R], 1e-12)), [R, C], [0]))]

    def cosine_similarity(b):  # three sums from one read of two tensors, one value per row
        x, y = b.create_input(F32, (R, C), "X"), b.create_input(F32, (R, C), "Y")
        xy, xx, yy = (b.reduce_sum(b.multiply(p, q), [1]) for p, q in ((x, y), (x, x), (y, y)))
        return [b.divide(xy, b.sqrt(b.multiply(xx, yy)))]

    def log_sum_exp(b):
        x = b.create_input(F32, (R, C), "X")
        mx = b.reduce_max(x, [1])
        s = b.reduce_sum(b.exp(b.subtract(x, b.broadcast_to(mx, [R, C], [0]))), [1])
        return [b.add(mx, b.log(s))]

    def rms_norm_16bit(T, suffix):  # 16-bit storage of x, the weight and the result, fp32 arithmetic between casts
        def make(b):
            x, g = b.create_input(T, (R, C), "X"), b.create_input(T, (C,), "G")
            xf, gf = b.cast(x, "float32"), b.cast(g, "float32")
            inv = b.rsqrt(b.scale(b.reduce_sum(b.multiply(xf, xf), [1]), 1.0 / C, 1e-6))
            return [b.cast(b.multiply(b.multiply(xf, b.broadcast_to(inv, [R, C], [0])), gf), suffix)]
        make.__name__ = "rms_norm_" + {"float16": "f16", "bfloat16": "bf16"}[suffix]
        return make

    return [rms_norm, standardise, log_softmax, l1_normalise, moments, min_max_normalise, rms_norm_plain,
            l2_normalise_eps, cosine_similarity, log_sum_exp, rms_norm_16bit(common.Float16(), "float16"),
            rms_norm_16bit(common.BFloat16(), "bfloat16")]


def builder_groups(programs, pattern):
    """(name, description) of the groups of `pattern` that the fusion pass forms from the given builder programs when
    it may form interpreted program groups."""
    import cinn_b200
    from cinn_b200.frontend import Computation, NetBuilder
    L = cinn_b200.lib()
    L.cinn_b200_set_option(b"fuse_interpreted_programs", 1)
    L.cinn_b200_set_option(b"enable_static_chains", 0)
    out = []
    try:
        for make in programs:
            b = NetBuilder(make.__name__)
            fetch = make(b)
            comp = Computation.build_and_compile(None, b, fetch=[str(f) for f in fetch], plan_only=True)
            k = 0
            for desc, pat in comp.groups():
                if pat.split()[0] == pattern:
                    lines = desc.splitlines()
                    name = make.__name__ + ("_%d" % k if k else "")
                    k += 1
                    lines[0] = "group fn_static_" + name
                    out.append((name, "\n".join(lines) + "\n"))
    finally:
        L.cinn_b200_set_option(b"fuse_interpreted_programs", 0)
        L.cinn_b200_set_option(b"enable_static_chains", 1)
    return out


def builder_dag_groups():
    return builder_groups(builder_programs(), "ew_dag")


VARIANT = {"_s0": (0, 0, "false"), "_s1": (1, 0, "false"), "_s3": (3, 0, "false"), "_s3t": (3, 2, "true"),
           "_s1o": (1, 0, "true"), "_s3o": (3, 0, "true")}
OUT_T = {"f32": "float", "f16": "__half", "bf16": "__nv_bfloat16", "bool": "uint8_t", "i32": "int32_t",
         "i64": "long long"}


def plan_of(desc):
    """(kernel name, [int args]) of the interpreted plan of one group, or None when it is not a float chain."""
    import cinn_b200
    g = cinn_b200.FusedGroup(desc)
    try:
        text = g.launch_text()
    finally:
        g.release()
    launches = [l for l in text.splitlines() if l.startswith("launch ")]
    kernel = launches[0].split()[2]
    if not re.match(r"(ew_chain_(f32|f16|bf16|bool|i32|i64)|chain_reduce_(row|col))_s", kernel):
        return None
    if kernel.startswith("ew_chain_") and len(launches) != 1:
        return None
    args = {}
    for l in text.splitlines():
        w = l.split()
        if w[0] == "launch" and w[1] != "0":
            break  # a second launch folds partials; the program lives in the first
        if w[0] == "arg" and w[2] == "int":
            args[int(w[1])] = int(w[3])
    return kernel, args


def dag_table_lines():
    import cinn_b200
    L = cinn_b200.lib()
    cinn_b200._lib.check(L.cinn_b200_set_option(b"enable_static_chains", 0))
    try:
        seen, lines, skipped = {}, [], []
        for name, desc in DAG_GROUPS + builder_dag_groups():
            cinn_b200._lib.check(L.cinn_b200_set_option(b"enable_static_chains", 0))
            try:
                g = cinn_b200.FusedGroup(desc)
            except cinn_b200.CinnB200Error as e:
                skipped.append("%s: %s" % (name, e))
                continue
            text = g.launch_text()
            g.release()
            launches = [l for l in text.splitlines() if l.startswith("launch ")]
            if len(launches) != 1 or launches[0].split()[2] != "ew_dag":
                skipped.append("%s: not a register program (%s)" % (name, launches[0].split()[2]))
                continue
            args = {int(l.split()[1]): int(l.split()[3]) for l in text.splitlines() if l.startswith("arg ") and l.split()[2] == "int"}
            meta, nsteps = args[14], args[31]
            sig = tuple(args[32 + k] & 0xffffffff for k in range(nsteps))
            if (meta, sig) in seen:
                skipped.append("%s: same program as %s" % (name, seen[(meta, sig)]))
                continue
            seen[(meta, sig)] = name
            lines.append("STATIC_DAG(%s, %d, %s);" % (name, meta, ", ".join("0x%08xu" % w for w in sig)))
        return lines, skipped
    finally:
        L.cinn_b200_set_option(b"enable_static_chains", 1)


def row_table_lines():
    import cinn_b200
    L = cinn_b200.lib()
    cinn_b200._lib.check(L.cinn_b200_set_option(b"enable_static_chains", 0))
    try:
        seen, lines, skipped = {}, [], []
        for name, desc in ROW_GROUPS + builder_groups(builder_row_programs(), "row_program"):
            cinn_b200._lib.check(L.cinn_b200_set_option(b"enable_static_chains", 0))
            try:
                g = cinn_b200.FusedGroup(desc)
            except cinn_b200.CinnB200Error as e:
                skipped.append("%s: %s" % (name, e))
                continue
            text = g.launch_text()
            g.release()
            launches = [l for l in text.splitlines() if l.startswith("launch ")]
            if len(launches) != 1 or launches[0].split()[2] != "row_program":
                skipped.append("%s: not a row program (%s)" % (name, launches[0].split()[2]))
                continue
            args = {int(l.split()[1]): int(l.split()[3]) for l in text.splitlines() if l.startswith("arg ") and l.split()[2] == "int"}
            meta, counts = args[16], args[17]
            nsteps = sum((counts >> (8 * k)) & 0xff for k in (0, 1, 2, 4, 5, 6))
            sig = tuple(args[34 + k] & 0xffffffff for k in range(nsteps))
            if (meta, counts, sig) in seen:
                skipped.append("%s: same program as %s" % (name, seen[(meta, counts, sig)]))
                continue
            seen[(meta, counts, sig)] = name
            lines.append("STATIC_ROW_PROGRAM(%s, %d, %d, %s);" % (name, meta, counts, ", ".join("0x%08xu" % w for w in sig)))
        return lines, skipped
    finally:
        L.cinn_b200_set_option(b"enable_static_chains", 1)


def table_lines(groups=None, reduce_table=False):
    import cinn_b200
    L = cinn_b200.lib()
    cinn_b200._lib.check(L.cinn_b200_set_option(b"enable_static_chains", 0))
    try:
        seen, lines, skipped = {}, [], []
        for name, desc in (GROUPS if groups is None else groups):
            try:
                got = plan_of(desc)
            except cinn_b200.CinnB200Error as e:
                skipped.append("%s: %s" % (name, e))
                continue
            if got is None:
                skipped.append("%s: not a single interpreted float chain" % name)
                continue
            kernel, args = got
            meta, nsteps = args[7], args[14]
            if reduce_table:
                m = re.match(r"chain_reduce_(row|col)(_s\w+)$", kernel)
                if not m:
                    skipped.append("%s: not a chain reduction (%s)" % (name, kernel))
                    continue
                ns, nt, _ = VARIANT[m.group(2)]
            else:
                m = re.match(r"ew_chain_(\w+?)(_s\w+)$", kernel)
                if not m:
                    skipped.append("%s: not an elementwise chain (%s)" % (name, kernel))
                    continue
                out_t, (ns, nt, st2) = OUT_T[m.group(1)], VARIANT[m.group(2)]
            sig = [args[15 + k] & 0xffffffff for k in range(nsteps)]
            if nsteps == 0:
                skipped.append("%s: empty program" % name)
                continue
            key = (kernel, meta, tuple(sig))
            if key in seen:
                skipped.append("%s: same program as %s" % (name, seen[key]))
                continue
            seen[key] = name
            sigs = ", ".join("0x%08xu" % s for s in sig)
            if reduce_table:
                lines.append('STATIC_CHAIN_REDUCE_%s(%s, "%s", %d, %d, %d, %s);' % (
                    m.group(1).upper(), name, kernel, ns, nt, meta, sigs))
            else:
                lines.append('STATIC_CHAIN(%s, "%s", %s, %d, %d, %s, %d, %s);' % (
                    name, kernel, out_t, ns, nt, st2, meta, sigs))
        return lines, skipped
    finally:
        L.cinn_b200_set_option(b"enable_static_chains", 1)


HEADER = ("// Generated by gen_static_chains.py -- do not edit.  STATIC_CHAIN(id, interpreted kernel, output type, side\n"
          "// inputs, temporaries, second output, meta word, low halves of the step words...).\n")


REDUCE_HEADER = ("// Generated by gen_static_chains.py -- do not edit.  STATIC_CHAIN_REDUCE_ROW / _COL(id, interpreted\n"
                 "// kernel, side inputs, temporaries, meta word (with the reduce op and result type), step words...).\n")


def tables():
    """[(file name, text, skipped notes)] of both generated tables."""
    lines, skipped = table_lines()
    rlines, rskipped = table_lines(REDUCE_GROUPS, reduce_table=True)
    dlines, dskipped = dag_table_lines()
    dag_header = ("// Generated by gen_static_chains.py -- do not edit.  STATIC_DAG(id, meta word, step words...).\n")
    return [("ew_static_table.inc", HEADER + "\n".join(lines) + "\n", skipped, len(lines)),
            ("chain_reduce_static_table.inc", REDUCE_HEADER + "\n".join(rlines) + "\n", rskipped, len(rlines)),
            ("ew_dag_static_table.inc", dag_header + "\n".join(dlines) + "\n", dskipped, len(dlines)),
            row_table(), int_table(), f64_table()]


def int_table():
    lines, skipped = int_table_lines()
    header = ("// Generated by gen_static_chains.py -- do not edit.  STATIC_INT_CHAIN(id, interpreted kernel, value type,\n"
              "// output type, side inputs, temporaries, meta word, step words...).\n")
    return ("ew_int_static_table.inc", header + "\n".join(lines) + "\n", skipped, len(lines))


def f64_table():
    lines, skipped = f64_table_lines()
    header = ("// Generated by gen_static_chains.py -- do not edit.  STATIC_F64_CHAIN(id, interpreted kernel, output type,\n"
              "// side inputs, temporaries, meta word, step words...).\n")
    return ("ew_f64_static_table.inc", header + "\n".join(lines) + "\n", skipped, len(lines))


def row_table():
    lines, skipped = row_table_lines()
    header = ("// Generated by gen_static_chains.py -- do not edit.  STATIC_ROW_PROGRAM(id, meta word, counts word, step\n"
              "// words...).\n")
    return ("row_prog_static_table.inc", header + "\n".join(lines) + "\n", skipped, len(lines))


def main():
    rc = 0
    for fname, text, skipped, count in tables():
        path = os.path.join(HERE, fname)
        if "--check" in sys.argv:
            ok = open(path).read() == text
            print("%s is %s" % (fname, "up to date" if ok else "OUT OF DATE"))
            rc = rc or (0 if ok else 1)
            continue
        with open(path, "w") as f:
            f.write(text)
        print("%s: %d kernels" % (fname, count))
        for s in skipped:
            print("  skipped", s)
    return rc


if __name__ == "__main__":
    sys.exit(main())
