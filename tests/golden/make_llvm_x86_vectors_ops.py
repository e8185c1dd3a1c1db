"""Generates tests/golden/llvm_x86_vectors_ops.npz: every unary and binary elementwise op of the registry, in float32 and
float64, as LLVM compiles the IR that CINN's x86 path emits for it, plus the integer ops of the int32 chains.

The two sibling scripts pin the benchmark groups and the decomposed groups; this one pins the op table itself.  For each
op a flat loop is written in LLVM IR the way CodeGenLLVM lowers the op (cinn/backends/llvm/llvm_intrin_rule.h:48-175:
exp / log / sqrt / floor / ceil / trunc / nearbyint / sin / cos / log2 / log10 / fabs / pow as llvm.* intrinsics; tanh
as the two-branch exp formula; rsqrt as 1 / sqrt; tan as sin / cos; sinh / cosh from two exps; erf, asin ... atanh as
calls of the host's libm (cinn/optim/map_extern_call.cc:42-74); cbrt through double (cinn/runtime/cpu/
host_intrinsics.cc:216); sigmoid as 1 / (1 + exp(-x)) (cinn/lang/builtin.h:79-82); max / min / relu as fcmp + select
(cinn/backends/llvm/codegen_llvm.cc:310-340); comparisons and logical ops yielding 0 / 1), compiled with llvmlite at O3
with the loop and SLP vectorisers and no fast-math flag, and run on seeded inputs that include zeros, signed zeros,
infinities, NaN, denormals and values at the functions' domain edges.  tests/test_oracle_pins.py requires the C oracle
(float32, float64) and the graph evaluator (int32) to reproduce every stored output bit for bit.

Float `mod` is left out: the reference's x86 path has no host symbol for it (the oracle documents that it follows the
reference's GPU runtime there).

Run: python tests/golden/make_llvm_x86_vectors_ops.py   (needs llvmlite; not needed to run the tests)
"""
import ctypes
import os

import llvmlite.binding as llvm
import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

# body templates: %v (and %w) are the loaded operands, the result must be named %r.  {T} float|double, {S} f32|f64,
# {f} the libm suffix ("f" or ""), {PI} / {HPI} / {NHPI} pi, pi / 2 and -pi / 2 rounded to the type.
UNARY = {
    "exp": "%r = call {T} @llvm.exp.{S}({T} %v)",
    "log": "%r = call {T} @llvm.log.{S}({T} %v)",
    "sqrt": "%r = call {T} @llvm.sqrt.{S}({T} %v)",
    "floor": "%r = call {T} @llvm.floor.{S}({T} %v)",
    "ceil": "%r = call {T} @llvm.ceil.{S}({T} %v)",
    "trunc": "%r = call {T} @llvm.trunc.{S}({T} %v)",
    "round": "%r = call {T} @llvm.nearbyint.{S}({T} %v)",
    "sin": "%r = call {T} @llvm.sin.{S}({T} %v)",
    "cos": "%r = call {T} @llvm.cos.{S}({T} %v)",
    "log2": "%r = call {T} @llvm.log2.{S}({T} %v)",
    "log10": "%r = call {T} @llvm.log10.{S}({T} %v)",
    "abs": "%r = call {T} @llvm.fabs.{S}({T} %v)",
    "negative": "%r = fneg {T} %v",
    "identity": "%r = fadd {T} %v, -0.0",
    "reciprocal": "%r = fdiv {T} 1.0, %v",
    "rsqrt": "%s = call {T} @llvm.sqrt.{S}({T} %v)\n  %r = fdiv {T} 1.0, %s",
    "sigmoid": "%n = fneg {T} %v\n  %e = call {T} @llvm.exp.{S}({T} %n)\n  %d = fadd {T} 1.0, %e\n  %r = fdiv {T} 1.0, %d",
    "tanh": ("%m2 = fmul {T} -2.0, %v\n  %p2 = fmul {T} 2.0, %v\n  %en = call {T} @llvm.exp.{S}({T} %m2)\n"
             "  %ep = call {T} @llvm.exp.{S}({T} %p2)\n  %pn = fsub {T} 1.0, %en\n  %pd = fadd {T} 1.0, %en\n"
             "  %tp = fdiv {T} %pn, %pd\n  %nn = fsub {T} %ep, 1.0\n  %nd = fadd {T} %ep, 1.0\n  %tn = fdiv {T} %nn, %nd\n"
             "  %ge = fcmp oge {T} %v, 0.0\n  %r = select i1 %ge, {T} %tp, {T} %tn"),
    "relu": "%c = fcmp ogt {T} %v, 0.0\n  %r = select i1 %c, {T} %v, {T} 0.0",
    "sign": ("%lt = fcmp olt {T} %v, 0.0\n  %gt = fcmp ogt {T} %v, 0.0\n  %eq = fcmp oeq {T} %v, 0.0\n"
             "  %z = select i1 %eq, {T} 0.0, {T} %v\n  %p = select i1 %gt, {T} 1.0, {T} %z\n  %r = select i1 %lt, {T} -1.0, {T} %p"),
    "tan": "%s = call {T} @llvm.sin.{S}({T} %v)\n  %c = call {T} @llvm.cos.{S}({T} %v)\n  %r = fdiv {T} %s, %c",
    "sinh": ("%n = fmul {T} %v, -1.0\n  %a = call {T} @llvm.exp.{S}({T} %v)\n  %b = call {T} @llvm.exp.{S}({T} %n)\n"
             "  %d = fsub {T} %a, %b\n  %r = fdiv {T} %d, 2.0"),
    "cosh": ("%n = fmul {T} %v, -1.0\n  %a = call {T} @llvm.exp.{S}({T} %v)\n  %b = call {T} @llvm.exp.{S}({T} %n)\n"
             "  %d = fadd {T} %a, %b\n  %r = fdiv {T} %d, 2.0"),
    "erf": "%r = call {T} @erf{f}({T} %v)",
    "asin": "%r = call {T} @asin{f}({T} %v)",
    "acos": "%r = call {T} @acos{f}({T} %v)",
    "atan": "%r = call {T} @atan{f}({T} %v)",
    "asinh": "%r = call {T} @asinh{f}({T} %v)",
    "acosh": "%r = call {T} @acosh{f}({T} %v)",
    "atanh": "%r = call {T} @atanh{f}({T} %v)",
    "cbrt": "%r = call {T} @cbrt_as_the_host_does({T} %v)",
    "isnan": "%c = fcmp uno {T} %v, %v\n  %r = uitofp i1 %c to {T}",
    "isinf": ("%a = call {T} @llvm.fabs.{S}({T} %v)\n  %c = fcmp oeq {T} %a, 0x7FF0000000000000\n  %r = uitofp i1 %c to {T}"),
    "isfinite": ("%a = call {T} @llvm.fabs.{S}({T} %v)\n  %c = fcmp one {T} %a, 0x7FF0000000000000\n  %r = uitofp i1 %c to {T}"),
    "logical_not": "%c = fcmp oeq {T} %v, 0.0\n  %r = uitofp i1 %c to {T}",
}
BINARY = {
    "add": "%r = fadd {T} %v, %w",
    "subtract": "%r = fsub {T} %v, %w",
    "multiply": "%r = fmul {T} %v, %w",
    "divide": "%r = fdiv {T} %v, %w",
    "max": "%c = fcmp ogt {T} %v, %w\n  %r = select i1 %c, {T} %v, {T} %w",
    "min": "%c = fcmp olt {T} %v, %w\n  %r = select i1 %c, {T} %v, {T} %w",
    "pow": "%r = call {T} @llvm.pow.{S}({T} %v, {T} %w)",
    "equal": "%c = fcmp oeq {T} %v, %w\n  %r = uitofp i1 %c to {T}",
    "not_equal": "%c = fcmp une {T} %v, %w\n  %r = uitofp i1 %c to {T}",
    "greater_than": "%c = fcmp ogt {T} %v, %w\n  %r = uitofp i1 %c to {T}",
    "less_than": "%c = fcmp olt {T} %v, %w\n  %r = uitofp i1 %c to {T}",
    "greater_equal": "%c = fcmp oge {T} %v, %w\n  %r = uitofp i1 %c to {T}",
    "less_equal": "%c = fcmp ole {T} %v, %w\n  %r = uitofp i1 %c to {T}",
    "floor_divide": "%q = fdiv {T} %v, %w\n  %r = call {T} @llvm.floor.{S}({T} %q)",
    "atan2": ("%q = fdiv {T} %v, %w\n  %at = call {T} @atan{f}({T} %q)\n  %bz = fcmp oeq {T} %w, 0.0\n"
              "  %az = fcmp oeq {T} %v, 0.0\n  %ap = fcmp ogt {T} %v, 0.0\n  %hp = select i1 %ap, {T} {HPI}, {T} {NHPI}\n"
              "  %zero = select i1 %az, {T} 0.0, {T} %hp\n  %bp = fcmp ogt {T} %w, 0.0\n  %age = fcmp oge {T} %v, 0.0\n"
              "  %plus = fadd {T} %at, {PI}\n  %minus = fsub {T} %at, {PI}\n  %other = select i1 %age, {T} %plus, {T} %minus\n"
              "  %nz = select i1 %bp, {T} %at, {T} %other\n  %r = select i1 %bz, {T} %zero, {T} %nz"),
    "logical_and": "%a = fcmp une {T} %v, 0.0\n  %b = fcmp une {T} %w, 0.0\n  %c = and i1 %a, %b\n  %r = uitofp i1 %c to {T}",
    "logical_or": "%a = fcmp une {T} %v, 0.0\n  %b = fcmp une {T} %w, 0.0\n  %c = or i1 %a, %b\n  %r = uitofp i1 %c to {T}",
    "logical_xor": "%a = fcmp une {T} %v, 0.0\n  %b = fcmp une {T} %w, 0.0\n  %c = xor i1 %a, %b\n  %r = uitofp i1 %c to {T}",
}
INT_BINARY = {
    "elementwise_add": "%r = add i32 %v, %w", "subtract": "%r = sub i32 %v, %w", "elementwise_mul": "%r = mul i32 %v, %w",
    "max": "%c = icmp sgt i32 %v, %w\n  %r = select i1 %c, i32 %v, i32 %w",
    "min": "%c = icmp slt i32 %v, %w\n  %r = select i1 %c, i32 %v, i32 %w",
    "bitwise_and": "%r = and i32 %v, %w", "bitwise_or": "%r = or i32 %v, %w", "bitwise_xor": "%r = xor i32 %v, %w",
}


def loop(name, ty, body, binary):
    args = f"{ty}* noalias %x, " + (f"{ty}* noalias %z, " if binary else "") + f"{ty}* noalias %y, i64 %count"
    load_w = f"  %pw = getelementptr {ty}, {ty}* %z, i64 %i\n  %w = load {ty}, {ty}* %pw\n" if binary else ""
    return (f"define void @{name}({args}) {{\nentry:\n  br label %loop\nloop:\n"
            f"  %i = phi i64 [ 0, %entry ], [ %i1, %loop ]\n  %pv = getelementptr {ty}, {ty}* %x, i64 %i\n"
            f"  %v = load {ty}, {ty}* %pv\n{load_w}  {body}\n  %py = getelementptr {ty}, {ty}* %y, i64 %i\n"
            f"  store {ty} %r, {ty}* %py\n  %i1 = add i64 %i, 1\n  %done = icmp eq i64 %i1, %count\n"
            f"  br i1 %done, label %exit, label %loop\nexit:\n  ret void\n}}\n")


def module_ir():
    parts = []
    for S, T in (("f32", "float"), ("f64", "double")):
        for fn in ("exp", "log", "sqrt", "floor", "ceil", "trunc", "nearbyint", "sin", "cos", "log2", "log10", "fabs"):
            parts.append(f"declare {T} @llvm.{fn}.{S}({T})")
        parts.append(f"declare {T} @llvm.pow.{S}({T}, {T})")
    for fn in ("erf", "asin", "acos", "atan", "asinh", "acosh", "atanh"):
        parts.append(f"declare float @{fn}f(float)\ndeclare double @{fn}(double)")
    parts.append("declare double @cbrt(double)")
    # cbrt: the host intrinsic promotes to double and rounds once
    parts.append("define float @cbrt_as_the_host_does_f32(float %v) {\n  %d = fpext float %v to double\n"
                 "  %c = call double @cbrt(double %d)\n  %r = fptrunc double %c to float\n  ret float %r\n}")
    parts.append("define double @cbrt_as_the_host_does_f64(double %v) {\n  %r = call double @cbrt(double %v)\n  ret double %r\n}")
    for S, T, f, pi, hpi, nhpi in (("f32", "float", "f", "0x400921FB60000000", "0x3FF921FB60000000", "0xBFF921FB60000000"),
                                   ("f64", "double", "", "0x400921FB54442D18", "0x3FF921FB54442D18", "0xBFF921FB54442D18")):
        def fill(body):
            return (body.replace("@cbrt_as_the_host_does", "@cbrt_as_the_host_does_" + S).replace("{T}", T)
                    .replace("{S}", S).replace("{f}", f).replace("{PI}", pi).replace("{NHPI}", nhpi).replace("{HPI}", hpi))
        for op, body in UNARY.items():
            parts.append(loop(f"u_{op}_{S}", T, fill(body), False))
        for op, body in BINARY.items():
            parts.append(loop(f"b_{op}_{S}", T, fill(body), True))
    for op, body in INT_BINARY.items():
        parts.append(loop(f"i_{op}_i32", "i32", body, True))
    return "\n".join(parts)


def compile_ir(ir):
    llvm.initialize_native_target()
    llvm.initialize_native_asmprinter()
    llvm.load_library_permanently("libm.so.6")
    mod = llvm.parse_assembly(ir)
    mod.verify()
    target = llvm.Target.from_default_triple()
    tm = target.create_target_machine(cpu=llvm.get_host_cpu_name(), features=llvm.get_host_cpu_features().flatten(), opt=3)
    pto = llvm.create_pipeline_tuning_options(speed_level=3, size_level=0)
    pto.loop_vectorization = True
    pto.slp_vectorization = True
    pto.loop_unrolling = True
    pb = llvm.create_pass_builder(tm, pto)
    pb.getModulePassManager().run(mod, pb)
    engine = llvm.create_mcjit_compiler(mod, tm)
    engine.finalize_object()
    return engine


def inputs(rng, dtype, n=1537):
    """Seeded values with the special cases in front: zeros, infinities, NaN, denormals, domain edges."""
    tiny = np.finfo(dtype).tiny
    special = np.array([0.0, -0.0, 1.0, -1.0, 0.5, -0.5, 2.0, -2.0, np.inf, -np.inf, np.nan, tiny / 4, -tiny / 4,
                        1e-7, -1e-7, 30.0, -30.0, 88.0, -88.0, 0.99999, -0.99999, 1.00001, 100.5, -100.5, 2.5, -2.5,
                        3.5, -3.5, 1e30, -1e30], dtype)
    body = np.concatenate([rng.standard_normal(n // 2) * 2.0, rng.uniform(-1, 1, n - n // 2)]).astype(dtype)
    return np.concatenate([special, body])


def main():
    engine = compile_ir(module_ir())
    vp, i64 = ctypes.c_void_p, ctypes.c_int64
    p = lambda a: a.ctypes.data_as(vp)  # noqa: E731
    rng = np.random.default_rng(4242)
    out = {}
    with np.errstate(all="ignore"):
        for S, dt in (("f32", np.float32), ("f64", np.float64)):
            x = inputs(rng, dt)
            w = np.roll(inputs(rng, dt), 7)  # the special values meet one another and ordinary ones
            out[f"x_{S}"], out[f"w_{S}"] = x, w
            for op in UNARY:
                y = np.empty_like(x)
                ctypes.CFUNCTYPE(None, vp, vp, i64)(engine.get_function_address(f"u_{op}_{S}"))(p(x), p(y), x.size)
                out[f"u_{op}_{S}"] = y
            for op in BINARY:
                y = np.empty_like(x)
                ctypes.CFUNCTYPE(None, vp, vp, vp, i64)(engine.get_function_address(f"b_{op}_{S}"))(p(x), p(w), p(y), x.size)
                out[f"b_{op}_{S}"] = y
        xi = rng.integers(-2**31, 2**31 - 1, 1031, dtype=np.int64).astype(np.int32)
        wi = rng.integers(-50000, 50000, 1031, dtype=np.int64).astype(np.int32)
        xi[:4] = [2**31 - 1, -2**31, 0, -1]
        out["x_i32"], out["w_i32"] = xi, wi
        for op in INT_BINARY:
            y = np.empty_like(xi)
            ctypes.CFUNCTYPE(None, vp, vp, vp, i64)(engine.get_function_address(f"i_{op}_i32"))(p(xi), p(wi), p(y), xi.size)
            out[f"i_{op}_i32"] = y
    np.savez_compressed(os.path.join(HERE, "llvm_x86_vectors_ops.npz"), **out)
    print("wrote %d arrays" % len(out))


if __name__ == "__main__":
    main()
