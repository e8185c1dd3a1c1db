"""Generates tests/golden/llvm_x86_vectors.npz: outputs of LLVM-compiled loops for the benchmark groups.

Why: the parity target is CINN's x86 path, which emits LLVM IR (cinn/backends/llvm/codegen_llvm.cc) and optimises it
at -O3 without fast-math (cinn/backends/llvm/llvm_optimizer.cc:124-163).  CINN itself cannot be built offline, so
the arithmetic cannot be observed directly; what CAN be observed is how LLVM lowers the IR constructs that CINN
emits for these groups: `llvm.fmuladd.f32` (from cinn/optim/lower_intrin.cc:41-59), `llvm.exp.f32` / `llvm.sqrt.f32`
(cinn/backends/llvm/llvm_intrin_rule.h:48-63), `fcmp ogt/oge` + `select` (codegen_llvm.cc:310-340), `fptrunc` to
half (codegen_llvm.cc:454-455), serial `fadd` reductions, after the loop vectoriser has run.  This script writes that
IR by hand for each group (flat loops over the output, producers inlined, as CodeGenLLVM would), JIT-compiles it with
llvmlite (LLVM 20 here; CINN pins LLVM 11) at O3 with loop and SLP vectorisation for the host CPU, runs it on small
seeded inputs and stores inputs and outputs.  tests/test_oracle_pins.py then requires the C oracle to reproduce the
stored outputs bit for bit, which pins the oracle's contraction, rounding and libm choices against a real LLVM build.

Run: python tests/golden/make_llvm_x86_vectors.py   (needs llvmlite; not needed to run the tests)
"""
import ctypes
import os

import llvmlite.binding as llvm
import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))

IR = r"""
declare float @llvm.fmuladd.f32(float, float, float)
declare float @llvm.exp.f32(float)
declare float @llvm.sqrt.f32(float)

; relu(A + B): max(x, 0) = fcmp ogt + select
define void @add_relu(float* noalias %a, float* noalias %b, float* noalias %y, i64 %n) {
entry:
  br label %loop
loop:
  %i = phi i64 [ 0, %entry ], [ %i1, %loop ]
  %pa = getelementptr float, float* %a, i64 %i
  %pb = getelementptr float, float* %b, i64 %i
  %va = load float, float* %pa
  %vb = load float, float* %pb
  %s = fadd float %va, %vb
  %c = fcmp ogt float %s, 0.0
  %r = select i1 %c, float %s, float 0.0
  %py = getelementptr float, float* %y, i64 %i
  store float %r, float* %py
  %i1 = add i64 %i, 1
  %done = icmp eq i64 %i1, %n
  br i1 %done, label %exit, label %loop
exit:
  ret void
}

; cast_f16(tanh(fmuladd(scale, x + bias[c], shift))) with tanh = x >= 0 ? (1-e^-2x)/(1+e^-2x) : (e^2x-1)/(e^2x+1)
define void @bias_scale_tanh_f16(float* noalias %x, float* noalias %bias, half* noalias %y, i64 %rows, i64 %cols,
                                 float %scale, float %shift) {
entry:
  br label %rowloop
rowloop:
  %r = phi i64 [ 0, %entry ], [ %r1, %rowend ]
  %rowoff = mul i64 %r, %cols
  br label %colloop
colloop:
  %c = phi i64 [ 0, %rowloop ], [ %c1, %colloop ]
  %idx = add i64 %rowoff, %c
  %px = getelementptr float, float* %x, i64 %idx
  %pb = getelementptr float, float* %bias, i64 %c
  %vx = load float, float* %px
  %vb = load float, float* %pb
  %s = fadd float %vx, %vb
  %t = call float @llvm.fmuladd.f32(float %scale, float %s, float %shift)
  %m2 = fmul float -2.0, %t
  %p2 = fmul float 2.0, %t
  %en = call float @llvm.exp.f32(float %m2)
  %ep = call float @llvm.exp.f32(float %p2)
  %pn = fsub float 1.0, %en
  %pd = fadd float 1.0, %en
  %tp = fdiv float %pn, %pd
  %nn = fsub float %ep, 1.0
  %nd = fadd float %ep, 1.0
  %tn = fdiv float %nn, %nd
  %ge = fcmp oge float %t, 0.0
  %th = select i1 %ge, float %tp, float %tn
  %h = fptrunc float %th to half
  %py = getelementptr half, half* %y, i64 %idx
  store half %h, half* %py
  %c1 = add i64 %c, 1
  %cdone = icmp eq i64 %c1, %cols
  br i1 %cdone, label %rowend, label %colloop
rowend:
  %r1 = add i64 %r, 1
  %rdone = icmp eq i64 %r1, %rows
  br i1 %rdone, label %exit, label %rowloop
exit:
  ret void
}

; reduce_sum over the last axis: init 0, serial fadd in index order
define void @reduce_sum_rows(float* noalias %x, float* noalias %y, i64 %rows, i64 %cols) {
entry:
  br label %rowloop
rowloop:
  %r = phi i64 [ 0, %entry ], [ %r1, %rowend ]
  %rowoff = mul i64 %r, %cols
  br label %colloop
colloop:
  %c = phi i64 [ 0, %rowloop ], [ %c1, %colloop ]
  %acc = phi float [ 0.0, %rowloop ], [ %acc1, %colloop ]
  %idx = add i64 %rowoff, %c
  %px = getelementptr float, float* %x, i64 %idx
  %vx = load float, float* %px
  %acc1 = fadd float %acc, %vx
  %c1 = add i64 %c, 1
  %cdone = icmp eq i64 %c1, %cols
  br i1 %cdone, label %rowend, label %colloop
rowend:
  %py = getelementptr float, float* %y, i64 %r
  store float %acc1, float* %py
  %r1 = add i64 %r, 1
  %rdone = icmp eq i64 %r1, %rows
  br i1 %rdone, label %exit, label %rowloop
exit:
  ret void
}

; softmax along the last axis: s = sum exp(x) (serial), y = exp(x) / s
define void @softmax_rows(float* noalias %x, float* noalias %y, i64 %rows, i64 %cols) {
entry:
  br label %rowloop
rowloop:
  %r = phi i64 [ 0, %entry ], [ %r1, %rowend ]
  %rowoff = mul i64 %r, %cols
  br label %sumloop
sumloop:
  %c = phi i64 [ 0, %rowloop ], [ %c1, %sumloop ]
  %acc = phi float [ 0.0, %rowloop ], [ %acc1, %sumloop ]
  %idx = add i64 %rowoff, %c
  %px = getelementptr float, float* %x, i64 %idx
  %vx = load float, float* %px
  %e = call float @llvm.exp.f32(float %vx)
  %acc1 = fadd float %acc, %e
  %c1 = add i64 %c, 1
  %cdone = icmp eq i64 %c1, %cols
  br i1 %cdone, label %divloop, label %sumloop
divloop:
  %d = phi i64 [ 0, %sumloop ], [ %d1, %divloop ]
  %idx2 = add i64 %rowoff, %d
  %px2 = getelementptr float, float* %x, i64 %idx2
  %vx2 = load float, float* %px2
  %e2 = call float @llvm.exp.f32(float %vx2)
  %q = fdiv float %e2, %acc1
  %py = getelementptr float, float* %y, i64 %idx2
  store float %q, float* %py
  %d1 = add i64 %d, 1
  %ddone = icmp eq i64 %d1, %cols
  br i1 %ddone, label %rowend, label %divloop
rowend:
  %r1 = add i64 %r, 1
  %rdone = icmp eq i64 %r1, %rows
  br i1 %rdone, label %exit, label %rowloop
exit:
  ret void
}

; layer_norm: mean = s1/N, var = max(s2/N - mean*mean, 0), rstd = 1/sqrt(var+eps),
; y = fmuladd((x - mean) * rstd, gamma, beta); x*x is materialised before it is summed
define void @layernorm_rows(float* noalias %x, float* noalias %gamma, float* noalias %beta, float* noalias %y,
                            i64 %rows, i64 %cols, float %eps) {
entry:
  %nf = uitofp i64 %cols to float
  br label %rowloop
rowloop:
  %r = phi i64 [ 0, %entry ], [ %r1, %rowend ]
  %rowoff = mul i64 %r, %cols
  br label %s1loop
s1loop:
  %c = phi i64 [ 0, %rowloop ], [ %c1, %s1loop ]
  %a1 = phi float [ 0.0, %rowloop ], [ %a1n, %s1loop ]
  %idx = add i64 %rowoff, %c
  %px = getelementptr float, float* %x, i64 %idx
  %vx = load float, float* %px
  %a1n = fadd float %a1, %vx
  %c1 = add i64 %c, 1
  %cdone = icmp eq i64 %c1, %cols
  br i1 %cdone, label %s2loop, label %s1loop
s2loop:
  %k = phi i64 [ 0, %s1loop ], [ %k1, %s2loop ]
  %a2 = phi float [ 0.0, %s1loop ], [ %a2n, %s2loop ]
  %idxk = add i64 %rowoff, %k
  %pxk = getelementptr float, float* %x, i64 %idxk
  %vxk = load float, float* %pxk
  %sq = fmul float %vxk, %vxk
  %a2n = fadd float %a2, %sq
  %k1 = add i64 %k, 1
  %kdone = icmp eq i64 %k1, %cols
  br i1 %kdone, label %stats, label %s2loop
stats:
  %mean = fdiv float %a1n, %nf
  %m2 = fdiv float %a2n, %nf
  %mm = fmul float %mean, %mean
  %dv = fsub float %m2, %mm
  %gt = fcmp ogt float %dv, 0.0
  %var = select i1 %gt, float %dv, float 0.0
  %ve = fadd float %var, %eps
  %sr = call float @llvm.sqrt.f32(float %ve)
  %rstd = fdiv float 1.0, %sr
  br label %outloop
outloop:
  %d = phi i64 [ 0, %stats ], [ %d1, %outloop ]
  %idxd = add i64 %rowoff, %d
  %pxd = getelementptr float, float* %x, i64 %idxd
  %vxd = load float, float* %pxd
  %pg = getelementptr float, float* %gamma, i64 %d
  %pbt = getelementptr float, float* %beta, i64 %d
  %vg = load float, float* %pg
  %vbt = load float, float* %pbt
  %xc = fsub float %vxd, %mean
  %xn = fmul float %xc, %rstd
  %yv = call float @llvm.fmuladd.f32(float %xn, float %vg, float %vbt)
  %py = getelementptr float, float* %y, i64 %idxd
  store float %yv, float* %py
  %d1 = add i64 %d, 1
  %ddone = icmp eq i64 %d1, %cols
  br i1 %ddone, label %rowend, label %outloop
rowend:
  %r1 = add i64 %r, 1
  %rdone = icmp eq i64 %r1, %rows
  br i1 %rdone, label %exit, label %rowloop
exit:
  ret void
}

; relu(batch_norm): max(((x - mean[c]) * scale[c]) / sqrt(var[c] + eps) + bias[c], 0) over [planes, hw]
define void @bn_relu(float* noalias %x, float* noalias %scale, float* noalias %bias, float* noalias %mean,
                     float* noalias %var, float* noalias %y, i64 %planes, i64 %channels, i64 %hw, float %eps) {
entry:
  br label %planeloop
planeloop:
  %p = phi i64 [ 0, %entry ], [ %p1, %planeend ]
  %ch = urem i64 %p, %channels
  %off = mul i64 %p, %hw
  %pm = getelementptr float, float* %mean, i64 %ch
  %ps = getelementptr float, float* %scale, i64 %ch
  %pb = getelementptr float, float* %bias, i64 %ch
  %pv = getelementptr float, float* %var, i64 %ch
  br label %inner
inner:
  %i = phi i64 [ 0, %planeloop ], [ %i1, %inner ]
  %idx = add i64 %off, %i
  %px = getelementptr float, float* %x, i64 %idx
  %vx = load float, float* %px
  %vm = load float, float* %pm
  %vs = load float, float* %ps
  %vb = load float, float* %pb
  %vv = load float, float* %pv
  %t1 = fsub float %vx, %vm
  %t2 = fmul float %t1, %vs
  %ve = fadd float %vv, %eps
  %sd = call float @llvm.sqrt.f32(float %ve)
  %t3 = fdiv float %t2, %sd
  %t4 = fadd float %t3, %vb
  %c = fcmp ogt float %t4, 0.0
  %r = select i1 %c, float %t4, float 0.0
  %py = getelementptr float, float* %y, i64 %idx
  store float %r, float* %py
  %i1 = add i64 %i, 1
  %idone = icmp eq i64 %i1, %hw
  br i1 %idone, label %planeend, label %inner
planeend:
  %p1 = add i64 %p, 1
  %pdone = icmp eq i64 %p1, %planes
  br i1 %pdone, label %exit, label %planeloop
exit:
  ret void
}
"""


def compile_ir():
    llvm.initialize_native_target()
    llvm.initialize_native_asmprinter()
    try:
        llvm.load_library_permanently("libm.so.6")
    except Exception:
        pass
    mod = llvm.parse_assembly(IR)
    mod.verify()
    target = llvm.Target.from_default_triple()
    tm = target.create_target_machine(cpu=llvm.get_host_cpu_name(), features=llvm.get_host_cpu_features().flatten(),
                                      opt=3)
    # O3 with loop and SLP vectorisation, no fast-math flags anywhere in the IR (as llvm_optimizer.cc:124-163)
    try:  # new pass manager (llvmlite >= 0.44)
        pto = llvm.create_pipeline_tuning_options(speed_level=3, size_level=0)
        pto.loop_vectorization = True
        pto.slp_vectorization = True
        pto.loop_unrolling = True
        pb = llvm.create_pass_builder(tm, pto)
        pb.getModulePassManager().run(mod, pb)
    except AttributeError:  # legacy pass manager
        pmb = llvm.create_pass_manager_builder()
        pmb.opt_level = 3
        pmb.loop_vectorize = True
        pmb.slp_vectorize = True
        pm = llvm.create_module_pass_manager()
        pmb.populate(pm)
        pm.run(mod)
    engine = llvm.create_mcjit_compiler(mod, tm)
    engine.finalize_object()
    return engine, str(mod)


def main():
    engine, optimised_ir = compile_ir()
    vp, i64, f32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_float
    fn = lambda name, *argtypes: ctypes.CFUNCTYPE(None, *argtypes)(engine.get_function_address(name))  # noqa: E731
    p = lambda a: a.ctypes.data_as(vp)  # noqa: E731
    rng = np.random.default_rng(2024)
    out = {}

    a = rng.uniform(-1, 1, 4099).astype(np.float32)
    b = rng.uniform(-1, 1, 4099).astype(np.float32)
    y = np.empty_like(a)
    fn("add_relu", vp, vp, vp, i64)(p(a), p(b), p(y), a.size)
    out.update(add_relu_a=a, add_relu_b=b, add_relu_y=y)

    x = (rng.standard_normal((37, 1000)) * 1.5).astype(np.float32)
    x[0, :8] = [0.0, -0.0, 1e-7, -1e-7, 30.0, -30.0, 1e-3, -1e-3]
    bias = (0.1 * rng.standard_normal(1000)).astype(np.float32)
    yh = np.empty(x.shape, np.float16)
    fn("bias_scale_tanh_f16", vp, vp, vp, i64, i64, f32, f32)(p(x), p(bias), p(yh), 37, 1000, 0.5, 0.0)
    out.update(tanh_x=x, tanh_bias=bias, tanh_y=yh)

    x = rng.standard_normal((29, 1031)).astype(np.float32)
    ys = np.empty(29, np.float32)
    fn("reduce_sum_rows", vp, vp, i64, i64)(p(x), p(ys), 29, 1031)
    out.update(sum_x=x, sum_y=ys)

    x = rng.standard_normal((23, 517)).astype(np.float32)
    y = np.empty_like(x)
    fn("softmax_rows", vp, vp, i64, i64)(p(x), p(y), 23, 517)
    out.update(softmax_x=x, softmax_y=y)

    x = rng.standard_normal((19, 777)).astype(np.float32)
    gamma = (1 + 0.02 * rng.standard_normal(777)).astype(np.float32)
    beta = (0.02 * rng.standard_normal(777)).astype(np.float32)
    y = np.empty_like(x)
    fn("layernorm_rows", vp, vp, vp, vp, i64, i64, f32)(p(x), p(gamma), p(beta), p(y), 19, 777, 1e-5)
    out.update(ln_x=x, ln_gamma=gamma, ln_beta=beta, ln_y=y)

    x = rng.standard_normal((3, 5, 11, 13)).astype(np.float32)
    mean = (0.1 * rng.standard_normal(5)).astype(np.float32)
    var = rng.uniform(0.5, 1.5, 5).astype(np.float32)
    scale = (1 + 0.1 * rng.standard_normal(5)).astype(np.float32)
    bb = (0.1 * rng.standard_normal(5)).astype(np.float32)
    y = np.empty_like(x)
    fn("bn_relu", vp, vp, vp, vp, vp, vp, i64, i64, i64, f32)(p(x), p(scale), p(bb), p(mean), p(var), p(y), 15, 5, 143,
                                                              1e-5)
    out.update(bn_x=x, bn_scale=scale, bn_bias=bb, bn_mean=mean, bn_var=var, bn_y=y)

    np.savez_compressed(os.path.join(HERE, "llvm_x86_vectors.npz"), **out)
    vectorised = "<8 x float>" in optimised_ir or "<16 x float>" in optimised_ir or "<4 x float>" in optimised_ir
    print("wrote llvm_x86_vectors.npz; LLVM %s, host cpu %s, loops vectorised: %s, fmuladd kept as intrinsic/fma: %s"
          % (".".join(map(str, llvm.llvm_version_info)), llvm.get_host_cpu_name(), vectorised,
             "fmuladd" in optimised_ir or "llvm.fma" in optimised_ir))


if __name__ == "__main__":
    main()
