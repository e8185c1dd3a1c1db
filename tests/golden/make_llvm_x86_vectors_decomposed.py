"""Generates tests/golden/llvm_x86_vectors_decomposed.npz: LLVM-compiled loops for the DECOMPOSED groups.

Companion of make_llvm_x86_vectors.py (same method, same reasons; read its header).  The groups here are the ones the
reference's decomposers produce (cinn/frontend/decomposer/batch_norm.cc, activation.cc) after inlining, written by
hand as the flat loops CodeGenLLVM would emit:

  bn_train_apply  y = fmuladd((x - mean) * (1 / sqrt(var + eps)), scale, bias)         one Add fed by a Mul
  bn_grad_apply   dx = t0 * ((dy * nhw - db) - ((x - mean) * S) / vae)                 no Add: nothing contracts
  softmax_safe    max by fcmp ogt + select from -FLT_MAX, exp(x - max), serial sum, true division
  gelu            x * fmuladd(0.5, erf(x * sqrt(0.5)), 0.5)                            erf is the host's erff

tests/test_oracle_pins.py requires oracle/x86_graph_eval.py, fed the same groups as text, to reproduce the bits.

Run: python tests/golden/make_llvm_x86_vectors_decomposed.py   (needs llvmlite; not needed to run the tests)
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
declare float @erff(float)

; x: [planes, hw], channel = plane % channels
define void @bn_train_apply(float* noalias %x, float* noalias %mean, float* noalias %var, float* noalias %scale,
                            float* noalias %bias, float* noalias %y, i64 %planes, i64 %channels, i64 %hw, float %eps) {
entry:
  br label %ploop
ploop:
  %p = phi i64 [ 0, %entry ], [ %p1, %pend ]
  %c = urem i64 %p, %channels
  %off = mul i64 %p, %hw
  %pm = getelementptr float, float* %mean, i64 %c
  %pv = getelementptr float, float* %var, i64 %c
  %ps = getelementptr float, float* %scale, i64 %c
  %pb = getelementptr float, float* %bias, i64 %c
  br label %iloop
iloop:
  %i = phi i64 [ 0, %ploop ], [ %i1, %iloop ]
  %idx = add i64 %off, %i
  %px = getelementptr float, float* %x, i64 %idx
  %vx = load float, float* %px
  %vm = load float, float* %pm
  %vv = load float, float* %pv
  %vs = load float, float* %ps
  %vb = load float, float* %pb
  %ve = fadd float %vv, %eps
  %sq = call float @llvm.sqrt.f32(float %ve)
  %inv = fdiv float 1.0, %sq
  %d = fsub float %vx, %vm
  %n = fmul float %d, %inv
  %r = call float @llvm.fmuladd.f32(float %n, float %vs, float %vb)
  %py = getelementptr float, float* %y, i64 %idx
  store float %r, float* %py
  %i1 = add i64 %i, 1
  %idone = icmp eq i64 %i1, %hw
  br i1 %idone, label %pend, label %iloop
pend:
  %p1 = add i64 %p, 1
  %pdone = icmp eq i64 %p1, %planes
  br i1 %pdone, label %exit, label %ploop
exit:
  ret void
}

define void @bn_grad_apply(float* noalias %x, float* noalias %dy, float* noalias %t0, float* noalias %db,
                           float* noalias %mean, float* noalias %s, float* noalias %vae, float* noalias %y,
                           i64 %planes, i64 %channels, i64 %hw, float %count) {
entry:
  br label %ploop
ploop:
  %p = phi i64 [ 0, %entry ], [ %p1, %pend ]
  %c = urem i64 %p, %channels
  %off = mul i64 %p, %hw
  %pt = getelementptr float, float* %t0, i64 %c
  %pd = getelementptr float, float* %db, i64 %c
  %pm = getelementptr float, float* %mean, i64 %c
  %ps = getelementptr float, float* %s, i64 %c
  %pv = getelementptr float, float* %vae, i64 %c
  br label %iloop
iloop:
  %i = phi i64 [ 0, %ploop ], [ %i1, %iloop ]
  %idx = add i64 %off, %i
  %px = getelementptr float, float* %x, i64 %idx
  %pdy = getelementptr float, float* %dy, i64 %idx
  %vx = load float, float* %px
  %vdy = load float, float* %pdy
  %vt = load float, float* %pt
  %vd = load float, float* %pd
  %vm = load float, float* %pm
  %vs = load float, float* %ps
  %vv = load float, float* %pv
  %t1 = fmul float %vdy, %count
  %a = fsub float %t1, %vd
  %xm = fsub float %vx, %vm
  %t30 = fmul float %xm, %vs
  %t3 = fdiv float %t30, %vv
  %b = fsub float %a, %t3
  %r = fmul float %vt, %b
  %py = getelementptr float, float* %y, i64 %idx
  store float %r, float* %py
  %i1 = add i64 %i, 1
  %idone = icmp eq i64 %i1, %hw
  br i1 %idone, label %pend, label %iloop
pend:
  %p1 = add i64 %p, 1
  %pdone = icmp eq i64 %p1, %planes
  br i1 %pdone, label %exit, label %ploop
exit:
  ret void
}

; three serial loops per row: max, sum of exp(x - max), exp(x - max) / sum
define void @softmax_safe_rows(float* noalias %x, float* noalias %y, i64 %rows, i64 %cols) {
entry:
  br label %rowloop
rowloop:
  %r = phi i64 [ 0, %entry ], [ %r1, %rowend ]
  %rowoff = mul i64 %r, %cols
  br label %maxloop
maxloop:
  %c = phi i64 [ 0, %rowloop ], [ %c1, %maxloop ]
  %mx = phi float [ 0xC7EFFFFFE0000000, %rowloop ], [ %mx1, %maxloop ]
  %idx = add i64 %rowoff, %c
  %px = getelementptr float, float* %x, i64 %idx
  %vx = load float, float* %px
  %gt = fcmp ogt float %mx, %vx
  %mx1 = select i1 %gt, float %mx, float %vx
  %c1 = add i64 %c, 1
  %cdone = icmp eq i64 %c1, %cols
  br i1 %cdone, label %sumpre, label %maxloop
sumpre:
  br label %sumloop
sumloop:
  %k = phi i64 [ 0, %sumpre ], [ %k1, %sumloop ]
  %acc = phi float [ 0.0, %sumpre ], [ %acc1, %sumloop ]
  %kidx = add i64 %rowoff, %k
  %pk = getelementptr float, float* %x, i64 %kidx
  %vk = load float, float* %pk
  %dk = fsub float %vk, %mx1
  %ek = call float @llvm.exp.f32(float %dk)
  %acc1 = fadd float %acc, %ek
  %k1 = add i64 %k, 1
  %kdone = icmp eq i64 %k1, %cols
  br i1 %kdone, label %outpre, label %sumloop
outpre:
  br label %outloop
outloop:
  %j = phi i64 [ 0, %outpre ], [ %j1, %outloop ]
  %jidx = add i64 %rowoff, %j
  %pj = getelementptr float, float* %x, i64 %jidx
  %vj = load float, float* %pj
  %dj = fsub float %vj, %mx1
  %ej = call float @llvm.exp.f32(float %dj)
  %q = fdiv float %ej, %acc1
  %py = getelementptr float, float* %y, i64 %jidx
  store float %q, float* %py
  %j1 = add i64 %j, 1
  %jdone = icmp eq i64 %j1, %cols
  br i1 %jdone, label %rowend, label %outloop
rowend:
  %r1 = add i64 %r, 1
  %rdone = icmp eq i64 %r1, %rows
  br i1 %rdone, label %exit, label %rowloop
exit:
  ret void
}

define void @gelu(float* noalias %x, float* noalias %y, i64 %n, float %p7) {
entry:
  br label %loop
loop:
  %i = phi i64 [ 0, %entry ], [ %i1, %loop ]
  %px = getelementptr float, float* %x, i64 %i
  %vx = load float, float* %px
  %s = fmul float %vx, %p7
  %e = call float @erff(float %s)
  %cdf = call float @llvm.fmuladd.f32(float 0.5, float %e, float 0.5)
  %r = fmul float %vx, %cdf
  %py = getelementptr float, float* %y, i64 %i
  store float %r, float* %py
  %i1 = add i64 %i, 1
  %done = icmp eq i64 %i1, %n
  br i1 %done, label %exit, label %loop
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
    rng = np.random.default_rng(2025)
    out = {}

    shape, c = (3, 5, 11, 13), 5
    x = rng.standard_normal(shape).astype(np.float32)
    mean = (0.1 * rng.standard_normal(c)).astype(np.float32)
    var = rng.uniform(0.5, 1.5, c).astype(np.float32)
    scale = (1 + 0.1 * rng.standard_normal(c)).astype(np.float32)
    bias = (0.1 * rng.standard_normal(c)).astype(np.float32)
    y = np.empty_like(x)
    fn("bn_train_apply", vp, vp, vp, vp, vp, vp, i64, i64, i64, f32)(p(x), p(mean), p(var), p(scale), p(bias), p(y), 15,
                                                                      c, 143, 1e-5)
    out.update(bnt_x=x, bnt_mean=mean, bnt_var=var, bnt_scale=scale, bnt_bias=bias, bnt_y=y)

    dy = rng.standard_normal(shape).astype(np.float32)
    t0 = rng.uniform(0.001, 0.01, c).astype(np.float32)
    db = rng.standard_normal(c).astype(np.float32)
    s = rng.standard_normal(c).astype(np.float32)
    vae = rng.uniform(0.5, 1.5, c).astype(np.float32)
    y = np.empty_like(x)
    fn("bn_grad_apply", vp, vp, vp, vp, vp, vp, vp, vp, i64, i64, i64, f32)(p(x), p(dy), p(t0), p(db), p(mean), p(s),
                                                                            p(vae), p(y), 15, c, 143, float(3 * 143))
    out.update(bng_x=x, bng_dy=dy, bng_t0=t0, bng_db=db, bng_mean=mean, bng_s=s, bng_vae=vae, bng_y=y)

    xs = (rng.standard_normal((23, 517)) * 3).astype(np.float32)
    ys = np.empty_like(xs)
    fn("softmax_safe_rows", vp, vp, i64, i64)(p(xs), p(ys), 23, 517)
    out.update(sms_x=xs, sms_y=ys)

    xg = (rng.standard_normal(4099) * 2).astype(np.float32)
    yg = np.empty_like(xg)
    fn("gelu", vp, vp, i64, f32)(p(xg), p(yg), xg.size, float(np.float32(np.sqrt(0.5))))
    out.update(gelu_x=xg, gelu_y=yg)

    np.savez_compressed(os.path.join(HERE, "llvm_x86_vectors_decomposed.npz"), **out)
    vectorised = any(t in optimised_ir for t in ("<8 x float>", "<16 x float>", "<4 x float>"))
    print("wrote llvm_x86_vectors_decomposed.npz; LLVM %s, host cpu %s, loops vectorised: %s"
          % (".".join(map(str, llvm.llvm_version_info)), llvm.get_host_cpu_name(), vectorised))


if __name__ == "__main__":
    main()
