"""MLIR modules of the shape the private rustc backend hands to a CodegenTarget.

The softmax, matmul-f16, matmul-f32, attention, GQA and matmul-transposed
modules restate the reference's own parser/emitter fixtures
(crates/tile_spec/tests/cucumber.rs:161-204,
crates/rustc_codegen_tile/src/mlir_to_linalg.rs:1941-1955, :2088-2102,
crates/rustc_codegen_tile/src/mlir_to_gpu.rs:2939-2955, :2974-2992) with other
kernel names and shapes; the bf16, causal-chain and generic-form modules are
this project's additions.  The rms_norm, reduce_sum / reduce_max and silu modules
restate crates/rustc_codegen_tile/src/mlir_to_linalg.rs:2629-2641, :2030-2056 and
:2143-2155; silu followed by mul is the pair the reference's NVIDIA emitter fuses
(crates/rustc_codegen_tile/src/mlir_to_gpu.rs:542-641).
"""


def module(name, nptr, body, ret=True):
    args = ", ".join(f"%arg{i}: !llvm.ptr<1>" for i in range(nptr))
    lines = "\n".join("    " + l for l in body)
    return (f"module {{\n  llvm.func @{name}({args}) attributes {{hacc.entry}} {{\n    ^bb0:\n{lines}\n"
            f"    llvm.return\n  }}\n}}\n")


def consts(**kv):
    return [f"%{k} = llvm.mlir.constant({v} : i32) : i32" for k, v in kv.items()]


def softmax(name="softmax_rows", rows=1, cols=1024, dt="f32"):
    return module(name, 2, consts(c0=0, r=rows, c=cols) + [
        f"%t0 = llvm.call @__tile_load_{dt}(%arg0, %r, %c) : (!llvm.ptr<1>, i32, i32) -> i32",
        f"%t1 = llvm.call @__tile_softmax_{dt}(%c0, %t0, %r, %c) : (i32, i32, i32, i32) -> i32",
        f"llvm.call @__tile_store_{dt}(%arg1, %t1, %r, %c) : (!llvm.ptr<1>, i32, i32, i32) -> ()"])


def matmul(name="tile_matmul", m=128, k=128, n=128, dt="f32", out_dt=None, transposed=False):
    out_dt = out_dt or dt
    op = f"__tile_matmul_transposed_{dt}" if transposed else f"__tile_matmul_{dt}"
    bshape = "%n, %k" if transposed else "%k, %n"
    return module(name, 3, consts(m=m, k=k, n=n) + [
        f"%a = llvm.call @__tile_load_{dt}(%arg0, %m, %k) : (!llvm.ptr<1>, i32, i32) -> i32",
        f"%b = llvm.call @__tile_load_{dt}(%arg1, {bshape}) : (!llvm.ptr<1>, i32, i32) -> i32",
        f"%y = llvm.call @{op}(%a, %a, %b, %m, %k, %n) : (i32, i32, i32, i32, i32, i32) -> i32",
        f"llvm.call @__tile_store_{out_dt}(%arg2, %y, %m, %n) : (!llvm.ptr<1>, i32, i32, i32) -> ()"])


def attention(name="tile_attention", seq=64, dim=64, dt="f32"):
    return module(name, 4, consts(s=seq, d=dim) + [
        f"%q = llvm.call @__tile_load_{dt}(%arg0, %s, %d) : (!llvm.ptr<1>, i32, i32) -> i32",
        f"%k = llvm.call @__tile_load_{dt}(%arg1, %s, %d) : (!llvm.ptr<1>, i32, i32) -> i32",
        f"%v = llvm.call @__tile_load_{dt}(%arg2, %s, %d) : (!llvm.ptr<1>, i32, i32) -> i32",
        f"%o = llvm.call @__tile_attention_{dt}(%q, %q, %k, %v, %s, %d) : (i32, i32, i32, i32, i32, i32) -> i32",
        f"llvm.call @__tile_store_{dt}(%arg3, %o, %s, %d) : (!llvm.ptr<1>, i32, i32, i32) -> ()"])


def attention_gqa(name="tile_attention_gqa", heads=8, kv_heads=2, seq=32, dim=64, dt="f32"):
    return module(name, 4, consts(nh=heads, nkv=kv_heads, seq=seq, hd=dim, qr=heads * seq, kr=kv_heads * seq) + [
        f"%q = llvm.call @__tile_load_{dt}(%arg0, %qr, %hd) : (!llvm.ptr<1>, i32, i32) -> i32",
        f"%k = llvm.call @__tile_load_{dt}(%arg1, %kr, %hd) : (!llvm.ptr<1>, i32, i32) -> i32",
        f"%v = llvm.call @__tile_load_{dt}(%arg2, %kr, %hd) : (!llvm.ptr<1>, i32, i32) -> i32",
        f"%out = llvm.call @__tile_attention_gqa_{dt}(%q, %q, %k, %v, %nh, %nkv, %seq, %hd) : "
        "(i32, i32, i32, i32, i32, i32, i32, i32) -> i32",
        f"llvm.call @__tile_store_{dt}(%arg3, %out, %qr, %hd) : (!llvm.ptr<1>, i32, i32, i32) -> ()"])


def causal_chain(name="causal_attention", seq=128, dim=64, scale=None, mask=True):
    """matmul_transposed -> scale -> causal_mask -> softmax -> matmul, f32."""
    scale = scale if scale is not None else dim ** -0.5
    body = consts(s=seq, d=dim, z=0) + [
        f"%sc = llvm.mlir.constant({scale!r} : f32) : f32",
        "%q = llvm.call @__tile_load_f32(%arg0, %s, %d) : (!llvm.ptr<1>, i32, i32) -> i32",
        "%k = llvm.call @__tile_load_f32(%arg1, %s, %d) : (!llvm.ptr<1>, i32, i32) -> i32",
        "%v = llvm.call @__tile_load_f32(%arg2, %s, %d) : (!llvm.ptr<1>, i32, i32) -> i32",
        "%s0 = llvm.call @__tile_matmul_transposed_f32(%z, %q, %k, %s, %d, %s) : (i32, i32, i32, i32, i32, i32) -> i32",
        "%s1 = llvm.call @__tile_scale_f32(%z, %s0, %sc, %s, %s) : (i32, i32, f32, i32, i32) -> i32"]
    last = "%s1"
    if mask:
        body.append("%s2 = llvm.call @__tile_causal_mask_f32(%z, %s1, %s, %s) : (i32, i32, i32, i32) -> i32")
        last = "%s2"
    body += [f"%p = llvm.call @__tile_softmax_f32(%z, {last}, %s, %s) : (i32, i32, i32, i32) -> i32",
             "%o = llvm.call @__tile_matmul_f32(%z, %p, %v, %s, %s, %d) : (i32, i32, i32, i32, i32, i32) -> i32",
             "llvm.call @__tile_store_f32(%arg3, %o, %s, %d) : (!llvm.ptr<1>, i32, i32, i32) -> ()"]
    return module(name, 4, body)


def softmax_bf16_io(name="softmax_bf16_io", rows=1, cols=4096):
    """bf16 load -> cast to f32 -> softmax -> cast to bf16 -> bf16 store."""
    return module(name, 2, consts(c0=0, r=rows, c=cols) + [
        "%t0 = llvm.call @__tile_load_bf16(%arg0, %r, %c) : (!llvm.ptr<1>, i32, i32) -> i32",
        "%t1 = llvm.call @__tile_cast_bf16_f32(%c0, %t0, %r, %c) : (i32, i32, i32, i32) -> i32",
        "%t2 = llvm.call @__tile_softmax_f32(%c0, %t1, %r, %c) : (i32, i32, i32, i32) -> i32",
        "%t3 = llvm.call @__tile_cast_f32_bf16(%c0, %t2, %r, %c) : (i32, i32, i32, i32) -> i32",
        "llvm.call @__tile_store_bf16(%arg1, %t3, %r, %c) : (!llvm.ptr<1>, i32, i32, i32) -> ()"])


def narrow_then_softmax(name="narrow_then_softmax", rows=1, cols=1024):
    """f32 load -> cast to f16 -> softmax_f16 -> f16 store: the operator would have to see ROUNDED inputs."""
    return module(name, 2, consts(c0=0, r=rows, c=cols) + [
        "%t0 = llvm.call @__tile_load_f32(%arg0, %r, %c) : (!llvm.ptr<1>, i32, i32) -> i32",
        "%t1 = llvm.call @__tile_cast_f32_f16(%c0, %t0, %r, %c) : (i32, i32, i32, i32) -> i32",
        "%t2 = llvm.call @__tile_softmax_f16(%c0, %t1, %r, %c) : (i32, i32, i32, i32) -> i32",
        "llvm.call @__tile_store_f16(%arg1, %t2, %r, %c) : (!llvm.ptr<1>, i32, i32, i32) -> ()"])


def cast_round_trip(name="cast_round_trip", rows=1, cols=1024, dt="bf16"):
    """f32 load -> cast to bf16 -> cast back to f32 -> f32 store (the reference's bf16 round-trip test,
    crates/rustc_codegen_tile/src/mlir_to_linalg.rs:2249-2263): a rounding in the middle of the kernel."""
    return module(name, 2, consts(c0=0, r=rows, c=cols) + [
        "%t0 = llvm.call @__tile_load_f32(%arg0, %r, %c) : (!llvm.ptr<1>, i32, i32) -> i32",
        f"%t1 = llvm.call @__tile_cast_f32_{dt}(%c0, %t0, %r, %c) : (i32, i32, i32, i32) -> i32",
        f"%t2 = llvm.call @__tile_cast_{dt}_f32(%c0, %t1, %r, %c) : (i32, i32, i32, i32) -> i32",
        "llvm.call @__tile_store_f32(%arg1, %t2, %r, %c) : (!llvm.ptr<1>, i32, i32, i32) -> ()"])


GENERIC_SOFTMAX = '''"builtin.module"() ({
  "llvm.func"() <{CConv = #llvm.cconv<ccc>, function_type = !llvm.func<void (ptr<1>, ptr<1>)>, linkage = #llvm.linkage<external>, sym_name = "softmax_generic"}> ({
  ^bb0(%arg0: !llvm.ptr<1>, %arg1: !llvm.ptr<1>):
    %0 = "llvm.mlir.constant"() <{value = 0 : i32}> : () -> i32
    %1 = "llvm.mlir.constant"() <{value = 2 : i32}> : () -> i32
    %2 = "llvm.mlir.constant"() <{value = 512 : i32}> : () -> i32
    %3 = "llvm.call"(%arg0, %1, %2) <{callee = @__tile_load_f32, fastmathFlags = #llvm.fastmath<none>}> : (!llvm.ptr<1>, i32, i32) -> i32
    %4 = "llvm.call"(%0, %3, %1, %2) <{callee = @__tile_softmax_f32, fastmathFlags = #llvm.fastmath<none>}> : (i32, i32, i32, i32) -> i32
    "llvm.call"(%arg1, %4, %1, %2) <{callee = @__tile_store_f32, fastmathFlags = #llvm.fastmath<none>}> : (!llvm.ptr<1>, i32, i32, i32) -> ()
    "llvm.return"() : () -> ()
  }) {hacc.entry} : () -> ()
}) : () -> ()
'''

OUT_OF_SCOPE = module("rope_test", 2, consts(r=1, c=256, pos=7) + [
    "%a = llvm.call @__tile_load_f32(%arg0, %r, %c) : (!llvm.ptr<1>, i32, i32) -> i32",
    "%s = llvm.call @__tile_rope_f32(%a, %a, %pos, %r, %c) : (i32, i32, i32, i32, i32) -> i32",
    "llvm.call @__tile_store_f32(%arg1, %s, %r, %c) : (!llvm.ptr<1>, i32, i32, i32) -> ()"])


def ewise_add(name="add_test", rows=1, cols=256, dt="f32"):
    return module(name, 3, consts(r=rows, c=cols) + [
        f"%a = llvm.call @__tile_load_{dt}(%arg0, %r, %c) : (!llvm.ptr<1>, i32, i32) -> i32",
        f"%b = llvm.call @__tile_load_{dt}(%arg1, %r, %c) : (!llvm.ptr<1>, i32, i32) -> i32",
        f"%s = llvm.call @__tile_add_{dt}(%a, %a, %b, %r, %c) : (i32, i32, i32, i32, i32) -> i32",
        f"llvm.call @__tile_store_{dt}(%arg2, %s, %r, %c) : (!llvm.ptr<1>, i32, i32, i32) -> ()"])


def ewise_chain(name="gelu_like", rows=2, cols=512, dt="f32", out_dt=None):
    """out = clamp(tanh(scale(x, 0.5)) * y + exp(neg(abs(x))), -0.75, 2.5) / max(sqrt(abs(y)), sigmoid(x)): thirteen
    operators, two inputs (x is used four times), one pass."""
    out_dt = out_dt or dt
    u = "(i32, i32, i32, i32) -> i32"
    b = "(i32, i32, i32, i32, i32) -> i32"
    return module(name, 3, consts(c0=0, r=rows, c=cols) + [
        "%half = llvm.mlir.constant(5.000000e-01 : f32) : f32",
        "%lo = llvm.mlir.constant(-7.500000e-01 : f32) : f32",
        "%hi = llvm.mlir.constant(2.500000e+00 : f32) : f32",
        f"%x = llvm.call @__tile_load_{dt}(%arg0, %r, %c) : (!llvm.ptr<1>, i32, i32) -> i32",
        f"%y = llvm.call @__tile_load_{dt}(%arg1, %r, %c) : (!llvm.ptr<1>, i32, i32) -> i32",
        f"%t1 = llvm.call @__tile_scale_f32(%c0, %x, %half, %r, %c) : (i32, i32, f32, i32, i32) -> i32",
        f"%t2 = llvm.call @__tile_tanh_f32(%c0, %t1, %r, %c) : {u}",
        f"%t3 = llvm.call @__tile_mul_f32(%c0, %t2, %y, %r, %c) : {b}",
        f"%t4 = llvm.call @__tile_abs_f32(%c0, %x, %r, %c) : {u}",
        f"%t5 = llvm.call @__tile_neg_f32(%c0, %t4, %r, %c) : {u}",
        f"%t6 = llvm.call @__tile_exp_f32(%c0, %t5, %r, %c) : {u}",
        f"%t7 = llvm.call @__tile_add_f32(%c0, %t3, %t6, %r, %c) : {b}",
        f"%t8 = llvm.call @__tile_clamp_f32(%c0, %t7, %lo, %hi, %r, %c) : (i32, i32, f32, f32, i32, i32) -> i32",
        f"%t9 = llvm.call @__tile_abs_f32(%c0, %y, %r, %c) : {u}",
        f"%t10 = llvm.call @__tile_sqrt_f32(%c0, %t9, %r, %c) : {u}",
        f"%t11 = llvm.call @__tile_sigmoid_f32(%c0, %x, %r, %c) : {u}",
        f"%t12 = llvm.call @__tile_max_f32(%c0, %t10, %t11, %r, %c) : {b}",
        f"%t13 = llvm.call @__tile_div_f32(%c0, %t8, %t12, %r, %c) : {b}",
        f"llvm.call @__tile_store_{out_dt}(%arg2, %t13, %r, %c) : (!llvm.ptr<1>, i32, i32, i32) -> ()"])


def ewise_misc(name="misc_ops", rows=3, cols=333, dt="f32"):
    """out = min(relu(x) - rsqrt(fill(4.0)), log(silu(x) * silu(x) + fill(1.0))): the remaining operators, odd width."""
    u = "(i32, i32, i32, i32) -> i32"
    b = "(i32, i32, i32, i32, i32) -> i32"
    return module(name, 2, consts(c0=0, r=rows, c=cols) + [
        "%four = llvm.mlir.constant(4.000000e+00 : f32) : f32",
        "%one = llvm.mlir.constant(1.000000e+00 : f32) : f32",
        f"%x = llvm.call @__tile_load_{dt}(%arg0, %r, %c) : (!llvm.ptr<1>, i32, i32) -> i32",
        f"%f4 = llvm.call @__tile_fill_f32(%c0, %four, %r, %c) : (i32, f32, i32, i32) -> i32",
        f"%f1 = llvm.call @__tile_fill_f32(%c0, %one, %r, %c) : (i32, f32, i32, i32) -> i32",
        f"%t1 = llvm.call @__tile_relu_f32(%c0, %x, %r, %c) : {u}",
        f"%t2 = llvm.call @__tile_rsqrt_f32(%c0, %f4, %r, %c) : {u}",
        f"%t3 = llvm.call @__tile_sub_f32(%c0, %t1, %t2, %r, %c) : {b}",
        f"%t4 = llvm.call @__tile_silu_f32(%c0, %x, %r, %c) : {u}",
        f"%t5 = llvm.call @__tile_mul_f32(%c0, %t4, %t4, %r, %c) : {b}",
        f"%t6 = llvm.call @__tile_add_f32(%c0, %t5, %f1, %r, %c) : {b}",
        f"%t7 = llvm.call @__tile_log_f32(%c0, %t6, %r, %c) : {u}",
        f"%t8 = llvm.call @__tile_min_f32(%c0, %t3, %t7, %r, %c) : {b}",
        f"llvm.call @__tile_store_{dt}(%arg1, %t8, %r, %c) : (!llvm.ptr<1>, i32, i32, i32) -> ()"])


def rms_norm(name="tile_rms", rows=1, cols=256, dt="f32", eps="1.0e-5"):
    return module(name, 2, consts(r=rows, c=cols) + [
        f"%eps = llvm.mlir.constant({eps} : f32) : f32",
        f"%x = llvm.call @__tile_load_{dt}(%arg0, %r, %c) : (!llvm.ptr<1>, i32, i32) -> i32",
        f"%y = llvm.call @__tile_rms_norm_{dt}(%x, %x, %eps, %r, %c) : (i32, i32, f32, i32, i32) -> i32",
        f"llvm.call @__tile_store_{dt}(%arg1, %y, %r, %c) : (!llvm.ptr<1>, i32, i32, i32) -> ()"])


def reduce(kind="sum", name=None, rows=1, cols=1024, dt="f32"):
    return module(name or f"tile_reduce_{kind}", 2, consts(r=rows, c=cols, one=1) + [
        f"%x = llvm.call @__tile_load_{dt}(%arg0, %r, %c) : (!llvm.ptr<1>, i32, i32) -> i32",
        f"%y = llvm.call @__tile_reduce_{kind}_{dt}(%x, %x, %r, %c) : (i32, i32, i32, i32) -> i32",
        f"llvm.call @__tile_store_{dt}(%arg1, %y, %r, %one) : (!llvm.ptr<1>, i32, i32, i32) -> ()"])


def silu(name="tile_silu", rows=1, cols=1024, dt="f32"):
    return module(name, 2, consts(r=rows, c=cols) + [
        f"%x = llvm.call @__tile_load_{dt}(%arg0, %r, %c) : (!llvm.ptr<1>, i32, i32) -> i32",
        f"%y = llvm.call @__tile_silu_{dt}(%x, %x, %r, %c) : (i32, i32, i32, i32) -> i32",
        f"llvm.call @__tile_store_{dt}(%arg1, %y, %r, %c) : (!llvm.ptr<1>, i32, i32, i32) -> ()"])


def silu_mul(name="tile_swiglu", rows=1, cols=1024, dt="f32", up_first=False):
    ops = "%u, %s" if up_first else "%s, %u"
    return module(name, 3, consts(c0=0, r=rows, c=cols) + [
        f"%g = llvm.call @__tile_load_{dt}(%arg0, %r, %c) : (!llvm.ptr<1>, i32, i32) -> i32",
        f"%u = llvm.call @__tile_load_{dt}(%arg1, %r, %c) : (!llvm.ptr<1>, i32, i32) -> i32",
        f"%s = llvm.call @__tile_silu_{dt}(%c0, %g, %r, %c) : (i32, i32, i32, i32) -> i32",
        f"%y = llvm.call @__tile_mul_{dt}(%c0, {ops}, %r, %c) : (i32, i32, i32, i32, i32) -> i32",
        f"llvm.call @__tile_store_{dt}(%arg2, %y, %r, %c) : (!llvm.ptr<1>, i32, i32, i32) -> ()"])
