"""The cuda_sm100 CodegenTarget and the registry, on the host.  Scenario shapes
follow the reference's behaviour specs (crates/tile_spec/features/
backend_emit_purity.feature, core_op_lowering.feature, registry_add_target.feature)
and registry unit tests (crates/tile_codegen/src/lib.rs:69-148)."""
import pytest

import mlir_fixtures as F


@pytest.fixture(scope="module")
def cg(pkg):
    return pkg.codegen


@pytest.fixture(scope="module")
def target(cg):
    t = cg.TargetRegistry.with_builtin().select("cuda_sm100")
    assert t is not None
    return t


def test_builtin_registry_has_debug_and_cuda_sm100(cg):
    r = cg.TargetRegistry.with_builtin()
    assert "debug" in r.names() and "cuda_sm100" in r.names()
    assert r.len() == 2 and not r.is_empty()
    assert r.select("nope") is None
    assert cg.TargetRegistry.new().is_empty()


def test_register_and_select_first_match_wins(cg):
    class MyAccel(cg.CodegenTarget):
        def name(self):
            return "myaccel"

        def emit(self, mlir_text, opts=cg.EmitOpts()):
            if not mlir_text.strip():
                raise cg.EmitError("empty MLIR module")
            return cg.EmitOut("// myaccel\n", "acc")

    r = cg.TargetRegistry.new()
    r.register(MyAccel())
    r.register(cg.EmitterTarget("myaccel", "txt", lambda s: "shadowed"))
    assert r.len() == 2 and r.names() == ["myaccel", "myaccel"]
    assert r.select("myaccel").emit("module {}").ext == "acc"
    lifted = cg.EmitterTarget("fake", "txt", lambda s: s.upper())
    assert lifted.emit("abc").source == "ABC" and lifted.emit("abc").ext == "txt"


def test_debug_target(cg):
    d = cg.DebugTarget()
    out = d.emit("module {\n func.func @f() { }\n}")
    assert out.ext == "mlir.txt" and "3 MLIR lines, 1 func.func op(s)" in out.source
    with pytest.raises(cg.EmitError):
        d.emit("  \n ")


CASES = {
    "softmax": (F.softmax(), ["softmax_rows_warp<float, 8, 4>", "d.cols = 1024", "tsm100::ops::softmax"]),
    "softmax_bf16_io": (F.softmax_bf16_io(), ["softmax_rows_cta<__nv_bfloat16, 4, 128>", "TSM100_BF16", "d.cols = 4096"]),
    "matmul_f32": (F.matmul(), ["gemm_tf32x3_kernel<false>", "d.m = 128", "tsm100::ops::gemm"]),
    "matmul_f32_odd": (F.matmul(m=33, k=30, n=17), ["gemm_simt_kernel<float, float", "d.k = 30"]),
    "matmul_f16": (F.matmul(dt="f16", m=64, k=128, n=64), ["gemm_tc_kernel<__half, false, false>", "TSM100_F16", "tcgen05"]),
    "matmul_bf16": (F.matmul(dt="bf16", m=8192, k=8192, n=8192), ["gemm_tc_kernel<__nv_bfloat16, false, true>", "d.k = 8192"]),
    "matmul_f16_acc_f32": (F.matmul(dt="f16", out_dt="f32"), ["gemm_tc_kernel<float, false, false>", "d.out_dtype = TSM100_F32"]),
    "matmul_transposed": (F.matmul(transposed=True, m=32, k=64, n=16), ["d.b_transposed = 1", "d.n = 16"]),
    "attention": (F.attention(), ["attention_simt_kernel<float>", "d.causal = 0", "d.seq = 64"]),
    "attention_bf16": (F.attention(seq=4096, dim=128, dt="bf16"), ["attention_fwd_kernel<true>", "d.head_dim = 128"]),
    "attention_gqa": (F.attention_gqa(), ["d.causal = 1", "d.heads_q = 8", "d.heads_kv = 2", "d.seq = 32"]),
    "causal_chain": (F.causal_chain(), ["d.causal = 1", "d.seq = 128", "d.head_dim = 64", "fused"]),
    "plain_chain": (F.causal_chain(mask=False), ["d.causal = 0"]),
    "generic_form": (F.GENERIC_SOFTMAX, ["softmax_generic_launch", "* 2;", "d.cols = 512"]),
    "rms_norm": (F.rms_norm(), ["row_op_kernel<float, tsm100::rowops::kRmsNorm, 2, 32, 128>", "d.eps = 9.99999975e-06f", "tsm100::ops::rms_norm"]),
    "rms_norm_bf16_wide": (F.rms_norm(rows=4, cols=4096, dt="bf16", eps="1.0e-6"),
                           ["row_op_kernel<__nv_bfloat16, tsm100::rowops::kRmsNorm, 4, 128, 128>", "blocks) * 4;", "TSM100_BF16"]),
    "reduce_sum": (F.reduce("sum"), ["row_op_kernel<float, tsm100::rowops::kReduceSum, 8, 32, 128>", "TSM100_REDUCE_SUM", "d.cols = 1024"]),
    "reduce_max": (F.reduce("max", cols=5000), ["row_op_kernel<float, tsm100::rowops::kReduceMax, 8, 256, 256>", "TSM100_REDUCE_MAX"]),
    "reduce_odd_width": (F.reduce("sum", cols=1001), ["row_op_stream_kernel<float, tsm100::rowops::kReduceSum, 512>"]),
    "ewise_add": (F.ewise_add(), ["add_test_ewise_vec", "a0[e] + a1[e]".replace("a0[e] + a1[e]", "v0 + v1"), "out = add(in0, in1)", "one pass"]),
    "ewise_chain": (F.ewise_chain(), ["gelu_like_ewise_vec(const float* __restrict__ p0, const float* __restrict__ p1, float* __restrict__ out",
                                      "tanhf(", "op_clamp(", "-0.75f, 2.5f", "op_sigmoid(", "fmaxf(", "* 0.5f", "blocks) * 2 * 512"]),
    "ewise_chain_bf16_to_f32": (F.ewise_chain(dt="bf16", out_dt="f32"), ["const __nv_bfloat16* __restrict__ p0", "float* __restrict__ out"]),
    "ewise_misc": (F.ewise_misc(), ["op_relu(", "op_rsqrt(", "op_silu(", "logf(", "fminf(", "4.0f", "misc_ops_ewise_scalar"]),
    "silu": (F.silu(), ["silu_mul_kernel<float, false, 4, 256>", "nullptr, args[1]", "tsm100::ops::silu_mul"]),
    "silu_mul": (F.silu_mul(), ["silu_mul_kernel<float, true, 4, 256>", "args[0], args[1], args[2]", "fused"]),
    "silu_mul_up_first_f16": (F.silu_mul(dt="f16", up_first=True, cols=4096), ["silu_mul_kernel<__half, true, 4, 256>", "args[0], args[1], args[2]"]),
}


@pytest.mark.parametrize("name", sorted(CASES))
def test_emit_idiom_purity_and_determinism(target, name):
    mlir, needles = CASES[name]
    out = target.emit(mlir)
    assert out.ext == "cu"
    assert "__global__" in out.source  # the CUDA idiom the reference's gpu rows require
    assert len(out.meta.kernel_names) == 1 and out.meta.kernel_names[0] + "_launch" in out.source
    for n in needles:
        assert n in out.source, (n, out.source)
    assert "TODO" not in out.source
    again = target.emit(mlir)
    assert again.source == out.source and again.meta.kernel_names == out.meta.kernel_names  # byte-identical re-emit


def test_two_kernels_in_one_module(target):
    two = F.softmax("k_one").rsplit("}", 1)[0] + F.matmul("k_two", dt="bf16").split("module {", 1)[1]
    out = target.emit(two)
    assert out.meta.kernel_names == ["k_one", "k_two"]


def test_non_entry_functions_are_ignored(target):
    m = F.softmax("entry_k").replace("module {", "module {\n  llvm.func @helper(%arg0: i32) -> i32 {\n    llvm.return %arg0 : i32\n  }")
    assert target.emit(m).meta.kernel_names == ["entry_k"]


@pytest.mark.parametrize("mlir,fragment", [
    ("", "empty MLIR module"), ("  \n\t ", "empty MLIR module"),
    ("module {\n}\n", "no entry kernel"),
    (F.softmax().replace(" attributes {hacc.entry}", ""), "no entry kernel"),
    (F.OUT_OF_SCOPE, "__tile_rope_f32 is outside the cuda_sm100 target"),
    (F.ewise_add().replace("(%arg1, %r, %c)", "(%arg1, %c, %r)"), "share the stored tile's shape"),
    (F.ewise_chain().replace("__tile_tanh_f32(%c0, %t1", "__tile_softmax_f32(%c0, %t1"), "may only consume loaded tiles"),
    (F.causal_chain(scale=0.5), "1/sqrt(head_dim)"),
    (F.reduce("sum").replace("%y, %r, %one)", "%y, %r, %c)"), "rows x 1 tile"),
    (F.silu_mul().replace("__tile_silu_f32(%c0, %g", "__tile_softmax_f32(%c0, %g"), "may only consume loaded tiles"),
    (F.rms_norm().replace("%eps, %r, %c) : (i32, i32, f32", "%eps, %r) : (i32, i32, f32"), "expects 5 operands"),
    (F.softmax().replace("%t0, %r, %c) : (i32", "%t0, %r) : (i32"), "expects 4 operands"),
    (F.softmax().replace("(%c0, %t0, %r, %c)", "(%c0, %t0, %r, %7)"), "not a compile-time integer constant"),
    (F.softmax().replace("(%arg0, %r, %c)", "(%c0, %r, %c)"), "not a global-memory pointer"),
    (F.matmul(dt="f16", out_dt="bf16"), "matmul output must be the input type or f32"),
    # casts are relabels only where they change no value; a rounding in the middle of a kernel is refused, not skipped
    (F.narrow_then_softmax(), "an operator reads a value narrowed to f16"),
    (F.cast_round_trip(), "already narrowed to bf16"),
    (F.softmax_bf16_io().replace("__tile_cast_f32_bf16", "__tile_cast_f32_f16"), "a value narrowed to f16 is stored as bf16"),
    (F.softmax_bf16_io().replace("__tile_cast_bf16_f32", "__tile_cast_f16_f32"), "must widen a freshly loaded f16 tile"),
    (F.matmul().replace("%m, %n) : (!llvm.ptr<1>, i32, i32, i32) -> ()", "%n, %n) : (!llvm.ptr<1>, i32, i32, i32) -> ()")
     .replace("%n = llvm.mlir.constant(128", "%n = llvm.mlir.constant(64"), "shapes disagree"),
])
def test_emit_rejects(target, cg, mlir, fragment):
    with pytest.raises(cg.EmitError) as e:
        target.emit(mlir)
    assert fragment in str(e.value), str(e.value)


def test_emitted_module_compiles(target, pkg, tmp_path):
    """nvcc accepts what emit produces (cross-compiled for sm_100a; no GPU needed): a library operator and
    two generated element-wise kernels in one module."""
    parts = [F.softmax("sm_compile_check", rows=2, cols=512), F.ewise_chain("chain_compile_check", dt="bf16", out_dt="f32"),
             F.ewise_misc("misc_compile_check")]
    mlir = parts[0].rsplit("}", 1)[0] + "".join(p.split("module {", 1)[1].rsplit("}", 1)[0] for p in parts[1:]) + "}\n"
    out = target.emit(mlir)
    assert out.meta.kernel_names == ["sm_compile_check", "chain_compile_check", "misc_compile_check"]
    so = pkg.build.build_module(out.source, tmp_path / "mod.so")
    assert so.exists() and so.stat().st_size > 0


def test_tile_kernel_descriptors(target, cg):
    """EmitOut.meta carries one TileKernel descriptor per entry kernel (tile_hal kernel.rs:93-212)."""
    out = target.emit(F.matmul("mm", 64, 128, 32, dt="f16", out_dt="f32"))
    (k,) = out.meta.kernels
    assert k.name == "mm" and k.mode == "General" and k.uses_matmul() and k.inferred_mode() == "General"
    assert (k.num_inputs, k.num_outputs) == (2, 1)
    assert [o.op for o in k.ops] == ["Load", "Load", "Matmul", "Store"]
    assert k.ops[2].params == {"m": 64, "k": 128, "n": 32}
    assert k.ops[3].params == {"rows": 64, "cols": 32, "dtype": "F32"}
    assert [(a.role, a.dtype, a.elements_per_block) for a in k.args] == [("input", "F16", 64 * 128), ("input", "F16", 128 * 32),
                                                                         ("output", "F32", 64 * 32)]
    assert k.args[2].bytes_for(3) == 3 * 64 * 32 * 4

    (k,) = target.emit(F.ewise_chain()).meta.kernels
    assert k.mode == "Vector" and not k.uses_matmul()
    assert [o.op for o in k.ops] == ["Load", "Load", "Scale", "Tanh", "Mul", "Abs", "Neg", "Exp", "Add", "Clamp", "Abs", "Sqrt",
                                     "Sigmoid", "Max", "Div", "Store"]
    assert k.ops[2].params == {"rows": 2, "cols": 512, "scalar": 0.5}
    assert k.ops[9].params == {"rows": 2, "cols": 512, "lo": -0.75, "hi": 2.5}

    (k,) = target.emit(F.rms_norm(rows=4, cols=4096, dt="bf16", eps="1.0e-6")).meta.kernels
    assert [o.op for o in k.ops] == ["Load", "RmsNorm", "Store"] and abs(k.ops[1].params["eps"] - 1e-6) < 1e-12
    (k,) = target.emit(F.reduce("max", rows=2, cols=1000)).meta.kernels
    assert [o.op for o in k.ops] == ["Load", "ReduceMax", "Store"]
    assert [(a.role, a.elements_per_block) for a in k.args] == [("input", 2000), ("output", 2)]
    (k,) = target.emit(F.attention_gqa()).meta.kernels
    assert k.mode == "General" and k.ops[3].op == "Attention" and k.ops[3].params["kv_heads"] == 2
    (k,) = target.emit(F.causal_chain()).meta.kernels
    assert [o.op for o in k.ops if o.op not in ("Load", "Store")] == ["Matmul", "Scale", "CausalMask", "Softmax", "Matmul"]
    assert k.ops[3].params["b_transposed"] is True
    two = F.softmax("k_one").rsplit("}", 1)[0] + F.matmul("k_two", dt="bf16").split("module {", 1)[1]
    assert [k.name for k in target.emit(two).meta.kernels] == ["k_one", "k_two"]
    with pytest.raises(cg.EmitError):
        target.describe("")
