"""The tile_hal mirror and emitted kernel modules on a real device, through the C ABI."""
import numpy as np
import pytest

import mlir_fixtures as F
import util

pytestmark = pytest.mark.gpu
torch = pytest.importorskip("torch")


def test_device_queries(dev, pkg):
    assert pkg.hal.CudaSm100Device.device_count() >= 1
    assert dev.ordinal() == 0 and "B200" in dev.name() or dev.sm_count() > 0
    mi = dev.mem_info()
    assert 0 < mi.free <= mi.total and mi.total > 100 << 30
    sel = pkg.hal.BackendSelector(pkg.hal.BackendKind.from_codegen_path("cuda_sm100"))
    d2 = sel.device(0)
    assert d2.name() == dev.name()
    d2.close()
    with pytest.raises(pkg.hal.KernelError):
        pkg.hal.CudaSm100Device(9999)


def test_buffer_round_trip_and_streams(dev):
    s = dev.create_stream()
    host = np.arange(100000, dtype=np.float32)
    buf = dev.alloc_from_slice(host, s)
    assert buf.len() == host.size and not buf.is_empty() and buf.as_raw_ptr() != 0
    assert np.array_equal(buf.copy_to_host(s), host)
    buf.copy_from_host(host[::-1].copy(), s)
    assert np.array_equal(buf.copy_to_host(s), host[::-1])
    empty = dev.alloc_f32(0)
    assert empty.is_empty() and empty.copy_to_host(s).size == 0
    s.synchronize()
    assert s.query()
    with pytest.raises(Exception):
        buf.copy_from_host(np.zeros(3, np.float32), s)


def test_events_time_a_kernel(dev, pkg):
    s = dev.create_stream()
    x = dev.alloc_from_slice(util.softmax_input(pkg.capi, 4096, 4096), s)
    y = dev.alloc(4096 * 4096, np.float32)
    e0, e1 = dev.create_event(), dev.create_event()
    e0.record(s)
    dev.softmax(pkg.capi.F32, 4096, 4096, x.as_raw_ptr(), y.as_raw_mut_ptr(), stream=s.raw)
    e1.record(s)
    e1.synchronize()
    ms = e0.elapsed_ms(e1)
    assert 0.0 < ms < 50.0
    assert abs(float(y.copy_to_host(s)[:4096].sum()) - 1.0) < 1e-5


def _module(pkg, tmp_path, mlir, name):
    out = pkg.codegen.CudaSm100Target().emit(mlir)
    so = pkg.build.build_module(out.source, tmp_path / f"{name}.so")
    return out, so


def test_emitted_softmax_module_launches(dev, pkg, oracle, tmp_path):
    """emit -> nvcc -> KernelLauncher.load -> launch(name, LaunchGrid, args, stream): the reference's flow."""
    rows_per_block, cols, blocks = 2, 1024, 37
    out, so = _module(pkg, tmp_path, F.softmax("softmax_tiles", rows_per_block, cols), "sm")
    launcher = dev.create_launcher()
    launcher.load(so, pkg.hal.KernelMode.Vector)
    s = dev.create_stream()
    x = util.softmax_input(pkg.capi, blocks * rows_per_block, cols)
    xb = dev.alloc_from_slice(x, s)
    yb = dev.alloc(x.size, np.float32)
    launcher.launch(out.meta.kernel_names[0], pkg.hal.LaunchGrid.blocks_(blocks), [xb.as_raw_ptr(), yb.as_raw_mut_ptr()], s)
    y = yb.copy_to_host(s).reshape(x.shape)
    m = oracle.compare(y, oracle.softmax_f32(x), floor_r=1e-30)
    assert m["rel_max"] <= util.F32_REL and m["max_elem_rel"] <= util.F32_REL, m
    with pytest.raises(pkg.hal.KernelError):
        launcher.launch("no_such_kernel", pkg.hal.LaunchGrid.blocks_(1), [0, 0], s)
    with pytest.raises(pkg.hal.KernelError):
        launcher.launch(out.meta.kernel_names[0], pkg.hal.LaunchGrid.blocks_(1), [xb.as_raw_ptr()], s)  # wrong arity


def test_emitted_gemm_and_attention_modules(dev, pkg, oracle, tmp_path):
    capi = pkg.capi
    two = (F.matmul("mm_bf16", 256, 192, 256, dt="bf16").rsplit("}", 1)[0]
           + F.attention_gqa("gqa_bf16", 4, 2, 256, 128, dt="bf16").split("module {", 1)[1])
    out, so = _module(pkg, tmp_path, two, "two")
    assert out.meta.kernel_names == ["mm_bf16", "gqa_bf16"]
    launcher = dev.create_launcher()
    launcher.load(so, pkg.hal.KernelMode.Matrix)
    s = dev.create_stream()
    blocks = 3  # three independent problems, one per block tile
    a = util.to_bf16(capi, util.gen_normal(capi, (blocks, 256, 192), 1, 0.3))
    b = util.to_bf16(capi, util.gen_normal(capi, (blocks, 192, 256), 2, 0.3))
    ab, bb = dev.alloc_from_slice(a, s), dev.alloc_from_slice(b, s)
    cb = dev.alloc(blocks * 256 * 256, np.uint16)
    launcher.launch("mm_bf16", pkg.hal.LaunchGrid.blocks_(blocks), [ab.as_raw_ptr(), bb.as_raw_ptr(), cb.as_raw_mut_ptr()], s)
    c = cb.copy_to_host(s).reshape(blocks, 256, 256)
    assert dev.status(s) == 0
    for i in range(blocks):
        ref32, _ = oracle.gemm_bf16(a[i], b[i])
        util.assert_16bit_close(oracle, oracle.bf16_to_f32(c[i]), ref32, i)
    q = util.to_bf16(capi, util.gen_normal(capi, (2, 4, 256, 128), 3))
    k = util.to_bf16(capi, util.gen_normal(capi, (2, 2, 256, 128), 4))
    v = util.to_bf16(capi, util.gen_normal(capi, (2, 2, 256, 128), 5))
    qb, kb, vb = (dev.alloc_from_slice(t, s) for t in (q, k, v))
    ob = dev.alloc(q.size, np.uint16)
    launcher.launch("gqa_bf16", pkg.hal.LaunchGrid.blocks_(2), [qb.as_raw_ptr(), kb.as_raw_ptr(), vb.as_raw_ptr(), ob.as_raw_mut_ptr()], s)
    o = ob.copy_to_host(s).reshape(q.shape)
    assert dev.status(s) == 0
    ref32, _ = oracle.attention_bf16(q, k, v, True)
    util.assert_16bit_close(oracle, oracle.bf16_to_f32(o), ref32)


def test_emitted_row_operator_modules(dev, pkg, oracle, tmp_path):
    """rms_norm, reduce_max and the fused silu * mul pair through emit -> nvcc -> load -> launch."""
    capi = pkg.capi
    rows_per_block, cols, blocks = 2, 2048, 19
    parts = [F.rms_norm("rms_tiles", rows_per_block, cols, eps="1.0e-6"), F.reduce("max", "max_tiles", rows_per_block, cols),
             F.silu_mul("swiglu_tiles", rows_per_block, cols)]
    mlir = parts[0].rsplit("}", 1)[0] + "".join(p.split("module {", 1)[1].rsplit("}", 1)[0] for p in parts[1:]) + "}\n"
    out, so = _module(pkg, tmp_path, mlir, "rowops")
    assert out.meta.kernel_names == ["rms_tiles", "max_tiles", "swiglu_tiles"]
    launcher = dev.create_launcher()
    launcher.load(so, pkg.hal.KernelMode.Vector)
    s = dev.create_stream()
    grid = pkg.hal.LaunchGrid.blocks_(blocks)
    rows = blocks * rows_per_block
    x = util.gen_normal(capi, (rows, cols), 601, 3.0)
    u = util.gen_normal(capi, (rows, cols), 603)
    xb, ub = dev.alloc_from_slice(x, s), dev.alloc_from_slice(u, s)
    yb, rb = dev.alloc(x.size, np.float32), dev.alloc(rows, np.float32)
    launcher.launch("rms_tiles", grid, [xb.as_raw_ptr(), yb.as_raw_mut_ptr()], s)
    m = oracle.compare(yb.copy_to_host(s).reshape(x.shape), oracle.rms_norm_f32(x, 1e-6, f64_acc=True))
    assert m["rel_max"] <= util.F32_REL, m
    launcher.launch("max_tiles", grid, [xb.as_raw_ptr(), rb.as_raw_mut_ptr()], s)
    assert np.array_equal(rb.copy_to_host(s), oracle.reduce_f32(x, "max"))
    launcher.launch("swiglu_tiles", grid, [xb.as_raw_ptr(), ub.as_raw_ptr(), yb.as_raw_mut_ptr()], s)
    m = oracle.compare(yb.copy_to_host(s).reshape(x.shape), oracle.silu_mul_f32(x, u, f64_acc=True))
    assert m["rel_max"] <= util.F32_REL, m
    assert dev.status(s) == 0


def test_generated_elementwise_kernels(dev, pkg, oracle, tmp_path):
    """Chains of element-wise intrinsics are emitted as one generated kernel each; results against the
    float64 statement of the same operators (oracle_np.EWISE)."""
    from oracle import oracle_np as onp
    E = onp.EWISE
    capi = pkg.capi
    parts = [F.ewise_chain("chain_f32", 2, 512), F.ewise_chain("chain_bf16", 2, 512, dt="bf16", out_dt="f32"),
             F.ewise_misc("misc_f32", 3, 333), F.ewise_add("add_f16", 1, 4096, dt="f16")]
    mlir = parts[0].rsplit("}", 1)[0] + "".join(p.split("module {", 1)[1].rsplit("}", 1)[0] for p in parts[1:]) + "}\n"
    out, so = _module(pkg, tmp_path, mlir, "ewise")
    assert out.meta.kernel_names == ["chain_f32", "chain_bf16", "misc_f32", "add_f16"]
    launcher = dev.create_launcher()
    launcher.load(so, pkg.hal.KernelMode.Vector)
    s = dev.create_stream()

    def chain(x, y):
        x, y = x.astype(np.float64), y.astype(np.float64)
        num = E["clamp"](E["add"](E["mul"](E["tanh"](E["scale"](x, 0.5)), y), E["exp"](E["neg"](E["abs"](x)))), -0.75, 2.5)
        return E["div"](num, E["max"](E["sqrt"](E["abs"](y)), E["sigmoid"](x)))

    blocks = 41
    x = util.gen_normal(capi, (blocks * 2, 512), 701, 2.0)
    y = util.gen_normal(capi, (blocks * 2, 512), 702, 1.5)
    xb, yb = dev.alloc_from_slice(x, s), dev.alloc_from_slice(y, s)
    ob = dev.alloc(x.size, np.float32)
    launcher.launch("chain_f32", pkg.hal.LaunchGrid.blocks_(blocks), [xb.as_raw_ptr(), yb.as_raw_ptr(), ob.as_raw_mut_ptr()], s)
    got = ob.copy_to_host(s).reshape(x.shape)
    ref = chain(x, y)
    assert np.abs(got - ref).max() / np.abs(ref).max() <= util.F32_REL
    assert np.abs(got - ref).max() <= 1e-5 * (1.0 + np.abs(ref).max())

    x16, y16 = util.to_bf16(capi, x), util.to_bf16(capi, y)
    xb16, yb16 = dev.alloc_from_slice(x16, s), dev.alloc_from_slice(y16, s)
    launcher.launch("chain_bf16", pkg.hal.LaunchGrid.blocks_(blocks), [xb16.as_raw_ptr(), yb16.as_raw_ptr(), ob.as_raw_mut_ptr()], s)
    got = ob.copy_to_host(s).reshape(x.shape)
    ref = chain(onp.bf16_bits_to_f32(x16), onp.bf16_bits_to_f32(y16))  # bf16 inputs widen exactly; the store is f32
    assert np.abs(got - ref).max() / np.abs(ref).max() <= util.F32_REL

    blocks = 7  # 7 * 3 * 333 elements: not a multiple of eight -> the scalar kernel
    z = util.gen_normal(capi, (blocks * 3, 333), 703, 2.0)
    zb = dev.alloc_from_slice(z, s)
    mb = dev.alloc(z.size, np.float32)
    launcher.launch("misc_f32", pkg.hal.LaunchGrid.blocks_(blocks), [zb.as_raw_ptr(), mb.as_raw_mut_ptr()], s)
    got = mb.copy_to_host(s).reshape(z.shape)
    z64 = z.astype(np.float64)
    sl = E["silu"](z64)
    ref = E["min"](E["sub"](E["relu"](z64), E["rsqrt"](np.full_like(z64, 4.0))), E["log"](E["add"](E["mul"](sl, sl), 1.0)))
    assert np.abs(got - ref).max() <= 1e-5 * (1.0 + np.abs(ref).max())

    a = util.f32_to_f16_bits(util.gen_normal(capi, (5, 4096), 704))
    b = util.f32_to_f16_bits(util.gen_normal(capi, (5, 4096), 705))
    ab, bb = dev.alloc_from_slice(a, s), dev.alloc_from_slice(b, s)
    cb = dev.alloc(a.size, np.uint16)
    launcher.launch("add_f16", pkg.hal.LaunchGrid.blocks_(5), [ab.as_raw_ptr(), bb.as_raw_ptr(), cb.as_raw_mut_ptr()], s)
    got = cb.copy_to_host(s).reshape(a.shape).view(np.float16)
    want = (a.view(np.float16).astype(np.float32) + b.view(np.float16).astype(np.float32)).astype(np.float16)
    assert np.array_equal(got, want)  # one exact f32 sum, one RNE rounding
    assert dev.status(s) == 0


def test_launch_with_tile_kernel_descriptor(dev, pkg, oracle, tmp_path):
    """KernelLauncher.launch_described: the descriptor emitted beside the binary sizes and validates the buffers."""
    rows_per_block, cols, blocks = 4, 512, 9
    out, so = _module(pkg, tmp_path, F.softmax("softmax_desc", rows_per_block, cols), "desc")
    (k,) = out.meta.kernels
    launcher = dev.create_launcher()
    launcher.load(so, pkg.hal.KernelMode[k.mode])
    s = dev.create_stream()
    x = util.softmax_input(pkg.capi, blocks * rows_per_block, cols)
    xb = dev.alloc_from_slice(x, s)
    yb = dev.alloc(k.args[1].elements_per_block * blocks, np.float32)
    launcher.launch_described(k, pkg.hal.LaunchGrid.blocks_(blocks), [xb, yb], s)
    m = oracle.compare(yb.copy_to_host(s).reshape(x.shape), oracle.softmax_f32(x), floor_r=1e-30)
    assert m["rel_max"] <= util.F32_REL, m
    with pytest.raises(pkg.hal.KernelError, match="blocks need"):
        launcher.launch_described(k, pkg.hal.LaunchGrid.blocks_(blocks + 1), [xb, yb], s)  # buffers too small for ten tiles
    with pytest.raises(pkg.hal.KernelError, match="takes 2 buffers"):
        launcher.launch_described(k, pkg.hal.LaunchGrid.blocks_(blocks), [xb], s)


def test_emitted_causal_chain_module_launches(dev, pkg, oracle, tmp_path):
    """matmul_transposed -> scale -> causal_mask -> softmax -> matmul is recognised as ONE fused causal attention;
    the emitted module is launched, one (batch, head) per block, and matches the oracle's causal attention."""
    seq, dim, blocks = 256, 64, 5
    out, so = _module(pkg, tmp_path, F.causal_chain("causal_attention", seq, dim), "causal")
    assert out.meta.kernel_names == ["causal_attention"]
    launcher = dev.create_launcher()
    launcher.load(so, pkg.hal.KernelMode.Matrix)
    s = dev.create_stream()
    q, k, v = (util.gen_normal(pkg.capi, (blocks, 1, seq, dim), 410 + i) for i in range(3))
    qb, kb, vb = (dev.alloc_from_slice(t, s) for t in (q, k, v))
    ob = dev.alloc(q.size, np.float32)
    launcher.launch("causal_attention", pkg.hal.LaunchGrid.blocks_(blocks),
                    [qb.as_raw_ptr(), kb.as_raw_ptr(), vb.as_raw_ptr(), ob.as_raw_mut_ptr()], s)
    o = ob.copy_to_host(s).reshape(q.shape)
    assert dev.status(s) == 0
    m = oracle.compare(o, oracle.attention_f32(q, k, v, True))
    assert m["rel_max"] <= util.F32_REL and m["rel_fro"] <= util.F32_REL, m
    # and without the mask the same chain is plain attention
    out2, so2 = _module(pkg, tmp_path, F.causal_chain("plain_attention", seq, dim, mask=False), "plain")
    l2 = dev.create_launcher()
    l2.load(so2, pkg.hal.KernelMode.Matrix)
    l2.launch("plain_attention", pkg.hal.LaunchGrid.blocks_(blocks),
              [qb.as_raw_ptr(), kb.as_raw_ptr(), vb.as_raw_ptr(), ob.as_raw_mut_ptr()], s)
    o2 = ob.copy_to_host(s).reshape(q.shape)
    m = oracle.compare(o2, oracle.attention_f32(q, k, v, False))
    assert m["rel_max"] <= util.F32_REL and m["rel_fro"] <= util.F32_REL, m


def test_a_bounded_wait_that_runs_out_is_reported_and_survivable(dev, pkg):
    """A one-CTA kernel waits 2 ms on a barrier nobody arrives at.  The wait gives up on its own: the kernel
    returns normally, the status word carries 0x1000 | site, the next synchronise raises the timeout error and
    clears the word, and the device goes on working.  Nothing traps, faults or spins without a limit."""
    import ctypes as C
    capi = pkg.capi
    assert dev.status() == 0
    seen = (C.c_uint32 * 2)()
    pkg.hal.check(capi.lib().tsm100_selftest_wait_timeout(dev._h, 2000, seen, None))
    assert seen[0] == 2             # both waiting threads left through the failure path
    assert 2000 <= seen[1] < 200000  # the first one after its 2 ms limit, not after the library's 2 s
    with pytest.raises(pkg.hal.RuntimeError_, match="0x103f"):
        pkg.hal.check(capi.lib().tsm100_stream_synchronize(dev._h, None))
    pkg.hal.check(capi.lib().tsm100_stream_synchronize(dev._h, None))  # reported once, then clear
    # a second expiry is reported through tsm100_device_status, and a real kernel runs right after it
    pkg.hal.check(capi.lib().tsm100_selftest_wait_timeout(dev._h, 1000, None, None))
    assert dev.status() == 0x1000 | 63
    assert dev.status() == 0
    x = util.softmax_input(capi, 64, 4096)
    xd = util.dev_tensor(torch, x)
    yd = torch.empty_like(xd)
    dev.softmax(capi.F32, 64, 4096, xd.data_ptr(), yd.data_ptr(), stream=util.cur_stream(torch))
    torch.cuda.synchronize()
    assert dev.status() == 0
    assert float((yd.sum(dim=1) - 1).abs().max()) < 1e-5
