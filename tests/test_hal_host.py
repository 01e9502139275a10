"""Host logic of the tile_hal mirror.  These follow the reference's own HAL unit
tests (crates/tile_hal/src/lib.rs:42-675): the codegen-path table, environment
selection, LaunchGrid builders and the Display text of HalError."""
import pytest


def test_from_codegen_path_table(pkg):
    K = pkg.hal.BackendKind
    table = {"cpp": K.Ascend, "pto": K.Ascend, "gpu": K.Cuda, "musa": K.Musa, "aie": K.Aie, "nki": K.Nki,
             "spirv": K.Spirv, "msl": K.Msl, "bang": K.Bang, "gaudi": K.Gaudi}
    for path, kind in table.items():
        assert K.from_codegen_path(path) is kind
    assert K.from_codegen_path("cuda_sm100") is K.Cuda  # the one added arm
    for unknown in ("", "linalg", "debug", "CUDA", "gpu "):
        assert K.from_codegen_path(unknown) is None
    assert K.Cuda.codegen_path() == "gpu" and K.Ascend.codegen_path() == "cpp"


def test_selector_from_env(pkg, monkeypatch):
    hal = pkg.hal
    monkeypatch.delenv("TILERS_CODEGEN_PATH", raising=False)
    monkeypatch.delenv("ACLRS_CODEGEN_PATH", raising=False)
    assert hal.BackendSelector.from_env().kind() is hal.BackendKind.Ascend  # default "cpp"
    monkeypatch.setenv("ACLRS_CODEGEN_PATH", "gpu")
    assert hal.BackendSelector.from_env().kind() is hal.BackendKind.Cuda
    monkeypatch.setenv("TILERS_CODEGEN_PATH", "cuda_sm100")  # takes precedence over the legacy variable
    assert hal.BackendSelector.from_env().kind() is hal.BackendKind.Cuda
    monkeypatch.setenv("TILERS_CODEGEN_PATH", "nonsense")
    with pytest.raises(hal.BackendNotAvailable) as e:
        hal.BackendSelector.from_env()
    assert str(e.value) == "backend not available: unknown codegen path: nonsense"


def test_backend_not_compiled(pkg):
    hal = pkg.hal
    with pytest.raises(hal.BackendNotAvailable) as e:
        hal.BackendSelector(hal.BackendKind.Msl).device(0)
    assert "Msl backend not compiled" in str(e.value)


def test_launch_grid_builders(pkg):
    G = pkg.hal.LaunchGrid
    g = G.blocks_(8)
    assert (g.blocks, g.threads_per_block, g.shared_mem_bytes) == (8, 1, 0)
    g = G.cuda(4, 256).with_shared_mem(4096)
    assert (g.blocks, g.threads_per_block, g.shared_mem_bytes) == (4, 256, 4096)


def test_hal_error_display(pkg):
    hal = pkg.hal
    assert str(hal.DeviceError("x")) == "device error: x"
    assert str(hal.MemoryError_("x")) == "memory error: x"
    assert str(hal.KernelError("x")) == "kernel error: x"
    assert str(hal.StreamError("x")) == "stream error: x"
    assert str(hal.BackendNotAvailable("x")) == "backend not available: x"
    assert str(hal.RuntimeError_("x")) == "runtime error: x"
    assert all(issubclass(c, hal.HalError) for c in (hal.DeviceError, hal.KernelError, hal.BackendNotAvailable))


def test_status_codes_map_to_error_variants(pkg):
    hal, capi = pkg.hal, pkg.capi
    hal.check(capi.OK)
    for code, exc in ((capi.ERR_INVALID, hal.KernelError), (capi.ERR_NO_DEVICE, hal.BackendNotAvailable),
                      (capi.ERR_MEMORY, hal.MemoryError_), (capi.ERR_LAUNCH, hal.KernelError),
                      (capi.ERR_STREAM, hal.StreamError), (capi.ERR_RUNTIME, hal.RuntimeError_),
                      (capi.ERR_TIMEOUT, hal.RuntimeError_)):
        with pytest.raises(exc):
            hal.check(code)
