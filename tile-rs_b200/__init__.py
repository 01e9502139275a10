"""tile-rs_b200: the sm_100a (B200) hot path of tile-rs — matmul, row softmax and
fused attention — behind the reference's two plugin seams.

* ``capi``    ctypes binding of ``include/tile_sm100.h`` (the C-ABI drop-in boundary)
* ``hal``     host-side mirror of ``tile_hal`` (Device / Stream / DeviceBuffer /
              KernelLauncher / BackendSelector / HalError) over that ABI
* ``codegen`` host-side mirror of ``tile_codegen`` (CodegenTarget / TargetRegistry)
              with the ``cuda_sm100`` target
* ``launcher`` the multi-GPU launcher (``tsm100_multi_run``) and the shard rule it and the
              process-per-GPU form share
* ``build``   nvcc recipe for ``libtile_sm100.so``

The directory name carries a hyphen, so it is imported under the module name
``tile_rs_b200`` (see ``__graft_entry__.load_package``).  There is no CPU
fallback anywhere in this package: compute calls fail with ``HalError`` when no
CUDA device is present.
"""
from . import build, capi, codegen, hal, launcher  # noqa: F401

__all__ = ["build", "capi", "codegen", "hal", "launcher"]
