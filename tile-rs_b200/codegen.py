"""Host-side mirror of the reference's ``tile_codegen`` crate with the
``cuda_sm100`` target.

* ``CodegenTarget`` / ``EmitOpts`` / ``EmitOut`` / ``TargetMeta`` / ``HardwareParams``
  crates/tile_codegen/src/target.rs:17-65
* ``TargetRegistry``   crates/tile_codegen/src/registry.rs:21-68
* ``DebugTarget`` / ``EmitterTarget``  crates/tile_codegen/src/targets.rs:32-102
* ``TileKernel`` / ``TileOp`` (the descriptor "the compiler emits alongside the compiled
  binary")  crates/tile_hal/src/kernel.rs:93-212

``CudaSm100Target.emit`` forwards to the C ABI's ``tsm100_emit`` (C++), so the
Rust implementation of the trait is the same few lines of forwarding.
"""
from __future__ import annotations

import ctypes as C
import json
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional

from . import capi


@dataclass(frozen=True)
class HardwareParams:
    ub_size: int = 0


@dataclass(frozen=True)
class EmitOpts:
    hw: HardwareParams = HardwareParams()


@dataclass(frozen=True)
class TileOp:
    """One ``TileOp`` of tile_hal (kernel.rs:93-158): the variant name and its fields."""
    op: str
    params: Dict[str, object] = field(default_factory=dict)


@dataclass(frozen=True)
class ArgInfo:
    """What a launcher needs to validate one pointer argument of a kernel."""
    index: int
    role: str                # "input" | "output" | "unused"
    dtype: str               # "F32" | "F16" | "BF16"
    elements_per_block: int

    def bytes_for(self, blocks: int) -> int:
        return blocks * self.elements_per_block * (4 if self.dtype == "F32" else 2)


@dataclass
class TileKernel:
    """``TileKernel`` of tile_hal (kernel.rs:160-212): the descriptor the compiler emits beside the binary."""
    name: str
    ops: List[TileOp]
    num_inputs: int
    num_outputs: int
    mode: str                # "Vector" | "Matrix" | "General"
    args: List[ArgInfo] = field(default_factory=list)

    def uses_matmul(self) -> bool:
        return any(o.op == "Matmul" for o in self.ops)

    def inferred_mode(self) -> str:
        return "General" if self.uses_matmul() else "Vector"


@dataclass
class TargetMeta:
    has_cube_kernel: bool = False
    kernel_names: List[str] = field(default_factory=list)
    kernels: List[TileKernel] = field(default_factory=list)   # one descriptor per entry kernel (cuda_sm100 only)


@dataclass
class EmitOut:
    source: str
    ext: str
    meta: TargetMeta = field(default_factory=TargetMeta)


class EmitError(Exception):
    """The ``Err(String)`` of ``CodegenTarget::emit``."""


class CodegenTarget:
    def name(self) -> str:
        raise NotImplementedError

    def emit(self, mlir_text: str, opts: EmitOpts = EmitOpts()) -> EmitOut:
        raise NotImplementedError


class DebugTarget(CodegenTarget):
    """targets.rs:32-53: echoes the module inside a banner."""

    def name(self) -> str:
        return "debug"

    def emit(self, mlir_text: str, opts: EmitOpts = EmitOpts()) -> EmitOut:
        if not mlir_text.strip():
            raise EmitError("empty MLIR module")
        lines = len(mlir_text.splitlines())
        funcs = mlir_text.count("func.func")
        return EmitOut(f"// tile-rs debug target\n// {lines} MLIR lines, {funcs} func.func op(s)\n{mlir_text}\n",
                       "mlir.txt", TargetMeta())


class EmitterTarget(CodegenTarget):
    """targets.rs:82-102: lifts a plain ``(mlir) -> source`` function into a target."""

    def __init__(self, name: str, ext: str, f: Callable[[str], str]):
        self._name, self._ext, self._f = name, ext, f

    def name(self) -> str:
        return self._name

    def emit(self, mlir_text: str, opts: EmitOpts = EmitOpts()) -> EmitOut:
        return EmitOut(self._f(mlir_text), self._ext, TargetMeta())


class CudaSm100Target(CodegenTarget):
    """The new target: MLIR text -> a CUDA translation unit that instantiates the
    hand-written sm_100a kernels for the shapes the module carries."""

    def name(self) -> str:
        return capi.lib().tsm100_target_name().decode()

    def emit(self, mlir_text: str, opts: EmitOpts = EmitOpts()) -> EmitOut:
        lib = capi.lib()
        raw = mlir_text.encode()
        src_len, names_len = C.c_size_t(), C.c_size_t()
        src_cap, names_cap = max(4096, 2 * len(raw) + 4096), 1024
        while True:
            src, names = C.create_string_buffer(src_cap), C.create_string_buffer(names_cap)
            st = lib.tsm100_emit(raw, len(raw), src, src_cap, C.byref(src_len), names, names_cap, C.byref(names_len))
            if st == capi.ERR_BUFFER:
                src_cap, names_cap = max(src_cap, src_len.value + 1), max(names_cap, names_len.value + 1)
                continue
            if st != capi.OK:
                raise EmitError(capi.last_error())
            break
        kernel_names = [n for n in names.value.decode().split("\n") if n]
        return EmitOut(src.value.decode(), lib.tsm100_target_ext().decode(),
                       TargetMeta(False, kernel_names, self.describe(mlir_text)))

    def describe(self, mlir_text: str) -> List[TileKernel]:
        """The TileKernel descriptors of the module's entry kernels."""
        lib = capi.lib()
        raw = mlir_text.encode()
        n = C.c_size_t()
        cap = max(4096, 4 * len(raw))
        while True:
            buf = C.create_string_buffer(cap)
            st = lib.tsm100_emit_descriptors(raw, len(raw), buf, cap, C.byref(n))
            if st == capi.ERR_BUFFER:
                cap = n.value + 1
                continue
            if st != capi.OK:
                raise EmitError(capi.last_error())
            break
        out = []
        for k in json.loads(buf.value.decode()):
            ops = [TileOp(o["op"], {f: v for f, v in o.items() if f != "op"}) for o in k["ops"]]
            args = [ArgInfo(a["index"], a["role"], a["dtype"], a["elements_per_block"]) for a in k["args"]]
            out.append(TileKernel(k["name"], ops, k["num_inputs"], k["num_outputs"], k["mode"], args))
        return out


class TargetRegistry:
    def __init__(self) -> None:
        self._targets: List[CodegenTarget] = []

    @staticmethod
    def new() -> "TargetRegistry":
        return TargetRegistry()

    @staticmethod
    def with_builtin() -> "TargetRegistry":
        r = TargetRegistry()
        r.register(DebugTarget())
        r.register(CudaSm100Target())
        return r

    def register(self, target: CodegenTarget) -> None:
        self._targets.append(target)

    def select(self, name: str) -> Optional[CodegenTarget]:
        """First match wins (registry.rs:42-52)."""
        for t in self._targets:
            if t.name() == name:
                return t
        return None

    def names(self) -> List[str]:
        return [t.name() for t in self._targets]

    def len(self) -> int:
        return len(self._targets)

    def __len__(self) -> int:
        return len(self._targets)

    def is_empty(self) -> bool:
        return not self._targets
