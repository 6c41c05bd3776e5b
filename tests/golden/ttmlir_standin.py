"""Stand-ins for the compiler's Python bindings (`ttmlir`), just enough to IMPORT the reference's
tools/golden/mapping.py outside a tt-mlir build.

mapping.py holds the torch goldens of every op; its only dependency beyond torch / numpy /
einops is `ttmlir` (MLIR attribute and type classes, dialect op classes used as dictionary keys).
The goldens themselves unwrap attributes with `unpack_mlir_attr(attr)` (`.value`, `list(attr)`)
and map element types with `mlir_type_to_torch_dtype(type)` (`isinstance` checks and `str()`), so
attribute classes that carry a value and type classes that print their MLIR spelling are all
they need.  Dialect modules hand out an empty class for any op name asked of them.

Only tests/golden/generate.py uses this, in the container where the reference checkout exists.
"""

import enum
import sys
import types

import numpy as np


class _AutoClassModule(types.ModuleType):
    """A module whose every attribute is a (cached) empty class named after the attribute."""

    def __getattr__(self, name):
        if name.startswith("__"):
            raise AttributeError(name)
        cls = type(name, (), {})
        setattr(self, name, cls)
        return cls


class _ValueAttr:
    def __init__(self, value):
        self.value = value

    @classmethod
    def get(cls, value, *a, **k):
        return cls(value)

    @classmethod
    def maybe_downcast(cls, attr):
        return attr


class IntegerAttr(_ValueAttr):
    pass


class BoolAttr(_ValueAttr):
    pass


class FloatAttr(_ValueAttr):
    pass


class StringAttr(_ValueAttr):
    pass


class ArrayAttr(list):
    pass


class DenseI64ArrayAttr(list):
    pass


class DenseI32ArrayAttr(list):
    pass


class DenseBoolArrayAttr(list):
    pass


class DenseElementsAttr:
    def __init__(self, array):
        self.array = np.asarray(array)

    def __array__(self, dtype=None, copy=None):
        return self.array if dtype is None else self.array.astype(dtype)


class Type:
    """An element type that prints as its MLIR spelling ("bf16", "f32", "si8", "i32" ...)."""

    def __init__(self, spelling):
        self.spelling = spelling

    def __str__(self):
        return self.spelling


class BF16Type(Type):
    def __init__(self):
        super().__init__("bf16")


class F16Type(Type):
    def __init__(self):
        super().__init__("f16")


class F32Type(Type):
    def __init__(self):
        super().__init__("f32")


class F64Type(Type):
    def __init__(self):
        super().__init__("f64")


class IntegerType(Type):
    def __init__(self, width, signed=True, unsigned=False):
        super().__init__(("ui" if unsigned else ("si" if signed else "i")) + str(width))
        self.width, self.is_signed, self.is_unsigned = width, signed and not unsigned, unsigned
        self.is_signless = not signed and not unsigned


def type_of(torch_dtype):
    import torch
    return {torch.bfloat16: BF16Type(), torch.float16: F16Type(), torch.float32: F32Type(), torch.float64: F64Type(),
            torch.int8: IntegerType(8), torch.uint8: IntegerType(8, unsigned=True), torch.int32: IntegerType(32),
            torch.int64: IntegerType(64), torch.bool: IntegerType(1)}[torch_dtype]


class ReduceType(enum.Enum):
    Sum = 0
    Mean = 1
    Max = 2
    Min = 3
    Std = 4
    Var = 5
    Prod = 6
    Invalid = 7


class MeshShardType(enum.Enum):
    Identity = 0
    Replicate = 1
    Maximal = 2
    Devices = 3


class MeshShardDirection(enum.Enum):
    FullToShard = 0
    ShardToFull = 1


class ReduceTypeAttr(_ValueAttr):
    pass


class MeshShardTypeAttr(_ValueAttr):
    pass


class MeshShardDirectionAttr(_ValueAttr):
    pass


def install():
    """Registers the stand-in `ttmlir` package in sys.modules (no-op if a real one is importable)."""
    try:
        import ttmlir  # noqa: F401
        if not getattr(ttmlir, "_is_standin", False):
            return
    except ImportError:
        pass
    pkg = types.ModuleType("ttmlir")
    pkg.__path__ = []
    pkg._is_standin = True
    dialects = types.ModuleType("ttmlir.dialects")
    dialects.__path__ = []
    mods = {"ttmlir": pkg, "ttmlir.dialects": dialects}
    for name in ("ttir", "stablehlo", "d2m", "ttnn", "ttcore", "sdy", "debug", "func"):
        m = _AutoClassModule("ttmlir.dialects." + name)
        setattr(dialects, name, m)
        mods[m.__name__] = m
    core_ir = _AutoClassModule("ttmlir.dialects.ttcore.ir")
    for cls in (ReduceType, MeshShardType, MeshShardDirection, ReduceTypeAttr, MeshShardTypeAttr, MeshShardDirectionAttr):
        setattr(core_ir, cls.__name__, cls)
    dialects.ttcore.ir = core_ir
    ir = _AutoClassModule("ttmlir.ir")
    exported = [IntegerAttr, BoolAttr, FloatAttr, StringAttr, ArrayAttr, DenseI64ArrayAttr, DenseI32ArrayAttr,
                DenseBoolArrayAttr, DenseElementsAttr, Type, BF16Type, F16Type, F32Type, F64Type, IntegerType]
    for cls in exported:
        setattr(ir, cls.__name__, cls)
    ir.np = np   # mapping.py reaches numpy through this star import
    ir.__all__ = [c.__name__ for c in exported] + ["np", "I64ElementsAttr", "Attribute", "Operation", "OpView", "Value",
                                                   "RankedTensorType", "Context", "Location"]
    passes = _AutoClassModule("ttmlir.passes")
    pkg.dialects, pkg.ir, pkg.passes = dialects, ir, passes
    mods.update({"ttmlir.ir": ir, "ttmlir.passes": passes})
    sys.modules.update(mods)


def load_mapping(reference_root):
    """Imports <reference_root>/tools/golden/mapping.py (unmodified) and returns the module."""
    import importlib.util
    import os
    install()
    path = os.path.join(reference_root, "tools", "golden", "mapping.py")
    spec = importlib.util.spec_from_file_location("tt_mlir_reference_golden_mapping", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod
