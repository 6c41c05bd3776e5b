"""`ttrt.runtime._ttmlir_runtime.binary`: the names runtime/python/binary/binary.cpp registers
(Flatbuffer, Binary, SystemDesc, GoldenTensor, load_*), over the C ABI."""

from . import api

GoldenTensor = api.GoldenTensor


class Flatbuffer(api.Binary):
    """binary.cpp:19-28.  version / schema_hash / ttmlir_git_hash / file_identifier are properties,
    check_schema_hash / as_json / store methods -- all inherited from the ctypes Binary."""


class Binary(Flatbuffer):
    """binary.cpp:30-52 (the program queries are inherited as well)."""


class SystemDesc(Flatbuffer):
    """binary.cpp:54-64."""


def _adopt(cls, b):
    out = cls(b._h)
    b._h = None          # ownership of the handle moves to the new wrapper
    return out


def load_from_path(path: str) -> Flatbuffer:
    return _adopt(Flatbuffer, api.Binary.load_from_path(path))


def load_binary_from_path(path: str) -> Binary:
    return _adopt(Binary, api.Binary.load_from_path(path))


def load_binary_from_bytes(data: bytes) -> Binary:
    return _adopt(Binary, api.Binary.load_from_memory(bytes(data)))


def load_binary_from_capsule(capsule) -> Binary:
    """The reference unwraps a PyCapsule holding a shared_ptr made by the compiler's Python bindings
    (binary.cpp:68-72).  Without those bindings the only portable hand-over is the serialized bytes."""
    if isinstance(capsule, (bytes, bytearray, memoryview)):
        return load_binary_from_bytes(bytes(capsule))
    raise TypeError("load_binary_from_capsule: pass the flatbuffer's bytes (no compiler bindings are loaded in this process)")


def load_system_desc_from_path(path: str) -> SystemDesc:
    return _adopt(SystemDesc, api.Binary.load_from_path(path))
