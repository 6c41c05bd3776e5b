"""Python face of the B200 runtime target, bound with ctypes over the C ABI in include/ttb_runtime.h.

Names and call shapes follow the reference's nanobind module (`ttrt.runtime` / `ttrt.binary`,
runtime/python/runtime/runtime.cpp and runtime/python/binary/binary.cpp), so a script written
for ttrt reads the same here:

    binary = Binary.load_from_path("model.ttnn")
    set_compatible_device_runtime(binary)
    device = open_mesh_device(MeshDeviceOptions(mesh_shape=[1, 1]))
    t = create_borrowed_host_tensor(x.data_ptr(), shape, stride, itemsize, DataType.BFloat16)
    t = to_layout(t, device, get_layout(binary, 0, 0))
    outs = submit(device, binary, 0, [t])
    host = to_host(outs[0], untilize=True)[0]

The library must have been built (`python tt-mlir_b200/build.py`); importing this module
without it raises.  There is no CPU fallback: every op runs on the GPU or fails.
"""

from __future__ import annotations

import ctypes
import enum
import os
import re
from typing import List, Optional, Sequence

_HERE = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_HERE)
LIB_PATH = os.path.join(_HERE, "lib", "libttb200.so")

if not os.path.exists(LIB_PATH):
    raise ImportError(f"{LIB_PATH} is missing: run `python tt-mlir_b200/build.py` first")

lib = ctypes.CDLL(LIB_PATH)


class DataType(enum.IntEnum):
    """tt::target::DataType (include/ttmlir/Target/Common/types.fbs:19-42)."""
    Float32 = 0
    Float16 = 1
    BFloat16 = 2
    UInt32 = 9
    UInt16 = 10
    UInt8 = 11
    Int32 = 12
    Int8 = 17


ITEMSIZE = {DataType.Float32: 4, DataType.Float16: 2, DataType.BFloat16: 2, DataType.UInt32: 4,
            DataType.UInt16: 2, DataType.UInt8: 1, DataType.Int32: 4, DataType.Int8: 1}


def declared_symbols() -> List[str]:
    """Every function declared in include/*.h (what the library promises to export)."""
    names = []
    inc = os.path.join(_ROOT, "include")
    for f in sorted(os.listdir(inc)):
        if f.endswith(".h"):
            text = open(os.path.join(inc, f)).read()
            names += re.findall(r"(?:TTB_API|TTRT_API)\s+[\w\s\*]+?\b(tt(?:b|rt)_\w+)\s*\(", text)
    return names


def check_exports() -> None:
    missing = [n for n in declared_symbols() if not hasattr(lib, n)]
    if missing:
        raise ImportError(f"libttb200.so does not export: {missing}")


check_exports()

lib.ttrt_last_error.restype = ctypes.c_char_p
lib.ttb_last_error.restype = ctypes.c_char_p
lib.ttb_launch_count.restype = ctypes.c_uint64
lib.ttb_dtype_size.restype = ctypes.c_size_t
lib.ttb_conv2d_workspace_bytes.restype = ctypes.c_size_t
lib.ttrt_free_string.argtypes = [ctypes.c_void_p]
lib.ttrt_perf_emitted.restype = ctypes.c_uint64
for _n in ("ttrt_binary_free", "ttrt_device_free", "ttrt_tensor_free", "ttrt_layout_free", "ttrt_tensor_ref_free"):
    getattr(lib, _n).argtypes = [ctypes.c_void_p]
    getattr(lib, _n).restype = None


class RuntimeError_(RuntimeError):
    pass


def _check(rc: int) -> None:
    if rc != 0:
        raise RuntimeError_(lib.ttrt_last_error().decode("utf-8", "replace"))


def _vp(x) -> ctypes.c_void_p:
    return ctypes.c_void_p(x)


def launch_count() -> int:
    """Kernels launched by the library in this process so far."""
    return int(lib.ttb_launch_count())


# ---------------------------------------------------------------------------------- Binary
class Binary:
    def __init__(self, handle: int):
        self._h = handle

    def __del__(self):
        if getattr(self, "_h", None) and lib is not None:  # module globals are gone at interpreter exit
            lib.ttrt_binary_free(self._h)
            self._h = None

    @staticmethod
    def load_from_path(path: str) -> "Binary":
        h = ctypes.c_void_p()
        _check(lib.ttrt_binary_load_from_path(path.encode(), ctypes.byref(h)))
        return Binary(h.value)

    @staticmethod
    def load_from_memory(data: bytes) -> "Binary":
        h = ctypes.c_void_p()
        _check(lib.ttrt_binary_load_from_memory(data, ctypes.c_size_t(len(data)), ctypes.byref(h)))
        return Binary(h.value)

    def store(self, path: str) -> None:
        _check(lib.ttrt_binary_store(_vp(self._h), path.encode()))

    @property
    def file_identifier(self) -> str:
        buf = ctypes.create_string_buffer(5)
        _check(lib.ttrt_binary_file_identifier(_vp(self._h), buf))
        return buf.value.decode()

    @property
    def version(self) -> str:
        buf = ctypes.create_string_buffer(64)
        _check(lib.ttrt_binary_version(_vp(self._h), buf, ctypes.c_size_t(64)))
        return buf.value.decode()

    @property
    def id(self) -> int:
        v = ctypes.c_uint64()
        _check(lib.ttrt_binary_id(_vp(self._h), ctypes.byref(v)))
        return v.value

    def check_schema_hash(self) -> bool:
        ok = ctypes.c_int()
        _check(lib.ttrt_binary_check_schema_hash(_vp(self._h), ctypes.byref(ok)))
        return bool(ok.value)

    def as_json(self) -> str:
        p = ctypes.c_void_p()
        _check(lib.ttrt_binary_as_json(_vp(self._h), ctypes.byref(p)))
        try:
            return ctypes.string_at(p.value).decode("utf-8", "replace")
        finally:
            lib.ttrt_free_string(p)

    def get_program_ops_as_json(self, program_index: int) -> str:
        p = ctypes.c_void_p()
        _check(lib.ttrt_binary_program_ops_as_json(_vp(self._h), ctypes.c_uint32(program_index), ctypes.byref(p)))
        try:
            return ctypes.string_at(p.value).decode("utf-8", "replace")
        finally:
            lib.ttrt_free_string(p)

    def get_num_programs(self) -> int:
        n = ctypes.c_uint32()
        _check(lib.ttrt_binary_num_programs(_vp(self._h), ctypes.byref(n)))
        return n.value

    def get_program_name(self, program_index: int) -> str:
        buf = ctypes.create_string_buffer(256)
        _check(lib.ttrt_binary_program_name(_vp(self._h), ctypes.c_uint32(program_index), buf, ctypes.c_size_t(256)))
        return buf.value.decode()

    def is_program_private(self, program_index: int) -> bool:
        v = ctypes.c_int()
        _check(lib.ttrt_binary_is_program_private(_vp(self._h), ctypes.c_uint32(program_index), ctypes.byref(v)))
        return bool(v.value)

    def get_num_program_inputs(self, program_index: int) -> int:
        n = ctypes.c_uint32()
        _check(lib.ttrt_binary_num_program_inputs(_vp(self._h), ctypes.c_uint32(program_index), ctypes.byref(n)))
        return n.value

    def get_num_program_outputs(self, program_index: int) -> int:
        n = ctypes.c_uint32()
        _check(lib.ttrt_binary_num_program_outputs(_vp(self._h), ctypes.c_uint32(program_index), ctypes.byref(n)))
        return n.value

    def _io_desc(self, program_index: int, is_output: bool, index: int):
        rank = ctypes.c_uint32()
        shape = (ctypes.c_uint32 * 8)()
        dt = ctypes.c_int()
        _check(lib.ttrt_binary_program_io_desc(_vp(self._h), ctypes.c_uint32(program_index), int(is_output),
                                               ctypes.c_uint32(index), ctypes.byref(rank), shape, ctypes.byref(dt)))
        return list(shape[:rank.value]), DataType(dt.value)

    def get_program_inputs(self, program_index: int):
        return [self._io_desc(program_index, False, i) for i in range(self.get_num_program_inputs(program_index))]

    def get_program_outputs(self, program_index: int):
        return [self._io_desc(program_index, True, i) for i in range(self.get_num_program_outputs(program_index))]

    def get_program_mesh_shape(self, program_index: int):
        y, x = ctypes.c_uint32(), ctypes.c_uint32()
        _check(lib.ttrt_binary_program_mesh_shape(_vp(self._h), ctypes.c_uint32(program_index), ctypes.byref(y),
                                                  ctypes.byref(x)))
        return (y.value, x.value)

    def _query(self, what: int, program_index: int = 0) -> str:
        p = ctypes.c_void_p()
        _check(lib.ttrt_binary_query_string(_vp(self._h), what, ctypes.c_uint32(program_index), ctypes.byref(p)))
        try:
            return ctypes.string_at(p.value).decode("utf-8", "replace")
        finally:
            lib.ttrt_free_string(p)

    def get_program_inputs_as_json(self, program_index: int) -> str:
        return self._query(0, program_index)

    def get_program_outputs_as_json(self, program_index: int) -> str:
        return self._query(1, program_index)

    def get_mlir_as_json(self) -> str:
        return self._query(2)

    def get_system_desc_as_json(self) -> str:
        return self._query(3)

    @property
    def schema_hash(self) -> str:
        return self._query(4)

    @property
    def ttmlir_git_hash(self) -> str:
        return self._query(5)

    def get_debug_info_golden(self, loc: str):
        """The golden tensors the compiler embedded under `loc` (Binary::getDebugInfoGolden): a dict
        device id -> GoldenTensor; empty when the binary carries none for that location."""
        n = ctypes.c_uint32()
        _check(lib.ttrt_binary_golden_devices(_vp(self._h), loc.encode(), None, 0, ctypes.byref(n)))
        if n.value == 0:
            return {}
        devs = (ctypes.c_uint32 * n.value)()
        _check(lib.ttrt_binary_golden_devices(_vp(self._h), loc.encode(), devs, n, ctypes.byref(n)))
        out = {}
        for d in devs:
            rank, dt = ctypes.c_uint32(), ctypes.c_int()
            shape, stride = (ctypes.c_int64 * 8)(), (ctypes.c_int64 * 8)()
            data, size = ctypes.c_void_p(), ctypes.c_size_t()
            _check(lib.ttrt_binary_golden_tensor(_vp(self._h), loc.encode(), ctypes.c_uint32(d), ctypes.byref(rank), shape, stride,
                                                 ctypes.byref(dt), ctypes.byref(data), ctypes.byref(size)))
            out[int(d)] = GoldenTensor(loc, list(shape[:rank.value]), list(stride[:rank.value]), DataType(dt.value),
                                       ctypes.string_at(data.value, size.value) if data.value else b"")
        return out


class GoldenTensor:
    """A tensor the compiler stored in a binary's debug info (tt.target.GoldenTensor)."""

    def __init__(self, name, shape, stride, dtype, data: bytes):
        self.name, self.shape, self.stride, self.dtype, self._data = name, shape, stride, dtype, data

    def get_data_buffer(self) -> bytearray:
        return bytearray(self._data)


# ---------------------------------------------------------------------------------- Device
class MeshDeviceOptions:
    def __init__(self, mesh_shape: Optional[Sequence[int]] = None, device_ids: Optional[Sequence[int]] = None,
                 process_rank: int = 0, process_count: int = 1, nccl_unique_id: Optional[bytes] = None):
        self.mesh_shape = list(mesh_shape) if mesh_shape is not None else [1, 1]
        self.device_ids = list(device_ids) if device_ids is not None else []
        self.process_rank = process_rank
        self.process_count = process_count
        self.nccl_unique_id = nccl_unique_id


class Device:
    def __init__(self, handle: int):
        self._h = handle

    def __del__(self):
        if getattr(self, "_h", None) and lib is not None:  # module globals are gone at interpreter exit
            lib.ttrt_device_free(self._h)
            self._h = None

    def get_mesh_shape(self):
        y, x = ctypes.c_uint32(), ctypes.c_uint32()
        _check(lib.ttrt_device_mesh_shape(_vp(self._h), ctypes.byref(y), ctypes.byref(x)))
        return [y.value, x.value]

    def get_device_ids(self) -> List[int]:
        n = ctypes.c_uint32()
        _check(lib.ttrt_device_ids(_vp(self._h), None, 0, ctypes.byref(n)))
        ids = (ctypes.c_int * max(n.value, 1))()
        _check(lib.ttrt_device_ids(_vp(self._h), ids, n, ctypes.byref(n)))
        return list(ids[:n.value])

    def num_local(self) -> int:
        n = ctypes.c_uint32()
        _check(lib.ttrt_device_num_local(_vp(self._h), ctypes.byref(n)))
        return n.value

    def stream(self, index: int = 0):
        """(cudaStream_t as int, CUDA device ordinal) of local coordinate `index`."""
        s = ctypes.c_void_p()
        d = ctypes.c_int()
        _check(lib.ttrt_device_stream(_vp(self._h), ctypes.c_uint32(index), ctypes.byref(s), ctypes.byref(d)))
        return (s.value or 0), d.value


def get_num_available_devices() -> int:
    n = ctypes.c_size_t()
    _check(lib.ttrt_get_num_available_devices(ctypes.byref(n)))
    return n.value


def get_current_system_desc(device: Optional["Device"] = None) -> Binary:
    """The machine (or `device`) described in the reference's system-descriptor format: a "TTSY"
    flatbuffer with as_json / store / version / file_identifier."""
    h = ctypes.c_void_p()
    _check(lib.ttrt_get_current_system_desc(_vp(device._h) if device is not None else None, ctypes.byref(h)))
    return Binary(h.value)


def create_sub_mesh_device(parent: "Device", mesh_shape: Sequence[int], mesh_offset: Optional[Sequence[int]] = None) -> "Device":
    h = ctypes.c_void_p()
    off = list(mesh_offset) if mesh_offset is not None else [0, 0]
    _check(lib.ttrt_create_sub_mesh_device(_vp(parent._h), ctypes.c_uint32(mesh_shape[0]), ctypes.c_uint32(mesh_shape[1]),
                                           int(mesh_offset is not None), ctypes.c_uint32(off[0]), ctypes.c_uint32(off[1]),
                                           ctypes.byref(h)))
    return Device(h.value)


def release_sub_mesh_device(sub: "Device") -> None:
    _check(lib.ttrt_release_sub_mesh_device(_vp(sub._h)))


def reshape_mesh_device(device: "Device", mesh_shape: Sequence[int]) -> None:
    _check(lib.ttrt_reshape_mesh_device(_vp(device._h), ctypes.c_uint32(mesh_shape[0]), ctypes.c_uint32(mesh_shape[1])))


def get_nccl_unique_id() -> bytes:
    buf = ctypes.create_string_buffer(128)
    _check(lib.ttrt_get_nccl_unique_id(buf))
    return buf.raw


def set_compatible_device_runtime(binary: Binary) -> None:
    _check(lib.ttrt_set_compatible_device_runtime(_vp(binary._h)))


def open_mesh_device(options: Optional[MeshDeviceOptions] = None) -> Device:
    o = options or MeshDeviceOptions()
    ids = (ctypes.c_int * len(o.device_ids))(*o.device_ids) if o.device_ids else None
    h = ctypes.c_void_p()
    nid = o.nccl_unique_id
    if nid is not None and len(nid) != 128:
        raise ValueError("nccl_unique_id must be 128 bytes")
    _check(lib.ttrt_open_mesh_device(ctypes.c_uint32(o.mesh_shape[0]), ctypes.c_uint32(o.mesh_shape[1]), ids,
                                     ctypes.c_uint32(len(o.device_ids)), ctypes.c_uint32(o.process_rank),
                                     ctypes.c_uint32(o.process_count), nid, ctypes.byref(h)))
    return Device(h.value)


def close_mesh_device(device: Device) -> None:
    _check(lib.ttrt_close_mesh_device(_vp(device._h)))


# ---------------------------------------------------------------------------------- Tensor
class Layout:
    def __init__(self, handle: int):
        self._h = handle

    def __del__(self):
        if getattr(self, "_h", None) and lib is not None:  # module globals are gone at interpreter exit
            lib.ttrt_layout_free(self._h)
            self._h = None


class Tensor:
    def __init__(self, handle: int, keepalive=None):
        self._h = handle
        self._keepalive = keepalive  # object owning borrowed memory

    def __del__(self):
        if getattr(self, "_h", None) and lib is not None:  # module globals are gone at interpreter exit
            lib.ttrt_tensor_free(self._h)
            self._h = None

    def _info(self):
        rank = ctypes.c_uint32()
        shape = (ctypes.c_uint32 * 8)()
        dt, st, al = ctypes.c_int(), ctypes.c_int(), ctypes.c_int()
        ns = ctypes.c_uint32()
        _check(lib.ttrt_tensor_info(_vp(self._h), ctypes.byref(rank), shape, ctypes.byref(dt), ctypes.byref(st),
                                    ctypes.byref(ns), ctypes.byref(al)))
        return list(shape[:rank.value]), DataType(dt.value), st.value, ns.value, bool(al.value)

    def get_shape(self):
        return self._info()[0]

    def get_dtype(self) -> DataType:
        return self._info()[1]

    def is_on_device(self) -> bool:
        return self._info()[2] == 1

    def get_num_shards(self) -> int:
        return self._info()[3]

    def host_ptr(self) -> int:
        """Address of a host tensor's data (no copy).  After to_host(..., blocking=False) call
        wait() first."""
        p = ctypes.c_void_p()
        _check(lib.ttrt_tensor_host_ptr(_vp(self._h), ctypes.byref(p)))
        return p.value

    def is_allocated(self) -> bool:
        return self._info()[4]

    def get_volume(self) -> int:
        v = 1
        for d in self.get_shape():
            v *= d
        return v

    def get_element_size(self) -> int:
        return ITEMSIZE[self.get_dtype()]

    def get_retain(self) -> bool:
        v = ctypes.c_int()
        _check(lib.ttrt_tensor_get_retain(_vp(self._h), ctypes.byref(v)))
        return bool(v.value)

    def set_retain(self, retain: bool) -> None:
        _check(lib.ttrt_tensor_set_retain(_vp(self._h), int(retain)))

    def get_data_buffer(self) -> bytes:
        n = self.get_volume() * self.get_element_size()
        buf = ctypes.create_string_buffer(n)
        _check(lib.ttrt_memcpy_to_ptr(buf, _vp(self._h), -1))
        return buf.raw


def _dims(shape, stride):
    rank = len(shape)
    return (ctypes.c_uint32 * max(rank, 1))(*shape), (ctypes.c_int64 * max(rank, 1))(*stride), rank


def create_borrowed_host_tensor(data_ptr: int, shape, stride, itemsize: int, dtype: DataType, keepalive=None) -> Tensor:
    s, st, rank = _dims(shape, stride)
    h = ctypes.c_void_p()
    _check(lib.ttrt_create_borrowed_host_tensor(_vp(data_ptr), s, st, ctypes.c_uint32(rank), ctypes.c_uint32(itemsize),
                                                int(dtype), ctypes.byref(h)))
    return Tensor(h.value, keepalive)


def create_owned_host_tensor(data_ptr: int, shape, stride, itemsize: int, dtype: DataType) -> Tensor:
    s, st, rank = _dims(shape, stride)
    h = ctypes.c_void_p()
    _check(lib.ttrt_create_owned_host_tensor(_vp(data_ptr), s, st, ctypes.c_uint32(rank), ctypes.c_uint32(itemsize),
                                             int(dtype), ctypes.byref(h)))
    return Tensor(h.value)


def create_multi_device_host_tensor_from_shards(shards: Sequence[Tensor], strategy: dict, mesh_shape) -> Tensor:
    arr = (ctypes.c_void_p * len(shards))(*[s._h for s in shards])
    h = ctypes.c_void_p()
    _check(lib.ttrt_create_multi_device_host_tensor(arr, ctypes.c_uint32(len(shards)), ctypes.c_uint32(mesh_shape[0]),
                                                    ctypes.c_uint32(mesh_shape[1]), ctypes.byref(h)))
    return Tensor(h.value, keepalive=list(shards))


def get_layout(binary: Binary, program_index: int, input_index: int) -> Layout:
    h = ctypes.c_void_p()
    _check(lib.ttrt_get_layout(_vp(binary._h), ctypes.c_uint32(program_index), ctypes.c_uint32(input_index),
                               ctypes.byref(h)))
    return Layout(h.value)


def to_layout(tensor: Tensor, device: Device, layout: Layout, retain: Optional[bool] = None) -> Tensor:
    h = ctypes.c_void_p()
    r = -1 if retain is None else int(retain)
    _check(lib.ttrt_to_layout(_vp(tensor._h), _vp(device._h), _vp(layout._h), r, ctypes.byref(h)))
    return Tensor(h.value)


def has_layout(tensor: Tensor, layout: Layout) -> bool:
    v = ctypes.c_int()
    _check(lib.ttrt_has_layout(_vp(tensor._h), _vp(layout._h), ctypes.byref(v)))
    return bool(v.value)


def to_host(tensor: Tensor, untilize: bool = False, blocking: bool = True) -> List[Tensor]:
    cap = 64
    arr = (ctypes.c_void_p * cap)()
    n = ctypes.c_uint32()
    _check(lib.ttrt_to_host(_vp(tensor._h), int(untilize), int(blocking), arr, ctypes.c_uint32(cap), ctypes.byref(n)))
    return [Tensor(arr[i]) for i in range(n.value)]


def memcpy(dst, src: Tensor, dtype: Optional[DataType] = None) -> None:
    """memcpy(ptr:int, Tensor[, dtype]) copies to host memory; memcpy(Tensor, Tensor) copies tensors."""
    if isinstance(dst, Tensor):
        _check(lib.ttrt_memcpy_tensor(_vp(dst._h), _vp(src._h)))
    else:
        _check(lib.ttrt_memcpy_to_ptr(_vp(dst), _vp(src._h), -1 if dtype is None else int(dtype)))


def wait(tensor_or_list) -> None:
    ts = tensor_or_list if isinstance(tensor_or_list, (list, tuple)) else [tensor_or_list]
    for t in ts:
        _check(lib.ttrt_wait_tensor(_vp(t._h)))


def deallocate_tensor(tensor: Tensor, force: bool = False) -> None:
    _check(lib.ttrt_deallocate_tensor(_vp(tensor._h), int(force)))


def submit(device: Device, binary: Binary, program_index: int, inputs: Sequence[Tensor]) -> List[Tensor]:
    n_in = len(inputs)
    arr = (ctypes.c_void_p * max(n_in, 1))(*[t._h for t in inputs])
    cap = 64
    outs = (ctypes.c_void_p * cap)()
    n = ctypes.c_uint32()
    _check(lib.ttrt_submit(_vp(device._h), _vp(binary._h), ctypes.c_uint32(program_index), arr, ctypes.c_uint32(n_in),
                           outs, ctypes.c_uint32(cap), ctypes.byref(n)))
    return [Tensor(outs[i]) for i in range(n.value)]


# ------------------------------------------------------- traces, const-eval cache, counters
def release_trace(device: Device, binary_id: int, main_program_index: int) -> None:
    """ttrt.runtime.release_trace: frees the traces recorded for one main program."""
    _check(lib.ttrt_release_trace(_vp(device._h), ctypes.c_uint64(binary_id), ctypes.c_size_t(main_program_index)))


def const_eval_cache_size() -> int:
    n = ctypes.c_size_t()
    _check(lib.ttrt_const_eval_cache_size(ctypes.byref(n)))
    return n.value


def clear_const_eval_cache() -> None:
    _check(lib.ttrt_const_eval_cache_clear())


def get_stat(name: str) -> int:
    """ttrt.runtime.DebugStats.get().get_stat(name)."""
    v = ctypes.c_int64()
    _check(lib.ttrt_stat_get(name.encode(), ctypes.byref(v)))
    return v.value


def clear_stats() -> None:
    _check(lib.ttrt_stats_clear())


# ---------------------------------------------------------------------------------- hooks
_OP_CB = ctypes.CFUNCTYPE(None, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p)


class OpContext:
    def __init__(self, ptr):
        self._p = ptr


class CallbackContext:
    def __init__(self, ptr):
        self._p = ptr


def get_op_loc_info(op: OpContext) -> str:
    buf = ctypes.create_string_buffer(1024)
    _check(lib.ttrt_op_loc_info(_vp(op._p), buf, ctypes.c_size_t(1024)))
    return buf.value.decode("utf-8", "replace")


def get_op_debug_str(op: OpContext) -> str:
    buf = ctypes.create_string_buffer(8192)
    _check(lib.ttrt_op_debug_string(_vp(op._p), buf, ctypes.c_size_t(8192)))
    return buf.value.decode("utf-8", "replace")


def get_op_output_tensor(op: OpContext, ctx: CallbackContext) -> Optional[Tensor]:
    h = ctypes.c_void_p()
    _check(lib.ttrt_op_output_tensor(_vp(op._p), _vp(ctx._p), ctypes.byref(h)))
    return Tensor(h.value) if h.value else None


def perf_env(dump_device_rate: int = 1000, enable_perf_trace: bool = False, program_metadata: str = "") -> bool:
    """perf::Env::get: the first call in a process fixes the settings.  Returns whether tracing is on."""
    on = ctypes.c_int()
    _check(lib.ttrt_perf_env_get(ctypes.c_uint32(dump_device_rate), int(enable_perf_trace), program_metadata.encode(),
                                 ctypes.byref(on)))
    return bool(on.value)


def perf_message(text: str, tag: int = 0) -> None:
    _check(lib.ttrt_perf_message(tag, text.encode()))


def perf_emitted() -> int:
    return int(lib.ttrt_perf_emitted())


class TensorRef:
    """Handle to a tensor of a running program (what hooks get from get_op_input_refs / get_op_output_refs)."""

    def __init__(self, handle: int):
        self._h = handle

    def __del__(self):
        if getattr(self, "_h", None) and lib is not None:
            lib.ttrt_tensor_ref_free(self._h)
            self._h = None

    def _info(self):
        rank, dt = ctypes.c_uint32(), ctypes.c_int()
        shape = (ctypes.c_uint32 * 8)()
        _check(lib.ttrt_tensor_ref_info(_vp(self._h), ctypes.byref(rank), shape, ctypes.byref(dt)))
        return list(shape[:rank.value]), DataType(dt.value)

    def get_shape(self):
        return self._info()[0]

    def get_dtype(self) -> DataType:
        return self._info()[1]


def _refs(fn, op: "OpContext") -> List[TensorRef]:
    n = ctypes.c_uint32()
    _check(fn(_vp(op._p), None, 0, ctypes.byref(n)))
    arr = (ctypes.c_void_p * max(n.value, 1))()
    _check(fn(_vp(op._p), arr, n, ctypes.byref(n)))
    return [TensorRef(arr[i]) for i in range(n.value)]


def get_op_input_refs(op: "OpContext") -> List[TensorRef]:
    return _refs(lib.ttrt_op_input_refs, op)


def get_op_output_refs(op: "OpContext") -> List[TensorRef]:
    return _refs(lib.ttrt_op_output_refs, op)


def retrieve_tensor_from_pool(ctx: "CallbackContext", ref: TensorRef, untilize: bool = True) -> Optional[Tensor]:
    h = ctypes.c_void_p()
    _check(lib.ttrt_retrieve_tensor_from_pool(_vp(ctx._p), _vp(ref._h), int(untilize), ctypes.byref(h)))
    return Tensor(h.value) if h.value else None


def update_tensor_in_pool(ctx: "CallbackContext", ref: TensorRef, src: Tensor) -> None:
    _check(lib.ttrt_update_tensor_in_pool(_vp(ctx._p), _vp(ref._h), _vp(src._h)))


def get_program_index(ctx: "CallbackContext") -> int:
    v = ctypes.c_size_t()
    _check(lib.ttrt_program_index(_vp(ctx._p), ctypes.byref(v)))
    return v.value


class DebugHooks:
    """debug::Hooks (runtime/include/tt/runtime/debug.h:77-158): callbacks get (binary_ptr,
    CallbackContext, OpContext); the contexts are only valid during the call."""
    _keep = []

    @staticmethod
    def get(pre_op=None, post_op=None) -> "DebugHooks":
        def wrap(fn):
            if fn is None:
                return ctypes.cast(None, _OP_CB)

            def tramp(bin_ptr, prog_ctx, op_ctx, _user):
                fn(bin_ptr, CallbackContext(prog_ctx), OpContext(op_ctx))
            return _OP_CB(tramp)
        pre_c, post_c = wrap(pre_op), wrap(post_op)
        DebugHooks._keep = [pre_c, post_c]
        _check(lib.ttrt_register_op_hooks(pre_c, post_c, None))
        return DebugHooks()


def unregister_hooks() -> None:
    _check(lib.ttrt_unregister_hooks())
    DebugHooks._keep = []


# ---------------------------------------------------------------------------------- torch helpers
def _torch_dtype_map():
    import torch
    return {torch.float32: DataType.Float32, torch.float16: DataType.Float16, torch.bfloat16: DataType.BFloat16,
            torch.int32: DataType.Int32, torch.uint8: DataType.UInt8, torch.int8: DataType.Int8,
            torch.uint16: DataType.UInt16, torch.uint32: DataType.UInt32}


def from_torch(t, owned: bool = False) -> Tensor:
    """Wraps a CPU torch tensor as a host tensor (borrowed: aliases t's memory and keeps t alive)."""
    dt = _torch_dtype_map()[t.dtype]
    if not owned:
        t = t.contiguous()
        return create_borrowed_host_tensor(t.data_ptr(), list(t.shape), list(t.stride()), t.element_size(), dt, keepalive=t)
    return create_owned_host_tensor(t.data_ptr(), list(t.shape), list(t.stride()), t.element_size(), dt)


def to_torch(t: Tensor):
    """Host copy of a (host or device) tensor as a torch tensor."""
    import torch
    inv = {v: k for k, v in _torch_dtype_map().items()}
    out = torch.empty(t.get_shape(), dtype=inv[t.get_dtype()])
    if out.numel():
        memcpy(out.data_ptr(), t)
    return out
