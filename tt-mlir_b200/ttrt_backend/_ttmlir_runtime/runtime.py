"""`ttrt.runtime._ttmlir_runtime.runtime`: the names runtime/python/runtime/runtime.cpp registers, over
the C ABI.  Functions that only mean something on Tenstorrent silicon (fabric configuration, memory
views per bank, the multi-host distributed controller) exist because `ttrt` calls them unconditionally;
they accept their arguments and do nothing, or raise where a result would be required."""

import enum
from typing import List, Optional, Sequence

from . import api
from .binary import Binary, SystemDesc, _adopt

# ---- handle types (runtime.cpp:41-66, 204-279) ---------------------------------------------------------
Device = api.Device
Tensor = api.Tensor
TensorRef = api.TensorRef
Layout = api.Layout
OpContext = api.OpContext
CallbackContext = api.CallbackContext
DataType = api.DataType            # runtime.cpp:287-307, values of tt::target::DataType


class Event:
    pass


class TensorDesc:
    """runtime.cpp:61-66."""

    def __init__(self, shape, stride, item_size, dtype):
        self.shape, self.stride, self.item_size, self.dtype = list(shape), list(stride), item_size, dtype
        self.physical_volume = 1
        for d in self.shape:
            self.physical_volume *= d


class MemoryBufferType(enum.IntEnum):     # runtime.cpp:281-285
    DRAM = 0
    L1 = 1
    L1_SMALL = 2
    TRACE = 3


class DeviceRuntime(enum.IntEnum):        # runtime.cpp:309-312; the CUDA target answers to "TTNN" binaries
    Disabled = 0
    TTNN = 1
    TTMetal = 2


class HostRuntime(enum.IntEnum):
    Local = 0
    Distributed = 1


class DistributedMode(enum.IntEnum):
    LocalSubprocess = 0
    MultiProcess = 1


class DispatchCoreType(enum.IntEnum):
    WORKER = 0
    ETH = 1


class FabricConfig(enum.IntEnum):
    DISABLED = 0
    FABRIC_1D = 1
    FABRIC_1D_RING = 2
    FABRIC_2D = 3
    FABRIC_2D_TORUS_X = 4
    FABRIC_2D_TORUS_Y = 5
    FABRIC_2D_TORUS_XY = 6
    CUSTOM = 7


class Arch(enum.IntEnum):
    WORMHOLE_B0 = 0
    BLACKHOLE = 1
    QUASAR = 2


class MemoryLogLevel(enum.IntFlag):
    NONE = 0
    PROGRAM = 1
    OPERATION = 2
    ANY = 3


class MeshDeviceOptions(api.MeshDeviceOptions):
    """runtime.cpp:68-129.  The reference's fields are accepted; those without a GPU meaning are kept as
    plain attributes."""

    def __init__(self):
        super().__init__()
        self.mesh_offset = [0, 0]
        self.num_hw_cqs = 1
        self.enable_program_cache = True
        self.l1_small_size = None
        self.trace_region_size = None
        self.dispatch_core_type = None


class MultiProcessArgs:
    @staticmethod
    def create(*a, **k):
        raise NotImplementedError("the multi-host distributed controller is not part of the CUDA target")


class DistributedOptions:
    def __init__(self):
        self.controller_port = 0
        self.mode = DistributedMode.LocalSubprocess
        self.multi_process_args = None
        self.worker_path = None


class _Env:
    """DebugEnv / PerfEnv / WorkaroundEnv: process-wide singletons whose `get(...)` takes the reference's
    positional switches.  The CUDA target keeps the values for printing and honours the ones it has a
    meaning for through its environment variables (TT_RUNTIME_SYNC_AFTER_OP ...)."""
    _instance = None

    def __init__(self):
        self.values = ()

    @classmethod
    def get(cls, *args, **kwargs):
        if cls._instance is None:
            cls._instance = cls()
        if args or kwargs:
            cls._instance.values = (args, kwargs)
        return cls._instance

    def __str__(self):
        return f"{type(self).__name__}{self.values}"


class DebugEnv(_Env):
    _instance = None


class WorkaroundEnv(_Env):
    _instance = None


class PerfEnv(_Env):
    """runtime.cpp:726-742.  The per-op messages go to the profiler ranges of the kernel library."""
    _instance = None

    def set_program_metadata(self, metadata: str):
        self.program_metadata = metadata

    def tracy_log_op_location(self, loc: str):
        api.perf_message(loc)

    def tracy_log_input_layout_conversion(self, converted: bool):
        api.perf_message(f"input_layout_conversion={bool(converted)}")

    def tracy_log_const_eval_program(self, const_eval: bool):
        api.perf_message(f"const_eval_program={bool(const_eval)}")

    def tracy_log_program_metadata(self, metadata: str):
        api.perf_message(metadata)


class DebugStats:
    """runtime.cpp:814-827."""
    _instance = None

    @classmethod
    def get(cls):
        if cls._instance is None:
            cls._instance = cls()
        return cls._instance

    def get_stat(self, stat: str) -> int:
        return api.get_stat(stat)

    def clear(self):
        api.clear_stats()

    def __str__(self):
        names = ("ConstEvalCacheHit", "ConstEvalCacheMiss", "TraceCacheMiss", "CapturedTrace", "ExecutedTrace")
        return "DebugStats{" + ", ".join(f"{n}: {api.get_stat(n)}" for n in names) + "}"


class DebugHooks:
    """runtime.cpp:744-812: DebugHooks.get(pre_op, post_op, pre_program, post_program).  Operation callbacks
    receive (binary, program_context, op_context), as in the reference."""

    @staticmethod
    def get(pre_op=None, post_op=None, pre_program=None, post_program=None):
        if pre_program is not None or post_program is not None:
            raise NotImplementedError("program-level callbacks are not exposed through the C ABI")
        return api.DebugHooks.get(pre_op, post_op)


# ---- runtime selection ---------------------------------------------------------------------------------
def set_mlir_home(mlir_home: str):
    pass


def set_metal_home(metal_home: str):
    pass


def set_memory_log_level(level):
    pass


def get_current_device_runtime():
    return DeviceRuntime.TTNN


def get_available_device_runtimes():
    return [DeviceRuntime.TTNN]


def set_current_device_runtime(runtime):
    if int(runtime) != int(DeviceRuntime.TTNN):
        raise RuntimeError("the CUDA target serves TTNN binaries only")


def set_compatible_device_runtime(binary):
    api.set_compatible_device_runtime(binary)


def get_current_host_runtime():
    return HostRuntime.Local


def get_available_host_runtimes():
    return [HostRuntime.Local]


def set_current_host_runtime(runtime):
    if int(runtime) != int(HostRuntime.Local):
        raise RuntimeError("the CUDA target has no distributed host runtime")


def launch_distributed_runtime(*a, **k):
    raise NotImplementedError("the multi-host distributed controller is not part of the CUDA target")


def shutdown_distributed_runtime():
    pass


def get_worker_debug_stats():
    return []


def get_current_system_desc(dispatch_core_type=None, mesh_device: Optional[Device] = None) -> SystemDesc:
    return _adopt(SystemDesc, api.get_current_system_desc(mesh_device))


def get_arch():
    return Arch.BLACKHOLE


# ---- devices ---------------------------------------------------------------------------------------------
get_num_available_devices = api.get_num_available_devices
open_mesh_device = api.open_mesh_device
close_mesh_device = api.close_mesh_device
create_sub_mesh_device = api.create_sub_mesh_device
release_sub_mesh_device = api.release_sub_mesh_device
reshape_mesh_device = api.reshape_mesh_device


def set_fabric_config(config):
    pass


# ---- tensors ---------------------------------------------------------------------------------------------
create_borrowed_host_tensor = api.create_borrowed_host_tensor
create_unsafe_borrowed_host_tensor = api.create_borrowed_host_tensor
create_owned_host_tensor = api.create_owned_host_tensor
create_multi_device_host_tensor_from_shards = api.create_multi_device_host_tensor_from_shards


def create_multi_device_host_tensor(ptrs: Sequence[int], shape, stride, item_size, dtype, strategy, mesh_shape) -> Tensor:
    shards = [api.create_owned_host_tensor(p, shape, stride, item_size, dtype) for p in ptrs]
    return api.create_multi_device_host_tensor_from_shards(shards, strategy, mesh_shape)


def create_multi_device_borrowed_host_tensor(ptrs: Sequence[int], shape, stride, item_size, dtype, strategy, mesh_shape) -> Tensor:
    shards = [api.create_borrowed_host_tensor(p, shape, stride, item_size, dtype) for p in ptrs]
    return api.create_multi_device_host_tensor_from_shards(shards, strategy, mesh_shape)


def create_empty_tensor(device, layout, shape, stride, item_size):
    raise NotImplementedError("create_empty_tensor is not exposed through the C ABI")


def wait(obj, cq_id=None):
    api.wait(obj)


def to_host(tensor, untilize: bool = False, blocking: bool = True) -> List[Tensor]:
    return api.to_host(tensor, untilize=untilize, blocking=blocking)


def get_device_tensors(tensor) -> List[Tensor]:
    return [tensor]


def get_num_shards(tensor) -> int:
    return tensor.get_num_shards()


def to_layout(tensor, device, layout, retain: Optional[bool] = None) -> Tensor:
    return api.to_layout(tensor, device, layout, retain)


get_layout = api.get_layout
memcpy = api.memcpy
deallocate_tensor = api.deallocate_tensor
submit = api.submit

# ---- debug hooks -------------------------------------------------------------------------------------------
get_op_debug_str = api.get_op_debug_str
get_op_loc_info = api.get_op_loc_info
get_op_output_refs = api.get_op_output_refs
get_op_input_refs = api.get_op_input_refs
retrieve_tensor_from_pool = api.retrieve_tensor_from_pool
update_tensor_in_pool = api.update_tensor_in_pool
get_program_index = api.get_program_index
unregister_hooks = api.unregister_hooks


def get_op_output_tensor(op_context, program_context):
    """runtime.cpp: a dict device id -> host tensor (empty when the op has no live output)."""
    t = api.get_op_output_tensor(op_context, program_context)
    return {0: t} if t is not None else {}


def walk_program(binary, program_index, callback):
    raise NotImplementedError("walk_program is not exposed through the C ABI")


def invoke_cpu_op(*a, **k):
    raise RuntimeError("CPU-hoisted ops are not executed by the CUDA target (no CPU fallback)")
