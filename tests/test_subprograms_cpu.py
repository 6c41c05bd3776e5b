"""Binaries with private sub-programs (const-eval functions, traced functions), as far as they
can be checked without a GPU: the builder emits the program set the compiler's trace hoisting
and const-eval hoisting produce, and the reader sees it."""

import json

from ttmlir_b200 import graphs


def _ops(binary, i):
    return [o["type_type"] for o in json.loads(binary.get_program_ops_as_json(i))]


def test_traced_binary_has_the_four_private_programs(rt):
    b = rt.Binary.load_from_memory(graphs.mlp_traced_binary(batch=32, d_in=64, d_hidden=48, d_out=10))
    names = [b.get_program_name(i) for i in range(b.get_num_programs())]
    assert names == ["mlp", "trace_0_mlp", "allocate_slots_trace_0_mlp", "run_and_capture_trace_0_mlp",
                     "execute_trace_0_mlp"]
    assert [b.is_program_private(i) for i in range(5)] == [False, True, True, True, True]
    # main: only the trace op; its input 0 (the activation) is host-staged, the parameters are on device
    assert _ops(b, 0) == ["GetDeviceOp", "CaptureOrExecuteTraceOp"]
    assert b.get_program_inputs(0)[0] == ([32, 64], rt.DataType.Float32)
    # traced function: (4 parameters, activation, output slot) -> nothing; results leave through CopyOp
    assert b.get_num_program_inputs(1) == 6 and b.get_num_program_outputs(1) == 0
    ops = _ops(b, 1)
    assert ops.count("MatmulOp") == 2 and "SoftmaxOp" in ops and ops.count("CopyOp") == 1
    # slot allocation: (device-resident inputs) -> input slots + output slots
    assert b.get_num_program_inputs(2) == 4 and b.get_num_program_outputs(2) == 6
    assert _ops(b, 2).count("EmptyOp") == 2
    # capture: (host input, 5 input slots, 1 output slot) -> trace id; write, call, begin, call, end, replay
    assert b.get_num_program_inputs(3) == 7
    assert b.get_program_outputs(3) == [([], rt.DataType.UInt32)]
    assert _ops(b, 3) == ["GetDeviceOp", "WriteTensorOp", "FuncCallOp", "BeginTraceCaptureOp", "FuncCallOp",
                          "EndTraceCaptureOp", "ExecuteTraceOp"]
    assert "DeallocateOp" not in _ops(b, 3) and "CopyOp" not in _ops(b, 3)
    # execute: (trace id) -> nothing
    assert b.get_program_inputs(4) == [([], rt.DataType.UInt32)] and _ops(b, 4) == ["GetDeviceOp", "ExecuteTraceOp"]


def test_const_eval_binary_has_a_load_cached_op(rt):
    b = rt.Binary.load_from_memory(graphs.w8_linear_const_eval_binary(m=64, k=128, n=96))
    assert b.get_num_programs() == 2
    assert b.get_program_name(1) == "w8_linear_const_eval_0" and b.is_program_private(1)
    assert _ops(b, 0)[:3] == ["GetDeviceOp", "LoadCachedOp", "LinearOp"]
    assert _ops(b, 1) == ["GetDeviceOp", "EltwiseQuantizationOp"]
    assert b.get_program_inputs(1) == [([96, 128], rt.DataType.Int8), ([96], rt.DataType.Float32)]
    assert b.get_program_outputs(1) == [([96, 128], rt.DataType.BFloat16)]


def test_stats_and_cache_api_without_gpu(rt):
    rt.clear_stats()
    assert rt.get_stat("ConstEvalCacheHit") == 0
    rt.clear_const_eval_cache()
    assert rt.const_eval_cache_size() == 0
    a = rt.Binary.load_from_memory(graphs.build_binary(graphs.mlp_graph))
    b = rt.Binary.load_from_memory(graphs.build_binary(graphs.mlp_graph))
    assert a.id != b.id
