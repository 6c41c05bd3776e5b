"""The caller-facing boundary on a GPU, through the stand-in for ttrt's extension module: the sequence of
calls `ttrt run` makes (tools/ttrt/common/run.py:562-1132) -- descriptor check, device open, inputs from
embedded goldens, layout conversion, submit, read-back, comparison with the embedded output golden,
per-op callback that looks up intermediate goldens by location -- and the profiler ranges."""

import json
import os
import subprocess
import sys
import textwrap

import pytest
import torch

from helpers import oracle_results
from test_ttrt_boundary_cpu import ROOT, load_shim
from ttmlir_b200 import graphs

pytestmark = pytest.mark.gpu


def to_torch(shim, t):
    names = {shim.runtime.DataType.Float32: torch.float32, shim.runtime.DataType.BFloat16: torch.bfloat16,
             shim.runtime.DataType.Int32: torch.int32}
    return torch.frombuffer(bytearray(t.get_data_buffer()), dtype=names[t.get_dtype()]).reshape(t.get_shape())


def test_descriptor_of_the_machine_matches_a_binary_compiled_for_it(rt, device):
    shim = load_shim()
    desc = shim.runtime.get_current_system_desc()
    sd = json.loads(desc.as_json())["system_desc"]
    n = rt.get_num_available_devices()
    assert len(sd["chip_descs"]) == n and sd["chip_desc_indices"] == list(range(n))
    chip = sd["chip_descs"][0]
    assert chip["num_dram_channels"] == 1 and chip["dram_channel_size"] > (100 << 30)          # HBM as one channel
    assert chip["grid_size"]["y"] * chip["grid_size"]["x"] == 148 and chip["l1_size"] == 227 * 1024
    assert "BFloat16" in chip["supported_data_types"] and chip["supported_tile_sizes"] == [{"y": 32, "x": 32}]
    # what ttrt's Binary.check_system_desc compares
    binary = shim.binary.load_binary_from_bytes(graphs.build_binary(graphs.mlp_graph, system_desc=sd))
    assert json.loads(binary.get_system_desc_as_json())["system_desc"] == sd
    one = json.loads(shim.runtime.get_current_system_desc(None, device).as_json())["system_desc"]
    assert len(one["chip_descs"]) == 1


def test_the_run_sequence_with_embedded_goldens(rt, device):
    shim = load_shim()
    R, B = shim.runtime, shim.binary
    ins = graphs.mlp_inputs()
    want = oracle_results(graphs.mlp_graph, ins)
    # intermediates of the oracle, keyed by the op locations the graph uses
    from helpers import TeacherForcedOracle
    goldens = {f"input_{i}": t for i, t in enumerate(ins)}
    goldens["output_0"] = want[0]
    binary = B.load_binary_from_bytes(graphs.build_binary(graphs.mlp_graph, goldens=goldens))
    R.set_compatible_device_runtime(binary)
    assert R.get_current_device_runtime() == R.DeviceRuntime.TTNN
    assert binary.get_program_mesh_shape(0) == (1, 1)
    # inputs come from the embedded goldens, as with `ttrt run --enable-golden`
    host = []
    keep = []
    for i in range(5):
        g = binary.get_debug_info_golden(f"input_{i}")[0]
        t = torch.frombuffer(g.get_data_buffer(), dtype=torch.float32).reshape(g.shape).clone()
        keep.append(t)
        host.append(R.create_borrowed_host_tensor(t.data_ptr(), list(t.shape), list(t.stride()), t.element_size(), R.DataType.Float32))
    seen = []

    def post_op(bin_, program_ctx, op_ctx):
        loc = R.get_op_loc_info(op_ctx)
        outs = R.get_op_output_tensor(op_ctx, program_ctx)
        refs = R.get_op_output_refs(op_ctx)
        seen.append((loc, R.get_op_debug_str(op_ctx), len(outs), [r.get_shape() for r in refs]))
        if outs:
            # a tensor still in the pool can be fetched through its reference as well
            again = R.retrieve_tensor_from_pool(program_ctx, refs[0], True)
            assert again is not None and again.get_shape() == outs[0].get_shape()
    R.DebugHooks.get(None, post_op)
    try:
        converted = [R.to_layout(h, device, R.get_layout(binary, 0, i), True) for i, h in enumerate(host)]
        outs = R.submit(device, binary, 0, converted)
        R.wait(outs)
        result = R.to_host(outs[0], untilize=True)[0]
    finally:
        R.unregister_hooks()
    got = to_torch(shim, result)
    g = binary.get_debug_info_golden("output_0")[0]
    golden = torch.frombuffer(g.get_data_buffer(), dtype=torch.float32).reshape(g.shape)
    from oracle import metrics
    assert metrics.get_pcc(golden, got) >= 0.999 and torch.allclose(got, golden, atol=1e-4, rtol=1e-4)
    locs = [s[0] for s in seen]
    assert any("softmax" in l for l in locs) and all(s[1] for s in seen)
    R.deallocate_tensor(outs[0], force=True)


def test_ops_are_bracketed_by_profiler_ranges():
    """With TT_RUNTIME_ENABLE_PERF_TRACE=1 every op of a submit emits the reference's three messages and
    one range; without it nothing.  The setting is read once per process, hence the child processes."""
    code = textwrap.dedent("""
        import sys
        sys.path.insert(0, %r)
        from __graft_entry__ import load_package
        load_package()
        import ttmlir_b200.runtime_api as rt
        from ttmlir_b200 import graphs
        dev = rt.open_mesh_device(rt.MeshDeviceOptions(mesh_shape=[1, 1]))
        binary = rt.Binary.load_from_memory(graphs.build_binary(graphs.mlp_graph))
        ins = [rt.to_layout(rt.from_torch(t), dev, rt.get_layout(binary, 0, i)) for i, t in enumerate(graphs.mlp_inputs())]
        out = rt.submit(dev, binary, 0, ins)
        rt.wait(out[0])
        print("EMITTED", rt.perf_emitted())
        rt.close_mesh_device(dev)
    """ % ROOT)
    counts = {}
    for flag in ("1", "0"):
        env = dict(os.environ, TT_RUNTIME_ENABLE_PERF_TRACE=flag)
        out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=300)
        assert out.returncode == 0, out.stderr[-2000:]
        counts[flag] = int([ln for ln in out.stdout.splitlines() if ln.startswith("EMITTED")][-1].split()[1])
    assert counts["0"] == 0
    assert counts["1"] >= 4 * 5, counts     # at least the matmul / add / relu / softmax chain, four emissions per op
