"""The caller-facing boundary without a GPU: the system descriptor in the reference's wire format,
goldens embedded in a binary, perf::Env, and the stand-in for ttrt's extension module
(tt-mlir_b200/ttrt_backend/_ttmlir_runtime).  Where a checkout of tenstorrent/tt-mlir is present
(TT_MLIR_ROOT, or a `reference` directory beside this repository), its own `ttrt` Python sources are laid over the stand-in and driven
unchanged."""

import importlib.util
import json
import os
import subprocess
import sys
import textwrap

import pytest
import torch

from ttmlir_b200 import graphs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SHIM = os.path.join(ROOT, "tt-mlir_b200", "ttrt_backend", "_ttmlir_runtime")
REFERENCE = os.environ.get("TT_MLIR_ROOT", os.path.join(os.path.dirname(ROOT), "reference"))

# Every name tools/ttrt/runtime/__init__.py and tools/ttrt/binary/__init__.py import from the extension module.
RUNTIME_NAMES = """Device Event Tensor TensorRef TensorDesc MemoryBufferType DataType DeviceRuntime HostRuntime DispatchCoreType
MemoryLogLevel DebugEnv PerfEnv DebugHooks DebugStats MeshDeviceOptions MultiProcessArgs DistributedOptions DistributedMode
set_mlir_home set_metal_home set_memory_log_level get_current_device_runtime set_current_device_runtime
set_compatible_device_runtime get_current_host_runtime set_current_host_runtime get_available_host_runtimes
get_current_system_desc launch_distributed_runtime shutdown_distributed_runtime get_num_available_devices open_mesh_device
close_mesh_device create_sub_mesh_device release_sub_mesh_device reshape_mesh_device submit create_borrowed_host_tensor
create_owned_host_tensor create_empty_tensor create_multi_device_host_tensor create_multi_device_borrowed_host_tensor
create_multi_device_host_tensor_from_shards create_unsafe_borrowed_host_tensor set_fabric_config wait to_host get_device_tensors
get_num_shards to_layout get_layout get_op_output_tensor get_op_output_refs get_op_input_refs retrieve_tensor_from_pool
update_tensor_in_pool get_program_index walk_program get_op_debug_str invoke_cpu_op memcpy deallocate_tensor WorkaroundEnv
get_op_loc_info unregister_hooks FabricConfig get_worker_debug_stats""".split()
BINARY_NAMES = "load_from_path load_binary_from_path load_binary_from_capsule load_system_desc_from_path Flatbuffer GoldenTensor".split()


def load_shim():
    if "_ttmlir_runtime" in sys.modules:
        return sys.modules["_ttmlir_runtime"]
    spec = importlib.util.spec_from_file_location("_ttmlir_runtime", os.path.join(SHIM, "__init__.py"),
                                                  submodule_search_locations=[SHIM])
    mod = importlib.util.module_from_spec(spec)
    sys.modules["_ttmlir_runtime"] = mod
    spec.loader.exec_module(mod)
    return mod


def test_stand_in_module_has_every_name_ttrt_imports():
    shim = load_shim()
    missing = [n for n in RUNTIME_NAMES if not hasattr(shim.runtime, n)] + [n for n in BINARY_NAMES if not hasattr(shim.binary, n)]
    assert not missing, missing
    assert shim.runtime.DataType.BFloat16 == 2 and shim.runtime.DataType.Int8 == 17
    assert shim.runtime.get_current_device_runtime() == shim.runtime.DeviceRuntime.TTNN


def test_system_descriptor_round_trip(rt, tmp_path):
    """getCurrentSystemDesc writes a "TTSY" flatbuffer (Common/system_desc.fbs) that loads, prints and
    stores like any other; a binary built with its `system_desc` compares equal to it, which is the
    check ttrt makes before running a binary (tools/ttrt/common/util.py:868-912)."""
    desc = rt.get_current_system_desc()
    assert desc.file_identifier == "TTSY" and desc.version == "0.1.0" and desc.check_schema_hash()
    j = json.loads(desc.as_json())
    sd = j["system_desc"]
    assert set(sd) >= {"cpu_descs", "chip_descs", "chip_desc_indices", "chip_capabilities", "chip_coords"}
    assert sd["cpu_descs"][0]["role"] == "Host"
    assert len(sd["chip_descs"]) == len(sd["chip_desc_indices"]) == rt.get_num_available_devices()
    path = str(tmp_path / "system_desc.ttsys")
    desc.store(path)
    again = rt.Binary.load_from_path(path)
    assert again.file_identifier == "TTSY" and json.loads(again.as_json()) == j
    with pytest.raises(RuntimeError, match="holds no programs"):
        again.get_num_programs()
    binary = rt.Binary.load_from_memory(graphs.build_binary(graphs.mlp_graph, system_desc=sd))
    assert json.loads(binary.get_system_desc_as_json())["system_desc"] == sd
    assert rt.Binary.load_from_memory(graphs.build_binary(graphs.mlp_graph)).get_system_desc_as_json() == ""


def test_embedded_goldens(rt):
    x = torch.randn(3, 5)
    y = torch.randn(2, 2).to(torch.bfloat16)
    binary = rt.Binary.load_from_memory(graphs.build_binary(graphs.mlp_graph, goldens={"input_0": x, 'loc("relu")': y}))
    g = binary.get_debug_info_golden("input_0")
    assert list(g) == [0] and g[0].shape == [3, 5] and g[0].stride == [5, 1] and g[0].dtype == rt.DataType.Float32
    assert torch.equal(torch.frombuffer(g[0].get_data_buffer(), dtype=torch.float32).reshape(3, 5), x)
    h = binary.get_debug_info_golden('loc("relu")')[0]
    assert h.dtype == rt.DataType.BFloat16 and torch.equal(torch.frombuffer(h.get_data_buffer(), dtype=torch.bfloat16).reshape(2, 2), y)
    assert binary.get_debug_info_golden("output_7") == {}


def test_perf_env_messages_are_counted():
    """perf::Env fixes its settings at the first call in a process, so this runs in a child process:
    with tracing on, each message is one NVTX mark; with tracing off nothing is emitted."""
    code = textwrap.dedent("""
        import sys
        sys.path.insert(0, %r)
        from __graft_entry__ import load_package
        load_package()
        import ttmlir_b200.runtime_api as rt
        on = rt.perf_env(1000, sys.argv[1] == "on", "model=decoder")
        before = rt.perf_emitted()
        rt.perf_message('loc("q_proj")')
        rt.perf_message("true", tag=1)
        rt.perf_message("model=decoder", tag=2)
        print(int(on), rt.perf_emitted() - before)
    """ % ROOT)
    for mode, want in (("on", "1 3"), ("off", "0 0")):
        env = {k: v for k, v in os.environ.items() if k != "TT_RUNTIME_ENABLE_PERF_TRACE"}
        out = subprocess.run([sys.executable, "-c", code, mode], capture_output=True, text=True, env=env, timeout=120)
        assert out.returncode == 0, out.stderr
        assert out.stdout.strip().splitlines()[-1] == want


@pytest.mark.skipif(not os.path.isdir(os.path.join(REFERENCE, "tools", "ttrt", "common")),
                    reason="needs a checkout of tenstorrent/tt-mlir (TT_MLIR_ROOT)")
def test_reference_ttrt_sources_run_on_the_stand_in(tmp_path):
    """tt-mlir's own `ttrt` package (tools/ttrt: __init__, binary/, common/, runtime/__init__.py), linked
    unmodified next to the stand-in for its extension module, imports, wraps a binary in its
    `ttrt.common.util.Binary`, and runs `ttrt read` over every section whose code matches the
    reference's own schema."""
    pkg = tmp_path / "ttrt"
    (pkg / "runtime").mkdir(parents=True)
    src = os.path.join(REFERENCE, "tools", "ttrt")
    for name in ("__init__.py", "__main__.py", "binary", "common", "library_tweaks.py"):
        os.symlink(os.path.join(src, name), pkg / name)
    os.symlink(os.path.join(src, "runtime", "__init__.py"), pkg / "runtime" / "__init__.py")
    os.symlink(SHIM, pkg / "runtime" / "_ttmlir_runtime")
    binary_path = tmp_path / "mlp.ttnn"
    binary_path.write_bytes(graphs.build_binary(graphs.mlp_graph, goldens={"input_0": torch.zeros(128, 784)}))
    code = textwrap.dedent("""
        import json, sys
        sys.path.insert(0, %r)
        import ttrt, ttrt.binary, ttrt.runtime
        from ttrt.common.api import API
        import ttrt.common.util as U
        API.initialize_apis()
        assert {"Read", "Run", "Query", "Perf", "Check"} <= set(API.registered_apis), API.registered_apis
        logger = U.Logger()
        b = U.Binary(logger, U.FileManager(logger), %r)
        assert b.check_version() and len(b.programs) == 1 and b.programs[0].num_inputs() == 5
        assert b.programs[0].inputs[0]["desc"]["shape"] == [128, 784]
        assert b.fbb.get_debug_info_golden("input_0")[0].shape == [128, 784]
        assert ttrt.binary.mlir_as_dict(b.fbb)["name"] == "ttnn"
        ok = {}
        for section in ("version", "mlir", "inputs", "outputs", "all"):
            args = {"binary": %r, "--section": section, "--log-file": "", "--result-file": %r, "--artifact-dir": %r,
                    "--clean-artifacts": False, "--save-artifacts": False, "--ignore-version": False}
            rc, _ = API.Read(args=args, logger=logger)()
            ok[section] = rc
        print("RESULT", json.dumps(ok))
    """ % (str(tmp_path), str(binary_path), str(binary_path), str(tmp_path / "read.json"), str(tmp_path / "artifacts")))
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300, cwd=str(tmp_path))
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    line = [ln for ln in out.stdout.splitlines() if ln.startswith("RESULT")][-1]
    assert set(json.loads(line[7:]).values()) == {0}, line
