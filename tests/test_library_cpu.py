"""Host-side behaviour that needs no GPU: the library loads, exports its ABI, reads and
rejects binaries, and fails loudly (never falls back) when there is no device."""

import json

import pytest

from ttmlir_b200 import graphs


def test_every_declared_symbol_is_exported(rt):
    names = rt.declared_symbols()
    assert len(names) > 100
    assert "ttb_quant_chain" in names and "ttrt_submit" in names and "ttb_gemm" in names
    missing = [n for n in names if not hasattr(rt.lib, n)]
    assert not missing


def test_binary_metadata(rt):
    buf = graphs.build_binary(graphs.decoder_block_graph, seq=128, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64,
                              ffn=512, tp=2, mesh_shape=(1, 2))
    b = rt.Binary.load_from_memory(buf)
    assert b.file_identifier == "TTNN"
    assert b.version == "0.1.0"
    assert b.check_schema_hash()
    assert b.get_num_programs() == 1 and b.get_program_name(0) == "main" and not b.is_program_private(0)
    assert b.get_program_mesh_shape(0) == (1, 2)
    ins = b.get_program_inputs(0)
    assert len(ins) == 12 and ins[0] == ([1, 128, 256], rt.DataType.BFloat16)
    assert b.get_program_outputs(0) == [([1, 128, 256], rt.DataType.BFloat16)]
    ops = json.loads(b.get_program_ops_as_json(0))
    kinds = [o["type"] for o in ops]
    assert kinds[0] == "GetDeviceOp" and kinds.count("AllReduceOp") == 2 and kinds.count("DistributeTensorOp") == 12
    assert kinds[-1] == "AggregateTensorOp" or "AggregateTensorOp" in kinds
    assert "DeallocateOp" in kinds
    doc = json.loads(b.as_json())
    assert doc["programs"][0]["name"] == "main"


def test_store_and_reload(rt, tmp_path):
    buf = graphs.build_binary(graphs.mlp_graph)
    b = rt.Binary.load_from_memory(buf)
    p = str(tmp_path / "mlp.ttnn")
    b.store(p)
    assert open(p, "rb").read() == buf
    assert rt.Binary.load_from_path(p).get_num_program_inputs(0) == 5


@pytest.mark.parametrize("damage", ["truncate", "identifier", "offsets", "tiny", "root"])
def test_corrupt_binaries_are_rejected(rt, damage):
    buf = bytearray(graphs.build_binary(graphs.mlp_graph))
    if damage == "truncate":
        buf = buf[: len(buf) // 2]
    elif damage == "identifier":
        buf[8:12] = b"TTM0"
    elif damage == "offsets":
        buf[40:72] = b"\xff" * 32
    elif damage == "tiny":
        buf = buf[:6]
    elif damage == "root":
        buf[4:8] = (0x7FFFFFF0).to_bytes(4, "little")
    with pytest.raises(RuntimeError):
        rt.Binary.load_from_memory(bytes(buf))


def test_missing_file(rt):
    with pytest.raises(RuntimeError, match="cannot open"):
        rt.Binary.load_from_path("/nonexistent/model.ttnn")


def test_no_silent_cpu_fallback(rt):
    if rt.get_num_available_devices() > 0:
        pytest.skip("a GPU is present")
    with pytest.raises(RuntimeError, match="no CUDA device"):
        rt.open_mesh_device()


def test_host_tensor_api_without_gpu(rt):
    import torch
    x = torch.arange(24, dtype=torch.float32).reshape(2, 3, 4)
    t = rt.from_torch(x)
    assert t.get_shape() == [2, 3, 4] and t.get_dtype() == rt.DataType.Float32 and not t.is_on_device()
    assert t.get_volume() == 24 and t.get_element_size() == 4
    assert torch.equal(rt.to_torch(t), x)
    # owned tensors gather strided input
    xt = x.permute(2, 0, 1)
    o = rt.create_owned_host_tensor(xt.data_ptr(), list(xt.shape), list(xt.stride()), 4, rt.DataType.Float32)
    assert torch.equal(rt.to_torch(o), xt.contiguous())
    # borrowed tensors must be contiguous
    with pytest.raises(RuntimeError, match="contiguous"):
        rt.create_borrowed_host_tensor(xt.data_ptr(), list(xt.shape), list(xt.stride()), 4, rt.DataType.Float32)
    with pytest.raises(RuntimeError, match="itemsize"):
        rt.create_borrowed_host_tensor(x.data_ptr(), [2, 3, 4], [12, 4, 1], 2, rt.DataType.Float32)
    # memcpy with dtype conversion on the host
    out = torch.empty(24, dtype=torch.bfloat16)
    rt.memcpy(out.data_ptr(), t, rt.DataType.BFloat16)
    assert torch.equal(out, x.reshape(-1).to(torch.bfloat16))
    # retain flag and deallocation of borrowed memory is a no-op
    t.set_retain(True)
    assert t.get_retain()
    rt.deallocate_tensor(t, force=True)
    assert t.is_allocated()
    rt.deallocate_tensor(o, force=True)
    assert not o.is_allocated()
