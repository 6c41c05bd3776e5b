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
    kinds = [o["type_type"] for o in ops]
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


def _flatc_style(x):
    """The Python reader's view of a table (unions as (name, table) pairs, absent fields None) in the
    shape of flatc's JSON text: "<field>_type" + "<field>" for unions, absent fields left out."""
    if isinstance(x, dict):
        out = {}
        for k, v in x.items():
            if v is None:
                continue
            if isinstance(v, tuple) and len(v) == 2 and isinstance(v[0], str) and isinstance(v[1], dict):
                out[k + "_type"] = v[0]
                out[k] = _flatc_style(v[1])
            else:
                out[k] = _flatc_style(v)
        return out
    if isinstance(x, (list, tuple)):
        return [_flatc_style(v) for v in x]
    if isinstance(x, (bytes, bytearray, memoryview)):
        return list(bytes(x))
    return x


def _drop_absent_unions(x):
    if isinstance(x, dict):
        return {k: _drop_absent_unions(v) for k, v in x.items() if not (k.endswith("_type") and v == "NONE")}
    if isinstance(x, list):
        return [_drop_absent_unions(v) for v in x]
    return x


def _close(a, b, path="$"):
    if isinstance(a, dict):
        assert isinstance(b, dict) and set(a) == set(b), f"{path}: keys {sorted(set(a) ^ set(b))}"
        for k in a:
            _close(a[k], b[k], f"{path}.{k}")
    elif isinstance(a, list):
        assert isinstance(b, list) and len(a) == len(b), path
        for i, (x, y) in enumerate(zip(a, b)):
            _close(x, y, f"{path}[{i}]")
    elif isinstance(a, float) or isinstance(b, float):
        assert abs(float(a) - float(b)) <= 1e-6 * max(1.0, abs(float(a))), f"{path}: {a} vs {b}"
    else:
        assert a == b, f"{path}: {a!r} vs {b!r}"


def _wide_ops_graph(b):
    """One op of every family that widens the op coverage: their tables go through the writer, the C++ reader /
    verifier and the generated JSON printers without a GPU."""
    bf = "BFloat16"
    x = b.input([2, 6, 6, 8], bf)
    v = b.input([4, 16], "Float32")
    outs = [b.cumprod(v, 1), b.prod(v, 1), b.upsample(x, 2), b.group_norm(b.reshape(x, [2, 1, 36, 8]), None, None, 2),
            b.bitcast_convert(v, "Int32"), b.assign(v, bf), b.pow_scalar(v, 2.0), b.dropout(v, 0.1, seed=3), b.rand([4, 4], "Float32"),
            b.region_end(b.region_start(b.annotate(v, "note"), "r"), "r")]
    b.print_message(v, "hello")
    b.breakpoint(v)
    b.memory_snapshot(v, "snapshot.txt")
    b.dump_tensor(v, "t.bin")
    outs.append(b.load_tensor("t.bin", [4, 16], "Float32"))
    mean, var = b.input([6], bf), b.input([6], bf)
    nchw = b.input([2, 6, 4, 4], bf)
    outs += [b.batch_norm_inference(nchw, mean, var, None, None), b.batch_norm_training(nchw, mean, var, None, None)]
    w = b.input([8, 4, 3, 3], bf)
    outs.append(b.conv_transpose2d(x, b.prepare_conv_transpose2d_weights(w, 2, 6, 6), None, 2, 6, 6))
    outs.append(b.conv1d(b.input([2, 10, 8], bf), b.input([4, 8, 3], bf), None, 2, 10))
    outs.append(b.conv3d(b.input([1, 1, 2 * 3 * 4 * 4, 8], bf), b.prepare_conv3d_weights(b.input([4, 8, 2, 2, 2], bf)), None, 2, 3, 4, 4))
    pooled, idx = b.max_pool2d_with_indices(b.reshape(x, [1, 1, 72, 8]), 2, 6, 6, 8)
    outs += [pooled, idx]
    q, k, vv = b.nlp_create_qkv_heads_decode(b.input([1, 1, 4, (2 + 2) * 32], bf), 2, 1)
    outs += [b.nlp_concat_heads_decode(q, 2), k, vv, b.nlp_concat_heads(b.input([1, 2, 4, 32], bf))]
    rx = b.input([1, 2, 32, 64], bf)
    outs.append(b.rotary_embedding_llama(rx, b.input([1, 1, 32, 64], bf), b.input([1, 1, 32, 64], bf), b.input([1, 1, 32, 32], bf)))
    nx = b.input([4, 64], bf)
    outs += [b.dit_rms_norm_unary_fused(nx, activation="silu"), b.distributed_rms_norm(nx), b.rms_norm_pre_all_gather(nx),
             b.layer_norm_post_all_gather(nx, b.layer_norm_pre_all_gather(nx))]
    b.create_global_semaphore(0)
    b.reset_global_semaphore(0)
    tok, sel = b.input([4, 1, 2, 16], bf), b.input([4, 1, 2, 2], "Int32")
    mp = b.input([1, 1, 4, 1], "Int32")
    disp, meta = b.all_to_all_dispatch(tok, sel, mp)
    mapping, reduced = b.moe_expert_token_remap(b.input([1, 4, 2, 4], bf), mp, meta, 8)
    sm = b.sparse_matmul(b.input([1, 1, 32, 16], bf), b.input([1, 4, 16, 16], bf), b.input([1, 1, 1, 4], bf), nnz=2)
    outs += [disp, mapping, reduced, sm, b.all_to_all_combine(b.input([4, 4, 2, 16], bf), meta, mp, 2)]
    d3, i3, s3 = b.all_to_all_dispatch_metadata(b.input([1, 1, 8, 16], bf), b.input([1, 1, 8, 2], "Int32"), b.input([1, 1, 8, 2], bf),
                                               b.input([1, 1, 1, 4], "Int32"))
    ri, rw = b.topk_router_gpt(b.input([32, 64], bf), b.input([64, 16], bf), b.input([32, 16], bf), 4)
    outs += [d3, i3, s3, ri, rw, b.all_reduce_async(nx), b.point_to_point(nx, [0, 0], [0, 0])]
    outs += [b.gelu_backward(nx, nx, "tanh"), b.embedding_backward(b.input([2, 3], "Int32"), b.input([10, 64], bf), b.input([2, 3, 64], bf))]
    b.adamw(b.input([8], "Float32"), b.input([8], "Float32"), b.input([8], "Float32"), b.input([8], "Float32"))
    qc = b.input([1, 2, 16, 32], bf)
    outs.append(b.chunked_scaled_dot_product_attention(qc, b.input([4, 1, 16, 32], bf), b.input([4, 1, 16, 32], bf),
                                                       b.input([1, 2], "Int32"), b.input([1], "Int32"), scale=0.2))
    outs.append(b.flash_mla_prefill(b.input([1, 2, 8, 48], bf), b.input([1, 1, 8, 48], bf), 32))
    outs.append(b.indexer_score_dsa(b.input([1, 4, 8, 32], bf), b.input([1, 1, 16, 32], bf), b.input([1, 4, 8, 1], bf), 8, cluster_axis=1))
    b.output(*outs)


@pytest.mark.parametrize("which", ["decoder", "quant", "traced", "pool", "wide"])
def test_json_views_print_every_declared_field(rt, which):
    """Binary::asJson / getProgramOpsAsJson (the generated printers) against the independent Python
    reader of the same buffer: every table, union, struct, enum and optional scalar of every op."""
    from ttmlir_b200.schema.fbs import Reader
    from ttmlir_b200.schema.ttnn_schema import S
    if which == "decoder":
        buf = graphs.build_binary(graphs.decoder_block_graph, seq=128, hidden=256, n_heads=4, n_kv_heads=2, head_dim=64,
                                  ffn=512, tp=2, mesh_shape=(1, 2))
    elif which == "quant":
        buf = graphs.build_binary(graphs.quant_chain_graph, rows=8, cols=8, keep_intermediates=True)
    elif which == "traced":
        buf = graphs.mlp_traced_binary(batch=4, d_in=8, d_hidden=8, d_out=4)
    elif which == "wide":
        buf = graphs.build_binary(_wide_ops_graph)
    else:
        def g(b):
            x = b.input([1, 1, 2 * 9 * 11, 8], "BFloat16")
            b.output(b.avg_pool2d(b.max_pool2d(x, 2, 9, 11, 8, (3, 3), (2, 2), (1, 2, 0, 1)), 2, 4, 6, 8, (2, 2), (2, 2), (0, 0),
                                  False, False), b.argmax(x, 2), b.pad(x, [0, 0, 0, 0, 1, 2, 0, 3], 1.5))
        buf = graphs.build_binary(g)
    want = _flatc_style(Reader(S, buf).root("TTNNBinary"))
    b = rt.Binary.load_from_memory(buf)
    got = _drop_absent_unions(json.loads(b.as_json()))
    _close(got, want)
    for i in range(b.get_num_programs()):
        ops = _drop_absent_unions(json.loads(b.get_program_ops_as_json(i)))
        _close(ops, want["programs"][i].get("operations", []), f"$.programs[{i}].operations")
