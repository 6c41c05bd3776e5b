"""Mesh programs (ttir.mesh_shard + collectives) on a 1xN device mesh driven by one process, as the
reference's runtime drives a mesh.  Needs at least two GPUs; skipped otherwise."""

import pytest
import torch

from helpers import assert_matches, oracle_results, run_body, run_program
from ttmlir_b200 import graphs

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mesh2(rt):
    if rt.get_num_available_devices() < 2:
        pytest.skip("needs two GPUs")
    dev = rt.open_mesh_device(rt.MeshDeviceOptions(mesh_shape=[1, 2]))
    yield dev
    rt.close_mesh_device(dev)


def host_graph(body, inputs, mesh):
    def graph(b):
        from helpers import DTYPE_NAME
        vals = [b.input(list(t.shape), DTYPE_NAME[t.dtype], on_device=False) for t in inputs]
        out = body(b, *vals)
        b.output(*(out if isinstance(out, (tuple, list)) else (out,)))
    return graph


def run_mesh(rt, dev, body, inputs):
    graph = host_graph(body, inputs, (1, 2))
    buf = graphs.build_binary(graph, mesh_shape=(1, 2))
    got = run_program(rt, dev, buf, inputs)
    want = oracle_results(graph, inputs, mesh_shape=(1, 2))
    return got, want


def test_shard_and_aggregate_round_trip(rt, mesh2):
    x = torch.randn(6, 8, 10)
    for dim in (0, 1, 2):
        got, want = run_mesh(rt, mesh2, lambda b, v: b.aggregate(b.distribute(v, dim), dim), [x])
        assert torch.equal(got[0], x) and torch.equal(want[0], x)
    got, _ = run_mesh(rt, mesh2, lambda b, v: b.aggregate(b.distribute(v, None), None), [x])
    assert torch.equal(got[0], x)


def test_all_reduce_all_gather_reduce_scatter(rt, mesh2):
    x = torch.randn(4, 6, 16)

    def body(b, v):
        s = b.distribute(v, 0)                       # each device holds [2, 6, 16]
        ar = b.aggregate(b.all_reduce(s), None)      # sum of the two halves, replicated
        ag0 = b.aggregate(b.all_gather(s, 0), None)  # gather on the leading dim
        ag2 = b.aggregate(b.all_gather(s, 2), None)  # gather on an inner dim
        rs = b.aggregate(b.reduce_scatter(s, 1), 1)  # reduce, scatter dim 1, concatenate back
        mp = b.aggregate(b.mesh_partition(b.distribute(v, None), 1), 1)
        return ar, ag0, ag2, rs, mp
    got, want = run_mesh(rt, mesh2, body, [x])
    for i, (g, w) in enumerate(zip(got, want)):
        assert_matches(g, w, f"collective {i}", (0.9999, 1e-5, 1e-5))
    assert torch.allclose(got[0], x[:2] + x[2:], atol=1e-6)
    assert torch.equal(got[1], x) and torch.equal(got[4], x)


def test_decoder_block_tensor_parallel(rt, mesh2):
    kw = dict(seq=256, hidden=512, n_heads=4, n_kv_heads=2, head_dim=128, ffn=1024)
    ins = graphs.decoder_block_inputs(**kw)
    buf = graphs.build_binary(graphs.decoder_block_graph, mesh_shape=(1, 2), tp=2, **kw)
    got = run_program(rt, mesh2, buf, ins)[0]
    want = oracle_results(graphs.decoder_block_graph, ins, mesh_shape=(1, 2), tp=2, **kw)[0]
    assert_matches(got, want, "decoder tp2", (0.999, 2e-2, 2.0 ** -6))


def test_bottleneck_data_parallel(rt, mesh2):
    kw = dict(batch=4, hw=8)
    ins = graphs.bottleneck_inputs(**kw)
    buf = graphs.build_binary(graphs.bottleneck_graph, mesh_shape=(1, 2), dp=2, **kw)
    got = run_program(rt, mesh2, buf, ins)[0]
    want = oracle_results(graphs.bottleneck_graph, ins, mesh_shape=(1, 2), dp=2, **kw)[0]
    assert_matches(got, want, "bottleneck dp2", (0.999, 2e-2, 2.0 ** -6))
    single = oracle_results(graphs.bottleneck_graph, ins, **kw)[0]
    assert torch.equal(want, single)   # data parallelism does not change the numbers


def test_presharded_multi_device_tensors(rt, mesh2):
    # per-device shards handed over as a multi-device host tensor, result read back per shard
    a = [torch.randn(3, 5), torch.randn(3, 5)]

    def graph(b):
        v = b.input([3, 5], "Float32")
        b.output(b.all_reduce(b.relu(v)))
    buf = graphs.build_binary(graph, mesh_shape=(1, 2))
    binary = rt.Binary.load_from_memory(buf)
    host = rt.create_multi_device_host_tensor_from_shards([rt.from_torch(t) for t in a], {}, [1, 2])
    dev_t = rt.to_layout(host, mesh2, rt.get_layout(binary, 0, 0))
    out = rt.submit(mesh2, binary, 0, [dev_t])[0]
    shards = rt.to_host(out, untilize=True)
    assert len(shards) == 2
    want = torch.relu(a[0]) + torch.relu(a[1])
    for s in shards:
        assert torch.allclose(rt.to_torch(s), want, atol=1e-6)
