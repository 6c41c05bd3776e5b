"""Host-side mesh logic on CPU ranks: the sharding helpers and the oracle's collective semantics
against real collectives (gloo, world size 2)."""

import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
from __graft_entry__ import load_package  # noqa: E402  (spawned workers import this module without conftest)

load_package()

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import ops
from ttmlir_b200 import graphs


def _worker(rank, world, port, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(5)
        full = torch.randn(4, 6, generator=g)
        mine = graphs.shard_inputs([full], [0], world, rank)[0]
        # all_reduce(sum) of the shards equals the oracle's all_reduce
        t = mine.clone()
        dist.all_reduce(t)
        want = ops.all_reduce(ops.mesh_shard_full_to_shard(full, world, 0))[rank]
        ok = torch.allclose(t, want)
        # all_gather along dim 0 restores the full tensor, as mesh_shard shard_to_full does
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        ok = ok and torch.equal(torch.cat(parts, 0), full)
        ok = ok and torch.equal(ops.mesh_shard_shard_to_full(parts, 0), full)
        # reduce_scatter = reduce then chunk
        rs = ops.reduce_scatter(ops.mesh_shard_full_to_shard(full, world, None), 1)[rank]
        ok = ok and torch.allclose(rs, torch.chunk(full * world, world, dim=1)[rank])
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_collective_semantics_with_gloo_ranks():
    world = 2
    port = 29500 + (os.getpid() % 2000)
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}


def _moe_worker(rank, world, port, ret):
    """The exchange the runtime performs for the mixture-of-experts ops, replayed with real collectives: dispatch =
    all-gather of tokens and expert indices + a local mask; combine = every rank writes, for every destination, the rows
    of the experts it owns (zeros elsewhere) and a sum reduce-scatter delivers them; the split normalisations exchange one
    statistic per row.  Each against the oracle's per-device results."""
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        g = torch.Generator().manual_seed(11)
        B, S, H, E, K = 4, 3, 8, 4, 2                           # per rank; experts 2r and 2r + 1 live on rank r
        tokens = [torch.randn(B, 1, S, H, generator=g) for _ in range(world)]
        select = [torch.stack([torch.randperm(E, generator=g)[:K] for _ in range(B * S)]).to(torch.int32).reshape(B, 1, S, K)
                  for _ in range(world)]
        mapping = torch.zeros(1, 1, E, world, dtype=torch.int32)
        for e in range(E):
            mapping[0, 0, e, e // 2] = 1
        want_disp, want_meta = ops.all_to_all_dispatch(tokens, select, mapping)
        # dispatch
        parts = [torch.empty(B, 1, S, H) for _ in range(world)]
        dist.all_gather(parts, tokens[rank])
        idx = [torch.empty(B, 1, S, K, dtype=torch.int32) for _ in range(world)]
        dist.all_gather(idx, select[rank])
        full, meta = torch.cat(parts, 0).reshape(1, world * B, S, H), torch.cat(idx, 0).reshape(1, world * B, S, K)
        mine = [e for e in range(E) if int(mapping[0, 0, e, rank])]
        routed = torch.isin(meta, torch.tensor(mine, dtype=torch.int32)).any(-1, keepdim=True)
        disp = torch.where(routed, full, torch.zeros_like(full))
        ok = torch.equal(disp, want_disp[rank]) and torch.equal(meta, want_meta[rank])
        # identity experts: local expert le hands every dispatched row back
        expert_out = torch.stack([disp[0]] * len(mine))           # [E_local, world * B, S, H]
        want_back = ops.all_to_all_combine([torch.stack([d[0]] * 2) for d in want_disp], meta, mapping, K)
        partial = torch.zeros(world, K, B, S, H)
        for p in range(world):
            for slot in range(K):
                for b in range(B):
                    for s_ in range(S):
                        e = int(meta[0, p * B + b, s_, slot])
                        if e in mine:
                            partial[p, slot, b, s_] = expert_out[mine.index(e), p * B + b, s_]
        dist.all_reduce(partial)                                # gloo has no reduce_scatter: reduce everything, keep the own block
        back = partial[rank]
        ok = ok and torch.equal(back, want_back[rank]) and torch.equal(back, torch.stack([tokens[rank].reshape(B, S, H)] * K))
        # distributed rms norm: local sums of squares, one all-reduce of a float per row, local normalisation
        x = [torch.randn(5, 16, generator=g) for _ in range(world)]
        w = [torch.rand(16, generator=g) + 0.5 for _ in range(world)]
        ss = x[rank].square().sum(-1, keepdim=True)
        dist.all_reduce(ss)
        got = x[rank] * torch.rsqrt(ss / (16 * world) + 1e-5) * w[rank]
        ok = ok and torch.allclose(got, ops.distributed_rms_norm(x, w, None, 1e-5)[rank], rtol=1e-6, atol=1e-6)
        # layer norm: pre statistics, all-gather along the last dimension, post
        stats = [torch.empty(5, 64) for _ in range(world)]
        dist.all_gather(stats, ops.layer_norm_pre_all_gather(x[rank], None, torch.float32))
        post = ops.layer_norm_post_all_gather(x[rank], torch.cat(stats, -1), w[rank], None, 1e-5)
        whole = torch.nn.functional.layer_norm(torch.cat(x, -1), [16 * world], torch.cat(w), None, 1e-5)
        ok = ok and torch.allclose(post, whole[:, 16 * rank: 16 * rank + 16], rtol=1e-5, atol=1e-5)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


def test_moe_exchange_and_split_norms_with_gloo_ranks():
    world = 2
    port = 31500 + (os.getpid() % 2000)
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_moe_worker, args=(world, port, ret), nprocs=world, join=True)
        assert dict(ret) == {0: True, 1: True}


def test_tensor_parallel_sharding_covers_every_weight_once():
    kw = dict(seq=64, hidden=128, n_heads=4, n_kv_heads=2, head_dim=32, ffn=256)
    ins = graphs.decoder_block_inputs(**kw)
    dims = graphs.decoder_shard_dims(**kw)
    for tp in (1, 2):
        shards = [graphs.shard_inputs(ins, dims, tp, r) for r in range(tp)]
        for i, (t, d) in enumerate(zip(ins, dims)):
            if d is None:
                assert all(torch.equal(s[i], t) for s in shards)
            else:
                assert torch.equal(torch.cat([s[i] for s in shards], dim=d), t)


def test_tensor_parallel_oracle_matches_single_device():
    kw = dict(seq=64, hidden=128, n_heads=4, n_kv_heads=2, head_dim=32, ffn=256)
    ins = graphs.decoder_block_inputs(**kw)
    from oracle.backend import OracleBuilder
    a = OracleBuilder(ins)
    graphs.decoder_block_graph(a, **kw)
    b = OracleBuilder(ins, mesh_shape=(1, 2))
    graphs.decoder_block_graph(b, tp=2, **kw)
    # the only difference is where the bf16 rounding of the partial sums happens
    assert torch.allclose(a.results()[0].float(), b.results()[0].float(), atol=0.07, rtol=0.02)


def test_mesh_program_structure():
    from ttmlir_b200.schema.fbs import Reader
    from ttmlir_b200.schema.ttnn_schema import S
    buf = graphs.build_binary(graphs.bottleneck_graph, mesh_shape=(1, 2), dp=2, batch=4, hw=8)
    prog = Reader(S, buf).root("TTNNBinary")["programs"][0]
    assert prog["mesh_shape"] == {"y": 1, "x": 2}
    ops_ = [o["type"] for o in prog["operations"]]
    dist_ops = [t for k, t in ops_ if k == "DistributeTensorOp"]
    assert dist_ops[0]["mapper_config"]["placements"] == [{"type": "Replicate", "dim": -1}, {"type": "Shard", "dim": 2}]
    assert all(p["mapper_config"]["placements"][1]["type"] == "Replicate" for p in dist_ops[1:])
    ag = next(t for k, t in ops_ if k == "AllGatherOp")
    assert ag["all_gather_dim"] == 2 and ag["cluster_axis"] == 1
    agg = next(t for k, t in ops_ if k == "AggregateTensorOp")
    assert agg["composer_config"]["dims"] == [0] and agg["composer_config"]["mesh_shape_override"] == [1]


def test_sequence_sharded_io_program_shape():
    """The tensor-parallel decoder program with sequence-sharded I/O: the activations arrive as
    1/N of the sequence, the first mesh op gathers them, the last op hands back this device's rows."""
    from ttmlir_b200.schema.fbs import Reader
    from ttmlir_b200.schema.ttnn_schema import S
    kw = dict(seq=64, hidden=128, n_heads=4, n_kv_heads=2, head_dim=32, ffn=256)
    buf = graphs.build_binary(graphs.decoder_block_graph, mesh_shape=(1, 2), tp=2, presharded=True, io_seq_sharded=True, **kw)
    prog = Reader(S, buf).root("TTNNBinary")["programs"][0]
    kinds = [op["type"][0] for op in prog["operations"] if op["type"][0] not in ("GetDeviceOp", "DeallocateOp")]
    assert kinds[0] == "AllGatherOp" and kinds[-1] == "MeshPartitionOp"
    assert kinds.count("AllReduceOp") == 2
    assert prog["inputs"][0]["desc"]["shape"] == [1, 32, 128]
    assert prog["outputs"][0]["desc"]["shape"] == [1, 32, 128]
    assert prog["mesh_shape"] == {"y": 1, "x": 2}
    dims = graphs.decoder_shard_dims(io_seq_sharded=True, **kw)
    assert dims[0] == 1 and dims[1] is None
    # without the option the activations are replicated and the result is the full sequence
    buf = graphs.build_binary(graphs.decoder_block_graph, mesh_shape=(1, 2), tp=2, presharded=True, **kw)
    prog = Reader(S, buf).root("TTNNBinary")["programs"][0]
    assert prog["inputs"][0]["desc"]["shape"] == [1, 64, 128] and prog["outputs"][0]["desc"]["shape"] == [1, 64, 128]


def test_sequence_sharded_indexer_scores_equal_the_single_device_scores():
    """indexer_score_dsa with the query sequence split over a mesh axis: every device's causal window starts behind the
    rows of the devices before it (the op's description, include/ttmlir/Dialect/TTNN/IR/TTNNOps.td:4378-4385), so the
    gathered scores are those of one device holding the whole sequence."""
    from oracle.backend import OracleBuilder
    torch.manual_seed(23)
    bf = torch.bfloat16
    q, k, w = (torch.randn(1, 4, 32, 64) * 0.3).to(bf), (torch.randn(1, 1, 48, 64) * 0.3).to(bf), torch.randn(1, 4, 32, 1).to(bf)

    def body(b, shard):
        qv, kv, wv = b.input(list(q.shape), "BFloat16"), b.input(list(k.shape), "BFloat16"), b.input(list(w.shape), "BFloat16")
        if not shard:
            return b.output(b.indexer_score_dsa(qv, kv, wv, 16))
        qs, ws = b.distribute(qv, 2), b.distribute(wv, 2)
        b.output(b.aggregate(b.indexer_score_dsa(qs, kv, ws, 16, cluster_axis=1), 2))
    whole = OracleBuilder([q, k, w])
    body(whole, False)
    split = OracleBuilder([q, k, w], mesh_shape=(1, 4))
    body(split, True)
    assert torch.equal(whole.results()[0], split.results()[0])
    assert torch.isneginf(whole.results()[0][0, 0, 0, 17:]).all() and torch.isfinite(whole.results()[0][0, 0, 31]).all()
    buf = graphs.build_binary(lambda b: body(b, True), mesh_shape=(1, 4))       # the same program as a flatbuffer
    assert len(buf) > 0
