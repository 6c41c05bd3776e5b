"""Generates tests/golden/ttir_cpu_golden.npz by running the reference's own CPU code.

Run where a checkout of tenstorrent/tt-mlir is available (path as the argument, or in the
TT_MLIR_ROOT environment variable):

    python tests/golden/generate.py /path/to/tt-mlir

It imports two files of the reference, unmodified, and records what their functions return on
small seeded inputs:

* tools/tt-alchemist/templates/python/local/ttir_cpu.py -- the pure-torch CPU implementation of
  the TTIR ops that the reference's CPU-hoist path targets;
* tools/golden/mapping.py -- the torch goldens of every op, for the ops that have no CPU lowering
  (quantization, rms_norm, attention, mesh_shard and the collectives, kv-cache ops, decode and
  paged attention, gather / scatter / sort / top-k).  That file imports the compiler's Python
  bindings; ttmlir_standin.py supplies attribute and type classes in their place, so the golden
  bodies that run are the reference's own text.

A third source, for the one op whose golden lives in a test file that cannot be imported (it needs the compiler's
builder): test/python/golden/ttir_ops/fusing/test_rope_fusing.py -- its `rotate_half` and `torch_rope` functions are
compiled from that file's own syntax tree (lift_functions), nothing else of the file runs.

Nothing in this script restates a golden.  The fixture travels with the repo; the reference tree
does not.  Two things have no golden to call and are recorded from torch directly, marked below:
per-axis quantization (torch.quantize_per_channel) and nothing else.
bf16 tensors are stored as their uint16 bit patterns.
"""

import importlib.util
import os
import sys

import numpy as np
import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import ttmlir_standin as standin  # noqa: E402


def load_ttir_cpu(root):
    path = os.path.join(root, "tools/tt-alchemist/templates/python/local/ttir_cpu.py")
    spec = importlib.util.spec_from_file_location("ttir_cpu_reference", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def lift_functions(path, names):
    """Compiles the named top-level functions of a Python file from its own syntax tree and returns them; the rest of
    the file (imports of the compiler's builder, test bodies) is not executed."""
    import ast
    with open(path) as f:
        tree = ast.parse(f.read(), path)
    ns = {"torch": torch}
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name in names:
            exec(compile(ast.Module([node], []), path, "exec"), ns)
    missing = [n for n in names if n not in ns]
    if missing:
        raise SystemExit(f"{path} no longer defines {missing}")
    return [ns[n] for n in names]


def store(out, name, t):
    if t.dtype == torch.bfloat16:
        out[name + "@bf16"] = t.contiguous().view(torch.uint16).numpy()
    else:
        out[name] = t.contiguous().numpy()


def main():
    root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("TT_MLIR_ROOT", "")
    if not root:
        raise SystemExit("usage: generate.py /path/to/tt-mlir")
    cpu = load_ttir_cpu(root)
    ref = standin.load_mapping(root)      # tools/golden/mapping.py, imported unmodified

    def gmt(t, mesh=(1, 1)):
        """A single-device value in the wrapper the goldens take."""
        return ref.GoldenMapTensor({0: t}, mesh)

    def one(v):
        return v.shard_at(0) if isinstance(v, ref.GoldenMapTensor) else v
    g = torch.Generator().manual_seed(1234)
    out = {}

    def rnd(*shape, scale=1.0):
        return torch.randn(*shape, generator=g) * scale

    # --- eltwise unary (ttir_cpu.py:94-232), f32
    x = rnd(7, 33) * 2
    store(out, "unary/x", x)
    for name in ["abs", "ceil", "cos", "floor", "gelu", "neg", "relu", "sigmoid", "sin", "sign", "tan", "tanh", "atan",
                 "exp", "erf", "erfc", "expm1", "relu6", "silu", "hardsigmoid", "mish", "asinh", "cbrt", "leaky_relu"]:
        store(out, f"unary/{name}", getattr(cpu, name)(x))
    xp = x.abs() + 0.1
    store(out, "unary/xpos", xp)
    for name in ["sqrt", "rsqrt", "reciprocal", "log", "log1p"]:
        store(out, f"unary/{name}", getattr(cpu, name)(xp))
    xu = torch.rand(7, 33, generator=g) * 1.8 - 0.9
    store(out, "unary/xunit", xu)
    for name in ["acos", "asin"]:
        store(out, f"unary/{name}", getattr(cpu, name)(xu))

    # --- eltwise binary with broadcasting (ttir_cpu.py:240-330)
    a, b = rnd(4, 5, 16), rnd(5, 16)
    b = torch.where(b.abs() < 0.05, torch.full_like(b, 0.5), b)
    store(out, "binary/a", a)
    store(out, "binary/b", b)
    for name in ["add", "subtract", "multiply", "div", "maximum", "minimum", "eq", "ne", "gt", "ge", "lt", "le"]:
        r = getattr(cpu, name)(a, b)
        store(out, f"binary/{name}", r.to(torch.float32))
    row = rnd(16)
    store(out, "binary/row", row)
    store(out, "binary/add_row", cpu.add(a, row))

    # --- matmul / linear (ttir_cpu.py:509-521)
    A, B, bias = rnd(37, 50), rnd(50, 29), rnd(29)
    store(out, "mm/a", A)
    store(out, "mm/b", B)
    store(out, "mm/bias", bias)
    store(out, "mm/matmul", cpu.matmul(A, B))
    store(out, "mm/linear", cpu.linear(A, B, bias))
    Bt = rnd(29, 50)
    store(out, "mm/bt", Bt)
    store(out, "mm/linear_tb", cpu.linear(A, Bt, bias, transpose_b=True))
    Ab, Bb = rnd(3, 8, 12), rnd(3, 12, 5)
    store(out, "mm/ab", Ab)
    store(out, "mm/bb", Bb)
    store(out, "mm/batched", cpu.matmul(Ab, Bb))

    # --- softmax (ttir_cpu.py:585)
    s = rnd(6, 10, 3) * 3
    store(out, "softmax/x", s)
    store(out, "softmax/last", cpu.softmax(s, dim=-1))
    store(out, "softmax/mid", cpu.softmax(s, dim=1))

    # --- reductions (ttir_cpu.py:374-397)
    r = rnd(3, 6, 8)
    store(out, "reduce/x", r)
    store(out, "reduce/sum_last", cpu.sum(r, dim=[2], keepdim=False))
    store(out, "reduce/mean_mid_keep", cpu.mean(r, dim=[1], keepdim=True))
    store(out, "reduce/max_last", cpu.max(r, dim=[2], keepdim=False))
    store(out, "reduce/min_first", cpu.min(r, dim=[0], keepdim=False))
    store(out, "reduce/sum_all", cpu.sum(r).reshape(1))

    # --- conv2d, NHWC activations / OIHW weights / bias [1,1,1,O] (ttir_cpu.py:772-815)
    cx, cw, cb = rnd(2, 9, 7, 8), rnd(6, 8, 3, 3) * 0.2, rnd(1, 1, 1, 6)
    store(out, "conv/x", cx)
    store(out, "conv/w", cw)
    store(out, "conv/b", cb)
    store(out, "conv/same", cpu.conv2d(cx, cw, cb, stride=(1, 1), padding=(1, 1, 1, 1)))
    store(out, "conv/stride2_asym", cpu.conv2d(cx, cw, cb, stride=(2, 2), padding=(0, 1, 1, 2)))
    cw1 = rnd(5, 8, 1, 1)
    store(out, "conv/w1", cw1)
    store(out, "conv/pointwise", cpu.conv2d(cx, cw1, None))

    # --- head split / merge (ttir_cpu.py:824-877)
    qkv = rnd(2, 6, (4 + 2 * 2) * 8)
    store(out, "heads/qkv", qkv)
    q, k, v = cpu.split_query_key_value_and_split_heads(qkv, None, num_heads=4, num_kv_heads=2)
    store(out, "heads/q", q)
    store(out, "heads/k", k)
    store(out, "heads/v", v)
    store(out, "heads/merged", cpu.concatenate_heads(q))

    # --- typecast (ttir_cpu.py:498)
    tc = rnd(5, 9) * 40
    store(out, "cast/x", tc)
    store(out, "cast/to_bf16", cpu.typecast(tc, torch.bfloat16))
    store(out, "cast/to_i32", cpu.typecast(tc, torch.int32))

    # --- quantization: quantize_golden / requantize_golden (tools/golden/mapping.py:2534-2582) and the
    #     registered golden of ttir.dequantize (torch.dequantize, mapping.py:9166), called as imported
    from ttmlir.dialects import ttir as ttir_ops   # the stand-in's op classes are the registry's keys
    dequantize_golden = ref.GOLDEN_MAPPINGS[ttir_ops.DequantizeOp]
    qx = (torch.randn(64, 48, generator=g)).to(torch.bfloat16)
    ties = torch.tensor([0.25, 0.75, 1.25, 3.0, -3.0, 0.01, -0.01, 0.03, -0.05, 2.55, -2.57, 100.0], dtype=torch.bfloat16)
    qx.view(-1)[: ties.numel()] = ties
    store(out, "quant/x", qx)
    for tag, scale, zp in [("s002_z0", 0.02, 0), ("s0037_z3", 0.037, 3)]:
        store(out, f"quant/{tag}/q_i8", ref.quantize_golden(qx.float(), scale, zp, torch.qint8))
        store(out, f"quant/{tag}/q_i32", ref.quantize_golden(qx.float(), scale, zp, torch.qint32))
        q8 = torch.quantize_per_tensor(qx.float(), scale, zp, torch.qint8)   # the quantized value the next goldens take
        store(out, f"quant/{tag}/deq", dequantize_golden(q8))
        rq = ref.requantize_golden(q8, scale * 2, zp + 1, torch.qint8)
        store(out, f"quant/{tag}/requant_i8", rq.int_repr())
        store(out, f"quant/{tag}/requant_deq", dequantize_golden(rq))
    # per-axis quantization has no golden in mapping.py (only the formula in TTIROps.td:6010-6013);
    # torch's per-channel quantizer is recorded as its stand-in
    ch_scale = torch.rand(64, generator=g) * 0.05 + 0.01
    store(out, "quant/ch_scale", ch_scale)
    qc = torch.quantize_per_channel(qx.float(), ch_scale.double(), torch.zeros(64, dtype=torch.int64), 0, torch.qint8)
    store(out, "quant/per_channel_q", qc.int_repr())
    store(out, "quant/per_channel_deq", torch.dequantize(qc))

    # --- rms_norm: ttir_rms_norm_golden (mapping.py:1265-1288)
    nx = rnd(5, 64).to(torch.bfloat16)
    nw = (1 + rnd(64) * 0.1).to(torch.bfloat16)
    store(out, "rms/x", nx)
    store(out, "rms/w", nw)
    store(out, "rms/out", one(ref.ttir_rms_norm_golden(gmt(nx), gmt(nw), None, standin.ArrayAttr([64]), standin.FloatAttr(1e-5),
                                                       standin.BF16Type())))

    # --- scaled dot product attention: ttir_sdpa_golden (mapping.py:8398-8500), grouped-query heads
    aq, ak, av = rnd(1, 4, 10, 16), rnd(1, 2, 10, 16), rnd(1, 2, 10, 16)
    store(out, "sdpa/q", aq)
    store(out, "sdpa/k", ak)
    store(out, "sdpa/v", av)
    for name, causal in (("causal", True), ("full", False)):
        store(out, f"sdpa/{name}", one(ref.ttir_sdpa_golden(gmt(aq), gmt(ak), gmt(av), None, standin.BoolAttr(causal), None,
                                                            standin.F32Type())))

    # --- layer_norm, argmax, cumsum, embedding, pad (ttir_cpu.py: layer_norm, argmax, cumsum, embedding, pad), f32
    lx, lw, lb = rnd(6, 4, 48), 1 + rnd(48) * 0.1, rnd(48) * 0.1
    store(out, "ln/x", lx)
    store(out, "ln/w", lw)
    store(out, "ln/b", lb)
    store(out, "ln/plain", cpu.layer_norm(lx, epsilon=1e-5))
    store(out, "ln/affine", cpu.layer_norm(lx, epsilon=1e-5, weight=lw, bias=lb))
    lw2 = 1 + rnd(4, 48) * 0.1
    store(out, "ln/w2", lw2)
    store(out, "ln/two_dims", cpu.layer_norm(lx, epsilon=1e-3, weight=lw2))
    ax = rnd(5, 7, 9)
    ax[1, 2, :] = ax[1, 2, 3]            # ties: the first index wins
    store(out, "arg/x", ax)
    for d in (0, 1, 2):
        store(out, f"arg/dim{d}", cpu.argmax(ax, dim=[d]))
    store(out, "arg/all", cpu.argmax(ax))
    store(out, "arg/keep", cpu.argmax(ax, dim=[1], keepdim=True))
    cx = rnd(4, 33, 5)
    store(out, "cum/x", cx)
    for d in (0, 1, 2):
        store(out, f"cum/dim{d}", cpu.cumsum(cx, dim=d))
    ci = torch.randint(-50, 50, (6, 40), generator=g, dtype=torch.int32)
    store(out, "cum/xi", ci)
    store(out, "cum/int", cpu.cumsum(ci, dim=1))
    ei = torch.randint(0, 30, (3, 11), generator=g, dtype=torch.int32)
    ew = rnd(1, 1, 30, 24)
    store(out, "emb/idx", ei)
    store(out, "emb/w", ew)
    store(out, "emb/out", cpu.embedding(ei, ew))
    px = rnd(2, 3, 5)
    store(out, "pad/x", px)
    store(out, "pad/out", cpu.pad(px, [1, 0, 0, 2, 3, 1], value=-1.5))

    # --- pooling over NHWC (ttir_cpu.py: max_pool2d, avg_pool2d, global_avg_pool2d); the reference's
    #     padding order at this level is (top, bottom, left, right)
    pool_x = rnd(2, 9, 11, 8)
    store(out, "pool/x", pool_x)
    flat = pool_x.reshape(1, 1, -1, 8)
    store(out, "pool/max_k2s2", cpu.max_pool2d(flat, 2, 9, 11, 8, [2, 2], [2, 2], [0, 0]))
    store(out, "pool/max_k3s2p1", cpu.max_pool2d(flat, 2, 9, 11, 8, [3, 3], [2, 2], [1, 1]))
    store(out, "pool/max_k3s2p1_ceil", cpu.max_pool2d(flat, 2, 9, 11, 8, [3, 3], [2, 2], [1, 1], ceil_mode=True))
    store(out, "pool/max_k3s1_dil2", cpu.max_pool2d(flat, 2, 9, 11, 8, [3, 3], [1, 1], [1, 1], dilation=[2, 2]))
    store(out, "pool/max_asym", cpu.max_pool2d(flat, 2, 9, 11, 8, [3, 2], [2, 1], [1, 0, 2, 1]))          # t, b, l, r
    store(out, "pool/max_asym_ceil", cpu.max_pool2d(flat, 2, 9, 11, 8, [3, 3], [2, 2], [0, 1, 0, 1], ceil_mode=True))
    store(out, "pool/avg_k2s2", cpu.avg_pool2d(flat, 2, 9, 11, 8, [2, 2], [2, 2], [0, 0]))
    store(out, "pool/avg_k3s2p1", cpu.avg_pool2d(flat, 2, 9, 11, 8, [3, 3], [2, 2], [1, 1]))
    store(out, "pool/avg_k3s2p1_nopad", cpu.avg_pool2d(flat, 2, 9, 11, 8, [3, 3], [2, 2], [1, 1], count_include_pad=False))
    store(out, "pool/avg_k3s2p1_ceil", cpu.avg_pool2d(flat, 2, 9, 11, 8, [3, 3], [2, 2], [1, 1], ceil_mode=True))
    store(out, "pool/avg_k3s2p1_ceil_nopad",
          cpu.avg_pool2d(flat, 2, 9, 11, 8, [3, 3], [2, 2], [1, 1], ceil_mode=True, count_include_pad=False))
    store(out, "pool/avg_asym", cpu.avg_pool2d(flat, 2, 9, 11, 8, [3, 3], [2, 2], [1, 0, 2, 1]))
    store(out, "pool/avg_asym_nopad", cpu.avg_pool2d(flat, 2, 9, 11, 8, [3, 3], [2, 2], [1, 0, 2, 1], count_include_pad=False))
    store(out, "pool/avg_bigpad", cpu.avg_pool2d(flat, 2, 9, 11, 8, [2, 2], [2, 2], [2, 2]))
    store(out, "pool/avg_bigpad_nopad", cpu.avg_pool2d(flat, 2, 9, 11, 8, [2, 2], [2, 2], [2, 2], count_include_pad=False))
    store(out, "pool/global", cpu.global_avg_pool2d(pool_x))

    # ===== goldens of tools/golden/mapping.py for ops with no CPU-hoist lowering, called as imported =====
    S = standin

    # --- more attention cases: additive mask, explicit scale, bf16 result (ttir_sdpa_golden)
    bq, bk, bv = rnd(2, 8, 24, 32).to(torch.bfloat16), rnd(2, 2, 40, 32).to(torch.bfloat16), rnd(2, 2, 40, 32).to(torch.bfloat16)
    bm = rnd(2, 1, 24, 40)
    for n, t in (("q", bq), ("k", bk), ("v", bv), ("mask", bm)):
        store(out, f"map/sdpa2/{n}", t)
    store(out, "map/sdpa2/masked", one(ref.ttir_sdpa_golden(gmt(bq), gmt(bk), gmt(bv), gmt(bm), S.BoolAttr(False),
                                                           S.FloatAttr(0.2), S.BF16Type())))
    store(out, "map/sdpa2/full", one(ref.ttir_sdpa_golden(gmt(bq), gmt(bk), gmt(bv), None, S.BoolAttr(False), None, S.BF16Type())))
    store(out, "map/sdpa2/causal_sq", one(ref.ttir_sdpa_golden(gmt(bq), gmt(bk[:, :, :24]), gmt(bv[:, :, :24]), None,
                                                              S.BoolAttr(True), None, S.BF16Type())))

    # --- rms_norm with a bias, f32 and bf16 (ttir_rms_norm_golden)
    rx, rw, rb = rnd(3, 7, 96), 1 + rnd(96) * 0.1, rnd(96) * 0.1
    for n, t in (("x", rx), ("w", rw), ("b", rb)):
        store(out, f"map/rms/{n}", t)
    store(out, "map/rms/f32_bias", one(ref.ttir_rms_norm_golden(gmt(rx), gmt(rw), gmt(rb), S.ArrayAttr([96]), S.FloatAttr(1e-6),
                                                               S.F32Type())))
    store(out, "map/rms/bf16_noweight", one(ref.ttir_rms_norm_golden(gmt(rx.to(torch.bfloat16)), None, None, S.ArrayAttr([96]),
                                                                    S.FloatAttr(1e-5), S.BF16Type())))

    # --- mesh_shard and the collectives on a 1x4 and a 2x2 mesh (mapping.py:4189-4235, 5658-5794)
    def sharded(t, mesh, dims):
        return ref.ttir_mesh_shard_golden(ref.GoldenMapTensor({0: t}, mesh), S.MeshShardTypeAttr(S.MeshShardType.Devices),
                                          S.MeshShardDirectionAttr(S.MeshShardDirection.FullToShard), S.DenseI64ArrayAttr([1, 1]),
                                          S.DenseI64ArrayAttr(dims), S.type_of(t.dtype))

    def store_shards(name, v):
        for i in sorted(v.shard_map):
            store(out, f"{name}/{i}", v.shard_at(i))
    mx = rnd(8, 12, 16)
    store(out, "map/mesh/x", mx)
    mxb = mx.to(torch.bfloat16)
    for mesh, dims, tag in (((1, 4), [-1, 0], "1x4_d0"), ((1, 4), [-1, 2], "1x4_d2"), ((2, 2), [0, 1], "2x2_d01")):
        sh = sharded(mx, mesh, dims)
        store_shards(f"map/mesh/{tag}/shards", sh)
        back = ref.ttir_mesh_shard_golden(sh, S.MeshShardTypeAttr(S.MeshShardType.Devices),
                                          S.MeshShardDirectionAttr(S.MeshShardDirection.ShardToFull), S.DenseI64ArrayAttr([1, 1]),
                                          S.DenseI64ArrayAttr(dims), S.F32Type())
        store(out, f"map/mesh/{tag}/full", one(back))
        for axis in ((1,) if mesh[0] == 1 else (0, 1)):
            for rt_name in ("Sum", "Max", "Min", "Mean"):
                r = ref.ttir_all_reduce_golden(sh, S.ReduceTypeAttr(S.ReduceType[rt_name]), S.IntegerAttr(axis), S.F32Type())
                store_shards(f"map/mesh/{tag}/all_reduce_{rt_name}_axis{axis}", r)
            store_shards(f"map/mesh/{tag}/all_gather_dim1_axis{axis}",
                         ref.ttir_all_gather_golden(sh, S.IntegerAttr(1), S.IntegerAttr(axis), S.F32Type()))
            store_shards(f"map/mesh/{tag}/reduce_scatter_dim1_axis{axis}",
                         ref.ttir_reduce_scatter_golden(sh, S.ReduceTypeAttr(S.ReduceType.Sum), S.IntegerAttr(1), S.IntegerAttr(axis),
                                                        S.F32Type()))
            store_shards(f"map/mesh/{tag}/mesh_partition_dim1_axis{axis}",
                         ref.ttir_mesh_partition_golden(sh, S.IntegerAttr(1), S.IntegerAttr(axis), S.F32Type()))
    shb = sharded(mxb, (1, 4), [-1, 0])
    store_shards("map/mesh/bf16_1x4_d0/all_reduce_Sum_axis1",
                 ref.ttir_all_reduce_golden(shb, S.ReduceTypeAttr(S.ReduceType.Sum), S.IntegerAttr(1), S.BF16Type()))
    rep = ref.ttir_mesh_shard_golden(ref.GoldenMapTensor({0: mx}, (1, 4)), S.MeshShardTypeAttr(S.MeshShardType.Replicate),
                                     S.MeshShardDirectionAttr(S.MeshShardDirection.FullToShard), S.DenseI64ArrayAttr([1, 1]),
                                     S.DenseI64ArrayAttr([-1, -1]), S.F32Type())
    store_shards("map/mesh/replicate_1x4", rep)

    # --- kv-cache ops and decode attention (mapping.py:3582-3670, 2417-2482)
    cache = rnd(4, 2, 64, 16)
    fill_in = rnd(1, 2, 40, 16)
    store(out, "map/cache/cache", cache)
    store(out, "map/cache/fill_in", fill_in)
    store(out, "map/cache/filled_user0", one(ref.fill_cache_golden(gmt(cache[:1].clone()), gmt(fill_in))))
    upd = rnd(1, 2, 4, 16)
    store(out, "map/cache/update_in", upd)
    store(out, "map/cache/updated_idx7", one(ref.update_cache_golden(gmt(cache.clone()), gmt(upd), gmt(torch.tensor([7], dtype=torch.int32)))))
    upd2 = rnd(1, 2, 2, 16)
    store(out, "map/cache/update_in2", upd2)
    store(out, "map/cache/updated_idx63_off2", one(ref.update_cache_golden(gmt(cache.clone()), gmt(upd2), gmt(torch.tensor([63], dtype=torch.int32)),
                                                                          batch_offset=S.IntegerAttr(2))))
    dq = rnd(1, 3, 8, 32).to(torch.bfloat16)
    dk, dv = rnd(3, 2, 96, 32).to(torch.bfloat16), rnd(3, 2, 96, 32).to(torch.bfloat16)
    pos = torch.tensor([5, 95, 40], dtype=torch.int32)
    dmask = rnd(3, 1, 8, 96)
    for n, t in (("q", dq), ("k", dk), ("v", dv), ("pos", pos), ("mask", dmask)):
        store(out, f"map/decode/{n}", t)
    store(out, "map/decode/causal", one(ref.sdpa_decode_golden(gmt(dq), gmt(dk), gmt(dv), gmt(pos), None, True, 32 ** -0.5)))
    store(out, "map/decode/masked", one(ref.sdpa_decode_golden(gmt(dq), gmt(dk), gmt(dv), None, gmt(dmask), False, 32 ** -0.5)))

    # --- gather / scatter / sort / top-k (mapping.py:5384-5437, 5624-5640, 5927-5958)
    gx = rnd(5, 9, 6)
    gi = torch.randint(0, 9, (5, 4, 6), generator=g, dtype=torch.int32)
    store(out, "map/gather/x", gx)
    store(out, "map/gather/idx_dim1", gi)
    store(out, "map/gather/dim1", one(ref.ttir_gather_golden(gmt(gx), gmt(gi), S.IntegerAttr(1), S.F32Type())))
    gi2 = torch.randint(0, 6, (5, 9, 3), generator=g, dtype=torch.int32)
    store(out, "map/gather/idx_dim2", gi2)
    store(out, "map/gather/dim2", one(ref.ttir_gather_golden(gmt(gx), gmt(gi2), S.IntegerAttr(2), S.F32Type())))
    # scatter: unique indices along the scatter dimension, so the result does not depend on write order
    si = torch.stack([torch.randperm(9, generator=g)[:4] for _ in range(5 * 6)]).reshape(5, 6, 4).permute(0, 2, 1).contiguous().to(torch.int32)
    ssrc = rnd(5, 4, 6)
    store(out, "map/scatter/idx", si)
    store(out, "map/scatter/src", ssrc)
    # the plain (no reduction) scatter is what ttnn.scatter computes; the golden selects it by ReduceType.Invalid
    store(out, "map/scatter/dim1", one(ref.ttir_scatter_golden(gmt(gx), gmt(si), gmt(ssrc), S.IntegerAttr(1),
                                                               S.ReduceTypeAttr(S.ReduceType.Invalid), S.F32Type())))
    store(out, "map/scatter/dim1_sum", one(ref.ttir_scatter_golden(gmt(gx), gmt(si), gmt(ssrc), S.IntegerAttr(1),
                                                                   S.ReduceTypeAttr(S.ReduceType.Sum), S.F32Type())))
    sx = rnd(6, 50)
    sx[2, 10] = sx[2, 30]                 # a tie: stable order keeps index 10 first
    store(out, "map/sort/x", sx)
    for desc in (False, True):
        vals, idx = ref.ttir_sort_golden(gmt(sx), S.IntegerAttr(-1), S.BoolAttr(desc), S.BoolAttr(True), S.F32Type())
        store(out, f"map/sort/values_desc{int(desc)}", one(vals))
        store(out, f"map/sort/indices_desc{int(desc)}", one(idx).to(torch.int32))
    vals, idx = ref.ttir_sort_golden(gmt(sx), S.IntegerAttr(0), S.BoolAttr(False), S.BoolAttr(True), S.F32Type())
    store(out, "map/sort/values_dim0", one(vals))
    store(out, "map/sort/indices_dim0", one(idx).to(torch.int32))
    tx = rnd(4, 3, 200).to(torch.bfloat16)
    store(out, "map/topk/x", tx)
    for k, largest in ((8, True), (32, True), (5, False)):
        vals, idx = ref.ttir_topk_golden(gmt(tx.float()), S.IntegerAttr(k), S.IntegerAttr(-1), S.BoolAttr(largest), S.BoolAttr(True),
                                         S.F32Type())
        store(out, f"map/topk/values_k{k}_l{int(largest)}", one(vals))
        store(out, f"map/topk/indices_k{k}_l{int(largest)}", one(idx).to(torch.int32))

    # --- paged caches and paged decode attention (mapping.py:8745-8844, 8926-9007)
    pcache = rnd(12, 2, 16, 32).to(torch.bfloat16)            # 12 blocks of 16 tokens
    ptable = torch.tensor([[3, 7, 1, 0], [5, 2, 9, 11], [4, 6, 8, 10]], dtype=torch.int32)
    store(out, "map/paged/cache", pcache)
    store(out, "map/paged/page_table", ptable)
    pin = rnd(3, 1, 2, 32).to(torch.bfloat16)                 # [batch, seq 1, heads, d]
    ppos = torch.tensor([17, 0, 63], dtype=torch.int32)
    store(out, "map/paged/update_in", pin)
    store(out, "map/paged/update_pos", ppos)
    store(out, "map/paged/updated", one(ref.ttir_paged_update_cache_golden(gmt(pcache.clone()), gmt(pin), gmt(ppos), S.BoolAttr(False),
                                                                           gmt(ptable), S.BF16Type())))
    pfill = rnd(1, 2, 40, 32).to(torch.bfloat16)              # one user's prompt
    store(out, "map/paged/fill_in", pfill)
    store(out, "map/paged/filled_user1", one(ref.ttir_paged_fill_cache_golden(gmt(pcache.clone()), gmt(pfill), gmt(ptable),
                                                                             gmt(torch.tensor([1], dtype=torch.int32)), S.BF16Type())))
    pv = rnd(12, 2, 16, 32).to(torch.bfloat16)
    pq = rnd(3, 1, 8, 32).to(torch.bfloat16)                  # [batch, seq 1, heads, d]
    store(out, "map/paged/v_cache", pv)
    store(out, "map/paged/q", pq)
    store(out, "map/paged/decode", one(ref.ttir_paged_sdpa_decode_golden(gmt(pq), gmt(pcache), gmt(pv), gmt(ptable), gmt(pq), S.BoolAttr(True),
                                                                         None, gmt(ppos), None, None, None, S.BF16Type())))

    # --- cumprod, prod, inference batch norm, upsampling (mapping.py:4308-4314, 2858-2900, 4948-4976, 3552-3578)
    cx = (rnd(4, 12, 5) * 0.5 + 1.0)
    store(out, "map/cumprod/x", cx)
    for d in (0, 1, 2):
        store(out, f"map/cumprod/dim{d}", one(ref.ttir_cumprod_golden(gmt(cx), S.IntegerAttr(d), S.F32Type())))
    cxb = cx.to(torch.bfloat16)
    store(out, "map/cumprod/x_bf16", cxb)
    store(out, "map/cumprod/bf16_dim1", one(ref.ttir_cumprod_golden(gmt(cxb), S.IntegerAttr(1), S.BF16Type())))
    ci = torch.randint(-3, 4, (3, 7), generator=g, dtype=torch.int32)
    store(out, "map/cumprod/x_i32", ci)
    store(out, "map/cumprod/i32_dim1", one(ref.ttir_cumprod_golden(gmt(ci), S.IntegerAttr(1), S.IntegerType(32))))
    store(out, "map/prod/all", one(ref.prod_golden(gmt(cx))).reshape(1))
    store(out, "map/prod/dim1", one(ref.prod_golden(gmt(cx), dim_arg=[1], keep_dim=False)))
    store(out, "map/prod/dim2_keep", one(ref.prod_golden(gmt(cx), dim_arg=[2], keep_dim=True)))
    store(out, "map/prod/i32_dim0", one(ref.prod_golden(gmt(ci), dim_arg=[0], keep_dim=False)).to(torch.int32))
    bx = rnd(3, 6, 5, 7)
    bmean, bvar = rnd(6) * 0.3, torch.rand(6, generator=g) + 0.5
    bw, bb = rnd(6) * 0.5 + 1.0, rnd(6) * 0.2
    for n, t in (("x", bx), ("mean", bmean), ("var", bvar), ("weight", bw), ("bias", bb)):
        store(out, f"map/batch_norm/{n}", t)
    store(out, "map/batch_norm/out", one(ref.ttir_batch_norm_inference_golden(gmt(bx), gmt(bw), gmt(bb), gmt(bmean), gmt(bvar),
                                                                             S.FloatAttr(1e-5), S.IntegerAttr(1), S.F32Type())))
    bxb = bx.to(torch.bfloat16)
    store(out, "map/batch_norm/out_bf16", one(ref.ttir_batch_norm_inference_golden(
        gmt(bxb), gmt(bw.to(torch.bfloat16)), gmt(bb.to(torch.bfloat16)), gmt(bmean.to(torch.bfloat16)), gmt(bvar.to(torch.bfloat16)),
        S.FloatAttr(1e-5), S.IntegerAttr(1), S.BF16Type())))
    ux = rnd(2, 6, 6, 5)                                        # NHWC, square (the golden's transpose assumes it)
    store(out, "map/upsample/x", ux)
    for mode in ("nearest", "bilinear"):
        spec = torch.empty(2, 12, 12, 5)
        store(out, f"map/upsample/{mode}_x2", one(ref.upsample2d_golden(gmt(ux), gmt(spec), 2, mode=mode)))
    spec3 = torch.empty(2, 18, 18, 5)
    store(out, "map/upsample/nearest_x3", one(ref.upsample2d_golden(gmt(ux), gmt(spec3), 3, mode="nearest")))

    # --- group_norm (channels-last), conv_transpose2d, conv1d (mapping.py:1541-1574, 804-893, 502-574)
    gx = rnd(2, 1, 20, 12)
    gw, gb = rnd(12) * 0.5 + 1.0, rnd(12) * 0.2
    for n, t in (("x", gx), ("weight", gw), ("bias", gb)):
        store(out, f"map/group_norm/{n}", t)
    store(out, "map/group_norm/g3", one(ref.ttir_group_norm_golden(gmt(gx), gmt(gw), gmt(gb), S.IntegerAttr(3), S.FloatAttr(1e-5), S.F32Type())))
    store(out, "map/group_norm/g12_noaffine", one(ref.ttir_group_norm_golden(gmt(gx), None, None, S.IntegerAttr(12), S.FloatAttr(1e-5),
                                                                            S.F32Type())))
    tx = rnd(2, 5, 6, 8)                                        # NHWC
    tw, tb = rnd(8, 6, 3, 3) * 0.3, rnd(1, 1, 1, 6) * 0.1       # [C_in, C_out, kH, kW]
    for n, t in (("x", tx), ("w", tw), ("b", tb)):
        store(out, f"map/conv_transpose/{n}", t)
    nhwc = (S.IntegerAttr(0), S.IntegerAttr(1), S.IntegerAttr(2), S.IntegerAttr(3))
    store(out, "map/conv_transpose/s2_p1_op1", one(ref.conv_transpose2d_golden(
        gmt(tx), gmt(tw), gmt(tb), S.DenseI32ArrayAttr([2, 2]), S.DenseI32ArrayAttr([1, 1]), S.DenseI32ArrayAttr([1, 1]),
        S.DenseI32ArrayAttr([1, 1]), S.IntegerAttr(1), *nhwc)))
    twg = rnd(8, 3, 2, 3) * 0.3                                 # groups 2: [C_in, C_out / 2, kH, kW]
    store(out, "map/conv_transpose/w_g2", twg)
    store(out, "map/conv_transpose/g2_s1x2_d2", one(ref.conv_transpose2d_golden(
        gmt(tx), gmt(twg), None, S.DenseI32ArrayAttr([1, 2]), S.DenseI32ArrayAttr([0, 1]), S.DenseI32ArrayAttr([0, 0]),
        S.DenseI32ArrayAttr([2, 1]), S.IntegerAttr(2), *nhwc)))
    ox = rnd(3, 17, 8)                                          # NLC
    ow, ob = rnd(10, 8, 4) * 0.3, rnd(1, 1, 10) * 0.1
    for n, t in (("x", ox), ("w", ow), ("b", ob)):
        store(out, f"map/conv1d/{n}", t)
    nlc = (S.IntegerAttr(0), S.IntegerAttr(1), S.IntegerAttr(2))
    store(out, "map/conv1d/s2_p1x2", one(ref.conv1d_golden(gmt(ox), gmt(ow), gmt(ob), S.IntegerAttr(2), S.DenseI32ArrayAttr([1, 2]),
                                                           S.IntegerAttr(1), S.IntegerAttr(1), *nlc)))

    # --- training batch norm (reuses the batch_norm inputs) and max_pool2d with indices (mapping.py:4979-5063, 5339-5378)
    tr = ref.ttir_batch_norm_training_golden(gmt(bx), gmt(bw), gmt(bb), gmt(bmean), gmt(bvar), S.FloatAttr(1e-5), S.IntegerAttr(1),
                                             S.FloatAttr(0.1), S.F32Type(), S.F32Type(), S.F32Type())
    for n, t in zip(("out", "new_mean", "new_var"), tr):
        store(out, f"map/batch_norm_training/{n}", one(t))
    mx = rnd(2, 9, 11, 6)                                       # NHWC
    store(out, "map/max_pool_indices/x", mx)
    for name, (k, st, pd, dl, ceil) in {"k3_s2_p1": ([3, 3], [2, 2], [1, 1, 1, 1], [1, 1], False),
                                       "k2x3_s1x2_d2_ceil": ([2, 3], [1, 2], [0, 1, 0, 1], [2, 1], True)}.items():
        v, ix = ref.ttir_max_pool2d_with_indices(gmt(mx), S.DenseI32ArrayAttr(k), S.DenseI32ArrayAttr(st), S.DenseI32ArrayAttr(pd),
                                                 S.DenseI32ArrayAttr(dl), S.BoolAttr(ceil), S.F32Type())
        store(out, f"map/max_pool_indices/{name}", one(v))
        store(out, f"map/max_pool_indices/{name}_idx", one(ix).to(torch.int32))

    # --- split normalisations (mapping.py:1291-1415, 7800-7921)
    nx, nres = rnd(6, 96), rnd(6, 96) * 0.5
    nw, nb = rnd(96) * 0.5 + 1.0, rnd(96) * 0.2
    for n, t in (("x", nx), ("residual", nres), ("weight", nw), ("bias", nb)):
        store(out, f"map/split_norm/{n}", t)
    store(out, "map/split_norm/dit_silu", one(ref.dit_rms_norm_unary_fused_golden(gmt(nx), gmt(nw), gmt(nb), gmt(nres), None, 1e-5, "silu")))
    store(out, "map/split_norm/dit_plain", one(ref.dit_rms_norm_unary_fused_golden(gmt(nx), gmt(nw), None, None, None, 1e-6, None)))
    store(out, "map/split_norm/rms_pre", one(ref.ttnn_rms_norm_pre_all_gather_golden(gmt(nx), gmt(nres), S.F32Type())))
    store(out, "map/split_norm/ln_pre", one(ref.ttnn_layer_norm_pre_all_gather_golden(gmt(nx), None, None, S.F32Type())))
    store(out, "map/split_norm/ln_post_1dev", one(ref.ttnn_layer_norm_post_all_gather_golden(
        gmt(nx), gmt(torch.zeros(6, 64)), gmt(nw), gmt(nb), S.FloatAttr(1e-5), S.F32Type())))
    xsh, rsh, wsh = sharded(nx, (1, 4), [-1, 1]), sharded(nres, (1, 4), [-1, 1]), sharded(nw, (1, 4), [-1, 0])
    store_shards("map/split_norm/dist_rms_1x4", ref.ttir_distributed_rms_norm_golden(xsh, wsh, rsh, S.IntegerAttr(1), S.FloatAttr(1e-5),
                                                                                     S.F32Type()))

    # --- mixture of experts (mapping.py:1596-1760, 2030-2150)
    sa, sb = rnd(2, 3, 32, 48).to(torch.bfloat16), (rnd(1, 4, 48, 40) * 0.2).to(torch.bfloat16)
    store(out, "map/moe/spmm_a", sa)
    store(out, "map/moe/spmm_b", sb)
    store(out, "map/moe/spmm_b_sparse", one(ref.ttir_sparse_matmul_golden(gmt(sa), gmt(sb), None, S.BoolAttr(False), S.BoolAttr(True), None,
                                                                          S.BF16Type())))
    sa2 = rnd(3, 4, 32, 48).to(torch.bfloat16)
    store(out, "map/moe/spmm_a2", sa2)
    store(out, "map/moe/spmm_a_sparse", one(ref.ttir_sparse_matmul_golden(gmt(sa2), gmt(sb), None, S.BoolAttr(True), S.BoolAttr(False), None,
                                                                          S.BF16Type())))
    # dispatch on a 1x4 mesh: 6 tokens per device, hidden 16, 2 of 8 experts per token, experts 2d and 2d+1 on device d
    D, Mt, Hh, Kk, Ee = 4, 6, 16, 2, 8
    tok = rnd(D * Mt, Hh)
    sel = torch.stack([torch.randperm(Ee, generator=g)[:Kk] for _ in range(D * Mt)]).to(torch.int32)
    scr = torch.rand(D * Mt, Kk, generator=g)
    store(out, "map/moe/tokens", tok)
    store(out, "map/moe/selected", sel)
    shard4 = lambda t: ref.GoldenMapTensor({d: t[d * Mt:(d + 1) * Mt].reshape(1, 1, Mt, -1).clone() for d in range(D)}, (1, D))
    owner = (torch.arange(Ee) // 2).to(torch.int32).reshape(1, 1, 1, Ee).repeat(1, 1, D, 1)        # entry [d, e] = owning device
    disp, idx_all, scr_all = ref.ttir_all_to_all_dispatch_metadata_golden(
        shard4(tok), shard4(sel), shard4(scr), ref.GoldenMapTensor({d: owner.clone() for d in range(D)}, (1, D)),
        S.IntegerAttr(D), S.IntegerAttr(1), S.F32Type(), S.IntegerType(32), S.F32Type())
    store_shards("map/moe/dispatched_1x4", disp)
    store(out, "map/moe/indices_gathered", idx_all.shard_at(0))
    # combine on one device: 4 experts, all local; 3 x 5 tokens, 2 slots
    cin = rnd(4, 3, 5, 16)
    cmeta = torch.stack([torch.randperm(4, generator=g)[:2] for _ in range(15)]).to(torch.int32).reshape(1, 3, 5, 2)
    store(out, "map/moe/combine_in", cin)
    store(out, "map/moe/combine_meta", cmeta)
    store(out, "map/moe/combine_out", one(ref.ttir_all_to_all_combine_golden(
        gmt(cin), gmt(cmeta), gmt(torch.ones(1, 1, 4, 1, dtype=torch.int32)), S.IntegerAttr(1), S.IntegerAttr(1), S.IntegerAttr(2),
        S.F32Type())))

    # --- GPT-OSS router (mapping.py:5960-5992): 32 tokens, hidden 64, 16 experts, top 4
    rx, rw, rb = rnd(32, 64).to(torch.bfloat16), (rnd(64, 16) * 0.3).to(torch.bfloat16), (rnd(32, 16) * 0.1).to(torch.bfloat16)
    for n, t in (("x", rx), ("w", rw), ("b", rb)):
        store(out, f"map/router/{n}", t)
    ridx, rwts = ref.ttir_topk_router_gpt_golden(gmt(rx), gmt(rw), gmt(rb), S.IntegerAttr(4), S.IntegerAttr(16), S.BF16Type())
    store(out, "map/router/indices", one(ridx).to(torch.int32))
    store(out, "map/router/weights", one(rwts))
    store(out, "map/moe/scores", scr)
    store(out, "map/moe/scores_gathered", scr_all.shard_at(0))

    # --- conv3d, gelu backward, embedding backward, adamw (mapping.py:714-801, 4379-4383, 5875-5912, 1155-1218)
    vx = rnd(2, 4, 5, 6, 8)                                     # NDHWC
    vw, vb = rnd(6, 4, 2, 3, 3) * 0.3, rnd(1, 1, 1, 1, 6) * 0.1  # groups 2: [O, C/2, kD, kH, kW]
    for n, t in (("x", vx), ("w", vw), ("b", vb)):
        store(out, f"map/conv3d/{n}", t)
    ndhwc = (S.IntegerAttr(0), S.IntegerAttr(1), S.IntegerAttr(2), S.IntegerAttr(3), S.IntegerAttr(4))
    store(out, "map/conv3d/s1x2x1_p1_g2", one(ref.conv3d_golden(gmt(vx), gmt(vw), gmt(vb), S.DenseI32ArrayAttr([1, 2, 1]),
                                                                S.DenseI32ArrayAttr([1, 1, 1]), S.IntegerAttr(2), *ndhwc, S.StringAttr("zeros"))))
    gg, gx = rnd(5, 40), rnd(5, 40) * 2
    store(out, "map/gelu_bw/grad", gg)
    store(out, "map/gelu_bw/x", gx)
    for ap in ("none", "tanh"):
        store(out, f"map/gelu_bw/{ap}", one(ref.ttir_gelu_backward_golden(gmt(gg), gmt(gx), approximate=ap)))
    ei = torch.randint(0, 10, (3, 7), generator=g, dtype=torch.int32)
    eg = rnd(3, 7, 16)
    store(out, "map/embedding_bw/indices", ei)
    store(out, "map/embedding_bw/grad", eg)
    store(out, "map/embedding_bw/out", one(ref.ttir_embedding_backward_golden(gmt(ei), gmt(torch.zeros(10, 16)), gmt(eg), S.F32Type())))
    ap_, ag = rnd(6, 50), rnd(6, 50).to(torch.bfloat16)
    am, av, amax = rnd(6, 50) * 0.1, torch.rand(6, 50, generator=g) * 0.01, torch.rand(6, 50, generator=g) * 0.01
    for n, t in (("param", ap_), ("grad", ag), ("m", am), ("v", av), ("vmax", amax)):
        store(out, f"map/adamw/{n}", t)
    for tag, vm in (("plain", None), ("amsgrad", amax)):
        res = ref.adamw_golden(gmt(ap_), gmt(ag), gmt(am), gmt(av), gmt(vm) if vm is not None else None, lr=1e-2, beta1=0.9, beta2=0.99,
                               beta1_pow=0.9 ** 3, beta2_pow=0.99 ** 3, epsilon=1e-8, weight_decay=0.1)
        for n, t in zip(("param", "m", "v", "vmax"), res):
            store(out, f"map/adamw/{tag}/{n}", one(t))

    # --- chunked prefill attention over a paged cache (mapping.py:8847-8912): 2 users, 4 q / 2 kv heads, block 16, 5 blocks each
    cq = rnd(2, 4, 24, 32)
    ck, cv = rnd(12, 2, 16, 32), rnd(12, 2, 16, 32)
    cpt = torch.stack([torch.randperm(12, generator=g)[:5] for _ in range(2)]).to(torch.int32)
    for n, t in (("q", cq), ("k", ck), ("v", cv), ("page_table", cpt)):
        store(out, f"map/chunked_sdpa/{n}", t)
    for start in (0, 40):
        store(out, f"map/chunked_sdpa/start{start}", one(ref.ttir_chunked_scaled_dot_product_attention_golden(
            gmt(cq), gmt(ck), gmt(cv), gmt(cpt), gmt(torch.tensor([start], dtype=torch.int32)), None, S.FloatAttr(0.2), S.F32Type())))

    # --- multi-latent attention prefill (mapping.py:8662-8692): 4 q / 1 kv heads, 24 tokens, 48-wide keys, 32-wide values
    lq, lk = rnd(2, 4, 24, 48), rnd(2, 1, 24, 48)
    lmask = torch.where(torch.rand(1, 1, 24, 24, generator=g) < 0.3, torch.tensor(float("-inf")), torch.tensor(0.0))
    lmask[..., 0] = 0.0                                        # no fully masked row
    for n, t in (("q", lq), ("k", lk), ("mask", lmask)):
        store(out, f"map/mla/{n}", t)
    store(out, "map/mla/causal", one(ref.flash_mla_prefill_golden(gmt(lq), gmt(lk), None, None, 32, True, None)))
    store(out, "map/mla/masked", one(ref.flash_mla_prefill_golden(gmt(lq), gmt(lk), None, gmt(lmask), 32, True, 0.2)))
    lv = rnd(2, 1, 24, 16)
    store(out, "map/mla/v", lv)
    store(out, "map/mla/own_values", one(ref.flash_mla_prefill_golden(gmt(lq), gmt(lk), gmt(lv), None, 16, False, None)))

    # --- paged multi-latent decode attention (mapping.py:8275-8365): 3 users, 4 heads on one latent head, block 8, 4 blocks each
    dq, dk = rnd(1, 3, 4, 48) * 0.5, rnd(14, 1, 8, 48) * 0.5
    dpt = torch.stack([torch.randperm(14, generator=g)[:4] for _ in range(3)]).to(torch.int32)
    dpos = torch.tensor([5, 31, 17], dtype=torch.int32)
    for n, t in (("q", dq), ("k", dk), ("page_table", dpt), ("cur_pos", dpos)):
        store(out, f"map/mla_decode/{n}", t)
    store(out, "map/mla_decode/latent", one(ref.ttir_paged_flash_multi_latent_attention_decode_golden(
        gmt(dq), gmt(dk), None, gmt(dpt), None, gmt(dpos), None, S.IntegerAttr(32), S.BoolAttr(True), None, S.F32Type())))
    dv = rnd(14, 1, 8, 16)
    store(out, "map/mla_decode/v", dv)
    store(out, "map/mla_decode/own_values", one(ref.ttir_paged_flash_multi_latent_attention_decode_golden(
        gmt(dq), gmt(dk), gmt(dv), gmt(dpt), None, gmt(dpos), None, S.IntegerAttr(16), S.BoolAttr(True), S.FloatAttr(0.15), S.F32Type())))

    # --- lightning-indexer scores of DeepSeek sparse attention (mapping.py:8695-8742): the shapes of the reference's own
    # test (test/python/golden/test_stablehlo_ops.py:2560-2596), dense and as the last chunk of a longer history, plus a
    # ragged case (5 heads, 19 queries, 75 keys) that fills no tile
    iq, ik, iw = (rnd(1, 8, 64, 128) * 0.3).to(torch.bfloat16), (rnd(1, 1, 128, 128) * 0.3).to(torch.bfloat16), rnd(1, 8, 64, 1).to(torch.bfloat16)
    for n, t in (("q", iq), ("k", ik), ("w", iw)):
        store(out, f"map/indexer/{n}", t)
    store(out, "map/indexer/dense", one(ref.indexer_score_dsa_golden(gmt(iq), gmt(ik), gmt(iw), 0)))
    store(out, "map/indexer/chunked", one(ref.indexer_score_dsa_golden(gmt(iq), gmt(ik), gmt(iw), 64)))
    rq, rk, rw = (rnd(2, 5, 19, 40) * 0.3).to(torch.bfloat16), (rnd(2, 1, 75, 40) * 0.3).to(torch.bfloat16), rnd(2, 5, 19, 1).to(torch.bfloat16)
    for n, t in (("q", rq), ("k", rk), ("w", rw)):
        store(out, f"map/indexer/ragged_{n}", t)
    store(out, "map/indexer/ragged", one(ref.indexer_score_dsa_golden(gmt(rq), gmt(rk), gmt(rw), 30)))

    # --- rotary embedding: the golden of the reference's fusing test (test_rope_fusing.py:23-33), cos / sin [1, S, D]
    # reshaped to [1, 1, S, D] and broadcast over batch and heads as the test's builder does; f32, and bf16 operands
    # evaluated in f32 with one rounding (the fused op's arithmetic)
    (torch_rope,) = lift_functions(os.path.join(root, "test/python/golden/ttir_ops/fusing/test_rope_fusing.py"), ["rotate_half", "torch_rope"])[1:]
    px = rnd(2, 4, 24, 64)
    ang = torch.arange(24, dtype=torch.float32).view(24, 1) * torch.pow(10000.0, -torch.arange(32, dtype=torch.float32) / 32).view(1, 32)
    pcos, psin = torch.cos(torch.cat([ang, ang], dim=-1)).view(1, 24, 64), torch.sin(torch.cat([ang, ang], dim=-1)).view(1, 24, 64)
    for n, t in (("x", px), ("cos", pcos), ("sin", psin)):
        store(out, f"rope/{n}", t)
    store(out, "rope/f32", torch_rope(px, pcos.view(1, 1, 24, 64), psin.view(1, 1, 24, 64)))
    bx, bc, bs = px.to(torch.bfloat16), pcos.to(torch.bfloat16), psin.to(torch.bfloat16)
    store(out, "rope/bf16_operands", torch_rope(bx.float(), bc.float().view(1, 1, 24, 64), bs.float().view(1, 1, 24, 64)).to(torch.bfloat16))

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ttir_cpu_golden.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    main()
