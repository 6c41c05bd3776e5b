"""Pins the CPU oracle (oracle/ops.py) against outputs of the reference's own code recorded in
tests/golden/ttir_cpu_golden.npz by tests/golden/generate.py: its CPU implementation of the TTIR
ops (ttir_cpu.py) and, under "map/", "quant/", "rms/" and "sdpa/", its torch goldens
(tools/golden/mapping.py) imported unmodified."""

import pytest
import torch

from oracle import metrics, ops

UNARY = {"abs": "Abs", "ceil": "Ceil", "cos": "Cos", "floor": "Floor", "gelu": "Gelu", "neg": "Neg", "relu": "Relu",
         "sigmoid": "Sigmoid", "sin": "Sin", "sign": "Sign", "tan": "Tan", "tanh": "Tanh", "atan": "Atan", "exp": "Exp",
         "erf": "Erf", "erfc": "Erfc", "expm1": "Expm1", "relu6": "Relu6", "silu": "Silu", "hardsigmoid": "Hardsigmoid",
         "mish": "Mish", "asinh": "Asinh", "cbrt": "Cbrt", "leaky_relu": "LeakyRelu"}
UNARY_POS = {"sqrt": "Sqrt", "rsqrt": "Rsqrt", "reciprocal": "Reciprocal", "log": "Log", "log1p": "Log1p"}
UNARY_UNIT = {"acos": "Acos", "asin": "Asin"}
BINARY = {"add": "Add", "subtract": "Subtract", "multiply": "Multiply", "div": "Divide", "maximum": "Maximum",
          "minimum": "Minimum", "eq": "Equal", "ne": "NotEqual", "gt": "GreaterThan", "ge": "GreaterEqual",
          "lt": "LessThan", "le": "LessEqual"}


def same(a, b):
    return torch.equal(a, b) or torch.allclose(a.float(), b.float(), rtol=0, atol=0, equal_nan=True)


@pytest.mark.parametrize("name", sorted(UNARY))
def test_unary(golden, name):
    assert same(ops.unary(UNARY[name], golden["unary/x"]), golden[f"unary/{name}"])


@pytest.mark.parametrize("name", sorted(UNARY_POS))
def test_unary_positive(golden, name):
    assert same(ops.unary(UNARY_POS[name], golden["unary/xpos"]), golden[f"unary/{name}"])


@pytest.mark.parametrize("name", sorted(UNARY_UNIT))
def test_unary_unit(golden, name):
    assert same(ops.unary(UNARY_UNIT[name], golden["unary/xunit"]), golden[f"unary/{name}"])


@pytest.mark.parametrize("name", sorted(BINARY))
def test_binary(golden, name):
    got = ops.binary(BINARY[name], golden["binary/a"], golden["binary/b"])
    assert same(got, golden[f"binary/{name}"])


def test_binary_row_broadcast(golden):
    assert same(ops.binary("Add", golden["binary/a"], golden["binary/row"]), golden["binary/add_row"])


def test_matmul_linear(golden):
    a, b, bias = golden["mm/a"], golden["mm/b"], golden["mm/bias"]
    assert same(ops.matmul(a, b), golden["mm/matmul"])
    assert same(ops.linear(a, b, bias), golden["mm/linear"])
    assert same(ops.linear(a, golden["mm/bt"], bias, transpose_b=True), golden["mm/linear_tb"])
    assert same(ops.matmul(golden["mm/ab"], golden["mm/bb"]), golden["mm/batched"])


def test_softmax(golden):
    assert same(ops.softmax(golden["softmax/x"], -1), golden["softmax/last"])
    assert same(ops.softmax(golden["softmax/x"], 1), golden["softmax/mid"])


def test_reductions(golden):
    x = golden["reduce/x"]
    assert same(ops.reduce("Sum", x, [2], False), golden["reduce/sum_last"])
    assert same(ops.reduce("Mean", x, [1], True), golden["reduce/mean_mid_keep"])
    assert same(ops.reduce("Max", x, [2], False), golden["reduce/max_last"])
    assert same(ops.reduce("Min", x, [0], False), golden["reduce/min_first"])
    assert same(ops.reduce("Sum", x, None, False).reshape(1), golden["reduce/sum_all"])


def test_conv2d(golden):
    x, w, b = golden["conv/x"], golden["conv/w"], golden["conv/b"]
    assert same(ops.conv2d(x, w, b, 2, 9, 7, (1, 1), (1, 1, 1, 1)), golden["conv/same"])
    assert same(ops.conv2d(x, w, b, 2, 9, 7, (2, 2), (0, 1, 1, 2)), golden["conv/stride2_asym"])
    assert same(ops.conv2d(x, golden["conv/w1"], None, 2, 9, 7), golden["conv/pointwise"])
    # the flattened [1,1,N*H*W,C] form the compiler emits gives the same numbers
    flat = ops.conv2d(x.reshape(1, 1, -1, 8), w, b, 2, 9, 7, (1, 1), (1, 1, 1, 1))
    assert same(flat.reshape(golden["conv/same"].shape), golden["conv/same"])


def test_heads(golden):
    q, k, v = ops.split_qkv(golden["heads/qkv"], None, 4, 2)
    assert same(q, golden["heads/q"]) and same(k, golden["heads/k"]) and same(v, golden["heads/v"])
    assert same(ops.concatenate_heads(q), golden["heads/merged"])


def test_typecast(golden):
    x = golden["cast/x"]
    assert same(ops.typecast(x, torch.bfloat16), golden["cast/to_bf16"])
    assert same(ops.typecast(x, torch.int32), golden["cast/to_i32"])


@pytest.mark.parametrize("tag,scale,zp", [("s002_z0", 0.02, 0), ("s0037_z3", 0.037, 3)])
def test_quantization_bit_exact(golden, tag, scale, zp):
    x = golden["quant/x"]
    q8 = ops.quantize(x, scale, zp, torch.int8)
    assert torch.equal(q8, golden[f"quant/{tag}/q_i8"])
    # int32 container, values clamped to the int8 range (how the compiler stores quantized tensors)
    assert torch.equal(ops.quantize(x, scale, zp, torch.int32, clamp_i8=True), golden[f"quant/{tag}/q_i8"].to(torch.int32))
    assert torch.equal(ops.quantize(x, scale, zp, torch.int32, clamp_i8=False), golden[f"quant/{tag}/q_i32"])
    assert torch.equal(ops.dequantize(q8, scale, zp), golden[f"quant/{tag}/deq"])
    rq = ops.requantize(q8, scale, zp, scale * 2, zp + 1)
    assert torch.equal(rq, golden[f"quant/{tag}/requant_i8"])
    assert torch.equal(ops.dequantize(rq, scale * 2, zp + 1), golden[f"quant/{tag}/requant_deq"])


def test_quantization_ties_round_to_even(golden):
    x = golden["quant/x"].reshape(-1)[:5]
    q = ops.quantize(x, 0.02, 0, torch.int8)
    assert q.tolist() == [12, 38, 62, 127, -128]  # 12.5 -> 12, 37.5 -> 38, 62.5 -> 62, clamps


def test_quantization_per_channel(golden):
    x, s = golden["quant/x"], golden["quant/ch_scale"]
    q = ops.quantize_per_axis(x, s, None, 0, torch.int8)
    assert torch.equal(q, golden["quant/per_channel_q"])
    assert torch.equal(ops.dequantize_per_axis(q, s, None, 0), golden["quant/per_channel_deq"])


def test_rms_norm(golden):
    assert same(ops.rms_norm(golden["rms/x"], golden["rms/w"], None, 1e-5), golden["rms/out"])


def test_sdpa(golden):
    q, k, v = golden["sdpa/q"], golden["sdpa/k"], golden["sdpa/v"]
    assert torch.allclose(ops.sdpa(q, k, v, True), golden["sdpa/causal"], atol=1e-6)
    assert torch.allclose(ops.sdpa(q, k, v, False), golden["sdpa/full"], atol=1e-6)


def test_sdpa_mask_scale_and_bf16(golden):
    """ttir_sdpa_golden as imported from the reference (tests/golden/generate.py): additive mask with
    an explicit scale, grouped-query heads with Sq != Skv, causal; bf16 in and out."""
    q, k, v, m = (golden[f"map/sdpa2/{n}"] for n in ("q", "k", "v", "mask"))
    assert torch.equal(ops.sdpa(q, k, v, False, m, 0.2), golden["map/sdpa2/masked"])
    assert torch.equal(ops.sdpa(q, k, v, False), golden["map/sdpa2/full"])
    assert torch.equal(ops.sdpa(q, k[:, :, :24], v[:, :, :24], True), golden["map/sdpa2/causal_sq"])


def test_rms_norm_bias_and_no_weight(golden):
    x, w, b = golden["map/rms/x"], golden["map/rms/w"], golden["map/rms/b"]
    assert same(ops.rms_norm(x, w, b, 1e-6), golden["map/rms/f32_bias"])
    assert same(ops.rms_norm(x.to(torch.bfloat16), None, None, 1e-5), golden["map/rms/bf16_noweight"])


def _shards(golden, name, n):
    return [golden[f"{name}/{i}"] for i in range(n)]


@pytest.mark.parametrize("tag,dim", [("1x4_d0", 0), ("1x4_d2", 2)])
def test_mesh_shard_and_collectives_on_a_row_mesh(golden, tag, dim):
    """mesh_shard, all_reduce (sum / max / min / mean), all_gather, reduce_scatter and mesh_partition
    against the reference's goldens on a 1x4 mesh."""
    x = golden["map/mesh/x"]
    base = f"map/mesh/{tag}"
    sh = ops.mesh_shard_full_to_shard(x, 4, dim)
    for got, want in zip(sh, _shards(golden, base + "/shards", 4)):
        assert torch.equal(got, want)
    assert torch.equal(ops.mesh_shard_shard_to_full(sh, dim), golden[base + "/full"])
    for code, name in enumerate(("Sum", "Mean", "Max", "Min")):
        for got, want in zip(ops.all_reduce(sh, code), _shards(golden, f"{base}/all_reduce_{name}_axis1", 4)):
            assert torch.equal(got, want), name
    for got, want in zip(ops.all_gather(sh, 1), _shards(golden, base + "/all_gather_dim1_axis1", 4)):
        assert torch.equal(got, want)
    for got, want in zip(ops.reduce_scatter(sh, 1), _shards(golden, base + "/reduce_scatter_dim1_axis1", 4)):
        assert torch.equal(got, want)
    for got, want in zip(ops.mesh_partition(sh, 1), _shards(golden, base + "/mesh_partition_dim1_axis1", 4)):
        assert torch.equal(got, want)


def test_collectives_bf16_and_replicate(golden):
    x = golden["map/mesh/x"]
    sh = ops.mesh_shard_full_to_shard(x.to(torch.bfloat16), 4, 0)
    for got, want in zip(ops.all_reduce(sh, 0), _shards(golden, "map/mesh/bf16_1x4_d0/all_reduce_Sum_axis1", 4)):
        assert torch.equal(got, want)
    for got, want in zip(ops.mesh_shard_full_to_shard(x, 4, None), _shards(golden, "map/mesh/replicate_1x4", 4)):
        assert torch.equal(got, want)


def test_collectives_on_a_2x2_mesh(golden):
    """Both cluster axes of a 2x2 mesh: a group is a row (axis 1) or a column (axis 0) of devices."""
    x = golden["map/mesh/x"]
    base = "map/mesh/2x2_d01"
    rows = torch.chunk(x, 2, dim=0)
    sh = [c.contiguous() for r in rows for c in torch.chunk(r, 2, dim=1)]
    for got, want in zip(sh, _shards(golden, base + "/shards", 4)):
        assert torch.equal(got, want)
    groups = {1: [[0, 1], [2, 3]], 0: [[0, 2], [1, 3]]}
    for axis, gs in groups.items():
        for g in gs:
            mine = [sh[i] for i in g]
            for j, i in enumerate(g):
                assert torch.equal(ops.all_reduce(mine, 0)[j], golden[f"{base}/all_reduce_Sum_axis{axis}/{i}"])
                assert torch.equal(ops.all_gather(mine, 1)[j], golden[f"{base}/all_gather_dim1_axis{axis}/{i}"])
                assert torch.equal(ops.reduce_scatter(mine, 1)[j], golden[f"{base}/reduce_scatter_dim1_axis{axis}/{i}"])
                assert torch.equal(ops.mesh_partition(mine, 1)[j], golden[f"{base}/mesh_partition_dim1_axis{axis}/{i}"])


def test_cache_ops_and_decode_attention(golden):
    """fill_cache, update_cache and decode attention against the reference's goldens."""
    cache = golden["map/cache/cache"]
    assert torch.equal(ops.fill_cache(cache[:1], golden["map/cache/fill_in"]), golden["map/cache/filled_user0"])
    assert torch.equal(ops.update_cache(cache, golden["map/cache/update_in"], torch.tensor([7])), golden["map/cache/updated_idx7"])
    assert torch.equal(ops.update_cache(cache, golden["map/cache/update_in2"], torch.tensor([63]), batch_offset=2),
                       golden["map/cache/updated_idx63_off2"])
    q, k, v, pos, m = (golden[f"map/decode/{n}"] for n in ("q", "k", "v", "pos", "mask"))
    assert torch.equal(ops.sdpa_decode(q, k, v, pos, None, True, 32 ** -0.5), golden["map/decode/causal"])
    assert torch.equal(ops.sdpa_decode(q, k, v, None, m, False, 32 ** -0.5), golden["map/decode/masked"])


def test_gather_scatter_sort_topk(golden):
    x = golden["map/gather/x"]
    assert torch.equal(ops.gather(x, golden["map/gather/idx_dim1"], 1), golden["map/gather/dim1"])
    assert torch.equal(ops.gather(x, golden["map/gather/idx_dim2"], 2), golden["map/gather/dim2"])
    idx, src = golden["map/scatter/idx"], golden["map/scatter/src"]
    assert torch.equal(ops.scatter(x, idx, src, 1), golden["map/scatter/dim1"])
    assert torch.equal(ops.scatter(x, idx, src, 1, "Sum"), golden["map/scatter/dim1_sum"])
    sx = golden["map/sort/x"]
    for desc in (False, True):
        v, i = ops.sort(sx, -1, desc)
        assert torch.equal(v, golden[f"map/sort/values_desc{int(desc)}"]) and torch.equal(i, golden[f"map/sort/indices_desc{int(desc)}"])
    v, i = ops.sort(sx, 0)
    assert torch.equal(v, golden["map/sort/values_dim0"]) and torch.equal(i, golden["map/sort/indices_dim0"])
    tx = golden["map/topk/x"].float()
    for k, largest in ((8, True), (32, True), (5, False)):
        v, i = ops.topk(tx, k, -1, largest)
        assert torch.equal(v, golden[f"map/topk/values_k{k}_l{int(largest)}"])
        assert torch.equal(i, golden[f"map/topk/indices_k{k}_l{int(largest)}"])


def test_paged_cache_and_paged_decode(golden):
    cache, table = golden["map/paged/cache"], golden["map/paged/page_table"]
    pos = golden["map/paged/update_pos"]
    assert torch.equal(ops.paged_update_cache(cache, golden["map/paged/update_in"], pos, table), golden["map/paged/updated"])
    assert torch.equal(ops.paged_fill_cache(cache, golden["map/paged/fill_in"], table, torch.tensor([1])), golden["map/paged/filled_user1"])
    got = ops.paged_sdpa_decode(golden["map/paged/q"], cache, golden["map/paged/v_cache"], table, pos)
    assert torch.equal(got, golden["map/paged/decode"])


def test_cumprod_prod_batch_norm_upsample(golden):
    """The restatements of cumprod, prod, inference batch norm and 2-D upsampling against the outputs of the reference's
    own goldens (tools/golden/mapping.py:4308-4314, 2858-2900, 4948-4976, 3552-3578), recorded by generate.py."""
    x = golden["map/cumprod/x"]
    for d in (0, 1, 2):
        assert torch.equal(ops.cumprod(x, d), golden[f"map/cumprod/dim{d}"])
    assert torch.equal(ops.cumprod(golden["map/cumprod/x_bf16"], 1), golden["map/cumprod/bf16_dim1"])
    xi = golden["map/cumprod/x_i32"]
    assert torch.equal(ops.cumprod(xi, 1), golden["map/cumprod/i32_dim1"])
    assert torch.equal(ops.prod(x).reshape(1), golden["map/prod/all"])
    assert torch.equal(ops.prod(x, 1), golden["map/prod/dim1"])
    assert torch.equal(ops.prod(x, 2, True), golden["map/prod/dim2_keep"])
    assert torch.equal(ops.prod(xi, 0).to(torch.int32), golden["map/prod/i32_dim0"])
    bx, mean, var, w, b = (golden[f"map/batch_norm/{n}"] for n in ("x", "mean", "var", "weight", "bias"))
    assert torch.equal(ops.batch_norm_inference(bx, mean, var, w, b, 1e-5), golden["map/batch_norm/out"])
    bf = torch.bfloat16
    # bf16: the golden lets torch evaluate in bf16; the CPU-hoist model (and the kernel) evaluates in f32 and rounds once
    got = ops.batch_norm_inference(bx.to(bf), mean.to(bf), var.to(bf), w.to(bf), b.to(bf), 1e-5)
    ok, report = metrics.check_close(golden["map/batch_norm/out_bf16"], got, 0.999, 2e-2, 2.0 ** -6)
    assert ok, report
    ux = golden["map/upsample/x"]
    assert torch.equal(ops.upsample2d(ux, 2, "nearest"), golden["map/upsample/nearest_x2"])
    assert torch.equal(ops.upsample2d(ux, 3, "nearest"), golden["map/upsample/nearest_x3"])
    assert torch.allclose(ops.upsample2d(ux, 2, "bilinear"), golden["map/upsample/bilinear_x2"], atol=1e-6, rtol=0)


def test_group_norm_conv_transpose_conv1d(golden):
    """Restatements against the reference's goldens (tools/golden/mapping.py:1541-1574, 804-893, 502-574)."""
    x, w, b = (golden[f"map/group_norm/{n}"] for n in ("x", "weight", "bias"))
    assert torch.equal(ops.group_norm(x, w, b, 3, 1e-5), golden["map/group_norm/g3"])
    assert torch.equal(ops.group_norm(x, None, None, 12, 1e-5), golden["map/group_norm/g12_noaffine"])
    x, w, b = (golden[f"map/conv_transpose/{n}"] for n in ("x", "w", "b"))
    assert torch.equal(ops.conv_transpose2d(x, w, b, 2, 5, 6, (2, 2), (1, 1), (1, 1), (1, 1), 1), golden["map/conv_transpose/s2_p1_op1"])
    assert torch.equal(ops.conv_transpose2d(x, golden["map/conv_transpose/w_g2"], None, 2, 5, 6, (1, 2), (0, 1), (0, 0), (2, 1), 2),
                       golden["map/conv_transpose/g2_s1x2_d2"])
    x, w, b = (golden[f"map/conv1d/{n}"] for n in ("x", "w", "b"))
    assert torch.equal(ops.conv1d(x, w, b, 2, (1, 2), 1, 1), golden["map/conv1d/s2_p1x2"])


def test_batch_norm_training_and_max_pool_indices(golden):
    """Restatements against the reference's goldens (tools/golden/mapping.py:4979-5063, 5339-5378)."""
    x, mean, var, w, b = (golden[f"map/batch_norm/{n}"] for n in ("x", "mean", "var", "weight", "bias"))
    y, m, v = ops.batch_norm_training(x, mean, var, w, b, 1e-5, 0.1)
    assert torch.allclose(y, golden["map/batch_norm_training/out"], rtol=1e-6, atol=1e-6)
    assert torch.allclose(m, golden["map/batch_norm_training/new_mean"], rtol=1e-6, atol=1e-7)
    assert torch.allclose(v, golden["map/batch_norm_training/new_var"], rtol=1e-6, atol=1e-7)
    x = golden["map/max_pool_indices/x"]
    for name, args in {"k3_s2_p1": ((3, 3), (2, 2), (1, 1), (1, 1), False), "k2x3_s1x2_d2_ceil": ((2, 3), (1, 2), (0, 1), (2, 1), True)}.items():
        val, idx = ops.max_pool2d_with_indices(x.reshape(1, 1, -1, 6), 2, 9, 11, 6, *args)
        want = golden[f"map/max_pool_indices/{name}"]
        assert torch.equal(val.reshape(want.shape), want)
        assert torch.equal(idx.reshape(want.shape).to(torch.int32), golden[f"map/max_pool_indices/{name}_idx"])


def test_decode_head_ops_and_llama_rotary():
    """The decode-step head ops are pure data movement; the llama rotary embedding with the pair-swap matrix equals the
    interleaved-pair rotation written out by hand."""
    torch.manual_seed(0)
    x = torch.randn(1, 1, 5, (4 + 2 * 2) * 8)
    q, k, v = ops.nlp_create_qkv_heads_decode(x, 4, 2)
    assert q.shape == (1, 5, 4, 8) and k.shape == (1, 5, 2, 8) and v.shape == (1, 5, 2, 8)
    assert torch.equal(q[0, 3, 2], x[0, 0, 3, 16:24]) and torch.equal(k[0, 1, 1], x[0, 0, 1, 40:48]) and torch.equal(v[0, 4, 0], x[0, 0, 4, 48:56])
    q2, _, _ = ops.nlp_create_qkv_heads_decode(x, 4, 2, batch_offset=2, slice_size=2)
    assert torch.equal(q2, q[:, 2:4])
    h = torch.randn(1, 5, 32, 8)
    assert torch.equal(ops.nlp_concat_heads_decode(h, 3)[0, 0, 4], h[0, 4, :3].reshape(-1))
    t = torch.zeros(32, 32)
    for i in range(0, 32, 2):                                   # (a, b) -> (-b, a)
        t[i, i + 1] = 1.0
        t[i + 1, i] = -1.0
    xs = torch.randn(1, 2, 6, 64)
    ang = torch.rand(1, 1, 6, 32).repeat_interleave(2, dim=-1)
    y = ops.rotary_embedding_llama(xs, torch.cos(ang), torch.sin(ang), t.reshape(1, 1, 32, 32), False)
    a, b = xs[..., 0::2], xs[..., 1::2]
    c, s_ = torch.cos(ang)[..., 0::2], torch.sin(ang)[..., 0::2]
    assert torch.allclose(y[..., 0::2], a * c - b * s_, atol=1e-6) and torch.allclose(y[..., 1::2], b * c + a * s_, atol=1e-6)


def test_split_normalisations(golden):
    """Restatements against the reference's goldens (tools/golden/mapping.py:1291-1415, 7800-7921)."""
    x, res, w, b = (golden[f"map/split_norm/{n}"] for n in ("x", "residual", "weight", "bias"))
    assert torch.allclose(ops.dit_rms_norm_unary_fused(x, w, b, res, 1e-5, "silu"), golden["map/split_norm/dit_silu"], rtol=1e-6, atol=1e-6)
    assert torch.allclose(ops.dit_rms_norm_unary_fused(x, w, None, None, 1e-6, None), golden["map/split_norm/dit_plain"], rtol=1e-6, atol=1e-6)
    assert torch.allclose(ops.rms_norm_pre_all_gather(x, res, torch.float32), golden["map/split_norm/rms_pre"], rtol=1e-6, atol=0)
    pre = ops.layer_norm_pre_all_gather(x, None, torch.float32)
    assert torch.allclose(pre, golden["map/split_norm/ln_pre"], rtol=1e-6, atol=1e-6)
    # one device: the statistics rebuild the shard's own layer norm, which is what the golden computes
    assert torch.allclose(ops.layer_norm_post_all_gather(x, pre, w, b, 1e-5), golden["map/split_norm/ln_post_1dev"], rtol=1e-5, atol=2e-6)
    # four devices: pre -> gather -> post equals the layer norm of the whole row
    xs = list(torch.chunk(x, 4, dim=-1))
    stats = torch.cat([ops.layer_norm_pre_all_gather(t, None, torch.float32) for t in xs], dim=-1)
    whole = torch.nn.functional.layer_norm(x, [96], w, b, 1e-5)
    for i, t in enumerate(xs):
        got = ops.layer_norm_post_all_gather(t, stats, w[24 * i: 24 * i + 24], b[24 * i: 24 * i + 24], 1e-5)
        assert torch.allclose(got, whole[:, 24 * i: 24 * i + 24], rtol=1e-5, atol=2e-6)
    got = ops.distributed_rms_norm(xs, list(torch.chunk(w, 4)), list(torch.chunk(res, 4, dim=-1)), 1e-5)
    for i, g in enumerate(got):
        assert torch.allclose(g, golden[f"map/split_norm/dist_rms_1x4/{i}"], rtol=1e-6, atol=1e-6)


def test_mixture_of_experts_ops(golden):
    """Restatements against the reference's goldens (tools/golden/mapping.py:1596-1760, 2030-2150)."""
    a, b = golden["map/moe/spmm_a"], golden["map/moe/spmm_b"]
    ones = torch.ones(2, 3, 1, 4)
    assert torch.equal(ops.sparse_matmul(a, b, ones, False), golden["map/moe/spmm_b_sparse"])
    sp = (torch.arange(24).reshape(2, 3, 1, 4) % 3 != 0).float()
    got = ops.sparse_matmul(a, b, sp, False)
    keep = sp.reshape(2, 3, 1, 4, 1, 1).bool().expand_as(got)
    assert torch.equal(got[keep], golden["map/moe/spmm_b_sparse"][keep]) and int(got[~keep].abs().sum()) == 0
    assert torch.equal(ops.sparse_matmul(golden["map/moe/spmm_a2"], b, torch.ones(1, 1, 3, 4), True), golden["map/moe/spmm_a_sparse"])
    # dispatch: 4 devices, experts 2d and 2d + 1 on device d
    tok, sel = golden["map/moe/tokens"], golden["map/moe/selected"]
    mapping = torch.zeros(1, 1, 8, 4, dtype=torch.int32)
    for e in range(8):
        mapping[0, 0, e, e // 2] = 1
    xs = [tok[6 * d: 6 * d + 6].reshape(6, 1, 1, 16) for d in range(4)]
    idx = [sel[6 * d: 6 * d + 6].reshape(6, 1, 1, 2) for d in range(4)]
    disp, meta = ops.all_to_all_dispatch(xs, idx, mapping)
    for d in range(4):
        assert torch.equal(disp[d].reshape(1, 24, 16), golden[f"map/moe/dispatched_1x4/{d}"])
        assert torch.equal(meta[d].reshape(1, 24, 2), golden["map/moe/indices_gathered"])
    cin, cmeta = golden["map/moe/combine_in"], golden["map/moe/combine_meta"]
    got = ops.all_to_all_combine([cin], cmeta, torch.ones(1, 1, 4, 1, dtype=torch.int32), 2)
    assert torch.equal(got[0], golden["map/moe/combine_out"])
    # dispatch -> identity experts -> combine hands every token back once per selected expert
    expert_out = [torch.stack([disp[d].reshape(24, 1, 16)] * 2) for d in range(4)]     # [E_local = 2, 24, 1, 16]
    back = ops.all_to_all_combine(expert_out, meta[0].reshape(1, 24, 1, 2), mapping, 2)
    for d in range(4):
        assert torch.equal(back[d], torch.stack([tok[6 * d: 6 * d + 6].reshape(6, 1, 16)] * 2))
    m, red = ops.moe_expert_token_remap(torch.rand(1, 24, 1, 8), mapping, meta[0].reshape(1, 24, 1, 2), 1, 8)
    assert m.shape == (1, 24, 1, 2) and red.shape == (1, 1, 3, 2)
    assert ((m != 0).reshape(24, 2) == torch.stack([(sel == 2).any(1), (sel == 3).any(1)], dim=1)).all()


def test_dispatch_metadata_and_router(golden):
    """Restatements against the reference's goldens (tools/golden/mapping.py:1656-1760, 5960-5992)."""
    tok, sel, scr = golden["map/moe/tokens"], golden["map/moe/selected"], golden["map/moe/scores"]
    owner = (torch.arange(8) // 2).to(torch.int32).reshape(1, 1, 1, 8).repeat(1, 1, 4, 1)
    part = lambda t: [t[6 * d: 6 * d + 6].reshape(1, 1, 6, -1) for d in range(4)]
    disp, idx, sc = ops.all_to_all_dispatch_metadata(part(tok), part(sel), part(scr), owner)
    for d in range(4):
        assert torch.equal(disp[d], golden[f"map/moe/dispatched_1x4/{d}"])
        assert torch.equal(idx[d], golden["map/moe/indices_gathered"]) and torch.equal(sc[d], golden["map/moe/scores_gathered"])
    x, w, b = (golden[f"map/router/{n}"] for n in ("x", "w", "b"))
    ridx, rw = ops.topk_router_gpt(x, w, b, 4)
    assert torch.equal(ridx.to(torch.int32), golden["map/router/indices"]) and torch.equal(rw, golden["map/router/weights"])


def test_conv3d_gelu_backward_embedding_backward_adamw(golden):
    """Restatements against the reference's goldens (tools/golden/mapping.py:714-801, 4379-4383, 5875-5912, 1155-1218)."""
    x, w, b = (golden[f"map/conv3d/{n}"] for n in ("x", "w", "b"))
    got = ops.conv3d(x, w, b, 2, 4, 5, 6, (1, 2, 1), (1, 1, 1), 2)
    assert torch.allclose(got, golden["map/conv3d/s1x2x1_p1_g2"], rtol=1e-5, atol=1e-5) and got.shape == golden["map/conv3d/s1x2x1_p1_g2"].shape
    rep = ops.conv3d(x, w, b, 2, 4, 5, 6, (1, 1, 1), (1, 1, 1), 2, "replicate")
    padded = torch.nn.functional.pad(x.permute(0, 4, 1, 2, 3), (1,) * 6, mode="replicate").permute(0, 2, 3, 4, 1).contiguous()
    assert torch.allclose(rep, ops.conv3d(padded, w, b, 2, 6, 7, 8, (1, 1, 1), (0, 0, 0), 2), rtol=1e-6, atol=1e-6)
    gg, gx = golden["map/gelu_bw/grad"], golden["map/gelu_bw/x"]
    for ap in ("none", "tanh"):
        assert torch.equal(ops.gelu_backward(gg, gx, ap), golden[f"map/gelu_bw/{ap}"])
    assert torch.allclose(ops.embedding_backward(golden["map/embedding_bw/indices"], [10, 16], golden["map/embedding_bw/grad"]),
                          golden["map/embedding_bw/out"], rtol=1e-6, atol=1e-6)
    p, g, m, v, vmax = (golden[f"map/adamw/{n}"] for n in ("param", "grad", "m", "v", "vmax"))
    for tag, vm in (("plain", None), ("amsgrad", vmax)):
        res = ops.adamw(p, g, m, v, vm, 1e-2, 0.9, 0.99, 0.9 ** 3, 0.99 ** 3, 1e-8, 0.1)
        for n, t in zip(("param", "m", "v", "vmax"), res):
            assert torch.allclose(t, golden[f"map/adamw/{tag}/{n}"], rtol=1e-6, atol=1e-7), (tag, n)


def test_chunked_prefill_attention(golden):
    """Restatement against the reference's golden (tools/golden/mapping.py:8847-8912)."""
    q, k, v, pt = (golden[f"map/chunked_sdpa/{n}"] for n in ("q", "k", "v", "page_table"))
    for start in (0, 40):
        assert torch.allclose(ops.chunked_sdpa(q, k, v, pt, start, 0.2), golden[f"map/chunked_sdpa/start{start}"], rtol=1e-6, atol=1e-6)


def test_multi_latent_attention_prefill(golden):
    """Restatement against the reference's golden (tools/golden/mapping.py:8662-8692)."""
    q, k, mask, v = (golden[f"map/mla/{n}"] for n in ("q", "k", "mask", "v"))
    assert torch.allclose(ops.flash_mla_prefill(q, k, None, None, 32, True), golden["map/mla/causal"], rtol=1e-6, atol=1e-6)
    assert torch.allclose(ops.flash_mla_prefill(q, k, None, mask, 32, True, 0.2), golden["map/mla/masked"], rtol=1e-6, atol=1e-6)
    assert torch.allclose(ops.flash_mla_prefill(q, k, v, None, 16, False), golden["map/mla/own_values"], rtol=1e-6, atol=1e-6)


def test_rotary_embedding_against_the_golden_of_the_fusing_test(golden):
    """The reference's own definition of the fused op's result (test/python/golden/ttir_ops/fusing/test_rope_fusing.py:23-33,
    lifted from the file by the fixture generator): bit for bit in f32, and for bf16 operands the f32 evaluation with
    one rounding."""
    x, cos, sin = golden["rope/x"], golden["rope/cos"], golden["rope/sin"]
    assert torch.equal(ops.rotary_embedding(x, cos, sin), golden["rope/f32"])
    bf = torch.bfloat16
    assert torch.equal(ops.rotary_embedding(x.to(bf), cos.to(bf), sin.to(bf)), golden["rope/bf16_operands"])


def test_indexer_score_dsa(golden):
    """Restatement against the reference's golden (tools/golden/mapping.py:8695-8742)."""
    q, k, w = (golden[f"map/indexer/{n}"] for n in ("q", "k", "w"))
    assert torch.equal(ops.indexer_score_dsa(q, k, w, 0), golden["map/indexer/dense"])
    assert torch.equal(ops.indexer_score_dsa(q, k, w, 64), golden["map/indexer/chunked"])
    q, k, w = (golden[f"map/indexer/ragged_{n}"] for n in ("q", "k", "w"))
    assert torch.equal(ops.indexer_score_dsa(q, k, w, 30), golden["map/indexer/ragged"])
    assert torch.isneginf(golden["map/indexer/dense"][0, 0, 0, 1:]).all() and torch.isfinite(golden["map/indexer/chunked"][0, 0, 0, :65]).all()


def test_paged_multi_latent_decode_attention(golden):
    """Restatement against the reference's golden (tools/golden/mapping.py:8275-8365)."""
    q, k, pt, pos, v = (golden[f"map/mla_decode/{n}"] for n in ("q", "k", "page_table", "cur_pos", "v"))
    assert torch.allclose(ops.paged_mla_decode(q, k, None, pt, pos, None, 32), golden["map/mla_decode/latent"], rtol=1e-6, atol=1e-6)
    assert torch.allclose(ops.paged_mla_decode(q, k, v, pt, pos, None, 16, True, 0.15), golden["map/mla_decode/own_values"], rtol=1e-6, atol=1e-6)


def test_layer_norm(golden):
    x, w, b = golden["ln/x"], golden["ln/w"], golden["ln/b"]
    assert same(ops.layer_norm(x), golden["ln/plain"])
    assert same(ops.layer_norm(x, w, b), golden["ln/affine"])
    assert same(ops.layer_norm(x, golden["ln/w2"], None, 1e-3), golden["ln/two_dims"])


def test_argmax_cumsum_embedding_pad(golden):
    x = golden["arg/x"]
    for d in (0, 1, 2):
        assert torch.equal(ops.argmax(x, d), golden[f"arg/dim{d}"])
    assert torch.equal(ops.argmax(x), golden["arg/all"])
    assert torch.equal(ops.argmax(x, 1, True), golden["arg/keep"])
    for d in (0, 1, 2):
        assert same(ops.cumsum(golden["cum/x"], d), golden[f"cum/dim{d}"])
    assert torch.equal(ops.cumsum(golden["cum/xi"], 1), golden["cum/int"])
    assert torch.equal(ops.embedding(golden["emb/idx"], golden["emb/w"]), golden["emb/out"])
    assert torch.equal(ops.pad(golden["pad/x"], [1, 0, 0, 2, 3, 1], -1.5), golden["pad/out"])


def test_pooling(golden):
    from helpers import POOL_CASES
    from ttmlir_b200.ttnn_builder import ProgramBuilder
    x = golden["pool/x"].reshape(1, 1, -1, 8)
    for name, (kind, kernel, stride, padding, dilation, ceil, include) in POOL_CASES.items():
        want = golden[f"pool/{name}"]
        if kind == "max":
            got = ops.max_pool2d(x, 2, 9, 11, 8, kernel, stride, padding, dilation, ceil)
        else:
            got = ops.avg_pool2d(x, 2, 9, 11, 8, kernel, stride, padding, ceil, include)
        assert same(got, want.reshape(1, 1, -1, 8)), name
        # the shape rule the builder (and the kernel library) uses gives the reference's extents
        ho, wo = ProgramBuilder.pool_out_hw("MaxPool2d" if kind == "max" else "AvgPool2d", 9, 11, kernel, stride, padding,
                                            dilation, ceil)
        assert (ho, wo) == tuple(want.shape[1:3]), name
    assert same(ops.global_avg_pool2d(golden["pool/x"]), golden["pool/global"])


def test_pool_out_shape_in_the_library_matches_the_builder(rt):
    import ctypes
    from helpers import POOL_CASES
    from ttmlir_b200.ttnn_builder import ProgramBuilder
    for h, w in ((9, 11), (7, 7), (56, 56), (5, 4)):
        for name, (kind, kernel, stride, padding, dilation, ceil, _) in POOL_CASES.items():
            if len(padding) == 4:
                pt, pl, pb, pr = padding
            else:
                pt = pb = padding[0]
                pl = pr = padding[1]
            ho, wo = ctypes.c_int(), ctypes.c_int()
            rc = rt.lib.ttb_pool2d_out_shape(int(kind == "max"), h, w, kernel[0], kernel[1], stride[0], stride[1], pt, pl, pb, pr,
                                             dilation[0], dilation[1], int(ceil), int(len(padding) == 4),
                                             ctypes.byref(ho), ctypes.byref(wo))
            want = ProgramBuilder.pool_out_hw("MaxPool2d" if kind == "max" else "AvgPool2d", h, w, kernel, stride, padding,
                                              dilation, ceil)
            if min(want) <= 0:
                assert rc != 0
            else:
                assert rc == 0 and (ho.value, wo.value) == want, (name, h, w)


def test_metrics_special_cases():
    a = torch.tensor([1.0, 2.0, 3.0])
    assert metrics.get_pcc(a, a) == 1.0
    assert metrics.get_pcc(a, -a) < -0.99
    assert metrics.get_pcc(torch.zeros(0), torch.zeros(0)) == 1.0
    assert metrics.get_pcc(torch.zeros(4), torch.ones(4)) == 0.0
    at, rt_ = metrics.get_atol_rtol(a, a + 0.5)
    assert abs(at - 0.5) < 1e-6
