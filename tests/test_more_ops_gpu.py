"""assign, pow_scalar, the debug / serialization ops, the decode-step head ops, rotary_embedding_llama, max_pool2d with
indices, training batch norm, dropout and rand through tt::runtime::submit, against the reference's goldens where it
has some (tests/golden, recorded from tools/golden/mapping.py), the oracle, and distribution properties for the two
random ops (their streams are this runtime's own)."""

import os

import pytest
import torch

from ttmlir_b200 import graphs
from helpers import DTYPE_NAME, assert_matches, run_body, run_program

pytestmark = pytest.mark.gpu


def run_gpu(rt, device, body, inputs):
    """Runs `body(b, *values)` on the GPU only (ops whose result the oracle cannot restate: random streams, files)."""
    def graph(b):
        vals = [b.input(list(t.shape), DTYPE_NAME[t.dtype]) for t in inputs]
        out = body(b, *vals)
        b.output(*(out if isinstance(out, (tuple, list)) else (out,)))
    return run_program(rt, device, graphs.build_binary(graph), inputs)


def test_assign_and_pow_scalar(rt, device):
    torch.manual_seed(0)
    x = torch.randn(7, 33)
    got, want = run_body(rt, device, lambda b, v: (b.assign(v), b.assign(v, "BFloat16")), [x])
    assert torch.equal(got[0], x) and torch.equal(got[1], x.to(torch.bfloat16)) and torch.equal(want[1], got[1])
    xp = torch.rand(5, 100) * 3 + 0.1
    got, want = run_body(rt, device, lambda b, v: (b.pow_scalar(v, 2.5), b.pow_scalar(v, 3), b.pow_scalar(v, -0.5)), [xp])
    for g, w in zip(got, want):
        assert torch.allclose(g, w, rtol=2e-6, atol=1e-7)
    xb = xp.to(torch.bfloat16)
    got, want = run_body(rt, device, lambda b, v: b.pow_scalar(v, 2.0), [xb])
    assert_matches(got[0], want[0], "pow_scalar bf16", (0.9999, 1e-2, 2.0 ** -7))


def test_debug_markers_pass_their_operand_on(rt, device, tmp_path, capfd):
    torch.manual_seed(1)
    x = torch.randn(4, 64)
    snap = str(tmp_path / "memory.txt")

    def body(b, v):
        a = b.annotate(v, "layer 3 input")
        r = b.region_start(a, "block0")
        y = b.binary("Add", r, r)
        e = b.region_end(y, "block0")
        b.print_message(e, "reached the end of block0")
        b.breakpoint(e)
        b.memory_snapshot(e, snap)
        return e
    got, want = run_body(rt, device, body, [x])
    assert torch.equal(got[0], x + x) and torch.equal(want[0], got[0])
    err = capfd.readouterr().err
    assert "reached the end of block0" in err and "breakpoint" in err
    text = open(snap).read()
    assert "Device 0 DRAM memory state" in text and "allocatedBytes=" in text


def test_dump_tensor_then_load_tensor(rt, device, tmp_path):
    torch.manual_seed(2)
    x = torch.randn(3, 5, 32).to(torch.bfloat16)
    path = str(tmp_path / "t.tensorbin")

    def dump(b, v):
        y = b.unary("Neg", v)
        b.dump_tensor(y, path)
        return y
    got = run_gpu(rt, device, dump, [x])
    assert torch.equal(got[0], -x) and os.path.getsize(path) > x.numel() * 2
    back = run_gpu(rt, device, lambda b: b.unary("Abs", b.load_tensor(path, [3, 5, 32], "BFloat16")), [])
    assert torch.equal(back[0], x.abs())
    with pytest.raises(RuntimeError, match="does not have the op's result type"):
        run_gpu(rt, device, lambda b: b.load_tensor(path, [3, 5, 32], "Float32"), [])
    bad = str(tmp_path / "bad.bin")
    open(bad, "wb").write(b"not a tensor file at all")
    with pytest.raises(RuntimeError, match="not a tensor file"):
        run_gpu(rt, device, lambda b: b.load_tensor(bad, [1], "Float32"), [])


def test_nlp_create_qkv_heads_decode_and_concat_heads_decode(rt, device):
    torch.manual_seed(3)
    x = torch.randn(1, 1, 32, (8 + 2 * 2) * 64).to(torch.bfloat16)
    got, want = run_body(rt, device, lambda b, v: b.nlp_create_qkv_heads_decode(v, 8, 2), [x])
    assert [tuple(g.shape) for g in got] == [(1, 32, 8, 64), (1, 32, 2, 64), (1, 32, 2, 64)]
    for g, w in zip(got, want):
        assert torch.equal(g, w)
    off = torch.tensor([8], dtype=torch.int32)
    got, want = run_body(rt, device, lambda b, v, o: b.nlp_create_qkv_heads_decode(v, 8, 2, batch_offset=o, slice_size=16), [x, off])
    assert tuple(got[0].shape) == (1, 16, 8, 64)
    for g, w in zip(got, want):
        assert torch.equal(g, w)
    h = torch.randn(1, 32, 32, 64).to(torch.bfloat16)          # heads padded to 32, 12 real
    got, want = run_body(rt, device, lambda b, v: b.nlp_concat_heads_decode(v, 12), [h])
    assert tuple(got[0].shape) == (1, 1, 32, 12 * 64) and torch.equal(got[0], want[0])
    # the decode step's attention front end: split, rotate, merge back
    got, want = run_body(rt, device, lambda b, v: b.nlp_concat_heads_decode(b.nlp_create_qkv_heads_decode(v, 8, 2)[0], 8), [x])
    assert torch.equal(got[0], x[..., : 8 * 64])


def pair_swap_matrix(dtype):
    t = torch.zeros(32, 32)
    for i in range(0, 32, 2):
        t[i, i + 1] = 1.0
        t[i + 1, i] = -1.0
    return t.reshape(1, 1, 32, 32).to(dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_rotary_embedding_llama_prefill_and_decode(rt, device, dtype):
    torch.manual_seed(4)
    tol = (0.9999, 1e-2, 2.0 ** -7) if dtype == torch.bfloat16 else (0.999999, 1e-5, 1e-5)
    t = pair_swap_matrix(dtype)
    for heads, seq, d in ((8, 128, 128), (3, 33, 64), (1, 32, 256)):
        x = torch.randn(1, heads, seq, d).to(dtype)
        ang = torch.rand(1, 1, seq, d // 2).repeat_interleave(2, dim=-1) * 6.28
        c, s = torch.cos(ang).to(dtype), torch.sin(ang).to(dtype)
        got, want = run_body(rt, device, lambda b, *v: b.rotary_embedding_llama(*v), [x, c, s, t])
        assert_matches(got[0], want[0], f"llama rotary prefill {heads}x{seq}x{d}", tol)
        a, bb = x.float()[..., 0::2], x.float()[..., 1::2]
        ref = torch.stack((a * c.float()[..., 0::2] - bb * s.float()[..., 0::2], bb * c.float()[..., 0::2] + a * s.float()[..., 0::2]),
                          dim=-1).reshape(x.shape)
        assert_matches(got[0], ref.to(dtype), "llama rotary against the pair rotation written out", tol)
    xd = torch.randn(1, 32, 8, 128).to(dtype)                   # decode: [1, batch, heads, D], one position per batch entry
    ang = torch.rand(1, 32, 1, 64).repeat_interleave(2, dim=-1) * 6.28
    c, s = torch.cos(ang).to(dtype), torch.sin(ang).to(dtype)
    got, want = run_body(rt, device, lambda b, *v: b.rotary_embedding_llama(*v, is_decode_mode=True), [xd, c, s, t])
    assert_matches(got[0], want[0], "llama rotary decode", tol)
    # a general (dense) transformation matrix
    dense = (torch.randn(1, 1, 32, 32) * 0.2).to(dtype)
    xg = torch.randn(1, 4, 32, 128).to(dtype)
    cg, sg = torch.randn(1, 1, 32, 128).to(dtype), torch.randn(1, 1, 32, 128).to(dtype)
    got, want = run_body(rt, device, lambda b, *v: b.rotary_embedding_llama(*v), [xg, cg, sg, dense])
    assert_matches(got[0], want[0], "llama rotary with a dense matrix", tol)


def test_max_pool2d_with_indices_matches_the_reference_goldens(rt, device, golden):
    x = golden["map/max_pool_indices/x"]
    flat = x.reshape(1, 1, -1, 6)
    cases = {"k3_s2_p1": dict(kernel=(3, 3), stride=(2, 2), padding=(1, 1)),
             "k2x3_s1x2_d2_ceil": dict(kernel=(2, 3), stride=(1, 2), padding=(0, 1), dilation=(2, 1), ceil_mode=True)}
    for name, kw in cases.items():
        got, want = run_body(rt, device, lambda b, v: b.max_pool2d_with_indices(v, 2, 9, 11, 6, **kw), [flat])
        ref_v, ref_i = golden[f"map/max_pool_indices/{name}"], golden[f"map/max_pool_indices/{name}_idx"]
        assert torch.equal(got[0].reshape(ref_v.shape), ref_v) and torch.equal(got[1].reshape(ref_i.shape), ref_i), name
        assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
    xb = torch.randn(1, 1, 4 * 28 * 28, 64, generator=torch.Generator().manual_seed(5)).to(torch.bfloat16)
    for idt in ("Int32", "UInt16"):
        got, want = run_body(rt, device, lambda b, v: b.max_pool2d_with_indices(v, 4, 28, 28, 64, kernel=(3, 3), stride=(2, 2), padding=(1, 1),
                                                                                index_dtype=idt), [xb])
        assert torch.equal(got[0], want[0]) and torch.equal(got[1].to(torch.int64), want[1].to(torch.int64))


def test_batch_norm_training_matches_the_reference_golden(rt, device, golden):
    x, mean, var, w, b_ = (golden[f"map/batch_norm/{n}"] for n in ("x", "mean", "var", "weight", "bias"))

    def body(b, xv, m, v, wv, bv):
        y = b.batch_norm_training(xv, m, v, wv, bv, 1e-5, 0.1)
        return y, b.assign(m), b.assign(v)                      # the running statistics after the in-place update
    got, want = run_body(rt, device, body, [x, mean, var, w, b_])
    for g, name in zip(got, ("out", "new_mean", "new_var")):
        assert torch.allclose(g, golden[f"map/batch_norm_training/{name}"], rtol=1e-5, atol=2e-6), name
    for g, w_ in zip(got, want):
        assert torch.allclose(g, w_, rtol=1e-5, atol=2e-6)
    bf = torch.bfloat16
    big = torch.randn(8, 32, 14, 14, generator=torch.Generator().manual_seed(6))
    ins = [big.to(bf), torch.zeros(32).to(bf), torch.ones(32).to(bf), (torch.rand(32) + 0.5).to(bf), torch.randn(32).to(bf)]
    got, want = run_body(rt, device, body, ins)
    assert_matches(got[0], want[0], "batch norm training bf16", (0.999, 2e-2, 2.0 ** -6))
    assert_matches(got[1], want[1], "running mean bf16", (0.99, 2e-2, 2.0 ** -7))
    assert_matches(got[2], want[2], "running var bf16", (0.99, 2e-2, 2.0 ** -7))


def test_dropout_drops_the_asked_fraction_and_scales_the_rest(rt, device):
    x = torch.rand(512, 1024) + 0.5
    got = run_gpu(rt, device, lambda b, v: (b.dropout(v, 0.25, seed=7), b.dropout(v, 0.25, seed=7), b.dropout(v, 0.25, seed=8),
                                            b.dropout(v, 0.0, seed=7), b.dropout(v, 1.0, scale=1.0, seed=7)), [x])
    a, a2, other, none, everything = got
    kept = a != 0
    assert abs((~kept).float().mean().item() - 0.25) < 0.004          # 524288 draws: sigma = 6e-4
    assert torch.allclose(a[kept], (x / 0.75)[kept], rtol=1e-6)
    assert torch.equal(a, a2) and not torch.equal(a, other)           # a function of the seed
    assert torch.equal(none, x) and int((everything != 0).sum()) == 0
    # no structure along rows or columns
    assert (kept.float().mean(dim=0) - 0.75).abs().max() < 0.1 and (kept.float().mean(dim=1) - 0.75).abs().max() < 0.07
    xb = x.to(torch.bfloat16)
    got = run_gpu(rt, device, lambda b, v: b.dropout(v, 0.5, seed=3), [xb])
    assert abs((got[0] == 0).float().mean().item() - 0.5) < 0.004
    assert torch.equal(got[0][got[0] != 0], (xb.float() * 2).to(torch.bfloat16)[got[0] != 0])


def test_rand_is_uniform_in_its_interval(rt, device):
    got = run_gpu(rt, device, lambda b: (b.rand([256, 1024], "Float32", -2.0, 3.0, seed=11), b.rand([256, 1024], "Float32", -2.0, 3.0, seed=11),
                                        b.rand([256, 1024], "Float32", -2.0, 3.0, seed=12), b.rand([64, 512], "BFloat16", 0.0, 1.0, seed=1)), [])
    a, a2, other, bf = got
    assert a.min() >= -2.0 and a.max() < 3.0 and torch.equal(a, a2) and not torch.equal(a, other)
    assert abs(a.mean().item() - 0.5) < 0.02 and abs(a.var().item() - 25.0 / 12.0) < 0.03
    hist = torch.histc(a, bins=20, min=-2.0, max=3.0) / a.numel()
    assert (hist - 0.05).abs().max() < 0.003
    assert bf.dtype == torch.bfloat16 and bf.min() >= 0 and bf.max() < 1 and abs(bf.float().mean().item() - 0.5) < 0.02
    assert len(torch.unique(bf)) > 200                                  # k / 256 for 256 values of k


def test_prepared_conv_transpose_weights_run_like_the_raw_ones(rt, device, golden):
    x, w, b_ = (golden[f"map/conv_transpose/{n}"] for n in ("x", "w", "b"))

    def body(b, xv, wv, bv):
        pw = b.prepare_conv_transpose2d_weights(wv, 2, 5, 6, stride=(2, 2), padding=(1, 1), output_padding=(1, 1))
        pb = b.prepare_conv_transpose2d_bias(bv, 8, 2, 5, 6, kernel=(3, 3), stride=(2, 2), padding=(1, 1))
        return b.conv_transpose2d(xv, pw, pb, 2, 5, 6, stride=(2, 2), padding=(1, 1), output_padding=(1, 1))
    got, want = run_body(rt, device, body, [x, w, b_])
    assert torch.allclose(got[0], golden["map/conv_transpose/s2_p1_op1"], rtol=1e-5, atol=1e-5) and torch.allclose(got[0], want[0], rtol=1e-5, atol=1e-5)


def test_split_normalisations_match_the_reference_goldens(rt, device, golden):
    x, res, w, b_ = (golden[f"map/split_norm/{n}"] for n in ("x", "residual", "weight", "bias"))
    got, want = run_body(rt, device, lambda b, xv, rv, wv, bv: (
        b.dit_rms_norm_unary_fused(xv, wv, bv, rv, 1e-5, "silu"), b.dit_rms_norm_unary_fused(xv, wv, epsilon=1e-6),
        b.rms_norm_pre_all_gather(xv, rv), b.layer_norm_pre_all_gather(xv),
        b.layer_norm_post_all_gather(xv, b.layer_norm_pre_all_gather(xv), wv, bv, 1e-5),
        b.distributed_rms_norm(xv, wv, rv)), [x, res, w, b_])
    names = ("dit_silu", "dit_plain", "rms_pre", "ln_pre", "ln_post_1dev")
    for g, w_, name in zip(got, want, names):
        assert torch.allclose(g, golden[f"map/split_norm/{name}"], rtol=1e-5, atol=2e-6), name
        assert torch.allclose(g, w_, rtol=1e-5, atol=2e-6), name
    # one device: the distributed form is the plain rms norm of x + residual
    xr = x + res
    assert torch.allclose(got[5], xr * torch.rsqrt(xr.square().mean(-1, keepdim=True) + 1e-5) * w, rtol=1e-5, atol=2e-6)
    assert got[2].shape == (6, 32) and int((got[2][:, 1:] != 0).sum()) == 0 and got[3].shape == (6, 64)
    bf = torch.bfloat16
    torch.manual_seed(9)
    xb, rb, wb = torch.randn(64, 4096).to(bf), torch.randn(64, 4096).to(bf), (torch.rand(4096) + 0.5).to(bf)
    for act in (None, "gelu", "relu6", "softplus", "tanh_approx"):
        got, want = run_body(rt, device, lambda b, xv, rv, wv: b.dit_rms_norm_unary_fused(xv, wv, None, rv, 1e-5, act), [xb, rb, wb])
        assert_matches(got[0], want[0], f"dit rms norm bf16 {act}", (0.9999, 1e-2, 2.0 ** -7))
    got, want = run_body(rt, device, lambda b, xv: b.layer_norm_pre_all_gather(xv, dtype="Float32"), [xb])
    assert torch.allclose(got[0], want[0], rtol=1e-5, atol=1e-3)


def test_global_semaphore_ops_are_accepted(rt, device):
    x = torch.randn(3, 32)

    def body(b, v):
        b.create_global_semaphore(0)
        y = b.unary("Neg", v)
        b.reset_global_semaphore(0)
        return y
    got, _ = run_body(rt, device, body, [x])
    assert torch.equal(got[0], -x)


def test_sparse_matmul_matches_the_reference_goldens(rt, device, golden):
    a, b_ = golden["map/moe/spmm_a"], golden["map/moe/spmm_b"]
    bf = torch.bfloat16
    got, want = run_body(rt, device, lambda b, av, bv, sv: b.sparse_matmul(av, bv, sv), [a, b_, torch.ones(2, 3, 1, 4).to(bf)])
    assert got[0].shape == golden["map/moe/spmm_b_sparse"].shape
    assert_matches(got[0], golden["map/moe/spmm_b_sparse"], "sparse_matmul, b sparse, all blocks", (0.9999, 1e-2, 2.0 ** -7))
    sp = (torch.arange(24).reshape(2, 3, 1, 4) % 3 != 0).to(bf)
    got, want = run_body(rt, device, lambda b, av, bv, sv: b.sparse_matmul(av, bv, sv, nnz=16), [a, b_, sp])
    assert_matches(got[0], want[0], "sparse_matmul with skipped blocks", (0.9999, 1e-2, 2.0 ** -7))
    keep = sp.reshape(2, 3, 1, 4, 1, 1).bool().expand_as(got[0])
    assert int(got[0][~keep].float().abs().sum()) == 0
    a2 = golden["map/moe/spmm_a2"]
    got, want = run_body(rt, device, lambda b, av, bv, sv: b.sparse_matmul(av, bv, sv, is_input_a_sparse=True, is_input_b_sparse=False),
                         [a2, b_, torch.ones(1, 1, 3, 4).to(bf)])
    assert_matches(got[0], golden["map/moe/spmm_a_sparse"], "sparse_matmul, a sparse", (0.9999, 1e-2, 2.0 ** -7))
    # an expert layer's shapes: 2 blocks of 32 tokens, 8 experts, 512 -> 1024, ragged n and k
    torch.manual_seed(12)
    xa, wb = torch.randn(2, 1, 32, 520).to(bf), (torch.randn(1, 8, 520, 1000) * 0.05).to(bf)
    mask = (torch.rand(2, 1, 1, 8) < 0.4).to(bf)
    got, want = run_body(rt, device, lambda b, av, bv, sv: b.sparse_matmul(av, bv, sv), [xa, wb, mask])
    assert_matches(got[0], want[0], "sparse_matmul at expert shapes", (0.9999, 2e-2, 2.0 ** -6))
    xh, wh = xa.to(torch.float16), wb.to(torch.float16)
    got, want = run_body(rt, device, lambda b, av, bv, sv: b.sparse_matmul(av, bv, sv), [xh, wh, mask.to(torch.float16)])
    assert_matches(got[0], want[0], "sparse_matmul f16", (0.9999, 1e-2, 2.0 ** -9))


def test_moe_routing_ops_on_one_device(rt, device, golden):
    cin, cmeta = golden["map/moe/combine_in"], golden["map/moe/combine_meta"]
    ones = torch.ones(1, 1, 4, 1, dtype=torch.int32)
    got, want = run_body(rt, device, lambda b, xv, mv, pv: b.all_to_all_combine(xv, mv, pv, 2), [cin, cmeta, ones])
    assert torch.equal(got[0], golden["map/moe/combine_out"]) and torch.equal(want[0], got[0])
    torch.manual_seed(13)
    x = torch.randn(6, 1, 5, 64).to(torch.bfloat16)
    sel = torch.stack([torch.randperm(4)[:2] for _ in range(30)]).to(torch.int32).reshape(6, 1, 5, 2)
    half = torch.tensor([[1, 0], [0, 1], [1, 0], [0, 1]], dtype=torch.int32).reshape(1, 1, 4, 2)   # this device owns experts 0 and 2
    got, want = run_body(rt, device, lambda b, xv, iv, pv: b.all_to_all_dispatch(xv, iv, pv), [x, sel, half])
    assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1]) and got[0].shape == (1, 6, 5, 64)
    routed = ((sel == 0) | (sel == 2)).any(-1).reshape(1, 6, 5, 1)
    assert torch.equal(got[0], torch.where(routed, x.reshape(1, 6, 5, 64), torch.zeros(1, 6, 5, 64).to(torch.bfloat16)))
    topk = torch.rand(1, 6, 5, 4).to(torch.bfloat16)
    for rdt in (None, "UInt16"):
        got, want = run_body(rt, device, lambda b, tv, pv, mv: b.moe_expert_token_remap(tv, pv, mv, 8, reduced_dtype=rdt),
                             [topk, half, sel.reshape(1, 6, 5, 2)])
        assert torch.equal(got[0], want[0]) and torch.equal(got[1].float(), want[1].float())
        assert got[0].shape == (1, 6, 5, 2) and got[1].shape == (1, 1, 4, 2)


def test_topk_router_gpt_matches_the_reference_golden(rt, device, golden):
    # The contraction's summation order differs from torch's, so a logit can land on the other side of a bf16 rounding
    # boundary and two near-equal experts swap places: the selections must agree on almost every token, and the
    # weights wherever they do.
    def check(got, idx, wts, what, tol):
        same = (got[0].to(torch.int32) == idx.to(torch.int32)).all(dim=-1)
        assert same.float().mean() >= 0.9, f"{what}: only {int(same.sum())} of {same.numel()} selections agree"
        assert_matches(got[1][same], wts[same], what, tol)
        assert got[0].dtype == torch.uint16 and torch.allclose(got[1].float().sum(-1), torch.ones(got[1].shape[0]), atol=2e-2)
    x, w, b_ = (golden[f"map/router/{n}"] for n in ("x", "w", "b"))
    got, want = run_body(rt, device, lambda b, xv, wv, bv: b.topk_router_gpt(xv, wv, bv, 4), [x, w, b_])
    check(got, golden["map/router/indices"], golden["map/router/weights"], "router against the reference golden", (0.999, 1e-2, 2.0 ** -7))
    check(got, want[0], want[1], "router against the oracle", (0.999, 1e-2, 2.0 ** -7))
    torch.manual_seed(14)
    xb = torch.randn(32, 2880).to(torch.bfloat16)                   # the GPT-OSS router's own shape: 128 experts, top 4
    wb, bb = (torch.randn(2880, 128) * 0.02).to(torch.bfloat16), torch.randn(32, 128).to(torch.bfloat16)
    got, want = run_body(rt, device, lambda b, xv, wv, bv: b.topk_router_gpt(xv, wv, bv, 4), [xb, wb, bb])
    check(got, want[0], want[1], "router at scale", (0.999, 2e-2, 2.0 ** -6))


def test_all_to_all_dispatch_metadata_on_one_device(rt, device):
    torch.manual_seed(15)
    x = torch.randn(1, 1, 24, 64).to(torch.bfloat16)
    sel = torch.stack([torch.randperm(8)[:2] for _ in range(24)]).to(torch.int32).reshape(1, 1, 24, 2)
    scr = torch.rand(1, 1, 24, 2).to(torch.bfloat16)
    owner = (torch.arange(8) % 2).to(torch.int32).reshape(1, 1, 1, 8)      # even experts here, odd ones on a device that is not in this mesh
    got, want = run_body(rt, device, lambda b, xv, iv, sv, ov: b.all_to_all_dispatch_metadata(xv, iv, sv, ov), [x, sel, scr, owner])
    for g, w_ in zip(got, want):
        assert torch.equal(g, w_)
    routed = (sel % 2 == 0).any(-1).reshape(1, 24, 1)
    assert torch.equal(got[0], torch.where(routed, x.reshape(1, 24, 64), torch.zeros(1, 24, 64).to(torch.bfloat16)))


def test_conv3d_matches_the_reference_golden(rt, device, golden):
    x, w, b_ = (golden[f"map/conv3d/{n}"] for n in ("x", "w", "b"))
    kw = dict(stride=(1, 2, 1), padding=(1, 1, 1), groups=2)
    got, want = run_body(rt, device, lambda b, xv, wv, bv: b.conv3d(xv, wv, bv, 2, 4, 5, 6, **kw), [x, w, b_])
    ref = golden["map/conv3d/s1x2x1_p1_g2"]
    assert got[0].shape == ref.shape and torch.allclose(got[0], ref, rtol=1e-5, atol=1e-5) and torch.allclose(got[0], want[0], rtol=1e-5, atol=1e-5)
    # flattened activations, prepared weights (carried through unchanged), replicate padding, bf16
    bf = torch.bfloat16
    xf = x.reshape(1, 1, -1, 8).to(bf)
    got, want = run_body(rt, device, lambda b, xv, wv, bv: b.conv3d(xv, b.prepare_conv3d_weights(wv, groups=2), bv, 2, 4, 5, 6,
                                                                   padding=(1, 1, 1), groups=2, padding_mode="replicate"),
                         [xf, w.to(bf), b_.to(bf)])
    assert list(got[0].shape) == [1, 1, 2 * 5 * 5 * 6, 6]
    assert_matches(got[0], want[0], "conv3d bf16 replicate", (0.9999, 2e-2, 2.0 ** -6))
    # TTNN's prepared weight matrix [kD*kH*kW*C, O] handed to conv3d directly (groups 1)
    w1 = (torch.randn(6, 8, 2, 3, 3, generator=torch.Generator().manual_seed(3)) * 0.2)
    prepared = w1.permute(2, 3, 4, 1, 0).reshape(2 * 3 * 3 * 8, 6).contiguous()

    def body(b, xv, wv):
        wv.filter_shape = [6, 8, 2, 3, 3]
        return b.conv3d(xv, wv, None, 2, 4, 5, 6, padding=(0, 1, 1))
    got = run_gpu(rt, device, body, [x, prepared])
    import oracle.ops as O
    assert torch.allclose(got[0], O.conv3d(x, w1, None, 2, 4, 5, 6, (1, 1, 1), (0, 1, 1), 1), rtol=1e-5, atol=1e-5)


def test_gelu_backward_and_embedding_backward(rt, device, golden):
    gg, gx = golden["map/gelu_bw/grad"], golden["map/gelu_bw/x"]
    got, want = run_body(rt, device, lambda b, g, x: (b.gelu_backward(g, x), b.gelu_backward(g, x, "tanh")), [gg, gx])
    for g, name in zip(got, ("none", "tanh")):
        assert torch.allclose(g, golden[f"map/gelu_bw/{name}"], rtol=2e-5, atol=2e-6), name
    got, want = run_body(rt, device, lambda b, g, x: b.gelu_backward(g, x), [gg.to(torch.bfloat16), gx.to(torch.bfloat16)])
    assert_matches(got[0], want[0], "gelu_bw bf16", (0.9999, 1e-2, 2.0 ** -7))
    ei, eg = golden["map/embedding_bw/indices"], golden["map/embedding_bw/grad"]
    table = torch.zeros(10, 16)
    got, want = run_body(rt, device, lambda b, i, w, g: b.embedding_backward(i, w, g), [ei, table, eg])
    assert torch.allclose(got[0], golden["map/embedding_bw/out"], rtol=1e-5, atol=1e-6) and torch.allclose(got[0], want[0], rtol=1e-5, atol=1e-6)
    torch.manual_seed(16)
    big_i = torch.randint(0, 1000, (4, 512), dtype=torch.int32)
    big_g = torch.randn(4, 512, 128).to(torch.bfloat16)
    got, want = run_body(rt, device, lambda b, i, w, g: b.embedding_backward(i, w, g), [big_i, torch.zeros(1000, 128).to(torch.bfloat16), big_g])
    assert_matches(got[0], want[0], "embedding_bw bf16", (0.9999, 2e-2, 2.0 ** -6))


def test_adamw_matches_the_reference_golden(rt, device, golden):
    p, g, m, v, vmax = (golden[f"map/adamw/{n}"] for n in ("param", "grad", "m", "v", "vmax"))
    hp = dict(lr=1e-2, beta1=0.9, beta2=0.99, beta1_pow=0.9 ** 3, beta2_pow=0.99 ** 3, epsilon=1e-8, weight_decay=0.1)

    def plain(b, pv, gv, mv, vv):
        b.adamw(pv, gv, mv, vv, **hp)
        return b.assign(pv), b.assign(mv), b.assign(vv)

    def ams(b, pv, gv, mv, vv, xv):
        b.adamw(pv, gv, mv, vv, xv, **hp)
        return b.assign(pv), b.assign(mv), b.assign(vv), b.assign(xv)
    got, want = run_body(rt, device, plain, [p, g, m, v])
    for t, w_, n in zip(got, want, ("param", "m", "v")):
        assert torch.allclose(t, golden[f"map/adamw/plain/{n}"], rtol=1e-5, atol=1e-7) and torch.allclose(t, w_, rtol=1e-5, atol=1e-7), n
    got, want = run_body(rt, device, ams, [p, g, m, v, vmax])
    for t, n in zip(got, ("param", "m", "v", "vmax")):
        assert torch.allclose(t, golden[f"map/adamw/amsgrad/{n}"], rtol=1e-5, atol=1e-7), n
    # bf16 parameters: round to nearest, then stochastic rounding (unbiased: the mean of many draws approaches the f32 value)
    bf = torch.bfloat16
    pb = torch.full((64, 1024), 1.0).to(bf)
    gb = torch.full((64, 1024), 0.37).to(bf)
    zeros = torch.zeros(64, 1024)

    def step(b, pv, gv, mv, vv, stochastic):
        b.adamw(pv, gv, mv, vv, lr=1e-3, beta1=0.9, beta2=0.999, beta1_pow=0.9, beta2_pow=0.999, stochastic_rounding=stochastic)
        return b.assign(pv)
    near = run_gpu(rt, device, lambda b, *v: step(b, *v, False), [pb, gb, zeros, zeros.clone()])[0]
    assert torch.equal(near, torch.full((64, 1024), 0.999).to(bf))       # 1 - 1e-3 rounds to the nearest bf16 (0.99609375 or 1.0)
    rnd = run_gpu(rt, device, lambda b, *v: step(b, *v, True), [pb, gb, zeros, zeros.clone()])[0].float()
    assert set(rnd.unique().tolist()) <= {0.99609375, 1.0} and abs(rnd.mean().item() - 0.999) < 2e-4


def test_chunked_prefill_attention(rt, device, golden):
    q, k, v, pt = (golden[f"map/chunked_sdpa/{n}"] for n in ("q", "k", "v", "page_table"))
    for start in (0, 40):                                        # head_dim 32, f32: the general kernel with a built mask
        st = torch.tensor([start], dtype=torch.int32)
        got, want = run_body(rt, device, lambda b, *t: b.chunked_scaled_dot_product_attention(*t, scale=0.2), [q, k, v, pt, st])
        assert torch.allclose(got[0], golden[f"map/chunked_sdpa/start{start}"], rtol=1e-4, atol=1e-5), start
        assert torch.allclose(got[0], want[0], rtol=1e-4, atol=1e-5)
    # the tensor-core kernel: head_dim 128, bf16, grouped heads, chunks of a 2048-token prefill over 64-token pages
    torch.manual_seed(18)
    bf = torch.bfloat16
    B, Hq, Hkv, D, bs, per_user = 2, 8, 2, 128, 64, 32
    kc, vc = torch.randn(80, Hkv, bs, D).to(bf), torch.randn(80, Hkv, bs, D).to(bf)
    table = torch.stack([torch.randperm(80)[:per_user] for _ in range(B)]).to(torch.int32)
    for start, sq in ((0, 256), (512, 384), (1792, 256), (1000, 200)):
        qc = torch.randn(B, Hq, sq, D).to(bf)
        st = torch.tensor([start], dtype=torch.int32)
        got, want = run_body(rt, device, lambda b, *t: b.chunked_scaled_dot_product_attention(*t), [qc, kc, vc, table, st])
        assert_matches(got[0], want[0], f"chunked attention, chunk [{start}, {start + sq})")
    # enough heads for the two-heads-per-CTA kernel
    qc = torch.randn(B, 32, 1024, D).to(bf)
    kc8, vc8 = torch.randn(80, 8, bs, D).to(bf), torch.randn(80, 8, bs, D).to(bf)
    got, want = run_body(rt, device, lambda b, *t: b.chunked_scaled_dot_product_attention(*t),
                         [qc, kc8, vc8, table, torch.tensor([960], dtype=torch.int32)])
    assert_matches(got[0], want[0], "chunked attention, 32 heads")


def test_flash_mla_prefill_matches_the_reference_goldens(rt, device, golden):
    q, k, mask, v = (golden[f"map/mla/{n}"] for n in ("q", "k", "mask", "v"))
    got, want = run_body(rt, device, lambda b, qv, kv: b.flash_mla_prefill(qv, kv, 32), [q, k])
    assert got[0].shape == (2, 4, 24, 32) and torch.allclose(got[0], golden["map/mla/causal"], rtol=1e-4, atol=1e-5)
    assert torch.allclose(got[0], want[0], rtol=1e-4, atol=1e-5)
    got, _ = run_body(rt, device, lambda b, qv, kv, mv: b.flash_mla_prefill(qv, kv, 32, mask=mv, scale=0.2), [q, k, mask])
    assert torch.allclose(got[0], golden["map/mla/masked"], rtol=1e-4, atol=1e-5)
    got, _ = run_body(rt, device, lambda b, qv, kv, vv: b.flash_mla_prefill(qv, kv, 16, v=vv, is_causal=False), [q, k, v])
    assert torch.allclose(got[0], golden["map/mla/own_values"], rtol=1e-4, atol=1e-5)
    # the latent widths of a DeepSeek-style layer: 576-wide keys (512 latent + 64 rotary), 512-wide values, one kv head
    torch.manual_seed(19)
    bf = torch.bfloat16
    qb, kb = (torch.randn(1, 8, 160, 576) * 0.3).to(bf), (torch.randn(1, 1, 160, 576) * 0.3).to(bf)
    got, want = run_body(rt, device, lambda b, qv, kv: b.flash_mla_prefill(qv, kv, 512), [qb, kb])
    assert got[0].shape == (1, 8, 160, 512)
    assert_matches(got[0], want[0], "flash_mla_prefill bf16, 576 / 512")


def _same_scores(got, want, what):
    """Masked keys agree exactly; the sums agree to one bf16 / f16 step (f32 sums taken in another order, one rounding)."""
    assert got.shape == want.shape and got.dtype == want.dtype, what
    assert torch.equal(torch.isneginf(got), torch.isneginf(want)), what
    seen = torch.isfinite(want)
    assert torch.isfinite(got[seen]).all(), what
    assert torch.allclose(got[seen].float(), want[seen].float(), rtol=2.0 ** -7, atol=1e-3), what


def test_indexer_score_dsa_matches_the_reference_goldens(rt, device, golden):
    q, k, w = (golden[f"map/indexer/{n}"] for n in ("q", "k", "w"))
    for start, name in ((0, "dense"), (64, "chunked")):
        got, want = run_body(rt, device, lambda b, qv, kv, wv: b.indexer_score_dsa(qv, kv, wv, start), [q, k, w])
        _same_scores(got[0], golden[f"map/indexer/{name}"], name)
        assert torch.equal(want[0], golden[f"map/indexer/{name}"])
    q, k, w = (golden[f"map/indexer/ragged_{n}"] for n in ("q", "k", "w"))
    got, _ = run_body(rt, device, lambda b, qv, kv, wv: b.indexer_score_dsa(qv, kv, wv, 30), [q, k, w])
    _same_scores(got[0], golden["map/indexer/ragged"], "5 heads, 19 queries, 75 keys of 40")
    # the indexer of a DeepSeek-style layer: 64 heads of 128, the last 200 positions of a 1000-token history, f16 too
    torch.manual_seed(21)
    for dt in (torch.bfloat16, torch.float16):
        qb, kb = (torch.randn(1, 64, 200, 128) * 0.2).to(dt), (torch.randn(1, 1, 1000, 128) * 0.2).to(dt)
        wb = torch.randn(1, 64, 200, 1).to(dt)
        got, want = run_body(rt, device, lambda b, qv, kv, wv: b.indexer_score_dsa(qv, kv, wv, 800), [qb, kb, wb])
        _same_scores(got[0], want[0], f"64 heads, {dt}")


def test_paged_multi_latent_decode_attention_matches_the_reference_goldens(rt, device, golden):
    q, k, pt, pos, v = (golden[f"map/mla_decode/{n}"] for n in ("q", "k", "page_table", "cur_pos", "v"))
    got, want = run_body(rt, device, lambda b, qv, kv, tv, pv: b.paged_flash_multi_latent_attention_decode(qv, kv, 32, tv, cur_pos=pv),
                         [q, k, pt, pos])
    assert got[0].shape == (1, 3, 4, 32) and torch.allclose(got[0], golden["map/mla_decode/latent"], rtol=1e-4, atol=1e-5)
    assert torch.allclose(got[0], want[0], rtol=1e-4, atol=1e-5)
    got, _ = run_body(rt, device, lambda b, qv, kv, tv, pv, vv: b.paged_flash_multi_latent_attention_decode(qv, kv, 16, tv, v_cache=vv,
                                                                                                          cur_pos=pv, scale=0.15),
                      [q, k, pt, pos, v])
    assert torch.allclose(got[0], golden["map/mla_decode/own_values"], rtol=1e-4, atol=1e-5)
    # latent widths of a DeepSeek-style layer, bf16: 32 users x 16 heads on one 576-wide latent head, 512-wide values
    torch.manual_seed(20)
    bf = torch.bfloat16
    qb = (torch.randn(1, 32, 16, 576) * 0.1).to(bf)
    kb = (torch.randn(160, 1, 32, 576) * 0.1).to(bf)
    table = torch.stack([torch.randperm(160)[:4] for _ in range(32)]).to(torch.int32)
    cur = torch.randint(0, 128, (32,), dtype=torch.int32)
    got, want = run_body(rt, device, lambda b, qv, kv, tv, pv: b.paged_flash_multi_latent_attention_decode(qv, kv, 512, tv, cur_pos=pv, scale=0.05),
                         [qb, kb, table, cur])
    assert got[0].shape == (1, 32, 16, 512)
    assert_matches(got[0], want[0], "paged MLA decode bf16, 576 / 512")
