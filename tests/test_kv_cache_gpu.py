"""fill_cache, update_cache and decode attention through tt::runtime::submit against the CPU
restatement of the reference's goldens (tools/golden/mapping.py: fill_cache_golden,
update_cache_golden, sdpa_decode_golden)."""

import math

import pytest
import torch

from helpers import assert_matches, run_body

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("users,heads,seq,max_seq,dim,offset,cache_users", [
    (1, 8, 100, 256, 64, 0, 1), (2, 4, 64, 64, 128, 1, 4), (3, 2, 33, 40, 96, 0, 3), (1, 8, 1000, 2048, 128, 2, 4)])
def test_fill_cache(rt, device, users, heads, seq, max_seq, dim, offset, cache_users):
    torch.manual_seed(seq)
    cache = torch.randn(cache_users, heads, max_seq, dim).to(torch.bfloat16)
    x = torch.randn(users, heads, seq, dim).to(torch.bfloat16)
    got, want = run_body(rt, device, lambda b, c, v: b.fill_cache(c, v, offset), [cache, x])
    assert torch.equal(got[0], want[0])
    assert torch.equal(got[0][offset:offset + users, :, :seq], x)
    untouched = [u for u in range(cache_users) if not offset <= u < offset + users]
    assert torch.equal(got[0][untouched], cache[untouched])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_update_cache_reads_its_index_from_a_tensor(rt, device, dtype):
    torch.manual_seed(3)
    cache = torch.randn(6, 4, 300, 128).to(dtype)
    x = torch.randn(1, 4, 3, 128).to(dtype)
    for idx, offset in ((0, 0), (299, 3), (77, 2)):
        index = torch.tensor([idx], dtype=torch.int32)
        got, want = run_body(rt, device, lambda b, c, v, i: b.update_cache(c, v, i, offset), [cache, x, index])
        assert torch.equal(got[0], want[0])
        assert torch.equal(got[0][offset:offset + 3, :, idx], x[0].permute(1, 0, 2))
        changed = (got[0] != cache).any(dim=-1)
        assert changed.sum().item() <= 3 * 4


CASES = [  # batch, heads, kv_heads, seq, head_dim
    (1, 8, 8, 100, 64), (2, 8, 2, 700, 128), (4, 32, 8, 2048, 128), (1, 16, 2, 1500, 256), (3, 4, 4, 513, 128),
    (2, 16, 2, 4100, 128)]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("B,H,Hkv,S,D", CASES)
def test_sdpa_decode_causal_positions(rt, device, dtype, B, H, Hkv, S, D):
    torch.manual_seed(B * S + H)
    q = torch.randn(1, B, H, D).to(dtype)
    k = torch.randn(B, Hkv, S, D).to(dtype)
    v = torch.randn(B, Hkv, S, D).to(dtype)
    pos = torch.tensor([(S - 1) if i == 0 else (i * 37) % S for i in range(B)], dtype=torch.int32)
    scale = 1.0 / math.sqrt(D)
    got, want = run_body(rt, device, lambda b, qq, kk, vv, pp: b.scaled_dot_product_attention_decode(qq, kk, vv, pp, None, True,
                                                                                                     scale), [q, k, v, pos])
    assert_matches(got[0], want[0], f"sdpa_decode {B}x{H}/{Hkv}x{S}x{D}", (0.999, 1e-2, 2.0 ** -6))
    again, _ = run_body(rt, device, lambda b, qq, kk, vv, pp: b.scaled_dot_product_attention_decode(qq, kk, vv, pp, None, True,
                                                                                                    scale), [q, k, v, pos])
    assert torch.equal(got[0], again[0]), "two runs differ"


def test_sdpa_decode_masks_and_no_scale(rt, device):
    torch.manual_seed(8)
    B, H, Hkv, S, D = 2, 8, 4, 600, 128
    q = (torch.randn(1, B, H, D) * 0.3).to(torch.bfloat16)
    k = (torch.randn(B, Hkv, S, D) * 0.3).to(torch.bfloat16)
    v = torch.randn(B, Hkv, S, D).to(torch.bfloat16)
    for mshape in ((B, 1, H, S), (1, 1, 1, S), (B, 1, 1, S), (1, 1, H, S)):
        mask = torch.zeros(mshape)
        mask[..., 400:] = float("-inf")
        mask[..., ::7] = -2.0
        mask = mask.to(torch.bfloat16)
        got, want = run_body(rt, device, lambda b, qq, kk, vv, mm: b.scaled_dot_product_attention_decode(qq, kk, vv, None, mm, False,
                                                                                                         0.125), [q, k, v, mask])
        assert_matches(got[0], want[0], f"sdpa_decode mask {mshape}", (0.999, 1e-2, 2.0 ** -6))
    # no scale on the op: the scores are used as they are; not causal and no positions: every key counts
    got, want = run_body(rt, device, lambda b, qq, kk, vv: b.scaled_dot_product_attention_decode(qq, kk, vv, None, None, False, None),
                         [q, k, v])
    assert_matches(got[0], want[0], "sdpa_decode without scale", (0.999, 1e-2, 2.0 ** -6))


def test_decode_step_updates_the_cache_then_attends(rt, device):
    """One decode step of a serving loop: the new key / value rows go into the caches at the current
    position, then the query attends to everything up to and including that position."""
    torch.manual_seed(21)
    B, H, Hkv, S, D, at = 4, 16, 4, 1024, 128, 333
    q = torch.randn(1, B, H, D).to(torch.bfloat16)
    kc = torch.randn(B, Hkv, S, D).to(torch.bfloat16)
    vc = torch.randn(B, Hkv, S, D).to(torch.bfloat16)
    kn = torch.randn(1, Hkv, B, D).to(torch.bfloat16)
    vn = torch.randn(1, Hkv, B, D).to(torch.bfloat16)
    index = torch.tensor([at], dtype=torch.int32)
    pos = torch.full((B,), at, dtype=torch.int32)

    def body(b, qq, kcc, vcc, knn, vnn, ii, pp):
        kcc = b.update_cache(kcc, knn, ii)
        vcc = b.update_cache(vcc, vnn, ii)
        return b.scaled_dot_product_attention_decode(qq, kcc, vcc, pp, None, True, 1.0 / math.sqrt(D)), kcc, vcc
    got, want = run_body(rt, device, body, [q, kc, vc, kn, vn, index, pos])
    assert_matches(got[0], want[0], "decode step", (0.999, 1e-2, 2.0 ** -6))
    assert torch.equal(got[1], want[1]) and torch.equal(got[2], want[2])
    assert torch.equal(got[1][:, :, at], kn[0].permute(1, 0, 2))


def test_bad_positions_and_indices_are_reported_not_followed(rt, device):
    """An update position outside the cache writes nothing, an embedding index outside the table reads
    row 0; neither touches memory it should not, and the next wait on a device tensor says so (once)."""
    from ttmlir_b200 import graphs
    cache = torch.randn(2, 2, 64, 64).to(torch.bfloat16)
    x = torch.randn(1, 2, 2, 64).to(torch.bfloat16)

    def run(graph, inputs):
        binary = rt.Binary.load_from_memory(graphs.build_binary(graph))
        ins = [rt.to_layout(rt.from_torch(t), device, rt.get_layout(binary, 0, i)) for i, t in enumerate(inputs)]
        return rt.submit(device, binary, 0, ins)

    def upd(b):
        c = b.input([2, 2, 64, 64], "BFloat16"); v = b.input([1, 2, 2, 64], "BFloat16"); i = b.input([1], "Int32")
        b.output(b.update_cache(c, v, i))
    out = run(upd, [cache, x, torch.tensor([64], dtype=torch.int32)])
    with pytest.raises(RuntimeError, match="outside the cache"):
        rt.wait(out[0])
    assert torch.equal(rt.to_torch(rt.to_host(out[0], untilize=True)[0]), cache)      # nothing was written
    rt.wait(out[0])                                                                    # reported once

    table = torch.randn(10, 32)

    def emb(b):
        i = b.input([4], "Int32"); w = b.input([10, 32], "Float32")
        b.output(b.embedding(i, w))
    out = run(emb, [torch.tensor([1, 10, -3, 9], dtype=torch.int32), table])
    with pytest.raises(RuntimeError, match="outside its table"):
        rt.wait(out[0])
    got = rt.to_torch(rt.to_host(out[0], untilize=True)[0])
    assert torch.equal(got, table[[1, 0, 0, 9]])
