"""gather / scatter / sort / top-k / sampling and the paged KV-cache ops through submit, against the
fixtures recorded from the reference's goldens (tests/golden, keys "map/...") and against the oracle on
larger seeded inputs.  Index results are bit-exact; values are copies of input elements, so they are
bit-exact too."""

import pytest
import torch

from helpers import run_body
from ttmlir_b200 import graphs

pytestmark = pytest.mark.gpu


def test_gather_and_scatter_match_the_reference_goldens(rt, device, golden):
    x = golden["map/gather/x"]
    for name, dim in (("dim1", 1), ("dim2", 2)):
        idx = golden[f"map/gather/idx_{name}"]
        got, want = run_body(rt, device, lambda b, v, i: b.gather(v, i, dim), [x, idx])
        assert torch.equal(got[0], golden[f"map/gather/{name}"]) and torch.equal(want[0], got[0])
    idx, src = golden["map/scatter/idx"], golden["map/scatter/src"]
    got, _ = run_body(rt, device, lambda b, v, i, s: (b.scatter(v, i, s, 1), b.scatter(v, i, s, 1, "Sum")), [x, idx, src])
    assert torch.equal(got[0], golden["map/scatter/dim1"]) and torch.equal(got[1], golden["map/scatter/dim1_sum"])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int32])
def test_gather_scatter_larger_with_duplicates(rt, device, dtype):
    """Duplicated indices: reduce modes apply them in increasing position along the dimension, the order of
    torch's CPU loop, so sums of bf16 values round the same way."""
    g = torch.Generator().manual_seed(3)
    x = (torch.randn(6, 40, 33, generator=g) * 4).to(dtype)
    src = (torch.randn(6, 25, 33, generator=g) * 4).to(dtype)
    idx = torch.randint(0, 40, (6, 25, 33), generator=g, dtype=torch.int32)
    got, want = run_body(rt, device, lambda b, v, i: b.gather(v, i, 1), [x, idx])
    assert torch.equal(got[0], want[0])
    modes = ["Sum", "Max", "Min"] + (["Prod"] if dtype != torch.int32 else [])
    got, want = run_body(rt, device, lambda b, v, i, s: tuple(b.scatter(v, i, s, 1, m) for m in modes), [x, idx, src])
    for m, gv, wv in zip(modes, got, want):
        assert torch.equal(gv, wv), m
    last = torch.randint(0, 33, (6, 40, 7), generator=g, dtype=torch.int32)
    got, want = run_body(rt, device, lambda b, v, i: b.gather(v, i, -1), [x, last])
    assert torch.equal(got[0], want[0])


def test_sort_matches_the_reference_goldens(rt, device, golden):
    x = golden["map/sort/x"]
    for desc in (False, True):
        got, _ = run_body(rt, device, lambda b, v: b.sort(v, -1, desc), [x])
        assert torch.equal(got[0], golden[f"map/sort/values_desc{int(desc)}"])
        assert torch.equal(got[1], golden[f"map/sort/indices_desc{int(desc)}"])
    got, _ = run_body(rt, device, lambda b, v: b.sort(v, 0), [x])
    assert torch.equal(got[0], golden["map/sort/values_dim0"]) and torch.equal(got[1], golden["map/sort/indices_dim0"])


@pytest.mark.parametrize("shape,dim", [((7, 3000), 1), ((4, 5000, 3), 1), ((2, 70000), -1), ((33, 17), 0)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int32])
def test_sort_is_stable_on_long_rows_with_ties(rt, device, shape, dim, dtype):
    """Rows longer than a shared-memory tile (global exchange steps), non-power-of-two lengths, many ties
    (few distinct values), NaN and infinities: values and positions must equal torch.sort(stable=True)."""
    g = torch.Generator().manual_seed(sum(shape))
    if dtype == torch.int32:
        x = torch.randint(-50, 50, shape, generator=g, dtype=torch.int32)
    else:
        x = (torch.randint(-200, 200, shape, generator=g).float() / 8).to(dtype)
        flat = x.view(-1)
        flat[::97] = float("nan")
        flat[1::101] = float("inf")
        flat[2::103] = float("-inf")
        flat[3::107] = -0.0
    for desc in (False, True):
        got, want = run_body(rt, device, lambda b, v: b.sort(v, dim, desc), [x])
        assert torch.equal(got[1], want[1]), (desc, "positions")
        assert torch.equal(got[0].view(torch.int32 if dtype != torch.bfloat16 else torch.int16),
                           want[0].view(torch.int32 if dtype != torch.bfloat16 else torch.int16)), (desc, "values")


def test_topk_matches_the_reference_goldens(rt, device, golden):
    x = golden["map/topk/x"].float()
    for k, largest in ((8, True), (32, True), (5, False)):
        got, _ = run_body(rt, device, lambda b, v: b.topk(v, k, -1, largest), [x])
        values, positions = golden[f"map/topk/values_k{k}_l{int(largest)}"], golden[f"map/topk/indices_k{k}_l{int(largest)}"]
        assert torch.equal(got[0], values)
        assert torch.equal(torch.gather(x, -1, got[1].long()), values)       # every position holds its value
        # Among equal values torch.topk's order is unspecified (the reference's golden says as much); here the
        # earlier position comes first.  Positions must agree wherever the value is unique in its row.
        unique = (x.unsqueeze(-1) == values.unsqueeze(-2)).sum(dim=-2) == 1
        assert torch.equal(got[1][unique], positions[unique])
        ties = ~unique
        if ties.any():
            same_set = torch.sort(torch.where(ties, got[1], -1), dim=-1).values == torch.sort(torch.where(ties, positions, -1), dim=-1).values
            first_tie = got[1][..., 1:][(values[..., 1:] == values[..., :-1])] > got[1][..., :-1][(values[..., 1:] == values[..., :-1])]
            assert first_tie.all()                                            # stable: earlier position first


def test_topk_over_a_vocabulary(rt, device):
    g = torch.Generator().manual_seed(9)
    logits = torch.randn(8, 128256, generator=g).to(torch.bfloat16).float()
    logits += torch.arange(128256) * 1e-9          # no exact ties: torch.topk's order among equals is unspecified
    got, want = run_body(rt, device, lambda b, v: b.topk(v, 64), [logits])
    assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])


def test_paged_cache_ops_match_the_reference_goldens(rt, device, golden):
    cache, table = golden["map/paged/cache"], golden["map/paged/page_table"]
    pos = golden["map/paged/update_pos"]

    def updated(b, c, x, p, t):
        b.paged_update_cache(c, x, p, t)
        return b.typecast(c, "BFloat16")            # an op that reads the cache: programs return values, not aliases
    got, _ = run_body(rt, device, updated, [cache, golden["map/paged/update_in"], pos, table])
    assert torch.equal(got[0], golden["map/paged/updated"])

    def filled(b, c, x, t, bi):
        b.paged_fill_cache(c, x, t, bi)
        return b.typecast(c, "BFloat16")
    got, _ = run_body(rt, device, filled, [cache, golden["map/paged/fill_in"], table, torch.tensor([1], dtype=torch.int32)])
    assert torch.equal(got[0], golden["map/paged/filled_user1"])
    got, _ = run_body(rt, device, lambda b, q, k, v, t, p: b.paged_scaled_dot_product_attention_decode(q, k, v, t, p),
                      [golden["map/paged/q"], cache, golden["map/paged/v_cache"], table, pos])
    want = golden["map/paged/decode"]
    assert torch.allclose(got[0].float(), want.float(), atol=1e-2, rtol=2.0 ** -7)


@pytest.mark.parametrize("heads,kv_heads,d", [(32, 8, 128), (8, 8, 64), (16, 2, 128)])
def test_paged_decode_equals_decode_over_the_unpaged_cache(rt, device, heads, kv_heads, d):
    """A shuffled page table over a block pool: attention through it must equal -- bit for bit, same kernel,
    same summation order -- attention over the contiguous cache the pages spell out."""
    g = torch.Generator().manual_seed(heads)
    users, block, pages = 5, 32, 40                    # 1280 positions per user: several key chunks
    blocks = users * pages + 7
    perm = torch.randperm(blocks, generator=g)[: users * pages].reshape(users, pages).to(torch.int32)
    kc = torch.randn(blocks, kv_heads, block, d, generator=g).to(torch.bfloat16)
    vc = torch.randn(blocks, kv_heads, block, d, generator=g).to(torch.bfloat16)
    q = torch.randn(users, 1, heads, d, generator=g).to(torch.bfloat16)
    pos = torch.tensor([0, 31, 32, 700, 1279], dtype=torch.int32)

    def unpage(c):
        return c[perm.long().reshape(-1)].reshape(users, pages, kv_heads, block, d).transpose(1, 2).reshape(users, kv_heads, pages * block, d).contiguous()
    scale = d ** -0.5
    got, want = run_body(rt, device, lambda b, qq, k, v, t, p: b.paged_scaled_dot_product_attention_decode(qq, k, v, t, p, scale=scale),
                         [q, kc, vc, perm, pos])
    assert torch.allclose(got[0].float(), want[0].float(), atol=1e-2, rtol=2.0 ** -7)
    flat, _ = run_body(rt, device, lambda b, qq, k, v, p: b.scaled_dot_product_attention_decode(qq, k, v, p, scale=scale),
                       [q.reshape(1, users, heads, d), unpage(kc), unpage(vc), pos])
    assert torch.equal(got[0].reshape(-1), flat[0].reshape(-1))


def sampling_body(seed):
    return lambda b, v, i, k, p, t: b.sampling(v, i, k, p, t, seed=seed)


def test_sampling_support_and_determinism(rt, device):
    """The draw is stochastic by definition (the reference's golden says so and switches comparison off):
    what can be pinned is the support -- k = 1 or a tiny p give the most probable candidate, the result is
    always among the k most probable -- and that (seed, row) determines the draw."""
    g = torch.Generator().manual_seed(17)
    rows, cand = 64, 50
    values = (torch.randn(rows, cand, generator=g) * 3).to(torch.bfloat16)
    indices = torch.stack([torch.randperm(100000, generator=g)[:cand] for _ in range(rows)]).to(torch.int32)
    temp = torch.full((rows,), 0.7, dtype=torch.bfloat16)
    best = indices[torch.arange(rows), values.float().argmax(dim=1)]
    one, _ = run_body(rt, device, sampling_body(1), [values, indices, torch.ones(rows, dtype=torch.int32).view(torch.int32), torch.ones(rows, dtype=torch.bfloat16), temp])
    assert torch.equal(one[0], best)
    tiny_p, _ = run_body(rt, device, sampling_body(2), [values, indices, torch.zeros(rows, dtype=torch.int32), torch.full((rows,), 1e-3, dtype=torch.bfloat16), temp])
    assert torch.equal(tiny_p[0], best)
    k5 = torch.full((rows,), 5, dtype=torch.int32)
    a, _ = run_body(rt, device, sampling_body(3), [values, indices, k5, torch.ones(rows, dtype=torch.bfloat16), temp])
    b2, _ = run_body(rt, device, sampling_body(3), [values, indices, k5, torch.ones(rows, dtype=torch.bfloat16), temp])
    c, _ = run_body(rt, device, sampling_body(4), [values, indices, k5, torch.ones(rows, dtype=torch.bfloat16), temp])
    assert torch.equal(a[0], b2[0]) and not torch.equal(a[0], c[0])
    top5 = torch.gather(indices, 1, values.float().topk(5, dim=1).indices)
    assert all(int(a[0][r]) in top5[r].tolist() for r in range(rows))


def test_sampling_follows_the_softmax_distribution(rt, device):
    """Many rows with the same six logits: the empirical frequencies must be close to softmax(values / temp)
    restricted to the nucleus (the golden's distribution, tools/golden/mapping.py:6008-6012)."""
    rows = 20000
    logits = torch.tensor([2.0, 1.0, 0.5, 0.0, -1.0, -3.0])
    values = logits.repeat(rows, 1).to(torch.float32)
    indices = torch.arange(6, dtype=torch.int32).repeat(rows, 1)
    temp = torch.full((rows,), 0.8)
    got, _ = run_body(rt, device, sampling_body(11), [values, indices, torch.zeros(rows, dtype=torch.int32), torch.ones(rows), temp])
    freq = torch.bincount(got[0].long(), minlength=6).float() / rows
    want = torch.softmax(logits / 0.8, dim=0)
    assert (freq - want).abs().max() < 0.015, (freq, want)
    # nucleus p = 0.8 keeps the first three candidates (mass 0.62, 0.80 reached with the second or third)
    got, _ = run_body(rt, device, sampling_body(12), [values, indices, torch.zeros(rows, dtype=torch.int32), torch.full((rows,), 0.8), temp])
    freq = torch.bincount(got[0].long(), minlength=6).float() / rows
    cum = torch.cumsum(want, 0)
    keep = int((cum < 0.8).sum().item()) + 1
    nucleus = torch.zeros(6)
    nucleus[:keep] = want[:keep] / want[:keep].sum()
    assert (freq - nucleus).abs().max() < 0.015 and freq[keep:].sum() == 0, (freq, nucleus)
