"""layer_norm, argmax, cumsum, embedding, pooling, pad through tt::runtime::submit, against the CPU
oracle and against the outputs of the reference's own CPU code recorded in tests/golden."""

import pytest
import torch

from helpers import POOL_CASES, assert_matches, pool_on, run_body

pytestmark = pytest.mark.gpu


def test_layer_norm_matches_the_reference_outputs(rt, device, golden):
    x, w, b = golden["ln/x"], golden["ln/w"], golden["ln/b"]
    got, want = run_body(rt, device, lambda bb, xv, wv, bv: (bb.layer_norm(xv), bb.layer_norm(xv, wv, bv)), [x, w, b])
    assert_matches(got[0], golden["ln/plain"], "layer_norm plain vs reference")
    assert_matches(got[1], golden["ln/affine"], "layer_norm affine vs reference")
    got, _ = run_body(rt, device, lambda bb, xv, wv: bb.layer_norm(xv, wv, None, 1e-3), [x, golden["ln/w2"]])
    assert_matches(got[0], golden["ln/two_dims"], "layer_norm over two dims vs reference")


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("rows,cols", [(1, 8), (37, 1000), (2048, 4096), (5, 12289)])
def test_layer_norm_sizes(rt, device, dtype, rows, cols):
    torch.manual_seed(rows + cols)
    x = (torch.randn(rows, cols) * 3 + 1.5).to(dtype)
    w = (1 + 0.1 * torch.randn(cols)).to(dtype)
    b = (0.1 * torch.randn(cols)).to(dtype)
    got, want = run_body(rt, device, lambda bb, xv, wv, bv: bb.layer_norm(xv, wv, bv), [x, w, b])
    assert_matches(got[0], want[0], f"layer_norm {rows}x{cols}")


def test_argmax_matches_the_reference_outputs(rt, device, golden):
    x = golden["arg/x"]
    got, _ = run_body(rt, device, lambda b, v: (b.argmax(v, 0), b.argmax(v, 1), b.argmax(v, 2), b.argmax(v),
                                                b.argmax(v, 1, True)), [x])
    for g, name in zip(got, ["dim0", "dim1", "dim2", "all", "keep"]):
        assert torch.equal(g, golden[f"arg/{name}"]), name


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int32])
def test_argmax_ties_nan_and_long_rows(rt, device, dtype):
    torch.manual_seed(5)
    x = torch.randint(-8, 8, (33, 5000)).to(dtype)          # many ties: the first maximum wins
    if dtype.is_floating_point:
        x[3, 1234] = float("nan")                            # a NaN counts as the maximum
        x[4, 7] = float("nan")
        x[4, 4000] = float("nan")                            # ... and the first NaN wins
    got, want = run_body(rt, device, lambda b, v: (b.argmax(v, 1), b.argmax(v, 0), b.argmax(v)), [x])
    for g, w in zip(got, want):
        assert torch.equal(g, w)


def test_cumsum_embedding_pad_match_the_reference_outputs(rt, device, golden):
    got, _ = run_body(rt, device, lambda b, v: (b.cumsum(v, 0), b.cumsum(v, 1), b.cumsum(v, 2)), [golden["cum/x"]])
    for d, g in enumerate(got):
        assert_matches(g, golden[f"cum/dim{d}"], f"cumsum dim {d}", (0.9999, 1e-5, 1e-5))
    got, _ = run_body(rt, device, lambda b, v: b.cumsum(v, 1), [golden["cum/xi"]])
    assert torch.equal(got[0], golden["cum/int"])
    got, _ = run_body(rt, device, lambda b, i, w: b.embedding(i, w), [golden["emb/idx"], golden["emb/w"]])
    assert torch.equal(got[0], golden["emb/out"])
    got, _ = run_body(rt, device, lambda b, v: b.pad(v, [1, 0, 0, 2, 3, 1], -1.5), [golden["pad/x"]])
    assert torch.equal(got[0], golden["pad/out"])


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_embedding_llm_sized_table(rt, device, dtype):
    torch.manual_seed(9)
    vocab, dim = 32000, 4096 if dtype == torch.bfloat16 else 1000
    table = torch.randn(vocab, dim).to(dtype)
    idx = torch.randint(0, vocab, (4, 512), dtype=torch.int32)
    idx[0, 0], idx[0, 1] = 0, vocab - 1
    got, want = run_body(rt, device, lambda b, i, w: b.embedding(i, w), [idx, table])
    assert torch.equal(got[0], want[0])
    # bf16 index tensors (what TTNN graphs often carry) hold the small integers exactly
    small = torch.randint(0, 256, (3, 40)).to(torch.bfloat16)
    got, want = run_body(rt, device, lambda b, i, w: b.embedding(i, w), [small, table])
    assert torch.equal(got[0], want[0])


@pytest.mark.parametrize("case", sorted(POOL_CASES))
def test_pooling_matches_the_reference_outputs(rt, device, golden, case):
    x = golden["pool/x"].reshape(1, 1, -1, 8)
    got, want = run_body(rt, device, lambda b, v: pool_on(b, v, case), [x])
    ref = golden[f"pool/{case}"].reshape(1, 1, -1, 8)
    if case.startswith("max"):
        assert torch.equal(got[0], ref)
    else:
        assert_matches(got[0], ref, f"{case} vs reference", (0.9999, 1e-6, 1e-5))
    # bf16 activations, channel count that is not a multiple of the 16-byte vector
    xb = golden["pool/x"][..., :7].contiguous().to(torch.bfloat16).reshape(1, 1, -1, 7)
    got, want = run_body(rt, device, lambda b, v: pool_on(b, v, case, channels=7), [xb])
    if case.startswith("max"):
        assert torch.equal(got[0], want[0])        # a maximum is exact; windows that lie in the padding give -inf
    else:
        assert_matches(got[0], want[0], f"{case} bf16 c=7")


def test_resnet_stem_pool_and_head(rt, device):
    """The pooling of a ResNet: 3x3 / 2 max pool with padding 1 over [8, 112, 112, 64] and the global
    average over [8, 7, 7, 2048], bf16."""
    torch.manual_seed(2)
    x = torch.randn(8, 112, 112, 64).to(torch.bfloat16)
    got, want = run_body(rt, device, lambda b, v: b.max_pool2d(b.reshape(v, [1, 1, 8 * 112 * 112, 64]), 8, 112, 112, 64,
                                                              (3, 3), (2, 2), (1, 1)), [x])
    assert list(got[0].shape) == [1, 1, 8 * 56 * 56, 64] and torch.equal(got[0], want[0])
    y = torch.randn(8, 7, 7, 2048).to(torch.bfloat16)
    got, want = run_body(rt, device, lambda b, v: b.global_avg_pool2d(v), [y])
    assert_matches(got[0], want[0], "global_avg_pool2d")


def test_pad_dtypes_and_ranks(rt, device):
    torch.manual_seed(4)
    for t in (torch.randn(3, 4, 5, 6).to(torch.bfloat16), torch.randint(-9, 9, (7, 9), dtype=torch.int32), torch.randn(17)):
        padding = [((i * 3) % 4, (i + 1) % 3) for i in range(t.dim())]
        flat = [p for pair in padding for p in pair]
        got, want = run_body(rt, device, lambda b, v: b.pad(v, flat, 2.0), [t])
        assert torch.equal(got[0], want[0])
