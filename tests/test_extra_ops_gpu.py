"""cumprod, prod, inference batch norm, 2-D upsampling and the conv2d preparation ops through tt::runtime::submit,
against the outputs of the reference's own goldens (tests/golden, recorded from tools/golden/mapping.py) and the oracle."""

import pytest
import torch

from helpers import assert_matches, run_body

pytestmark = pytest.mark.gpu


def test_cumprod_matches_the_reference_goldens(rt, device, golden):
    x = golden["map/cumprod/x"]
    for d in (0, 1, 2):
        got, want = run_body(rt, device, lambda b, v: b.cumprod(v, d), [x])
        assert torch.equal(got[0], golden[f"map/cumprod/dim{d}"]) and torch.equal(want[0], got[0])
    xi = golden["map/cumprod/x_i32"]
    got, _ = run_body(rt, device, lambda b, v: b.cumprod(v, 1), [xi])
    assert torch.equal(got[0], golden["map/cumprod/i32_dim1"])
    # bf16: the running product is f32 on both sides, every prefix rounded once
    xb = golden["map/cumprod/x_bf16"]
    got, _ = run_body(rt, device, lambda b, v: b.cumprod(v, 1), [xb])
    assert torch.equal(got[0], golden["map/cumprod/bf16_dim1"])


def test_prod_matches_the_reference_goldens(rt, device, golden):
    x = golden["map/cumprod/x"]
    got, want = run_body(rt, device, lambda b, v: (b.prod(v, 1), b.prod(v, 2, keep_dim=True), b.prod(v, None, keep_dim=True)), [x])
    for g, w, name in zip(got, want, ("map/prod/dim1", "map/prod/dim2_keep", None)):
        assert torch.allclose(g, w, rtol=1e-5, atol=1e-7)            # f32 products: the order of the factors differs
        if name:
            assert torch.allclose(g, golden[name], rtol=1e-5, atol=1e-7) and g.shape == golden[name].shape
    assert torch.allclose(got[2].reshape(1), golden["map/prod/all"], rtol=1e-5, atol=0)
    xi = golden["map/cumprod/x_i32"]
    got, _ = run_body(rt, device, lambda b, v: b.prod(v, 0), [xi])
    assert torch.equal(got[0], golden["map/prod/i32_dim0"])                 # integers: exact


@pytest.mark.parametrize("shape", [(5, 1000), (3, 7, 4096), (2, 33)])
def test_prod_shapes(rt, device, shape):
    torch.manual_seed(len(shape))
    x = torch.rand(*shape) * 0.2 + 0.9
    for dim in range(len(shape)):
        got, want = run_body(rt, device, lambda b, v: b.prod(v, dim), [x])
        assert torch.allclose(got[0], want[0], rtol=2e-5, atol=1e-30), f"dim {dim}"
    xb = x.to(torch.bfloat16)
    got, want = run_body(rt, device, lambda b, v: b.prod(v, -1), [xb])
    assert_matches(got[0], want[0], "prod bf16", (0.999, 1e-2, 2.0 ** -6))


def test_batch_norm_inference_matches_the_reference_golden(rt, device, golden):
    x, mean, var, w, b_ = (golden[f"map/batch_norm/{n}"] for n in ("x", "mean", "var", "weight", "bias"))
    got, want = run_body(rt, device, lambda b, *v: b.batch_norm_inference(v[0], v[1], v[2], v[3], v[4], 1e-5), [x, mean, var, w, b_])
    # torch folds the statistics into one multiplier and one offset per channel first; same value up to f32 rounding
    assert torch.allclose(got[0], golden["map/batch_norm/out"], rtol=1e-5, atol=1e-6)
    assert torch.allclose(got[0], want[0], rtol=1e-5, atol=1e-6)
    got, _ = run_body(rt, device, lambda b, *v: b.batch_norm_inference(v[0], v[1], v[2], None, None, 1e-5), [x, mean, var])
    ref = (x - mean[None, :, None, None]) / torch.sqrt(var[None, :, None, None] + 1e-5)
    assert torch.allclose(got[0], ref, rtol=1e-5, atol=1e-6)
    bf = torch.bfloat16
    got, want = run_body(rt, device, lambda b, *v: b.batch_norm_inference(v[0], v[1], v[2], v[3], v[4], 1e-5),
                         [t.to(bf) for t in (x, mean, var, w, b_)])
    assert_matches(got[0], want[0], "batch norm bf16", (0.999, 1e-2, 2.0 ** -7))
    assert_matches(got[0], golden["map/batch_norm/out_bf16"], "batch norm bf16 vs torch's bf16 evaluation", (0.999, 2e-2, 2.0 ** -6))


def test_upsample_matches_the_reference_goldens(rt, device, golden):
    x = golden["map/upsample/x"]
    got, want = run_body(rt, device, lambda b, v: (b.upsample(v, 2), b.upsample(v, 3), b.upsample(v, 2, "bilinear")), [x])
    assert torch.equal(got[0], golden["map/upsample/nearest_x2"]) and torch.equal(got[1], golden["map/upsample/nearest_x3"])
    assert torch.allclose(got[2], golden["map/upsample/bilinear_x2"], atol=1e-5, rtol=0)
    assert torch.equal(want[0], got[0]) and torch.allclose(want[2], got[2], atol=1e-5, rtol=0)


def test_upsample_non_square_and_two_scales(rt, device):
    torch.manual_seed(11)
    x = torch.randn(3, 5, 9, 16).to(torch.bfloat16)
    got, want = run_body(rt, device, lambda b, v: (b.upsample(v, (2, 3)), b.upsample(v, (3, 2), "bilinear")), [x])
    assert torch.equal(got[0], want[0])
    assert_matches(got[1], want[1], "bilinear (3, 2)", (0.999, 1e-2, 2.0 ** -7))


def test_conv2d_through_prepared_weights_and_bias(rt, device):
    """The optimizer puts prepare_conv2d_weights / prepare_conv2d_bias in front of conv2d and declares TTNN's prepared
    layout as their result type; here they hand the tensors on, and the convolution must give exactly what it gives on the
    raw weights."""
    torch.manual_seed(5)
    n, hw, c, o = 2, 10, 64, 96
    x = torch.randn(1, 1, n * hw * hw, c).to(torch.bfloat16)
    w = (torch.randn(o, c, 3, 3) * 0.05).to(torch.bfloat16)
    bias = torch.randn(1, 1, 1, o).to(torch.bfloat16)

    def prepared(b, xv, wv, bv):
        pw = b.prepare_conv2d_weights(wv, n, hw, hw, padding=(1, 1, 1, 1))
        pb = b.prepare_conv2d_bias(bv, list(w.shape), n, hw, hw, padding=(1, 1, 1, 1))
        return b.relu(b.conv2d(xv, pw, pb, n, hw, hw, padding=(1, 1, 1, 1)))

    def raw(b, xv, wv, bv):
        return b.relu(b.conv2d(xv, wv, bv, n, hw, hw, padding=(1, 1, 1, 1)))
    got, want = run_body(rt, device, prepared, [x, w, bias])
    direct, _ = run_body(rt, device, raw, [x, w, bias])
    assert torch.equal(got[0], direct[0])
    assert_matches(got[0], want[0], "conv2d on prepared weights", (0.999, 2e-2, 2.0 ** -6))


def test_group_norm_matches_the_reference_goldens(rt, device, golden):
    x, w, b_ = (golden[f"map/group_norm/{n}"] for n in ("x", "weight", "bias"))
    got, want = run_body(rt, device, lambda b, xv, wv, bv: b.group_norm(xv, wv, bv, 3, 1e-5), [x, w, b_])
    assert torch.allclose(got[0], golden["map/group_norm/g3"], rtol=1e-5, atol=2e-6) and torch.allclose(got[0], want[0], rtol=1e-5, atol=2e-6)
    got, _ = run_body(rt, device, lambda b, xv: b.group_norm(xv, None, None, 12, 1e-5), [x])
    assert torch.allclose(got[0], golden["map/group_norm/g12_noaffine"], rtol=1e-5, atol=2e-6)
    torch.manual_seed(2)
    xb = torch.randn(3, 1, 196, 64).to(torch.bfloat16)
    wb, bb = (torch.randn(64) * 0.5 + 1).to(torch.bfloat16), (torch.randn(64) * 0.2).to(torch.bfloat16)
    got, want = run_body(rt, device, lambda b, xv, wv, bv: b.group_norm(xv, wv, bv, 8, 1e-5), [xb, wb, bb])
    assert_matches(got[0], want[0], "group norm bf16", (0.999, 1e-2, 2.0 ** -7))


def test_conv_transpose2d_matches_the_reference_goldens(rt, device, golden):
    x, w, b_ = (golden[f"map/conv_transpose/{n}"] for n in ("x", "w", "b"))
    got, want = run_body(rt, device, lambda b, xv, wv, bv: b.conv_transpose2d(xv, wv, bv, 2, 5, 6, stride=(2, 2), padding=(1, 1),
                                                                              output_padding=(1, 1)), [x, w, b_])
    assert got[0].shape == golden["map/conv_transpose/s2_p1_op1"].shape
    assert torch.allclose(got[0], golden["map/conv_transpose/s2_p1_op1"], rtol=1e-5, atol=1e-5)
    assert torch.allclose(got[0], want[0], rtol=1e-5, atol=1e-5)
    wg = golden["map/conv_transpose/w_g2"]
    got, _ = run_body(rt, device, lambda b, xv, wv: b.conv_transpose2d(xv, wv, None, 2, 5, 6, stride=(1, 2), padding=(0, 1),
                                                                       dilation=(2, 1), groups=2), [x, wg])
    assert torch.allclose(got[0], golden["map/conv_transpose/g2_s1x2_d2"], rtol=1e-5, atol=1e-5)
    torch.manual_seed(3)                                        # bf16, flattened activations as the compiler emits them
    xb = torch.randn(1, 1, 2 * 7 * 7, 32).to(torch.bfloat16)
    wb = (torch.randn(32, 16, 2, 2) * 0.1).to(torch.bfloat16)
    got, want = run_body(rt, device, lambda b, xv, wv: b.conv_transpose2d(xv, wv, None, 2, 7, 7, stride=(2, 2)), [xb, wb])
    assert list(got[0].shape) == [1, 1, 2 * 14 * 14, 16]
    assert_matches(got[0], want[0], "conv_transpose2d bf16", (0.999, 1e-2, 2.0 ** -7))


def test_conv1d_matches_the_reference_golden(rt, device, golden):
    x, w, b_ = (golden[f"map/conv1d/{n}"] for n in ("x", "w", "b"))
    got, want = run_body(rt, device, lambda b, xv, wv, bv: b.conv1d(xv, wv, bv, 3, 17, stride=2, padding=(1, 2)), [x, w, b_])
    assert got[0].shape == golden["map/conv1d/s2_p1x2"].shape
    assert torch.allclose(got[0], golden["map/conv1d/s2_p1x2"], rtol=1e-4, atol=1e-5) and torch.allclose(got[0], want[0], rtol=1e-4, atol=1e-5)
    torch.manual_seed(4)
    xb = torch.randn(2, 300, 64).to(torch.bfloat16)
    wb = (torch.randn(128, 64, 3) * 0.05).to(torch.bfloat16)
    bb = torch.randn(1, 1, 128).to(torch.bfloat16)
    got, want = run_body(rt, device, lambda b, xv, wv, bv: b.conv1d(xv, wv, bv, 2, 300, padding=(1, 1)), [xb, wb, bb])
    assert_matches(got[0], want[0], "conv1d bf16", (0.999, 2e-2, 2.0 ** -6))


def test_bitcast_convert_and_nlp_concat_heads(rt, device):
    torch.manual_seed(6)
    x = torch.randn(4, 33)
    got, want = run_body(rt, device, lambda b, v: b.bitcast_convert(v, "Int32"), [x])
    assert torch.equal(got[0], x.view(torch.int32)) and torch.equal(want[0], got[0])
    h = torch.randn(2, 4, 9, 32).to(torch.bfloat16)
    got, want = run_body(rt, device, lambda b, v: b.nlp_concat_heads(v), [h])
    assert torch.equal(got[0], h.permute(0, 2, 1, 3).reshape(2, 1, 9, 128)) and torch.equal(want[0], got[0])
