"""Per-op parity on the GPU: every op runs through the runtime's C ABI and is compared with the
fixtures recorded from the reference's CPU code and with the CPU oracle."""

import pytest
import torch

from helpers import assert_matches, run_body

pytestmark = pytest.mark.gpu

UNARY = {"abs": "Abs", "ceil": "Ceil", "cos": "Cos", "floor": "Floor", "gelu": "Gelu", "neg": "Neg", "relu": "Relu",
         "sigmoid": "Sigmoid", "sin": "Sin", "sign": "Sign", "tan": "Tan", "tanh": "Tanh", "atan": "Atan", "exp": "Exp",
         "erf": "Erf", "erfc": "Erfc", "expm1": "Expm1", "relu6": "Relu6", "silu": "Silu", "hardsigmoid": "Hardsigmoid",
         "mish": "Mish", "asinh": "Asinh"}
UNARY_POS = {"sqrt": "Sqrt", "rsqrt": "Rsqrt", "reciprocal": "Reciprocal", "log": "Log"}
F32 = (0.999, 1e-4, 1e-4)


@pytest.mark.parametrize("name", sorted(UNARY))
def test_unary_vs_reference_fixture(rt, device, golden, name):
    got, want = run_body(rt, device, lambda b, x: b.unary(UNARY[name], x), [golden["unary/x"]])
    assert_matches(got[0], golden[f"unary/{name}"], name, F32)
    assert_matches(got[0], want[0], name + " (oracle)", F32)


@pytest.mark.parametrize("name", sorted(UNARY_POS))
def test_unary_positive(rt, device, golden, name):
    got, _ = run_body(rt, device, lambda b, x: b.unary(UNARY_POS[name], x), [golden["unary/xpos"]])
    assert_matches(got[0], golden[f"unary/{name}"], name, F32)


def test_unary_bf16_rounds_once(rt, device):
    x = (torch.randn(33, 65) * 3).to(torch.bfloat16)
    for kind in ["Exp", "Silu", "Sigmoid", "Relu", "Neg", "Tanh"]:
        got, want = run_body(rt, device, lambda b, v: b.unary(kind, v), [x])
        assert_matches(got[0], want[0], kind)


def test_leaky_relu_param(rt, device, golden):
    got, _ = run_body(rt, device, lambda b, x: b.unary("LeakyRelu", x, 0.01), [golden["unary/x"]])
    assert_matches(got[0], golden["unary/leaky_relu"], "leaky_relu", F32)


BINARY = {"add": "Add", "subtract": "Subtract", "multiply": "Multiply", "div": "Divide", "maximum": "Maximum",
          "minimum": "Minimum", "eq": "Equal", "ne": "NotEqual", "gt": "GreaterThan", "ge": "GreaterEqual",
          "lt": "LessThan", "le": "LessEqual"}


@pytest.mark.parametrize("name", sorted(BINARY))
def test_binary_broadcast(rt, device, golden, name):
    got, _ = run_body(rt, device, lambda b, x, y: b.binary(BINARY[name], x, y), [golden["binary/a"], golden["binary/b"]])
    assert_matches(got[0], golden[f"binary/{name}"], name, F32)


def test_binary_row_vector_and_int(rt, device, golden):
    got, _ = run_body(rt, device, lambda b, x, y: b.add(x, y), [golden["binary/a"], golden["binary/row"]])
    assert_matches(got[0], golden["binary/add_row"], "add row", F32)
    a = torch.randint(-2 ** 30, 2 ** 30, (5, 7), dtype=torch.int32)
    c = torch.randint(-2 ** 30, 2 ** 30, (5, 7), dtype=torch.int32)
    got, want = run_body(rt, device, lambda b, x, y: (b.add(x, y), b.subtract(x, y), b.binary("BitwiseAnd", x, y)), [a, c])
    for g, w in zip(got, want):
        assert_matches(g, w, "int32 binary")


def test_where_and_clamp(rt, device):
    c = (torch.rand(4, 9) > 0.5).to(torch.float32)
    a, b_ = torch.randn(4, 9), torch.randn(4, 9)
    got, want = run_body(rt, device, lambda b, cc, x, y: (b.where(cc, x, y), b.clamp(x, -0.5, 0.25)), [c, a, b_])
    assert_matches(got[0], want[0], "where")
    assert_matches(got[1], want[1], "clamp")


def test_matmul_linear_vs_fixture(rt, device, golden):
    a, bm, bias, bt = golden["mm/a"], golden["mm/b"], golden["mm/bias"], golden["mm/bt"]
    got, _ = run_body(rt, device, lambda b, x, y, z, w: (b.matmul(x, y), b.linear(x, y, z), b.linear(x, w, z, transpose_b=True)),
                      [a, bm, bias, bt])
    assert_matches(got[0], golden["mm/matmul"], "matmul", F32)
    assert_matches(got[1], golden["mm/linear"], "linear", F32)
    assert_matches(got[2], golden["mm/linear_tb"], "linear transpose_b", F32)
    got, _ = run_body(rt, device, lambda b, x, y: b.matmul(x, y), [golden["mm/ab"], golden["mm/bb"]])
    assert_matches(got[0], golden["mm/batched"], "batched matmul", F32)


@pytest.mark.parametrize("m,n,k,ta,tb", [(1, 1, 1, False, False), (17, 5, 3, False, True), (64, 64, 16, True, False),
                                           (70, 130, 33, True, True), (3, 200, 129, False, False)])
def test_matmul_ragged_shapes(rt, device, m, n, k, ta, tb):
    a = torch.randn((k, m) if ta else (m, k))
    bm = torch.randn((n, k) if tb else (k, n))
    got, want = run_body(rt, device, lambda b, x, y: b.matmul(x, y, transpose_a=ta, transpose_b=tb), [a, bm])
    assert_matches(got[0], want[0], f"matmul {m}x{n}x{k}", (0.999, 1e-4, 1e-4))


def test_softmax(rt, device, golden):
    got, _ = run_body(rt, device, lambda b, x: (b.softmax(x, -1), b.softmax(x, 1)), [golden["softmax/x"]])
    assert_matches(got[0], golden["softmax/last"], "softmax last", F32)
    assert_matches(got[1], golden["softmax/mid"], "softmax mid", F32)


def test_reductions(rt, device, golden):
    x = golden["reduce/x"]
    got, _ = run_body(rt, device, lambda b, v: (b.reduce("Sum", v, [2], False), b.reduce("Mean", v, [1], True),
                                                 b.reduce("Max", v, [2], False), b.reduce("Min", v, [0], False),
                                                 b.reduce("Sum", v, None, False)), [x])
    assert_matches(got[0], golden["reduce/sum_last"], "sum", F32)
    assert_matches(got[1], golden["reduce/mean_mid_keep"], "mean", F32)
    assert_matches(got[2], golden["reduce/max_last"], "max", F32)
    assert_matches(got[3], golden["reduce/min_first"], "min", F32)
    assert_matches(got[4].reshape(1), golden["reduce/sum_all"], "sum all", (0.999, 1e-4, 1e-5))


def test_conv2d_vs_fixture(rt, device, golden):
    x, w, bias, w1 = golden["conv/x"], golden["conv/w"], golden["conv/b"], golden["conv/w1"]
    got, _ = run_body(rt, device, lambda b, xx, ww, bb, w1_: (
        b.conv2d(xx, ww, bb, 2, 9, 7, padding=(1, 1, 1, 1)),
        b.conv2d(xx, ww, bb, 2, 9, 7, stride=(2, 2), padding=(0, 1, 1, 2)),
        b.conv2d(xx, w1_, None, 2, 9, 7)), [x, w, bias, w1])
    assert_matches(got[0], golden["conv/same"], "conv same", F32)
    assert_matches(got[1], golden["conv/stride2_asym"], "conv stride 2", F32)
    assert_matches(got[2], golden["conv/pointwise"], "conv 1x1", F32)


def test_heads_and_typecast(rt, device, golden):
    got, _ = run_body(rt, device, lambda b, x: b.split_query_key_value_and_split_heads(x, None, 4, 2), [golden["heads/qkv"]])
    for g, n in zip(got, ["q", "k", "v"]):
        assert_matches(g, golden[f"heads/{n}"], n)
    got, _ = run_body(rt, device, lambda b, x: b.concatenate_heads(x), [golden["heads/q"]])
    assert_matches(got[0], golden["heads/merged"], "merged")
    got, _ = run_body(rt, device, lambda b, x: (b.typecast(x, "BFloat16"), b.typecast(x, "Int32")), [golden["cast/x"]])
    assert_matches(got[0], golden["cast/to_bf16"], "to bf16", (1.0, 0.0, 0.0))
    assert_matches(got[1], golden["cast/to_i32"], "to i32")


@pytest.mark.parametrize("tag,scale,zp", [("s002_z0", 0.02, 0), ("s0037_z3", 0.037, 3)])
@pytest.mark.parametrize("container", ["Int8", "Int32"])
def test_quantization_bit_exact(rt, device, golden, tag, scale, zp, container):
    x = golden["quant/x"]

    def body(b, v):
        q = b.quantize(v, scale, zp, out_dtype=container)
        rq = b.requantize(q, scale, zp, scale * 2, zp + 1, out_dtype=container)
        return q, b.dequantize(q, scale, zp), rq, b.dequantize(rq, scale * 2, zp + 1)
    got, want = run_body(rt, device, body, [x])
    dt = torch.int8 if container == "Int8" else torch.int32
    assert torch.equal(got[0], golden[f"quant/{tag}/q_i8"].to(dt))
    assert torch.equal(got[1], golden[f"quant/{tag}/deq"])
    assert torch.equal(got[2], golden[f"quant/{tag}/requant_i8"].to(dt))
    assert torch.equal(got[3], golden[f"quant/{tag}/requant_deq"])
    for g, w in zip(got, want):
        assert torch.equal(g, w)


def test_quantization_per_channel(rt, device, golden):
    x, s = golden["quant/x"], golden["quant/ch_scale"]

    def body(b, v, sc):
        q = b.quantize(v, sc, 0, out_dtype="Int8", axis=0)
        return q, b.dequantize(q, sc, 0, axis=0)
    got, _ = run_body(rt, device, body, [x, s])
    assert torch.equal(got[0], golden["quant/per_channel_q"])
    assert torch.equal(got[1], golden["quant/per_channel_deq"])


def test_rms_norm(rt, device, golden):
    got, _ = run_body(rt, device, lambda b, x, w: b.rms_norm(x, w), [golden["rms/x"], golden["rms/w"]])
    assert_matches(got[0], golden["rms/out"], "rms_norm")
    for cols in [48, 4096, 8192, 10000]:
        x = torch.randn(7, cols).to(torch.bfloat16)
        w = (1 + 0.1 * torch.randn(cols)).to(torch.bfloat16)
        got, want = run_body(rt, device, lambda b, xx, ww: b.rms_norm(xx, ww), [x, w])
        assert_matches(got[0], want[0], f"rms_norm cols={cols}")


def test_sdpa_small_vs_fixture(rt, device, golden):
    q, k, v = golden["sdpa/q"], golden["sdpa/k"], golden["sdpa/v"]
    got, _ = run_body(rt, device, lambda b, a, c, d: (b.scaled_dot_product_attention(a, c, d, True),
                                                      b.scaled_dot_product_attention(a, c, d, False)), [q, k, v])
    assert_matches(got[0], golden["sdpa/causal"], "sdpa causal", F32)
    assert_matches(got[1], golden["sdpa/full"], "sdpa full", F32)


@pytest.mark.parametrize("seq,causal", [(64, True), (200, True), (256, False), (77, False)])
def test_sdpa_flash_kernel(rt, device, seq, causal):
    torch.manual_seed(seq)
    q = torch.randn(2, 4, seq, 128).to(torch.bfloat16)
    k = torch.randn(2, 2, seq, 128).to(torch.bfloat16)
    v = torch.randn(2, 2, seq, 128).to(torch.bfloat16)
    got, want = run_body(rt, device, lambda b, a, c, d: b.scaled_dot_product_attention(a, c, d, causal), [q, k, v])
    assert_matches(got[0], want[0], f"flash seq={seq} causal={causal}")


def test_sdpa_with_mask(rt, device):
    q, k, v = torch.randn(1, 2, 9, 32), torch.randn(1, 2, 12, 32), torch.randn(1, 2, 12, 32)
    mask = torch.where(torch.rand(1, 1, 9, 12) > 0.3, 0.0, -1e9)
    got, want = run_body(rt, device, lambda b, a, c, d, m: b.scaled_dot_product_attention(a, c, d, False, mask=m), [q, k, v, mask])
    assert_matches(got[0], want[0], "sdpa mask", F32)


def test_rotary_embedding(rt, device):
    from ttmlir_b200.graphs import rope_tables
    cos, sin = rope_tables(40, 64)
    x = torch.randn(2, 3, 40, 64).to(torch.bfloat16)
    got, want = run_body(rt, device, lambda b, xx, c, s: b.rotary_embedding(xx, c, s), [x, cos, sin])
    assert_matches(got[0], want[0], "rope")


def test_rotary_embedding_matches_the_golden_of_the_fusing_test(rt, device, golden):
    """The fixture is what torch_rope of test/python/golden/ttir_ops/fusing/test_rope_fusing.py returns (f32 evaluation
    of bf16 operands, one rounding), cos / sin broadcast over batch and heads."""
    bf = torch.bfloat16
    x, cos, sin = golden["rope/x"].to(bf), golden["rope/cos"].to(bf).reshape(1, 1, 24, 64), golden["rope/sin"].to(bf).reshape(1, 1, 24, 64)
    got, want = run_body(rt, device, lambda b, xx, c, s: b.rotary_embedding(xx, c, s), [x, cos, sin])
    assert_matches(got[0], golden["rope/bf16_operands"], "rope against the reference's golden")
    assert torch.equal(want[0], golden["rope/bf16_operands"])


def test_data_movement(rt, device):
    x = torch.randn(3, 4, 5, 6)

    def body(b, v):
        return (b.permute(v, [0, 2, 1, 3]), b.transpose(v, -1, -2), b.slice(v, [0, 1, 0, 2], [3, 4, 5, 6], [1, 2, 1, 1]),
                b.concat([v, v], 2), b.repeat(v, [1, 2, 1, 2]), b.repeat_interleave(v, 3, 1), b.reshape(v, [12, 30]))
    got, want = run_body(rt, device, body, [x])
    for i, (g, w) in enumerate(zip(got, want)):
        assert_matches(g, w, f"movement {i}", (1.0, 0.0, 0.0))
    xb = torch.randn(2, 64, 8, 128).to(torch.bfloat16)  # the head split of the decoder block
    got, want = run_body(rt, device, lambda b, v: b.permute(v, [0, 2, 1, 3]), [xb])
    assert torch.equal(got[0], want[0])


def test_creation_ops(rt, device):
    data = torch.arange(12, dtype=torch.float32).reshape(3, 4)

    def body(b, v):
        c = b.constant(data.numpy().tobytes(), [3, 4], "Float32")
        return (b.add(v, b.full([3, 4], 2.5, "Float32")), b.add(v, b.ones([3, 4], "Float32")), b.add(v, b.zeros([3, 4], "Float32")),
                b.add(v, c), b.arange(0, 10, 2, "Float32"))
    got, want = run_body(rt, device, body, [torch.randn(3, 4)])
    for i, (g, w) in enumerate(zip(got, want)):
        assert_matches(g, w, f"creation {i}", F32)


def test_empty_tensor(rt, device):
    x = torch.zeros(0, 16)
    got, want = run_body(rt, device, lambda b, v: b.relu(v), [x])
    assert list(got[0].shape) == [0, 16]


@pytest.mark.parametrize("c,o,k,stride,pad,dil", [
    (64, 64, 3, (1, 1), (1, 1, 1, 1), (1, 1)),
    (64, 40, 3, (2, 2), (0, 1, 1, 2), (1, 1)),
    (128, 256, 3, (1, 1), (2, 2, 2, 2), (2, 2)),
    (64, 72, 5, (1, 2), (2, 2, 2, 2), (1, 1)),
    (192, 64, 1, (2, 2), (0, 0, 0, 0), (1, 1)),
])
def test_conv2d_implicit_gemm(rt, device, c, o, k, stride, pad, dil):
    """Channel counts that are multiples of 64 take the tensor-core kernel's gathering producer
    (no im2col operand in memory): strides, asymmetric padding, dilation, several k-blocks per
    tap, ragged pixel and channel tails, with the relu and residual-add epilogues."""
    torch.manual_seed(c + o + k)
    n, h, w = 3, 13, 11
    x = torch.randn(n, h, w, c).to(torch.bfloat16)
    wt = (torch.randn(o, c, k, k) * (2.0 / (c * k * k)) ** 0.5).to(torch.bfloat16)
    bias = torch.randn(1, 1, 1, o).to(torch.bfloat16)
    ho = (h + pad[0] + pad[2] - dil[0] * (k - 1) - 1) // stride[0] + 1
    wo = (w + pad[1] + pad[3] - dil[1] * (k - 1) - 1) // stride[1] + 1
    res = torch.randn(n, ho, wo, o).to(torch.bfloat16)

    def body(b, xx, ww, bb, rr):
        plain = b.conv2d(xx, ww, bb, n, h, w, stride=stride, padding=pad, dilation=dil)
        act = b.relu(b.conv2d(xx, ww, bb, n, h, w, stride=stride, padding=pad, dilation=dil))
        fused = b.relu(b.add(b.conv2d(xx, ww, None, n, h, w, stride=stride, padding=pad, dilation=dil), rr))
        return plain, act, fused
    got, want = run_body(rt, device, body, [x, wt, bias, res])
    for g, wnt, name in zip(got, want, ["plain", "relu", "add+relu"]):
        assert_matches(g, wnt, f"conv {c}->{o} k{k} {name}")
