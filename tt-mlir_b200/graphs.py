"""The benchmark graphs, written once against the builder interface, plus their seeded inputs.

Each `*_graph(b, ...)` function only calls methods of a builder `b`; handed a
`ttnn_builder.ProgramBuilder` it emits the TTNN program, handed the CPU oracle's builder it
computes the expected result.  Shapes default to the full benchmark configurations; tests pass
smaller ones.  Inputs are synthetic (seeded torch CPU generator) with the distributions each
configuration states.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence, Tuple

import torch


# ---------------------------------------------------------------- config 1: f32 MLP
def mlp_body(b, x, w1, b1, w2, b2):
    h = b.relu(b.add(b.matmul(x, w1, loc="fc1"), b1, loc="fc1_bias"), loc="relu")
    y = b.add(b.matmul(h, w2, loc="fc2"), b2, loc="fc2_bias")
    return b.softmax(y, dim=-1, loc="softmax")


def mlp_graph(b, batch=128, d_in=784, d_hidden=256, d_out=10, dtype="Float32"):
    x = b.input([batch, d_in], dtype)
    w1 = b.input([d_in, d_hidden], dtype)
    b1 = b.input([d_hidden], dtype)
    w2 = b.input([d_hidden, d_out], dtype)
    b2 = b.input([d_out], dtype)
    b.output(mlp_body(b, x, w1, b1, w2, b2))


def mlp_traced_binary(batch=128, d_in=784, d_hidden=256, d_out=10, dtype="Float32") -> bytes:
    """The MLP as the compiler emits it with `enable-trace=true`: program 0 takes the same five
    inputs as `mlp_graph` (the activation on host, the parameters on device) and holds one
    CaptureOrExecuteTraceOp; the ops live in a private traced function (see
    ttnn_builder.BinaryBuilder.hoist_trace)."""
    from .ttnn_builder import BinaryBuilder
    bb = BinaryBuilder()
    main = bb.program("mlp")
    x = main.input([batch, d_in], dtype, on_device=False)
    w1 = main.input([d_in, d_hidden], dtype)
    b1 = main.input([d_hidden], dtype)
    w2 = main.input([d_hidden, d_out], dtype)
    b2 = main.input([d_out], dtype)
    outs = bb.hoist_trace(main, "mlp", [w1, b1, w2, b2, x],
                          lambda p, a: [mlp_body(p, a[4], a[0], a[1], a[2], a[3])])
    main.output(*outs)
    return bb.finish()


def mlp_inputs(batch=128, d_in=784, d_hidden=256, d_out=10, seed=0, dtype=torch.float32):
    g = torch.Generator().manual_seed(seed)
    x = torch.rand(batch, d_in, generator=g) * 2 - 1
    w1 = torch.randn(d_in, d_hidden, generator=g) / math.sqrt(d_in)
    w2 = torch.randn(d_hidden, d_out, generator=g) / math.sqrt(d_hidden)
    return [t.to(dtype) for t in (x, w1, torch.zeros(d_hidden), w2, torch.zeros(d_out))]


# ---------------------------------------------------------------- config 2: quantization chain
def quant_chain_graph(b, rows=4096, cols=4096, scale1=0.02, scale2=0.04, zp1=0, zp2=0, container="Int32",
                      keep_intermediates=False, out_dtype="Float32"):
    x = b.input([rows, cols], "BFloat16")
    q1 = b.quantize(x, scale1, zp1, out_dtype=container, loc="quantize")
    q2 = b.requantize(q1, scale1, zp1, scale2, zp2, out_dtype=container, loc="requantize")
    y = b.dequantize(q2, scale2, zp2, out_dtype=out_dtype, loc="dequantize")
    if keep_intermediates:
        b.output(y, q1, q2)
    else:
        b.output(y)


def quant_chain_inputs(rows=4096, cols=4096, seed=1):
    g = torch.Generator().manual_seed(seed)
    return [torch.randn(rows, cols, generator=g).to(torch.bfloat16)]


# ---------------------------------------------------------------- config 3: int8-weight linear
def w8_linear_graph(b, m=2048, k=4096, n=11008):
    a = b.input([m, k], "BFloat16")
    wq = b.input([n, k], "Int8")
    scales = b.input([n], "Float32")
    bias = b.input([n], "BFloat16")
    w = b.dequantize(wq, scales, 0, out_dtype="BFloat16", axis=0, loc="dequant_weight")
    b.output(b.linear(a, w, bias, transpose_b=True, loc="linear"))


def w8_linear_const_eval_binary(m=2048, k=4096, n=11008) -> bytes:
    """Config 3 as the compiler emits it with `enable-const-eval=true`: the weight's dequantization
    depends on parameters only, so it is hoisted into a private const-eval function that program 0
    reaches through a LoadCachedOp; the runtime evaluates it on the first submit and caches the
    bf16 weight.  Same inputs, same results as `w8_linear_graph`."""
    from .ttnn_builder import BinaryBuilder
    bb = BinaryBuilder()
    main = bb.program("w8_linear")
    a = main.input([m, k], "BFloat16")
    wq = main.input([n, k], "Int8")
    scales = main.input([n], "Float32")
    bias = main.input([n], "BFloat16")
    ce = bb.private_program("w8_linear_const_eval_0")
    c_wq = ce.input([n, k], "Int8")
    c_scales = ce.input([n], "Float32")
    ce.output(ce.dequantize(c_wq, c_scales, 0, out_dtype="BFloat16", axis=0, loc="dequant_weight"))
    (w,) = main.load_cached(ce, [wq, scales])
    main.output(main.linear(a, w, bias, transpose_b=True, loc="linear"))
    return bb.finish()


def w8_linear_inputs(m=2048, k=4096, n=11008, seed=2):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(m, k, generator=g).to(torch.bfloat16)
    wf = torch.randn(n, k, generator=g) * 0.02
    s = wf.abs().amax(dim=1) / 127.0
    wq = torch.clamp(torch.round(wf / s[:, None]), -127, 127).to(torch.int8)
    bias = (torch.randn(n, generator=g) * 0.01).to(torch.bfloat16)
    return [a, wq, s.to(torch.float32), bias]


def w8a8_linear_graph(b, m=2048, k=4096, n=11008, act_scale=0.04, fused_dequant=True):
    """Config 3's shapes with BOTH operands quantized: activations per tensor (scale `act_scale`), weights
    per output channel.  The contraction runs on the 8-bit values with an Int32 accumulator and the
    dequantize after it carries the product of the scales per output channel -- the form the compiler
    produces when it commutes dequantize below a quantizable op (QuantDequantConversion.cpp).  Inputs:
    activations bf16 [m, k], weights Int8 [n, k], combined scales f32 [n] (= act_scale * weight scale),
    bias bf16 [n]."""
    a = b.input([m, k], "BFloat16")
    wq = b.input([n, k], "Int8")
    scales = b.input([n], "Float32")
    bias = b.input([n], "BFloat16")
    aq = b.quantize(a, act_scale, 0, out_dtype="Int8", loc="quantize_activation")
    acc = b.matmul(aq, wq, transpose_b=True, out_dtype="Int32", loc="int_matmul")
    y = b.dequantize(acc, scales, 0, out_dtype="BFloat16", axis=1, loc="dequantize_result")
    b.output(b.add(y, bias, loc="bias"))


def w8a8_linear_inputs(m=2048, k=4096, n=11008, seed=2, act_scale=0.04):
    a, wq, s, bias = w8_linear_inputs(m, k, n, seed)
    return [a, wq, (s * act_scale).to(torch.float32), bias]


def quantized_conv_graph(b, batch=8, hw=28, c_in=64, c_out=128, kernel=3, x_scale=0.05, container="Int8"):
    """A convolution on quantized operands: input quantized per tensor, weight Int8 per output channel,
    Int32 accumulator, dequantize with the per-channel product of the scales."""
    x = b.input([1, 1, batch * hw * hw, c_in], "BFloat16")
    wq = b.input([c_out, c_in, kernel, kernel], container)
    scales = b.input([c_out], "Float32")
    xq = b.quantize(x, x_scale, 0, out_dtype=container, loc="quantize_input")
    pad = kernel // 2
    acc = b.conv2d(xq, wq, None, batch, hw, hw, padding=(pad, pad, pad, pad), out_dtype="Int32", loc="int_conv")
    b.output(b.dequantize(acc, scales, 0, out_dtype="Float32", axis=3, loc="dequantize_result"))


def quantized_conv_inputs(batch=8, hw=28, c_in=64, c_out=128, kernel=3, seed=7, x_scale=0.05, container=torch.int8):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(1, 1, batch * hw * hw, c_in, generator=g).to(torch.bfloat16)
    wf = torch.randn(c_out, c_in, kernel, kernel, generator=g) * (2.0 / (c_in * kernel * kernel)) ** 0.5
    s = wf.abs().amax(dim=(1, 2, 3)) / 127.0
    wq = torch.clamp(torch.round(wf / s[:, None, None, None]), -127, 127).to(container)
    return [x, wq, (s * x_scale).to(torch.float32)]


# ---------------------------------------------------------------- config 4: Llama-style decoder block
def rope_tables(seq, head_dim, theta=500000.0, dtype=torch.bfloat16):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    ang = torch.outer(torch.arange(seq, dtype=torch.float32), inv)
    emb = torch.cat((ang, ang), dim=-1)
    return emb.cos().to(dtype).reshape(1, 1, seq, head_dim), emb.sin().to(dtype).reshape(1, 1, seq, head_dim)


DECODER_WEIGHTS = ["attn_norm", "wq", "wk", "wv", "wo", "ffn_norm", "w_gate", "w_up", "w_down"]


def decoder_shapes(seq=2048, hidden=4096, n_heads=32, n_kv_heads=8, head_dim=128, ffn=14336, batch=1):
    """Full (unsharded) shapes of the block's inputs, and the dim each is sharded on under
    1xN tensor parallelism (None = replicated): column-parallel q/k/v/gate/up, row-parallel o/down."""
    return {
        "x": ([batch, seq, hidden], None),
        "attn_norm": ([hidden], None),
        "wq": ([n_heads * head_dim, hidden], 0),
        "wk": ([n_kv_heads * head_dim, hidden], 0),
        "wv": ([n_kv_heads * head_dim, hidden], 0),
        "wo": ([hidden, n_heads * head_dim], 1),
        "ffn_norm": ([hidden], None),
        "w_gate": ([ffn, hidden], 0),
        "w_up": ([ffn, hidden], 0),
        "w_down": ([hidden, ffn], 1),
        "cos": ([1, 1, seq, head_dim], None),
        "sin": ([1, 1, seq, head_dim], None),
    }


DECODER_ORDER = ["x", "attn_norm", "wq", "wk", "wv", "wo", "ffn_norm", "w_gate", "w_up", "w_down", "cos", "sin"]


def decoder_block_graph(b, seq=2048, hidden=4096, n_heads=32, n_kv_heads=8, head_dim=128, ffn=14336, batch=1,
                        tp=1, eps=1e-5, presharded=False, dtype="BFloat16", io_seq_sharded=False):
    """RMSNorm -> q/k/v -> RoPE -> causal GQA attention -> o_proj (+all_reduce) -> residual ->
    RMSNorm -> SwiGLU FFN (+all_reduce) -> residual.  `tp` is the 1xN mesh width.  With
    `presharded` the program's inputs are already per-device device tensors (what a frontend
    that shards its own arguments hands over) and the output stays on the mesh.  With
    `io_seq_sharded` (presharded, tp > 1) every device receives and returns only its 1/tp of the
    sequence: the block starts with an all_gather of the activations over NVLink and ends with a
    mesh_partition, so host traffic per step is one copy of the activations in each direction in
    total instead of one per device."""
    io_seq_sharded = bool(io_seq_sharded and presharded and tp > 1)
    if io_seq_sharded:
        assert seq % tp == 0, "sequence length must divide by the mesh width"
    shapes = decoder_shapes(seq, hidden, n_heads, n_kv_heads, head_dim, ffn, batch)
    v = {}
    for name in DECODER_ORDER:
        shape, sdim = shapes[name]
        if tp == 1:
            v[name] = b.input(shape, dtype)
        elif presharded:
            local = list(shape)
            if sdim is not None:
                local[sdim] //= tp
            if name == "x" and io_seq_sharded:
                local[1] //= tp
            v[name] = b.input(local, dtype)
        else:
            full = b.input(shape, dtype, on_device=False)
            v[name] = b.distribute(full, sdim, loc=f"shard_{name}")
    hq, hkv = n_heads // tp, n_kv_heads // tp
    x = v["x"]
    if io_seq_sharded:
        x = b.all_gather(x, 1, loc="gather_sequence")
    h = b.rms_norm(x, v["attn_norm"], epsilon=eps, loc="attn_norm")
    q = b.linear(h, v["wq"], transpose_b=True, loc="q_proj")
    k = b.linear(h, v["wk"], transpose_b=True, loc="k_proj")
    val = b.linear(h, v["wv"], transpose_b=True, loc="v_proj")
    q = b.permute(b.reshape(q, [batch, seq, hq, head_dim]), [0, 2, 1, 3], loc="q_heads")
    k = b.permute(b.reshape(k, [batch, seq, hkv, head_dim]), [0, 2, 1, 3], loc="k_heads")
    val = b.permute(b.reshape(val, [batch, seq, hkv, head_dim]), [0, 2, 1, 3], loc="v_heads")
    q = b.rotary_embedding(q, v["cos"], v["sin"], loc="q_rope")
    k = b.rotary_embedding(k, v["cos"], v["sin"], loc="k_rope")
    a = b.scaled_dot_product_attention(q, k, val, is_causal=True, loc="attention")
    a = b.concatenate_heads(a, loc="merge_heads")
    o = b.linear(a, v["wo"], transpose_b=True, loc="o_proj")
    if tp > 1:
        o = b.all_reduce(o, loc="o_proj_all_reduce")
    x1 = b.add(x, o, loc="attn_residual")
    h2 = b.rms_norm(x1, v["ffn_norm"], epsilon=eps, loc="ffn_norm")
    g = b.linear(h2, v["w_gate"], transpose_b=True, loc="gate_proj")
    u = b.linear(h2, v["w_up"], transpose_b=True, loc="up_proj")
    act = b.multiply(b.silu(g, loc="silu"), u, loc="swiglu")
    d = b.linear(act, v["w_down"], transpose_b=True, loc="down_proj")
    if tp > 1:
        d = b.all_reduce(d, loc="down_proj_all_reduce")
    out = b.add(x1, d, loc="ffn_residual")
    if tp > 1 and not presharded:
        out = b.aggregate(out, None, loc="gather_output")
    if io_seq_sharded:
        out = b.mesh_partition(out, 1, loc="own_rows")
    b.output(out)


def decoder_block_inputs(seq=2048, hidden=4096, n_heads=32, n_kv_heads=8, head_dim=128, ffn=14336, batch=1, seed=3,
                         dtype=torch.bfloat16) -> List[torch.Tensor]:
    g = torch.Generator().manual_seed(seed)
    shapes = decoder_shapes(seq, hidden, n_heads, n_kv_heads, head_dim, ffn, batch)
    cos, sin = rope_tables(seq, head_dim, dtype=dtype)
    out = []
    for name in DECODER_ORDER:
        shape, _ = shapes[name]
        if name == "cos":
            out.append(cos)
        elif name == "sin":
            out.append(sin)
        elif name in ("attn_norm", "ffn_norm"):
            out.append((1.0 + torch.randn(shape, generator=g) * 0.02).to(dtype))
        elif name == "x":
            # activations of order one, as a block in the middle of a network sees them
            out.append(torch.randn(shape, generator=g).to(dtype))
        else:
            out.append((torch.randn(shape, generator=g) * 0.02).to(dtype))
    return out


def shard_inputs(inputs: Sequence[torch.Tensor], shard_dims: Sequence[Optional[int]], tp: int, rank: int):
    """The slice of every input that mesh coordinate `rank` owns."""
    out = []
    for t, d in zip(inputs, shard_dims):
        out.append(t if d is None else torch.chunk(t, tp, dim=d)[rank].contiguous())
    return out


def decoder_shard_dims(io_seq_sharded=False, **kw) -> List[Optional[int]]:
    shapes = decoder_shapes(**kw)
    dims = [shapes[n][1] for n in DECODER_ORDER]
    if io_seq_sharded:
        dims[DECODER_ORDER.index("x")] = 1  # the activations arrive split along the sequence
    return dims


def decoder_block_flops(seq=2048, hidden=4096, n_heads=32, n_kv_heads=8, head_dim=128, ffn=14336, batch=1,
                        causal_discount=False) -> float:
    t = batch * seq
    proj = 2 * t * hidden * (n_heads * head_dim) * 2 + 2 * t * hidden * (n_kv_heads * head_dim) * 2
    attn = 2 * 2 * batch * n_heads * seq * seq * head_dim
    if causal_discount:
        attn /= 2
    mlp = 3 * 2 * t * hidden * ffn
    return float(proj + attn + mlp)


# ---------------------------------------------------------------- config 5: ResNet bottleneck
def bottleneck_graph(b, batch=64, hw=56, c_in=64, c_mid=64, c_out=256, dp=1, presharded=False, dtype="BFloat16"):
    """1x1 -> relu -> 3x3 (pad 1) -> relu -> 1x1, plus a 1x1 projection of the input as the
    residual, then relu.  Activations are NHWC flattened to [1, 1, N*H*W, C] as the compiler
    emits them (lib/Dialect/TTIR/Transforms/FlattenSlidingWindow.cpp).  `dp` shards the batch
    over a 1xN mesh and gathers the result."""
    nb = batch // dp
    full_shape = [1, 1, batch * hw * hw, c_in]
    wshapes = [[c_mid, c_in, 1, 1], [1, 1, 1, c_mid], [c_mid, c_mid, 3, 3], [1, 1, 1, c_mid], [c_out, c_mid, 1, 1],
               [1, 1, 1, c_out], [c_out, c_in, 1, 1], [1, 1, 1, c_out]]
    if dp == 1:
        x = b.input(full_shape, dtype)
        ws = [b.input(s, dtype) for s in wshapes]
    elif presharded:
        x = b.input([1, 1, nb * hw * hw, c_in], dtype)
        ws = [b.input(s, dtype) for s in wshapes]
    else:
        x = b.distribute(b.input(full_shape, dtype, on_device=False), 2, loc="shard_batch")
        ws = [b.distribute(b.input(s, dtype, on_device=False), None, loc=f"replicate_w{i}") for i, s in enumerate(wshapes)]
    w1, b1, w2, b2, w3, b3, wp, bp = ws
    y = b.relu(b.conv2d(x, w1, b1, nb, hw, hw, loc="conv1"), loc="relu1")
    y = b.relu(b.conv2d(y, w2, b2, nb, hw, hw, padding=(1, 1, 1, 1), loc="conv2"), loc="relu2")
    y = b.conv2d(y, w3, b3, nb, hw, hw, loc="conv3")
    r = b.conv2d(x, wp, bp, nb, hw, hw, loc="proj")
    y = b.relu(b.add(y, r, loc="residual"), loc="relu3")
    if dp > 1:
        y = b.all_gather(y, 2, loc="gather_batch")
        if not presharded:
            y = b.aggregate(y, None, loc="to_host")
    b.output(y)


def bottleneck_inputs(batch=64, hw=56, c_in=64, c_mid=64, c_out=256, seed=4, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)

    def kaiming(o, c, kh, kw):
        return (torch.randn(o, c, kh, kw, generator=g) * math.sqrt(2.0 / (c * kh * kw))).to(dtype)

    def bias(o):
        return (torch.randn(1, 1, 1, o, generator=g) * 0.05).to(dtype)  # folded batch-norm shift
    x = torch.randn(batch, hw, hw, c_in, generator=g).to(dtype).reshape(1, 1, batch * hw * hw, c_in)
    return [x, kaiming(c_mid, c_in, 1, 1), bias(c_mid), kaiming(c_mid, c_mid, 3, 3), bias(c_mid),
            kaiming(c_out, c_mid, 1, 1), bias(c_out), kaiming(c_out, c_in, 1, 1), bias(c_out)]


BOTTLENECK_SHARD_DIMS = [2, None, None, None, None, None, None, None, None]


# ---------------------------------------------------------------- helpers
# ---------------------------------------------------------------- serving: one decode step's attention
def decode_attention_graph(b, batch=32, heads=32, kv_heads=8, seq=8192, head_dim=128, dtype="BFloat16"):
    """A decode step's attention for `batch` users: the new key / value rows are written into the
    caches at `index`, then every user's single query attends to its cache up to its position."""
    q = b.input([1, batch, heads, head_dim], dtype)
    k_cache = b.input([batch, kv_heads, seq, head_dim], dtype)
    v_cache = b.input([batch, kv_heads, seq, head_dim], dtype)
    k_new = b.input([1, kv_heads, batch, head_dim], dtype)
    v_new = b.input([1, kv_heads, batch, head_dim], dtype)
    index = b.input([1], "Int32")
    pos = b.input([batch], "Int32")
    k_cache = b.update_cache(k_cache, k_new, index, loc="update_k")
    v_cache = b.update_cache(v_cache, v_new, index, loc="update_v")
    b.output(b.scaled_dot_product_attention_decode(q, k_cache, v_cache, pos, None, True, 1.0 / math.sqrt(head_dim),
                                                   loc="decode_attention"))


def decode_attention_inputs(batch=32, heads=32, kv_heads=8, seq=8192, head_dim=128, seed=6, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    mk = lambda *s: torch.randn(*s, generator=g).to(dtype)
    at = seq - 1
    return [mk(1, batch, heads, head_dim), mk(batch, kv_heads, seq, head_dim), mk(batch, kv_heads, seq, head_dim),
            mk(1, kv_heads, batch, head_dim), mk(1, kv_heads, batch, head_dim), torch.tensor([at], dtype=torch.int32),
            torch.full((batch,), at, dtype=torch.int32)]


class _TracedBody:
    """Stands between a `*_graph(b, ...)` function and the program that holds the traced function:
    `input()` hands out the traced function's arguments in order, `output()` collects the results,
    every op goes to the program."""

    def __init__(self, program, args):
        self._p, self._args, self.results = program, list(args), []

    def input(self, shape, dtype, on_device=True):
        v = self._args.pop(0)
        assert list(v.shape) == list(shape) and v.dtype == dtype, "traced body and main program disagree on an input"
        return v

    def output(self, *values):
        self.results.extend(values)

    def __getattr__(self, name):
        return getattr(self._p, name)


def traced_binary(graph_fn, host_inputs=(0,), name="main", **kw) -> bytes:
    """`graph_fn` the way the compiler emits it with `enable-trace=true` on one device: program 0 has
    the graph's inputs (those listed in `host_inputs` on host, the rest on device, i.e. parameters)
    and one CaptureOrExecuteTraceOp; the ops live in a private traced function
    (ttnn_builder.BinaryBuilder.hoist_trace)."""
    from .ttnn_builder import BinaryBuilder
    # a first pass over the graph only to learn its inputs
    probe = BinaryBuilder().program("probe")
    graph_fn(probe, **kw)
    bb = BinaryBuilder()
    main = bb.program(name)
    ins = [main.input(v.shape, v.dtype, on_device=(i not in host_inputs)) for i, v in enumerate(probe.inputs)]
    order = sorted(range(len(ins)), key=lambda i: 0 if ins[i].on_device else 1)   # hoist_trace's argument order

    def body(p, args):
        by_index = {i: a for i, a in zip(order, args)}
        tb = _TracedBody(p, [by_index[i] for i in range(len(ins))])
        graph_fn(tb, **kw)
        return tb.results
    main.output(*bb.hoist_trace(main, name, [ins[i] for i in order], body))
    return bb.finish()


def decoder_block_traced_binary(**kw) -> bytes:
    """The single-device decoder block as a trace: activations staged from host, weights and rotary tables resident."""
    return traced_binary(decoder_block_graph, host_inputs=(0,), name="decoder_block", **kw)


def build_binary(graph_fn, mesh_shape=(1, 1), name="main", goldens=None, system_desc=None, **kw) -> bytes:
    """Emits a one-program .ttnn binary for `graph_fn(b, **kw)`.  `goldens` ({key: torch tensor}) are embedded
    in the program's debug info; `system_desc` (the "system_desc" dictionary of a descriptor's JSON view)
    becomes the binary's record of the system it was compiled for."""
    from .ttnn_builder import BinaryBuilder
    bb = BinaryBuilder(system_desc=system_desc)
    p = bb.program(name, mesh_shape)
    graph_fn(p, **kw)
    for key, t in (goldens or {}).items():
        p.golden(key, t)
    return bb.finish()
