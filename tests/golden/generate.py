"""Generates tests/golden/ttir_cpu_golden.npz by running the reference's own CPU code.

Run where a checkout of tenstorrent/tt-mlir is available (path as the argument, or in the
TT_MLIR_ROOT environment variable):

    python tests/golden/generate.py /path/to/tt-mlir

It imports tools/tt-alchemist/templates/python/local/ttir_cpu.py -- the pure-torch CPU
implementation of the TTIR ops that the reference's CPU-hoist path targets -- and records its
outputs on small seeded inputs.  For ops the reference defines only through a torch golden in
tools/golden/mapping.py (that file needs the compiler's Python bindings and cannot be
imported), the golden's body is the single torch call cited beside each entry below, and that
call is recorded.  The fixture travels with the repo; the reference tree does not.
bf16 tensors are stored as their uint16 bit patterns.
"""

import importlib.util
import os
import sys

import numpy as np
import torch


def load_ttir_cpu(root):
    path = os.path.join(root, "tools/tt-alchemist/templates/python/local/ttir_cpu.py")
    spec = importlib.util.spec_from_file_location("ttir_cpu_reference", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


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

    # --- quantization goldens: torch.quantize_per_tensor(...).int_repr(), torch.dequantize,
    #     requantize = quantize(dequantize(q))  (tools/golden/mapping.py:2534-2582)
    qx = (torch.randn(64, 48, generator=g)).to(torch.bfloat16)
    ties = torch.tensor([0.25, 0.75, 1.25, 3.0, -3.0, 0.01, -0.01, 0.03, -0.05, 2.55, -2.57, 100.0], dtype=torch.bfloat16)
    qx.view(-1)[: ties.numel()] = ties
    store(out, "quant/x", qx)
    for tag, scale, zp in [("s002_z0", 0.02, 0), ("s0037_z3", 0.037, 3)]:
        q8 = torch.quantize_per_tensor(qx.float(), scale, zp, torch.qint8)
        store(out, f"quant/{tag}/q_i8", q8.int_repr())
        q32 = torch.quantize_per_tensor(qx.float(), scale, zp, torch.qint32)
        store(out, f"quant/{tag}/q_i32", q32.int_repr())
        store(out, f"quant/{tag}/deq", torch.dequantize(q8))
        rq = torch.quantize_per_tensor(torch.dequantize(q8), scale * 2, zp + 1, torch.qint8)
        store(out, f"quant/{tag}/requant_i8", rq.int_repr())
        store(out, f"quant/{tag}/requant_deq", torch.dequantize(rq))
    ch_scale = torch.rand(64, generator=g) * 0.05 + 0.01
    store(out, "quant/ch_scale", ch_scale)
    qc = torch.quantize_per_channel(qx.float(), ch_scale.double(), torch.zeros(64, dtype=torch.int64), 0, torch.qint8)
    store(out, "quant/per_channel_q", qc.int_repr())
    store(out, "quant/per_channel_deq", torch.dequantize(qc))

    # --- rms_norm golden: torch.nn.functional.rms_norm on float input (mapping.py:1221-1290)
    nx = rnd(5, 64).to(torch.bfloat16)
    nw = (1 + rnd(64) * 0.1).to(torch.bfloat16)
    store(out, "rms/x", nx)
    store(out, "rms/w", nw)
    store(out, "rms/out", torch.nn.functional.rms_norm(nx.float(), (64,), weight=nw, eps=1e-5).to(torch.bfloat16))

    # --- scaled dot product attention golden body (mapping.py:8398-8500): GQA repeat, scale,
    #     causal -inf mask above the diagonal, f32 softmax, f32 P.V, cast
    aq, ak, av = rnd(1, 4, 10, 16), rnd(1, 2, 10, 16), rnd(1, 2, 10, 16)
    store(out, "sdpa/q", aq)
    store(out, "sdpa/k", ak)
    store(out, "sdpa/v", av)
    kk = torch.repeat_interleave(ak, 2, dim=1)
    vv = torch.repeat_interleave(av, 2, dim=1)
    qk = torch.matmul(aq, kk.transpose(-2, -1)) * (1.0 / 16 ** 0.5)
    causal = qk + torch.triu(torch.full((10, 10), float("-inf")), diagonal=1)
    store(out, "sdpa/causal", torch.matmul(torch.softmax(causal, dim=-1), vv))
    store(out, "sdpa/full", torch.matmul(torch.softmax(qk, dim=-1), vv))

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

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "ttir_cpu_golden.npz")
    np.savez_compressed(path, **out)
    print(f"wrote {path}: {len(out)} arrays, {os.path.getsize(path)} bytes")


if __name__ == "__main__":
    main()
