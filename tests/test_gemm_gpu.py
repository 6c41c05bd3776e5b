"""The tcgen05 tensor-core GEMM against the CUDA-core GEMM and an f32 reference, through the
kernel-level C ABI (ttb_gemm picks the tensor-core kernel, ttb_gemm_simt forces the other)."""

import ctypes

import pytest
import torch

from helpers import KernelHarness, assert_matches

pytestmark = pytest.mark.gpu

BF16, F32 = 2, 0
ACT = {None: 0, "relu": 1, "silu": 2}


def run_gemm(h, fn, a, b, bias, m, n, k, act=0, round_steps=0, out_dtype=torch.bfloat16):
    da, db = h.upload(a), h.upload(b)
    dbias = h.upload(bias) if bias is not None else None
    dc = h.empty((m, n), out_dtype)
    i64 = ctypes.c_int64
    rc = fn(da, db, dbias, dc, BF16, BF16, BF16 if out_dtype == torch.bfloat16 else F32, i64(1), i64(m), i64(n), i64(k),
            0, 1, i64(0), i64(0), act, round_steps, h.stream)
    if rc != 0:
        raise RuntimeError(h.lib.ttb_last_error().decode())
    return h.download(dc, (m, n), out_dtype)


def tc_status(h):
    st = ctypes.c_int(-1)
    assert h.lib.ttb_gemm_tcgen05_status(ctypes.byref(st)) == 0
    return st.value


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (128, 64, 128), (128, 128, 256), (256, 512, 1024),
                                   (200, 136, 72), (1000, 1000, 520), (77, 264, 4096), (4096, 64, 576),
                                   (2048, 4096, 4096),
                                   # CTA pairs (256 rows and more, K of 512 and more) with ragged edges: a second CTA
                                   # with one valid row, none at all in the last tile, 8 columns, K tails
                                   (257, 264, 512), (385, 8, 1032), (513, 520, 2056), (300, 1032, 640)])
def test_tcgen05_matches_simt_and_f32(rt, device, m, n, k):
    torch.manual_seed(m + n + k)
    a = torch.randn(m, k).to(torch.bfloat16)
    b = (torch.randn(n, k) * 0.05).to(torch.bfloat16)
    h = KernelHarness(rt)
    try:
        fast = run_gemm(h, h.lib.ttb_gemm, a, b, None, m, n, k)
        assert tc_status(h) == 0, "a wait inside the tensor-core kernel timed out"
        slow = run_gemm(h, h.lib.ttb_gemm_simt, a, b, None, m, n, k)
    finally:
        h.close()
    ref = (a.float() @ b.float().t())
    assert_matches(slow, ref.to(torch.bfloat16), f"simt {m}x{n}x{k}")
    assert_matches(fast, ref.to(torch.bfloat16), f"tcgen05 {m}x{n}x{k}")
    # both accumulate in f32 and round once: they may differ only where f32 summation order
    # moves a value across a bf16 rounding boundary
    diff = (fast.float() - slow.float()).abs()
    assert (diff > 2.0 ** -6 * ref.abs() + 1e-3).sum().item() == 0


@pytest.mark.parametrize("act,round_steps", [(None, 0), ("relu", 0), ("silu", 2), ("relu", 3)])
def test_tcgen05_epilogue(rt, device, act, round_steps):
    m, n, k = 256, 384, 512
    torch.manual_seed(7)
    a = torch.randn(m, k).to(torch.bfloat16)
    b = (torch.randn(n, k) * 0.05).to(torch.bfloat16)
    bias = torch.randn(n).to(torch.bfloat16)
    h = KernelHarness(rt)
    try:
        fast = run_gemm(h, h.lib.ttb_gemm, a, b, bias, m, n, k, ACT[act], round_steps)
        slow = run_gemm(h, h.lib.ttb_gemm_simt, a, b, bias, m, n, k, ACT[act], round_steps)
        assert tc_status(h) == 0
    finally:
        h.close()
    acc = a.float() @ b.float().t()
    if round_steps & 1:
        acc = acc.to(torch.bfloat16).float()
    acc = acc + bias.float()
    if round_steps & 2:
        acc = acc.to(torch.bfloat16).float()
    if act == "relu":
        acc = torch.relu(acc)
    elif act == "silu":
        acc = torch.nn.functional.silu(acc)
    assert_matches(fast, acc.to(torch.bfloat16), "tcgen05 epilogue")
    assert_matches(slow, acc.to(torch.bfloat16), "simt epilogue")


def test_tcgen05_f32_output(rt, device):
    m, n, k = 256, 256, 256
    a = torch.randn(m, k).to(torch.bfloat16)
    b = torch.randn(n, k).to(torch.bfloat16)
    h = KernelHarness(rt)
    try:
        fast = run_gemm(h, h.lib.ttb_gemm, a, b, None, m, n, k, out_dtype=torch.float32)
        assert tc_status(h) == 0
    finally:
        h.close()
    assert_matches(fast, a.float() @ b.float().t(), "f32 out", (0.999, 1e-3, 1e-4))


@pytest.mark.parametrize("extra_op", [1, 2])
@pytest.mark.parametrize("m,n,k,with_bias", [(256, 384, 512, False), (200, 136, 72, True), (2048, 1024, 256, False),
                                             (8, 16, 32, False)])
def test_gemm_fused_extra_operand(rt, device, extra_op, m, n, k, with_bias):
    """ttb_gemm_fused: residual add (1) and SwiGLU gating (2) in the GEMM's epilogue equal the
    chain of separate ops, with every intermediate rounded to bf16.  The last shape is too small
    for the tensor-core kernel and exercises the composed fallback."""
    torch.manual_seed(m + extra_op)
    a = torch.randn(m, k).to(torch.bfloat16)
    b = (torch.randn(n, k) * 0.05).to(torch.bfloat16)
    bias = torch.randn(n).to(torch.bfloat16) if with_bias else None
    extra = torch.randn(m, n).to(torch.bfloat16)
    h = KernelHarness(rt)
    try:
        da, db, de = h.upload(a), h.upload(b), h.upload(extra)
        dbias = h.upload(bias) if with_bias else None
        dc = h.empty((m, n), torch.bfloat16)
        i64 = ctypes.c_int64
        rc = h.lib.ttb_gemm_fused(da, db, dbias, dc, BF16, BF16, BF16, i64(1), i64(m), i64(n), i64(k), 0, 1, i64(0), i64(0),
                                  0, 0, de, extra_op, h.stream)
        assert rc == 0, h.lib.ttb_last_error().decode()
        got = h.download(dc, (m, n), torch.bfloat16)
        assert tc_status(h) == 0
    finally:
        h.close()
    acc = a.float() @ b.float().t()
    if with_bias:
        acc = acc + bias.float()
    r = acc.to(torch.bfloat16).float()
    if extra_op == 1:
        want = (r + extra.float()).to(torch.bfloat16)
    else:
        s = torch.nn.functional.silu(extra.float()).to(torch.bfloat16).float()
        want = (s * r).to(torch.bfloat16)
    assert_matches(got, want, f"gemm_fused op={extra_op} {m}x{n}x{k}")


def test_pointwise_conv_shape_bias_relu(rt, device):
    """The memory-bound shape of config 5's 1x1 convolutions (every pixel of [64,56,56,64] times a
    [256,64] weight) with the bias + relu epilogue, against an f32 reference."""
    m, n, k = 200704, 256, 64
    torch.manual_seed(3)
    a = torch.randn(m, k).to(torch.bfloat16)
    b = (torch.randn(n, k) * 0.1).to(torch.bfloat16)
    bias = torch.randn(n).to(torch.bfloat16)
    h = KernelHarness(rt)
    try:
        got = run_gemm(h, h.lib.ttb_gemm, a, b, bias, m, n, k, ACT["relu"], 0)
        assert tc_status(h) == 0
    finally:
        h.close()
    want = torch.relu(a.float() @ b.float().t() + bias.float()).to(torch.bfloat16)
    assert_matches(got, want, "pointwise conv shape")


@pytest.mark.parametrize("m,k,ns", [(2048, 4096, (4096, 1024, 1024)), (200, 264, (136, 72)), (256, 512, (512, 128, 128)),
                                    (64, 64, (16, 16))])
def test_gemm_grouped_matches_separate_calls(rt, device, m, k, ns):
    """ttb_gemm_grouped (several products sharing A in one launch) gives exactly what separate
    ttb_gemm calls give; the last case is too small for the tensor-core kernel (loop fallback)."""
    torch.manual_seed(m + k)
    a = torch.randn(m, k).to(torch.bfloat16)
    bs = [(torch.randn(n, k) * 0.05).to(torch.bfloat16) for n in ns]
    h = KernelHarness(rt)
    try:
        da = h.upload(a)
        dbs = [h.upload(b) for b in bs]
        dcs = [h.empty((m, n), torch.bfloat16) for n in ns]
        i64 = ctypes.c_int64
        cnt = len(ns)
        bp = (ctypes.c_void_p * cnt)(*[p.value for p in dbs])
        cp = (ctypes.c_void_p * cnt)(*[p.value for p in dcs])
        nn = (ctypes.c_int64 * cnt)(*ns)
        rc = h.lib.ttb_gemm_grouped(da, bp, cp, nn, cnt, BF16, BF16, i64(m), i64(k), h.stream)
        assert rc == 0, h.lib.ttb_last_error().decode()
        got = [h.download(dc, (m, n), torch.bfloat16) for dc, n in zip(dcs, ns)]
        assert tc_status(h) == 0
        sep = [run_gemm(h, h.lib.ttb_gemm, a, b, None, m, n, k) for b, n in zip(bs, ns)]
    finally:
        h.close()
    for g, s_, b in zip(got, sep, bs):
        assert torch.equal(g, s_), "grouped and separate launches differ"
        assert_matches(g, (a.float() @ b.float().t()).to(torch.bfloat16), "grouped gemm")


@pytest.mark.parametrize("m,n,k1,k2,act,biases", [(200704 // 8, 256, 64, 64, 1, True), (300, 136, 72, 264, 0, True),
                                                   (1024, 64, 128, 64, 1, False), (130, 512, 64, 576, 1, True)])
def test_gemm_dual_add_equals_the_chain_of_launches(rt, device, m, n, k1, k2, act, biases):
    """ttb_gemm_dual_add (two products in two accumulators of one launch, summed in the epilogue) gives bit for bit
    what the second product as its own launch followed by the first with the residual-add epilogue gives, and what
    the f32 reference of the op chain with its bf16 roundings gives within tolerance."""
    torch.manual_seed(m + n + k1)
    a1 = torch.randn(m, k1).to(torch.bfloat16)
    a2 = torch.randn(m, k2).to(torch.bfloat16)
    b1 = (torch.randn(n, k1) * 0.1).to(torch.bfloat16)
    b2 = (torch.randn(n, k2) * 0.1).to(torch.bfloat16)
    bias1 = torch.randn(n).to(torch.bfloat16) if biases else None
    bias2 = torch.randn(n).to(torch.bfloat16) if biases else None
    h = KernelHarness(rt)
    try:
        i64 = ctypes.c_int64
        d = {k: h.upload(v) for k, v in dict(a1=a1, a2=a2, b1=b1, b2=b2).items()}
        db1 = h.upload(bias1) if biases else None
        db2 = h.upload(bias2) if biases else None
        out = h.empty((m, n), torch.bfloat16)
        rc = h.lib.ttb_gemm_dual_add(d["a1"], d["b1"], db1, d["a2"], d["b2"], db2, out, BF16, BF16, i64(m), i64(n), i64(k1), i64(k2),
                                     act, h.stream)
        assert rc == 0, h.lib.ttb_last_error().decode()
        got = h.download(out, (m, n), torch.bfloat16)
        assert tc_status(h) == 0
        second = h.empty((m, n), torch.bfloat16)
        assert h.lib.ttb_gemm(d["a2"], d["b2"], db2, second, BF16, BF16, BF16, i64(1), i64(m), i64(n), i64(k2), 0, 1, i64(0), i64(0),
                              0, 0, h.stream) == 0
        chain = h.empty((m, n), torch.bfloat16)
        assert h.lib.ttb_gemm_fused(d["a1"], d["b1"], db1, chain, BF16, BF16, BF16, i64(1), i64(m), i64(n), i64(k1), 0, 1, i64(0),
                                    i64(0), 0, 0, second, 3 if act else 1, h.stream) == 0
        want_chain = h.download(chain, (m, n), torch.bfloat16)
    finally:
        h.close()
    assert torch.equal(got, want_chain), f"{(got != want_chain).sum().item()} of {got.numel()} elements differ from the chain"
    v1 = (a1.float() @ b1.float().t() + (bias1.float() if biases else 0)).to(torch.bfloat16)
    v2 = (a2.float() @ b2.float().t() + (bias2.float() if biases else 0)).to(torch.bfloat16)
    ref = (v1.float() + v2.float())
    ref = (torch.relu(ref) if act else ref).to(torch.bfloat16)
    assert_matches(got, ref, "dual add")


@pytest.mark.parametrize("batch,seq,k,ns,mask", [(1, 2048, 4096, (4096, 1024, 1024), 3), (2, 200, 264, (256, 128, 128), 3),
                                                 (1, 512, 512, (512, 128, 128), 2), (1, 300, 128, (128, 384), 1)])
def test_gemm_grouped_with_rotary_embedding_epilogue(rt, device, batch, seq, k, ns, mask):
    """ttb_gemm_grouped_rope: the problems in the mask come out rotated, bit for bit what the grouped product
    followed by the rotary embedding (f32 arithmetic on the rounded product, one rounding) gives; the others
    are the plain product.  Rows are (batch, position) pairs; ragged row counts exercise the clipped tiles."""
    m = batch * seq
    torch.manual_seed(m + k)
    a = torch.randn(m, k).to(torch.bfloat16)
    bs = [(torch.randn(n, k) * 0.05).to(torch.bfloat16) for n in ns]
    pos = torch.arange(seq, dtype=torch.float32)[:, None]
    freq = 1.0 / (10000.0 ** (torch.arange(0, 64, dtype=torch.float32) / 64))
    ang = torch.cat([pos * freq, pos * freq], dim=1)
    cos, sin = ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)
    h = KernelHarness(rt)
    try:
        da = h.upload(a)
        dbs = [h.upload(b) for b in bs]
        dcs = [h.empty((m, n), torch.bfloat16) for n in ns]
        dcos, dsin = h.upload(cos), h.upload(sin)
        i64 = ctypes.c_int64
        cnt = len(ns)
        bp = (ctypes.c_void_p * cnt)(*[p.value for p in dbs])
        cp = (ctypes.c_void_p * cnt)(*[p.value for p in dcs])
        nn = (ctypes.c_int64 * cnt)(*ns)
        rc = h.lib.ttb_gemm_grouped_rope(da, bp, cp, nn, cnt, BF16, i64(m), i64(k), dcos, dsin, mask, i64(seq), i64(128), h.stream)
        assert rc == 0, h.lib.ttb_last_error().decode()
        got = [h.download(dc, (m, n), torch.bfloat16) for dc, n in zip(dcs, ns)]
        assert tc_status(h) == 0
        rc = h.lib.ttb_gemm_grouped(da, bp, cp, nn, cnt, BF16, BF16, i64(m), i64(k), h.stream)
        assert rc == 0, h.lib.ttb_last_error().decode()
        plain = [h.download(dc, (m, n), torch.bfloat16) for dc, n in zip(dcs, ns)]
    finally:
        h.close()
    for i, (g, pl, n) in enumerate(zip(got, plain, ns)):
        if not (mask >> i) & 1:
            assert torch.equal(g, pl), f"problem {i} is not in the mask and must be the plain product"
            continue
        x = pl.float().view(batch, seq, n // 128, 128)
        c, s_ = cos.float()[None, :, None, :], sin.float()[None, :, None, :]
        rot = torch.cat([-x[..., 64:], x[..., :64]], dim=-1)
        want = (x * c + rot * s_).to(torch.bfloat16).view(m, n)
        assert torch.equal(g, want), f"problem {i}: {(g != want).sum().item()} of {g.numel()} elements differ"


@pytest.mark.parametrize("m,n,k", [(256, 384, 512), (2048, 1792, 1024), (200, 136, 72), (8, 16, 32), (1280, 14336, 256),
                                   (130, 64, 64)])
def test_gemm_swiglu_equals_the_chain_of_launches(rt, device, m, n, k):
    """ttb_gemm_swiglu (gate and up projections in one accumulator, silu(gate) * up in the epilogue)
    gives bit for bit what linear, linear + silu-multiply epilogue give as two launches, and matches
    the f32 reference of the op chain with its bf16 roundings.  (8, 16, 32) is below the tensor-core
    kernel's size limit and runs the composed fallback."""
    torch.manual_seed(m + n + k)
    a = torch.randn(m, k).to(torch.bfloat16)
    wg = (torch.randn(n, k) * 0.05).to(torch.bfloat16)
    wu = (torch.randn(n, k) * 0.05).to(torch.bfloat16)
    h = KernelHarness(rt)
    try:
        da, dg, du = h.upload(a), h.upload(wg), h.upload(wu)
        i64 = ctypes.c_int64
        out = h.empty((m, n), torch.bfloat16)
        rc = h.lib.ttb_gemm_swiglu(da, dg, du, out, BF16, i64(m), i64(n), i64(k), h.stream)
        assert rc == 0, h.lib.ttb_last_error().decode()
        got = h.download(out, (m, n), torch.bfloat16)
        assert tc_status(h) == 0
        gate = h.empty((m, n), torch.bfloat16)
        two = h.empty((m, n), torch.bfloat16)
        assert h.lib.ttb_gemm(da, dg, None, gate, BF16, BF16, BF16, i64(1), i64(m), i64(n), i64(k), 0, 1, i64(0), i64(0), 0, 0,
                              h.stream) == 0
        assert h.lib.ttb_gemm_fused(da, du, None, two, BF16, BF16, BF16, i64(1), i64(m), i64(n), i64(k), 0, 1, i64(0), i64(0), 0, 0,
                                    gate, 2, h.stream) == 0
        chain = h.download(two, (m, n), torch.bfloat16)
    finally:
        h.close()
    assert torch.equal(got, chain), "one launch and two launches differ"
    g = (a.float() @ wg.float().t()).to(torch.bfloat16).float()
    u = (a.float() @ wu.float().t()).to(torch.bfloat16).float()
    want = (torch.nn.functional.silu(g).to(torch.bfloat16).float() * u).to(torch.bfloat16)
    # three roundings in a row (gate, silu, product): a one-ulp flip of an intermediate, which a different
    # f32 summation order can cause, moves the result by up to two ulps
    assert_matches(got, want, f"swiglu {m}x{n}x{k}", (0.999, 2e-2, 2.0 ** -6))
