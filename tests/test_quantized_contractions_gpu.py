"""Contractions on quantized (8-bit integer) operands: matmul / linear / conv2d with an exact Int32
accumulator on the tensor cores (tcgen05.mma kind::i8) and on the CUDA-core fallback, and the dequantize
that follows them fused into the epilogue.  Integer results must equal an integer matmul on the CPU bit
for bit; dequantized results are float(acc) * scale with one rounding, also bit for bit."""

import ctypes

import pytest
import torch

from helpers import KernelHarness, check_graph, oracle_results, run_program
from ttmlir_b200 import graphs

pytestmark = pytest.mark.gpu

I8, U8, I32, F32, BF16 = 17, 11, 12, 0, 2
TORCH = {I8: torch.int8, U8: torch.uint8, I32: torch.int32, F32: torch.float32, BF16: torch.bfloat16}


def int_matmul(a, b, ta, tb):
    x, y = a.double(), b.double()
    if ta:
        x = x.transpose(-2, -1)
    if tb:
        y = y.transpose(-2, -1)
    return torch.matmul(x, y).to(torch.int64)      # exact: |products| <= 2^16, sums far below 2^53


def call(h, fn, a, b, out_dtype, batch, m, n, k, ta, tb, scale=None, scalar=0.0):
    i64 = ctypes.c_int64
    da, db = h.upload(a), h.upload(b)
    dc = h.empty((batch, m, n), TORCH[out_dtype])
    ds = h.upload(scale) if scale is not None else None
    adt = I8 if a.dtype == torch.int8 else U8
    bdt = I8 if b.dtype == torch.int8 else U8
    rc = fn(da, db, dc, adt, bdt, out_dtype, i64(batch), i64(m), i64(n), i64(k), int(ta), int(tb),
            i64(0 if a.dim() == 2 else m * k), i64(0 if b.dim() == 2 else k * n), ds, ctypes.c_float(scalar), h.stream)
    assert rc == 0, h.lib.ttb_last_error().decode()
    return h.download(dc, (batch, m, n), TORCH[out_dtype])


@pytest.mark.parametrize("m,n,k", [(128, 256, 128), (2048, 1024, 4096), (130, 72, 80), (257, 520, 1040), (64, 64, 4096),
                                   (1000, 24, 48)])
@pytest.mark.parametrize("signs", ["ss", "us", "su"])
def test_int8_gemm_weight_layout_is_exact(rt, device, m, n, k, signs):
    """A[M, K] B[N, K]^T: the tensor-core kernel where it applies (k a multiple of 16, n of 4), tails in
    every dimension, signed and unsigned operands; the CUDA-core kernel must give the same integers."""
    h = KernelHarness(rt)
    try:
        g = torch.Generator().manual_seed(m + n + k)
        mk = lambda s, shape: (torch.randint(-128, 128, shape, generator=g, dtype=torch.int32).to(torch.int8) if s == "s"
                               else torch.randint(0, 256, shape, generator=g, dtype=torch.int32).to(torch.uint8))
        a, b = mk(signs[0], (m, k)), mk(signs[1], (n, k))
        want = int_matmul(a, b, False, True).to(torch.int32)
        got = call(h, h.lib.ttb_gemm_i8, a, b, I32, 1, m, n, k, False, True)[0]
        assert torch.equal(got, want)
        ref = call(h, h.lib.ttb_gemm_i8_simt, a, b, I32, 1, m, n, k, False, True)[0]
        assert torch.equal(ref, want)
        st = ctypes.c_int(-1)
        assert h.lib.ttb_gemm_tcgen05_status(ctypes.byref(st)) == 0 and st.value == 0
    finally:
        h.close()


@pytest.mark.parametrize("ta,tb", [(False, False), (True, False), (True, True)])
def test_int8_gemm_other_layouts_and_batches(rt, device, ta, tb):
    h = KernelHarness(rt)
    try:
        g = torch.Generator().manual_seed(5)
        batch, m, n, k = 3, 70, 45, 100
        a = torch.randint(-128, 128, (batch, k, m) if ta else (batch, m, k), generator=g, dtype=torch.int32).to(torch.int8)
        b = torch.randint(-128, 128, (batch, n, k) if tb else (batch, k, n), generator=g, dtype=torch.int32).to(torch.int8)
        got = call(h, h.lib.ttb_gemm_i8, a, b, I32, batch, m, n, k, ta, tb)
        assert torch.equal(got, int_matmul(a, b, ta, tb).to(torch.int32))
    finally:
        h.close()


@pytest.mark.parametrize("out_dtype", [F32, BF16])
@pytest.mark.parametrize("per_channel", [False, True])
@pytest.mark.parametrize("m,n,k", [(256, 384, 512), (130, 72, 80), (33, 20, 50)])
def test_int8_gemm_with_fused_dequantize(rt, device, out_dtype, per_channel, m, n, k):
    """float(acc) * scale, rounded once to the result type: what dequantize computes from the Int32
    accumulator ((q - 0) * scale in f32, tools/golden/mapping.py:9166 = torch.dequantize)."""
    h = KernelHarness(rt)
    try:
        g = torch.Generator().manual_seed(m * 3 + n)
        a = torch.randint(-128, 128, (m, k), generator=g, dtype=torch.int32).to(torch.int8)
        b = torch.randint(-128, 128, (n, k), generator=g, dtype=torch.int32).to(torch.int8)
        scale = (torch.rand(n, generator=g) * 1e-3 + 1e-4).to(torch.float32) if per_channel else None
        scalar = 0.00037
        acc = int_matmul(a, b, False, True).to(torch.int32)
        s = scale[None, :] if per_channel else torch.tensor(scalar, dtype=torch.float32)
        want = (acc.to(torch.float32) * s).to(TORCH[out_dtype])
        for fn in (h.lib.ttb_gemm_i8, h.lib.ttb_gemm_i8_simt):
            got = call(h, fn, a, b, out_dtype, 1, m, n, k, False, True, scale, scalar)[0]
            assert torch.equal(got, want)
    finally:
        h.close()


@pytest.mark.parametrize("kw", [dict(m=64, k=128, n=96), dict(m=256, k=512, n=384), dict(m=130, k=200, n=72)])
def test_quantized_linear_graph(rt, device, kw):
    """quantize(activations) -> matmul on Int8 -> dequantize(per channel) -> add(bias) through submit.  The
    matmul and the dequantize run as one launch; with debug hooks registered (nothing fused) the program
    must give the same bits, and the Int32 accumulator seen by the hook must be exact."""
    ins = graphs.w8a8_linear_inputs(**kw)
    buf = graphs.build_binary(graphs.w8a8_linear_graph, **kw)
    fused = run_program(rt, device, buf, ins)[0]
    want = oracle_results(graphs.w8a8_linear_graph, ins, **kw)[0]
    assert torch.equal(fused, want)                    # integer contraction, one rounding per op: nothing to tolerate
    outputs = {}

    def post(_bin, ctx, op):
        t = rt.get_op_output_tensor(op, ctx)
        if t is not None:
            outputs[rt.get_op_loc_info(op)] = rt.to_torch(t)
    rt.DebugHooks.get(None, post)
    try:
        unfused = run_program(rt, device, buf, ins)[0]
    finally:
        rt.unregister_hooks()
    assert torch.equal(unfused, fused)
    aq = torch.quantize_per_tensor(ins[0].float(), 0.04, 0, torch.qint8).int_repr()
    assert torch.equal(outputs['loc("quantize_activation")'], aq)
    assert torch.equal(outputs['loc("int_matmul")'], int_matmul(aq, ins[1], False, True).to(torch.int32))


def test_quantized_linear_full_size(rt, device):
    """Config 3's shapes with both operands quantized (2048 x 4096 by 11008 x 4096): the whole result
    against the oracle, bit for bit."""
    ins = graphs.w8a8_linear_inputs()
    buf = graphs.build_binary(graphs.w8a8_linear_graph)
    got = run_program(rt, device, buf, ins)[0]
    want = oracle_results(graphs.w8a8_linear_graph, ins)[0]
    assert list(got.shape) == [2048, 11008] and torch.equal(got, want)


@pytest.mark.parametrize("container", ["Int8", "Int32"])
@pytest.mark.parametrize("kw", [dict(batch=2, hw=8, c_in=16, c_out=24, kernel=3), dict(batch=3, hw=9, c_in=20, c_out=8, kernel=1),
                                dict(batch=4, hw=14, c_in=64, c_out=128, kernel=3), dict(batch=2, hw=7, c_in=128, c_out=64, kernel=1)])
def test_quantized_conv_graph(rt, device, container, kw):
    """conv2d on quantized input and weight (Int8 tensors, or the Int32 containers the compiler uses by
    default) -> dequantize per output channel; fused and op-by-op must agree with the oracle exactly."""
    tdt = torch.int8 if container == "Int8" else torch.int32
    ins = graphs.quantized_conv_inputs(container=tdt, **kw)
    buf = graphs.build_binary(graphs.quantized_conv_graph, container=container, **kw)
    got = run_program(rt, device, buf, ins)[0]
    want = oracle_results(graphs.quantized_conv_graph, ins, container=container, **kw)[0]
    assert torch.equal(got, want)
    seen = {}
    rt.DebugHooks.get(None, lambda _b, ctx, op: seen.__setitem__(rt.get_op_loc_info(op), True))
    try:
        unfused = run_program(rt, device, buf, ins)[0]
    finally:
        rt.unregister_hooks()
    assert 'loc("int_conv")' in seen and torch.equal(unfused, got)
