"""ttb_conv2d_static: the convolution entry point that takes its workspace from a buffer built
into the library instead of from the caller.

It exists for hosts that may not allocate device memory where they run the convolution (a
serving loop living inside someone else's memory arena, a plugin whose application forbids
cudaMalloc after start-up).  The test drives it through the C ABI next to the ordinary
ttb_conv2d (which gets a workspace allocated here) and requires identical bytes, twice in a
row with different data, so that whatever the first call left in the shared buffer cannot
leak into the second.  The file name sorts last on purpose: a run that stops at the first
failure has then already executed every other test.
"""

import ctypes

import pytest
import torch

from helpers import KernelHarness

pytestmark = pytest.mark.gpu

BF16, F32 = 2, 0


def pool_in_use(lib, reset=False):
    """(bytes handed out by the device's memory pool now, high-water mark since the last reset)."""
    used, high = ctypes.c_uint64(), ctypes.c_uint64()
    assert lib.ttb_mempool_stats(None, ctypes.byref(used), ctypes.byref(high), int(reset)) == 0
    return used.value, high.value


def conv_pair(h, seed, n, hh, ww, c, o, k, pad, dtype=torch.bfloat16):
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(n, hh, ww, c, generator=g).to(dtype)
    w = (torch.randn(o, c, k, k, generator=g) * 0.1).to(dtype)
    b = torch.randn(o, generator=g).to(dtype)
    BF16 = 2 if dtype == torch.bfloat16 else 0   # the dtype tag both calls below pass
    dx, dw, db = h.upload(x), h.upload(w), h.upload(b)
    ho, wo = hh + 2 * pad - k + 1, ww + 2 * pad - k + 1
    padding = (ctypes.c_int * 4)(pad, pad, pad, pad)
    i64 = ctypes.c_int64
    lib = h.lib
    need = lib.ttb_conv2d_workspace_bytes(BF16, i64(n), i64(hh), i64(ww), i64(c), i64(o), k, k, 1, 1, padding, 1, 1, 1)
    assert 0 <= need <= (28 << 20)
    ws = h.empty((max(need, 16),), torch.uint8)
    out_ref = h.empty((n, ho, wo, o), dtype)
    out_new = h.empty((n, ho, wo, o), dtype)
    rc = lib.ttb_conv2d(dx, dw, db, out_ref, BF16, BF16, i64(n), i64(hh), i64(ww), i64(c), i64(o), k, k, 1, 1, padding,
                        1, 1, 1, 1, ws, h.stream)
    assert rc == 0, lib.ttb_last_error().decode()
    h.sync()
    # From here to the end of the call under test nothing may come out of the memory pool: the
    # high-water mark of the pool's use is reset, and must still equal the current use afterwards.
    pool_in_use(lib, reset=True)
    before, _ = pool_in_use(lib)
    rc = lib.ttb_conv2d_static(dx, dw, db, out_new, BF16, BF16, i64(n), i64(hh), i64(ww), i64(c), i64(o), k, k, 1, 1,
                               padding, 1, 1, 1, 1, h.stream)
    assert rc == 0, lib.ttb_last_error().decode()
    h.sync()
    after, high = pool_in_use(lib)
    assert after == before and high <= before, f"the static entry point allocated: in use {before} -> {after}, high {high}"
    shape = (n, ho, wo, o)
    return h.download(out_ref, shape, dtype), h.download(out_new, shape, dtype), x, w, b


def test_static_scratch_conv_matches_workspace_conv_twice(rt, device):
    h = KernelHarness(rt)
    try:
        ref1, new1, x, w, b = conv_pair(h, 11, 2, 20, 18, 64, 96, 3, 1)
        assert torch.equal(ref1, new1)
        # and both agree with a float reference of the same convolution (+ bias, relu)
        want = torch.nn.functional.conv2d(x.float().permute(0, 3, 1, 2), w.float(), b.float(), padding=1)
        want = torch.relu(want).permute(0, 2, 3, 1)
        assert torch.allclose(new1.float(), want, atol=1e-2, rtol=2.0 ** -7)
        # second call, other data and a smaller problem: stale scratch contents must not matter
        ref2, new2, *_ = conv_pair(h, 12, 1, 9, 13, 32, 40, 3, 1)
        assert torch.equal(ref2, new2)
        assert not torch.equal(new1.reshape(-1)[: new2.numel()], new2.reshape(-1))
    finally:
        h.close()


@pytest.mark.parametrize("dtype,shape", [
    (torch.float32, (1, 8, 8, 32, 32, 3, 1)),      # f32: the CUDA-core contraction, which splits K = 288 over blocks
    (torch.bfloat16, (1, 4, 4, 32, 32, 3, 1)),     # 16-bit but too small for the tensor-core kernel: same path
    (torch.float32, (2, 6, 5, 24, 16, 1, 0)),      # pointwise: no workspace at all, the contraction may still split
])
def test_static_scratch_conv_on_the_cuda_core_path_allocates_nothing(rt, device, dtype, shape):
    """Shapes the tensor-core kernel declines reach the CUDA-core contraction, whose split-K mode
    needs scratch for partial sums: under the static entry point that scratch is the tail of the
    built-in buffer, so the results equal the ordinary entry point's bit for bit and the memory pool
    is not touched (checked inside conv_pair).  Twice in a row, as above."""
    h = KernelHarness(rt)
    try:
        for seed in (21, 22):
            ref, new, x, w, b = conv_pair(h, seed, *shape, dtype=dtype)
            assert torch.equal(ref, new)
            want = torch.nn.functional.conv2d(x.float().permute(0, 3, 1, 2), w.float(), b.float(), padding=shape[-1])
            want = torch.relu(want).permute(0, 2, 3, 1)
            tol = dict(atol=1e-4, rtol=1e-4) if dtype == torch.float32 else dict(atol=1e-2, rtol=2.0 ** -7)
            assert torch.allclose(new.float(), want, **tol)
    finally:
        h.close()


def test_static_scratch_refuses_oversized_problem(rt, device):
    h = KernelHarness(rt)
    try:
        i64 = ctypes.c_int64
        padding = (ctypes.c_int * 4)(1, 1, 1, 1)
        dummy = h.empty((16,), torch.uint8)
        # 48 channels are not whole 64-channel blocks, so the gathered input is materialised:
        # 64 x 56 x 56 pixels x 432 taps x 2 bytes = 173 MB, beyond the 32 MiB buffer.  The call must
        # refuse before touching any tensor (the pointers here are 16-byte dummies).
        rc = h.lib.ttb_conv2d_static(dummy, dummy, None, dummy, BF16, BF16, i64(64), i64(56), i64(56), i64(48), i64(64),
                                     3, 3, 1, 1, padding, 1, 1, 1, 0, h.stream)
        assert rc != 0
        msg = h.lib.ttb_last_error().decode()
        assert "scratch" in msg and "ttb_conv2d" in msg
        # extents that are not positive, or whose byte count overflows, are refused as well
        rc = h.lib.ttb_conv2d_static(dummy, dummy, None, dummy, BF16, BF16, i64(-3), i64(56), i64(56), i64(48), i64(64),
                                     3, 3, 1, 1, padding, 1, 1, 1, 0, h.stream)
        assert rc != 0
        rc = h.lib.ttb_conv2d_static(dummy, dummy, None, dummy, BF16, BF16, i64(1 << 40), i64(1 << 20), i64(1 << 20), i64(48),
                                     i64(64), 3, 3, 1, 1, padding, 1, 1, 1, 0, h.stream)
        assert rc != 0
    finally:
        h.close()
