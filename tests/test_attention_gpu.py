"""Attention kernels through the kernel-level C ABI (ttb_sdpa), checked against the oracle's f32
softmax (oracle/ops.py sdpa, which restates tools/golden/mapping.py:8398-8500).  Covers the
tcgen05 kernel's tile edges: ragged query / key tails, causal diagonal tiles, grouped-query heads,
different query and key lengths, both 16-bit formats."""

import ctypes

import pytest
import torch

from helpers import KernelHarness, assert_matches
from oracle import ops as O

pytestmark = pytest.mark.gpu

DT = {torch.bfloat16: 2, torch.float16: 1}


@pytest.fixture(scope="module")
def kh(rt):
    return KernelHarness(rt)


def run_sdpa(kh, q, k, v, causal, scale=None):
    B, Hq, Sq, D = q.shape
    _, Hkv, Skv, _ = k.shape
    if scale is None:
        scale = 1.0 / D ** 0.5
    dq, dk, dv = kh.upload(q), kh.upload(k), kh.upload(v)
    out = kh.empty(q.shape, q.dtype)
    i64 = ctypes.c_int64
    rc = kh.lib.ttb_sdpa(dq, dk, dv, None, out, DT[q.dtype], i64(B), i64(Hq), i64(Hkv), i64(Sq), i64(Skv), i64(D),
                         i64(0), i64(0), int(causal), ctypes.c_float(scale), kh.stream)
    kh._check(rc)
    got = kh.download(out, q.shape, q.dtype)
    st = ctypes.c_int(-1)
    kh._check(kh.lib.ttb_sdpa_tcgen05_status(ctypes.byref(st)))
    assert st.value == 0, f"tcgen05 attention gave up at wait site {st.value >> 8}"
    return got


CASES = [
    # B, Hq, Hkv, Sq, Skv, causal
    (1, 1, 1, 128, 128, False),
    (1, 1, 1, 128, 128, True),
    (1, 2, 2, 256, 256, True),
    (2, 4, 2, 200, 200, True),
    (2, 4, 2, 77, 77, False),
    (1, 8, 2, 1024, 1024, True),
    (1, 2, 1, 128, 384, False),
    (1, 2, 1, 130, 515, False),
    (1, 2, 2, 384, 512, True),
    (1, 2, 2, 1, 300, False),
    # tensor-parallel shards of the decoder block (few heads)
    (1, 4, 1, 2048, 2048, True),
    (1, 8, 2, 2048, 2048, True),
    # few heads and long sequences: the causal key ranges are split over several CTAs and merged
    (1, 2, 1, 4096, 4096, True),
    (1, 2, 2, 3333, 3333, True),
    (1, 1, 1, 3000, 3000, True),
    # enough CTAs for the kernel that gives one CTA two heads of a grouped-query group
    (1, 16, 4, 2432, 2432, True),
    (1, 16, 8, 2400, 2400, False),
    (2, 8, 4, 2500, 2500, True),
]


@pytest.mark.parametrize("B,Hq,Hkv,Sq,Skv,causal", CASES)
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_sdpa_head_dim_128(kh, B, Hq, Hkv, Sq, Skv, causal, dtype):
    torch.manual_seed(Sq * 7 + Skv)
    q = torch.randn(B, Hq, Sq, 128).to(dtype)
    k = torch.randn(B, Hkv, Skv, 128).to(dtype)
    v = torch.randn(B, Hkv, Skv, 128).to(dtype)
    got = run_sdpa(kh, q, k, v, causal)
    want = O.sdpa(q, k, v, is_causal=causal)
    assert_matches(got, want, f"sdpa B{B} H{Hq}/{Hkv} S{Sq}x{Skv} causal={causal} {dtype}")


def test_sdpa_large_scores_and_scale(kh):
    # Scores far from zero exercise the running-maximum rescale across key tiles.
    torch.manual_seed(5)
    q = (torch.randn(1, 2, 256, 128) * 4).to(torch.bfloat16)
    k = (torch.randn(1, 2, 640, 128) * 4).to(torch.bfloat16)
    v = torch.randn(1, 2, 640, 128).to(torch.bfloat16)
    got = run_sdpa(kh, q, k, v, False, scale=0.25)
    want = O.sdpa(q, k, v, is_causal=False, scale=0.25)
    assert_matches(got, want, "sdpa large scores")


def test_sdpa_two_heads_per_cta_with_frequent_rescales(kh):
    # Enough CTAs for the two-heads-per-CTA kernel, and keys whose magnitude grows along the sequence, so that rows
    # raise their running maximum (and rescale O) at different tiles: the softmax warps of a head drift apart, which is
    # what their barrier protocol has to survive.
    torch.manual_seed(17)
    B, Hq, Hkv, S = 2, 16, 4, 2048
    q = (torch.randn(B, Hq, S, 128) * 2).to(torch.bfloat16)
    growth = (1.0 + 6.0 * torch.arange(S) / S).reshape(1, 1, S, 1) * (torch.rand(B, Hkv, S, 1) > 0.5)
    k = (torch.randn(B, Hkv, S, 128) * growth).to(torch.bfloat16)
    v = torch.randn(B, Hkv, S, 128).to(torch.bfloat16)
    for causal in (True, False):
        got = run_sdpa(kh, q, k, v, causal, scale=0.2)
        want = O.sdpa(q, k, v, is_causal=causal, scale=0.2)
        assert_matches(got, want, f"sdpa with growing scores, causal={causal}")


def test_sdpa_kernels_agree(kh, monkeypatch):
    # Two calls in a row give the same bits (no state carried between launches).
    torch.manual_seed(9)
    q = torch.randn(1, 4, 512, 128).to(torch.bfloat16)
    k = torch.randn(1, 4, 512, 128).to(torch.bfloat16)
    v = torch.randn(1, 4, 512, 128).to(torch.bfloat16)
    a = run_sdpa(kh, q, k, v, True)
    b = run_sdpa(kh, q, k, v, True)
    assert torch.equal(a, b)
