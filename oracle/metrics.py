"""Comparison metrics used by the reference's runners, restated (tools/golden/metrics.py:19-127):
max absolute / relative error and the Pearson correlation coefficient with the same special
cases (empty tensors, all-NaN, constant tensors, single elements)."""

from __future__ import annotations

import numpy as np
import torch


def _as_float(t: torch.Tensor) -> torch.Tensor:
    t = t.detach().clone()
    if not torch.is_floating_point(t):
        return t.to(torch.float64)
    if t.dtype in (torch.bfloat16, torch.float16):
        return t.to(torch.float32)
    return t


def get_atol_rtol(golden: torch.Tensor, calculated: torch.Tensor):
    g, c = _as_float(golden), _as_float(calculated)
    if g.numel() == 0 or c.numel() == 0:
        return 0.0, 0.0
    g, c = g.double(), c.double()
    atol = torch.max(torch.abs(g - c)).item()
    rtol = torch.max(torch.abs((g - c) / c)).item()
    return atol, rtol


def get_pcc(golden: torch.Tensor, calculated: torch.Tensor, atol: float = 1e-8, rtol: float = 1e-5) -> float:
    g, c = _as_float(golden), _as_float(calculated)
    if g.numel() == 0 and c.numel() == 0:
        return 1.0 if g.shape == c.shape else 0.0
    if g.numel() == 0 or c.numel() == 0:
        return 0.0
    if g.numel() == 1 and g.item() != 0:
        cs = torch.nn.functional.cosine_similarity(g.float().reshape(1, 1), c.float().reshape(1, 1), dim=0)
        return 1.0 if cs.item() else 0.0
    if torch.all(torch.isnan(g)) and torch.all(torch.isnan(c)):
        return 1.0
    if torch.any(g.bool()) != torch.any(c.bool()):
        return 0.0
    if torch.all(torch.isnan(g)) or torch.all(torch.isnan(c)):
        return 0.0
    g = torch.where(torch.isfinite(g), g, torch.zeros_like(g))
    c = torch.where(torch.isfinite(c), c, torch.zeros_like(c))
    if torch.equal(g, c):
        return 1.0
    if g.numel() == 1:
        return float(torch.isclose(g, c, atol=atol, rtol=rtol).item())
    if torch.max(g) == torch.min(g) and torch.max(c) == torch.min(c):
        return float(torch.isclose(torch.max(g), torch.max(c), atol=atol, rtol=rtol).item())
    m = np.corrcoef(g.double().numpy().ravel(), c.double().numpy().ravel())
    v = float(m[0, 1])
    return 1.0 if np.isnan(v) else v


def check_close(golden: torch.Tensor, calculated: torch.Tensor, pcc: float, atol: float, rtol: float):
    """Returns (ok, report).  A float result passes when PCC >= `pcc` and every element satisfies
    |calc - golden| <= atol + rtol * |golden| (torch.allclose form, as the reference's own
    check in tools/ttrt/common/run.py:925-931 uses)."""
    a, r = get_atol_rtol(golden, calculated)
    p = get_pcc(golden, calculated)
    g, c = _as_float(golden).double(), _as_float(calculated).double()
    close = bool(torch.all(torch.abs(g - c) <= atol + rtol * torch.abs(g)).item()) if g.numel() else True
    ok = p >= pcc and close and golden.shape == calculated.shape
    return ok, f"pcc={p:.6f} (>= {pcc}) max_abs={a:.3e} max_rel={r:.3e} allclose(atol={atol}, rtol={rtol})={close}"
