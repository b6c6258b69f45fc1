"""Tolerance checker used by the parity tests (test infrastructure only).

Restates tests/lib.py:8-73 (``check_is_allclose``): positions of +inf, -inf and
NaN must coincide exactly; every other element must satisfy an absolute OR a
relative bound; and a global cosine difference bound must hold.
"""
from __future__ import annotations

import torch


def cosine_diff(x: torch.Tensor, y: torch.Tensor) -> float:
    """1 - 2<x,y>/(|x|^2+|y|^2), in float64 (tests/lib.py:15-24)."""
    x, y = x.double(), y.double()
    den = float((x * x + y * y).sum())
    if den == 0.0:
        return 0.0
    return 1.0 - 2.0 * float((x * y).sum()) / den


def check_is_allclose(name: str, ans: torch.Tensor, ref: torch.Tensor,
                      abs_tol: float = 1e-5, rel_tol: float = 1e-2,
                      cos_diff_tol: float = 1e-7, verbose: bool = True) -> bool:
    if ans.shape != ref.shape:
        raise AssertionError(f"{name}: shape {tuple(ans.shape)} vs {tuple(ref.shape)}")
    ans = ans.detach().to("cpu", torch.float32).clone()
    ref = ref.detach().to("cpu", torch.float32).clone()

    ok = True
    for kind, sel in (("+inf", lambda t: t == float("inf")),
                      ("-inf", lambda t: t == float("-inf")),
                      ("nan", lambda t: t != t)):
        ma, mr = sel(ans), sel(ref)
        if not torch.equal(ma, mr):
            if verbose:
                print(f"{name}: {kind} positions differ ({int(ma.sum())} vs {int(mr.sum())})")
            ok = False
        ans[ma] = 0.0
        ref[mr] = 0.0
    if not ok:
        return False

    err = (ans - ref).abs()
    rel = err / (ref.abs() + 1e-6)
    good = (err < abs_tol) | (rel < rel_tol)
    if not bool(good.all()):
        if verbose:
            bad = (~good).flatten().nonzero()[:1]
            i = int(bad[0]) if bad.numel() else 0
            print(f"{name}: {int((~good).sum())}/{good.numel()} elements out of tolerance; "
                  f"max abs {float(err.max()):.3e}; first bad flat idx {i}: "
                  f"{float(ans.flatten()[i])} vs {float(ref.flatten()[i])}")
        return False
    cd = cosine_diff(ans, ref)
    if abs(cd) > cos_diff_tol:
        if verbose:
            print(f"{name}: cosine diff {cd:.3e} > {cos_diff_tol:.3e}")
        return False
    return True


def max_abs_diff(ans: torch.Tensor, ref: torch.Tensor) -> float:
    """Largest |ans-ref| over finite reference positions; infinities must match."""
    a = ans.detach().to("cpu", torch.float32)
    r = ref.detach().to("cpu", torch.float32)
    fin = torch.isfinite(r)
    if not torch.equal(a[~fin], r[~fin]) and not (a[~fin] != a[~fin]).all():
        return float("inf")
    if fin.sum() == 0:
        return 0.0
    return float((a[fin] - r[fin]).abs().max())
