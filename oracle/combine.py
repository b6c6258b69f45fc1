"""Split-KV combine oracle (test infrastructure only).

Restates csrc/smxx/mla_combine.cu:71-107 (merge of base-2 log-sum-exps) and
:128-151 (weighted sum of normalised fp32 partial outputs).
"""
from __future__ import annotations

import math

import torch


def combine_ref(lse_accum: torch.Tensor, o_accum: torch.Tensor):
    """lse_accum [n, rows] base-2 (-inf = empty part); o_accum [n, rows, dv] fp32.

    Returns (o [rows, dv] fp32, lse [rows] natural log; +inf where every part is
    empty, and the output row is then 0).
    """
    lse_accum = lse_accum.float()
    o_accum = o_accum.float()
    mx = lse_accum.max(dim=0).values
    mx = torch.where(torch.isinf(mx) & (mx < 0), torch.zeros_like(mx), mx)   # :86
    s = torch.exp2(lse_accum - mx).sum(dim=0)                                # :89-94
    glse = torch.where((s == 0) | torch.isnan(s), torch.full_like(s, float("inf")),
                       torch.log2(s) + mx)                                   # :96
    w = torch.exp2(lse_accum - glse)                                         # :102-104
    w = torch.where(torch.isnan(w), torch.zeros_like(w), w)
    o = (w.unsqueeze(-1) * torch.where(w.unsqueeze(-1) != 0, o_accum, torch.zeros_like(o_accum))).sum(dim=0)
    return o, glse / math.log2(math.e)                                       # :98
