"""Sparse MLA prefill oracle (test infrastructure only).

Restates ``reference_torch`` of tests/test_flash_mla_prefill.py:72-90 and the
definition in README.md:201-217: logits are q.k * sm_scale * log2(e); an index
< 0 or >= s_kv is masked; ``max_logits`` and ``lse`` are in base 2; rows with no
valid index give out = 0 (NaN in the reference's 0*inf arithmetic is replaced
by the kernel contract: out 0, max_logits -inf, lse -inf,
csrc/sm100/prefill/sparse/fwd.cu:399-417, 438-445).
"""
from __future__ import annotations

import math
from typing import Tuple

import torch


def sparse_prefill_ref(q: torch.Tensor, kv: torch.Tensor, indices: torch.Tensor,
                       sm_scale: float, d_v: int = 512
                       ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """q [s_q, h_q, d_qk]; kv [s_kv, 1, d_qk]; indices [s_q, 1, topk] int32.
    Returns (out fp32 [s_q, h_q, d_v], max_logits [s_q, h_q], lse [s_q, h_q])."""
    s_q, h_q, d_qk = q.shape
    s_kv = kv.shape[0]
    idx = indices[:, 0, :].long()
    bad = (idx < 0) | (idx >= s_kv)                                   # :78
    qs = q.float()
    kvs = kv[:, 0, :].float()
    g = kvs.index_select(0, idx.masked_fill(bad, 0).flatten()).view(s_q, -1, d_qk)   # :82
    p = qs @ g.transpose(1, 2)                                        # [s_q, h_q, topk]
    p = p.masked_fill(bad.unsqueeze(1), float("-inf"))
    p = p * (sm_scale * math.log2(math.e))                            # :85
    max_logits = p.max(dim=-1).values
    lse = torch.logsumexp(p * math.log(2.0), dim=-1) * math.log2(math.e)   # :73-74
    w = torch.exp2(p - lse.unsqueeze(-1))
    empty = bad.all(dim=-1)                                           # rows with nothing to attend
    w = torch.where(empty.view(-1, 1, 1), torch.zeros_like(w), w)
    out = w @ g[:, :, :d_v]
    return out, max_logits, lse
