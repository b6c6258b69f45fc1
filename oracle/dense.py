"""Dense varlen MHA forward/backward oracle (test infrastructure only).

Restates tests/test_fmha_sm100.py:19-44 (bias mask + fp32 sdpa) and :99-115 (the
per-sequence loop); gradients come from torch autograd through the same fp32
graph, as the reference test obtains them (:135-140).  Causal masking is
bottom-right aligned: query i of a sequence with s_q queries and s_k keys sees
keys j <= i + (s_k - s_q) (:19-23).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch


def attn_bias(s_q: int, s_k: int, causal: bool) -> torch.Tensor:
    bias = torch.zeros(s_q, s_k, dtype=torch.float32)
    if causal:
        keep = torch.ones(s_q, s_k, dtype=torch.bool).tril(diagonal=s_k - s_q)
        bias.masked_fill_(keep.logical_not(), float("-inf"))
    return bias


def _sdpa(q, k, v, bias, scale):
    """q [s_q, h, d], k [s_k, h_k, d], v [s_k, h_k, dv] -> (out [s_q,h,dv], lse [s_q,h])."""
    h, h_k = q.shape[1], k.shape[1]
    qq = q.float().transpose(0, 1)
    kk = k.float().transpose(0, 1).repeat_interleave(h // h_k, dim=0)
    vv = v.float().transpose(0, 1).repeat_interleave(h // h_k, dim=0)
    w = (qq @ kk.transpose(-2, -1)) * scale + bias
    lse = w.logsumexp(dim=-1)
    p = torch.softmax(w, dim=-1, dtype=torch.float32)
    # rows with no visible key: softmax gives NaN; the kernels define out = 0, lse = -inf
    p = torch.where(torch.isnan(p), torch.zeros_like(p), p)
    return (p @ vv).transpose(0, 1), lse.transpose(0, 1)


def dense_fwd_ref(q, k, v, cu_q, cu_k, causal: bool, softmax_scale: Optional[float] = None
                  ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Packed varlen inputs; returns (out fp32 [Tq, h, dv], lse fp32 [Tq, h])."""
    scale = q.shape[-1] ** -0.5 if softmax_scale is None else softmax_scale
    outs, lses = [], []
    for i in range(len(cu_q) - 1):
        a, b = int(cu_q[i]), int(cu_q[i + 1])
        c, d = int(cu_k[i]), int(cu_k[i + 1])
        o, l = _sdpa(q[a:b], k[c:d], v[c:d], attn_bias(b - a, d - c, causal), scale)
        outs.append(o)
        lses.append(l)
    return torch.cat(outs), torch.cat(lses)


def dense_fwd_bwd_ref(q, k, v, d_out, cu_q, cu_k, causal: bool,
                      softmax_scale: Optional[float] = None):
    """Returns (out, lse, dq, dk, dv), all fp32, gradients w.r.t. the fp32 graph."""
    q2 = q.detach().float().requires_grad_()
    k2 = k.detach().float().requires_grad_()
    v2 = v.detach().float().requires_grad_()
    out, lse = dense_fwd_ref(q2, k2, v2, cu_q, cu_k, causal, softmax_scale)
    out.backward(d_out.float())
    return out.detach(), lse.detach(), q2.grad, k2.grad, v2.grad
