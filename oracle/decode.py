"""MLA decode oracle: dense BF16 paged KV and sparse (top-k) attention
(test infrastructure only).

``decode_ref`` restates ``reference_torch`` of tests/test_flash_mla_decoding.py:124-205
(fp32 math, output rounded to bf16, natural-log LSE, +inf / zero rows where no
key can be attended).  ``decode_sparse_physical_ref`` states the same softmax
over the *physical* cache slots the public API receives (README.md:176), so a
kernel can be checked without the logical->physical map.
``fallback_ref`` restates flash_mla/flash_mla_interface.py:166-248, the torch path
the reference runs on a CPU (non-causal / s_q == 1 cases only: its causal mask
is top-left aligned, unlike the kernels and the tests).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch


def cdiv(a: int, b: int) -> int:
    return (a + b - 1) // b


def _attend(query: torch.Tensor, kv: torch.Tensor, dv: int, mask: Optional[torch.Tensor],
            softmax_scale: Optional[float]) -> Tuple[torch.Tensor, torch.Tensor]:
    """query [h_q, s_q, d] , kv [h_kv, s_k, d]; mask [s_q, s_k] bool (True = keep)."""
    h_q, h_kv = query.shape[0], kv.shape[0]
    query = query.float()
    kv = kv.float()
    if h_kv != 1:
        kv = kv.repeat_interleave(h_q // h_kv, dim=0)        # :155-156
    kv = torch.where(kv != kv, torch.zeros_like(kv), kv)      # NaN -> 0, :157
    w = query @ kv.transpose(-2, -1)                          # [h_q, s_q, s_k]
    if mask is not None:
        w = w.masked_fill(mask.logical_not().unsqueeze(0), float("-inf"))   # :159-169
    scale = (1.0 / math.sqrt(query.shape[-1])) if softmax_scale is None else softmax_scale
    w = w * scale                                             # :170
    lse = torch.logsumexp(w, dim=-1)                          # :171
    p = torch.softmax(w, dim=-1, dtype=torch.float32)
    out = p @ kv[..., :dv]
    lonely = lse == float("-inf")                             # :175-178
    out = out.masked_fill(lonely.unsqueeze(-1), 0.0)
    lse = lse.masked_fill(lonely, float("inf"))
    return out, lse


def decode_ref(cache_seqlens: torch.Tensor, block_table: torch.Tensor, q: torch.Tensor,
               blocked_k: torch.Tensor, dv: int, is_causal: bool,
               abs_indices: Optional[torch.Tensor] = None,
               softmax_scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """q [b, s_q, h_q, d]; blocked_k [num_blocks, block, h_kv, d] (already
    de-quantised for FP8 caches); abs_indices [b, s_q, topk] = LOGICAL token
    positions, -1 = padding.  Returns (out bf16 [b,s_q,h_q,dv], lse fp32 [b,h_q,s_q])."""
    b, s_q, h_q, d = q.shape
    block = blocked_k.shape[1]
    h_kv = blocked_k.shape[2]
    out = torch.empty(b, s_q, h_q, dv, dtype=torch.float32)
    lse = torch.empty(b, h_q, s_q, dtype=torch.float32)
    lens = cache_seqlens.to("cpu")
    for i in range(b):
        L = int(lens[i])
        nblk = cdiv(L, block)
        pages = block_table[i, :nblk].long()
        kv = blocked_k[pages].reshape(-1, h_kv, d)[:L]        # :191-193
        mask = None
        if (is_causal and s_q > 1) or abs_indices is not None:
            mask = torch.ones(s_q, L, dtype=torch.bool)
            if is_causal:
                assert abs_indices is None
                mask = mask.tril(diagonal=L - s_q)            # bottom-right aligned, :163
            if abs_indices is not None:
                sel = torch.zeros(s_q, L, dtype=torch.bool)
                for r in range(s_q):
                    idx = abs_indices[i, r]
                    sel[r, idx[idx != -1].long()] = True      # :133-139
                mask &= sel
        o, l = _attend(q[i].transpose(0, 1), kv.transpose(0, 1), dv, mask, softmax_scale)
        out[i] = o.transpose(0, 1)
        lse[i] = l
    # the result takes the dtype of q (bf16, or fp16 for fp16 inputs), tests/test_flash_mla_decoding.py:347-359
    return out.to(q.dtype if q.dtype in (torch.bfloat16, torch.float16) else torch.bfloat16), lse


def decode_sparse_physical_ref(q: torch.Tensor, blocked_k: torch.Tensor, indices: torch.Tensor,
                               dv: int, softmax_scale: Optional[float] = None
                               ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sparse decode stated on physical slots: indices [b, s_q, topk] hold
    page*block + offset into ``blocked_k`` (h_kv == 1), or -1 / out-of-range for
    padding.  Duplicated slots count once each (the reference generator never
    produces duplicates).  Same outputs as ``decode_ref``."""
    b, s_q, h_q, d = q.shape
    flat = blocked_k.reshape(-1, d).float()
    flat = torch.where(flat != flat, torch.zeros_like(flat), flat)
    n_slots = flat.shape[0]
    scale = (1.0 / math.sqrt(d)) if softmax_scale is None else softmax_scale
    out = torch.empty(b, s_q, h_q, dv, dtype=torch.float32)
    lse = torch.empty(b, h_q, s_q, dtype=torch.float32)
    for i in range(b):
        for r in range(s_q):
            idx = indices[i, r].long()
            valid = (idx >= 0) & (idx < n_slots)
            rows = flat[idx.clamp(0, n_slots - 1)]            # [topk, d]
            w = (q[i, r].float() @ rows.t())                  # [h_q, topk]
            w = w.masked_fill(valid.logical_not().unsqueeze(0), float("-inf")) * scale
            l = torch.logsumexp(w, dim=-1)
            p = torch.softmax(w, dim=-1, dtype=torch.float32)
            o = p @ rows[:, :dv]
            lonely = l == float("-inf")
            out[i, r] = o.masked_fill(lonely.unsqueeze(-1), 0.0)
            lse[i, :, r] = l.masked_fill(lonely, float("inf"))
    return out.to(torch.bfloat16), lse


def fallback_ref(q: torch.Tensor, k_cache: torch.Tensor, block_table: torch.Tensor,
                 cache_seqlens: torch.Tensor, head_dim_v: int,
                 softmax_scale: Optional[float] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """The reference's CPU-runnable torch path for dense, non-causal decode
    (flash_mla/flash_mla_interface.py:166-248): per request, gather pages, fp32
    scores * scale, logsumexp / softmax, P@V, cast to q.dtype."""
    b, s_q, h_q, d = q.shape
    block = k_cache.shape[1]
    h_kv = k_cache.shape[2]
    scale = d ** -0.5 if softmax_scale is None else softmax_scale
    out = torch.empty(b, s_q, h_q, head_dim_v, dtype=q.dtype)
    lse = torch.empty(b, h_q, s_q, dtype=torch.float32)
    kf = k_cache.float()
    for i in range(b):
        L = int(cache_seqlens[i])
        if L == 0:                                            # :208-211
            out[i].zero_()
            lse[i].fill_(float("inf"))
            continue
        pages = block_table[i, :cdiv(L, block)].long()
        kv = kf[pages].reshape(-1, h_kv, d)[:L].transpose(0, 1)     # [h_kv, L, d]
        if h_kv != 1:
            kv = kv.repeat_interleave(h_q // h_kv, dim=0)
        qq = q[i].transpose(0, 1).float()                     # [h_q, s_q, d]
        w = (qq @ kv.transpose(-2, -1)) * scale
        l = torch.logsumexp(w, dim=-1)
        p = torch.softmax(w, dim=-1, dtype=torch.float32)
        o = p @ kv[..., :head_dim_v]
        out[i] = o.transpose(0, 1).to(q.dtype)
        lse[i] = l
    return out, lse
