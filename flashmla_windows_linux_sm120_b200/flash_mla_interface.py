"""Public Python API: the same functions, argument meaning, defaults, shapes and
error behaviour as the reference's flash_mla/flash_mla_interface.py, routed to
the sm_100a kernels only.  There is no torch/CPU fallback: the reference sends
every non-"sm120" build to `_fallback_flash_mla_with_kvcache`
(flash_mla_interface.py:147-149, 286-297); here a missing or failing CUDA
library raises.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import cuda_sm100 as flash_mla_cuda

FLASH_MLA_LOADED_VARIANT = flash_mla_cuda.__flash_mla_variant__
TILE_SCHEDULER_METADATA_SIZE = 8


def get_mla_metadata(cache_seqlens: torch.Tensor, num_q_tokens_per_head_k: int, num_heads_k: int,
                     num_heads_q: Optional[int] = None, is_fp8_kvcache: bool = False,
                     topk: Optional[int] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Split-KV schedule for a decode batch (reference: flash_mla_interface.py:116-163).

    cache_seqlens: (batch,) int32.  num_q_tokens_per_head_k = s_q * num_heads_q // num_heads_k.
    topk: if given, sparse attention is scheduled (every request has `topk` tokens).
    Returns (tile_scheduler_metadata (num_sm_parts, 8) int32, num_splits (batch+1,) int32).
    """
    md, ns = flash_mla_cuda.get_mla_decoding_metadata(cache_seqlens, num_q_tokens_per_head_k, num_heads_k,
                                                      num_heads_q, is_fp8_kvcache, topk)
    return md, ns


def flash_mla_with_kvcache(q: torch.Tensor, k_cache: torch.Tensor, block_table: torch.Tensor,
                           cache_seqlens: torch.Tensor, head_dim_v: int, tile_scheduler_metadata: torch.Tensor,
                           num_splits: torch.Tensor, softmax_scale: Optional[float] = None, causal: bool = False,
                           is_fp8_kvcache: bool = False, indices: Optional[torch.Tensor] = None
                           ) -> Tuple[torch.Tensor, torch.Tensor]:
    """MLA decode over a paged KV cache (reference: flash_mla_interface.py:251-312).

    q (b, s_q, h_q, 576); k_cache (num_blocks, 64, h_k, 576) bf16, or (num_blocks, 64, 1, 656)
    FP8 records when is_fp8_kvcache; block_table (b, max_blocks) int32; cache_seqlens (b,) int32;
    indices (b, s_q, topk) int32 physical slots (page*64 + offset), -1 / out-of-range = padding.
    Returns (out (b, s_q, h_q, head_dim_v), softmax_lse (b, h_q, s_q) fp32).
    """
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    if indices is not None:
        assert causal == False, "causal must be `false` if sparse attention is enabled."  # noqa: E712
    out, lse = flash_mla_cuda.fwd_kvcache_mla(q, k_cache, head_dim_v, cache_seqlens, block_table, softmax_scale,
                                              causal, tile_scheduler_metadata, num_splits, is_fp8_kvcache, indices)
    return out, lse


def flash_mla_sparse_decode_logical_indices(q: torch.Tensor, k_cache: torch.Tensor, block_table: torch.Tensor,
                                            cache_seqlens: torch.Tensor, head_dim_v: int,
                                            tile_scheduler_metadata: torch.Tensor, num_splits: torch.Tensor,
                                            indices: torch.Tensor, softmax_scale: Optional[float] = None
                                            ) -> Tuple[torch.Tensor, torch.Tensor]:
    """Sparse FP8 decode whose `indices` (b, s_q, topk) hold token POSITIONS of each request (what a top-k indexer
    produces; < 0 or >= cache_seqlens[b] = padding) instead of physical slots: the kernel maps them through
    block_table itself, which saves the caller's remap (README.md:176 of the reference).  No counterpart in the
    reference API; everything else as flash_mla_with_kvcache(..., is_fp8_kvcache=True)."""
    if softmax_scale is None:
        softmax_scale = q.shape[-1] ** (-0.5)
    out, lse = flash_mla_cuda.fwd_kvcache_mla(q, k_cache, head_dim_v, cache_seqlens, block_table, softmax_scale,
                                              False, tile_scheduler_metadata, num_splits, True, indices,
                                              indices_logical=True)
    return out, lse


def flash_mla_sparse_fwd(q: torch.Tensor, kv: torch.Tensor, indices: torch.Tensor, sm_scale: float,
                         d_v: int = 512) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Sparse attention prefill (reference: flash_mla_interface.py:315-342).

    q [s_q, h_q, 576] bf16; kv [s_kv, 1, 576] bf16; indices [s_q, 1, topk] int32 (-1 or >= s_kv = padding).
    Returns (output [s_q, h_q, d_v] bf16, max_logits [s_q, h_q] fp32, lse [s_q, h_q] fp32 base-2).
    """
    out, max_logits, lse = flash_mla_cuda.sparse_prefill_fwd(q, kv, indices, sm_scale, d_v)
    return out, max_logits, lse


def _flash_attn_varlen_forward(q, k, v, cu_seqlens_qo, cu_seqlens_kv, max_seqlen_qo, max_seqlen_kv,
                               out=None, lse=None, causal=False, softmax_scale=None, is_varlen=True):
    """reference: flash_mla_interface.py:345-389 (without its unused 32 MiB workspace allocation)."""
    total_q, h_q, d_qk = q.shape
    _, _, d_vo = v.shape
    if softmax_scale is None:
        softmax_scale = d_qk ** (-0.5)
    if out is None:
        out = torch.empty(total_q, h_q, d_vo, device=q.device, dtype=q.dtype)
    if lse is None:
        lse = torch.empty(h_q, total_q, device=q.device, dtype=torch.float32).T   # contiguous along tokens
    flash_mla_cuda.dense_prefill_fwd(None, q, k, v, cu_seqlens_qo, cu_seqlens_kv, out, lse, 1 if causal else 0,
                                     softmax_scale, max_seqlen_qo, max_seqlen_kv, is_varlen)
    return out, lse


def _flash_attn_varlen_backward(do, q, k, v, out, lse, cu_seqlens_qo, cu_seqlens_kv, max_seqlen_qo, max_seqlen_kv,
                                dq=None, dk=None, dv=None, causal=False, softmax_scale=None, is_varlen=True):
    """reference: flash_mla_interface.py:392-456."""
    total_q, h_q, d_qk = q.shape
    total_k, h_k, d_vo = v.shape
    if h_q != h_k:
        raise ValueError(f"SM100 bwd doesn't support GQA now. num_qo_heads: {h_q}, num_kv_heads: {h_k}.")
    if softmax_scale is None:
        softmax_scale = d_qk ** (-0.5)
    if dq is None:
        dq = torch.empty(total_q, h_q, d_qk, device=q.device, dtype=q.dtype)
    if dk is None:
        dk = torch.empty(total_k, h_k, d_qk, device=q.device, dtype=q.dtype)
    if dv is None:
        dv = torch.empty(total_k, h_k, d_vo, device=q.device, dtype=q.dtype)
    ws_bytes = flash_mla_cuda.lib.fmla_dense_bwd_workspace_bytes(total_q, h_q, d_qk)
    workspace = torch.empty(ws_bytes, dtype=torch.uint8, device=q.device)
    if do.stride(-1) != 1:
        do = do.contiguous()
    flash_mla_cuda.dense_prefill_bwd(workspace, do, q, k, v, out, lse, cu_seqlens_qo, cu_seqlens_kv, dq, dk, dv,
                                     1 if causal else 0, softmax_scale, max_seqlen_qo, max_seqlen_kv, is_varlen)
    return dq, dk, dv


class FlashAttnVarlenFunc(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, cu_seqlens_qo, cu_seqlens_kv, max_seqlen_qo, max_seqlen_kv, causal=False,
                softmax_scale=None, is_varlen=True):
        out, lse = _flash_attn_varlen_forward(q, k, v, cu_seqlens_qo, cu_seqlens_kv, max_seqlen_qo, max_seqlen_kv,
                                              causal=causal, softmax_scale=softmax_scale, is_varlen=is_varlen)
        ctx.save_for_backward(q, k, v, out, lse, cu_seqlens_qo, cu_seqlens_kv)
        ctx.max_seqlen_qo, ctx.max_seqlen_kv = max_seqlen_qo, max_seqlen_kv
        ctx.causal, ctx.softmax_scale, ctx.is_varlen = causal, softmax_scale, is_varlen
        ctx.mark_non_differentiable(lse)
        return out, lse

    @staticmethod
    def backward(ctx, do, dlse):
        del dlse  # LSE has no gradient, as in the reference
        q, k, v, out, lse, cu_q, cu_k = ctx.saved_tensors
        dq, dk, dv = _flash_attn_varlen_backward(do, q, k, v, out, lse, cu_q, cu_k, ctx.max_seqlen_qo,
                                                 ctx.max_seqlen_kv, causal=ctx.causal,
                                                 softmax_scale=ctx.softmax_scale, is_varlen=ctx.is_varlen)
        return dq, dk, dv, None, None, None, None, None, None, None


def flash_attn_varlen_func(q, k, v, cu_seqlens_qo, cu_seqlens_kv, max_seqlen_qo, max_seqlen_kv, dropout_p=0.0,
                           softmax_scale=None, causal=False, deterministic=False, is_varlen=True):
    """Dense varlen MHA, forward + autograd backward (reference: flash_mla_interface.py:503-523).
    Returns (out [total_q, h, d_v], lse [total_q, h] natural log)."""
    assert dropout_p == 0.0
    del deterministic   # accepted: the backward here is always bitwise reproducible (the reference asserts False)
    return FlashAttnVarlenFunc.apply(q, k, v, cu_seqlens_qo, cu_seqlens_kv, max_seqlen_qo, max_seqlen_kv, causal,
                                     softmax_scale, is_varlen)


def flash_attn_varlen_qkvpacked_func(qkv, cu_seqlens, max_seqlen, head_dim_qk, dropout_p=0.0, softmax_scale=None,
                                     causal=False, deterministic=False, is_varlen=True):
    """reference: flash_mla_interface.py:526-545.  qkv [total, h, 2*head_dim_qk + d_v]."""
    assert dropout_p == 0.0
    del deterministic   # accepted: the backward here is always bitwise reproducible (the reference asserts False)
    return FlashAttnVarlenFunc.apply(qkv[:, :, :head_dim_qk], qkv[:, :, head_dim_qk:head_dim_qk * 2],
                                     qkv[:, :, head_dim_qk * 2:], cu_seqlens, cu_seqlens, max_seqlen, max_seqlen,
                                     causal, softmax_scale, is_varlen)


def flash_attn_varlen_kvpacked_func(q, kv, cu_seqlens_qo, cu_seqlens_kv, max_seqlen_qo, max_seqlen_kv, head_dim_qk,
                                    dropout_p=0.0, softmax_scale=None, causal=False, deterministic=False,
                                    is_varlen=True):
    """reference: flash_mla_interface.py:548-566.  kv [total_k, h_k, head_dim_qk + d_v]."""
    assert dropout_p == 0.0
    del deterministic   # accepted: the backward here is always bitwise reproducible (the reference asserts False)
    return FlashAttnVarlenFunc.apply(q, kv[:, :, :head_dim_qk], kv[:, :, head_dim_qk:], cu_seqlens_qo, cu_seqlens_kv,
                                     max_seqlen_qo, max_seqlen_kv, causal, softmax_scale, is_varlen)
