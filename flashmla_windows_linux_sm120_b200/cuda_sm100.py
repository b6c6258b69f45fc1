"""The "extension module" the public interface calls: same five functions, same
positional signatures and return conventions as the module csrc/pybind.cpp
builds in the reference (:870-911), implemented as a thin marshalling layer
over the C ABI.  Tensors are allocated with torch (device memory, streams);
everything else happens inside libflashmla_b200.so.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional

import torch

from . import _cabi
from ._cabi import DecodeParams, DenseParams, SparsePrefillParams, check, lib

__flash_mla_variant__ = lib.fmla_variant().decode()
TILE_SCHEDULER_METADATA_SIZE = 8


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


# Arrival counters of the in-kernel merge of split requests (fmla_decode_params.arrival_counters): zero on entry,
# left zero by the kernel, so one array per (device, stream) is allocated once and reused -- calls on one stream
# are ordered, calls on different streams get different arrays.
_arrival_counters = {}
_MERGE_IN_KERNEL_DEFAULT = os.environ.get("FMLA_MERGE_IN_KERNEL", "0") == "1"


def _counters_for(t: torch.Tensor, n: int) -> torch.Tensor:
    key = (t.device.index, _stream(t))
    buf = _arrival_counters.get(key)
    if buf is None or buf.numel() < n:
        buf = torch.zeros((max(n, 4096),), dtype=torch.int32, device=t.device)
        _arrival_counters[key] = buf
    return buf


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _cuda(t: torch.Tensor, name: str) -> None:
    _require(t.is_cuda, f"{name} must be on CUDA")


def get_mla_decoding_metadata(seqlens_k: torch.Tensor, num_q_tokens_per_head_k: int, h_k: int,
                              h_q: Optional[int] = None, is_fp8_kvcache: bool = False,
                              topk: Optional[int] = None) -> List[torch.Tensor]:
    """csrc/pybind.cpp:383-428.  Returns [tile_scheduler_metadata int32[num_sm_parts, 8], num_splits int32[b+1]]."""
    is_sparse = topk is not None
    _cuda(seqlens_k, "seqlens_k")
    _require(seqlens_k.is_contiguous(), "seqlens_k must be contiguous")
    _require(seqlens_k.dtype == torch.int32, "seqlens_k must have dtype int32")
    if is_sparse:
        _require(h_q is not None, "num_heads_q must be provided when topk is provided")
    n = C.c_int(0)
    check(lib.fmla_get_num_sm_parts(seqlens_k.device.index or 0, int(num_q_tokens_per_head_k), int(h_k),
                                    int(h_q) if h_q is not None else 0, int(bool(is_fp8_kvcache)), int(is_sparse),
                                    C.byref(n)))
    b = seqlens_k.shape[0]
    with torch.cuda.device(seqlens_k.device):
        md = torch.empty((n.value, TILE_SCHEDULER_METADATA_SIZE), dtype=torch.int32, device=seqlens_k.device)
        ns = torch.empty((b + 1,), dtype=torch.int32, device=seqlens_k.device)
        check(lib.fmla_get_mla_metadata(seqlens_k.data_ptr(), b, n.value, int(topk) if is_sparse else -1,
                                        md.data_ptr(), ns.data_ptr(), _stream(seqlens_k)))
    return [md, ns]


def fwd_kvcache_mla(q: torch.Tensor, kcache: torch.Tensor, head_size_v: int, seqlens_k: torch.Tensor,
                    block_table: torch.Tensor, softmax_scale: float, is_causal: bool,
                    tile_scheduler_metadata: torch.Tensor, num_splits: torch.Tensor, is_fp8: bool = False,
                    indices: Optional[torch.Tensor] = None, profile_events=None,
                    indices_logical: bool = False, merge_in_kernel: Optional[bool] = None) -> List[torch.Tensor]:
    """csrc/pybind.cpp:430-720.  Returns [out [b,s_q,h_q,dv] (q dtype), softmax_lse [b,h_q,s_q] fp32].
    profile_events: optional (begin, end) pair of torch.cuda.Event(enable_timing=True) recorded around the
    attention kernel alone (they must have been recorded once already so that their handles exist).
    merge_in_kernel: dense decode with a multiple of 128 heads per kv head only -- the CTA that delivers the last
    partial of a split request merges it (one kernel per step) instead of a second, dependent-launched merge kernel.
    Default: the environment variable FMLA_MERGE_IN_KERNEL=1, else off (the inline merge stalls the pipeline of the
    merging CTA for longer than the separate kernel takes)."""
    sparse = indices is not None
    _require(q.dtype in (torch.bfloat16, torch.float16), "q must be bfloat16 or float16")
    if not is_fp8:
        _require(kcache.dtype == q.dtype, "query and key must have the same dtype")
    else:
        _require(kcache.dtype in (torch.float8_e4m3fn, torch.int8, torch.uint8),
                 "key must have dtype fp8_e4m3fn or int8 or uint8")
    _require(seqlens_k.dtype == torch.int32, "seqlens_k must have dtype int32")
    _require(block_table.dtype == torch.int32, "block_table must have dtype torch.int32")
    _require(tile_scheduler_metadata.dtype == torch.int32, "tile_scheduler_metadata must have dtype int32")
    _require(num_splits.dtype == torch.int32, "num_splits must have dtype int32")
    _require(not sparse or indices.dtype == torch.int32, "indices must have dtype int32")
    for t, n in ((q, "q"), (kcache, "kcache"), (seqlens_k, "seqlens_k"), (block_table, "block_table"),
                 (tile_scheduler_metadata, "tile_scheduler_metadata"), (num_splits, "num_splits")):
        _cuda(t, n)
    if sparse:
        _cuda(indices, "indices")
    _require(q.dim() == 4 and kcache.dim() == 4, "q and kcache must be 4-D")
    _require(q.stride(-1) == 1, "q must have contiguous last dimension")
    _require(kcache.stride(-1) == 1, "kcache must have contiguous last dimension")
    _require(seqlens_k.is_contiguous(), "seqlens_k must be contiguous")
    _require(block_table.stride(-1) == 1, "block_table must have contiguous last dimension")
    _require(tile_scheduler_metadata.is_contiguous() and num_splits.is_contiguous(),
             "tile_scheduler_metadata and num_splits must be contiguous")
    _require(not sparse or indices.stride(-1) == 1, "indices must have contiguous last dimension")

    b, s_q, h_q, d = q.shape
    num_blocks, page, h_k, last = kcache.shape
    _require(tile_scheduler_metadata.dim() == 2 and tile_scheduler_metadata.shape[1] == TILE_SCHEDULER_METADATA_SIZE,
             "tile_scheduler_metadata must be [num_sm_parts, 8]")
    _require(tuple(seqlens_k.shape) == (b,), "seqlens_k must be [batch]")
    _require(tuple(num_splits.shape) == (b + 1,), "num_splits must be [batch + 1]")
    _require(block_table.dim() == 2 and block_table.shape[0] == b, "block_table must be [batch, max_blocks]")
    if is_fp8:
        _require(last == 656, "FP8 kcache must have 656 bytes per token")
    else:
        _require(last == d, "kcache head dim must equal q head dim")
    topk = -1
    if sparse:
        _require(indices.dim() == 3 and indices.shape[0] == b and indices.shape[1] == s_q, "indices must be [b, s_q, topk]")
        topk = indices.shape[2]
    if q.dtype == torch.float16 and (sparse or is_fp8):
        raise RuntimeError("flashmla_b200: unsupported configuration: float16 queries are supported for the dense "
                           "(float16 cache) decode only")

    num_sm_parts = tile_scheduler_metadata.shape[0]
    with torch.cuda.device(q.device):
        out = torch.empty((b, s_q, h_q, head_size_v), dtype=q.dtype, device=q.device)
        lse = torch.empty((b, h_q, s_q), dtype=torch.float32, device=q.device)
        slots = b + num_sm_parts
        lse_accum = torch.empty((slots, s_q * h_q), dtype=torch.float32, device=q.device)
        o_accum = torch.empty((slots, s_q * h_q, head_size_v), dtype=torch.float32, device=q.device)
        p = DecodeParams()
        p.b, p.s_q, p.h_q, p.h_k, p.d, p.d_v = b, s_q, h_q, h_k, d, int(head_size_v)
        p.num_blocks, p.page_block_size = num_blocks, page
        p.is_causal, p.is_fp8, p.topk = int(bool(is_causal)), int(bool(is_fp8)), topk
        p.q_dtype = 1 if q.dtype == torch.float16 else 0
        p.softmax_scale = float(softmax_scale)
        p.q, p.q_stride_b, p.q_stride_s, p.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1), q.stride(2)
        p.kcache = kcache.data_ptr()
        p.k_stride_block, p.k_stride_row, p.k_stride_head = kcache.stride(0), kcache.stride(1), kcache.stride(2)
        p.block_table, p.block_table_stride_b = block_table.data_ptr(), block_table.stride(0)
        p.seqlens_k = seqlens_k.data_ptr()
        if sparse:
            p.indices, p.indices_stride_b, p.indices_stride_s = indices.data_ptr(), indices.stride(0), indices.stride(1)
            p.indices_logical = int(bool(indices_logical))
        p.tile_scheduler_metadata, p.num_sm_parts = tile_scheduler_metadata.data_ptr(), num_sm_parts
        p.num_splits = num_splits.data_ptr()
        p.out, p.o_stride_b, p.o_stride_s, p.o_stride_h = out.data_ptr(), out.stride(0), out.stride(1), out.stride(2)
        p.softmax_lse, p.lse_accum, p.o_accum = lse.data_ptr(), lse_accum.data_ptr(), o_accum.data_ptr()
        if merge_in_kernel is None:
            merge_in_kernel = _MERGE_IN_KERNEL_DEFAULT
        if merge_in_kernel and not sparse and (h_q // h_k) % 128 == 0:
            p.arrival_counters = _counters_for(q, b * s_q * (h_q // 64)).data_ptr()
        p.no_split_hint = int(_no_request_is_split(num_splits, b))
        if profile_events is not None:
            p.profile_event_begin = profile_events[0].cuda_event
            p.profile_event_end = profile_events[1].cuda_event
        check(lib.fmla_fwd_kvcache_mla(C.byref(p), _stream(q)))
    return [out, lse]


def _no_request_is_split(num_splits: torch.Tensor, b: int) -> bool:
    """True when the schedule gives every request to one partition (num_splits[b] == b): the merge kernel is then
    not launched.  Read back from the device once per metadata tensor (one synchronisation, remembered on the
    tensor object; a decode step reuses its metadata for every layer); unknown -- and therefore False -- while the
    stream is being captured into a CUDA graph before that first read."""
    known = getattr(num_splits, "_fmla_no_split", None)
    if known is None:
        if torch.cuda.is_current_stream_capturing():
            return False
        known = bool(int(num_splits[b].item()) == b)
        num_splits._fmla_no_split = known
    return known


def sparse_prefill_fwd(q: torch.Tensor, kv: torch.Tensor, indices: torch.Tensor, sm_scale: float,
                       d_v: int = 512) -> List[torch.Tensor]:
    """csrc/pybind.cpp:730-814.  Returns [out bf16 [s_q,h_q,d_v], max_logits fp32 [s_q,h_q], lse fp32 [s_q,h_q]]."""
    for t, n in ((q, "q"), (kv, "kv"), (indices, "indices")):
        _cuda(t, n)
    _require(q.dtype == torch.bfloat16 and kv.dtype == torch.bfloat16, "q and kv must be bfloat16")
    _require(indices.dtype == torch.int32, "indices must be int32")
    _require(q.dim() == 3 and kv.dim() == 3 and indices.dim() == 3, "q, kv, indices must be 3-D")
    _require(q.stride(-1) == 1 and kv.stride(-1) == 1 and indices.stride(-1) == 1, "last dimensions must be contiguous")
    s_q, h_q, d_qk = q.shape
    s_kv, h_kv, _ = kv.shape
    topk = indices.shape[2]
    _require(kv.shape[2] == d_qk, "q and kv head dims differ")
    _require(tuple(indices.shape[:2]) == (s_q, h_kv), "indices must be [s_q, h_kv, topk]")
    with torch.cuda.device(q.device):
        out = torch.empty((s_q, h_q, d_v), dtype=torch.bfloat16, device=q.device)
        mx = torch.empty((s_q, h_q), dtype=torch.float32, device=q.device)
        lse = torch.empty((s_q, h_q), dtype=torch.float32, device=q.device)
        p = SparsePrefillParams()
        p.s_q, p.s_kv, p.h_q, p.h_kv, p.d_qk, p.d_v, p.topk = s_q, s_kv, h_q, h_kv, d_qk, int(d_v), topk
        p.sm_scale = float(sm_scale)
        p.q, p.q_stride_s, p.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1)
        p.kv, p.kv_stride_s, p.kv_stride_h = kv.data_ptr(), kv.stride(0), kv.stride(1)
        p.indices, p.indices_stride_s, p.indices_stride_h = indices.data_ptr(), indices.stride(0), indices.stride(1)
        p.out, p.max_logits, p.lse = out.data_ptr(), mx.data_ptr(), lse.data_ptr()
        check(lib.fmla_sparse_prefill_fwd(C.byref(p), _stream(q)))
    return [out, mx, lse]


def _dense_params(q, k, v, cu_q, cu_k, o, lse, mask_mode_code, softmax_scale, max_q, max_k) -> DenseParams:
    for t, n in ((q, "q"), (k, "k"), (v, "v"), (cu_q, "cumulative_seqlen_q"), (cu_k, "cumulative_seqlen_kv"),
                 (o, "o"), (lse, "lse")):
        _cuda(t, n)
    _require(q.dtype == torch.bfloat16 and k.dtype == torch.bfloat16 and v.dtype == torch.bfloat16 and
             o.dtype == torch.bfloat16, "q, k, v, o must be bfloat16")
    _require(lse.dtype == torch.float32, "lse must be float32")
    _require(cu_q.dtype == torch.int32 and cu_k.dtype == torch.int32, "cumulative seqlens must be int32")
    _require(q.dim() == 3 and k.dim() == 3 and v.dim() == 3 and o.dim() == 3 and lse.dim() == 2, "bad ranks")
    _require(q.stride(-1) == 1 and k.stride(-1) == 1 and v.stride(-1) == 1 and o.stride(-1) == 1,
             "last dimensions must be contiguous")
    _require(cu_q.is_contiguous() and cu_k.is_contiguous(), "cumulative seqlens must be contiguous")
    p = DenseParams()
    p.batch = cu_q.shape[0] - 1
    p.total_q, p.h_q, p.d_qk = q.shape
    p.total_k, p.h_k, p.d_v = v.shape
    _require(k.shape[0] == v.shape[0] and k.shape[1] == v.shape[1] and k.shape[2] == q.shape[2], "k shape mismatch")
    _require(tuple(o.shape) == (q.shape[0], q.shape[1], v.shape[2]), "o shape mismatch")
    _require(tuple(lse.shape) == (q.shape[0], q.shape[1]), "lse must be [total_q, h_q]")
    p.max_seqlen_q, p.max_seqlen_k = int(max_q), int(max_k)
    p.is_causal = 1 if mask_mode_code == 1 else 0
    p.softmax_scale = float(softmax_scale)
    p.q, p.q_stride_t, p.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1)
    p.k, p.k_stride_t, p.k_stride_h = k.data_ptr(), k.stride(0), k.stride(1)
    p.v, p.v_stride_t, p.v_stride_h = v.data_ptr(), v.stride(0), v.stride(1)
    p.cu_seqlens_q, p.cu_seqlens_k = cu_q.data_ptr(), cu_k.data_ptr()
    p.o, p.o_stride_t, p.o_stride_h = o.data_ptr(), o.stride(0), o.stride(1)
    p.lse, p.lse_stride_t, p.lse_stride_h = lse.data_ptr(), lse.stride(0), lse.stride(1)
    return p


def dense_prefill_fwd(workspace_buffer, q, k, v, cumulative_seqlen_q, cumulative_seqlen_kv, o, lse,
                      mask_mode_code: int, softmax_scale: float, max_seqlen_q: int, max_seqlen_kv: int,
                      is_varlen: bool = True) -> None:
    """csrc/pybind.cpp:817-839.  Writes o and lse in place.  workspace_buffer is accepted and unused
    (the reference's forward does not use it either, fmha_cutlass_fwd_sm100.cuh:302-306)."""
    p = _dense_params(q, k, v, cumulative_seqlen_q, cumulative_seqlen_kv, o, lse, mask_mode_code, softmax_scale,
                      max_seqlen_q, max_seqlen_kv)
    with torch.cuda.device(q.device):
        check(lib.fmla_dense_prefill_fwd(C.byref(p), _stream(q)))


def dense_prefill_bwd(workspace_buffer, d_o, q, k, v, o, lse, cumulative_seqlen_q, cumulative_seqlen_kv,
                      dq, dk, dv, mask_mode_code: int, softmax_scale: float, max_seqlen_q: int,
                      max_seqlen_kv: int, is_varlen: bool = True) -> None:
    """csrc/pybind.cpp:841-867.  Writes dq, dk, dv in place."""
    p = _dense_params(q, k, v, cumulative_seqlen_q, cumulative_seqlen_kv, o, lse, mask_mode_code, softmax_scale,
                      max_seqlen_q, max_seqlen_kv)
    for t, n in ((d_o, "d_o"), (dq, "dq"), (dk, "dk"), (dv, "dv"), (workspace_buffer, "workspace_buffer")):
        _cuda(t, n)
        _require(t.stride(-1) == 1, f"{n} must have contiguous last dimension")
    _require(all(t.dtype == torch.bfloat16 for t in (d_o, dq, dk, dv)), "d_o, dq, dk, dv must be bfloat16")
    _require(tuple(d_o.shape) == tuple(o.shape) and tuple(dq.shape) == tuple(q.shape) and
             tuple(dk.shape) == tuple(k.shape) and tuple(dv.shape) == tuple(v.shape), "gradient shape mismatch")
    p.d_o, p.do_stride_t, p.do_stride_h = d_o.data_ptr(), d_o.stride(0), d_o.stride(1)
    p.dq, p.dq_stride_t, p.dq_stride_h = dq.data_ptr(), dq.stride(0), dq.stride(1)
    p.dk, p.dk_stride_t, p.dk_stride_h = dk.data_ptr(), dk.stride(0), dk.stride(1)
    p.dv, p.dv_stride_t, p.dv_stride_h = dv.data_ptr(), dv.stride(0), dv.stride(1)
    need = lib.fmla_dense_bwd_workspace_bytes(p.total_q, p.h_q, p.d_qk)
    _require(workspace_buffer.numel() * workspace_buffer.element_size() >= need,
             f"workspace_buffer too small: need {need} bytes")
    p.workspace, p.workspace_bytes = workspace_buffer.data_ptr(), workspace_buffer.numel() * workspace_buffer.element_size()
    with torch.cuda.device(q.device):
        check(lib.fmla_dense_prefill_bwd(C.byref(p), _stream(q)))


def combine_partials(lse_accum: torch.Tensor, o_accum: torch.Tensor):
    """Merge [num_parts, rows] base-2 LSEs and [num_parts, rows, 512] fp32 partial outputs.
    Returns (out bf16 [rows, 512], lse fp32 [rows] natural log)."""
    _require(lse_accum.is_cuda and o_accum.is_cuda and lse_accum.is_contiguous() and o_accum.is_contiguous(),
             "partials must be contiguous CUDA tensors")
    _require(lse_accum.dtype == torch.float32 and o_accum.dtype == torch.float32, "partials must be float32")
    n, rows = lse_accum.shape
    _require(tuple(o_accum.shape) == (n, rows, 512), "o_accum must be [num_parts, rows, 512]")
    with torch.cuda.device(o_accum.device):
        out = torch.empty((rows, 512), dtype=torch.bfloat16, device=o_accum.device)
        lse = torch.empty((rows,), dtype=torch.float32, device=o_accum.device)
        check(lib.fmla_combine_partials(lse_accum.data_ptr(), o_accum.data_ptr(), n, rows, 512, out.data_ptr(), 512,
                                        lse.data_ptr(), _stream(o_accum)))
    return out, lse


def quantize_kv_fp8(kv: torch.Tensor, cache: Optional[torch.Tensor] = None,
                    dst_slots: Optional[torch.Tensor] = None) -> torch.Tensor:
    """bf16 [n, 576] (or [num_blocks, 64, 1, 576]) -> FP8 records.  Without `cache` a fresh
    [*, 656] float8_e4m3fn tensor of the same leading shape is returned."""
    _require(kv.is_cuda and kv.dtype == torch.bfloat16 and kv.shape[-1] == 576, "kv must be CUDA bf16 [..., 576]")
    lead = kv.shape[:-1]
    flat = kv.reshape(-1, 576)
    _require(flat.stride(-1) == 1, "kv rows must be contiguous")
    with torch.cuda.device(kv.device):
        if cache is None:
            cache = torch.empty((*lead, 656), dtype=torch.float8_e4m3fn, device=kv.device)
        cflat = cache.view(torch.uint8).reshape(-1, 656)
        slots_ptr = None
        if dst_slots is not None:
            _require(dst_slots.is_cuda and dst_slots.dtype == torch.int32 and dst_slots.is_contiguous(),
                     "dst_slots must be a contiguous CUDA int32 tensor")
            slots_ptr = dst_slots.data_ptr()
        check(lib.fmla_quantize_kv_fp8(flat.data_ptr(), flat.stride(0), flat.shape[0], slots_ptr, cflat.data_ptr(),
                                       cflat.stride(0), _stream(kv)))
    return cache
