"""ctypes binding of libflashmla_b200.so (declarations: include/flashmla_b200.h).

The library is the only compute path: if it cannot be loaded the import of the
package fails; there is no Python / torch fallback.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libflashmla_b200.so")

i32, i64, f32, vp = C.c_int32, C.c_int64, C.c_float, C.c_void_p


class DecodeParams(C.Structure):
    _fields_ = [
        ("b", i32), ("s_q", i32), ("h_q", i32), ("h_k", i32), ("d", i32), ("d_v", i32),
        ("num_blocks", i32), ("page_block_size", i32), ("is_causal", i32), ("is_fp8", i32),
        ("topk", i32), ("q_dtype", i32), ("softmax_scale", f32),
        ("q", vp), ("q_stride_b", i64), ("q_stride_s", i64), ("q_stride_h", i64),
        ("kcache", vp), ("k_stride_block", i64), ("k_stride_row", i64), ("k_stride_head", i64),
        ("block_table", vp), ("block_table_stride_b", i64),
        ("seqlens_k", vp),
        ("indices", vp), ("indices_stride_b", i64), ("indices_stride_s", i64),
        ("tile_scheduler_metadata", vp), ("num_sm_parts", i32), ("num_splits", vp),
        ("out", vp), ("o_stride_b", i64), ("o_stride_s", i64), ("o_stride_h", i64),
        ("softmax_lse", vp), ("lse_accum", vp), ("o_accum", vp),
        ("profile_event_begin", vp), ("profile_event_end", vp),
        ("indices_logical", i32),
        ("arrival_counters", vp),
        ("no_split_hint", i32),
    ]


class SparsePrefillParams(C.Structure):
    _fields_ = [
        ("s_q", i32), ("s_kv", i32), ("h_q", i32), ("h_kv", i32), ("d_qk", i32), ("d_v", i32), ("topk", i32),
        ("sm_scale", f32),
        ("q", vp), ("q_stride_s", i64), ("q_stride_h", i64),
        ("kv", vp), ("kv_stride_s", i64), ("kv_stride_h", i64),
        ("indices", vp), ("indices_stride_s", i64), ("indices_stride_h", i64),
        ("out", vp), ("max_logits", vp), ("lse", vp),
    ]


class DenseParams(C.Structure):
    _fields_ = [
        ("batch", i32), ("total_q", i32), ("total_k", i32), ("h_q", i32), ("h_k", i32), ("d_qk", i32), ("d_v", i32),
        ("max_seqlen_q", i32), ("max_seqlen_k", i32), ("is_causal", i32), ("softmax_scale", f32),
        ("q", vp), ("q_stride_t", i64), ("q_stride_h", i64),
        ("k", vp), ("k_stride_t", i64), ("k_stride_h", i64),
        ("v", vp), ("v_stride_t", i64), ("v_stride_h", i64),
        ("cu_seqlens_q", vp), ("cu_seqlens_k", vp),
        ("o", vp), ("o_stride_t", i64), ("o_stride_h", i64),
        ("lse", vp), ("lse_stride_t", i64), ("lse_stride_h", i64),
        ("d_o", vp), ("do_stride_t", i64), ("do_stride_h", i64),
        ("dq", vp), ("dq_stride_t", i64), ("dq_stride_h", i64),
        ("dk", vp), ("dk_stride_t", i64), ("dk_stride_h", i64),
        ("dv", vp), ("dv_stride_t", i64), ("dv_stride_h", i64),
        ("workspace", vp), ("workspace_bytes", C.c_size_t),
    ]


class PeerPush(C.Structure):
    _fields_ = [("slot", i32), ("num_dst", i32), ("dst_o", vp * 8), ("dst_lse", vp * 8), ("dst_flag", vp * 8),
                ("epoch", C.c_uint32), ("counter", vp)]


# every symbol include/flashmla_b200.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "fmla_status_string": (C.c_char_p, [C.c_int]),
    "fmla_last_error_message": (C.c_char_p, []),
    "fmla_version": (C.c_char_p, []),
    "fmla_variant": (C.c_char_p, []),
    "fmla_get_num_sm_parts": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(C.c_int)]),
    "fmla_get_mla_metadata": (C.c_int, [vp, C.c_int, C.c_int, C.c_int, vp, vp, vp]),
    "fmla_decode_scratch_bytes": (C.c_int, [C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,
                                            C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
    "fmla_fwd_kvcache_mla": (C.c_int, [C.POINTER(DecodeParams), vp]),
    "fmla_fwd_kvcache_mla_static_scratch": (C.c_int, [C.POINTER(DecodeParams), vp]),
    "fmla_static_scratch_max_rows": (C.c_size_t, []),
    "fmla_fwd_kvcache_mla_push_partial": (C.c_int, [C.POINTER(DecodeParams), C.POINTER(PeerPush), vp]),
    "fmla_merge_peer_partials": (C.c_int, [vp, vp, C.c_int, C.c_int, C.c_int, vp, C.c_uint32, C.c_int, vp, i64, vp, vp]),
    "fmla_sizeof_peer_push": (C.c_size_t, []),
    "fmla_combine_partials": (C.c_int, [vp, vp, C.c_int, C.c_int, C.c_int, vp, i64, vp, vp]),
    "fmla_sparse_prefill_fwd": (C.c_int, [C.POINTER(SparsePrefillParams), vp]),
    "fmla_dense_prefill_fwd": (C.c_int, [C.POINTER(DenseParams), vp]),
    "fmla_dense_bwd_workspace_bytes": (C.c_size_t, [C.c_int, C.c_int, C.c_int]),
    "fmla_dense_prefill_bwd": (C.c_int, [C.POINTER(DenseParams), vp]),
    "fmla_quantize_kv_fp8": (C.c_int, [vp, i64, C.c_int, vp, vp, i64, vp]),
    "fmla_device_status": (C.c_int, [C.POINTER(C.c_int), C.c_int]),
    "fmla_sizeof_decode_params": (C.c_size_t, []),
    "fmla_sizeof_sparse_prefill_params": (C.c_size_t, []),
    "fmla_sizeof_dense_params": (C.c_size_t, []),
}


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python flashmla_windows_linux_sm120_b200/build.py` "
            "(needs nvcc). There is no fallback path.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)      # AttributeError if the library does not export it
        fn.restype = res
        fn.argtypes = args
    for cls, fn in ((DecodeParams, lib.fmla_sizeof_decode_params),
                    (SparsePrefillParams, lib.fmla_sizeof_sparse_prefill_params),
                    (DenseParams, lib.fmla_sizeof_dense_params), (PeerPush, lib.fmla_sizeof_peer_push)):
        if C.sizeof(cls) != fn():
            raise ImportError(f"struct layout mismatch for {cls.__name__}: {C.sizeof(cls)} vs {fn()}")
    return lib


lib = _load()


def check(status: int) -> None:
    """Raise RuntimeError (what TORCH_CHECK raises in the reference) on a non-zero status."""
    if status != 0:
        msg = lib.fmla_last_error_message().decode()
        kind = lib.fmla_status_string(status).decode()
        raise RuntimeError(f"flashmla_b200: {kind}: {msg}")
