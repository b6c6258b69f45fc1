"""CPU checks of the C-ABI library: it loads, exports every symbol the public
header declares, and its host-only entry points behave (no GPU needed)."""
import ctypes as C
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared_symbols():
    text = open(os.path.join(ROOT, "include", "flashmla_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fmla_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    from flashmla_windows_linux_sm120_b200 import _cabi
    names = _declared_symbols()
    assert len(names) >= 15
    for n in names:
        assert hasattr(_cabi.lib, n), f"{n} declared in include/flashmla_b200.h but not exported"
        assert n in _cabi.SYMBOLS, f"{n} has no ctypes prototype"
    assert sorted(_cabi.SYMBOLS) == names


def test_host_only_entry_points():
    from flashmla_windows_linux_sm120_b200._cabi import DecodeParams, DenseParams, SparsePrefillParams, lib
    assert lib.fmla_status_string(0) == b"ok"
    assert b"invalid" in lib.fmla_status_string(1)
    assert lib.fmla_version().decode().count(".") == 2
    assert lib.fmla_sizeof_decode_params() == C.sizeof(DecodeParams)
    assert lib.fmla_sizeof_sparse_prefill_params() == C.sizeof(SparsePrefillParams)
    assert lib.fmla_sizeof_dense_params() == C.sizeof(DenseParams)
    a, b = C.c_size_t(0), C.c_size_t(0)
    assert lib.fmla_decode_scratch_bytes(128, 1, 128, 74, 512, C.byref(a), C.byref(b)) == 0
    assert a.value == (128 + 74) * 128 * 4 and b.value == (128 + 74) * 128 * 512 * 4
    assert lib.fmla_dense_bwd_workspace_bytes(1000, 4, 192) >= 1000 * 4 * 4


def test_argument_validation_without_gpu():
    """Rejected arguments return a status and a message before any CUDA call."""
    from flashmla_windows_linux_sm120_b200._cabi import DecodeParams, lib
    p = DecodeParams()
    assert lib.fmla_fwd_kvcache_mla(C.byref(p), None) == 1
    assert b"batch" in lib.fmla_last_error_message()
    assert lib.fmla_fwd_kvcache_mla(None, None) == 1
    assert lib.fmla_get_mla_metadata(None, 1, 1, -1, None, None, None) == 1
    assert lib.fmla_combine_partials(None, None, 1, 1, 512, None, 512, None, None) == 1
    n = C.c_int(0)
    assert lib.fmla_get_num_sm_parts(0, 128, 1, 128, 1, 0, C.byref(n)) == 2     # dense FP8: unsupported


def test_python_api_surface_matches_reference_names():
    import flashmla_windows_linux_sm120_b200 as fm
    for name in ["get_mla_metadata", "flash_mla_with_kvcache", "flash_attn_varlen_func",
                 "flash_attn_varlen_qkvpacked_func", "flash_attn_varlen_kvpacked_func", "flash_mla_sparse_fwd",
                 "FLASH_MLA_LOADED_VARIANT"]:
        assert hasattr(fm, name)
    import inspect
    sig = inspect.signature(fm.flash_mla_with_kvcache)
    assert list(sig.parameters) == ["q", "k_cache", "block_table", "cache_seqlens", "head_dim_v",
                                    "tile_scheduler_metadata", "num_splits", "softmax_scale", "causal",
                                    "is_fp8_kvcache", "indices"]
    sig = inspect.signature(fm.get_mla_metadata)
    assert list(sig.parameters) == ["cache_seqlens", "num_q_tokens_per_head_k", "num_heads_k", "num_heads_q",
                                    "is_fp8_kvcache", "topk"]
