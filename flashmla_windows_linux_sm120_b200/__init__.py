"""flashmla_windows_linux_sm120_b200: B200 (sm_100a) implementation of the
FlashMLA attention path behind the reference's Python API
(flash_mla/__init__.py:3-21 exports the same names)."""
__version__ = "0.1.0"

from .flash_mla_interface import (  # noqa: F401
    FLASH_MLA_LOADED_VARIANT,
    flash_attn_varlen_func,
    flash_attn_varlen_kvpacked_func,
    flash_attn_varlen_qkvpacked_func,
    flash_mla_sparse_fwd,
    flash_mla_with_kvcache,
    flash_mla_sparse_decode_logical_indices,
    get_mla_metadata,
)

__all__ = [
    "get_mla_metadata",
    "flash_mla_with_kvcache",
    "flash_mla_sparse_decode_logical_indices",
    "flash_attn_varlen_func",
    "flash_attn_varlen_qkvpacked_func",
    "flash_attn_varlen_kvpacked_func",
    "flash_mla_sparse_fwd",
    "FLASH_MLA_LOADED_VARIANT",
]
