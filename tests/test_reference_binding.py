"""The reference's UNCHANGED Python interface bound over this package's extension module.

`flash_mla/flash_mla_interface.py` of the reference imports a module object (its first candidate is
`flash_mla.cuda_sm120`, :22-28) and calls five attributes of it positionally (:152-159, 299-311, 339-341,
373-387, 436-454).  Here `flashmla_windows_linux_sm120_b200.cuda_sm100` is registered under that name, the
reference package is imported as it stands, and every public entry point of the reference is driven with CPU
tensors while the five extension functions are replaced by recorders that bind the received positional /
keyword arguments against the REAL signatures of this package's functions: a change of arity, order or a
renamed keyword on either side fails the bind.  No kernel runs (no GPU needed).

The reference tree is looked for in $FMLA_REFERENCE_DIR and next to the repository (../reference); the
binding test is skipped where it is absent.  The seven public signatures are pinned either way.
"""
import importlib
import inspect
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _reference_dir():
    for cand in (os.environ.get("FMLA_REFERENCE_DIR"), os.path.join(os.path.dirname(ROOT), "reference")):
        if cand and os.path.exists(os.path.join(cand, "flash_mla", "flash_mla_interface.py")):
            return cand
    return None


PUBLIC = {
    "get_mla_metadata": ["cache_seqlens", "num_q_tokens_per_head_k", "num_heads_k", "num_heads_q", "is_fp8_kvcache", "topk"],
    "flash_mla_with_kvcache": ["q", "k_cache", "block_table", "cache_seqlens", "head_dim_v", "tile_scheduler_metadata",
                               "num_splits", "softmax_scale", "causal", "is_fp8_kvcache", "indices"],
    "flash_mla_sparse_fwd": ["q", "kv", "indices", "sm_scale", "d_v"],
    "flash_attn_varlen_func": ["q", "k", "v", "cu_seqlens_qo", "cu_seqlens_kv", "max_seqlen_qo", "max_seqlen_kv", "dropout_p",
                               "softmax_scale", "causal", "deterministic", "is_varlen"],
    "flash_attn_varlen_qkvpacked_func": ["qkv", "cu_seqlens", "max_seqlen", "head_dim_qk", "dropout_p", "softmax_scale", "causal",
                                         "deterministic", "is_varlen"],
    "flash_attn_varlen_kvpacked_func": ["q", "kv", "cu_seqlens_qo", "cu_seqlens_kv", "max_seqlen_qo", "max_seqlen_kv", "head_dim_qk",
                                        "dropout_p", "softmax_scale", "causal", "deterministic", "is_varlen"],
}


def test_all_public_signatures_are_pinned():
    import flashmla_windows_linux_sm120_b200 as fm
    for name, params in PUBLIC.items():
        assert list(inspect.signature(getattr(fm, name)).parameters) == params, name
    assert isinstance(fm.FLASH_MLA_LOADED_VARIANT, str)


@pytest.fixture
def reference_over_our_extension(monkeypatch):
    ref_dir = _reference_dir()
    if ref_dir is None:
        pytest.skip("reference tree not available")
    from flashmla_windows_linux_sm120_b200 import cuda_sm100
    for m in [k for k in sys.modules if k == "flash_mla" or k.startswith("flash_mla.")]:
        monkeypatch.delitem(sys.modules, m)
    monkeypatch.setitem(sys.modules, "flash_mla.cuda_sm120", cuda_sm100)
    monkeypatch.syspath_prepend(ref_dir)
    ref = importlib.import_module("flash_mla")
    calls = []

    def recorder(name, result):
        real = getattr(cuda_sm100, name)
        sig = inspect.signature(real)

        def spy(*args, **kwargs):
            bound = sig.bind(*args, **kwargs)          # TypeError on an arity / keyword mismatch
            calls.append((name, dict(bound.arguments)))
            return result(bound.arguments)
        return spy

    def md(a):
        return [torch.zeros((4, 8), dtype=torch.int32), torch.zeros((a["seqlens_k"].shape[0] + 1,), dtype=torch.int32)]

    def dec(a):
        b, s_q, h_q, _ = a["q"].shape
        return [torch.zeros((b, s_q, h_q, a["head_size_v"]), dtype=a["q"].dtype), torch.zeros((b, h_q, s_q))]

    def pre(a):
        s_q, h_q, _ = a["q"].shape
        return [torch.zeros((s_q, h_q, a["d_v"]), dtype=torch.bfloat16), torch.zeros((s_q, h_q)), torch.zeros((s_q, h_q))]

    for name, result in (("get_mla_decoding_metadata", md), ("fwd_kvcache_mla", dec), ("sparse_prefill_fwd", pre),
                         ("dense_prefill_fwd", lambda a: None), ("dense_prefill_bwd", lambda a: None)):
        monkeypatch.setattr(cuda_sm100, name, recorder(name, result))
    yield ref, calls
    for m in [k for k in sys.modules if k == "flash_mla" or k.startswith("flash_mla.")]:
        sys.modules.pop(m, None)


def test_reference_interface_binds_every_call_site(reference_over_our_extension):
    ref, calls = reference_over_our_extension
    assert ref.FLASH_MLA_LOADED_VARIANT == "sm120"          # otherwise decode would be routed to the torch fallback (:148, 287)
    # the public signatures of both packages agree parameter by parameter (names and defaults)
    import flashmla_windows_linux_sm120_b200 as fm
    for name in PUBLIC:
        ours, theirs = inspect.signature(getattr(fm, name)), inspect.signature(getattr(ref, name))
        assert [(p.name, p.default) for p in ours.parameters.values()] == [(p.name, p.default) for p in theirs.parameters.values()], name

    lens = torch.tensor([100, 200], dtype=torch.int32)
    bf = torch.bfloat16
    md, ns = ref.get_mla_metadata(lens, 128, 1)
    ref.get_mla_metadata(lens, 128, 1, 128, True, 2048)
    q = torch.zeros((2, 1, 128, 576), dtype=bf)
    kc = torch.zeros((8, 64, 1, 576), dtype=bf)
    bt = torch.zeros((2, 4), dtype=torch.int32)
    ref.flash_mla_with_kvcache(q, kc, bt, lens, 512, md, ns, causal=True)
    idx = torch.zeros((2, 1, 64), dtype=torch.int32)
    ref.flash_mla_with_kvcache(q, torch.zeros((8, 64, 1, 656), dtype=torch.uint8), bt, lens, 512, md, ns, is_fp8_kvcache=True, indices=idx)
    ref.flash_mla_sparse_fwd(torch.zeros((3, 128, 576), dtype=bf), torch.zeros((64, 1, 576), dtype=bf),
                             torch.zeros((3, 1, 128), dtype=torch.int32), 0.04)
    cu = torch.tensor([0, 5], dtype=torch.int32)
    mk = lambda d: torch.zeros((5, 4, d), dtype=bf, requires_grad=True)
    qq, kk, vv = mk(192), mk(192), mk(128)
    out, lse = ref.flash_attn_varlen_func(qq, kk, vv, cu, cu, 5, 5, causal=True)
    out.sum().backward()
    qkv = torch.zeros((5, 4, 192 + 192 + 128), dtype=bf)
    ref.flash_attn_varlen_qkvpacked_func(qkv, cu, 5, head_dim_qk=192, causal=True)
    ref.flash_attn_varlen_kvpacked_func(torch.zeros((5, 4, 192), dtype=bf), torch.zeros((5, 4, 192 + 128), dtype=bf), cu, cu, 5, 5,
                                        head_dim_qk=192)

    names = [n for n, _ in calls]
    assert names.count("get_mla_decoding_metadata") == 2 and names.count("fwd_kvcache_mla") == 2
    assert names.count("sparse_prefill_fwd") == 1 and names.count("dense_prefill_fwd") == 3 and names.count("dense_prefill_bwd") == 1
    by = lambda n, i=0: [a for m, a in calls if m == n][i]
    a = by("get_mla_decoding_metadata", 1)
    assert (a["num_q_tokens_per_head_k"], a["h_k"], a["h_q"], a["is_fp8_kvcache"], a["topk"]) == (128, 1, 128, True, 2048)
    a = by("fwd_kvcache_mla", 0)
    assert a["head_size_v"] == 512 and a["is_causal"] is True and a["is_fp8"] is False and a["indices"] is None
    assert a["seqlens_k"] is lens and a["block_table"] is bt and abs(a["softmax_scale"] - 576 ** -0.5) < 1e-9
    a = by("fwd_kvcache_mla", 1)
    assert a["is_fp8"] is True and a["indices"] is idx and a["is_causal"] is False
    a = by("sparse_prefill_fwd")
    assert abs(a["sm_scale"] - 0.04) < 1e-9 and a["d_v"] == 512
    a = by("dense_prefill_fwd", 0)
    assert a["mask_mode_code"] == 1 and a["max_seqlen_q"] == 5 and a["max_seqlen_kv"] == 5 and a["is_varlen"] is True
    assert a["workspace_buffer"].dtype == torch.uint8 and tuple(a["lse"].shape) == (5, 4) and a["lse"].stride(0) == 1
    a = by("dense_prefill_bwd")
    assert a["mask_mode_code"] == 1 and tuple(a["dq"].shape) == (5, 4, 192) and tuple(a["dv"].shape) == (5, 4, 128)
    assert tuple(a["d_o"].shape) == (5, 4, 128) and a["cumulative_seqlen_q"] is cu
