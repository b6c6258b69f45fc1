"""Pins the CPU oracle against outputs of the reference's own Python
(tests/golden/*.npz, produced by tests/golden/make_golden.py)."""
import math

import pytest
import torch

from golden_io import load
from oracle import combine, decode, dense, quant, sparse_prefill
from oracle.check import check_is_allclose


@pytest.mark.parametrize("name", ["decode_dense_causal", "decode_dense_plain", "decode_dense_zero"])
def test_decode_dense(name):
    g = load(name)
    out, lse = decode.decode_ref(g["cache_seqlens"], g["block_table"], g["q"], g["blocked_k"], 512,
                                 bool(g["is_causal"]))
    assert torch.equal(torch.isinf(lse), torch.isinf(g["lse"]))
    assert check_is_allclose("out", out, g["out"], abs_tol=1e-6, rel_tol=1e-2, cos_diff_tol=1e-9)
    assert check_is_allclose("lse", lse, g["lse"], abs_tol=1e-6, rel_tol=1e-6)


@pytest.mark.parametrize("name", ["decode_sparse_fp8", "decode_sparse_fp8_pad"])
def test_decode_sparse_and_codec(name):
    g = load(name)
    # codec: bit-exact bytes and bit-exact de-quantised bf16
    qk = quant.quantize_k_cache(g["blocked_k"], 512, 128)
    used = ~torch.isnan(g["blocked_k"].float()).any(dim=-1).reshape(-1)
    a = qk.view(torch.uint8).reshape(-1, 656)[used]
    b = g["blocked_k_quant"].view(torch.uint8).reshape(-1, 656)[used]
    assert torch.equal(a, b)
    dq = quant.dequantize_k_cache(g["blocked_k_quant"])
    assert torch.equal(dq.view(torch.int16).reshape(-1, 576)[used],
                       g["blocked_k_dequant"].view(torch.int16).reshape(-1, 576)[used])
    # attention, stated on logical and on physical indices
    out, lse = decode.decode_ref(g["cache_seqlens"], g["block_table"], g["q"], g["blocked_k_dequant"], 512,
                                 False, g["abs_indices"])
    assert check_is_allclose("out", out, g["out"], abs_tol=1e-6, rel_tol=1e-2, cos_diff_tol=1e-9)
    assert check_is_allclose("lse", lse, g["lse"], abs_tol=1e-6, rel_tol=1e-6)
    out2, lse2 = decode.decode_sparse_physical_ref(g["q"], g["blocked_k_dequant"], g["indices"], 512)
    assert check_is_allclose("out_phys", out2, g["out"], abs_tol=2e-5, rel_tol=1e-2, cos_diff_tol=1e-8)
    assert check_is_allclose("lse_phys", lse2, g["lse"], abs_tol=2e-6, rel_tol=1e-6)


def test_fallback_path():
    g = load("decode_fallback_path")
    out, lse = decode.fallback_ref(g["q"], g["blocked_k"], g["block_table"], g["cache_seqlens"], 512)
    assert check_is_allclose("out", out, g["out"], abs_tol=1e-6, rel_tol=1e-2, cos_diff_tol=1e-9)
    assert check_is_allclose("lse", lse, g["lse"], abs_tol=1e-6, rel_tol=1e-6)
    # and the test reference agrees with the fallback for non-causal dense decode
    out2, lse2 = decode.decode_ref(g["cache_seqlens"], g["block_table"], g["q"], g["blocked_k"], 512, False)
    assert check_is_allclose("out2", out2, g["out"], abs_tol=8e-4, rel_tol=2.01 / 128, cos_diff_tol=5e-6)
    assert check_is_allclose("lse2", lse2, g["lse"], abs_tol=1e-5, rel_tol=1e-5)


@pytest.mark.parametrize("name", ["prefill_oob", "prefill_irregular"])
def test_sparse_prefill(name):
    g = load(name)
    out, mx, lse = sparse_prefill.sparse_prefill_ref(g["q"], g["kv"], g["indices"], g["sm_scale"])
    assert check_is_allclose("out", out, g["out"], abs_tol=1e-5, rel_tol=1e-2, cos_diff_tol=1e-9)
    assert check_is_allclose("max_logits", mx, g["max_logits"], abs_tol=1e-6, rel_tol=1e-6)
    assert check_is_allclose("lse", lse, g["lse"], abs_tol=1e-6, rel_tol=1e-6)


@pytest.mark.parametrize("name", ["dense_mla192_causal", "dense_128_plain_gqa"])
def test_dense(name):
    g = load(name)
    causal = bool(g["causal"])
    if "dq" in g:
        out, lse, dq, dk, dv = dense.dense_fwd_bwd_ref(g["q"], g["k"], g["v"], g["d_out"], g["cu_q"], g["cu_k"],
                                                       causal, g["scale"])
        # the reference's leaves are bf16, so its stored gradients carry one bf16 rounding (2^-9 relative)
        assert check_is_allclose("dq", dq, g["dq"], abs_tol=1e-4, rel_tol=2e-2, cos_diff_tol=4e-6)
        assert check_is_allclose("dk", dk, g["dk"], abs_tol=1e-4, rel_tol=2e-2, cos_diff_tol=4e-6)
        assert check_is_allclose("dv", dv, g["dv"], abs_tol=1e-4, rel_tol=2e-2, cos_diff_tol=4e-6)
    else:
        out, lse = dense.dense_fwd_ref(g["q"], g["k"], g["v"], g["cu_q"], g["cu_k"], causal, g["scale"])
    assert check_is_allclose("out", out, g["out"], abs_tol=1e-5, rel_tol=1e-2, cos_diff_tol=1e-8)
    assert check_is_allclose("lse", lse, g["lse"], abs_tol=1e-6, rel_tol=1e-6)


def test_combine_closed_form():
    torch.manual_seed(0)
    n, rows, dv = 5, 7, 16
    # partial softmaxes over disjoint key sets must merge to the softmax over the union
    logits = torch.randn(rows, n, 9) * 3
    vals = torch.randn(rows, n, 9, dv)
    lse_parts = torch.logsumexp(logits, dim=-1) * math.log2(math.e)          # base 2
    o_parts = (torch.softmax(logits, -1).unsqueeze(-1) * vals).sum(-2)
    lse_parts[2, 1] = float("-inf")
    logits[2, 1] = float("-inf")
    o, lse = combine.combine_ref(lse_parts.t().contiguous(), o_parts.transpose(0, 1).contiguous())
    full = logits.reshape(rows, -1)
    p = torch.softmax(full, -1)
    ref = (p.unsqueeze(-1) * vals.reshape(rows, -1, dv)).sum(1)
    assert torch.allclose(o, ref, atol=1e-5)
    assert torch.allclose(lse, torch.logsumexp(full, -1), atol=1e-5)
    o2, lse2 = combine.combine_ref(torch.full((3, 2), float("-inf")), torch.zeros(3, 2, dv))
    assert torch.isinf(lse2).all() and (lse2 > 0).all() and (o2 == 0).all()
