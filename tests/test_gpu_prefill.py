"""GPU parity of flash_mla_sparse_fwd (cases of tests/test_flash_mla_prefill.py:139-172)."""
import math

import pytest
import torch

import gpu_util as U
from golden_io import load
from oracle import gen, sparse_prefill
from oracle.check import check_is_allclose, max_abs_diff

pytestmark = pytest.mark.gpu


def _check(q, kv, idx, sm_scale):
    import flashmla_windows_linux_sm120_b200 as fm
    out, mx, lse = fm.flash_mla_sparse_fwd(q.cuda(), kv.cuda(), idx.cuda(), sm_scale)
    torch.cuda.synchronize()
    r_out, r_mx, r_lse = sparse_prefill.sparse_prefill_ref(q, kv, idx, sm_scale)
    assert check_is_allclose("out", out, r_out, abs_tol=8e-4, rel_tol=2.01 / 128, cos_diff_tol=7e-6)
    assert check_is_allclose("max_logits", mx, r_mx, abs_tol=1e-6, rel_tol=2.01 / 65536)
    assert check_is_allclose("lse", lse, r_lse, abs_tol=1e-6, rel_tol=2.01 / 65536)
    assert max_abs_diff(out, r_out) <= U.TARGET_OUT_MAXABS * max(1.0, float(r_out.abs().max()))
    fin = torch.isfinite(r_lse)
    if fin.any():
        assert (lse.cpu()[fin] - r_lse[fin]).abs().max() <= U.TARGET_LSE_MAXABS * max(1.0, float(r_lse[fin].abs().max()))


@pytest.mark.parametrize("s_kv,topk", [(128, 128), (256, 256), (512, 512), (592, 128), (1840, 256), (1592, 384),
                                       (1521, 512), (95, 128), (153, 256), (114, 384), (32, 2048), (64, 8192)])
@pytest.mark.parametrize("s_q", [1, 62])
def test_sparse_prefill(s_kv, topk, s_q):
    q, kv, idx = gen.make_prefill_case(gen.PrefillCase(s_q=s_q, s_kv=s_kv, topk=topk))
    _check(q, kv, idx, 1 / math.sqrt(576))


def test_sparse_prefill_rows_without_valid_index():
    q, kv, idx = gen.make_prefill_case(gen.PrefillCase(s_q=5, s_kv=300, topk=128))
    idx[1] = -1
    idx[3] = 2147480000
    _check(q, kv, idx, 1 / math.sqrt(576))


def test_sparse_prefill_causal_restricted_h64():
    q, kv, idx = gen.make_prefill_case(gen.PrefillCase(s_q=48, s_kv=4096, topk=512, h_q=64, causal_restrict=True))
    _check(q, kv, idx, 1 / math.sqrt(576))


@pytest.mark.parametrize("name", ["prefill_irregular", "prefill_oob"])
def test_sparse_prefill_golden(name):
    import flashmla_windows_linux_sm120_b200 as fm
    g = load(name)
    h_q = g["q"].shape[1]
    # fixtures were generated with few heads to stay small: replicate heads to a full 64-head tile
    q = g["q"].repeat(1, 64 // h_q, 1)
    out, mx, lse = fm.flash_mla_sparse_fwd(q.cuda(), g["kv"].cuda(), g["indices"].cuda(), g["sm_scale"])
    out, mx, lse = out.cpu()[:, :h_q], mx.cpu()[:, :h_q], lse.cpu()[:, :h_q]
    assert check_is_allclose("out", out, g["out"], abs_tol=8e-4, rel_tol=2.01 / 128, cos_diff_tol=7e-6)
    assert check_is_allclose("max_logits", mx, g["max_logits"], abs_tol=1e-6, rel_tol=2.01 / 65536)
    assert check_is_allclose("lse", lse, g["lse"], abs_tol=1e-6, rel_tol=2.01 / 65536)
