"""GPU parity of flash_mla_sparse_fwd (cases of tests/test_flash_mla_prefill.py:139-172)."""
import math

import pytest
import torch

import gpu_util as U
from golden_io import load
from oracle import gen, sparse_prefill
from oracle.check import check_is_allclose, max_abs_diff

pytestmark = pytest.mark.gpu


def _check(q, kv, idx, sm_scale, what="", logit_tol=None):
    """logit_tol: absolute bound for max_logits / lse when the logits are far larger than in the reference's tests
    (their fp32 rounding grows with their magnitude); None = the reference's bounds and the build target."""
    import flashmla_windows_linux_sm120_b200 as fm
    out, mx, lse = fm.flash_mla_sparse_fwd(q.cuda(), kv.cuda(), idx.cuda(), sm_scale)
    torch.cuda.synchronize()
    r_out, r_mx, r_lse = sparse_prefill.sparse_prefill_ref(q, kv, idx, sm_scale)
    assert check_is_allclose("out", out, r_out, abs_tol=8e-4, rel_tol=2.01 / 128, cos_diff_tol=7e-6)
    assert check_is_allclose("max_logits", mx, r_mx, abs_tol=logit_tol or 1e-6, rel_tol=2.01 / 65536)
    assert check_is_allclose("lse", lse, r_lse, abs_tol=logit_tol or 1e-6, rel_tol=2.01 / 65536)
    # build-target bounds; max_logits and lse are base-2 quantities here (README.md:201-217), i.e. log2(e)
    # times the natural-log LSE the 1e-4 bound is stated for
    e_out, e_lse, e_mx = max_abs_diff(out, r_out), max_abs_diff(lse, r_lse), max_abs_diff(mx, r_mx)
    print(f"[parity prefill {what}] out max-abs {e_out:.3e} (bound {U.out_bound(r_out):.1e})  lse(base 2) max-abs {e_lse:.3e}  "
          f"max_logits max-abs {e_mx:.3e} (bound {U.TARGET_LSE_MAXABS * math.log2(math.e):.2e})")
    assert e_out <= U.out_bound(r_out)
    lim = logit_tol or U.TARGET_LSE_MAXABS * math.log2(math.e)
    assert e_lse <= lim and e_mx <= lim


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


@pytest.mark.parametrize("s_q,h_q,s_kv,topk", [(300, 128, 4096, 512), (700, 128, 4096, 512), (333, 64, 2048, 256)])
def test_sparse_prefill_more_query_tokens_than_resident_ctas(s_q, h_q, s_kv, topk):
    """The kernel is persistent: min(s_q, SMs / head tiles) CTAs per head tile walk the query tokens.  With
    s_q above 74 (128 heads) or 148 (64 heads) every CTA takes several tokens in turn, which exercises the
    re-use of the Q tile, of the accumulators and of every barrier phase across tokens."""
    q, kv, idx = gen.make_prefill_case(gen.PrefillCase(s_q=s_q, s_kv=s_kv, topk=topk, h_q=h_q, causal_restrict=True))
    _check(q, kv, idx, 1 / math.sqrt(576), what=f"s_q={s_q} h_q={h_q}")


def test_sparse_prefill_leading_blocks_without_valid_index_and_very_negative_logits():
    """The first 64-index blocks of some rows hold only padding, and the first visible keys then have logits
    far below -128 (base 2): the running scale has to be taken from them, not rescaled from zero."""
    q, kv, idx = gen.make_prefill_case(gen.PrefillCase(s_q=6, s_kv=1024, topk=256))
    q = (q.float() * 100).to(torch.bfloat16)
    kv = (kv.float() * 10).to(torch.bfloat16)
    kv[:, 0, :] = -(q[0, 0].float().sign() * kv[:, 0, :].float().abs()).to(torch.bfloat16)    # q[0, head 0] . k << 0 for every key
    idx[0, 0, :128] = -1
    idx[3, 0, :64] = 2147480000
    q2 = q.clone()
    q2[3] = q[0]
    # logits reach -200 here: a 576-term fp32 dot product of that size carries ~2e-4 of rounding, so 1e-3 is the bound
    _check(q2, kv, idx, 1 / math.sqrt(576), what="leading padding", logit_tol=1e-3)


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
