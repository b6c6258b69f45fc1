"""Helpers shared by the GPU parity tests."""
import torch

from oracle.check import check_is_allclose, max_abs_diff

# Tolerances (stated once, used by every parity test):
#  * the reference tests' own element-wise bounds (tests/test_flash_mla_decoding.py:252-253,
#    tests/test_flash_mla_prefill.py:123-125, tests/test_fmha_sm100.py:126-133), and
#  * the build target: bf16 outputs max-abs <= 2e-3 (scaled by max(1, max|ref|), one bf16 ulp
#    of the largest output), LSE max-abs <= 1e-4.
OUT_ABS, OUT_REL, OUT_COS = 8e-4, 2.01 / 128, 5e-6
LSE_ABS, LSE_REL = 1e-6, 8.01 / 65536
TARGET_OUT_MAXABS = 2e-3
TARGET_LSE_MAXABS = 1e-4


def cuda_available() -> bool:
    return torch.cuda.is_available()


def dev(t):
    return None if t is None else t.cuda()


def assert_out_lse(out, lse, ref_out, ref_lse, out_cos=OUT_COS):
    assert check_is_allclose("out", out, ref_out, abs_tol=OUT_ABS, rel_tol=OUT_REL, cos_diff_tol=out_cos)
    assert check_is_allclose("lse", lse, ref_lse, abs_tol=LSE_ABS, rel_tol=LSE_REL)
    scale = max(1.0, float(ref_out.float().abs().max()))
    assert max_abs_diff(out, ref_out) <= TARGET_OUT_MAXABS * scale, max_abs_diff(out, ref_out)
    assert max_abs_diff(lse, ref_lse) <= TARGET_LSE_MAXABS * max(1.0, float(ref_lse[torch.isfinite(ref_lse)].abs().max()) if torch.isfinite(ref_lse).any() else 1.0)
