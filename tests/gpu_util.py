"""Helpers shared by the GPU parity tests."""
import math

import torch

from oracle.check import check_is_allclose, max_abs_diff

# Tolerances (stated once, used by every parity test):
#  * the reference tests' own element-wise bounds (tests/test_flash_mla_decoding.py:252-253,
#    tests/test_flash_mla_prefill.py:123-125, tests/test_fmha_sm100.py:126-133), and
#  * the build target: 16-bit outputs max-abs <= 2e-3 against the fp32 reference, LSE max-abs <= 1e-4.
#    The output bound is applied as stated wherever the reference output stays within [-1, 1].  A 16-bit
#    output of magnitude in [B/2, B) is rounded with a step of up to 1.95e-3 * B, so above 1 the bound is
#    2.5e-3 * B with B = the power of two above the largest reference magnitude (the rounding step plus the
#    same relative allowance for the arithmetic).  The LSE bound is applied as stated, unscaled.
# Every helper prints the error it measured, so a test log shows the margin, not only pass / fail.
OUT_ABS, OUT_REL, OUT_COS = 8e-4, 2.01 / 128, 5e-6
LSE_ABS, LSE_REL = 1e-6, 8.01 / 65536
TARGET_OUT_MAXABS = 2e-3
TARGET_LSE_MAXABS = 1e-4


def cuda_available() -> bool:
    return torch.cuda.is_available()


def dev(t):
    return None if t is None else t.cuda()


def out_bound(ref_out) -> float:
    m = float(ref_out.float().abs().max())
    return TARGET_OUT_MAXABS if m <= 1.0 else 2.5e-3 * 2.0 ** math.ceil(math.log2(m))


def assert_target_bounds(out, lse, ref_out, ref_lse, what: str = "") -> dict:
    """The build-target bounds alone (max-abs of out and of the finite LSE entries); prints and returns the
    measured errors."""
    e_out = max_abs_diff(out, ref_out)
    e_lse = max_abs_diff(lse, ref_lse)
    bound = out_bound(ref_out)
    print(f"[parity{' ' + what if what else ''}] out max-abs {e_out:.3e} (bound {bound:.1e}, max|ref| "
          f"{float(ref_out.float().abs().max()):.3f})  lse max-abs {e_lse:.3e} (bound {TARGET_LSE_MAXABS:.0e})")
    assert e_out <= bound, (e_out, bound)
    assert e_lse <= TARGET_LSE_MAXABS, e_lse
    return {"out_max_abs": e_out, "lse_max_abs": e_lse}


def assert_out_lse(out, lse, ref_out, ref_lse, out_cos=OUT_COS, what: str = "") -> dict:
    assert check_is_allclose("out", out, ref_out, abs_tol=OUT_ABS, rel_tol=OUT_REL, cos_diff_tol=out_cos)
    assert check_is_allclose("lse", lse, ref_lse, abs_tol=LSE_ABS, rel_tol=LSE_REL)
    return assert_target_bounds(out, lse, ref_out, ref_lse, what)
