"""Generate golden fixtures by running the REFERENCE's own Python on a CPU.

Run once in a container that has the reference checkout (it cannot travel to the
GPU box):

    python tests/golden/make_golden.py /path/to/reference

It imports the reference's test modules (tests/test_flash_mla_decoding.py,
tests/test_flash_mla_prefill.py, tests/test_fmha_sm100.py, tests/quant.py) and
flash_mla/flash_mla_interface.py, with
  * a stub registered as ``flash_mla.cuda_sm120`` (the CUDA extension does not
    exist here), and
  * ``Tensor.cuda()`` / ``torch.cuda.synchronize`` patched to no-ops,
runs their generators and fp32 torch references on small seeded cases, and
stores inputs and outputs as ``tests/golden/*.npz``.  bf16 tensors are stored as
their raw 16-bit patterns (suffix ``__bf16``), e4m3 bytes as uint8.
"""
from __future__ import annotations

import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _pack(d):
    out = {}
    for k, v in d.items():
        if v is None:
            continue
        if isinstance(v, torch.Tensor):
            v = v.detach().cpu()
            if v.dtype == torch.bfloat16:
                out[k + "__bf16"] = v.contiguous().view(torch.int16).numpy()
            elif v.dtype == torch.float8_e4m3fn:
                out[k + "__e4m3"] = v.contiguous().view(torch.uint8).numpy()
            else:
                out[k] = v.contiguous().numpy()
        else:
            out[k] = np.asarray(v)
    return out


def save(name, **d):
    path = os.path.join(HERE, name + ".npz")
    np.savez_compressed(path, **_pack(d))
    print("wrote", path, os.path.getsize(path) // 1024, "KiB")


def main(ref_root: str):
    sys.path.insert(0, ref_root)
    sys.path.insert(0, os.path.join(ref_root, "tests"))
    stub = types.ModuleType("flash_mla.cuda_sm120")
    sys.modules["flash_mla.cuda_sm120"] = stub
    torch.Tensor.cuda = lambda self, *a, **k: self          # generators call .cuda()
    torch.cuda.synchronize = lambda *a, **k: None
    torch.cuda.manual_seed = lambda *a, **k: None

    import flash_mla.flash_mla_interface as iface            # noqa: E402
    import quant as rquant                                    # noqa: E402
    import test_flash_mla_decoding as tdec                    # noqa: E402
    import test_flash_mla_prefill as tpre                     # noqa: E402
    import test_fmha_sm100 as tfmha                           # noqa: E402

    torch.set_default_dtype(torch.bfloat16)                   # as the reference tests' main()

    # ---- dense decode (reference_torch) -------------------------------------
    for name, tp in [
        ("decode_dense_causal", tdec.TestParam(2, 2, 140, True, True, False, None, h_q=16)),
        ("decode_dense_plain", tdec.TestParam(3, 1, 100, True, False, False, None, h_q=8)),
        ("decode_dense_zero", tdec.TestParam(4, 2, 150, True, True, False, None, h_q=8,
                                             have_zero_seqlen_k=True)),
    ]:
        lens, q, bt, bk, _, _ = tdec.generate_test_data(tp)
        out, lse = tdec.reference_torch(lens, bt, q, bk, tp.dv, tp.is_causal, None)
        save(name, cache_seqlens=lens, q=q, block_table=bt, blocked_k=bk, out=out, lse=lse,
             is_causal=int(tp.is_causal))

    # ---- sparse FP8 decode + codec ------------------------------------------
    for name, tp in [
        ("decode_sparse_fp8", tdec.TestParam(2, 2, 200, True, False, True, 128, h_q=16)),
        ("decode_sparse_fp8_pad", tdec.TestParam(2, 1, 60, False, False, True, 128, h_q=8)),
    ]:
        lens, q, bt, bk, abs_idx, phys_idx = tdec.generate_test_data(tp)
        bkq = rquant.quantize_k_cache(bk, tp.dv, 128)
        bkd = rquant.dequantize_k_cache(bkq)
        out, lse = tdec.reference_torch(lens, bt, q, bkd, tp.dv, False, abs_idx)
        save(name, cache_seqlens=lens, q=q, block_table=bt, blocked_k=bk, blocked_k_quant=bkq,
             blocked_k_dequant=bkd, abs_indices=abs_idx, indices=phys_idx, out=out, lse=lse)

    # ---- the reference's CPU torch path (dense, non-causal) ------------------
    tp = tdec.TestParam(2, 1, 128, False, False, False, None, h_q=16)
    lens, q, bt, bk, _, _ = tdec.generate_test_data(tp)
    os.environ["FLASH_MLA_FORCE_FALLBACK"] = "1"
    out, lse = iface.flash_mla_with_kvcache(q, bk, bt, lens, tp.dv, None, None, causal=False)
    save("decode_fallback_path", cache_seqlens=lens, q=q, block_table=bt, blocked_k=bk, out=out, lse=lse)

    # ---- sparse prefill ------------------------------------------------------
    for name, pp in [
        ("prefill_oob", tpre.TestParam(1, 3, 95, 128, h_q=8)),
        ("prefill_irregular", tpre.TestParam(1, 2, 592, 128, h_q=16)),
    ]:
        tc = tpre.generate_testcase(pp)
        sm_scale = 1 / (pp.d_qk ** 0.5)
        mx, lse, out = tpre.reference_torch(pp, tc, sm_scale)
        save(name, q=tc.q[0], kv=tc.kv[0], indices=tc.indices[0], sm_scale=sm_scale,
             out=out.float(), max_logits=mx.float(), lse=lse.float())

    # ---- dense MHA forward / backward ---------------------------------------
    for name, (b, msq, msk, varlen, h, h_k, d, dv, causal) in [
        ("dense_mla192_causal", (2, 48, 48, True, 4, 4, 192, 128, True)),
        ("dense_128_plain_gqa", (2, 40, 56, True, 4, 2, 128, 128, False)),
    ]:
        import random
        torch.manual_seed(0)
        random.seed(0)
        tfmha.h, tfmha.h_k = h, h_k                            # module globals read by sdpa()
        sq = torch.full((b,), msq, dtype=torch.int32)
        sk = torch.full((b,), msk, dtype=torch.int32)
        for i in range(b):
            sq[i] = max(random.normalvariate(msq, msq / 2), 1)
        for i in range(b):
            sk[i] = max(random.normalvariate(msk, msk / 2), sq[i].item())
        cu_q = torch.cumsum(torch.nn.functional.pad(sq, (1, 0)), 0, dtype=torch.int32)
        cu_k = torch.cumsum(torch.nn.functional.pad(sk, (1, 0)), 0, dtype=torch.int32)
        tq, tk = int(sq.sum()), int(sk.sum())
        q = torch.randn(tq, h, d) / 10
        k = torch.randn(tk, h_k, d) / 10
        v = torch.randn(tk, h_k, dv) / 10
        go = torch.randn(tq, h, dv) / 10
        scale = (d + 100) ** (-0.5)
        q2, k2, v2 = (t.clone().requires_grad_() for t in (q, k, v))
        outs, lses = [], []
        for i in range(b):
            o, l = tfmha.sdpa(q2[cu_q[i].item():cu_q[i + 1].item()],
                              k2[cu_k[i].item():cu_k[i + 1].item()],
                              v2[cu_k[i].item():cu_k[i + 1].item()],
                              attn_bias=tfmha.get_attn_bias(sq[i].item(), sk[i].item(), causal, 0),
                              softmax_scale=scale)
            outs.append(o.transpose(-3, -2))
            lses.append(l.transpose(-2, -1))
        out = torch.cat(outs)
        lse = torch.cat(lses)
        extra = {}
        if h == h_k:
            out.backward(go)
            extra = dict(dq=q2.grad.float(), dk=k2.grad.float(), dv=v2.grad.float())
        save(name, q=q, k=k, v=v, d_out=go, cu_q=cu_q, cu_k=cu_k, scale=scale, causal=int(causal),
             out=out.detach().float(), lse=lse.detach().float(), **extra)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path of the reference checkout>")
    main(sys.argv[1])
