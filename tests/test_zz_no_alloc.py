"""The decode entry point that brings its own scratch (fmla_fwd_kvcache_mla_static_scratch).

A caller that may not allocate device memory at call time (fixed arena handed out at start-up, a
plugin's enqueue hook, work recorded into a stream) uses this entry point instead of
fmla_fwd_kvcache_mla; the partial-result scratch then comes from arrays built into the library.
The test drives it through the C ABI, twice in a row with different problems (the second run sees
whatever the first left in the shared arrays), and checks each result against the regular entry
point fed with caller-allocated scratch: the two run the same kernels on the same schedule in a fixed
order, so the results have to be bit-identical; one of the two problems is also checked against the
CPU oracle.  Collected last on purpose (file name), so a failure here
cannot hide a failure elsewhere under `pytest -x`.
"""
import ctypes as C

import pytest
import torch

import gpu_util as U
from oracle import gen

pytestmark = pytest.mark.gpu


def _params(d, t, md, ns, out, lse, lse_accum, o_accum):
    from flashmla_windows_linux_sm120_b200._cabi import DecodeParams
    q, kc, bt, lens = d["q"], d["kcache"], d["block_table"], d["lens"]
    p = DecodeParams()
    p.b, p.s_q, p.h_q, p.h_k, p.d, p.d_v = t.b, t.s_q, t.h_q, t.h_kv, 576, 512
    p.num_blocks, p.page_block_size = kc.shape[0], 64
    p.is_causal, p.is_fp8, p.topk, p.q_dtype = int(t.is_causal), 0, -1, 0
    p.softmax_scale = 576 ** -0.5
    p.q, p.q_stride_b, p.q_stride_s, p.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1), q.stride(2)
    p.kcache, p.k_stride_block, p.k_stride_row, p.k_stride_head = kc.data_ptr(), kc.stride(0), kc.stride(1), kc.stride(2)
    p.block_table, p.block_table_stride_b = bt.data_ptr(), bt.stride(0)
    p.seqlens_k = lens.data_ptr()
    p.tile_scheduler_metadata, p.num_sm_parts, p.num_splits = md.data_ptr(), md.shape[0], ns.data_ptr()
    p.out, p.o_stride_b, p.o_stride_s, p.o_stride_h = out.data_ptr(), out.stride(0), out.stride(1), out.stride(2)
    p.softmax_lse = lse.data_ptr()
    p.lse_accum = lse_accum.data_ptr() if lse_accum is not None else None
    p.o_accum = o_accum.data_ptr() if o_accum is not None else None
    return p


def _run_both(t):
    import flashmla_windows_linux_sm120_b200 as fm
    from flashmla_windows_linux_sm120_b200._cabi import check, lib
    data = gen.make_decode_case(t)
    d = dict(q=data.q.cuda(), kcache=data.blocked_k.cuda(), block_table=data.block_table.cuda(),
             lens=data.cache_seqlens.cuda())
    md, ns = fm.get_mla_metadata(d["lens"], t.s_q * t.h_q // t.h_kv, t.h_kv)
    assert int(ns[-1]) > t.b, "the case must contain split requests, otherwise no scratch is exercised"
    stream = torch.cuda.current_stream().cuda_stream
    slots = t.b + md.shape[0]

    def outputs():
        return (torch.full((t.b, t.s_q, t.h_q, 512), float("nan"), dtype=torch.bfloat16, device="cuda"),
                torch.full((t.b, t.h_q, t.s_q), float("nan"), dtype=torch.float32, device="cuda"))

    out_a, lse_a = outputs()
    lse_acc = torch.empty((slots, t.s_q * t.h_q), dtype=torch.float32, device="cuda")
    o_acc = torch.empty((slots, t.s_q * t.h_q, 512), dtype=torch.float32, device="cuda")
    pa = _params(d, t, md, ns, out_a, lse_a, lse_acc, o_acc)
    check(lib.fmla_fwd_kvcache_mla(C.byref(pa), stream))

    out_b, lse_b = outputs()
    pb = _params(d, t, md, ns, out_b, lse_b, None, None)        # no scratch pointers at all
    check(lib.fmla_fwd_kvcache_mla_static_scratch(C.byref(pb), stream))
    torch.cuda.synchronize()
    return data, (out_a.cpu(), lse_a.cpu()), (out_b.cpu(), lse_b.cpu())


def test_static_scratch_matches_regular_entry_point_twice_in_a_row():
    cases = [gen.DecodeCase(b=3, s_q=2, s_k=3000, is_varlen=True, is_causal=True, h_q=128, seed=11),
             gen.DecodeCase(b=2, s_q=1, s_k=1500, is_varlen=True, is_causal=False, h_q=64, seed=12)]
    from oracle import decode
    for n, t in enumerate(cases):
        data, (out_a, lse_a), (out_b, lse_b) = _run_both(t)
        assert not torch.isnan(out_b.float()).any() and not torch.isnan(lse_b).any()
        assert torch.equal(out_b, out_a) and torch.equal(lse_b, lse_a)
        if n == 0:
            ref_out, ref_lse = decode.decode_ref(data.cache_seqlens, data.block_table, data.q, data.blocked_k, 512, t.is_causal)
            U.assert_out_lse(out_b, lse_b, ref_out, ref_lse, what="static scratch vs oracle")


def test_static_scratch_rejects_oversized_problems():
    from flashmla_windows_linux_sm120_b200._cabi import DecodeParams, lib
    limit = lib.fmla_static_scratch_max_rows()
    p = DecodeParams()
    p.b, p.s_q, p.h_q, p.h_k, p.d, p.d_v, p.num_sm_parts = 4096, 2, 128, 1, 576, 512, 37
    assert (p.b + p.num_sm_parts) * p.s_q * p.h_q > limit
    assert lib.fmla_fwd_kvcache_mla_static_scratch(C.byref(p), None) == 1
    msg = lib.fmla_last_error_message().decode()
    assert str(limit) in msg and "partial rows" in msg
