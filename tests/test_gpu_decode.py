"""GPU parity of get_mla_metadata + flash_mla_with_kvcache against the CPU oracle
(grid modelled on tests/test_flash_mla_decoding.py:293-321 of the reference)."""
import pytest
import torch

import gpu_util as U
from golden_io import load
from oracle import decode, gen, quant, scheduler

pytestmark = pytest.mark.gpu


def _api():
    import flashmla_windows_linux_sm120_b200 as fm
    return fm


def _run_dense(d: gen.DecodeData, t: gen.DecodeCase):
    fm = _api()
    lens = d.cache_seqlens.cuda()
    md, ns = fm.get_mla_metadata(lens, t.s_q * t.h_q // t.h_kv, t.h_kv)
    out, lse = fm.flash_mla_with_kvcache(d.q.cuda(), d.blocked_k.cuda(), d.block_table.cuda(), lens, t.dv, md, ns,
                                         causal=t.is_causal)
    torch.cuda.synchronize()
    return out.cpu(), lse.cpu(), md.cpu(), ns.cpu()


@pytest.mark.parametrize("b,s_q,s_k,varlen,causal,h_q,h_kv", [
    (1, 1, 20, False, False, 128, 1),
    (2, 2, 140, True, True, 128, 1),
    (6, 4, 140, True, True, 128, 1),
    (6, 1, 1500, True, False, 128, 1),
    (2, 2, 4096, True, True, 128, 1),
    (3, 2, 300, True, True, 16, 1),
    (3, 4, 300, False, False, 64, 1),
    (2, 2, 260, True, True, 32, 2),
    (64, 1, 140, True, False, 128, 1),
])
def test_dense_decode(b, s_q, s_k, varlen, causal, h_q, h_kv):
    t = gen.DecodeCase(b=b, s_q=s_q, s_k=s_k, is_varlen=varlen, is_causal=causal, h_q=h_q, h_kv=h_kv)
    d = gen.make_decode_case(t)
    out, lse, md, ns = _run_dense(d, t)
    ref_out, ref_lse = decode.decode_ref(d.cache_seqlens, d.block_table, d.q, d.blocked_k, t.dv, causal)
    U.assert_out_lse(out, lse, ref_out, ref_lse)
    scheduler.check_schedule_invariants(md.tolist(), ns.tolist(), d.cache_seqlens.tolist())


@pytest.mark.parametrize("b,s_q,s_k,varlen,causal,h_q,h_kv", [
    (6, 1, 1500, True, False, 128, 1),
    (2, 2, 4096, True, True, 128, 1),
    (2, 2, 260, True, True, 32, 2),
])
def test_dense_decode_fp16(b, s_q, s_k, varlen, causal, h_q, h_kv):
    """float16 queries and cache (the reference test's --dtype fp16, tests/test_flash_mla_decoding.py:347-359)."""
    t = gen.DecodeCase(b=b, s_q=s_q, s_k=s_k, is_varlen=varlen, is_causal=causal, h_q=h_q, h_kv=h_kv)
    d = gen.make_decode_case(t)
    d.q = d.q.to(torch.float16)
    d.blocked_k = d.blocked_k.to(torch.float16)
    out, lse, md, ns = _run_dense(d, t)
    assert out.dtype == torch.float16
    ref_out, ref_lse = decode.decode_ref(d.cache_seqlens, d.block_table, d.q, d.blocked_k, t.dv, causal)
    U.assert_out_lse(out, lse, ref_out, ref_lse)


@pytest.mark.parametrize("seed", range(10))
def test_dense_decode_random_shapes(seed):
    """Seeded random shapes: batch, queries per request, heads, kv heads, lengths (some zero), causal or not."""
    import random
    rng = random.Random(1000 + seed)
    h_kv = rng.choice([1, 1, 2])
    h_q = rng.choice([16, 64, 128]) * h_kv if h_kv == 2 else rng.choice([16, 64, 128])
    t = gen.DecodeCase(b=rng.randint(1, 9), s_q=rng.choice([1, 1, 2, 3]), s_k=rng.choice([30, 200, 700, 2300]),
                       is_varlen=True, is_causal=rng.random() < 0.5, h_q=min(h_q, 128), h_kv=h_kv,
                       zero_seqlen=rng.random() < 0.3, seed=seed)
    d = gen.make_decode_case(t)
    out, lse, md, ns = _run_dense(d, t)
    ref_out, ref_lse = decode.decode_ref(d.cache_seqlens, d.block_table, d.q, d.blocked_k, t.dv, t.is_causal)
    U.assert_out_lse(out, lse, ref_out, ref_lse)
    scheduler.check_schedule_invariants(md.tolist(), ns.tolist(), d.cache_seqlens.tolist())


def test_dense_decode_zero_length_requests():
    t = gen.DecodeCase(b=16, s_q=2, s_k=500, is_varlen=True, is_causal=True, zero_seqlen=True)
    d = gen.make_decode_case(t)
    assert (d.cache_seqlens == 0).any()
    out, lse, _, _ = _run_dense(d, t)
    ref_out, ref_lse = decode.decode_ref(d.cache_seqlens, d.block_table, d.q, d.blocked_k, t.dv, True)
    U.assert_out_lse(out, lse, ref_out, ref_lse)


def test_dense_decode_unit_normal_values():
    # benchmark value distribution: bf16 N(0,1) q and kv
    t = gen.DecodeCase(b=4, s_q=1, s_k=1024, h_q=16, unit_normal=True)
    d = gen.make_decode_case(t)
    out, lse, _, _ = _run_dense(d, t)
    ref_out, ref_lse = decode.decode_ref(d.cache_seqlens, d.block_table, d.q, d.blocked_k, t.dv, False)
    U.assert_out_lse(out, lse, ref_out, ref_lse, out_cos=2e-5)


@pytest.mark.parametrize("name", ["decode_dense_causal", "decode_dense_plain", "decode_dense_zero", "decode_fallback_path"])
def test_dense_decode_golden(name):
    """CUDA path against outputs stored from the reference's own torch code."""
    fm = _api()
    g = load(name)
    b, s_q, h_q, _ = g["q"].shape
    lens = g["cache_seqlens"].cuda()
    md, ns = fm.get_mla_metadata(lens, s_q * h_q, 1)
    out, lse = fm.flash_mla_with_kvcache(g["q"].cuda(), g["blocked_k"].cuda(), g["block_table"].cuda(), lens, 512, md, ns,
                                         causal=bool(g.get("is_causal", 0)))
    U.assert_out_lse(out.cpu(), lse.cpu(), g["out"], g["lse"])


def _run_sparse(d: gen.DecodeData, t: gen.DecodeCase, kq):
    fm = _api()
    lens = d.cache_seqlens.cuda()
    md, ns = fm.get_mla_metadata(lens, t.s_q * t.h_q // t.h_kv, t.h_kv, t.h_q, True, t.topk)
    out, lse = fm.flash_mla_with_kvcache(d.q.cuda(), kq.cuda(), d.block_table.cuda(), lens, t.dv, md, ns,
                                         is_fp8_kvcache=True, indices=d.indices.cuda())
    torch.cuda.synchronize()
    return out.cpu(), lse.cpu()


@pytest.mark.parametrize("b,s_q,s_k,topk,h_q,invalid", [
    (1, 1, 140, 128, 128, False),
    (2, 2, 4096, 128, 128, False),
    (6, 4, 4096, 2048, 128, False),
    (2, 2, 1000, 2048, 128, False),       # fewer tokens than topk: -1 padding
    (3, 1, 600, 256, 64, False),
    (4, 2, 4096, 128, 128, True),         # every index invalid
])
def test_sparse_fp8_decode(b, s_q, s_k, topk, h_q, invalid):
    t = gen.DecodeCase(b=b, s_q=s_q, s_k=s_k, is_varlen=True, topk=topk, h_q=h_q, all_indices_invalid=invalid)
    d = gen.make_decode_case(t)
    kq = quant.quantize_k_cache(d.blocked_k, t.dv, 128)
    kd = quant.dequantize_k_cache(kq)
    out, lse = _run_sparse(d, t, kq)
    ref_out, ref_lse = decode.decode_ref(d.cache_seqlens, d.block_table, d.q, kd, t.dv, False, d.abs_indices)
    U.assert_out_lse(out, lse, ref_out, ref_lse)


def test_sparse_fp8_decode_logical_indices():
    """Token positions mapped through the block table inside the kernel give exactly what the caller-side remap
    to physical slots gives."""
    fm = _api()
    t = gen.DecodeCase(b=5, s_q=2, s_k=700, is_varlen=True, topk=128, h_q=128)
    d = gen.make_decode_case(t)
    kq = quant.quantize_k_cache(d.blocked_k, t.dv, 128)
    out_p, lse_p = _run_sparse(d, t, kq)
    lens = d.cache_seqlens.cuda()
    md, ns = fm.get_mla_metadata(lens, t.s_q * t.h_q, 1, t.h_q, True, t.topk)
    out_l, lse_l = fm.flash_mla_sparse_decode_logical_indices(d.q.cuda(), kq.cuda(), d.block_table.cuda(), lens, t.dv, md, ns,
                                                              d.abs_indices.cuda())
    torch.cuda.synchronize()
    assert torch.equal(out_l.cpu(), out_p) and torch.equal(lse_l.cpu(), lse_p)


@pytest.mark.parametrize("name", ["decode_sparse_fp8", "decode_sparse_fp8_pad"])
def test_sparse_fp8_decode_golden(name):
    fm = _api()
    g = load(name)
    b, s_q, h_q, _ = g["q"].shape
    topk = g["indices"].shape[-1]
    lens = g["cache_seqlens"].cuda()
    md, ns = fm.get_mla_metadata(lens, s_q * h_q, 1, h_q, True, topk)
    out, lse = fm.flash_mla_with_kvcache(g["q"].cuda(), g["blocked_k_quant"].cuda(), g["block_table"].cuda(), lens, 512,
                                         md, ns, is_fp8_kvcache=True, indices=g["indices"].cuda())
    U.assert_out_lse(out.cpu(), lse.cpu(), g["out"], g["lse"])


def test_decode_step_replays_from_a_cuda_graph():
    """Scheduler + attention + combine of one decode step captured into a CUDA graph (after one eager warm-up
    call) and replayed on new query values give the eager result bit for bit."""
    fm = _api()
    t = gen.DecodeCase(b=8, s_q=1, s_k=900, is_varlen=True, h_q=128)
    d = gen.make_decode_case(t)
    lens, bt, cache = d.cache_seqlens.cuda(), d.block_table.cuda(), d.blocked_k.cuda()
    q_static = d.q.cuda().clone()

    def step(q):
        md, ns = fm.get_mla_metadata(lens, t.s_q * t.h_q // t.h_kv, t.h_kv)
        return fm.flash_mla_with_kvcache(q, cache, bt, lens, t.dv, md, ns, causal=False)

    step(q_static)                       # warm-up: driver entry points, function attributes, allocator pools
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out_g, lse_g = step(q_static)
    for seed in (1, 2):
        torch.manual_seed(seed)
        q_new = (torch.randn_like(q_static.float()) / 10).to(q_static.dtype)
        q_static.copy_(q_new)
        graph.replay()
        torch.cuda.synchronize()
        out_e, lse_e = step(q_new)
        torch.cuda.synchronize()
        assert torch.equal(out_g, out_e) and torch.equal(lse_g, lse_e)


def test_argument_errors():
    fm = _api()
    t = gen.DecodeCase(b=1, s_q=1, s_k=64, h_q=16)
    d = gen.make_decode_case(t)
    lens = d.cache_seqlens.cuda()
    md, ns = fm.get_mla_metadata(lens, 16, 1)
    with pytest.raises(RuntimeError):
        fm.flash_mla_with_kvcache(d.q.cuda()[..., :512].contiguous(), d.blocked_k.cuda(), d.block_table.cuda(), lens, 512, md, ns)
    with pytest.raises(RuntimeError):
        fm.flash_mla_with_kvcache(d.q.cuda(), d.blocked_k.cuda(), d.block_table.cuda().long(), lens, 512, md, ns)
    with pytest.raises(RuntimeError):   # query and cache must have one dtype
        fm.flash_mla_with_kvcache(d.q.cuda().half(), d.blocked_k.cuda(), d.block_table.cuda(), lens, 512, md, ns)


@pytest.mark.parametrize("s_q", [1, 2])
def test_dense_decode_merge_in_kernel_is_bit_equal_to_the_merge_kernel(s_q):
    """128 heads: the CTA pair kernel can merge split requests itself (arrival counters) instead of leaving it to
    the dependent-launched merge kernel.  Same partials, same order of summation: identical bits, twice in a row
    (the counters must have returned to zero)."""
    from flashmla_windows_linux_sm120_b200 import cuda_sm100
    fm = _api()
    t = gen.DecodeCase(b=6, s_q=s_q, s_k=2500, is_varlen=True, is_causal=True, h_q=128, seed=5)
    d = gen.make_decode_case(t)
    lens, bt, cache, q = d.cache_seqlens.cuda(), d.block_table.cuda(), d.blocked_k.cuda(), d.q.cuda()
    md, ns = fm.get_mla_metadata(lens, t.s_q * t.h_q, 1)
    assert int(ns[-1]) > t.b
    ref = cuda_sm100.fwd_kvcache_mla(q, cache, 512, lens, bt, 576 ** -0.5, True, md, ns, merge_in_kernel=False)
    for _ in range(2):
        got = cuda_sm100.fwd_kvcache_mla(q, cache, 512, lens, bt, 576 ** -0.5, True, md, ns, merge_in_kernel=True)
        torch.cuda.synchronize()
        assert torch.equal(got[0], ref[0]) and torch.equal(got[1], ref[1])
    r_out, r_lse = decode.decode_ref(d.cache_seqlens, d.block_table, d.q, d.blocked_k, 512, True)
    U.assert_out_lse(got[0].cpu(), got[1].cpu(), r_out, r_lse, what=f"merge in kernel s_q={s_q}")


def _device_status(reset=True):
    import ctypes as C

    from flashmla_windows_linux_sm120_b200._cabi import lib
    st = C.c_int(0)
    rc = lib.fmla_device_status(C.byref(st), int(reset))
    return rc, st.value


@pytest.mark.parametrize("h_q,b", [(128, 21), (64, 42)])
def test_no_merge_kernel_when_no_request_is_split(h_q, b):
    """Requests of equal cost (2 blocks + 5 of overhead) whose number makes the pitch of the cuts equal to that
    cost: the schedule splits none of them, the binding reads that back once (remembered on the metadata tensor)
    and the merge kernel is not launched.  Same results."""
    fm = _api()
    t = gen.DecodeCase(b=b, s_q=1, s_k=600, is_varlen=True, topk=128, h_q=h_q)
    d = gen.make_decode_case(t)
    kq = quant.quantize_k_cache(d.blocked_k, t.dv, 128)
    kd = quant.dequantize_k_cache(kq)
    lens = d.cache_seqlens.cuda()
    md, ns = fm.get_mla_metadata(lens, t.s_q * t.h_q, 1, t.h_q, True, t.topk)
    assert int(ns[t.b]) == t.b                      # no request is split
    for _ in range(2):                              # the second call uses the remembered answer
        out, lse = fm.flash_mla_with_kvcache(d.q.cuda(), kq.cuda(), d.block_table.cuda(), lens, t.dv, md, ns,
                                             is_fp8_kvcache=True, indices=d.indices.cuda())
        torch.cuda.synchronize()
        assert ns._fmla_no_split is True
        ref_out, ref_lse = decode.decode_ref(d.cache_seqlens, d.block_table, d.q, kd, t.dv, False, d.abs_indices)
        U.assert_out_lse(out.cpu(), lse.cpu(), ref_out, ref_lse)
    assert _device_status() == (0, 0)


def test_a_wrong_no_split_hint_is_reported():
    """A caller that rules out split requests although the schedule has some gets a device status, not silently
    unmerged partials."""
    fm = _api()
    t = gen.DecodeCase(b=3, s_q=1, s_k=900, h_q=128, is_varlen=True)
    d = gen.make_decode_case(t)
    lens = d.cache_seqlens.cuda()
    md, ns = fm.get_mla_metadata(lens, t.s_q * t.h_q, 1)
    assert int(ns[t.b]) > t.b                       # some request is split
    ns._fmla_no_split = True                        # what a stale or wrong answer would look like
    fm.flash_mla_with_kvcache(d.q.cuda(), d.blocked_k.cuda(), d.block_table.cuda(), lens, t.dv, md, ns, causal=False)
    torch.cuda.synchronize()
    rc, code = _device_status(reset=True)
    assert rc == 5 and code == 41
    assert _device_status() == (0, 0)
    ns._fmla_no_split = False
    out, lse = fm.flash_mla_with_kvcache(d.q.cuda(), d.blocked_k.cuda(), d.block_table.cuda(), lens, t.dv, md, ns, causal=False)
    torch.cuda.synchronize()
    ref_out, ref_lse = decode.decode_ref(d.cache_seqlens, d.block_table, d.q, d.blocked_k, t.dv, False)
    U.assert_out_lse(out.cpu(), lse.cpu(), ref_out, ref_lse)
