"""Bit-exact scheduler parity, combine parity, FP8 cache writer parity (GPU)."""
import ctypes as C
import math

import pytest
import torch

from oracle import combine, gen, quant, scheduler

pytestmark = pytest.mark.gpu


def _gpu_metadata(seqlens, parts, topk):
    from flashmla_windows_linux_sm120_b200._cabi import check, lib
    s = torch.tensor(seqlens, dtype=torch.int32, device="cuda")
    md = torch.full((parts, 8), -7, dtype=torch.int32, device="cuda")
    ns = torch.full((len(seqlens) + 1,), -7, dtype=torch.int32, device="cuda")
    check(lib.fmla_get_mla_metadata(s.data_ptr(), len(seqlens), parts, topk, md.data_ptr(), ns.data_ptr(),
                                    torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    return md.cpu().tolist(), ns.cpu().tolist()


@pytest.mark.parametrize("seqlens,parts,topk", [
    ([1024] * 4, 74, -1),
    ([4096] * 8, 4, -1),
    ([0, 100, 0, 5000], 10, -1),
    ([1], 148, -1),
    ([0], 3, -1),
    ([37, 64, 65, 128, 129, 4095, 4097, 1, 0, 20000], 74, -1),
    ([5] * 64, 74, 2048),
    ([5] * 3, 37, 128),
    (list(range(3072, 5120, 16)), 74, -1),
    (list(range(1, 700)), 148, -1),
    ([1 << 20], 74, -1),
    ([4096] * 3000, 74, -1),                       # more requests than one pass of the block-wide scan
    ([2048] * 64, 74, 2048),
])
def test_scheduler_bit_exact(seqlens, parts, topk):
    """The CUDA scheduler against the integer statement of its own algorithm (oracle.scheduler.schedule_cut_ref),
    plus the invariants every consumer relies on; the balance is compared with the reference's greedy walk."""
    md, ns = _gpu_metadata(seqlens, parts, topk)
    rmd, rns = scheduler.schedule_cut_ref(seqlens, parts, topk)
    assert md == rmd
    assert ns == rns
    scheduler.check_schedule_invariants(md, ns, seqlens, topk)
    assert ns[-1] <= len(seqlens) + parts


def test_num_sm_parts_formula():
    from flashmla_windows_linux_sm120_b200._cabi import check, lib
    sm = torch.cuda.get_device_properties(0).multi_processor_count
    for (rows, h_k, h_q, sparse) in [(128, 1, 128, False), (256, 1, 128, False), (16, 1, 16, False), (64, 2, 128, False),
                                     (128, 1, 128, True), (256, 1, 128, True), (64, 1, 64, True)]:
        n = C.c_int(0)
        check(lib.fmla_get_num_sm_parts(0, rows, h_k, h_q, int(sparse), int(sparse), C.byref(n)))
        assert n.value == scheduler.num_sm_parts_ref(sm, rows, h_k, h_q, sparse)


@pytest.mark.parametrize("nparts,rows", [(2, 128), (8, 128), (3, 5), (100, 17), (148, 64)])
def test_combine_partials(nparts, rows):
    from flashmla_windows_linux_sm120_b200 import cuda_sm100
    torch.manual_seed(nparts * 1000 + rows)
    lse = torch.randn(nparts, rows) * 4
    lse[torch.rand(nparts, rows) < 0.2] = float("-inf")
    lse[:, 0] = float("-inf")                              # a row with no contribution at all
    o = torch.randn(nparts, rows, 512)
    o[torch.isinf(lse)] = 0
    out, glse = cuda_sm100.combine_partials(lse.cuda(), o.cuda())
    ref_o, ref_lse = combine.combine_ref(lse, o)
    assert torch.equal(torch.isinf(glse.cpu()), torch.isinf(ref_lse))
    fin = torch.isfinite(ref_lse)
    assert (glse.cpu()[fin] - ref_lse[fin]).abs().max() <= 1e-5
    assert (out.cpu().float() - ref_o.to(torch.bfloat16).float()).abs().max() <= 2 ** -7 * max(1.0, float(ref_o.abs().max()))
    assert (out.cpu()[0] == 0).all() and glse.cpu()[0] == float("inf")


def test_fp8_cache_writer_bit_exact():
    from flashmla_windows_linux_sm120_b200 import cuda_sm100
    torch.manual_seed(3)
    kv = (torch.randn(6, 64, 1, 576) * torch.rand(6, 64, 1, 1) * 3).to(torch.bfloat16)
    ref = quant.quantize_k_cache(kv, 512, 128).view(torch.uint8)
    got = cuda_sm100.quantize_kv_fp8(kv.cuda()).view(torch.uint8).cpu()
    assert torch.equal(got.reshape(-1, 656), ref.reshape(-1, 656))
    # scattered write into an existing cache
    cache = torch.zeros(10 * 64, 656, dtype=torch.uint8, device="cuda")
    slots = torch.randperm(10 * 64)[:6 * 64].to(torch.int32)
    cuda_sm100.quantize_kv_fp8(kv.cuda().reshape(-1, 576), cache=cache.view(torch.float8_e4m3fn), dst_slots=slots.cuda())
    assert torch.equal(cache.cpu()[slots.long()], ref.reshape(-1, 656))
