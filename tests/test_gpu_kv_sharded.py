"""KV-sharded decode: the per-rank push kernel and the flag-waiting merge kernel.

On one GPU the ranks are emulated in sequence inside one process (every "peer" buffer is local and all
pushes have completed before the merge is launched, so no kernel ever waits for another launch).
With two or more GPUs the same path runs as one process per GPU over symmetric memory
(tests/multi_gpu/run_kv_sharded.py), peer transport against the NCCL all_gather baseline.
"""
import ctypes as C
import os
import subprocess
import sys

import pytest
import torch

import gpu_util as U
from oracle import decode, gen

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _status(reset=True):
    from flashmla_windows_linux_sm120_b200._cabi import lib
    st = C.c_int(0)
    rc = lib.fmla_device_status(C.byref(st), int(reset))
    return rc, st.value


@pytest.mark.parametrize("world,seqlen,h_q,b", [(4, 5000, 128, 1), (8, 700, 64, 2), (2, 64, 128, 1)])
def test_emulated_ranks_on_one_gpu(world, seqlen, h_q, b):
    import flashmla_windows_linux_sm120_b200 as fm
    from flashmla_windows_linux_sm120_b200 import parallel
    t = gen.DecodeCase(b=b, s_q=1, s_k=seqlen, h_q=h_q, seed=21)
    d = gen.make_decode_case(t)
    q, kc = d.q.cuda(), d.blocked_k.cuda()
    buf = parallel.PartialBuffers(world, b * h_q, "cuda")
    counter = torch.zeros((1,), dtype=torch.int32, device="cuda")
    for epoch in (1, 2, 3):                            # three steps: both buffer sets, flags and counter reused
        dst = [buf.ptrs(epoch)]
        for r in range(world):
            lo, hi = parallel.shard_kv_pages(seqlen, world)[r]
            bt = d.block_table[:, lo // 64:(hi + 63) // 64].contiguous()
            if bt.shape[1] == 0:
                bt = torch.zeros((b, 1), dtype=torch.int32)
            lens = torch.full((b,), hi - lo, dtype=torch.int32).cuda()
            md, ns = fm.get_mla_metadata(lens, h_q, 1)
            parallel.push_partial(q, kc, bt.cuda(), lens, md, ns, 576 ** -0.5, r, dst, epoch, counter)
        torch.cuda.synchronize()
        assert buf.flags[epoch & 1].cpu().tolist() == [epoch] * world and int(counter) == 0
        out, lse = parallel.merge_partials(buf, epoch, max_polls=1000)
        torch.cuda.synchronize()
        ref_out, ref_lse = decode.decode_ref(d.cache_seqlens, d.block_table, d.q, d.blocked_k, 512, False)
        U.assert_out_lse(out.cpu().view(b, 1, h_q, 512), lse.cpu().view(b, h_q, 1), ref_out, ref_lse)
    assert _status() == (0, 0)


def test_merge_times_out_on_a_flag_that_never_arrives():
    """A rank that never publishes: the merge gives up after its poll budget, reports through the status
    word and leaves the GPU usable."""
    from flashmla_windows_linux_sm120_b200 import parallel
    buf = parallel.PartialBuffers(2, 128, "cuda")
    buf.lse.fill_(0.0)
    buf.flags[1, 0] = 7                                # epoch 7 uses buffer set 1; rank 1 never writes its flag
    out, lse = parallel.merge_partials(buf, 7, max_polls=200)
    torch.cuda.synchronize()
    # the next library call on this device sees the failure without anybody asking for it
    with pytest.raises(RuntimeError, match="bounded device-side wait"):
        parallel.merge_partials(buf, 7, max_polls=200)
    rc, code = _status(reset=True)
    assert rc == 5 and code == 20                      # FMLA_ERR_DEVICE_TIMEOUT, merge code
    assert _status() == (0, 0)                         # cleared; the context still works
    buf.flags[1, 1] = 7
    out, lse = parallel.merge_partials(buf, 7, max_polls=200)
    torch.cuda.synchronize()
    assert _status() == (0, 0) and torch.isfinite(lse).all()


def test_a_fast_rank_may_push_the_next_step_before_a_slow_rank_has_merged():
    """Rank 0 runs ahead: it pushes step 2 while the partials of step 1 have not been merged yet.  The two
    steps use different buffer sets, so the merge of step 1 still finds every slot of step 1 intact (with a
    single set it would find epoch 2 in slot 0 and run out of polls)."""
    import flashmla_windows_linux_sm120_b200 as fm
    from flashmla_windows_linux_sm120_b200 import parallel
    world, seqlen, h_q, b = 2, 3000, 128, 1
    d1 = gen.make_decode_case(gen.DecodeCase(b=b, s_q=1, s_k=seqlen, h_q=h_q, seed=31))
    d2 = gen.make_decode_case(gen.DecodeCase(b=b, s_q=1, s_k=seqlen, h_q=h_q, seed=32))
    buf = parallel.PartialBuffers(world, b * h_q, "cuda")
    counter = torch.zeros((1,), dtype=torch.int32, device="cuda")

    def push(d, r, epoch):
        lo, hi = parallel.shard_kv_pages(seqlen, world)[r]
        bt = d.block_table[:, lo // 64:(hi + 63) // 64].contiguous().cuda()
        lens = torch.full((b,), hi - lo, dtype=torch.int32).cuda()
        md, ns = fm.get_mla_metadata(lens, h_q, 1)
        parallel.push_partial(d.q.cuda(), d.blocked_k.cuda(), bt, lens, md, ns, 576 ** -0.5, r, [buf.ptrs(epoch)], epoch, counter)

    push(d1, 0, 1)
    push(d1, 1, 1)
    push(d2, 0, 2)              # rank 0 is already one step ahead
    out1, lse1 = parallel.merge_partials(buf, 1, max_polls=1000)
    push(d2, 1, 2)
    out2, lse2 = parallel.merge_partials(buf, 2, max_polls=1000)
    torch.cuda.synchronize()
    assert _status() == (0, 0)
    for d, out, lse in ((d1, out1, lse1), (d2, out2, lse2)):
        ref_out, ref_lse = decode.decode_ref(d.cache_seqlens, d.block_table, d.q, d.blocked_k, 512, False)
        U.assert_out_lse(out.cpu().view(b, 1, h_q, 512), lse.cpu().view(b, h_q, 1), ref_out, ref_lse)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs 2 GPUs")
def test_two_gpus_peer_memory_vs_nccl():
    n = min(torch.cuda.device_count(), 8)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}", "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(ROOT, "tests", "multi_gpu", "run_kv_sharded.py"), "--seqlen", "20000"]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-3000:] + r.stderr[-3000:]
    assert "OK" in r.stdout
