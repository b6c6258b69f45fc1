"""Parity at the benchmarked configurations, with the benchmark's own value distribution (bf16 N(0,1)).

Each test builds the workload object `bench.py` times (same generator, same seed, same API call), runs one
step on the GPU at full size, and compares a sample of the outputs with the CPU oracle: the oracle cannot
finish the full shapes in seconds, so it is run on a subset of requests / query tokens / heads that covers
the corner positions of the schedule (first and last request of the batch, first and last query token a
persistent CTA walks, shortest and longest sequence).  `bench.py` repeats the same check after its timed
region and reports it as `parity_checked`.
Reference for checking performance shapes for correctness too: tests/test_flash_mla_prefill.py:174-179,
tests/test_flash_mla_decoding.py:323-332.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(key, **kw):
    import bench
    wl = bench.make_workload(key)
    for k, v in kw.items():
        setattr(wl, k, v)
    wl.setup(torch.device("cuda", 0), 0)
    try:
        d = wl.parity()
    finally:
        wl.release()
    print(f"[parity {key}] {d}")
    assert d["ok"], d
    return d


@pytest.mark.parametrize("key", ["dense_decode", "dense_decode_sq2"])
def test_dense_decode_b128_unit_normal(key):
    """b = 128, h_q = 128, lengths U[3072, 5120], s_q = 1 and 2 (causal): 16 requests against decode_ref."""
    d = _run(key)
    assert d["out_max_abs"] <= 2e-3 and d["lse_max_abs"] <= 1e-4      # outputs stay far below 1: the unscaled bounds


def test_dense_decode_b64_h64_single_cta_kernel():
    """The same shape through the one-CTA-per-64-heads kernel (the path every other head count takes):
    h_q = 64 requests."""
    import bench
    wl = bench.DenseDecode(1, batch=64, h_q=64)
    wl.setup(torch.device("cuda", 0), 1)
    try:
        d = wl.parity()
    finally:
        wl.release()
    print(f"[parity dense_decode h_q=64] {d}")
    assert d["ok"], d


def test_sparse_fp8_decode_b64_topk2048():
    """b = 64, s_k = 32768, top-k 2048 of a cache quantised from N(0,1): 4 requests, de-quantised by the codec oracle."""
    _run("sparse_decode")


def test_sparse_prefill_sq4096_topk2048():
    """s_q = 4096 (55-56 query tokens per persistent CTA), s_kv = 32768, top-k 2048: 70 query tokens incl. the
    first and last token of a lane."""
    _run("sparse_prefill")


def test_dense_mha_fwd_bwd_8_sequences():
    """8 sequences U[1024, 8192], h = 128, N(0,1): heads 0 and 127 of the shortest and the longest sequence,
    out / lse / dq / dk / dv against the fp32 autograd oracle."""
    _run("dense_fwd_bwd")
