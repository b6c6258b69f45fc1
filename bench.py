#!/usr/bin/env python
"""Benchmark of the MLA attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

One "step" = one pass of the hot path (the public API call) over one batch of
seeded synthetic input.  Default workload: dense BF16 MLA decode at the
DeepSeek-V3 shape (batch 128 per GPU, s_q 1, 128 heads, d 576/512, sequence
lengths uniform in [3072, 5120], paged cache with a shuffled block table).
Prints ONE JSON line (rank 0).  Timing: CUDA events on the launching stream, W
warm-up steps, K timed steps bracketed by barrier + synchronize, max over ranks.
The working set (~600 MB) is several times the 126 MB L2, so no flush is needed.

`--impl reference` times the reference's CPU algorithm for the same workload
(the oracle port of its torch path) on the host cores, on a bounded sample.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# dram__bytes_read + dram__bytes_write per launch of the dominant kernel, from the committed ncu capture
# of this kernel on this workload (summary committed under profiles/)
TRAFFIC_BYTES = {"dense_decode": 708.7e6}

FALLBACK_HBM_GBS = 6650.0
FALLBACK_BF16_TFLOPS = 1590.0


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            d = json.load(open(path))
            return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                        bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
        except Exception:
            pass
    return dict(hbm_gbs=FALLBACK_HBM_GBS, bf16_tflops=FALLBACK_BF16_TFLOPS, bf16_tflops_sustained=1400.0,
                source="fallback")


# ---------------------------------------------------------------------------------------------
# clocks: sampled in-process through NVML (read-only) while the timed region runs
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting", 0x10: "sync_boost"}

    def __init__(self, index: int, period_s: float = 0.004):
        self.samples, self.reasons, self.period = [], set(), period_s
        self.max_mhz = None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    r = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in self.REASONS.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period)

    def start(self):
        if self.nv is not None:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()

    def stop(self):
        if self._thr is not None:
            self._stop.set()
            self._thr.join(timeout=2)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---------------------------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------------------------
class DenseDecode:
    """Dense BF16 MLA decode at the DeepSeek-V3 shape."""
    metric, unit, dtype = "dense_bf16_mla_decode_bandwidth", "GB/s", "bf16"
    bound = "hbm"
    kernel_name = "mla_tc_kernel<kDense>"
    launches_per_step = 2          # split-KV attention + combine

    def __init__(self, s_q: int = 1, batch: int = 128, h_q: int = 128):
        self.s_q, self.b, self.h_q = s_q, batch, h_q
        self.name = f"dense_bf16_decode b={batch}/gpu s_q={s_q} h_q={h_q} h_kv=1 d=576 dv=512 seqlen~U[3072,5120] page=64"

    def make_host(self, seed: int):
        g = torch.Generator().manual_seed(seed)
        self.lens = torch.randint(3072, 5121, (self.b,), generator=g, dtype=torch.int32)
        nblk = (self.lens + 63) // 64
        total = int(nblk.sum())
        perm = torch.randperm(total, generator=g, dtype=torch.int32)
        self.block_table = torch.full((self.b, int(nblk.max())), 2147480000, dtype=torch.int32)
        o = 0
        for i in range(self.b):
            n = int(nblk[i])
            self.block_table[i, :n] = perm[o:o + n]
            o += n
        self.num_pages = total

    def setup(self, device, seed: int):
        import flashmla_windows_linux_sm120_b200 as fm
        self.fm = fm
        self.make_host(seed)
        torch.manual_seed(seed)
        self.cache = torch.randn((self.num_pages, 64, 1, 576), dtype=torch.bfloat16, device=device)
        self.q = torch.randn((self.b, self.s_q, self.h_q, 576), dtype=torch.bfloat16, device=device)
        self.d_lens = self.lens.to(device)
        self.d_bt = self.block_table.to(device)
        self.md, self.ns = fm.get_mla_metadata(self.d_lens, self.s_q * self.h_q, 1)
        self.h_q_pin = self.q.cpu().pin_memory()
        self.h_bt_pin = self.block_table.pin_memory()
        self.h_lens_pin = self.lens.pin_memory()
        self.h_out = torch.empty((self.b, self.s_q, self.h_q, 512), dtype=torch.bfloat16).pin_memory()
        self.h_lse = torch.empty((self.b, self.h_q, self.s_q), dtype=torch.float32).pin_memory()
        self.device = device

    # reference formulas: tests/test_flash_mla_decoding.py:255-268
    def alg_bytes(self, lens=None):
        lens = self.lens if lens is None else lens
        return int(len(lens) * (self.s_q * self.h_q * 576 * 2 + self.s_q * self.h_q * 512 * 2) + int(lens.sum()) * 1152)

    def alg_flops(self, lens=None):
        lens = self.lens if lens is None else lens
        return int(self.h_q * self.s_q * 2 * (576 + 512) * int(lens.sum()))

    def step(self, events=None):
        from flashmla_windows_linux_sm120_b200 import cuda_sm100
        return cuda_sm100.fwd_kvcache_mla(self.q, self.cache, 512, self.d_lens, self.d_bt, 576 ** -0.5, True, self.md,
                                          self.ns, False, None, profile_events=events)

    # End to end = the serving loop a user of the API writes: the inputs of a step come from pinned host memory,
    # the results go back to pinned host memory, and the copies of neighbouring steps overlap with the kernels
    # (three streams, two sets of buffers).  Every step copies its own inputs and reads its own results.
    def e2e_begin(self):
        dev = self.device
        if not hasattr(self, "_s_in"):
            self._s_in, self._s_cmp, self._s_out = (torch.cuda.Stream(dev) for _ in range(3))
            self._d_q = [torch.empty_like(self.q) for _ in range(2)]
            self._d_bt = [torch.empty_like(self.d_bt) for _ in range(2)]
            self._d_lens = [torch.empty_like(self.d_lens) for _ in range(2)]
            self._h_out = [torch.empty_like(self.h_out).pin_memory() for _ in range(2)]
            self._h_lse = [torch.empty_like(self.h_lse).pin_memory() for _ in range(2)]
            self._ev_in = [torch.cuda.Event() for _ in range(2)]
            self._ev_cmp = [torch.cuda.Event() for _ in range(2)]
            self._ev_out = [torch.cuda.Event() for _ in range(2)]
            self._keep = [None, None]
        self._k = 0
        main = torch.cuda.current_stream(dev)
        for st in (self._s_in, self._s_cmp, self._s_out):
            st.wait_stream(main)

    def step_e2e(self):
        i = self._k & 1
        self._k += 1
        with torch.cuda.stream(self._s_in):
            if self._k > 2:
                self._s_in.wait_event(self._ev_cmp[i])      # the decode that read this set of inputs two steps ago
            self._d_q[i].copy_(self.h_q_pin, non_blocking=True)
            self._d_bt[i].copy_(self.h_bt_pin, non_blocking=True)
            self._d_lens[i].copy_(self.h_lens_pin, non_blocking=True)
            self._ev_in[i].record(self._s_in)
        with torch.cuda.stream(self._s_cmp):
            self._s_cmp.wait_event(self._ev_in[i])
            if self._k > 2:
                # the results of two steps ago are dropped below; whatever reuses their memory on this
                # stream must come after their read-back
                self._s_cmp.wait_event(self._ev_out[i])
            out, lse = self.fm.flash_mla_with_kvcache(self._d_q[i], self.cache, self._d_bt[i], self._d_lens[i], 512,
                                                      self.md, self.ns, causal=True)
            self._ev_cmp[i].record(self._s_cmp)
        with torch.cuda.stream(self._s_out):
            self._s_out.wait_event(self._ev_cmp[i])
            self._h_out[i].copy_(out, non_blocking=True)
            self._h_lse[i].copy_(lse, non_blocking=True)
            self._ev_out[i].record(self._s_out)
        self._keep[i] = (out, lse)

    def e2e_end(self):
        main = torch.cuda.current_stream(self.device)
        for st in (self._s_in, self._s_cmp, self._s_out):
            main.wait_stream(st)

    def e2e_bytes(self):
        h2d = self.h_q_pin.numel() * 2 + self.h_bt_pin.numel() * 4 + self.h_lens_pin.numel() * 4
        d2h = self.h_out.numel() * 2 + self.h_lse.numel() * 4
        return h2d, d2h

    def value_from(self, seconds_per_step, n_gpus_bytes):
        return n_gpus_bytes / seconds_per_step / 1e9

    def cpu_sample(self, n_req: int = 32):
        """The reference's CPU torch path on the first n_req requests of this workload."""
        from oracle import decode
        lens = self.lens[:n_req]
        nb = int(((lens + 63) // 64).max())
        bt = self.block_table[:n_req, :nb].clone()
        used = torch.unique(bt[bt < self.num_pages])
        remap = torch.full((self.num_pages,), -1, dtype=torch.int64)
        remap[used.long()] = torch.arange(len(used))
        bt = torch.where(bt < self.num_pages, remap[bt.clamp(max=self.num_pages - 1).long()].to(torch.int32), bt)
        torch.manual_seed(1)
        cache = torch.randn((len(used), 64, 1, 576), dtype=torch.bfloat16)
        q = torch.randn((n_req, self.s_q, self.h_q, 576), dtype=torch.bfloat16)

        def run():
            return decode.decode_ref(lens, bt, q, cache, 512, self.s_q > 1)
        return run, self.alg_bytes(lens), f"first {n_req} of {self.b} requests ({int(lens.sum())} tokens), oracle.decode.decode_ref"


class SparseDecode:
    """Sparse FP8 MLA decode, batch 64, top-k 2048 of 32768 cached tokens."""
    metric, unit, dtype = "sparse_fp8_mla_decode_tflops", "TFLOP/s", "bf16 (fp8 e4m3 cache)"
    bound = "tensor"
    kernel_name = "mla_tc_kernel<kSparseDecode>"
    launches_per_step = 2

    def __init__(self, batch: int = 64, topk: int = 2048, seqlen: int = 32768, h_q: int = 128):
        self.b, self.topk, self.seqlen, self.h_q, self.s_q = batch, topk, seqlen, h_q, 1
        self.name = f"sparse_fp8_decode b={batch}/gpu s_q=1 h_q={h_q} topk={topk} seqlen_k={seqlen} 656B/token page=64"

    def make_host(self, seed: int):
        pass

    def setup(self, device, seed: int):
        import flashmla_windows_linux_sm120_b200 as fm
        from flashmla_windows_linux_sm120_b200 import cuda_sm100
        self.fm = fm
        torch.manual_seed(seed)
        pages_per = self.seqlen // 64
        npages = self.b * pages_per
        g = torch.Generator(device="cpu").manual_seed(seed)
        perm = torch.randperm(npages, generator=g, dtype=torch.int32)
        self.block_table = perm.view(self.b, pages_per).to(device)
        self.lens = torch.full((self.b,), self.seqlen, dtype=torch.int32, device=device)
        self.cache = torch.empty((npages, 64, 1, 656), dtype=torch.float8_e4m3fn, device=device)
        chunk = 4096
        for p0 in range(0, npages, chunk):     # quantise N(0,1) bf16 KV page by page on the device
            kv = torch.randn((min(chunk, npages - p0), 64, 1, 576), dtype=torch.bfloat16, device=device)
            self.cache[p0:p0 + kv.shape[0]] = cuda_sm100.quantize_kv_fp8(kv)
        idx = torch.empty((self.b, 1, self.topk), dtype=torch.int32, device=device)
        for i in range(self.b):
            logical = torch.randperm(self.seqlen, device=device)[:self.topk]
            idx[i, 0] = self.block_table[i, (logical // 64).long()] * 64 + (logical % 64).to(torch.int32)
        idx[:, :, ::97] = -1                                      # some padding slots
        self.indices = idx
        self.q = torch.randn((self.b, 1, self.h_q, 576), dtype=torch.bfloat16, device=device)
        self.md, self.ns = fm.get_mla_metadata(self.lens, self.h_q, 1, self.h_q, True, self.topk)
        self.device = device

    def alg_bytes(self):
        return int(self.b * (self.h_q * 576 * 2 + self.topk * 656 + self.h_q * 512 * 2))

    def alg_flops(self):
        return int(self.b * self.h_q * 2 * (576 + 512) * self.topk)

    def step(self, events=None):
        return self.fm.flash_mla_with_kvcache(self.q, self.cache, self.block_table, self.lens, 512, self.md, self.ns,
                                              is_fp8_kvcache=True, indices=self.indices)


class SparsePrefill:
    """Sparse MLA prefill forward, s_q 4096, s_kv 32768, top-k 2048 (causally restricted)."""
    metric, unit, dtype = "sparse_mla_prefill_fwd_tflops", "TFLOP/s", "bf16"
    bound = "tensor"
    kernel_name = "mla_tc_kernel<kSparsePrefill>"
    launches_per_step = 1

    def __init__(self, s_q: int = 4096, s_kv: int = 32768, topk: int = 2048, h_q: int = 128):
        self.s_q, self.s_kv, self.topk, self.h_q, self.b = s_q, s_kv, topk, h_q, 1
        self.name = f"sparse_prefill_fwd s_q={s_q}/gpu h_q={h_q} s_kv={s_kv} topk={topk} causal-restricted indices"

    def make_host(self, seed: int):
        pass

    def setup(self, device, seed: int):
        import flashmla_windows_linux_sm120_b200 as fm
        self.fm = fm
        torch.manual_seed(seed)
        self.q = torch.randn((self.s_q, self.h_q, 576), dtype=torch.bfloat16, device=device)
        self.kv = torch.randn((self.s_kv, 1, 576), dtype=torch.bfloat16, device=device)
        idx = torch.empty((self.s_q, 1, self.topk), dtype=torch.int32, device=device)
        for t in range(self.s_q):                       # query t sits at position s_kv - s_q + t
            hi = self.s_kv - self.s_q + t + 1
            idx[t, 0] = torch.randperm(hi, device=device)[:self.topk].to(torch.int32)
        self.indices = idx
        self.scale = 576 ** -0.5

    def alg_bytes(self):
        return int(self.q.numel() * 2 + self.kv.numel() * 2 + self.indices.numel() * 4 + self.s_q * self.h_q * 512 * 2)

    def alg_flops(self):
        return int(2 * (self.h_q * 576 * self.topk + self.h_q * 512 * self.topk) * self.s_q)

    def step(self, events=None):
        return self.fm.flash_mla_sparse_fwd(self.q, self.kv, self.indices, self.scale)


class DenseFwdBwd:
    """Dense causal varlen MHA forward + backward, h 128, d 192/128, 8 sequences U[1024,8192]."""
    metric, unit, dtype = "dense_mha_varlen_fwd_bwd_tflops", "TFLOP/s", "bf16"
    bound = "tensor"
    kernel_name = "dense_fwd_tc_kernel<192> + dense_bwd_*"
    launches_per_step = 4

    def __init__(self, nseq: int = 8, h: int = 128):
        self.nseq, self.h, self.b = nseq, h, nseq
        self.name = f"dense_mha_varlen fwd+bwd {nseq} seqs/gpu L~U[1024,8192] h={h} d=192/128 causal"

    def make_host(self, seed: int):
        pass

    def setup(self, device, seed: int):
        import flashmla_windows_linux_sm120_b200 as fm
        self.fm = fm
        g = torch.Generator().manual_seed(seed)
        lens = torch.randint(1024, 8193, (self.nseq,), generator=g, dtype=torch.int32)
        self.lens = lens
        cu = torch.cumsum(torch.nn.functional.pad(lens, (1, 0)), 0, dtype=torch.int32)
        T = int(lens.sum())
        torch.manual_seed(seed)
        mk = lambda d: torch.randn((T, self.h, d), dtype=torch.bfloat16, device=device).requires_grad_()
        self.q, self.k, self.v = mk(192), mk(192), mk(128)
        self.d_out = torch.randn((T, self.h, 128), dtype=torch.bfloat16, device=device)
        self.cu = cu.to(device)
        self.max_len = int(lens.max())
        self.pairs = int(sum(int(l) * (int(l) + 1) // 2 for l in lens))

    def alg_bytes(self):
        T = self.q.shape[0]
        return int(T * self.h * (192 * 2 * 2 + 128 * 2 * 2) * 2)   # q,k,v,o,do read + dq,dk,dv written (approx.)

    def alg_flops(self):
        return int(self.pairs * self.h * 2 * ((192 + 128) + (3 * 192 + 2 * 128)))

    def step(self, events=None):
        self.q.grad = self.k.grad = self.v.grad = None
        out, lse = self.fm.flash_attn_varlen_func(self.q, self.k, self.v, self.cu, self.cu, self.max_len, self.max_len,
                                                  causal=True)
        out.backward(self.d_out)
        return out, lse


class DenseFwd(DenseFwdBwd):
    """The same workload, forward only (the reference quotes forward and backward separately)."""
    metric = "dense_mha_varlen_fwd_tflops"
    kernel_name = "dense_fwd_tc_kernel<192>"
    launches_per_step = 1

    def __init__(self, nseq: int = 8, h: int = 128):
        super().__init__(nseq, h)
        self.name = f"dense_mha_varlen fwd {nseq} seqs/gpu L~U[1024,8192] h={h} d=192/128 causal"

    def alg_flops(self):
        return int(self.pairs * self.h * 2 * (192 + 128))

    def step(self, events=None):
        with torch.no_grad():
            return self.fm.flash_attn_varlen_func(self.q, self.k, self.v, self.cu, self.cu, self.max_len, self.max_len, causal=True)


WORKLOADS = {
    "dense_fwd": lambda: DenseFwd(),
    "dense_decode": lambda: DenseDecode(1),
    "dense_decode_sq2": lambda: DenseDecode(2),
    "sparse_decode": lambda: SparseDecode(),
    "sparse_prefill": lambda: SparsePrefill(),
    "dense_fwd_bwd": lambda: DenseFwdBwd(),
}


# ---------------------------------------------------------------------------------------------
def dist_env():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    return rank, world, local


def use_all_host_threads():
    """The launcher of multi-process runs sets OMP_NUM_THREADS=1; the CPU legs use every core they can get."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(max(1, n))
    return torch.get_num_threads()


def time_cpu(run, steps, warmup):
    for _ in range(warmup):
        run()
    ts = []
    for _ in range(steps):
        t0 = time.perf_counter()
        run()
        ts.append(time.perf_counter() - t0)
    return statistics.median(ts)


def run_reference(args, wl):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    if not hasattr(wl, "cpu_sample"):
        print(json.dumps({"impl": "reference", "unavailable": "no CPU sample is defined for this workload; the default workload has one"}))
        return
    wl.make_host(args.seed)
    use_all_host_threads()
    run, nbytes, sample = wl.cpu_sample()
    steps = max(1, min(args.steps, 5))
    warm = max(1, min(args.warmup, 1))
    sec = time_cpu(run, steps, warm)
    val = nbytes / sec / 1e9
    cores = torch.get_num_threads()
    line = {"impl": "reference", "metric": wl.metric, "value": val, "unit": wl.unit, "n_gpus": args.gpus, "steps": steps,
            "warmup": warm, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": {"workload": wl.name, "sample": sample},
            "cpu_baseline": {"value": val, "unit": wl.unit, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="dense_decode", choices=sorted(WORKLOADS))
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    wl = WORKLOADS[args.workload]()

    if args.impl == "reference":
        run_reference(args, wl)
        return

    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path (use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    use_dist = world > 1
    if use_dist:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)

    wl.setup(device, args.seed + rank)
    stream = torch.cuda.current_stream()

    def barrier():
        if use_dist:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing (value) + per-kernel timing (roofline) -------------------------
    for _ in range(args.warmup):
        wl.step()
    pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    for a, b in pairs:            # create the handles
        a.record(stream)
        b.record(stream)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)
    barrier()
    sampler.start()
    e0.record(stream)
    for i in range(args.steps):
        wl.step(pairs[i] if wl.bound == "hbm" else None)
    e1.record(stream)
    barrier()
    clocks = sampler.stop()
    total_ms = e0.elapsed_time(e1)
    kern_ms = [a.elapsed_time(b) for a, b in pairs] if wl.bound == "hbm" else []
    t = torch.tensor([total_ms], dtype=torch.float64, device=device)
    if use_dist:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_per_step = float(t.item()) / args.steps
    nbytes = torch.tensor([float(wl.alg_bytes())], dtype=torch.float64, device=device)
    nflops = torch.tensor([float(wl.alg_flops())], dtype=torch.float64, device=device)
    if use_dist:
        dist.all_reduce(nbytes)
        dist.all_reduce(nflops)
    gbs = float(nbytes.item()) / (ms_per_step * 1e-3) / 1e9
    tflops = float(nflops.item()) / (ms_per_step * 1e-3) / 1e12
    value = gbs if wl.bound == "hbm" else tflops

    # ---- end to end through the public API with host buffers -----------------------------------
    e2e = None
    if hasattr(wl, "step_e2e"):
        wl.e2e_begin()
        for _ in range(3):
            wl.step_e2e()
        wl.e2e_end()
        barrier()
        e0.record(stream)
        wl.e2e_begin()
        for _ in range(args.steps):
            wl.step_e2e()
        wl.e2e_end()
        e1.record(stream)
        barrier()
        t = torch.tensor([e0.elapsed_time(e1)], dtype=torch.float64, device=device)
        if use_dist:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item()) / args.steps
        h2d, d2h = wl.e2e_bytes()
        e2e = {"value": float(nbytes.item()) / (e2e_ms * 1e-3) / 1e9, "unit": wl.unit, "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "note": "every step copies q, block_table, cache_seqlens from pinned host memory and reads out, lse back; copies and kernels of neighbouring steps overlap (3 streams, 2 buffer sets); the KV cache is resident device state"}

    if rank == 0:
        peaks = measured_peaks()
        if wl.bound == "hbm":
            k_ms = statistics.mean(kern_ms)
            achieved = wl.alg_bytes() / (k_ms * 1e-3) / 1e9
            roof = {"bound": "hbm", "kernel": wl.kernel_name, "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"], "kernel_ms": k_ms,
                    "algorithmic_bytes_per_launch": wl.alg_bytes(), "traffic": TRAFFIC_BYTES.get(args.workload),
                    "tensor_tflops": wl.alg_flops() / (k_ms * 1e-3) / 1e12,
                    "tensor_frac_of_burst": wl.alg_flops() / (k_ms * 1e-3) / 1e12 / peaks["bf16_tflops"]}
        else:   # whole step timed (these workloads launch their kernels back to back with nothing else)
            achieved = wl.alg_flops() / (ms_per_step * 1e-3) / 1e12
            roof = {"bound": "tensor", "kernel": wl.kernel_name, "achieved": achieved, "peak": peaks["bf16_tflops"],
                    "unit": "TFLOP/s", "frac": achieved / peaks["bf16_tflops"], "peak_source": peaks["source"],
                    "kernel_ms": ms_per_step, "algorithmic_flops_per_launch": wl.alg_flops(), "traffic": None}
        cpu = None
        if not args.no_cpu_baseline and hasattr(wl, "cpu_sample"):
            use_all_host_threads()
            run, cbytes, sample = wl.cpu_sample()
            sec = time_cpu(run, 3, 1)
            cpu = {"value": cbytes / sec / 1e9, "unit": wl.unit, "cores": torch.get_num_threads(), "kind": "port",
                   "sample": sample, "seconds": sec}
        line = {"metric": wl.metric, "value": value, "unit": wl.unit, "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak",
                "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
                "config": {"workload": wl.name, "global_batch": wl.b * world, "parallelism": f"requests sharded x{world}, no collective",
                           "l2": "inputs (>=600 MB per GPU) larger than the 126 MB L2; no flush"},
                "tflops": tflops, "roofline": roof, "cpu_baseline": cpu,
                "e2e": e2e, "gb_per_s": gbs,
                "gpu_launches": wl.launches_per_step * args.steps, "clocks": clocks}
        print(json.dumps(line))
    if use_dist:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
