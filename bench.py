#!/usr/bin/env python
"""Benchmark of the MLA attention hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]
                    [--small] [--no-extras] [--no-cpu-baseline] [--no-sustained] [--no-graph]

One "step" = one pass of the hot path (the public API call) over one batch of seeded synthetic input.
Default workload: dense BF16 MLA decode at the DeepSeek-V3 shape (batch 128 per GPU, s_q 1, 128 heads,
d 576/512, sequence lengths uniform in [3072, 5120], paged cache with a shuffled block table).
Prints ONE JSON line (rank 0).  Timing: CUDA events on the launching stream, W warm-up steps, K timed
steps bracketed by barrier + synchronize, max over ranks.  Every working set is several times the 126 MB
L2 (or, for the sparse prefill, L2-resident by the nature of the workload), so no flush is needed.

The line of the default run also carries, outside the headline timing:
  parity_checked  a sample of the step's outputs compared with the CPU oracle after the timed region
  sustained       the same step repeated for at least one second (clocks sampled over that stretch)
  workloads       the other configurations (sparse FP8 decode, sparse prefill, dense MHA forward and
                  forward+backward, dense decode at s_q = 2, the KV-sharded 1 M-token decode), each for
                  >= 20 steps with its own roofline fraction, parity sample and clocks
  e2e.copy_only   the same host<->device copies without the kernel (what the host fabric alone allows)

`--impl reference` times the reference's CPU algorithm for the same workload (the oracle port of its torch
path) on the host cores, on a bounded sample.  `--small` shrinks every workload to a few hundred MB for
profiler captures.
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
import traceback

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# dram__bytes_read + dram__bytes_write per launch of the dominant kernel, from ncu captures of that kernel
# (summaries under profiles/).  "full" = captured on the full workload; otherwise bytes per unit of a small
# case, scaled by the units one launch of the benchmark workload processes (traffic grows in proportion).
TRAFFIC = {
    # mla_pair_kernel<decode>: 640.56 MB read + 27.04 MB written in one launch over 526 851 cached tokens
    "dense_decode": {"per_token": (640556288 + 27036672) / 526851, "unit": "cached token", "source": "full-size capture (3 metrics, 1 pass)"},
    # mla_pair_kernel<sparse decode>, --small case (16 requests): 27.26 MB read + 0.03 MB written
    "sparse_decode": {"per_request": (27259648 + 25856) / 16, "unit": "request of 2048 indices", "source": "small case (16 requests), scaled by requests"},
    # mla_pair_kernel<prefill>, --small case (512 query tokens): 125.76 MB read + 45.35 MB written, of which the
    # kv tensor (37.7 MB) is read once whatever the number of query tokens
    "sparse_prefill": {"fixed": 32768 * 1152.0, "per_query_token": (125763840 + 45354240 - 32768 * 1152) / 512, "unit": "query token",
                       "source": "small case (512 query tokens), scaled by query tokens"},
}

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
# clocks: sampled in-process through NVML (read-only) while a timed region runs
# ---------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake_slowdown", 0x2: "applications_clocks_setting", 0x10: "sync_boost"}

    def __init__(self, index: int, period_s: float = 0.002):
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
        return self

    def stop(self):
        if self._thr is not None:
            self._stop.set()
            self._thr.join(timeout=2)
        return {"sm_mhz": statistics.median(self.samples) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def out_bound(ref_out) -> float:
    """2e-3 while the reference output stays within [-1, 1].  A 16-bit output of magnitude in [B/2, B) is rounded
    with a step of up to 1.95e-3 * B, so above 1 the bound is 2.5e-3 * B, B = the power of two above the largest
    reference magnitude (rounding step plus the same relative allowance for the arithmetic)."""
    m = float(ref_out.float().abs().max())
    return 2e-3 if m <= 1.0 else 2.5e-3 * 2.0 ** math.ceil(math.log2(m))


def _errs(out, ref_out, lse=None, ref_lse=None):
    """Largest absolute errors against the oracle; a NaN anywhere counts as an infinite error (it would otherwise
    vanish in a `max()` with an earlier finite value)."""
    from oracle.check import max_abs_diff

    def err(a, b):
        e = max_abs_diff(a, b)
        return e if e == e else float("inf")
    d = {"out_max_abs": err(out, ref_out), "out_bound": out_bound(ref_out)}
    if lse is not None:
        d["lse_max_abs"] = err(lse, ref_lse)
    return d


# ---------------------------------------------------------------------------------------------
# workloads
# ---------------------------------------------------------------------------------------------
class Workload:
    """One benchmarked configuration.  `units` of work are bytes for the HBM-bound decode and FLOPs for the
    others (the reference's own formulas)."""
    scaling = "weak"
    e2e_buffers = 1          # sets of device input / host output buffers of the end-to-end loop
    e2e_max_steps = 5
    world = 1
    rank = 0
    sharding = "requests sharded, no collective"

    # ---- end to end through the public API: inputs from pinned host memory, results back to pinned host memory.
    # With two buffer sets the copies of neighbouring steps overlap with the kernels (three streams).
    def e2e_begin(self):
        dev = self.device
        if not hasattr(self, "_E"):
            n = self.e2e_buffers
            E = self._E = argparse.Namespace()
            E.n = n
            E.s_in, E.s_cmp, E.s_out = (torch.cuda.Stream(dev) for _ in range(3))
            E.h_in = {k: (v if v.is_pinned() else v.pin_memory()) for k, v in self.host_inputs().items()}
            E.d_in = [{k: torch.empty(v.shape, dtype=v.dtype, device=dev) for k, v in E.h_in.items()} for _ in range(n)]
            E.h_out = [None] * n
            E.ev_in = [torch.cuda.Event() for _ in range(n)]
            E.ev_cmp = [torch.cuda.Event() for _ in range(n)]
            E.ev_out = [torch.cuda.Event() for _ in range(n)]
            E.keep = [None] * n
            E.d2h = 0
        self._E.k = 0
        main = torch.cuda.current_stream(dev)
        for st in (self._E.s_in, self._E.s_cmp, self._E.s_out):
            st.wait_stream(main)

    def step_e2e(self, run_kernel: bool = True):
        E = self._E
        i = E.k % E.n
        E.k += 1
        later = E.k > E.n
        with torch.cuda.stream(E.s_in):
            if later:
                E.s_in.wait_event(E.ev_cmp[i])       # the step that read this set of inputs
            for k, v in E.h_in.items():
                E.d_in[i][k].copy_(v, non_blocking=True)
            E.ev_in[i].record(E.s_in)
        with torch.cuda.stream(E.s_cmp):
            E.s_cmp.wait_event(E.ev_in[i])
            if later:
                E.s_cmp.wait_event(E.ev_out[i])      # results of that step have been read back
            outs = self.run_from(E.d_in[i]) if run_kernel or E.keep[i] is None else E.keep[i]
            E.ev_cmp[i].record(E.s_cmp)
        if E.h_out[i] is None:
            E.h_out[i] = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in outs]
            E.d2h = sum(o.numel() * o.element_size() for o in outs)
        with torch.cuda.stream(E.s_out):
            E.s_out.wait_event(E.ev_cmp[i])
            for h, o in zip(E.h_out[i], outs):
                h.copy_(o, non_blocking=True)
            E.ev_out[i].record(E.s_out)
        E.keep[i] = outs

    def e2e_end(self):
        main = torch.cuda.current_stream(self.device)
        for st in (self._E.s_in, self._E.s_cmp, self._E.s_out):
            main.wait_stream(st)

    def e2e_bytes(self):
        h2d = sum(v.numel() * v.element_size() for v in self._E.h_in.values())
        return h2d, self._E.d2h

    def release(self):
        self._graph_out = None
        self._graph = None
        for k in list(self.__dict__):
            if isinstance(self.__dict__[k], (torch.Tensor, list, dict, argparse.Namespace)):
                del self.__dict__[k]
        torch.cuda.empty_cache()

    def imbalance(self):
        return None

    def traffic(self):
        return None

    # Launch-bound steps (a decode step is two kernels of ~0.15 ms) are timed as replays of a CUDA graph that holds
    # one captured step: the host then issues one call per step whatever the cost of the Python launch path.
    graphable = False

    def capture(self):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._graph_out = self.step()
        self._graph = g

    def timed_step(self):
        """What the timed region runs: a replay of the captured step when there is one, else a plain step."""
        if getattr(self, "_graph", None) is not None:
            self._graph.replay()
            return self._graph_out
        return self.step()


class DenseDecode(Workload):
    """Dense BF16 MLA decode at the DeepSeek-V3 shape."""
    metric, unit, dtype = "dense_bf16_mla_decode_bandwidth", "GB/s", "bf16"
    bound = "hbm"
    kernel_name = "mla_pair_kernel<decode> (+ decode_combine_kernel)"
    launches_per_step = 2          # split-KV attention + combine
    graphable = True
    e2e_buffers = 2
    e2e_max_steps = 10 ** 9

    def __init__(self, s_q: int = 1, batch: int = 128, h_q: int = 128, small: bool = False):
        if small:
            batch = 16
        self.s_q, self.b, self.h_q = s_q, batch, h_q
        self.key = "dense_decode" if s_q == 1 else f"dense_decode_sq{s_q}"
        if s_q > 1:
            self.metric, self.unit, self.bound = "dense_bf16_mla_decode_tflops", "TFLOP/s", "tensor"
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

    def setup(self, device, seed: int, rank: int = 0, world: int = 1):
        import flashmla_windows_linux_sm120_b200 as fm
        self.fm, self.device, self.rank, self.world = fm, device, rank, world
        self.make_host(seed + rank)
        torch.manual_seed(seed + rank)
        self.cache = torch.randn((self.num_pages, 64, 1, 576), dtype=torch.bfloat16, device=device)
        self.q = torch.randn((self.b, self.s_q, self.h_q, 576), dtype=torch.bfloat16, device=device)
        self.d_lens = self.lens.to(device)
        self.d_bt = self.block_table.to(device)
        self.md, self.ns = fm.get_mla_metadata(self.d_lens, self.s_q * self.h_q, 1)

    # reference formulas: tests/test_flash_mla_decoding.py:255-268
    def alg_bytes(self, lens=None):
        lens = self.lens if lens is None else lens
        return int(len(lens) * (self.s_q * self.h_q * 576 * 2 + self.s_q * self.h_q * 512 * 2) + int(lens.sum()) * 1152)

    def alg_flops(self, lens=None):
        lens = self.lens if lens is None else lens
        return int(self.h_q * self.s_q * 2 * (576 + 512) * int(lens.sum()))

    def traffic(self):
        return TRAFFIC["dense_decode"]["per_token"] * int(self.lens.sum()) if self.s_q == 1 else None

    def step(self, events=None):
        from flashmla_windows_linux_sm120_b200 import cuda_sm100
        return cuda_sm100.fwd_kvcache_mla(self.q, self.cache, 512, self.d_lens, self.d_bt, 576 ** -0.5, True, self.md,
                                          self.ns, False, None, profile_events=events)

    def host_inputs(self):
        return {"q": self.q.cpu(), "bt": self.block_table, "lens": self.lens}

    def run_from(self, d):
        return self.fm.flash_mla_with_kvcache(d["q"], self.cache, d["bt"], d["lens"], 512, self.md, self.ns, causal=True)

    def parity(self, n_req: int = 16):
        """Outputs of one more step against the CPU oracle on n_req requests spread over the batch."""
        from oracle import decode
        out, lse = self.timed_step()
        torch.cuda.synchronize()
        sel = sorted(set(int(round(i * (self.b - 1) / max(n_req - 1, 1))) for i in range(min(n_req, self.b))))
        lens = self.lens[sel]
        nb = int(((lens + 63) // 64).max())
        bt = self.block_table[sel, :nb].clone()
        used = torch.unique(bt[bt < self.num_pages])
        remap = torch.full((self.num_pages,), -1, dtype=torch.int64)
        remap[used.long()] = torch.arange(len(used))
        bt = torch.where(bt < self.num_pages, remap[bt.clamp(max=self.num_pages - 1).long()].to(torch.int32), bt)
        cache = self.cache[used.to(self.device).long()].cpu()
        r_out, r_lse = decode.decode_ref(lens, bt, self.q[sel].cpu(), cache, 512, self.s_q > 1)
        d = _errs(out[sel].cpu(), r_out, lse[sel].cpu(), r_lse)
        d.update(sample=f"{len(sel)} of {self.b} requests, oracle.decode.decode_ref", ok=bool(d["out_max_abs"] <= d["out_bound"] and d["lse_max_abs"] <= 1e-4))
        return d

    def cpu_sample(self, n_req: int = 32):
        """The reference's CPU torch path on n_req requests with the sequence lengths of this workload."""
        from oracle import decode
        n_req = min(n_req, self.b)
        lens = self.lens[:n_req]
        nblk = (lens + 63) // 64
        total = int(nblk.sum())
        bt = torch.full((n_req, int(nblk.max())), 2147480000, dtype=torch.int32)
        perm = torch.randperm(total, generator=torch.Generator().manual_seed(1), dtype=torch.int32)
        o = 0
        for i in range(n_req):
            bt[i, :int(nblk[i])] = perm[o:o + int(nblk[i])]
            o += int(nblk[i])
        torch.manual_seed(1)
        cache = torch.randn((total, 64, 1, 576), dtype=torch.bfloat16)
        q = torch.randn((n_req, self.s_q, self.h_q, 576), dtype=torch.bfloat16)

        def run():
            return decode.decode_ref(lens, bt, q, cache, 512, self.s_q > 1)
        units = self.alg_bytes(lens) if self.bound == "hbm" else self.alg_flops(lens)
        return run, units, f"first {n_req} of {self.b} requests ({int(lens.sum())} tokens), oracle.decode.decode_ref"


class SparseDecode(Workload):
    """Sparse FP8 MLA decode, batch 64, top-k 2048 of 32768 cached tokens."""
    metric, unit, dtype = "sparse_fp8_mla_decode_tflops", "TFLOP/s", "bf16 (fp8 e4m3 cache)"
    bound = "tensor"
    key = "sparse_decode"
    kernel_name = "mla_pair_kernel<sparse decode> (+ decode_combine_kernel)"
    launches_per_step = 2
    graphable = True

    def traffic(self):
        return TRAFFIC["sparse_decode"]["per_request"] * self.b if (self.topk, self.h_q) == (2048, 128) else None

    def __init__(self, batch: int = 64, topk: int = 2048, seqlen: int = 32768, h_q: int = 128, small: bool = False):
        if small:
            batch = 16
        self.b, self.topk, self.seqlen, self.h_q, self.s_q = batch, topk, seqlen, h_q, 1
        self.name = f"sparse_fp8_decode b={batch}/gpu s_q=1 h_q={h_q} topk={topk} seqlen_k={seqlen} 656B/token page=64"

    def make_host(self, seed: int):
        pass

    def setup(self, device, seed: int, rank: int = 0, world: int = 1):
        import flashmla_windows_linux_sm120_b200 as fm
        from flashmla_windows_linux_sm120_b200 import cuda_sm100
        self.fm, self.device, self.rank, self.world = fm, device, rank, world
        torch.manual_seed(seed + rank)
        pages_per = self.seqlen // 64
        npages = self.b * pages_per
        g = torch.Generator(device="cpu").manual_seed(seed + rank)
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

    def alg_bytes(self):
        return int(self.b * (self.h_q * 576 * 2 + self.topk * 656 + self.h_q * 512 * 2))

    def alg_flops(self):
        return int(self.b * self.h_q * 2 * (576 + 512) * self.topk)

    def step(self, events=None):
        return self.fm.flash_mla_with_kvcache(self.q, self.cache, self.block_table, self.lens, 512, self.md, self.ns,
                                              is_fp8_kvcache=True, indices=self.indices)

    def host_inputs(self):
        return {"q": self.q.cpu(), "idx": self.indices.cpu(), "bt": self.block_table.cpu(), "lens": self.lens.cpu()}

    def run_from(self, d):
        return self.fm.flash_mla_with_kvcache(d["q"], self.cache, d["bt"], d["lens"], 512, self.md, self.ns,
                                              is_fp8_kvcache=True, indices=d["idx"])

    def parity(self, n_req: int = 4):
        """n_req requests: their 2048 records are fetched, de-quantised by the codec oracle and attended on the CPU."""
        from oracle import decode, quant
        out, lse = self.timed_step()
        torch.cuda.synchronize()
        sel = sorted(set(int(round(i * (self.b - 1) / max(n_req - 1, 1))) for i in range(min(n_req, self.b))))
        e_out = e_lse = 0.0
        bound = 0.0
        flat = self.cache.view(torch.uint8).view(-1, 656)
        for i in sel:
            idx = self.indices[i, 0]
            rows = flat[idx.clamp(min=0).long()].cpu()                                  # [topk, 656]
            deq = quant.dequantize_k_cache(rows.view(self.topk // 64, 64, 1, 656))      # [topk/64, 64, 1, 576] bf16
            local = torch.arange(self.topk, dtype=torch.int32)
            local[idx.cpu() < 0] = -1
            r_out, r_lse = decode.decode_sparse_physical_ref(self.q[i:i + 1].cpu(), deq, local.view(1, 1, -1), 512)
            d = _errs(out[i:i + 1].cpu(), r_out, lse[i:i + 1].cpu(), r_lse)
            e_out, e_lse, bound = max(e_out, d["out_max_abs"]), max(e_lse, d["lse_max_abs"]), max(bound, d["out_bound"])
        return {"out_max_abs": e_out, "out_bound": bound, "lse_max_abs": e_lse, "ok": bool(e_out <= bound and e_lse <= 1e-4),
                "sample": f"{len(sel)} of {self.b} requests, oracle.quant.dequantize_k_cache + oracle.decode.decode_sparse_physical_ref"}

    def cpu_sample(self, n_req: int = 4):
        from oracle import decode, quant
        torch.manual_seed(2)
        kv = torch.randn((n_req * self.topk // 64, 64, 1, 576), dtype=torch.bfloat16)
        cache = quant.quantize_k_cache(kv)
        q = torch.randn((n_req, 1, self.h_q, 576), dtype=torch.bfloat16)
        idx = torch.stack([torch.randperm(self.topk, dtype=torch.int32) + i * self.topk for i in range(n_req)]).view(n_req, 1, -1)

        def run():
            deq = quant.dequantize_k_cache(cache)
            return decode.decode_sparse_physical_ref(q, deq, idx, 512)
        return run, int(n_req * self.h_q * 2 * (576 + 512) * self.topk), f"{n_req} of {self.b} requests, de-quantisation + oracle.decode.decode_sparse_physical_ref"


class SparsePrefill(Workload):
    """Sparse MLA prefill forward, s_q 4096, s_kv 32768, top-k 2048 (causally restricted)."""
    metric, unit, dtype = "sparse_mla_prefill_fwd_tflops", "TFLOP/s", "bf16"
    bound = "tensor"
    key = "sparse_prefill"
    kernel_name = "mla_pair_kernel<prefill>"
    e2e_buffers = 2
    launches_per_step = 1
    scaling = "strong"
    sharding = "query tokens sharded (kv replicated), no collective"

    def traffic(self):
        t = TRAFFIC["sparse_prefill"]
        return t["fixed"] + t["per_query_token"] * self.s_q if (self.s_kv, self.topk, self.h_q) == (32768, 2048, 128) else None

    def __init__(self, s_q: int = 4096, s_kv: int = 32768, topk: int = 2048, h_q: int = 128, small: bool = False):
        if small:
            s_q = 512
        self.s_q_total, self.s_kv, self.topk, self.h_q, self.b = s_q, s_kv, topk, h_q, 1
        self.name = f"sparse_prefill_fwd s_q={s_q} h_q={h_q} s_kv={s_kv} topk={topk} causal-restricted indices"

    def make_host(self, seed: int):
        pass

    def setup(self, device, seed: int, rank: int = 0, world: int = 1):
        import flashmla_windows_linux_sm120_b200 as fm
        from flashmla_windows_linux_sm120_b200 import parallel
        self.fm, self.device, self.rank, self.world = fm, device, rank, world
        self.lo, self.hi = parallel.shard_query_tokens(self.s_q_total, world)[rank]
        self.s_q = self.hi - self.lo
        g = torch.Generator(device=device).manual_seed(seed)            # the same kv on every rank
        self.kv = torch.randn((self.s_kv, 1, 576), dtype=torch.bfloat16, device=device, generator=g)
        torch.manual_seed(seed + 1000 + rank)
        self.q = torch.randn((self.s_q, self.h_q, 576), dtype=torch.bfloat16, device=device)
        idx = torch.empty((self.s_q, 1, self.topk), dtype=torch.int32, device=device)
        for t in range(self.s_q):                       # query t sits at position s_kv - s_q_total + (lo + t)
            hi = self.s_kv - self.s_q_total + self.lo + t + 1
            idx[t, 0] = torch.randperm(hi, device=device)[:self.topk].to(torch.int32)
        self.indices = idx
        self.scale = 576 ** -0.5

    def alg_bytes(self):
        return int(self.q.numel() * 2 + self.kv.numel() * 2 + self.indices.numel() * 4 + self.s_q * self.h_q * 512 * 2)

    def alg_flops(self):
        return int(2 * (self.h_q * 576 * self.topk + self.h_q * 512 * self.topk) * self.s_q)

    def step(self, events=None):
        return self.fm.flash_mla_sparse_fwd(self.q, self.kv, self.indices, self.scale)

    def host_inputs(self):
        return {"q": self.q.cpu(), "idx": self.indices.cpu()}

    def run_from(self, d):
        return self.fm.flash_mla_sparse_fwd(d["q"], self.kv, d["idx"], self.scale)

    def parity(self, n_tok: int = 64):
        """n_tok query tokens incl. the first and the last token that a persistent CTA walks."""
        from oracle import sparse_prefill
        from oracle.check import max_abs_diff
        out, mx, lse = self.step()
        torch.cuda.synchronize()
        g = torch.Generator().manual_seed(3)
        lanes = 74 if self.h_q == 128 else 148
        base = [0, 1, lanes - 1, lanes, self.s_q - lanes, self.s_q - 1]
        sel = sorted(set([t for t in base if 0 <= t < self.s_q] + torch.randint(0, self.s_q, (n_tok,), generator=g).tolist()))[:n_tok + 6]
        r_out, r_mx, r_lse = sparse_prefill.sparse_prefill_ref(self.q[sel].cpu(), self.kv.cpu(), self.indices[sel].cpu(), self.scale)
        d = _errs(out[sel].cpu(), r_out, lse[sel].cpu(), r_lse)
        d["max_logits_max_abs"] = max_abs_diff(mx[sel].cpu(), r_mx)
        lim = 1e-4 * math.log2(math.e)      # base-2 quantities
        d.update(sample=f"{len(sel)} of {self.s_q} query tokens, oracle.sparse_prefill.sparse_prefill_ref",
                 ok=bool(d["out_max_abs"] <= d["out_bound"] and d["lse_max_abs"] <= lim and d["max_logits_max_abs"] <= lim))
        return d

    def cpu_sample(self, n_tok: int = 64):
        from oracle import sparse_prefill
        torch.manual_seed(4)
        q = torch.randn((n_tok, self.h_q, 576), dtype=torch.bfloat16)
        kv = torch.randn((self.s_kv, 1, 576), dtype=torch.bfloat16)
        idx = torch.stack([torch.randperm(self.s_kv)[:self.topk].to(torch.int32) for _ in range(n_tok)]).view(n_tok, 1, -1)
        scale = 576 ** -0.5

        def run():
            return sparse_prefill.sparse_prefill_ref(q, kv, idx, scale)
        return run, int(2 * self.h_q * (576 + 512) * self.topk * n_tok), f"{n_tok} of {self.s_q_total} query tokens, oracle.sparse_prefill.sparse_prefill_ref"


class DenseFwdBwd(Workload):
    """Dense causal varlen MHA forward + backward, h 128, d 192/128, 8 sequences U[1024,8192]."""
    metric, unit, dtype = "dense_mha_varlen_fwd_bwd_tflops", "TFLOP/s", "bf16"
    bound = "tensor"
    key = "dense_fwd_bwd"
    kernel_name = "dense_fwd_tc_kernel<192> + dense_bwd_*"
    launches_per_step = 4
    scaling = "strong"
    sharding = "sequences sharded (longest first), no collective"
    backward = True
    e2e_max_steps = 3

    def __init__(self, nseq: int = 8, h: int = 128, small: bool = False):
        self.nseq, self.h, self.b, self.small = nseq, h, nseq, small
        self.name = f"dense_mha_varlen {'fwd+bwd' if self.backward else 'fwd'} {nseq} seqs L~U[1024,8192] h={h} d=192/128 causal"

    def make_host(self, seed: int):
        g = torch.Generator().manual_seed(seed)
        self.all_lens = torch.randint(1024, 8193, (self.nseq,), generator=g, dtype=torch.int32)
        if self.small:
            self.all_lens = self.all_lens[:2].clamp(max=2048)

    def setup(self, device, seed: int, rank: int = 0, world: int = 1):
        import flashmla_windows_linux_sm120_b200 as fm
        from flashmla_windows_linux_sm120_b200 import parallel
        self.fm, self.device, self.rank, self.world = fm, device, rank, world
        self.make_host(seed)                                            # the same lengths on every rank
        mine = parallel.shard_sequences(self.all_lens.tolist(), world)[rank]
        lens = self.all_lens[mine] if mine else torch.zeros((0,), dtype=torch.int32)
        self.lens = lens
        self.mine = mine
        cu = torch.cumsum(torch.nn.functional.pad(lens, (1, 0)), 0, dtype=torch.int32)
        T = int(lens.sum())
        torch.manual_seed(seed + rank)
        mk = lambda d: torch.randn((max(T, 1), self.h, d), dtype=torch.bfloat16, device=device)[:T].requires_grad_(self.backward)
        self.q, self.k, self.v = mk(192), mk(192), mk(128)
        self.d_out = torch.randn((T, self.h, 128), dtype=torch.bfloat16, device=device)
        self.cu = cu.to(device)
        self.cu_host = cu
        self.max_len = int(lens.max()) if len(lens) else 0
        self.pairs = int(sum(int(l) * (int(l) + 1) // 2 for l in lens))
        allp = [int(l) * (int(l) + 1) // 2 for l in self.all_lens]
        loads = [sum(allp[i] for i in s) for s in parallel.shard_sequences(self.all_lens.tolist(), world)]
        self._imb = max(loads) / (sum(loads) / world) if sum(loads) else None

    def imbalance(self):
        return self._imb

    def alg_bytes(self):
        T = self.q.shape[0]
        return int(T * self.h * (192 * 2 * 2 + 128 * 2 * 2) * (2 if self.backward else 1))

    def alg_flops(self):
        f = (192 + 128) + ((3 * 192 + 2 * 128) if self.backward else 0)
        return int(self.pairs * self.h * 2 * f)

    def _run(self, q, k, v, d_out):
        if len(self.lens) == 0:
            return ()
        if not self.backward:
            with torch.no_grad():
                return self.fm.flash_attn_varlen_func(q, k, v, self.cu, self.cu, self.max_len, self.max_len, causal=True)
        q.grad = k.grad = v.grad = None
        out, lse = self.fm.flash_attn_varlen_func(q, k, v, self.cu, self.cu, self.max_len, self.max_len, causal=True)
        out.backward(d_out)
        return out.detach(), lse, q.grad, k.grad, v.grad

    def step(self, events=None):
        return self._run(self.q, self.k, self.v, self.d_out)

    def host_inputs(self):
        d = {"q": self.q.detach().cpu(), "k": self.k.detach().cpu(), "v": self.v.detach().cpu()}
        if self.backward:
            d["d_out"] = self.d_out.cpu()
        return d

    def run_from(self, d):
        q, k, v = d["q"], d["k"], d["v"]
        if self.backward:       # fresh autograd leaves over the device buffers (the buffers themselves are overwritten in place)
            q, k, v = (t.detach().requires_grad_(True) for t in (q, k, v))
        return self._run(q, k, v, d.get("d_out"))

    def parity(self, heads=(0, 127)):
        """Heads `heads` of the shortest and of the longest sequence of this rank against the fp32 autograd oracle."""
        from oracle import dense
        from oracle.check import max_abs_diff
        if len(self.lens) == 0:
            return {"ok": True, "sample": "no sequence on this rank"}
        res = self.step()
        torch.cuda.synchronize()
        seqs = sorted(set([int(torch.argmin(self.lens)), int(torch.argmax(self.lens))]))
        hs = [h for h in heads if h < self.h]
        d = {"out_max_abs": 0.0, "out_bound": 0.0, "lse_max_abs": 0.0}
        if self.backward:
            d.update(dq_max_abs=0.0, dk_max_abs=0.0, dv_max_abs=0.0, grad_bound=0.0)
        for s in seqs:
            a, b = int(self.cu_host[s]), int(self.cu_host[s + 1])
            sl = lambda t: t.detach()[a:b][:, hs].float().cpu()
            cu = torch.tensor([0, b - a], dtype=torch.int32)
            if self.backward:
                r = dense.dense_fwd_bwd_ref(sl(self.q), sl(self.k), sl(self.v), sl(self.d_out), cu, cu, True)
            else:
                r = dense.dense_fwd_ref(sl(self.q), sl(self.k), sl(self.v), cu, cu, True)
            e = _errs(sl(res[0]), r[0], res[1][a:b][:, hs].cpu(), r[1])
            d["out_max_abs"], d["out_bound"] = max(d["out_max_abs"], e["out_max_abs"]), max(d["out_bound"], e["out_bound"])
            d["lse_max_abs"] = max(d["lse_max_abs"], e["lse_max_abs"])
            if self.backward:
                for n, got, ref in (("dq", res[2], r[2]), ("dk", res[3], r[3]), ("dv", res[4], r[4])):
                    d[n + "_max_abs"] = max(d[n + "_max_abs"], max_abs_diff(sl(got), ref))
                    d["grad_bound"] = max(d["grad_bound"], 4 * out_bound(ref))
        ok = d["out_max_abs"] <= d["out_bound"] and d["lse_max_abs"] <= 1e-4
        if self.backward:
            ok = ok and all(d[n + "_max_abs"] <= d["grad_bound"] for n in ("dq", "dk", "dv"))
        d.update(ok=bool(ok), sample=f"heads {hs} of sequences {[int(self.lens[s]) for s in seqs]} tokens, oracle.dense (fp32 autograd)")
        return d

    def cpu_sample(self, L: int = 2048, heads: int = 8):
        from oracle import dense
        torch.manual_seed(5)
        mk = lambda d: torch.randn((L, heads, d), dtype=torch.bfloat16)
        q, k, v, do = mk(192), mk(192), mk(128), mk(128)
        cu = torch.tensor([0, L], dtype=torch.int32)

        def run():
            if self.backward:
                return dense.dense_fwd_bwd_ref(q, k, v, do, cu, cu, True)
            return dense.dense_fwd_ref(q, k, v, cu, cu, True)
        f = (192 + 128) + ((3 * 192 + 2 * 128) if self.backward else 0)
        return run, int(L * (L + 1) // 2 * heads * 2 * f), f"one {L}-token sequence, {heads} of {self.h} heads, oracle.dense (fp32 autograd)"


class DenseFwd(DenseFwdBwd):
    """The same workload, forward only (the reference quotes forward and backward separately)."""
    metric = "dense_mha_varlen_fwd_tflops"
    key = "dense_fwd"
    kernel_name = "dense_fwd_tc_kernel<192>"
    launches_per_step = 1
    backward = False


class KVShardedDecode(Workload):
    """One 1 M-token context, batch 1, cache pages sharded along the sequence over the ranks; the per-rank
    partial outputs are merged through peer memory (NVLink stores + flags).  The NCCL all_gather variant is
    timed beside it."""
    metric, unit, dtype = "kv_sharded_decode_bandwidth", "GB/s", "bf16"
    bound = "hbm"
    key = "kv_sharded_decode"
    kernel_name = "mla_pair_kernel<decode> + push/merge"
    launches_per_step = 3
    scaling = "strong"
    sharding = "KV pages of one context sharded along the sequence; peer-memory merge of O / LSE"

    def __init__(self, seqlen: int = 1 << 20, h_q: int = 128, small: bool = False):
        if small:
            seqlen = 1 << 17
        self.seqlen, self.h_q, self.b = seqlen, h_q, 1
        self.name = f"kv_sharded_decode b=1 s_q=1 h_q={h_q} seqlen={seqlen} d=576 dv=512"

    def make_host(self, seed: int):
        pass

    def setup(self, device, seed: int, rank: int = 0, world: int = 1):
        import flashmla_windows_linux_sm120_b200 as fm
        from flashmla_windows_linux_sm120_b200 import parallel
        self.fm, self.device, self.rank, self.world, self.parallel = fm, device, rank, world, parallel
        lo, hi = parallel.shard_kv_pages(self.seqlen, world)[rank]
        self.n_local = hi - lo
        npages = max((self.n_local + 63) // 64, 1)
        g = torch.Generator(device="cpu").manual_seed(seed)             # the same q on every rank
        self.q = torch.randn((1, 1, self.h_q, 576), generator=g).to(torch.bfloat16).to(device)
        torch.manual_seed(seed + 100 + rank)
        self.cache = torch.randn((npages, 64, 1, 576), dtype=torch.bfloat16, device=device)
        self.bt = torch.randperm(npages, device=device).to(torch.int32).view(1, npages)
        self.lens = torch.tensor([self.n_local], dtype=torch.int32, device=device)
        self.nccl_ms = None
        if world > 1:
            self.dec = parallel.KVShardedDecode(1, self.h_q, device, transport="peer")
            self.dec_nccl = parallel.KVShardedDecode(1, self.h_q, device, transport="nccl")
        else:
            self.md, self.ns = fm.get_mla_metadata(self.lens, self.h_q, 1)

    def alg_bytes(self):
        return int(self.n_local * 1152 + (self.h_q * 576 * 2 + self.h_q * 512 * 2) / self.world)

    def alg_flops(self):
        return int(self.h_q * 2 * (576 + 512) * self.n_local)

    def step(self, events=None):
        if self.world > 1:
            return self.dec(self.q, self.cache, self.bt, self.lens)
        return self.fm.flash_mla_with_kvcache(self.q, self.cache, self.bt, self.lens, 512, self.md, self.ns)

    def step_nccl(self):
        return self.dec_nccl(self.q, self.cache, self.bt, self.lens)

    def host_inputs(self):
        return {"q": self.q.cpu()}

    def run_from(self, d):
        if self.world > 1:
            return self.dec(d["q"], self.cache, self.bt, self.lens)
        return self.fm.flash_mla_with_kvcache(d["q"], self.cache, self.bt, self.lens, 512, self.md, self.ns)

    def parity(self, heads: int = 8):
        """The merged result for the first `heads` heads against the CPU oracle over the whole context."""
        import torch.distributed as dist
        from oracle import decode
        out, lse = self.step()
        torch.cuda.synchronize()
        kv_local = self.cache[self.bt[0].long()].reshape(-1, 576)[:self.n_local]
        if self.world > 1:
            n_max = (self.seqlen // 64 // self.world + 1) * 64
            pad = torch.zeros((n_max, 576), dtype=torch.bfloat16, device=self.device)
            pad[:self.n_local] = kv_local
            allkv = torch.empty((self.world, n_max, 576), dtype=torch.bfloat16, device=self.device)
            dist.all_gather_into_tensor(allkv, pad)
            sizes = [b - a for a, b in self.parallel.shard_kv_pages(self.seqlen, self.world)]
            kv = torch.cat([allkv[r, :sizes[r]] for r in range(self.world)]).cpu()
        else:
            kv = kv_local.cpu()
        if self.rank != 0:
            return {"ok": True}
        L = kv.shape[0]
        padn = (-L) % 64
        blocked = torch.cat([kv, torch.zeros(padn, 576, dtype=kv.dtype)]).view(-1, 64, 1, 576)
        r_out, r_lse = decode.decode_ref(torch.tensor([L], dtype=torch.int32), torch.arange(blocked.shape[0], dtype=torch.int32).view(1, -1),
                                         self.q[:, :, :heads].cpu(), blocked, 512, False)
        d = _errs(out[:, :, :heads].cpu(), r_out, lse[:, :heads].cpu(), r_lse)
        d.update(sample=f"{heads} of {self.h_q} heads over all {L} tokens, oracle.decode.decode_ref",
                 ok=bool(d["out_max_abs"] <= d["out_bound"] and d["lse_max_abs"] <= 1e-4))
        return d

    def cpu_sample(self, L: int = 1 << 16, heads: int = 16):
        from oracle import decode
        torch.manual_seed(6)
        kv = torch.randn((L // 64, 64, 1, 576), dtype=torch.bfloat16)
        q = torch.randn((1, 1, heads, 576), dtype=torch.bfloat16)
        lens, bt = torch.tensor([L], dtype=torch.int32), torch.arange(L // 64, dtype=torch.int32).view(1, -1)

        def run():
            return decode.decode_ref(lens, bt, q, kv, 512, False)
        return run, int(L * 1152), f"{L} of {self.seqlen} tokens, {heads} of {self.h_q} heads, oracle.decode.decode_ref"


def make_workload(key: str, small: bool = False) -> Workload:
    return {
        "dense_decode": lambda: DenseDecode(1, small=small),
        "dense_decode_sq2": lambda: DenseDecode(2, small=small),
        "sparse_decode": lambda: SparseDecode(small=small),
        "sparse_prefill": lambda: SparsePrefill(small=small),
        "dense_fwd": lambda: DenseFwd(small=small),
        "dense_fwd_bwd": lambda: DenseFwdBwd(small=small),
        "kv_sharded_decode": lambda: KVShardedDecode(small=small),
    }[key]()


WORKLOADS = ["dense_decode", "dense_decode_sq2", "sparse_decode", "sparse_prefill", "dense_fwd", "dense_fwd_bwd", "kv_sharded_decode"]


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


def unit_scale(wl):
    return 1e9 if wl.unit == "GB/s" else 1e12


def run_reference(args, wl):
    rank, world, _ = dist_env()
    if rank != 0:
        return
    wl.make_host(args.seed)
    use_all_host_threads()
    run, units, sample = wl.cpu_sample()
    steps = max(1, min(args.steps, 5))
    warm = max(1, min(args.warmup, 1))
    sec = time_cpu(run, steps, warm)
    val = units / sec / unit_scale(wl)
    cores = torch.get_num_threads()
    line = {"impl": "reference", "metric": wl.metric, "value": val, "unit": wl.unit, "n_gpus": args.gpus, "steps": steps,
            "warmup": warm, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": wl.scaling, "vs_baseline": None,
            "dtype": "f32", "data": "synthetic", "config": {"workload": wl.name, "sample": sample},
            "cpu_baseline": {"value": val, "unit": wl.unit, "cores": cores, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": wl.unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line))


class Runner:
    """Times one workload on this rank; every rank runs the same sequence of collectives."""

    def __init__(self, device, local, rank, world, seed):
        self.device, self.local, self.rank, self.world, self.seed = device, local, rank, world, seed
        self.stream = torch.cuda.current_stream()
        self.sustained = True
        self.use_graph = True
        if world > 1:
            import torch.distributed as dist
            self.dist = dist

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def allmax(self, x: float) -> float:
        t = torch.tensor([x], dtype=torch.float64, device=self.device)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def allsum(self, x: float) -> float:
        t = torch.tensor([x], dtype=torch.float64, device=self.device)
        if self.world > 1:
            self.dist.all_reduce(t)
        return float(t.item())

    def all_ok(self, ok: bool) -> bool:
        return self.allmax(0.0 if ok else 1.0) == 0.0

    def timed(self, fn, steps, per_kernel=False):
        """Returns (ms per step as the max over ranks, [kernel ms], clocks)."""
        pairs = None
        if per_kernel:
            pairs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
            for a, b in pairs:            # create the handles
                a.record(self.stream)
                b.record(self.stream)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        sampler = ClockSampler(self.local).start()
        e0.record(self.stream)
        for i in range(steps):
            fn(pairs[i]) if per_kernel else fn(None)
        e1.record(self.stream)
        self.barrier()
        clocks = sampler.stop()
        ms = self.allmax(e0.elapsed_time(e1)) / steps
        kern = [a.elapsed_time(b) for a, b in pairs] if per_kernel else []
        return ms, kern, clocks

    def e2e(self, wl, steps, run_kernel=True):
        wl.e2e_begin()
        for _ in range(min(3, steps)):
            wl.step_e2e(run_kernel)
        wl.e2e_end()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        self.barrier()
        e0.record(self.stream)
        wl.e2e_begin()
        for _ in range(steps):
            wl.step_e2e(run_kernel)
        wl.e2e_end()
        e1.record(self.stream)
        self.barrier()
        return self.allmax(e0.elapsed_time(e1)) / steps

    def measure(self, wl, steps, warmup, headline: bool, do_cpu: bool):
        """Set-up, warm-up, K timed steps, roofline, parity sample, end-to-end loop.  Returns a dict (rank 0 uses it)."""
        peaks = measured_peaks()
        r = {"name": wl.key, "workload": wl.name, "metric": wl.metric, "unit": wl.unit, "dtype": wl.dtype, "scaling": wl.scaling,
             "steps": steps, "warmup": warmup}
        ok = True
        try:
            wl.setup(self.device, self.seed, self.rank, self.world)
            for _ in range(warmup):
                wl.step()
            torch.cuda.synchronize()
        except Exception as e:      # noqa: BLE001
            ok = False
            r["error"] = f"setup: {type(e).__name__}: {e}"
            traceback.print_exc(file=sys.stderr)
        if not self.all_ok(ok):
            r.setdefault("error", "set-up failed on another rank")
            return r
        per_kernel = wl.bound == "hbm" and wl.key.startswith("dense_decode")
        ms_eager, kern, clocks = self.timed(lambda ev: wl.step(ev) if per_kernel else wl.step(), steps, per_kernel)
        ms = ms_eager
        captured = False
        if wl.graphable and self.use_graph:
            try:
                wl.capture()
                for _ in range(3):
                    wl.timed_step()
                torch.cuda.synchronize()
                captured = True
            except Exception as e:      # noqa: BLE001
                wl._graph = None
                r["graph_capture_error"] = f"{type(e).__name__}: {e}"
            if self.all_ok(captured):
                ms, _, clocks = self.timed(lambda ev: wl.timed_step(), steps, False)
                r["launch"] = "replays of a CUDA graph that holds one captured step (scheduler metadata fixed, as in a serving loop)"
                r["ms_per_step_eager"] = ms_eager
            else:
                wl._graph = None
        nbytes, nflops = self.allsum(float(wl.alg_bytes())), self.allsum(float(wl.alg_flops()))
        gbs, tflops = nbytes / (ms * 1e-3) / 1e9, nflops / (ms * 1e-3) / 1e12
        r.update(value=gbs if wl.unit == "GB/s" else tflops, ms_per_step=ms, gb_per_s=gbs, tflops=tflops, clocks=clocks,
                 gpu_launches=wl.launches_per_step * steps)
        if wl.imbalance() is not None:
            r["imbalance_max_over_mean"] = wl.imbalance()
        # roofline of the dominant kernel: this rank's algorithmic work / this rank's kernel time
        if wl.bound == "hbm":
            k_ms = statistics.mean(kern) if kern else ms
            ach = wl.alg_bytes() / (k_ms * 1e-3) / 1e9
            r["roofline"] = {"bound": "hbm", "kernel": wl.kernel_name, "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                             "frac": ach / peaks["hbm_gbs"], "peak_source": peaks["source"], "kernel_ms": k_ms,
                             "kernel_timed": "CUDA events around the attention kernel, recorded by the library" if kern else "whole step",
                             "algorithmic_bytes_per_launch": wl.alg_bytes(), "traffic": wl.traffic(),
                             "tensor_tflops": wl.alg_flops() / (k_ms * 1e-3) / 1e12,
                             "tensor_frac_of_burst": wl.alg_flops() / (k_ms * 1e-3) / 1e12 / peaks["bf16_tflops"]}
        else:   # whole step timed (these workloads launch their kernels back to back with nothing else)
            ach = wl.alg_flops() / (ms * 1e-3) / 1e12
            long_step = ms * steps > 500.0          # a stretch of seconds runs under the power cap: sustained peak
            peak = peaks["bf16_tflops_sustained"] if long_step else peaks["bf16_tflops"]
            r["roofline"] = {"bound": "tensor", "kernel": wl.kernel_name, "achieved": ach, "peak": peak, "unit": "TFLOP/s",
                             "frac": ach / peak, "frac_of_burst": ach / peaks["bf16_tflops"], "peak_source": peaks["source"],
                             "peak_kind": "sustained" if long_step else "burst", "kernel_ms": ms,
                             "algorithmic_flops_per_launch": wl.alg_flops(), "traffic": wl.traffic()}
        # parity of a sample of the outputs the timed path produces
        try:
            par = wl.parity()
        except Exception as e:      # noqa: BLE001
            par = {"ok": False, "error": f"{type(e).__name__}: {e}"}
            traceback.print_exc(file=sys.stderr)
        par["ok"] = self.all_ok(bool(par.get("ok")))
        r["parity_checked"] = par
        if isinstance(wl, KVShardedDecode) and self.world > 1:
            ms_n, _, _ = self.timed(lambda ev: wl.step_nccl(), steps)
            r["nccl_all_gather_baseline_ms"] = ms_n
            r["peer_merge_ms"] = ms
        # sustained: the same step for at least a second
        if headline and self.sustained:
            t0 = time.perf_counter()
            n, tot = 0, 0.0
            sampler = ClockSampler(self.local).start()
            while tot < 1000.0 and time.perf_counter() - t0 < 20.0:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                self.barrier()
                e0.record(self.stream)
                for _ in range(steps * 5):
                    wl.timed_step()
                e1.record(self.stream)
                self.barrier()
                tot += self.allmax(e0.elapsed_time(e1))
                n += steps * 5
            c = sampler.stop()
            r["sustained"] = {"value": (nbytes if wl.unit == "GB/s" else nflops) / (tot / n * 1e-3) / unit_scale(wl), "unit": wl.unit,
                              "steps": n, "seconds": tot / 1e3, "ms_per_step": tot / n, "clocks": c}
        # end to end through the public API with host buffers
        try:
            e_steps = max(1, min(steps, wl.e2e_max_steps))
            e_ms = self.e2e(wl, e_steps)
            h2d, d2h = wl.e2e_bytes()
            units = nbytes if wl.unit == "GB/s" else nflops
            r["e2e"] = {"value": units / (e_ms * 1e-3) / unit_scale(wl), "unit": wl.unit, "ms_per_step": e_ms, "steps": e_steps,
                        "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                        "note": "every step copies its inputs from pinned host memory and reads its results back; "
                                + (f"copies and kernels of neighbouring steps overlap (3 streams, {wl.e2e_buffers} buffer sets); " if wl.e2e_buffers > 1 else "")
                                + "the KV cache / kv tensor is resident device state"}
            if headline:
                c_ms = self.e2e(wl, e_steps, run_kernel=False)
                r["e2e"]["copy_only"] = {"ms_per_step": c_ms, "fraction_of_copy_only": c_ms / e_ms,
                                         "note": "the same copies without the kernel: what the host fabric alone allows at this N"}
        except Exception as e:      # noqa: BLE001
            r["e2e"] = None
            r["e2e_error"] = f"{type(e).__name__}: {e}"
            traceback.print_exc(file=sys.stderr)
        if do_cpu and self.rank == 0:
            try:
                use_all_host_threads()
                run, units, sample = wl.cpu_sample()
                sec = time_cpu(run, 3 if headline else 1, 1)
                r["cpu_baseline"] = {"value": units / sec / unit_scale(wl), "unit": wl.unit, "cores": torch.get_num_threads(), "kind": "port",
                                     "sample": sample, "seconds": sec}
            except Exception as e:      # noqa: BLE001
                r["cpu_baseline"] = None
                r["cpu_baseline_error"] = f"{type(e).__name__}: {e}"
        return r


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="dense_decode", choices=WORKLOADS)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--small", action="store_true", help="shrink the workload (profiler captures)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="do not run the other workloads after the default one")
    ap.add_argument("--no-graph", action="store_true", help="time plain per-step launches instead of CUDA graph replays")
    ap.add_argument("--no-sustained", action="store_true", help="skip the one-second sustained stretch (profiler captures)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    wl = make_workload(args.workload, args.small)

    if args.impl == "reference":
        run_reference(args, wl)
        return

    rank, world, local = dist_env()
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path (use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)

    runner = Runner(device, local, rank, world, args.seed)
    runner.sustained = not args.no_sustained
    runner.use_graph = not args.no_graph
    head = runner.measure(wl, args.steps, args.warmup, headline=True, do_cpu=not args.no_cpu_baseline and world == 1)
    wl.release()

    extras = []
    if args.workload == "dense_decode" and not args.no_extras and not args.small and "error" not in head:
        for key in WORKLOADS:
            if key == "dense_decode":
                continue
            w = make_workload(key)
            steps = 20
            r = runner.measure(w, steps, 3, headline=False, do_cpu=not args.no_cpu_baseline and world == 1)
            w.release()
            extras.append(r)

    if rank == 0:
        if "error" in head:
            print(json.dumps({"metric": wl.metric, "error": head["error"]}))
        else:
            line = {"metric": wl.metric, "value": head["value"], "unit": wl.unit, "n_gpus": world, "steps": args.steps,
                    "warmup": args.warmup, "ms_per_step": head["ms_per_step"], "higher_is_better": True, "scaling": wl.scaling,
                    "vs_baseline": None, "dtype": wl.dtype, "data": "synthetic",
                    "config": {"workload": wl.name, "global_batch": wl.b * world if wl.scaling == "weak" else wl.b,
                               "parallelism": f"{wl.sharding} x{world}",
                               "l2": "inputs (>=600 MB per GPU) larger than the 126 MB L2; no flush"},
                    "tflops": head["tflops"], "gb_per_s": head["gb_per_s"], "roofline": head["roofline"],
                    "cpu_baseline": head.get("cpu_baseline"), "e2e": head.get("e2e"), "parity_checked": head.get("parity_checked"),
                    "sustained": head.get("sustained"), "gpu_launches": head["gpu_launches"], "clocks": head["clocks"]}
            for k in ("imbalance_max_over_mean", "nccl_all_gather_baseline_ms", "peer_merge_ms", "e2e_error", "ms_per_step_eager",
                      "graph_capture_error"):
                if k in head:
                    line[k] = head[k]
            if "launch" in head:
                line["config"]["launch"] = head["launch"]
            if extras:
                line["workloads"] = extras
            print(json.dumps(line))
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
