"""Seeded synthetic inputs for the parity tests (test infrastructure only).

CPU restatements of the reference tests' generators, which cannot run on a CPU
as written (they call ``.cuda()`` / set the default device):
  decode         tests/test_flash_mla_decoding.py:34-121
  sparse prefill tests/test_flash_mla_prefill.py:34-63
  dense MHA      tests/test_fmha_sm100.py:51-78
Unused cache pages and the tail of the last page are NaN-poisoned, unused
block-table slots hold 2147480000, as in the reference, so any out-of-range read
shows up in the result.
"""
from __future__ import annotations

import dataclasses
import random
from typing import Optional

import torch


def cdiv(a: int, b: int) -> int:
    return (a + b - 1) // b


@dataclasses.dataclass
class DecodeCase:
    b: int
    s_q: int
    s_k: int
    is_varlen: bool = False
    is_causal: bool = False
    topk: Optional[int] = None
    all_indices_invalid: bool = False
    zero_seqlen: bool = False
    block_size: int = 64
    h_q: int = 128
    h_kv: int = 1
    d: int = 576
    dv: int = 512
    seed: int = 0
    unit_normal: bool = False      # N(0,1) values (benchmark distribution) instead of randn/10


@dataclasses.dataclass
class DecodeData:
    cache_seqlens: torch.Tensor    # [b] int32
    q: torch.Tensor                # [b, s_q, h_q, d] bf16
    block_table: torch.Tensor      # [b, max_blocks] int32
    blocked_k: torch.Tensor        # [num_blocks, block, h_kv, d] bf16
    abs_indices: Optional[torch.Tensor]     # [b, s_q, topk] logical positions / -1
    indices: Optional[torch.Tensor]         # [b, s_q, topk] physical slots / -1


def make_decode_case(t: DecodeCase) -> DecodeData:
    random.seed(t.seed)
    torch.manual_seed(t.seed)
    lens = torch.full((t.b,), t.s_k, dtype=torch.int32)
    if t.is_varlen:
        for i in range(t.b):
            lens[i] = max(random.normalvariate(t.s_k, t.s_k / 2), t.s_q)
    if t.zero_seqlen:
        lens[torch.randn(t.b) > 0] = 0
    max_pad = cdiv(max(int(lens.max()), 1), 256) * 256
    q = torch.randn(t.b, t.s_q, t.h_q, t.d)
    per = max_pad // t.block_size
    block_table = torch.arange(t.b * per, dtype=torch.int32)
    block_table = block_table[torch.randperm(block_table.numel())].view(t.b, per)
    blocked_k = torch.randn(block_table.numel(), t.block_size, t.h_kv, t.d)
    if not t.unit_normal:
        q.clamp_(-1.0, 1.0)
        blocked_k = (blocked_k / 10).clamp_(-1.0, 1.0)
    q = q.to(torch.bfloat16)
    blocked_k = blocked_k.to(torch.bfloat16)

    if t.topk is None:
        for i in range(t.b):
            L = int(lens[i])
            nb = cdiv(L, t.block_size)
            blocked_k[block_table[i, nb:].long()] = float("nan")
            if L % t.block_size != 0:
                blocked_k[int(block_table[i, nb - 1]), L % t.block_size:] = float("nan")
            block_table[i, nb:] = 2147480000
        return DecodeData(lens, q, block_table, blocked_k, None, None)

    abs_idx = torch.empty(t.b, t.s_q, t.topk, dtype=torch.int32)
    phys = torch.empty(t.b, t.s_q, t.topk, dtype=torch.int32)
    for i in range(t.b):
        for j in range(t.s_q):
            a = torch.randperm(int(lens[i]))[:t.topk]
            p = block_table[i, (a // t.block_size).long()].long() * t.block_size + (a % t.block_size)
            if len(a) < t.topk:
                pad = torch.full((t.topk - len(a),), -1, dtype=a.dtype)
                a = torch.cat([a, pad])
                p = torch.cat([p, pad])
            perm = torch.randperm(t.topk)
            a, p = a[perm], p[perm]
            if t.all_indices_invalid:
                a = torch.full_like(a, -1)
                p = torch.full_like(p, -1)
            abs_idx[i, j] = a
            phys[i, j] = p
    used = torch.unique(phys.flatten())
    used = used[used >= 0].long()
    flat = blocked_k.view(-1, t.h_kv, t.d)
    unused = torch.ones(flat.shape[0], dtype=torch.bool)
    unused[used] = False
    flat[unused] = float("nan")
    return DecodeData(lens, q, block_table, blocked_k, abs_idx, phys)


@dataclasses.dataclass
class PrefillCase:
    s_q: int
    s_kv: int
    topk: int
    h_q: int = 128
    d_qk: int = 576
    d_v: int = 512
    seed: int = 0
    causal_restrict: bool = False   # indices of query t drawn from [0, t_pos] (benchmark shape)


def make_prefill_case(t: PrefillCase):
    """Returns (q [s_q,h_q,d_qk] bf16, kv [s_kv,1,d_qk] bf16, indices [s_q,1,topk] int32)."""
    torch.manual_seed(t.seed)
    random.seed(t.seed)
    q = (torch.randn(t.s_q, t.h_q, t.d_qk) / 10).clamp_(-10, 10).to(torch.bfloat16)
    kv = (torch.randn(t.s_kv, 1, t.d_qk) / 10).clamp_(-10, 10).to(torch.bfloat16)
    idx = torch.full((t.s_q, 1, t.topk), t.s_kv, dtype=torch.int32)
    for s in range(t.s_q):
        if t.causal_restrict:
            hi = max(1, min(t.s_kv, (s + 1) * t.s_kv // t.s_q))
            cur = torch.randperm(hi)[:t.topk]
        else:
            n = min(t.topk, t.s_kv)
            near = torch.randint(0, 32, (n,)) < 31
            cur = torch.randperm(t.s_kv)[:t.topk]
            cur[near] = torch.randint(max(0, t.s_kv - 20000), max(t.s_kv - 1, 1), (int(near.sum()),))
        if len(cur) < t.topk:
            cur = torch.cat([cur, torch.full((t.topk - len(cur),), 2147480000)])
        idx[s, 0] = cur[torch.randperm(t.topk)].to(torch.int32)
    return q, kv, idx


@dataclasses.dataclass
class DenseCase:
    b: int
    mean_sq: int
    mean_sk: int
    varlen: bool
    h: int
    h_k: int
    d: int
    dv: int
    causal: bool
    seed: int = 0


def make_dense_case(t: DenseCase):
    """Returns dict with q,k,v,d_out (bf16, packed varlen), cu_q, cu_k (int32), max_q, max_k, scale."""
    torch.manual_seed(t.seed)
    random.seed(t.seed)
    sq = torch.full((t.b,), t.mean_sq, dtype=torch.int32)
    sk = torch.full((t.b,), t.mean_sk, dtype=torch.int32)
    if t.varlen:
        for i in range(t.b):
            sq[i] = max(random.normalvariate(t.mean_sq, t.mean_sq / 2), 1)
        for i in range(t.b):
            sk[i] = max(random.normalvariate(t.mean_sk, t.mean_sk / 2), int(sq[i]))
    cu_q = torch.cumsum(torch.nn.functional.pad(sq, (1, 0)), 0, dtype=torch.int32)
    cu_k = torch.cumsum(torch.nn.functional.pad(sk, (1, 0)), 0, dtype=torch.int32)
    tq, tk = int(sq.sum()), int(sk.sum())
    mk = lambda *s: (torch.randn(*s) / 10).to(torch.bfloat16)
    return dict(q=mk(tq, t.h, t.d), k=mk(tk, t.h_k, t.d), v=mk(tk, t.h_k, t.dv),
                d_out=mk(tq, t.h, t.dv), cu_q=cu_q, cu_k=cu_k,
                max_q=int(sq.max()), max_k=int(sk.max()),
                scale=(t.d + 100) ** -0.5)
