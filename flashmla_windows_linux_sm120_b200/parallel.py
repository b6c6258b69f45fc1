"""Multi-GPU use of the attention path.

Most of the path shards without any exchange: decode requests, varlen sequences and
sparse-prefill query tokens are independent, so each rank simply owns a subset
(`shard_requests`, `shard_sequences`, `shard_query_tokens`) and runs the single-GPU
API on it.  The one case with a real exchange step is a single very long context
whose cache pages are split along the sequence over the ranks (`shard_kv_pages`):
every rank attends to its shard and the per-rank partial outputs are merged with
the same log-sum-exp arithmetic as the split-KV merge inside one GPU.

`KVShardedDecode` implements that exchange two ways:
  transport="peer"  each rank's merge kernel stores its normalised fp32 partial
                    and a flag straight into every peer's buffer (symmetric memory,
                    plain stores over NVLink); the final merge kernel polls the
                    flags with a bound and reduces the N slots.  No NCCL call on the
                    data path.
  transport="nccl"  the baseline: all_gather of the partials, then the local merge.

The reference has no multi-GPU code at all; the merge math is its
csrc/smxx/mla_combine.cu:71-151.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple

import torch

LOG2E = 1.4426950408889634


# ---------------------------------------------------------------------------------------------------
# sharding of independent work (host-side, pure Python)
# ---------------------------------------------------------------------------------------------------
def _lpt(costs: Sequence[float], world_size: int) -> List[List[int]]:
    """Longest-processing-time-first assignment of items to `world_size` bins; ties broken by index."""
    bins: List[List[int]] = [[] for _ in range(world_size)]
    load = [0.0] * world_size
    for i in sorted(range(len(costs)), key=lambda j: (-costs[j], j)):
        r = min(range(world_size), key=lambda k: (load[k], k))
        bins[r].append(i)
        load[r] += costs[i]
    for b in bins:
        b.sort()
    return bins


def shard_requests(cache_seqlens: Sequence[int], world_size: int) -> List[List[int]]:
    """Decode requests -> ranks, balanced by cached tokens (+5 blocks of fixed cost per request, the
    scheduler's own overhead model, csrc/smxx/get_mla_metadata.cu:37)."""
    return _lpt([int(s) + 5 * 64 for s in cache_seqlens], world_size)


def shard_sequences(lengths: Sequence[int], world_size: int, causal: bool = True) -> List[List[int]]:
    """Varlen prefill sequences -> ranks, balanced by attention work (L^2/2 when causal)."""
    return _lpt([float(l) * float(l) * (0.5 if causal else 1.0) for l in lengths], world_size)


def shard_query_tokens(s_q: int, world_size: int) -> List[Tuple[int, int]]:
    """Sparse-prefill query tokens -> contiguous [begin, end) ranges, sizes differing by at most one."""
    base, rem = divmod(s_q, world_size)
    out, lo = [], 0
    for r in range(world_size):
        hi = lo + base + (1 if r < rem else 0)
        out.append((lo, hi))
        lo = hi
    return out


def shard_kv_pages(seqlen: int, world_size: int, block: int = 64) -> List[Tuple[int, int]]:
    """One context of `seqlen` tokens -> contiguous page-aligned token ranges [begin, end), one per rank."""
    nblk = (seqlen + block - 1) // block
    out = []
    for lo_b, hi_b in shard_query_tokens(nblk, world_size):
        out.append((min(lo_b * block, seqlen), min(hi_b * block, seqlen)))
    return out


# ---------------------------------------------------------------------------------------------------
# KV-sharded decode
# ---------------------------------------------------------------------------------------------------
class PartialBuffers:
    """Two sets (selected by the parity of the step's epoch) of N slots of (partial O [rows, 512] fp32,
    base-2 LSE [rows] fp32, flag uint32) living on one GPU.

    Why two sets: a rank may start the push of step e+1 as soon as its own merge of step e is done, which
    only needs the peers' pushes of step e, not their merges.  With one set it could overwrite a slot that a
    slower peer has not merged yet.  With two, the push of step e+2 (the next one into the same set) comes
    after this rank's merge of e+1, which waited for the peer's push of e+1, which the peer's stream ordered
    after its merge of e: the slot is free by construction, without any extra flag.
    """

    def __init__(self, num_slots: int, rows: int, device, tensors=None):
        self.num_slots, self.rows = num_slots, rows
        if tensors is None:
            o = torch.zeros((2, num_slots, rows, 512), dtype=torch.float32, device=device)
            lse = torch.zeros((2, num_slots, rows), dtype=torch.float32, device=device)
            flags = torch.zeros((2, num_slots), dtype=torch.int32, device=device)
            tensors = (o, lse, flags)
        self.o, self.lse, self.flags = tensors

    def offsets(self, epoch: int) -> Tuple[int, int, int]:
        """Byte offsets of the set used by `epoch` inside the o / lse / flags allocations."""
        par = epoch & 1
        return (par * self.num_slots * self.rows * 512 * 4, par * self.num_slots * self.rows * 4, par * self.num_slots * 4)

    def ptrs(self, epoch: int, bases: Optional[Tuple[int, int, int]] = None) -> Tuple[int, int, int]:
        """Device addresses of the set used by `epoch`; `bases` = the allocations' addresses as another rank sees them."""
        if bases is None:
            bases = (self.o.data_ptr(), self.lse.data_ptr(), self.flags.data_ptr())
        off = self.offsets(epoch)
        return (bases[0] + off[0], bases[1] + off[1], bases[2] + off[2])


def push_partial(q, k_cache, block_table, cache_seqlens, tile_scheduler_metadata, num_splits, softmax_scale,
                 slot: int, dst_ptrs: Sequence[Tuple[int, int, int]], epoch: int, counter: torch.Tensor) -> None:
    """Dense decode over the local shard; the merged partial goes to slot `slot` of every destination
    given as (o_ptr, lse_ptr, flag_ptr) device addresses of the buffer set of this epoch
    (`PartialBuffers.ptrs(epoch, ...)`)."""
    from ._cabi import DecodeParams, PeerPush, check, lib
    b, s_q, h_q, d = q.shape
    num_blocks, page, h_k, _ = k_cache.shape
    parts = tile_scheduler_metadata.shape[0]
    with torch.cuda.device(q.device):
        lse_accum = torch.empty((b + parts, s_q * h_q), dtype=torch.float32, device=q.device)
        o_accum = torch.empty((b + parts, s_q * h_q, 512), dtype=torch.float32, device=q.device)
        p = DecodeParams()
        p.b, p.s_q, p.h_q, p.h_k, p.d, p.d_v = b, s_q, h_q, h_k, d, 512
        p.num_blocks, p.page_block_size = num_blocks, page
        p.is_causal, p.is_fp8, p.topk, p.q_dtype = 0, 0, -1, 0
        p.softmax_scale = float(softmax_scale)
        p.q, p.q_stride_b, p.q_stride_s, p.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1), q.stride(2)
        p.kcache = k_cache.data_ptr()
        p.k_stride_block, p.k_stride_row, p.k_stride_head = k_cache.stride(0), k_cache.stride(1), k_cache.stride(2)
        p.block_table, p.block_table_stride_b = block_table.data_ptr(), block_table.stride(0)
        p.seqlens_k = cache_seqlens.data_ptr()
        p.tile_scheduler_metadata, p.num_sm_parts = tile_scheduler_metadata.data_ptr(), parts
        p.num_splits = num_splits.data_ptr()
        p.lse_accum, p.o_accum = lse_accum.data_ptr(), o_accum.data_ptr()
        push = PeerPush()
        push.slot, push.num_dst, push.epoch, push.counter = slot, len(dst_ptrs), epoch, counter.data_ptr()
        for i, (po, pl, pf) in enumerate(dst_ptrs):
            push.dst_o[i], push.dst_lse[i], push.dst_flag[i] = po, pl, pf
        check(lib.fmla_fwd_kvcache_mla_push_partial(C.byref(p), C.byref(push),
                                                    torch.cuda.current_stream(q.device).cuda_stream))


def merge_partials(buf: PartialBuffers, epoch: int, max_polls: int = 5_000_000):
    """Waits (bounded) for all slots of the buffer set of `epoch` to carry `epoch`, merges them.  Returns
    (out bf16 [rows,512], lse fp32 [rows] natural log).  If the wait runs out the outputs are not written; the
    condition is reported by `fmla_device_status` and by the next library call on this device."""
    from ._cabi import check, lib
    dev = buf.o.device
    po, pl, pf = buf.ptrs(epoch)
    with torch.cuda.device(dev):
        out = torch.empty((buf.rows, 512), dtype=torch.bfloat16, device=dev)
        lse = torch.empty((buf.rows,), dtype=torch.float32, device=dev)
        check(lib.fmla_merge_peer_partials(pl, po, buf.num_slots, buf.rows, 512, pf, epoch, max_polls,
                                           out.data_ptr(), 512, lse.data_ptr(),
                                           torch.cuda.current_stream(dev).cuda_stream))
    return out, lse


class KVShardedDecode:
    """Decode of requests whose KV cache is sharded along the sequence over the ranks of `group`.

    Every rank calls it with the same q [b, 1, h_q, 576] and its own local cache shard
    (k_cache, block_table, cache_seqlens = tokens held locally, possibly 0).  Every rank gets the
    full result (out [b, 1, h_q, 512] bf16, lse [b, h_q, 1] fp32).
    """

    def __init__(self, b: int, h_q: int, device, group=None, transport: str = "peer"):
        import torch.distributed as dist
        assert transport in ("peer", "nccl")
        self.dist, self.group, self.transport = dist, group, transport
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.b, self.h_q, self.rows, self.device = b, h_q, b * h_q, device
        self.epoch = 0
        self.counter = torch.zeros((1,), dtype=torch.int32, device=device)
        if transport == "peer":
            import torch.distributed._symmetric_memory as symm
            n = self.world
            # one symmetric allocation per array: every rank can address every peer's copy
            self._o = symm.empty((2, n, self.rows, 512), dtype=torch.float32, device=device)
            self._lse = symm.empty((2, n, self.rows), dtype=torch.float32, device=device)
            self._flags = symm.empty((2, n), dtype=torch.int32, device=device)
            self._flags.zero_()
            gname = group.group_name if group is not None else dist.group.WORLD.group_name
            self._h = [symm.rendezvous(t, gname) for t in (self._o, self._lse, self._flags)]
            self.buf = PartialBuffers(n, self.rows, device, (self._o, self._lse, self._flags))
            self.peer_bases = [(int(self._h[0].buffer_ptrs[r]), int(self._h[1].buffer_ptrs[r]), int(self._h[2].buffer_ptrs[r]))
                               for r in range(n)]
            torch.cuda.synchronize(device)
            dist.barrier(group)
        else:
            self.buf = PartialBuffers(self.world, self.rows, device)
            self.local = PartialBuffers(1, self.rows, device)

    def __call__(self, q, k_cache, block_table, cache_seqlens, softmax_scale: Optional[float] = None):
        from .flash_mla_interface import get_mla_metadata
        b, s_q, h_q, d = q.shape
        assert s_q == 1 and b == self.b and h_q == self.h_q, "KV-sharded decode handles s_q == 1 queries"
        if softmax_scale is None:
            softmax_scale = d ** -0.5
        md, ns = get_mla_metadata(cache_seqlens, s_q * h_q // k_cache.shape[2], k_cache.shape[2])
        self.epoch += 1
        if self.transport == "peer":
            dst = [self.buf.ptrs(self.epoch, bases) for bases in self.peer_bases]
            push_partial(q, k_cache, block_table, cache_seqlens, md, ns, softmax_scale, self.rank, dst,
                         self.epoch, self.counter)
            out, lse = merge_partials(self.buf, self.epoch)
        else:
            loc = self.local
            par = self.epoch & 1
            push_partial(q, k_cache, block_table, cache_seqlens, md, ns, softmax_scale, 0,
                         [loc.ptrs(self.epoch)], self.epoch, self.counter)
            self.dist.all_gather_into_tensor(self.buf.o[par], loc.o[par, 0], group=self.group)
            self.dist.all_gather_into_tensor(self.buf.lse[par], loc.lse[par, 0], group=self.group)
            self.buf.flags[par].fill_(self.epoch)
            out, lse = merge_partials(self.buf, self.epoch)
        # rows are ordered (batch, head): regrouped row index of a kv head == head for s_q == 1, h_k == 1
        return out.view(b, 1, h_q, 512), lse.view(b, h_q, 1)
