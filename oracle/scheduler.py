"""Integer oracles of the split-KV tile scheduler (test infrastructure only).

`get_mla_metadata_ref` follows the reference, csrc/smxx/get_mla_metadata.cu:25-88 (the single-warp greedy walk)
with the partition sizing of csrc/pybind.cpp:288-380; it documents the output contract and is the yardstick for
the balance of any other schedule.  `schedule_cut_ref` is the integer statement of the schedule this library's
kernel computes (proportional cuts of the cost line, snapped to request boundaries): the CUDA scheduler must
match it bit for bit.  Both satisfy `check_schedule_invariants`, which is all a consumer relies on (the two
tensors are opaque to callers, flash_mla_interface.py:116-163).
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

TILE_SCHEDULER_METADATA_SIZE = 8  # csrc/params.h:51
FIXED_OVERHEAD_NUM_BLOCKS = 5     # csrc/pybind.cpp:308,323,341
BLOCK_SIZE_N = 64                 # csrc/pybind.cpp:309,324,342


def cdiv(a: int, b: int) -> int:
    return (a + b - 1) // b


def num_sm_parts_ref(sm_count: int, num_q_tokens_per_head_k: int, h_k: int,
                     h_q: Optional[int], is_sparse: bool) -> int:
    """How many partitions the schedule is cut into.

    Dense: the Hopper formula, csrc/pybind.cpp:321-325 (the reference has no
    dense Blackwell kernel and refuses at :349-355; one CTA handles 64 query rows
    here as well, so the same formula applies).
    Sparse FP8: the Blackwell formula, csrc/pybind.cpp:339-343.
    """
    if is_sparse:
        assert h_q is not None and h_q % h_k == 0
        s_q = num_q_tokens_per_head_k * h_k // h_q
        return max(sm_count // h_k // (cdiv(h_q // h_k, 64) * s_q), 1)
    return max(sm_count // h_k // cdiv(num_q_tokens_per_head_k, 64), 1)


def get_mla_metadata_ref(seqlens_k: Sequence[int], num_sm_parts: int,
                         topk: int = -1,
                         block_size_n: int = BLOCK_SIZE_N,
                         fixed_overhead_num_blocks: int = FIXED_OVERHEAD_NUM_BLOCKS,
                         ) -> Tuple[List[List[int]], List[int]]:
    """Returns (tile_scheduler_metadata [num_sm_parts][8], num_splits [b+1]).

    Row layout (csrc/params.h:52): [begin_idx, begin_block_idx, end_idx
    (inclusive), end_block_idx (exclusive), begin_n_split_idx, 0, 0, 0].
    Unlike the reference (which leaves words 5..7 uninitialised) the unused words
    are defined to be zero.
    """
    b = len(seqlens_k)
    # get_mla_metadata.cu:26-41: per-request block counts; a zero-length request
    # still counts as one block.
    lens = [int(s) if topk == -1 else int(topk) for s in seqlens_k]
    last_block = [max(l - 1, 0) // block_size_n for l in lens]
    num_blocks = [lb + 1 for lb in last_block]
    total = sum(nb + fixed_overhead_num_blocks for nb in num_blocks)

    # get_mla_metadata.cu:47-48
    payload = cdiv(total, num_sm_parts) + fixed_overhead_num_blocks

    md = [[0] * TILE_SCHEDULER_METADATA_SIZE for _ in range(num_sm_parts)]
    num_splits = [0] * (b + 1)
    now_idx = now_block = now_n_split_idx = cum = 0
    for i in range(num_sm_parts):                       # :52
        md[i][0] = now_idx
        md[i][1] = now_block                            # first block idx is always 0
        md[i][4] = now_n_split_idx
        remain = payload
        while now_idx < b:                              # :58-75
            rem_blocks = num_blocks[now_idx] - now_block
            if remain >= rem_blocks + fixed_overhead_num_blocks:
                cum += now_n_split_idx + 1
                num_splits[now_idx + 1] = cum
                remain -= rem_blocks + fixed_overhead_num_blocks
                now_idx += 1
                now_block = 0
                now_n_split_idx = 0
            else:
                if remain - fixed_overhead_num_blocks > 0:
                    now_block += remain - fixed_overhead_num_blocks
                    now_n_split_idx += 1
                    remain = 0
                break
        # :76-77 ; when the walk stopped exactly on a request boundary the part
        # ends with the previous request (end_block = its block count, or 0 for a
        # zero-length request).  Parts past the end of the batch get
        # begin_idx == b, which consumers treat as "nothing to do".
        if now_block > 0:
            md[i][2] = now_idx
            md[i][3] = now_block
        else:
            md[i][2] = now_idx - 1
            if now_idx >= 1:
                md[i][3] = 0 if lens[now_idx - 1] == 0 else last_block[now_idx - 1] + 1
            else:
                md[i][3] = 0
    assert now_idx == b and now_block == 0 and now_n_split_idx == 0, \
        "schedule did not cover the batch"              # :82
    return md, num_splits


SNAP_BLOCKS = 0     # a cut this close to a request boundary moves onto it (0: only cuts inside an overhead stretch move)


def schedule_cut_ref(seqlens_k: Sequence[int], num_sm_parts: int, topk: int = -1,
                     block_size_n: int = BLOCK_SIZE_N,
                     fixed_overhead_num_blocks: int = FIXED_OVERHEAD_NUM_BLOCKS,
                     snap: int = SNAP_BLOCKS) -> Tuple[List[List[int]], List[int]]:
    """The schedule of this library (same output contract as `get_mla_metadata_ref`).

    Every request costs its block count (a zero-length request counts one block) plus a fixed overhead, laid out
    on a line as [overhead | blocks] per request.  Cut k of num_sm_parts + 1 sits at k * pitch on that line.
    With more requests than parts pitch = ceil(total / parts): every part then carries at most that many cost
    units plus one overhead for starting in the middle of a request, the same bound as the reference's greedy
    walk.  With at most one request per part pitch = ceil(total / parts) + overhead: the slack lets a batch of
    similar requests fall one request per part instead of being cut everywhere (the last parts may then stay
    empty).  A cut inside an overhead stretch (or within `snap` blocks of either end of a request's blocks)
    moves to that request boundary.  Part k is everything between cuts k and k+1; equal cuts give an empty
    part (begin_idx = batch).  Each cut depends only on the prefix sums, so the parts are computed
    independently of each other, in parallel on the GPU.
    """
    b = len(seqlens_k)
    lens = [int(s) if topk == -1 else int(topk) for s in seqlens_k]
    real = [0 if l == 0 else cdiv(l, block_size_n) for l in lens]
    nblk = [max(r, 1) for r in real]
    pre = [0] * (b + 1)
    for i in range(b):
        pre[i + 1] = pre[i] + nblk[i] + fixed_overhead_num_blocks
    total = pre[b]
    pitch = cdiv(total, num_sm_parts) + (fixed_overhead_num_blocks if b <= num_sm_parts else 0)

    def cut(k: int) -> Tuple[int, int]:
        x = k * pitch
        if k >= num_sm_parts or x >= total:
            return (b, 0)
        lo, hi = 0, b                     # last request r with pre[r] <= x
        while hi - lo > 1:
            mid = (lo + hi) // 2
            if pre[mid] <= x:
                lo = mid
            else:
                hi = mid
        r = lo
        off = x - pre[r] - fixed_overhead_num_blocks
        if off <= snap:
            return (r, 0)
        if nblk[r] - off <= snap:
            return (r + 1, 0)
        return (r, off)

    cuts = [cut(k) for k in range(num_sm_parts + 1)]
    md = [[0] * TILE_SCHEDULER_METADATA_SIZE for _ in range(num_sm_parts)]
    counts = [1] * b
    for k in range(num_sm_parts):
        (r0, o0), (r1, o1) = cuts[k], cuts[k + 1]
        if (r0, o0) == (r1, o1):
            md[k][0], md[k][2] = b, b - 1
            continue
        # distinct earlier cuts strictly inside request r0 = position of this part among the parts of r0
        split = 0
        if o0 > 0:
            j = k
            while j >= 1 and cuts[j][0] == r0 and cuts[j][1] > 0:
                if cuts[j] != cuts[j - 1]:
                    split += 1
                j -= 1
            counts[r0] = max(counts[r0], split + 1)
        md[k][0], md[k][1], md[k][4] = r0, o0, split
        if o1 > 0:
            md[k][2], md[k][3] = r1, o1
        else:
            md[k][2], md[k][3] = r1 - 1, real[r1 - 1]
    num_splits = [0] * (b + 1)
    for i in range(b):
        num_splits[i + 1] = num_splits[i] + counts[i]
    return md, num_splits


def max_part_cost(md, seqlens_k, topk: int = -1, block_size_n: int = BLOCK_SIZE_N,
                  fixed_overhead_num_blocks: int = FIXED_OVERHEAD_NUM_BLOCKS) -> int:
    """Largest cost of a part (blocks + overhead per visited request): what the slowest CTA has to do."""
    b = len(seqlens_k)
    lens = [int(s) if topk == -1 else int(topk) for s in seqlens_k]
    nblk = [0 if l == 0 else cdiv(l, block_size_n) for l in lens]
    worst = 0
    for bi, bb, ei, eb in (row[:4] for row in md):
        if bi >= b:
            continue
        c = 0
        for r in range(bi, ei + 1):
            c += (eb if r == ei else nblk[r]) - (bb if r == bi else 0) + fixed_overhead_num_blocks
        worst = max(worst, c)
    return worst


def check_schedule_invariants(md, num_splits, seqlens_k, topk: int = -1,
                              block_size_n: int = BLOCK_SIZE_N) -> None:
    """Coverage / disjointness invariants of any valid schedule."""
    b = len(seqlens_k)
    lens = [int(s) if topk == -1 else int(topk) for s in seqlens_k]
    nblk = [0 if l == 0 else cdiv(l, block_size_n) for l in lens]
    covered = [[0] * max(n, 1) for n in nblk]
    visits = [0] * b
    for row in md:
        bi, bb, ei, eb, ns = row[:5]
        if bi >= b:
            continue
        for r in range(bi, ei + 1):
            lo = bb if r == bi else 0
            hi = eb if r == ei else nblk[r]
            split_idx = ns if r == bi else 0
            assert split_idx == visits[r], (r, split_idx, visits[r])
            visits[r] += 1
            for k in range(lo, hi):
                covered[r][k] += 1
    for r in range(b):
        assert all(c == 1 for c in covered[r][:nblk[r]]), ("coverage", r, covered[r])
        assert visits[r] >= 1, ("request never visited", r)
        assert num_splits[r + 1] - num_splits[r] == visits[r], (r, num_splits, visits)
    assert num_splits[0] == 0
