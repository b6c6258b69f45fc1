"""world_size-2 CPU run of the KV-sharded decode: the pages of one context are split over the ranks
(parallel.shard_kv_pages), each rank attends to its shard (oracle), partials are exchanged
(all_gather = the baseline transport) and merged with the split-KV merge arithmetic; the result must
match attention over the whole context."""
import math
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from flashmla_windows_linux_sm120_b200 import parallel   # noqa: E402
from oracle import combine, decode, gen                   # noqa: E402

dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
t = gen.DecodeCase(b=1, s_q=1, s_k=700, h_q=8, seed=9)
d = gen.make_decode_case(t)
L = int(d.cache_seqlens[0])
lo, hi = parallel.shard_kv_pages(L, world)[rank]
nb_lo, nb_hi = lo // 64, (hi + 63) // 64
local_bt = d.block_table[:, nb_lo:nb_hi].contiguous()
local_len = torch.tensor([hi - lo], dtype=torch.int32)
o, lse = decode.decode_ref(local_len, local_bt, d.q, d.blocked_k, 512, False)   # bf16 o, natural lse (+inf if empty)
part_o = o.float().view(-1, 512)
part_lse2 = torch.where(torch.isinf(lse), torch.full_like(lse, float("-inf")), lse * math.log2(math.e)).view(-1)
go = [torch.empty_like(part_o) for _ in range(world)]
gl = [torch.empty_like(part_lse2) for _ in range(world)]
dist.all_gather(go, part_o)
dist.all_gather(gl, part_lse2)
merged_o, merged_lse = combine.combine_ref(torch.stack(gl), torch.stack(go))
full_o, full_lse = decode.decode_ref(d.cache_seqlens, d.block_table, d.q, d.blocked_k, 512, False)
assert (merged_o - full_o.float().view(-1, 512)).abs().max() < 2e-3
assert (merged_lse - full_lse.view(-1)).abs().max() < 1e-4
if rank == 0:
    print("OK kv sharding", parallel.shard_kv_pages(L, world))
dist.destroy_process_group()
