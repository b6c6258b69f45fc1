"""world_size-2 CPU run of request-sharded decode: each rank takes its shard of the batch
(parallel.shard_requests), computes it independently (oracle in place of the kernel), and the
gathered result must equal the full-batch result.  No data-path collective: the gather is only the
test's way to compare."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from flashmla_windows_linux_sm120_b200 import parallel   # noqa: E402
from oracle import decode, gen                            # noqa: E402

dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
t = gen.DecodeCase(b=6, s_q=2, s_k=300, is_varlen=True, is_causal=True, h_q=8, seed=5)
d = gen.make_decode_case(t)
shards = parallel.shard_requests(d.cache_seqlens.tolist(), world)
mine = shards[rank]
idx = torch.tensor(mine, dtype=torch.long)
out, lse = decode.decode_ref(d.cache_seqlens[idx], d.block_table[idx], d.q[idx], d.blocked_k, 512, True)
gathered = [None] * world
dist.all_gather_object(gathered, (mine, out, lse))
if rank == 0:
    full_out, full_lse = decode.decode_ref(d.cache_seqlens, d.block_table, d.q, d.blocked_k, 512, True)
    got_out, got_lse = torch.empty_like(full_out), torch.empty_like(full_lse)
    for ids, o, l in gathered:
        got_out[ids], got_lse[ids] = o, l
    assert torch.equal(got_out, full_out) and torch.equal(got_lse, full_lse)
    print("OK request sharding", shards)
dist.destroy_process_group()
