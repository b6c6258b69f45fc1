"""CPU tests of the multi-GPU host logic: sharding helpers, and world_size-2 gloo runs of the two
sharded paths (request sharding without any exchange; KV sharding + log-sum-exp merge of partials)
with the oracle standing in for the kernels."""
import os
import subprocess
import sys

import pytest

from flashmla_windows_linux_sm120_b200 import parallel

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_requests_balanced_and_complete():
    lens = [4096, 100, 5000, 3000, 64, 4000, 7, 2500]
    for n in (1, 2, 3, 8):
        shards = parallel.shard_requests(lens, n)
        assert sorted(i for s in shards for i in s) == list(range(len(lens)))
        loads = [sum(lens[i] + 320 for i in s) for s in shards]
        assert max(loads) - min(loads) <= max(lens) + 320
    assert parallel.shard_requests([], 2) == [[], []]


def test_shard_sequences_by_quadratic_cost():
    shards = parallel.shard_sequences([8192, 1024, 1024, 1024, 1024, 1024, 1024, 1024], 2)
    assert [0] in shards            # the long sequence is alone: 8192^2 dominates 7 * 1024^2


def test_shard_query_tokens_and_kv_pages():
    assert parallel.shard_query_tokens(10, 4) == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert parallel.shard_query_tokens(2, 4) == [(0, 1), (1, 2), (2, 2), (2, 2)]
    sh = parallel.shard_kv_pages(1000, 4)
    assert sh[0][0] == 0 and sh[-1][1] == 1000
    assert all(a % 64 == 0 for a, _ in sh) and all(x[1] == y[0] for x, y in zip(sh, sh[1:]))
    assert parallel.shard_kv_pages(100, 8)[-1] == (100, 100)     # more ranks than pages: empty shards
    assert parallel.shard_kv_pages(1 << 20, 8) == [(i << 17, (i + 1) << 17) for i in range(8)]


@pytest.mark.parametrize("script", ["gloo_request_sharding.py", "gloo_kv_sharding.py"])
def test_world_size_2_gloo(script):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29517", os.path.join(ROOT, "tests", "multi_gpu", script)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-2000:]
    assert "OK" in r.stdout
