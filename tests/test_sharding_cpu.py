"""CPU suite for the multi-GPU plumbing: event sharding, and the rank meeting (gloo, 2 processes)
that the bench uses to take the maximum time over ranks."""
import os
import subprocess
import sys
import textwrap

import numpy as np

from conftest import ROOT
from hgcalml_b200.sharding import shard_events, local_row_splits, merge_indices


def test_shards_partition_the_batch():
    rng = np.random.default_rng(0)
    for world in (1, 2, 3, 4, 8):
        sizes = rng.integers(0, 1000, 37)
        rs = np.concatenate([[0], np.cumsum(sizes)])
        shards = shard_events(rs, world)
        assert len(shards) == world
        covered = []
        for a, b in shards:
            covered += list(range(a, b))
        assert covered == list(range(37))
        hits = [rs[b] - rs[a] for a, b in shards]
        assert max(hits) <= rs[-1] / world + sizes.max()


def test_equal_events_split_evenly():
    rs = np.arange(65) * 200000
    for world in (1, 2, 4, 8):
        shards = shard_events(rs, world)
        assert [b - a for a, b in shards] == [64 // world] * world


def test_sharded_search_equals_whole_batch(oracle):
    """Searching shards separately and re-offsetting equals one search over the batch."""
    from hgcalml_b200 import synth
    c, _, rs = synth.shower_batch([700, 20, 0, 900, 400], dims=4, n_feat=1, seed=3)
    whole_i, whole_d = oracle.canonical_knn(*oracle.BinnedSelectKnn(12, c, rs))
    parts_i, parts_d = [], []
    for a, b in shard_events(rs, 2):
        lrs, off = local_row_splits(rs, a, b)
        i, d = oracle.BinnedSelectKnn(12, c[off:off + lrs[-1]], lrs)
        parts_i.append(merge_indices(i, off))
        parts_d.append(d)
    got_i, got_d = oracle.canonical_knn(np.concatenate(parts_i), np.concatenate(parts_d))
    assert np.array_equal(got_i, whole_i) and np.array_equal(got_d.view(np.uint32), whole_d.view(np.uint32))


def test_two_ranks_meet_over_gloo(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(textwrap.dedent(f"""
        import os, sys
        sys.path.insert(0, {ROOT!r})
        import numpy as np, torch, torch.distributed as dist
        from hgcalml_b200.sharding import shard_events
        dist.init_process_group("gloo")
        rank, world = dist.get_rank(), dist.get_world_size()
        rs = np.arange(9) * 1000
        a, b = shard_events(rs, world)[rank]
        t = torch.tensor([10.0 + rank, float(b - a)], dtype=torch.float64)
        dist.all_reduce(t[:1], op=dist.ReduceOp.MAX)
        dist.all_reduce(t[1:], op=dist.ReduceOp.SUM)
        assert t[0].item() == 10.0 + world - 1 and t[1].item() == 8.0, t
        dist.barrier()
        dist.destroy_process_group()
        print("rank", rank, "ok")
    """))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT="29533")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                        "--master-addr", "127.0.0.1", "--master-port", "29533", str(script)],
                       env=env, capture_output=True, text=True, timeout=300)
    assert r.returncode == 0, r.stdout + r.stderr
    assert r.stdout.count("ok") == 2
