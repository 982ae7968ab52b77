"""world_size-2 check of the replica path on CPU (gloo): sharding covers every sequence once,
the max-over-ranks timing reduction works, and each rank plans the same model independently."""
import os
import subprocess
import sys
import textwrap

from fluidml_b200.replicas import aggregate_throughput, shard

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_shard_partitions_items():
    items = list(range(11))
    parts = [shard(items, r, 4) for r in range(4)]
    assert sorted(sum(parts, [])) == items
    assert max(map(len, parts)) - min(map(len, parts)) <= 1
    assert aggregate_throughput([100, 100], [1.0, 2.0]) == 100.0


def test_two_ranks_gloo(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(textwrap.dedent(f"""
        import os, sys, json
        sys.path.insert(0, {ROOT!r})
        import torch, torch.distributed as dist
        from fluidml_b200 import models
        from fluidml_b200.executor import Executor
        from fluidml_b200.replicas import shard
        dist.init_process_group("gloo")
        rank, world = dist.get_rank(), dist.get_world_size()
        mine = shard(list(range(9)), rank, world)
        st = Executor.make_dp_greedy("bert").plan(models.build_bert(layers=1, vocab=200, hidden=64, heads=4, ffn=128, seq=16).to_bytes())
        t = torch.tensor([1.0 + rank], dtype=torch.float64)
        dist.barrier()
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        got = [None] * world
        dist.all_gather_object(got, (mine, st["peak_arena_bytes"]))
        if rank == 0:
            print(json.dumps({{"max": t.item(), "got": got}}))
        dist.destroy_process_group()
    """))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29731", str(script)],
                         capture_output=True, text=True, env=env, timeout=240)
    assert out.returncode == 0, out.stderr[-2000:]
    import json
    res = json.loads([l for l in out.stdout.splitlines() if l.startswith("{")][-1])
    assert res["max"] == 2.0
    items = sorted(res["got"][0][0] + res["got"][1][0])
    assert items == list(range(9))
    assert res["got"][0][1] == res["got"][1][1]  # both replicas plan the same arena
