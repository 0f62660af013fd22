"""The N>1 form of the decode path (independent replicas, no data-path collective):
host-side sharding and timing aggregation, run as two ``gloo`` ranks on CPU."""
import os
import socket
import subprocess
import sys
import textwrap

import pytest

from adam_b200.replicas import combine_timings, dist_env, shard_sequences

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


@pytest.mark.parametrize("n,world", [(0, 1), (1, 2), (7, 2), (8, 8), (33, 4), (3, 8)])
def test_shard_sequences_is_a_balanced_partition(n, world):
    parts = [shard_sequences(n, r, world) for r in range(world)]
    flat = [i for p in parts for i in p]
    assert flat == list(range(n))                                  # disjoint, ordered, complete
    sizes = [len(p) for p in parts]
    assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        shard_sequences(n, world, world)


def test_single_process_defaults():
    env = {k: os.environ.pop(k, None) for k in ("RANK", "LOCAL_RANK", "WORLD_SIZE")}
    try:
        assert dist_env() == (0, 0, 1)
        c = combine_timings(2.0, 10, 4000.0, 1)
        assert c["value"] == pytest.approx(5000.0) and c["e2e"] == pytest.approx(4000.0) and c["tokens"] == 10
    finally:
        for k, v in env.items():
            if v is not None:
                os.environ[k] = v


_RANK_SCRIPT = textwrap.dedent("""
    import json, os, sys
    sys.path.insert(0, %r)
    import torch.distributed as dist
    from adam_b200.replicas import combine_timings, dist_env, gather_generated, shard_sequences
    rank, local_rank, world = dist_env()
    dist.init_process_group("gloo")
    # every rank decodes its own share of 5 sequences; rank 1 is the slow one
    mine = shard_sequences(5, rank, world)
    local = [[100 * s + t for t in range(3)] for s in mine]
    ms = 10.0 if rank == 0 else 16.0
    comb = combine_timings(ms, 3 * len(mine), 1000.0 - 100.0 * rank, world)
    allseq = gather_generated(local, world)
    dist.barrier()
    if rank == 0:
        print(json.dumps({"comb": comb, "seqs": allseq, "world": world}))
    dist.destroy_process_group()
""")


def test_two_gloo_ranks_aggregate_like_the_bench(tmp_path):
    script = tmp_path / "rank.py"
    script.write_text(_RANK_SCRIPT % ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), str(script)]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=240, cwd=ROOT)
    assert out.returncode == 0, out.stderr[-2000:]
    import json
    line = [l for l in out.stdout.splitlines() if l.startswith("{")][-1]
    res = json.loads(line)
    assert res["world"] == 2
    # 5 sequences x 3 tokens over the slowest rank's 16 ms; e2e = world x slowest rank's rate
    assert res["comb"]["tokens"] == 15
    assert res["comb"]["ms"] == pytest.approx(16.0)
    assert res["comb"]["value"] == pytest.approx(15 / 16e-3)
    assert res["comb"]["e2e"] == pytest.approx(2 * 900.0)
    assert res["seqs"] == [[100 * s + t for t in range(3)] for s in range(5)]     # rank order = sequence order


def test_reference_arm_other_ranks_do_no_work():
    """Under a multi-rank launch only rank 0 runs the CPU reference arm; the others exit 0 silently."""
    env = dict(os.environ, RANK="1", LOCAL_RANK="1", WORLD_SIZE="2")
    out = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2"],
                         capture_output=True, text=True, timeout=120, cwd=ROOT, env=env)
    assert out.returncode == 0, out.stderr[-2000:]
    assert out.stdout.strip() == ""
