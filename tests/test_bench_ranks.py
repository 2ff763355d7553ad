"""The multi-GPU arm of bench.py is replicas only (one independent sequence per GPU, no data-path collective); what the
ranks share is the barrier and the max-over-ranks timing.  Exercised here with two gloo ranks on the CPU."""
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import json, os, sys
sys.path.insert(0, {root!r})
import bench
rank, world, local = bench.dist_env()
r = bench.Ranks(rank, world, local, "gloo")
mine = 0.5 + rank            # rank 1 is the slow one
agg = r.aggregate_rate(100.0, mine)
mx = r.barrier_max(mine)
r.close()
print(json.dumps({{"rank": rank, "world": world, "max": mx, "rate": agg}}))
"""


def test_two_gloo_ranks_agree_on_the_slowest(tmp_path):
    script = tmp_path / "child.py"
    script.write_text(CHILD.format(root=ROOT))
    procs = []
    for rank in range(2):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE="2", LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT="29631")
        procs.append(subprocess.Popen([sys.executable, str(script)], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = []
    for p in procs:
        out, err = p.communicate(timeout=120)
        assert p.returncode == 0, err[-2000:]
        outs.append(json.loads(out.strip().splitlines()[-1]))
    assert sorted(o["rank"] for o in outs) == [0, 1]
    for o in outs:
        assert o["world"] == 2 and o["max"] == 1.5            # both ranks see the slower rank's time
        assert abs(o["rate"] - 2 * 100.0 / 1.5) < 1e-9        # whole-job units over the slowest rank's time


def test_single_rank_needs_no_process_group():
    sys.path.insert(0, ROOT)
    import bench
    r = bench.Ranks(0, 1, 0, "gloo")
    assert r.barrier_max(0.25) == 0.25 and r.aggregate_rate(10, 0.5) == 20.0
    r.close()
