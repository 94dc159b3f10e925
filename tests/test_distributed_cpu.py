"""World-size-2 `gloo` test of the benchmark's multi-rank plumbing (no GPU): rendezvous on 127.0.0.1,
barrier, maximum over ranks, and that the rank shards tile the batch exactly like the library's own slicing."""
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import os, sys, json
sys.path.insert(0, %r)
from thnets_b200.distributed import Ranks
r = Ranks("gloo")
r.barrier()
worst = r.max(10.0 + r.rank)          # rank 1 is "slower"
total = r.sum(256)                    # every rank processed 256 images (weak scaling)
off, cnt = r.shard(251)
r.barrier()
# host-side hand-over: rank 1 blocks on the store (no collective in flight) until rank 0 has done its solo work
import time
if r.rank == 0:
    time.sleep(0.5)
    open(os.path.join(%r, "solo_done"), "w").write("x")
    r.host_signal("solo")
else:
    r.host_wait("solo", 60)
    assert os.path.exists(os.path.join(%r, "solo_done"))
r.barrier()
print(json.dumps(dict(rank=r.rank, world=r.world, worst=worst, total=total, off=off, cnt=cnt)))
r.close()
"""


def test_two_ranks_gloo(tmp_path):
    script = tmp_path / "child.py"
    script.write_text(CHILD % (ROOT, str(tmp_path), str(tmp_path)))
    port = 29500 + os.getpid() % 2000
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), WORLD_SIZE="2", OMP_NUM_THREADS="1")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(i), LOCAL_RANK=str(i)),
                              stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for i in range(2)]
    import json
    outs = []
    for p in procs:
        out, err = p.communicate(timeout=180)
        assert p.returncode == 0, err[-2000:]
        outs.append(json.loads(out.strip().splitlines()[-1]))
    outs.sort(key=lambda o: o["rank"])
    assert [o["world"] for o in outs] == [2, 2]
    assert all(o["worst"] == 11.0 for o in outs)       # max over ranks, seen by every rank
    assert all(o["total"] == 512.0 for o in outs)
    assert (outs[0]["off"], outs[0]["cnt"], outs[1]["off"], outs[1]["cnt"]) == (0, 126, 126, 125)


def test_single_rank_is_a_no_op():
    sys.path.insert(0, ROOT)
    from thnets_b200.distributed import Ranks
    env_backup = {k: os.environ.pop(k, None) for k in ("RANK", "WORLD_SIZE", "LOCAL_RANK")}
    try:
        r = Ranks()
        assert (r.rank, r.world) == (0, 1) and r.max(3.5) == 3.5 and r.shard(10) == (0, 10)
        r.barrier()
        r.close()
    finally:
        for k, v in env_backup.items():
            if v is not None:
                os.environ[k] = v
