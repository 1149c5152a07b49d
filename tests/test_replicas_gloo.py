"""The multi-GPU path is N independent replicas plus a gloo control plane; this
runs that control plane with two CPU ranks."""
import os
import socket
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r"""
import os, sys, json
sys.path.insert(0, %r)
from megaqwen_b200.replicas import dist_env, init_control_plane, barrier, max_over_ranks, aggregate_throughput, replica_seed
from megaqwen_b200.spec import QWEN3_TINY
from megaqwen_b200.synthetic import random_prompt
rank, world, local = dist_env()
dist = init_control_plane(world)
barrier(dist)
# every rank times its own replica: rank r took (1 + r) seconds for 100 units
slow = max_over_ranks(dist, [1.0 + rank, 5.0 - rank])
prompt = random_prompt(QWEN3_TINY, 8, 2, replica_seed(0, rank)).tolist()
barrier(dist)
out = {"world": world, "slow": slow, "value": aggregate_throughput(100, world, slow[0]), "prompt": prompt}
with open(os.path.join(%r, "rank%%d.json" %% rank), "w") as fh:
    json.dump(out, fh)
"""


def free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def test_two_rank_control_plane(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text(WORKER % (ROOT, str(tmp_path)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", str(free_port()), str(script)]
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=240)
    assert res.returncode == 0, res.stderr[-2000:]
    import json
    d0 = json.load(open(tmp_path / "rank0.json"))
    d1 = json.load(open(tmp_path / "rank1.json"))
    assert d0["world"] == 2
    assert d0["slow"] == [2.0, 5.0] == d1["slow"]     # max over ranks of (1+r, 5-r)
    assert abs(d0["value"] - 100.0) < 1e-9            # 2 replicas x 100 units / 2 s
    assert d0["prompt"] != d1["prompt"]               # every replica decodes its own prompt


def test_single_process_is_identity():
    from megaqwen_b200.replicas import aggregate_throughput, barrier, init_control_plane, max_over_ranks
    assert init_control_plane(1) is None
    barrier(None)
    assert max_over_ranks(None, [3.0, 1.0]) == [3.0, 1.0]
    assert aggregate_throughput(256, 8, 0.5) == 4096.0
