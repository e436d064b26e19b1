"""CPU-only coverage of the multi-rank logic of bench.py: the batch split and the gather of the
per-rank outputs to rank 0, with two gloo ranks (no GPU involved)."""
import os
import socket
import sys

import numpy as np

from conftest import ROOT

sys.path.insert(0, ROOT)
import bench  # noqa: E402


def test_shard_covers_the_batch_exactly():
    for total in (256, 255, 7, 1):
        for world in (1, 2, 3, 4, 8):
            spans = [bench.shard(total, world, r) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == total
            for a, b in zip(spans, spans[1:]):
                assert a[1] == b[0]
            sizes = [e - b for b, e in spans]
            assert max(sizes) - min(sizes) <= 1


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


RANK_SCRIPT = r"""
import os, sys
import numpy as np
import torch
import torch.distributed as dist
sys.path.insert(0, sys.argv[1])
import bench
total, out_path = int(sys.argv[2]), sys.argv[3]
dist.init_process_group("gloo")        # RANK / WORLD_SIZE / MASTER_* from the environment, as under torchrun
rank, world = dist.get_rank(), dist.get_world_size()
begin, end = bench.shard(total, world, rank)
# stand-in for the rank's forward pass: row i of the global output holds i everywhere
local = torch.arange(begin, end, dtype=torch.float32).unsqueeze(1).repeat(1, 10)
counts = [bench.shard(total, world, r)[1] - bench.shard(total, world, r)[0] for r in range(world)]
gathered = [torch.empty(c, 10) for c in counts] if rank == 0 else None
dist.gather(local, gathered, dst=0)
t = torch.tensor([float(rank + 1)])
dist.all_reduce(t, op=dist.ReduceOp.MAX)        # the max-over-ranks reduction the timing uses
if rank == 0:
    np.save(out_path, np.concatenate([torch.cat(gathered).numpy().reshape(-1), t.numpy()]))
dist.destroy_process_group()
"""


def test_two_rank_gather_reassembles_the_global_batch(tmp_path):
    import subprocess
    total, world = 12, 2        # the gather needs equal shards; 256 divides by 1, 2, 4 and 8
    out = str(tmp_path / "gathered.npy")
    port = _free_port()
    procs = []
    for rank in range(world):
        env = dict(os.environ, RANK=str(rank), WORLD_SIZE=str(world), LOCAL_RANK=str(rank), MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
        procs.append(subprocess.Popen([sys.executable, "-c", RANK_SCRIPT, ROOT, str(total), out], env=env))
    for p in procs:
        assert p.wait(timeout=300) == 0
    data = np.load(out)
    full, tmax = data[:-1].reshape(total, 10), data[-1]
    assert np.array_equal(full[:, 0], np.arange(total, dtype=np.float32))
    assert tmax == world


def test_reference_arm_json_line_shape():
    """--impl reference prints the contract's keys (a tiny sample here)."""
    import subprocess, json
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                       capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stderr
    line = json.loads(r.stdout.strip().splitlines()[-1])
    for key in ("metric", "value", "unit", "n_gpus", "steps", "warmup", "ms_per_step", "higher_is_better", "scaling", "dtype", "data",
                "config", "impl", "cpu_baseline", "e2e"):
        assert key in line
    assert line["impl"] == "reference" and line["cpu_baseline"]["kind"] in ("reference", "port")
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["value"] > 0
