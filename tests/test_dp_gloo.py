"""Data-parallel host logic on CPU: two gloo ranks shard a fraction by sequence, each computes the
gradients of its shard (with the checker, standing in for the GPU kernels), the all-reduced sum must
equal the single-process gradient of the whole fraction, and the summed error the whole error."""
import os
import subprocess
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys
import numpy as np
import torch
import torch.distributed as dist
sys.path[:0] = [os.path.join(ROOT, "project-currennt-public_b200"), os.path.join(ROOT, "oracle"),
                os.path.join(ROOT, "tests"), os.path.join(ROOT, "tests", "golden")]
from b2lstm import dp, workloads
from make_golden import run as run_checker
import parity

dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
layers = [dict(type="input", size=6), dict(type="blstm", size=10, bias=1.0), dict(type="lstm", size=4, bias=1.0),
          dict(type="feedforward_identity", size=3, bias=1.0), dict(type="sse", size=3)]
P, lens = 5, workloads.make_lengths(5, 6, 14, 77)
x, tg = workloads.make_fraction(6, 3, P, lens, 78, 79)
w = workloads.make_weights(layers, 80, 0.2)
full = run_checker("port", layers, P, lens, x, tg, w)
lens_r, x_r, tg_r = dp.shard_fraction(lens, x, tg, rank, world)
mine = run_checker("port", layers, len(lens_r), lens_r, x_r, tg_r, w)
loss = torch.tensor([mine["loss"]], dtype=torch.float64)
dist.all_reduce(loss)
assert abs(loss.item() - full["loss"]) <= 1e-5 * abs(full["loss"]), (loss.item(), full["loss"])
for i in w:
    g = torch.from_numpy(mine["dw%d" % i].copy())
    dist.all_reduce(g)
    parity.assert_grads_close(layers, i, g.numpy(), full["dw%d" % i], "rank %d" % rank)
frames = dp.frames_per_rank(lens, world)
assert sum(frames) == int(lens.sum()) and max(frames) - min(frames) <= int(lens.max())
dist.destroy_process_group()
print("rank", rank, "ok")
'''


def test_two_rank_gradient_sum_equals_single_process(tmp_path):
    script = tmp_path / "worker.py"
    script.write_text("ROOT = %r\n" % ROOT + WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29611", str(script)],
                         capture_output=True, text=True, timeout=300, env=env)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert out.stdout.count("ok") == 2


def test_round_robin_sharding_balances_sorted_lengths():
    sys.path.insert(0, os.path.join(ROOT, "project-currennt-public_b200"))
    from b2lstm import dp, workloads
    lens = workloads.make_lengths(256, 600, 1000, 4004)
    assert (np.diff(lens) <= 0).all()
    for world in (2, 4, 8):
        fr = dp.frames_per_rank(lens, world)
        assert sum(fr) == int(lens.sum())
        assert (max(fr) - min(fr)) / (sum(fr) / world) < 0.01
        seen = np.concatenate([dp.shard_indices(256, r, world) for r in range(world)])
        assert sorted(seen.tolist()) == list(range(256))
