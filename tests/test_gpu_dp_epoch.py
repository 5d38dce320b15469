"""Two-GPU test of data-parallel training from a sharded .nc data set: two ranks, each with its shard
of every fraction and a full weight replica, must end an epoch with the weights a single GPU reaches
on the unsharded fractions (same gradient sums up to fp32 summation order), including a last fraction
that leaves one rank without a sequence.  Skipped on a box with fewer than two GPUs."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

WORKER = r'''
import os, sys
import numpy as np
import torch
import torch.distributed as dist
sys.path[:0] = [os.path.join(ROOT, "project-currennt-public_b200")]
import b2lstm
from b2lstm import workloads

rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
torch.cuda.set_device(int(os.environ["LOCAL_RANK"]))
dist.init_process_group("nccl")
layers = [dict(type="input", size=9), dict(type="blstm", size=64, bias=1.0), dict(type="feedforward_identity", size=4, bias=1.0),
          dict(type="sse", size=4)]
P = 2
w = workloads.make_weights(layers, 5, 0.1)
net = b2lstm.Net(layers, P, 40)
for i, wi in w.items():
    net.set_weights(i, wi)
idt = torch.zeros(128, dtype=torch.uint8, device="cuda")
if rank == 0:
    idt.copy_(torch.frombuffer(bytearray(b2lstm.dp_unique_id()), dtype=torch.uint8))
dist.broadcast(idt, 0)
net.dp_attach(rank, world, bytes(idt.cpu().numpy().tobytes()))
ds = b2lstm.DataSet(PATH, P, shard_rank=rank, shard_count=world)
out = [b2lstm.train_epoch(net, ds, 1e-3, 0.9) for _ in range(2)]
net.synchronize()
np.savez(os.path.join(OUT, "rank%d.npz" % rank), err=np.array([o[0] for o in out]), frames=np.array([o[1] for o in out]),
         **{"w%d" % i: net.get_weights(i) for i in w})
net.dp_detach()
dist.destroy_process_group()
print("rank", rank, "ok")
'''


def test_two_ranks_on_shards_match_one_gpu_on_whole_fractions(tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import b2lstm
    from b2lstm import workloads
    rng = np.random.default_rng(3)
    lens = [12, 30, 7, 22, 18, 25, 9, 14, 27]          # 9 sequences, 4 per global fraction: the last one holds 1
    n = int(sum(lens))
    x = rng.standard_normal((n, 9)).astype(np.float32)
    y = rng.standard_normal((n, 4)).astype(np.float32)
    path = str(tmp_path / "dp.nc")
    b2lstm.write_nc(path, ["s%02d" % i for i in range(len(lens))], lens, x, y)
    script = tmp_path / "worker.py"
    script.write_text("ROOT = %r\nPATH = %r\nOUT = %r\n" % (ROOT, path, str(tmp_path)) + WORKER)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                          "--master-addr", "127.0.0.1", "--master-port", "29631", str(script)],
                         capture_output=True, text=True, timeout=600, env=env)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert out.stdout.count("ok") == 2

    # one GPU, the same sequences in fractions of 2 x 2
    layers = [dict(type="input", size=9), dict(type="blstm", size=64, bias=1.0), dict(type="feedforward_identity", size=4, bias=1.0),
              dict(type="sse", size=4)]
    w = workloads.make_weights(layers, 5, 0.1)
    net = b2lstm.Net(layers, 4, 40)
    for i, wi in w.items():
        net.set_weights(i, wi)
    ds = b2lstm.DataSet(path, 4)
    want = [b2lstm.train_epoch(net, ds, 1e-3, 0.9) for _ in range(2)]
    r0, r1 = np.load(tmp_path / "rank0.npz"), np.load(tmp_path / "rank1.npz")
    for i in w:
        assert np.array_equal(r0["w%d" % i], r1["w%d" % i])                     # replicas stay identical
        ref = net.get_weights(i)
        assert np.allclose(r0["w%d" % i], ref, rtol=1e-4, atol=1e-6), np.abs(r0["w%d" % i] - ref).max()
        assert not np.array_equal(ref, w[i])
    for k in range(2):
        assert r0["frames"][k] == r1["frames"][k] == want[k][1] == sum(lens)
        assert abs(r0["err"][k] - want[k][0]) <= 1e-4 * abs(want[k][0])
        assert r0["err"][k] == r1["err"][k]
    net.close()
