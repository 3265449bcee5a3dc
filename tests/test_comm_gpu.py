"""The C ABI's NCCL allreduce of fp32 partials (thor_b200_comm_*): one rank on one GPU, and two ranks as two
processes when the machine has two GPUs (NVLS off, plain rings: the ranks only exchange 64 KiB)."""
import os
import subprocess
import sys
import tempfile

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_single_rank_allreduce_is_the_identity():
    from thor_b200.sharding import Communicator

    comm = Communicator(1, 0, Communicator.unique_id())
    x = torch.arange(16384, dtype=torch.float32, device="cuda")
    want = x.clone()
    for op in ("sum", "max", "min"):
        comm.allreduce(x, op)
    torch.cuda.synchronize()
    assert torch.equal(x, want)
    # the grouped statistics call: sums, NaN-propagating maxima and minima through ordered keys, identity on one rank
    mx = torch.tensor([float("-inf"), -2.5, -0.0, 0.0, 3.0, float("inf"), float("nan")], device="cuda")
    mn = mx.clone()
    keep = mx.clone()
    comm.allreduce_stats(sums=x, maxima=mx, minima=mn)
    torch.cuda.synchronize()
    assert torch.equal(x, want)
    for got in (mx, mn):
        assert torch.equal(got[:-1].view(torch.int32), keep[:-1].view(torch.int32)) and torch.isnan(got[-1])
    comm.close()


_RANK_SCRIPT = r"""
import os, sys, time, torch
rank, world, id_path = int(sys.argv[1]), int(sys.argv[2]), sys.argv[3]
torch.cuda.set_device(rank)
from thor_b200.sharding import Communicator
if rank == 0:
    uid = Communicator.unique_id()
    with open(id_path + ".tmp", "wb") as f: f.write(uid)
    os.replace(id_path + ".tmp", id_path)
else:
    for _ in range(600):
        if os.path.exists(id_path): break
        time.sleep(0.05)
    uid = open(id_path, "rb").read()
comm = Communicator(world, rank, uid)
sums = torch.full((16384,), float(rank + 1), device="cuda")
maxima = torch.tensor([float(rank), -float(rank)], device="cuda")
comm.allreduce(sums, "sum")
comm.allreduce(maxima, "max")
torch.cuda.synchronize()
assert bool((sums == sum(range(1, world + 1))).all()), sums[:4]
assert maxima.tolist() == [float(world - 1), 0.0], maxima
# one group for a step's statistics; a NaN in exactly one rank's shard is the global extreme
s2 = torch.full((2,), float(rank + 1), device="cuda")
mx = torch.tensor([float(rank), float("nan") if rank == world - 1 else 1.0], device="cuda")
mn = torch.tensor([float(rank), float("nan") if rank == 0 else 1.0], device="cuda")
comm.allreduce_stats(sums=s2, maxima=mx, minima=mn)
torch.cuda.synchronize()
assert s2.tolist() == [float(sum(range(1, world + 1)))] * 2, s2
assert mx[0].item() == world - 1 and torch.isnan(mx[1]) and mn[0].item() == 0 and torch.isnan(mn[1]), (mx, mn)
# the overlapped combiner: four steps over two slots, sums rounded to bf16 once after the combine
from thor_b200.sharding import Combiner
cb = Combiner(comm, 2)
sums = [torch.zeros(2, 4096, device="cuda") for _ in range(2)]
rounded = [torch.zeros(2, 4096, device="cuda", dtype=torch.bfloat16) for _ in range(2)]
mx = [torch.zeros(1, device="cuda") for _ in range(2)]
bound = [cb.bind(b, sums=sums[b], maxima=mx[b], rounded_sums=rounded[b]) for b in range(2)]  # the same calls with everything resolved once
for step in range(4):
    b = step & 1
    cb.wait(b) if step < 2 else bound[b].wait()
    sums[b].fill_(float(rank + 1) * (step + 1) + 0.001)
    mx[b].fill_(float(rank * (step + 1)))
    cb.submit(b, sums=sums[b], maxima=mx[b], rounded_sums=rounded[b]) if step < 2 else bound[b].submit()
cb.drain()
torch.cuda.synchronize()
total = sum(range(1, world + 1))
for b, step in ((0, 2), (1, 3)):
    want = torch.full((2, 4096), 0.0, device="cuda")
    for r in range(world):
        want += float(r + 1) * (step + 1) + 0.001
    assert torch.equal(sums[b], want), (sums[b][0, :2], want[0, :2])
    assert torch.equal(rounded[b], want.bfloat16()) and mx[b].item() == (world - 1) * (step + 1)
cb.close()
comm.close()
print("rank", rank, "ok")
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_combine_partials():
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    with tempfile.TemporaryDirectory() as d:
        id_path = os.path.join(d, "nccl_id")
        procs = [subprocess.Popen([sys.executable, "-c", _RANK_SCRIPT, str(r), "2", id_path], env=env, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
                 for r in range(2)]
        outs = []
        for p in procs:
            try:
                out, _ = p.communicate(timeout=120)
            except subprocess.TimeoutExpired:
                p.kill()
                out, _ = p.communicate()
            outs.append(out)
        for r, (p, out) in enumerate(zip(procs, outs)):
            assert p.returncode == 0 and f"rank {r} ok" in out, out[-2000:]
