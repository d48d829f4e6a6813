"""Data-parallel training that outlives a rank (CPU ranks): the last rank leaves after two steps; the
others get an error out of backward() or step(), rebuild the trainer on a communicator of the survivors
and train on.  Afterwards every surviving replica holds the same finite parameters."""
import sys
from pathlib import Path

import numpy as np
import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
import aluminum_b200 as al  # noqa: E402
from aluminum_b200.parallel.host_ddp import HostDataParallel  # noqa: E402

comm = al.HostComm()
p, me = comm.size, comm.rank
torch.manual_seed(3)
model = torch.nn.Sequential(torch.nn.Linear(16, 64), torch.nn.ReLU(), torch.nn.Linear(64, 4))
dp = HostDataParallel(model, comm, bucket_bytes=2048, lr=0.05)
g = torch.Generator().manual_seed(100)
data, target = torch.randn(64, 16, generator=g), torch.randn(64, 4, generator=g)


def train_step(k):
    rows = torch.arange(me + k, 64, max(p, 1)) % 64
    loss = torch.nn.functional.mse_loss(dp(data[rows]), target[rows])
    loss.backward()
    dp.step()
    return float(loss.detach())


lost = False
for k in range(6):
    if k == 2 and me == p - 1:
        print(f"rank {me} leaves")
        sys.exit(0)
    try:
        train_step(k)
    except al.AlError:
        assert k == 2 and not lost, k
        lost = True
        alive = al.alive_ranks()
        while len(alive) != p - 1:
            alive = al.alive_ranks()
        dp.rebuild(al.HostComm.from_ranks(alive))
        train_step(k)
assert lost
flat = dp.flat_param.numpy()
allp = np.empty(flat.size * dp.comm.size, dtype=np.float32)
dp.comm.allgather(flat, allp)
assert np.isfinite(allp).all()
assert all(np.array_equal(allp[:flat.size], allp[flat.size * r:flat.size * (r + 1)]) for r in range(dp.comm.size))
print(f"rank {me}: trained on with {dp.comm.size} ranks, steps {dp.steps}")
