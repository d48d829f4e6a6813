"""Data-parallel training on CPU ranks must reproduce single-process training on the whole batch.

Every rank builds the same model from the same seed, trains on its shard of each global batch with
HostDataParallel (bucketed non-blocking allreduce on the progress thread) and, on its own, trains
a second copy on the full batch with the same optimizer; after a few steps the parameters must
agree.  Also checks checkpoint save / load."""
import io
import sys
from pathlib import Path

import torch
from torch import nn

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
import aluminum_b200 as al  # noqa: E402
from aluminum_b200.parallel.host_ddp import HostDataParallel  # noqa: E402

torch.set_num_threads(1)
comm = al.HostComm()
p, me = comm.size, comm.rank


def make():
    torch.manual_seed(7)
    return nn.Sequential(nn.Linear(20, 64), nn.Tanh(), nn.Linear(64, 64), nn.Tanh(), nn.Linear(64, 5))


dp = HostDataParallel(make(), comm, bucket_bytes=8 * 1024, lr=0.05, momentum=0.9, weight_decay=1e-3)
ref = HostDataParallel(make(), None, bucket_bytes=8 * 1024, lr=0.05, momentum=0.9, weight_decay=1e-3)
assert len(dp.buckets) > 1
loss_fn = nn.MSELoss()
gen = torch.Generator().manual_seed(123)
per = 6
for step in range(5):
    x = torch.randn(per * p, 20, generator=gen)
    y = torch.randn(per * p, 5, generator=gen)
    xs, ys = x[me * per:(me + 1) * per], y[me * per:(me + 1) * per]
    loss_fn(dp(xs), ys).backward()
    dp.step()
    loss_fn(ref(x), y).backward()   # mean over the whole batch == mean of the shard means
    ref.step()
    if step == 2:
        buf = io.BytesIO()
        torch.save(dp.state_dict(), buf)
        buf.seek(0)
        dp.load_state_dict(torch.load(buf))
err = (dp.flat_param - ref.flat_param).abs().max().item()
assert err < 1e-5, err
# every rank holds the same parameters bit for bit
mine = dp.flat_param.numpy().copy()
lo, hi = mine.copy(), mine.copy()
comm.allreduce(lo, op="min")
comm.allreduce(hi, op="max")
assert (lo == hi).all()
print(f"rank {me}: data parallel on CPU ok ({len(dp.buckets)} buckets, max err {err:.2e})")
