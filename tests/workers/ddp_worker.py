"""Data-parallel training over real ranks (one GPU each): after a few steps every rank must hold the
parameters that single-process training on the concatenated batch produces."""
import os
import sys
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
import aluminum_b200 as al  # noqa: E402
from aluminum_b200.models import MLP  # noqa: E402
from aluminum_b200.parallel import DataParallel, Trainer  # noqa: E402

local = int(os.environ.get("AL_LOCAL_RANK", os.environ.get("LOCAL_RANK", "0")))
torch.cuda.set_device(local)
al.init()
comm = al.DeviceComm()
p, me = comm.size, comm.rank
torch.manual_seed(7)                       # same initial weights everywhere (also broadcast by DataParallel)
model = MLP(32, 64, 10).cuda()
ref = MLP(32, 64, 10).cuda()
ref.load_state_dict(model.state_dict())
dp = DataParallel(model, comm, bucket_bytes=8 * 1024, lr=0.05, momentum=0.9)   # tiny buckets: several allreduces
tr = Trainer(dp, autocast_dtype=None)
opt = torch.optim.SGD(ref.parameters(), lr=0.05, momentum=0.9)
lossf = torch.nn.CrossEntropyLoss()
g = torch.Generator().manual_seed(11)
for step in range(4):
    x = torch.randn(8 * p, 32, generator=g).cuda()
    y = torch.randint(0, 10, (8 * p,), generator=g).cuda()
    tr.step_device(x[me * 8:(me + 1) * 8].contiguous(), y[me * 8:(me + 1) * 8].contiguous())
    opt.zero_grad()
    lossf(ref(x), y).backward()           # mean over the global batch = mean of the ranks' means
    opt.step()
torch.cuda.synchronize()
for a, b in zip(model.parameters(), ref.parameters()):
    torch.testing.assert_close(a, b, rtol=2e-4, atol=2e-5)
assert len(dp.buckets) > 1 and dp.launches >= 4 * (len(dp.buckets) + 1)
st = comm.stats()
assert st["timeouts"] == 0
print(f"rank {me} ok: {len(dp.buckets)} buckets, allreduce kernels nvls={st['nvls']} zero_copy={st['nvls_zero_copy']} "
      f"one_shot={st['one_shot']} two_shot={st['two_shot']}")
comm.close()
al.finalize()
