"""Parallelism components over REAL ranks (one process and one GPU each; run under alrun with 2 or 4 ranks):

* tensor + sequence parallel MLP (ColumnParallelLinear -> GELU -> RowParallelLinear with the sequence
  allgathered on entry and reduce-scattered on exit) trains to the same losses and weights as the same MLP
  on one device;
* Ulysses sequence <-> head exchange and expert dispatch / combine: results, gradients, and the kernel list
  of the exchange (one library kernel, no torch copy kernel);
* pipeline: a two-stage GPipe schedule (forward + backward over micro-batches) matches single-device autograd;
* ring attention with the key / value rotation overlapped with the block computation.
"""
import math
import os
import sys
from pathlib import Path

import torch
from torch import nn

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
import aluminum_b200 as al  # noqa: E402
from aluminum_b200.parallel import autograd as ag  # noqa: E402
from aluminum_b200.parallel import context, expert, ulysses  # noqa: E402
from aluminum_b200.parallel.pipeline import PipelineStage  # noqa: E402

local = int(os.environ.get("AL_LOCAL_RANK", os.environ.get("LOCAL_RANK", "0")))
torch.cuda.set_device(local)
al.init()
comm = al.DeviceComm()
p, me = comm.size, comm.rank
comm.set_timeout_ms(8000)
torch.backends.cuda.matmul.allow_tf32 = False
torch.backends.cudnn.allow_tf32 = False

# ---- 1. tensor + sequence parallel MLP vs one device -----------------------------------------------------------
S, B, H = 8 * p, 3, 32
fc1 = ag.ColumnParallelLinear(comm, H, 4 * H, sequence_parallel=True, seed=11)
fc2 = ag.RowParallelLinear(comm, 4 * H, H, sequence_parallel=True, seed=12)
tp = nn.Sequential(fc1, nn.GELU(), fc2)
ref = nn.Sequential(nn.Linear(H, 4 * H), nn.GELU(), nn.Linear(4 * H, H)).cuda()
with torch.no_grad():
    w1, b1 = ag._full_weight(4 * H, H, 11, "cuda", torch.float32)
    w2, b2 = ag._full_weight(H, 4 * H, 12, "cuda", torch.float32)
    ref[0].weight.copy_(w1); ref[0].bias.copy_(b1); ref[2].weight.copy_(w2); ref[2].bias.copy_(b2)
opt = torch.optim.SGD(tp.parameters(), lr=0.05)
ropt = torch.optim.SGD(ref.parameters(), lr=0.05)
g = torch.Generator().manual_seed(3)
for step in range(4):
    x = torch.randn(S, B, H, generator=g).cuda()
    t = torch.randn(S, B, H, generator=g).cuda()
    xs, ts = x.chunk(p, dim=0)[me].contiguous(), t.chunk(p, dim=0)[me].contiguous()
    opt.zero_grad()
    loss = ((tp(xs) - ts) ** 2).sum() / (S * B * H)      # every rank's share of the global mean
    loss.backward()
    ag.sync_replicated_grads(comm, tp)
    opt.step()
    total = loss.detach().clone().view(1)
    comm.allreduce(total)
    ropt.zero_grad()
    rloss = ((ref(x) - t) ** 2).mean()
    rloss.backward()
    ropt.step()
    torch.cuda.synchronize()
    torch.testing.assert_close(total[0], rloss.detach(), rtol=1e-4, atol=1e-6)
n1 = 4 * H // p
torch.testing.assert_close(fc1.weight, ref[0].weight[me * n1:(me + 1) * n1], rtol=1e-4, atol=1e-5)
torch.testing.assert_close(fc2.weight, ref[2].weight[:, me * n1:(me + 1) * n1], rtol=1e-4, atol=1e-5)
torch.testing.assert_close(fc2.bias, ref[2].bias, rtol=1e-4, atol=1e-5)

# without sequence parallelism: replicated input, allreduced output
fc1r = ag.ColumnParallelLinear(comm, H, 4 * H, seed=11)
fc2r = ag.RowParallelLinear(comm, 4 * H, H, seed=12)
x = torch.randn(5, H, generator=g).cuda().requires_grad_(True)
xr = x.detach().clone().requires_grad_(True)
ref2 = nn.Sequential(nn.Linear(H, 4 * H), nn.GELU(), nn.Linear(4 * H, H)).cuda()
with torch.no_grad():
    ref2[0].weight.copy_(w1); ref2[0].bias.copy_(b1); ref2[2].weight.copy_(w2); ref2[2].bias.copy_(b2)
y = fc2r(nn.functional.gelu(fc1r(x)))
y.sum().backward()
yr = ref2(xr)
yr.sum().backward()
torch.cuda.synchronize()
torch.testing.assert_close(y, yr, rtol=1e-4, atol=1e-5)
torch.testing.assert_close(x.grad, xr.grad, rtol=1e-4, atol=1e-5)

# ---- 2. Ulysses and expert exchange: values, gradients, kernel list ------------------------------------------------
s, h, d = 6, 2 * p, 8
full = torch.randn(s * p, h, d, generator=g).cuda()
shard = full.chunk(p, dim=0)[me].contiguous().requires_grad_(True)
heads = ag.seq_to_head(comm, shard)
torch.cuda.synchronize()
assert torch.equal(heads, full[:, me * 2:(me + 1) * 2])
back = ag.head_to_seq(comm, heads * 2.0)
back.sum().backward()
torch.cuda.synchronize()
assert torch.equal(back, shard.detach() * 2) and torch.all(shard.grad == 2.0)

from torch.profiler import ProfilerActivity, profile  # noqa: E402
with profile(activities=[ProfilerActivity.CUDA]) as prof:
    hh = ulysses.seq_to_head(comm, shard.detach())
    bb = ulysses.head_to_seq(comm, hh)
    torch.cuda.synchronize()
def _dev_time(e):
    return getattr(e, "device_time_total", getattr(e, "cuda_time_total", 0))


names = [e.key for e in prof.key_averages() if _dev_time(e) > 0]
kernels = [k for k in names if "memcpy" not in k.lower() and "memset" not in k.lower()]
if kernels:  # (an empty list means the profiler could not attach in this process: nothing to judge)
    assert all("rows_kernel" in k for k in kernels), f"unexpected kernels around the Ulysses exchange: {names}"
    assert not any("copy" in k.lower() or "elementwise" in k.lower() for k in names), names
ulysses_kernels = kernels

toks = torch.randn(10 + me, 16, generator=torch.Generator().manual_seed(50 + me)).cuda()
dest = torch.randint(0, p, (toks.shape[0],), generator=torch.Generator().manual_seed(60 + me)).cuda()
got, state = expert.dispatch(comm, toks, dest)
want = []
for r in range(p):
    tr = torch.randn(10 + r, 16, generator=torch.Generator().manual_seed(50 + r)).cuda()
    dr = torch.randint(0, p, (tr.shape[0],), generator=torch.Generator().manual_seed(60 + r)).cuda()
    want.append(tr[torch.argsort(dr, stable=True)][torch.sort(dr, stable=True).values == me])
torch.cuda.synchronize()
assert torch.equal(got, torch.cat(want))
res = expert.combine(comm, got * 3.0, state)
torch.cuda.synchronize()
torch.testing.assert_close(res, toks * 3.0)

# ---- 3. pipeline: two stages, forward + backward over micro-batches ----------------------------------------------------
torch.manual_seed(21)
l0, l1 = nn.Linear(16, 32).cuda(), nn.Linear(32, 4).cuda()      # same weights on every rank (same seed)
mbs = [torch.randn(5, 16, generator=torch.Generator().manual_seed(70 + i)).cuda() for i in range(3)]
tgt = [torch.randn(5, 4, generator=torch.Generator().manual_seed(80 + i)).cuda() for i in range(3)]
r0, r1 = nn.Linear(16, 32).cuda(), nn.Linear(32, 4).cuda()
r0.load_state_dict(l0.state_dict()); r1.load_state_dict(l1.state_dict())
ref_losses = []
for x, t in zip(mbs, tgt):
    l = ((r1(torch.relu(r0(x))) - t) ** 2).mean()
    l.backward()
    ref_losses.append(l.detach())
if me < 2:
    stage = PipelineStage(comm, nn.Sequential(l0, nn.ReLU()) if me == 0 else l1, stages=[0, 1])
    out = stage.run(mbs, act_shape=(5, 32), loss_fn=lambda y, t: ((y - t) ** 2).mean(), targets=tgt)
    torch.cuda.synchronize()
    if me == 1:
        for a, b in zip(out, ref_losses):
            torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
        torch.testing.assert_close(l1.weight.grad, r1.weight.grad, rtol=1e-4, atol=1e-6)
    else:
        torch.testing.assert_close(l0.weight.grad, r0.weight.grad, rtol=1e-4, atol=1e-6)
comm.barrier()

# ---- 4. ring attention, transfers overlapped with the block computation ----------------------------------------------
sq, hh_, dd = 5, 2, 8
q, k, v = (torch.randn(sq * p, hh_, dd, generator=torch.Generator().manual_seed(90 + i)).cuda() for i in range(3))
scores = torch.einsum("qhd,khd->qhk", q, k) / math.sqrt(dd)
want = torch.einsum("qhk,khd->qhd", torch.softmax(scores, dim=-1), v)
out = context.ring_attention(comm, q.chunk(p)[me].contiguous(), k.chunk(p)[me].contiguous(), v.chunk(p)[me].contiguous())
torch.cuda.synchronize()
torch.testing.assert_close(out, want.chunk(p)[me], rtol=1e-4, atol=1e-4)

assert comm.status()["code"] == 0
print(f"rank {me} parallel components ok: rows={comm.stats()['rows']} window={comm.stats()['window']} ll={comm.stats()['ll']} "
      f"kernels around the Ulysses exchange: {sorted(set(k.split('(')[0].split('::')[-1] for k in ulysses_kernels))}")
comm.close()
al.finalize()
