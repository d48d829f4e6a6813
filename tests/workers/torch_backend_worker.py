"""torch.distributed on the "aluminum" backend: every collective against a locally computed
expectation, a sub-group, and DistributedDataParallel against full-batch training.
CPU tensors by default; `cuda` as first argument puts every tensor on this rank's GPU."""
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import aluminum_b200 as al  # noqa: E402
import aluminum_b200.torch_backend  # noqa: E402,F401  (registers the backend)

al.init()
me, p = al.world_rank(), al.world_size()
dev = torch.device("cpu")
if len(sys.argv) > 1 and sys.argv[1] == "cuda":
    torch.cuda.set_device(al.local_rank() % torch.cuda.device_count())
    dev = torch.device("cuda", torch.cuda.current_device())
E = lambda *shape, **kw: torch.empty(*shape, device=dev, **kw)  # noqa: E731
os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
os.environ.setdefault("MASTER_PORT", os.environ.get("AL_TEST_PORT", "29611"))
dist.init_process_group("aluminum", rank=me, world_size=p)
assert dist.get_backend() == "aluminum" and dist.get_rank() == me and dist.get_world_size() == p


def vec(r, n=1000, dtype=torch.float32):
    return (torch.arange(n, dtype=torch.float32, device=dev) * 0.25 + r).to(dtype)


# allreduce: sum / max / avg, a non-contiguous tensor, int64
x = vec(me)
dist.all_reduce(x)
assert torch.allclose(x, sum(vec(r) for r in range(p)))
x = vec(me)
dist.all_reduce(x, op=dist.ReduceOp.MAX)
assert torch.equal(x, vec(p - 1))
x = vec(me)
dist.all_reduce(x, op=dist.ReduceOp.AVG)
assert torch.allclose(x, sum(vec(r) for r in range(p)) / p)
m = torch.full((6, 8), float(me), device=dev)[:, ::2]
dist.all_reduce(m)
assert not m.is_contiguous() and torch.all(m == sum(range(p)))
k = torch.tensor([me, 2 * me, 7], dtype=torch.int64, device=dev)
dist.all_reduce(k)
assert k.tolist() == [sum(range(p)), 2 * sum(range(p)), 7 * p]

# broadcast / reduce
b = vec(me)
dist.broadcast(b, src=p - 1)
assert torch.equal(b, vec(p - 1))
r_ = vec(me)
dist.reduce(r_, dst=0)
assert torch.allclose(r_, sum(vec(r) for r in range(p))) if me == 0 else torch.equal(r_, vec(me))

# allgather (list and tensor forms), reduce_scatter (list and tensor forms)
outs = [E(1000) for _ in range(p)]
dist.all_gather(outs, vec(me))
assert all(torch.equal(outs[r], vec(r)) for r in range(p))
flat = E(p * 1000)
dist.all_gather_into_tensor(flat, vec(me))
assert torch.equal(flat, torch.cat([vec(r) for r in range(p)]))
full = torch.cat([vec(me + d, 10) for d in range(p)])
rs = E(10)
dist.reduce_scatter_tensor(rs, full)
assert torch.allclose(rs, sum(vec(r + me, 10) for r in range(p)))
rs2 = E(10)
dist.reduce_scatter(rs2, [vec(me + d, 10) for d in range(p)])
assert torch.allclose(rs2, rs)

# all_to_all (single, equal and unequal splits; list form)
a = torch.arange(p * 3, dtype=torch.float32, device=dev) + 100 * me
o = E(p * 3)
dist.all_to_all_single(o, a)
assert torch.equal(o, torch.cat([torch.arange(me * 3, me * 3 + 3, dtype=torch.float32, device=dev) + 100 * r for r in range(p)]))
in_split = [d + 1 for d in range(p)]            # rank r sends d+1 rows to rank d
out_split = [me + 1] * p                        # so it receives me+1 rows from everyone
a = torch.cat([torch.full((d + 1, 2), float(10 * me + d), device=dev) for d in range(p)])
o = E(sum(out_split), 2)
dist.all_to_all_single(o, a, out_split, in_split)
assert torch.equal(o, torch.cat([torch.full((me + 1, 2), float(10 * r + me), device=dev) for r in range(p)]))
outs = [E(2) for _ in range(p)]
dist.all_to_all(outs, [torch.full((2,), float(me * p + d), device=dev) for d in range(p)])
assert all(torch.all(outs[r] == r * p + me) for r in range(p))

# gather / scatter / barrier / send-recv
g = [E(5) for _ in range(p)] if me == 0 else None
dist.gather(vec(me, 5), g, dst=0)
assert me != 0 or all(torch.equal(g[r], vec(r, 5)) for r in range(p))
s = E(5)
dist.scatter(s, [vec(r + 50, 5) for r in range(p)] if me == 1 % p else None, src=1 % p)
assert torch.equal(s, vec(me + 50, 5))
dist.barrier()
if p >= 2:
    if me == 0:
        dist.send(vec(7, 33), dst=1)
    elif me == 1:
        got = E(33)
        dist.recv(got, src=0)
        assert torch.equal(got, vec(7, 33))

# a sub-group of the even ranks: only its members build a communicator
evens = list(range(0, p, 2))
sub = dist.new_group(evens)
if me in evens:
    y = torch.full((4,), float(me), device=dev)
    dist.all_reduce(y, group=sub)
    assert torch.all(y == sum(evens))

# DistributedDataParallel: averaged gradients equal the full-batch gradients
torch.manual_seed(0)
model = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Tanh(), torch.nn.Linear(16, 3)).to(dev)
ref = torch.nn.Sequential(torch.nn.Linear(8, 16), torch.nn.Tanh(), torch.nn.Linear(16, 3)).to(dev)
ref.load_state_dict(model.state_dict())
ddp = torch.nn.parallel.DistributedDataParallel(model)
data = torch.randn(4 * p, 8).to(dev)
target = torch.randn(4 * p, 3).to(dev)
opt = torch.optim.SGD(ddp.parameters(), lr=0.1)
ropt = torch.optim.SGD(ref.parameters(), lr=0.1)
for _ in range(3):
    opt.zero_grad()
    torch.nn.functional.mse_loss(ddp(data[4 * me:4 * me + 4]), target[4 * me:4 * me + 4]).backward()
    opt.step()
    ropt.zero_grad()
    torch.nn.functional.mse_loss(ref(data), target).backward()
    ropt.step()
for a_, b_ in zip(model.parameters(), ref.parameters()):
    assert torch.allclose(a_, b_, rtol=1e-5, atol=1e-6), (a_ - b_).abs().max()

if dev.type == "cuda":
    torch.cuda.synchronize()
dist.destroy_process_group()
print(f"rank {me}: torch backend ok")
