"""World-size-2 CPU plumbing check: fp32 allreduce of 1,048,576 values drawn U(-1,1) from seed 0
per rank (blocking, then non-blocking + wait) and an int32 alltoall of 4096 values per peer holding
rank*1e6 + index, each compared with a serial computation."""
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
import aluminum_b200 as al  # noqa: E402

comm = al.HostComm()
p, me = comm.size, comm.rank
n = 1 << 20


def data(rank):
    return np.random.default_rng(0 + 1000 * rank).uniform(-1, 1, n).astype(np.float32)


want = np.zeros(n, dtype=np.float32)
for r in range(p):  # serial reduction in rank order
    want = want + data(r) if r else data(0).copy()
x = data(me)
out = np.zeros_like(x)
comm.allreduce(x, out)
assert np.allclose(out, want, rtol=1e-6, atol=1e-6), "blocking allreduce"
assert np.array_equal(x, data(me)), "send buffer must stay untouched"
y = data(me)
req = comm.allreduce(y, nonblocking=True)
req.wait()
assert req.test()
assert np.allclose(y, want, rtol=1e-6, atol=1e-6), "non-blocking allreduce"
per = 4096
send = (me * 1_000_000 + np.arange(per * p)).astype(np.int32)
recv = np.zeros_like(send)
comm.alltoall(send, recv)
for r in range(p):
    exp = r * 1_000_000 + np.arange(me * per, (me + 1) * per)
    assert np.array_equal(recv[r * per:(r + 1) * per], exp), "alltoall"
# split: singleton groups still work
sub = comm.split(me, 0)
z = np.ones(5, dtype=np.float64)
sub.allreduce(z)
assert sub.size == 1 and np.all(z == 1)
sub.close()
comm.barrier()
comm.close()
al.finalize()
print(f"rank {me} ok")
