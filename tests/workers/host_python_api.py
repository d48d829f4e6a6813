"""Python HostComm: vector collectives, rooted operations, point-to-point and requests on CPU ranks."""
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
import aluminum_b200 as al  # noqa: E402

c = al.HostComm()
p, me = c.size, c.rank
# allgatherv with rank-dependent counts
counts = [3 + r for r in range(p)]
displs = [sum(counts[:r]) for r in range(p)]
mine = np.full(counts[me], me, dtype=np.int64)
out = np.zeros(sum(counts), dtype=np.int64)
c.allgatherv(mine, out, counts, displs)
assert np.array_equal(out, np.concatenate([np.full(counts[r], r) for r in range(p)]))
# reduce_scatterv
full = np.arange(sum(counts), dtype=np.float64) + me
got = np.zeros(counts[me])
c.reduce_scatterv(full, got, counts)
want = sum(np.arange(sum(counts), dtype=np.float64) + r for r in range(p))[displs[me]:displs[me] + counts[me]]
assert np.allclose(got, want)
# bcast / gather / scatter / reduce with a non-zero root
root = p - 1
b = np.full(7, me, dtype=np.float32)
c.bcast(b, root=root)
assert np.all(b == root)
g = np.zeros(4 * p, dtype=np.int32)
c.gather(np.full(4, me, dtype=np.int32), g, root=root)
if me == root:
    assert np.array_equal(g, np.repeat(np.arange(p), 4))
s = np.zeros(4, dtype=np.int32)
c.scatter(np.arange(4 * p, dtype=np.int32), s, root=root)
assert np.array_equal(s, np.arange(4 * me, 4 * me + 4))
r = np.ones(5, dtype=np.float32) * (me + 1)
ro = np.zeros(5, dtype=np.float32)
c.reduce(r, ro, op="max", root=root)
if me == root:
    assert np.all(ro == p)
# ring sendrecv, non-blocking
snd = np.full(1000, me, dtype=np.float32)
rcv = np.zeros(1000, dtype=np.float32)
req = c.sendrecv(snd, (me + 1) % p, rcv, (me - 1) % p, nonblocking=True)
while not req.test():
    pass
assert np.all(rcv == (me - 1) % p)
# avg and logical operators
a = np.full(9, float(me), dtype=np.float32)
c.allreduce(a, op="avg")
assert np.allclose(a, (p - 1) / 2)
l = np.array([me % 2, 1, 0], dtype=np.int32)
c.allreduce(l, op="land")
assert list(l) == [1 if p == 1 and me % 2 else 0, 1, 0] or list(l)[1:] == [1, 0]
# trace snapshot through the C API
print(f"rank {me} ok")
c.close()
al.finalize()
