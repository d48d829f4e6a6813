"""Recovery after a lost rank, on CPU ranks: the last rank leaves between steps; the others get an
error from the next collective, look which processes are still there, build a new communicator
from exactly those and carry on - here with a data-parallel model whose replicas must stay equal."""
import sys
import time
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
import aluminum_b200 as al  # noqa: E402

comm = al.HostComm()
p, me = comm.size, comm.rank
w = np.zeros(64, dtype=np.float32)          # the "model": every replica applies the averaged gradient


def step(c, k):
    g = np.full(64, float(c.rank + k), dtype=np.float32)
    c.allreduce(g)
    return w - 0.1 * g / c.size


w = step(comm, 0)
if me == p - 1:
    print(f"rank {me} leaves")
    sys.exit(0)                              # host-side fault: the process is gone, nothing in flight
time.sleep(0.2)
t0 = time.time()
try:
    step(comm, 1)
    print("ERROR: the collective returned although a rank is missing")
    sys.exit(2)
except al.AlError as e:
    t_seen = time.time()
    assert t_seen - t0 < 10, t_seen - t0
comm.abort("a rank was lost")
# A survivor that noticed first may already be past this point; nobody else has left.
alive = al.alive_ranks()
deadline = time.time() + 5
while len(alive) != p - 1 and time.time() < deadline:
    time.sleep(0.05)
    alive = al.alive_ranks()
assert alive == list(range(p - 1)), alive
assert not al.peer_alive(p - 1) and al.peer_alive(me)
new = al.HostComm.from_ranks(alive)
t_new = time.time()
assert new.size == p - 1 and new.rank == me
for k in range(1, 4):
    w = step(new, k)
# replicas agree after recovery
allw = np.empty(64 * new.size, dtype=np.float32)
new.allgather(w, allw)
assert all(np.array_equal(allw[:64], allw[64 * r:64 * (r + 1)]) for r in range(new.size))
expect = -0.1 * (sum(range(p)) / p) - 0.1 * sum((sum(range(p - 1)) + k * (p - 1)) / (p - 1) for k in range(1, 4))
assert np.allclose(w, expect, rtol=1e-5), (w[0], expect)
new.close()
print(f"rank {me}: recovered with {len(alive)} ranks (failure seen after {1e3 * (t_seen - t0):.1f} ms, "
      f"new communicator {1e3 * (t_new - t_seen):.1f} ms later)")
