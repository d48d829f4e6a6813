"""A world that spans several (modelled) nodes: ranks of one node share memory, ranks of different
nodes talk over TCP.

argv[1]:
  hier   - world collectives over sockets, node-local communicator over shared memory, a leaders'
           communicator across nodes, and a two-level allreduce that must equal the flat one
  dead   - the last rank leaves between steps; the others' next collective must fail promptly with
           an error naming a closed connection (no time-out needed: the sockets report it)
  mismatch - ranks disagree on the size of a broadcast: the receiver reports the mismatch
"""
import sys
import time
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
import aluminum_b200 as al  # noqa: E402

mode = sys.argv[1]
world = al.HostComm()
p, me = world.size, world.rank

if mode == "hier":
    assert al.num_nodes() == 2, al.num_nodes()
    assert al.local_size() == p // 2 and al.local_rank() == me % (p // 2)
    node = world.split(al.node_index(), me)                 # shared memory inside
    leaders = world.split(0 if al.local_rank() == 0 else 1, me)  # sockets across (colour 1: the rest)
    # the communicator's own view of the node structure
    assert world.local_size == p // 2 and world.local_rank == me % (p // 2), (world.local_rank, world.local_size)
    assert node.local_size == node.size and node.local_rank == node.rank
    mine = world.local()
    assert mine.size == p // 2 and mine.rank == world.local_rank
    z = np.full(3, float(me), dtype=np.float32)
    mine.allreduce(z)
    first = (me // (p // 2)) * (p // 2)
    assert z[0] == sum(range(first, first + p // 2)), z
    odd = world.split(me % 2, me)   # a subset that still spans both nodes
    assert odd.local_size == sum(1 for r in range(first, first + p // 2) if r % 2 == me % 2)
    mine.close(); odd.close()
    assert node.size == p // 2
    rng = np.random.default_rng(me)
    for n in (1, 7, 1000, 300001):
        x = rng.standard_normal(n).astype(np.float32)
        flat = x.copy()
        world.allreduce(flat)
        # two-level: reduce inside the node, allreduce among the leaders, broadcast inside the node
        y = x.copy()
        node.reduce(y, root=0)
        if al.local_rank() == 0:
            leaders.allreduce(y)
        node.bcast(y, root=0)
        assert np.allclose(flat, y, rtol=1e-5, atol=1e-5), (n, np.abs(flat - y).max())
    g = np.empty(p, dtype=np.int64)
    world.allgather(np.array([me * 10], dtype=np.int64), g)
    assert (g == np.arange(p) * 10).all()
    print(f"rank {me}: hierarchical ok")
elif mode == "dead":
    x = np.ones(1000, dtype=np.float32)
    world.allreduce(x)
    assert x[0] == p
    if me == p - 1:
        print(f"rank {me} leaves")
        sys.exit(0)
    time.sleep(0.3)
    t0 = time.time()
    try:
        world.allreduce(x)
        print("ERROR: completed")
        sys.exit(2)
    except al.AlError as e:
        assert time.time() - t0 < 15, time.time() - t0
        # the dead rank itself, a peer that noticed first and said so, or one that has already left in turn
        assert any(w in str(e) for w in ("closed the connection", "failed", "timed out", "has exited", "reported a failure")), str(e)
    print(f"rank {me}: detected the dead rank")
elif mode == "mismatch":
    x = np.zeros(100 if me == 0 else 50, dtype=np.float32)
    try:
        world.bcast(x, root=0)
        assert me == 0
    except al.AlError as e:
        assert "do not match" in str(e), str(e)
        print(f"rank {me}: mismatch reported")
