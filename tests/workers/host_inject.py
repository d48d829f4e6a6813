"""Host-side fault injection, abort and counters on CPU ranks.

argv[1] selects the scenario:
  skip   - rank 1 never signals the communicator's second collective: it gets an error at once, the
           others time out cleanly; all of them can then build a new communicator that works
  delay  - rank 1 signals its second collective 300 ms late: everybody still gets the right answer
  abort  - rank 0 aborts while a non-blocking receive can never complete: the request ends with an
           error, later calls raise, counters show the failure
  jitter - every rank sleeps a random time before every publish: results stay exact
"""
import sys
import time
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
import aluminum_b200 as al  # noqa: E402

mode = sys.argv[1]
comm = al.HostComm()
p, me = comm.size, comm.rank


def expect_sum(x, scale=1.0):
    assert np.allclose(x, scale * p * (p + 1) / 2), x[:4]


if mode == "skip":
    x = np.full(64, me + 1, dtype=np.float32)
    comm.allreduce(x)
    expect_sum(x)
    y = np.full(64, me + 1, dtype=np.float32)
    t0 = time.time()
    try:
        comm.allreduce(y)
        print("ERROR: completed")
        sys.exit(2)
    except al.AlError as e:
        msg = str(e)
        if me == 1:
            assert "injected fault" in msg, msg
        else:  # told by the failing rank through the shared workspace, or (had that rank hung) by the time-out
            assert "reported a failure" in msg or "timed out" in msg, msg
        assert time.time() - t0 < 20
    assert comm.stats()["failures"] >= 1
    # Recovery path: a new communicator over the same ranks (the injection names operation 2 of a
    # communicator, so switch it off first).
    al.set_tuning("fault_kind", 0)
    comm.close()
    fresh = al.HostComm()
    z = np.full(64, me + 1, dtype=np.float32)
    fresh.allreduce(z)
    expect_sum(z)
    print(f"rank {me}: recovered")
elif mode == "delay":
    for it in range(3):
        x = np.full(1000, me + 1, dtype=np.float64)
        t0 = time.time()
        comm.allreduce(x)
        dt = time.time() - t0
        expect_sum(x)
        if it == 1:
            assert dt > 0.2, dt  # everybody waited for the late rank
    print(f"rank {me}: delayed op ok")
elif mode == "abort":
    x = np.zeros(8, dtype=np.float32)
    comm.barrier()
    if me == 0:
        req = comm.recv(x, 1, nonblocking=True)   # rank 1 never sends
        time.sleep(0.2)
        assert not req.test()
        comm.abort("test abort")
        try:
            req.wait()
            sys.exit(2)
        except al.AlError as e:
            assert "test abort" in str(e), str(e)
        try:
            comm.barrier()
            sys.exit(3)
        except al.AlError as e:
            assert "failed" in str(e), str(e)
        s = comm.stats()
        assert s["failures"] >= 1 and s["collectives"] == 1 and s["p2p_ops"] == 1, s
    else:
        time.sleep(1.0)   # stay alive: a rank that exits is noticed by its peers, which is not what is tested here
    print(f"rank {me}: abort ok")
elif mode == "jitter":
    rng = np.random.default_rng(1234)
    for it in range(40):
        n = int(rng.integers(1, 5000))
        x = np.full(n, me + 1, dtype=np.float32)
        comm.allreduce(x)
        expect_sum(x)
        a = np.full(n * p, me, dtype=np.int32)
        b = np.empty(n * p, dtype=np.int32)
        comm.alltoall(a, b)
        assert all((b[r * n:(r + 1) * n] == r).all() for r in range(p))
    s = comm.stats()
    assert s["collectives"] == 80 and s["bytes"] > 0, s
    print(f"rank {me}: jitter ok")
