"""Failure detection on CPU ranks: rank 1 never joins the second collective (it exits between
steps, with nothing in flight); rank 0 must get an exception promptly instead of hanging - the
closed control connection tells it long before the wait limit (60 s here) - and the communicator
must then refuse further work."""
import sys
import time
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
import aluminum_b200 as al  # noqa: E402

comm = al.HostComm()
x = np.ones(16, dtype=np.float32)
comm.allreduce(x)          # both ranks take part
assert x[0] == comm.size
if comm.rank == 1:
    print("rank 1 leaves")
    sys.exit(0)            # host-side fault: the rank is simply gone
t0 = time.time()
try:
    comm.allreduce(x)
    print("ERROR: the collective returned although a rank is missing")
    sys.exit(2)
except al.AlError as e:
    dt = time.time() - t0
    assert "has exited" in str(e), str(e)
    assert dt < 5, dt
try:
    comm.allreduce(x)
    sys.exit(3)
except al.AlError as e:
    assert "failed" in str(e)
print("rank 0 detected the failure")
