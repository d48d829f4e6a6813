"""Data paths of the device backend over REAL ranks (one process and one GPU each; run under alrun):

* low-latency packets, staged, pipelined and window operations against a locally computed expectation
  (every rank can compute every rank's input from the seed);
* window operations on symmetric tensors (multimem.st / multimem.ld_reduce where the GPUs have NVLS) and on
  ordinary torch tensors registered through CUDA IPC, at equal and at different offsets;
* the zero-copy NVLS allreduce on a sub-range of a symmetric tensor whose length is not a multiple of 16 bytes
  (must not touch the elements behind it);
* reduce_scatter of private buffers reduced by the switch (staged NVLS; more than two ranks): odd lengths,
  several chunks, unaligned and in-place outputs, avg and max, against the locally computed expectation;
* large messages: pipelined staged NVLS allreduce (private, 160 MiB), zero-copy allreduce (symmetric),
  pipelined reduce_scatter / allgather / alltoall (64 MiB per rank) - only with AL_TEST_LARGE=1;
* a rank that passes a private buffer where the others pass a symmetric one: every rank must get a clear
  "different paths" error at once, not a time-out, and a new communicator must work afterwards;
* one-sided Get next to Put; a communicator over a subset of the ranks (from_ranks).
"""
import os
import sys
import time
from pathlib import Path

import torch

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
import aluminum_b200 as al  # noqa: E402

local = int(os.environ.get("AL_LOCAL_RANK", os.environ.get("LOCAL_RANK", "0")))
torch.cuda.set_device(local)
al.init()
comm = al.DeviceComm()
p, me = comm.size, comm.rank
comm.set_timeout_ms(8000)
LARGE = os.environ.get("AL_TEST_LARGE") == "1"


def data(rank, n, seed, dtype=torch.float32):
    g = torch.Generator(device="cuda").manual_seed(1000 * seed + rank)
    return (torch.randint(-16, 17, (n,), generator=g, device="cuda").float() / 8).to(dtype)


def check(name, got, want, exact=True):
    torch.cuda.synchronize()
    st = comm.status()
    assert st["code"] == 0, f"{name}: status {st}"
    if exact:
        assert torch.equal(got, want), f"rank {me}: {name} differs"
    else:
        torch.testing.assert_close(got.double(), want.double(), rtol=2e-2, atol=2e-2, msg=f"rank {me}: {name}")


def all_inputs(n, seed, dtype=torch.float32):
    return [data(r, n, seed, dtype) for r in range(p)]


# ---- 1. packets, staged, window on private / symmetric / registered buffers ----------------------------
seed = 0
for n in (1, 33, 2048, 70_000, 1_000_003):  # floats per rank slice
    seed += 1
    xs = all_inputs(n, seed)
    out = torch.empty(n, device="cuda")
    comm.allreduce(xs[me], out)
    check(f"allreduce {n}", out, torch.stack(xs).sum(0), exact=False)
    big = all_inputs(n * p, seed + 100)
    rs = torch.empty(n, device="cuda")
    comm.reduce_scatter(big[me], rs)
    check(f"reduce_scatter {n}", rs, torch.stack(big).sum(0)[me * n:(me + 1) * n], exact=False)
    ag = torch.empty(n * p, device="cuda")
    comm.allgather(xs[me], ag)
    check(f"allgather {n}", ag, torch.cat(xs))
    a2 = torch.empty(n * p, device="cuda")
    comm.alltoall(big[me], a2)
    check(f"alltoall {n}", a2, torch.cat([big[q][me * n:(me + 1) * n] for q in range(p)]))

ll_ops = comm.stats()["ll"]
assert ll_ops >= 8, comm.stats()

for n in (4, 1000, 262_144):
    seed += 1
    xs = all_inputs(n, seed)
    big = all_inputs(n * p, seed + 100)
    sym_out = comm.symm_empty((n * p + 4,), torch.float32)     # same offset everywhere: multimem where available
    sym_in = comm.symm_empty((n * p,), torch.float32)
    reg_out = torch.full((n * p + 64,), -1.0, device="cuda")  # ordinary tensors, registered; used at rank-dependent offsets
    reg_in = torch.empty(n * p + 64, device="cuda")
    w_out, w_in = comm.register(reg_out), comm.register(reg_in)
    assert w_out >= 0 and w_in >= 0, "CUDA IPC registration of torch tensors failed"
    before = comm.stats()["window"]
    # allgather / alltoall / bcast into symmetric and into registered receive buffers
    for name, recv in (("symm", sym_out[:n * p]), ("registered", reg_out[4 * me:4 * me + n * p])):
        comm.allgather(xs[me], recv, algo="window")
        check(f"window allgather {name} {n}", recv, torch.cat(xs))
        comm.alltoall(big[me], recv, algo="window")
        check(f"window alltoall {name} {n}", recv, torch.cat([big[q][me * n:(me + 1) * n] for q in range(p)]))
        b = recv[:n]
        root = (n + 1) % p
        b.copy_(xs[me])
        comm.bcast(b, root=root, algo="window")
        check(f"window bcast {name} {n}", b, xs[root])
    assert torch.all(sym_out[n * p:] == 0) and torch.all(reg_out[4 * me + n * p:] == -1.0), "written past the end"
    # reduce_scatter out of symmetric and out of registered send buffers
    for name, send in (("symm", sym_in), ("registered", reg_in[4 * me:4 * me + n * p])):
        send.copy_(big[me])
        comm.barrier()
        for op in ("sum", "max", "avg"):
            rs = torch.zeros(n, device="cuda")
            comm.reduce_scatter(send, rs, op=op, algo="window")
            st = torch.stack(big)
            want = {"sum": st.sum(0), "max": st.max(0).values, "avg": st.mean(0)}[op][me * n:(me + 1) * n]
            check(f"window reduce_scatter {name} {op} {n}", rs, want, exact=False)
    assert comm.stats()["window"] == before + 12, comm.stats()
    comm.unregister(reg_out)
    comm.unregister(reg_in)
    comm.symm_free(sym_out)
    comm.symm_free(sym_in)

# bf16 reduce_scatter through the switch (multimem.ld_reduce with fp32 accumulation) and through peer loads
n = 65_536
bx = [data(r, n * p, 77, torch.bfloat16) for r in range(p)]
sym = comm.symm_empty((n * p,), torch.bfloat16)
sym.copy_(bx[me])
comm.barrier()
for multimem in (1, 0):
    al.set_tuning("window_multimem", multimem)
    rs = torch.zeros(n, dtype=torch.bfloat16, device="cuda")
    comm.reduce_scatter(sym, rs, algo="window")
    check(f"window reduce_scatter bf16 multimem={multimem}", rs,
          torch.stack([b.float() for b in bx]).sum(0)[me * n:(me + 1) * n], exact=False)
al.set_tuning("window_multimem", 1)
comm.symm_free(sym)

# ---- 2. zero-copy NVLS allreduce on a sub-range that does not end on a 16-byte boundary ---------------------
if comm.has_multicast:
    for count in (5, 1023, 4097):
        t = comm.symm_empty((8192,), torch.float32)
        t.fill_(float(me + 1))
        comm.barrier()
        torch.cuda.synchronize()
        comm.allreduce(t[:count], algo="nvls")
        torch.cuda.synchronize()
        assert torch.all(t[:count] == p * (p + 1) / 2), f"rank {me}: nvls allreduce of {count} wrong"
        assert torch.all(t[count:] == float(me + 1)), f"rank {me}: nvls allreduce of {count} touched the elements behind it"
        comm.symm_free(t)

# ---- 2b. staged NVLS reduce_scatter of private buffers (the switch reduces) ----------------------------------
if comm.has_multicast and p > 2:
    before = comm.stats()["rs_nvls"]
    calls = 0
    for dt, ops in ((torch.float32, ("sum", "avg")), (torch.bfloat16, ("sum", "max"))):
        for n in (5, 1000, 262_147, 3_000_001):
            src = [data(r, n * p, 40 + n % 7, dt) for r in range(p)]
            st = torch.stack([t.float() for t in src])
            for op in ops:
                want = {"sum": st.sum(0), "avg": st.mean(0), "max": st.max(0).values}[op][me * n:(me + 1) * n]
                out = torch.full((n + 3,), -7.0, dtype=dt, device="cuda")
                comm.reduce_scatter(src[me], out[1:1 + n], op=op, algo="nvls")       # output one element into its allocation
                check(f"nvls reduce_scatter {dt} {op} {n}", out[1:1 + n].float(), want, exact=False)
                assert out[0] == -7.0 and torch.all(out[1 + n:] == -7.0), "nvls reduce_scatter wrote outside its output"
                calls += 1
            buf = src[me].clone()
            comm.reduce_scatter(buf, op="sum", algo="nvls")                            # in place: result at the start
            check(f"nvls reduce_scatter in place {dt} {n}", buf[:n].float(), st.sum(0)[me * n:(me + 1) * n], exact=False)
            calls += 1
    assert comm.stats()["rs_nvls"] == before + calls, comm.stats()

# ---- 3. large messages ----------------------------------------------------------------------------------------
if LARGE:
    n = 40 * 1024 * 1024  # 160 MiB of fp32
    x = torch.full((n,), float(me + 1), device="cuda")
    x[::1000] = float(me)
    comm.allreduce(x)                                   # private: staged NVLS, pipelined
    torch.cuda.synchronize()
    assert torch.all(x[1::1000] == p * (p + 1) / 2) and torch.all(x[::1000] == p * (p - 1) / 2), "large private allreduce"
    s = comm.symm_empty((n,), torch.float32)
    s.fill_(float(me + 1))
    comm.barrier()
    comm.allreduce(s)                                   # symmetric: zero-copy
    torch.cuda.synchronize()
    assert torch.all(s == p * (p + 1) / 2), "large symmetric allreduce"
    comm.symm_free(s)
    del x
    for dt in (torch.float32, torch.bfloat16):
        n = (64 * 1024 * 1024) // torch.empty((), dtype=dt).element_size()   # 64 MiB per rank slice
        src = torch.arange(n * p, device="cuda").remainder(241).to(dt) + me   # exact in bf16 (small integers)
        rs = torch.empty(n, dtype=dt, device="cuda")
        comm.reduce_scatter(src, rs)
        base = torch.arange(me * n, (me + 1) * n, device="cuda").remainder(241).to(torch.float32)
        check(f"large reduce_scatter {dt}", rs.float(), base * p + p * (p - 1) / 2, exact=False)
        del rs, base
        ag = torch.empty(n * p, dtype=dt, device="cuda")
        comm.allgather(src[:n], ag)
        torch.cuda.synchronize()
        for q in range(p):
            assert torch.equal(ag[q * n:(q + 1) * n], torch.arange(n, device="cuda").remainder(241).to(dt) + q), "large allgather"
        comm.alltoall(src, ag)
        torch.cuda.synchronize()
        for q in range(p):
            assert torch.equal(ag[q * n:(q + 1) * n], torch.arange(me * n, (me + 1) * n, device="cuda").remainder(241).to(dt) + q), "large alltoall"
        del ag, src
    torch.cuda.empty_cache()

# ---- 4. one-sided Get next to Put; a communicator over a subset ---------------------------------------------
right, left = (me + 1) % p, (me + p - 1) % p
mine = torch.full((4096,), float(me), device="cuda")
got = torch.zeros(4096, device="cuda")
if me % 2 == 0:
    r_right = comm.attach(mine, right); r_left = comm.attach(mine, left)
else:
    r_left = comm.attach(mine, left); r_right = comm.attach(mine, right)
comm.barrier()                     # every rank's `mine` is filled before anybody reads it
comm.get(got, right, r_right)
torch.cuda.synchronize()
assert torch.all(got == float(right)), "get"
comm.barrier()
torch.cuda.synchronize()
comm.detach(r_right, right)
comm.detach(r_left, left)

if p >= 3:
    members = list(range(0, p, 2))
    if me in members:
        sub = al.DeviceComm.from_ranks(members)
        t = torch.full((1000,), float(me), device="cuda")
        sub.allreduce(t)
        torch.cuda.synchronize()
        assert torch.all(t == float(sum(members))), "from_ranks allreduce"
        sub.close()
comm.barrier()
torch.cuda.synchronize()

# ---- 5. ranks that disagree about registration get a clear error, not a time-out ------------------------------
n = 600_000                                      # 2.4 MB per pair of ranks: beyond the packet path on any number of ranks
al.set_tuning("window_min_bytes", 256 << 10)   # left to itself the library keeps messages of this size on the staged path
bad = al.DeviceComm()
bad.set_timeout_ms(15000)
sym = bad.symm_empty((n * p,), torch.float32)
priv = torch.empty(n * p, device="cuda")
t0 = time.time()
raised = ""
try:
    bad.allgather(data(me, n, 5), priv if me == p - 1 else sym)   # the last rank passes a private buffer
    torch.cuda.synchronize()
    bad.barrier()
    torch.cuda.synchronize()
except al.AlError as e:
    raised = str(e)
dt = time.time() - t0
assert "different paths" in raised, f"rank {me}: expected a path-mismatch error, got '{raised}'"
assert dt < 5.0, f"rank {me}: the mismatch took {dt:.1f} s to surface"
assert bad.status()["code"] == 3
fresh = al.DeviceComm()
t = torch.ones(10, device="cuda")
fresh.allreduce(t)
torch.cuda.synchronize()
assert torch.all(t == p)
fresh.close()

print(f"rank {me} device paths ok: ll={comm.stats()['ll']} window={comm.stats()['window']} "
      f"multicast={int(comm.has_multicast)} large={int(LARGE)}")
comm.close()
al.finalize()
