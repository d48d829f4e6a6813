"""Device collectives on ONE GPU: all ranks of a communicator are emulated in one
process and every call is a single cooperative launch of the same kernels the
multi-GPU path uses (flag protocol included).  Results are compared with plain
PyTorch fp32 references of the same operation.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu

SIZES = [1, 7, 256, 1000, 4099, 65536, 300001]


@pytest.fixture(scope="module")
def al():
    import aluminum_b200 as al
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    al.init()
    yield al


@pytest.fixture(scope="module", params=[2, 4, 8])
def comm(al, request):
    c = al.DeviceComm(emulate=request.param)
    yield c
    c.close()


@pytest.fixture(scope="module")
def small_stage_comm(al):
    """Tiny staging halves force the multi-chunk paths (chunk loop + closing barrier)."""
    old = al.get_tuning("dev_stage_bytes")
    al.set_tuning("dev_stage_bytes", 65536)
    c = al.DeviceComm(emulate=4)
    al.set_tuning("dev_stage_bytes", old)
    yield c
    c.close()


def rand(n, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if dtype.is_floating_point:
        return (torch.randint(-16, 17, (n,), generator=g, device="cuda").float() / 8).to(dtype)
    if dtype == torch.uint8:
        return torch.randint(0, 7, (n,), generator=g, device="cuda").to(dtype)
    return torch.randint(-6, 7, (n,), generator=g, device="cuda").to(dtype)


def ref_reduce(xs, op):
    st = torch.stack([x.float() for x in xs])
    if op == "sum":
        return st.sum(0)
    if op == "avg":
        return st.mean(0)
    if op == "min":
        return st.min(0).values
    if op == "max":
        return st.max(0).values
    if op == "prod":
        return st.prod(0)
    raise ValueError(op)


@pytest.mark.parametrize("n", SIZES)
@pytest.mark.parametrize("algo", ["one_shot", "two_shot", "auto"])
def test_allreduce_f32(comm, n, algo):
    p = comm.size
    xs = [rand(n, torch.float32, 10 + r) for r in range(p)]
    want = ref_reduce(xs, "sum")
    outs = [torch.zeros(n, device="cuda") for _ in range(p)]
    comm.allreduce(xs, outs, algo=algo)
    torch.cuda.synchronize()
    for o in outs:
        torch.testing.assert_close(o, want, rtol=1e-5, atol=1e-5)
    # in place
    ys = [x.clone() for x in xs]
    comm.allreduce(ys, algo=algo)
    torch.cuda.synchronize()
    for y in ys:
        torch.testing.assert_close(y, want, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16, torch.float64, torch.int32, torch.int64, torch.uint8, torch.int8])
@pytest.mark.parametrize("op", ["sum", "min", "max", "prod", "avg"])
def test_allreduce_types_ops(comm, dtype, op):
    p, n = comm.size, 5003
    if op == "prod":
        xs = [(torch.randint(0, 2, (n,), device="cuda") * 2 - 1).to(dtype) if dtype != torch.uint8
              else torch.ones(n, device="cuda", dtype=dtype) for _ in range(p)]
    else:
        xs = [rand(n, dtype, 20 + r) for r in range(p)]
    if op == "avg" and not dtype.is_floating_point:
        want = torch.stack([x.to(torch.int64) for x in xs]).sum(0)
        want = torch.div(want, p, rounding_mode="trunc").float()
    else:
        want = ref_reduce(xs, op)
    ys = [x.clone() for x in xs]
    comm.allreduce(ys, op=op, algo="two_shot")
    zs = [x.clone() for x in xs]
    comm.allreduce(zs, op=op, algo="one_shot")
    torch.cuda.synchronize()
    tol = dict(rtol=2e-2, atol=2e-2) if dtype in (torch.bfloat16, torch.float16) else dict(rtol=1e-6, atol=1e-6)
    for y, z in zip(ys, zs):
        torch.testing.assert_close(y.float(), want.float(), **tol)
        torch.testing.assert_close(z.float(), want.float(), **tol)
        assert torch.equal(y, ys[0]), "ranks disagree bitwise"


def test_allreduce_bitwise_logical(comm):
    p, n = comm.size, 777
    xs = [torch.randint(0, 256, (n,), device="cuda", dtype=torch.int32) for _ in range(p)]
    for op, fn in (("bor", torch.bitwise_or), ("band", torch.bitwise_and), ("bxor", torch.bitwise_xor)):
        want = xs[0].clone()
        for x in xs[1:]:
            want = fn(want, x)
        ys = [x.clone() for x in xs]
        comm.allreduce(ys, op=op)
        torch.cuda.synchronize()
        assert all(torch.equal(y, want) for y in ys), op
    bs = [torch.randint(0, 2, (n,), device="cuda", dtype=torch.int32) * 5 for _ in range(p)]
    st = torch.stack([b != 0 for b in bs])
    for op, want in (("lor", st.any(0)), ("land", st.all(0)), ("lxor", (st.sum(0) % 2 == 1))):
        ys = [b.clone() for b in bs]
        comm.allreduce(ys, op=op)
        torch.cuda.synchronize()
        assert all(torch.equal(y != 0, want) for y in ys), op


def test_allreduce_fused_cast_scale(comm):
    """fp32 in -> bf16 on the wire -> fp32 out with a fused scale; bf16 in -> fp32 out."""
    p, n = comm.size, 40000
    xs = [rand(n, torch.float32, 30 + r) for r in range(p)]
    want = ref_reduce(xs, "sum") * 0.5
    outs = [torch.zeros(n, device="cuda") for _ in range(p)]
    comm.allreduce(xs, outs, scale=0.5, wire_dtype=torch.bfloat16, algo="two_shot")
    torch.cuda.synchronize()
    for o in outs:
        torch.testing.assert_close(o, want, rtol=2e-2, atol=2e-2)
    bs = [x.to(torch.bfloat16) for x in xs]
    outs = [torch.zeros(n, device="cuda") for _ in range(p)]
    comm.allreduce(bs, outs, algo="one_shot")
    torch.cuda.synchronize()
    for o in outs:
        torch.testing.assert_close(o, ref_reduce(bs, "sum"), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("n", [1, 513, 70001])
def test_reduce_and_bcast(comm, n):
    p = comm.size
    for root in (0, p - 1):
        xs = [rand(n, torch.float32, 40 + r) for r in range(p)]
        outs = [torch.full((n,), -1.0, device="cuda") for _ in range(p)]
        comm.reduce(xs, outs, root=root)
        torch.cuda.synchronize()
        torch.testing.assert_close(outs[root], ref_reduce(xs, "sum"))
        for r in range(p):
            if r != root:
                assert torch.all(outs[r] == -1.0)
        bufs = [x.clone() for x in xs]
        comm.bcast(bufs, root=root)
        torch.cuda.synchronize()
        for b in bufs:
            assert torch.equal(b, xs[root])


@pytest.mark.parametrize("n", [1, 33, 10007, 131072])
def test_reduce_scatter_allgather_alltoall(comm, n):
    p = comm.size
    xs = [rand(n * p, torch.float32, 50 + r) for r in range(p)]
    want = ref_reduce(xs, "sum")
    outs = [torch.zeros(n, device="cuda") for _ in range(p)]
    comm.reduce_scatter(xs, outs)
    torch.cuda.synchronize()
    for r in range(p):
        torch.testing.assert_close(outs[r], want[r * n:(r + 1) * n])
    # in place: result in the first n elements
    ys = [x.clone() for x in xs]
    comm.reduce_scatter(ys)
    torch.cuda.synchronize()
    for r in range(p):
        torch.testing.assert_close(ys[r][:n], want[r * n:(r + 1) * n])
    # allgather
    ss = [rand(n, torch.float32, 60 + r) for r in range(p)]
    full = torch.cat(ss)
    outs = [torch.zeros(n * p, device="cuda") for _ in range(p)]
    comm.allgather(ss, outs)
    torch.cuda.synchronize()
    assert all(torch.equal(o, full) for o in outs)
    ips = [torch.zeros(n * p, device="cuda") for _ in range(p)]
    for r in range(p):
        ips[r][r * n:(r + 1) * n] = ss[r]
    comm.allgather(ips)
    torch.cuda.synchronize()
    assert all(torch.equal(o, full) for o in ips)
    # alltoall
    outs = [torch.zeros(n * p, device="cuda") for _ in range(p)]
    comm.alltoall(xs, outs)
    ys = [x.clone() for x in xs]
    comm.alltoall(ys)
    torch.cuda.synchronize()
    for d in range(p):
        want_d = torch.cat([xs[r][d * n:(d + 1) * n] for r in range(p)])
        assert torch.equal(outs[d], want_d)
        assert torch.equal(ys[d], want_d)


def test_gather_scatter(comm):
    p, n = comm.size, 3001
    for root in (0, 1 % p):
        ss = [rand(n, torch.int32, 70 + r) for r in range(p)]
        outs = [torch.zeros(n * p, device="cuda", dtype=torch.int32) for _ in range(p)]
        comm.gather(ss, outs, root=root)
        torch.cuda.synchronize()
        assert torch.equal(outs[root], torch.cat(ss))
        src = [rand(n * p, torch.int32, 80 + r) for r in range(p)]
        dst = [torch.zeros(n, device="cuda", dtype=torch.int32) for _ in range(p)]
        comm.scatter(src, dst, root=root)
        torch.cuda.synchronize()
        for r in range(p):
            assert torch.equal(dst[r], src[root][r * n:(r + 1) * n])


def test_vector_collectives(comm):
    p, base = comm.size, 1000
    # alltoallv with pair-dependent counts
    cnt = lambda a, b: base + 37 * ((a + b) % 3)
    sc = [[cnt(r, d) for d in range(p)] for r in range(p)]
    sd = [[sum(row[:d]) for d in range(p)] for row in sc]
    xs = [rand(sum(sc[r]), torch.float32, 90 + r) for r in range(p)]
    outs = [torch.zeros(sum(sc[r]), device="cuda") for r in range(p)]
    comm.alltoallv(xs, sc, sd, outs, sc, sd)
    torch.cuda.synchronize()
    for d in range(p):
        want = torch.cat([xs[r][sd[r][d]:sd[r][d] + sc[r][d]] for r in range(p)])
        assert torch.equal(outs[d], want)
    # allgatherv / reduce_scatterv with rank-dependent counts
    counts = [base + 11 * r for r in range(p)]
    displs = [sum(counts[:r]) for r in range(p)]
    ss = [rand(counts[r], torch.float32, 100 + r) for r in range(p)]
    outs = [torch.zeros(sum(counts), device="cuda") for _ in range(p)]
    comm.allgatherv(ss, outs, [counts] * p, [displs] * p)
    torch.cuda.synchronize()
    assert all(torch.equal(o, torch.cat(ss)) for o in outs)
    xs = [rand(sum(counts), torch.float32, 110 + r) for r in range(p)]
    outs = [torch.zeros(counts[r], device="cuda") for r in range(p)]
    comm.reduce_scatterv(xs, outs, [counts] * p)
    torch.cuda.synchronize()
    want = ref_reduce(xs, "sum")
    for r in range(p):
        torch.testing.assert_close(outs[r], want[displs[r]:displs[r] + counts[r]])
    # gatherv / scatterv
    outs = [torch.zeros(sum(counts), device="cuda") for _ in range(p)]
    comm.gatherv(ss, outs, [counts] * p, [displs] * p, root=p - 1)
    src = [rand(sum(counts), torch.float32, 120 + r) for r in range(p)]
    dst = [torch.zeros(counts[r], device="cuda") for r in range(p)]
    comm.scatterv(src, dst, [counts] * p, [displs] * p, root=0)
    torch.cuda.synchronize()
    assert torch.equal(outs[p - 1], torch.cat(ss))
    for r in range(p):
        assert torch.equal(dst[r], src[0][displs[r]:displs[r] + counts[r]])


def test_multichunk_paths(small_stage_comm):
    """Messages many times larger than a staging half, back to back, mixed with small ones."""
    comm = small_stage_comm
    p, n = comm.size, 200003
    for it in range(3):
        xs = [rand(n, torch.float32, 130 + r + it) for r in range(p)]
        want = ref_reduce(xs, "sum")
        for algo in ("two_shot", "one_shot"):
            ys = [x.clone() for x in xs]
            comm.allreduce(ys, algo=algo)
            small = [torch.full((5,), float(r), device="cuda") for r in range(p)]
            comm.allreduce(small)
            torch.cuda.synchronize()
            for y in ys:
                torch.testing.assert_close(y, want, rtol=1e-5, atol=1e-5)
            assert all(torch.all(s == sum(range(p))) for s in small)
        a2a = [rand(30011 * p, torch.float32, 140 + r) for r in range(p)]
        outs = [torch.zeros_like(a2a[0]) for _ in range(p)]
        comm.alltoall(a2a, outs)
        torch.cuda.synchronize()
        for d in range(p):
            assert torch.equal(outs[d], torch.cat([a2a[r][d * 30011:(d + 1) * 30011] for r in range(p)]))


def test_pipelined_schedule(al):
    """Large uniform reduce_scatter / allgather / alltoall: publisher and consumer CTAs, many chunks."""
    old = al.get_tuning("pipeline_min_bytes")
    al.set_tuning("pipeline_min_bytes", 16384)
    try:
        for p in (2, 8):
            comm = al.DeviceComm(emulate=p)
            n = 1_500_007  # per-rank slice, not a multiple of anything
            for it in range(2):
                ss = [rand(n, torch.float32, 200 + r + it) for r in range(p)]
                outs = [torch.zeros(n * p, device="cuda") for _ in range(p)]
                comm.allgather(ss, outs)
                xs = [rand(n * p, torch.float32, 210 + r + it) for r in range(p)]
                rs = [torch.zeros(n, device="cuda") for _ in range(p)]
                comm.reduce_scatter(xs, rs)
                a2 = [torch.zeros(n * p, device="cuda") for _ in range(p)]
                comm.alltoall(xs, a2)
                small = [torch.full((3,), float(r), device="cuda") for r in range(p)]
                comm.allreduce(small)
                torch.cuda.synchronize()
                full, want = torch.cat(ss), ref_reduce(xs, "sum")
                for r in range(p):
                    assert torch.equal(outs[r], full)
                    torch.testing.assert_close(rs[r], want[r * n:(r + 1) * n])
                    assert torch.equal(a2[r], torch.cat([xs[q][r * n:(r + 1) * n] for q in range(p)]))
                    assert torch.all(small[r] == sum(range(p)))
            assert comm.status()["code"] == 0
            comm.close()
    finally:
        al.set_tuning("pipeline_min_bytes", old)


def test_barrier_nonblocking_and_stats(comm):
    p = comm.size
    comm.barrier()
    xs = [torch.full((1000,), float(r), device="cuda") for r in range(p)]
    req = comm.allreduce(xs, nonblocking=True)
    req.wait()
    torch.cuda.synchronize()
    assert req.test()
    assert all(torch.all(x == sum(range(p))) for x in xs)
    st = comm.stats()
    assert st["ops"] > 0 and st["kernels"] > 0 and st["timeouts"] == 0
    assert comm.status()["code"] == 0


def test_p2p_sendrecv_ring(comm):
    p, n = comm.size, 100003
    src = [rand(n, torch.float32, 150 + r) for r in range(p)]
    dst = [torch.zeros(n, device="cuda") for _ in range(p)]
    items = []
    for r in range(p):
        items.append((True, (r + 1) % p, src[r], r))
        items.append((False, (r - 1) % p, dst[r], r))
    comm.p2p(items)
    torch.cuda.synchronize()
    for r in range(p):
        assert torch.equal(dst[r], src[(r - 1) % p])
    assert comm.status()["code"] == 0


def test_p2p_in_place_exchange(comm):
    """The same buffer is sent and then overwritten by what arrives (in-place SendRecv)."""
    p, n = comm.size, 50001
    bufs = [rand(n, torch.float32, 170 + r) for r in range(p)]
    snap = [b.clone() for b in bufs]
    items = []
    for r in range(p):
        items.append((True, (r + 1) % p, bufs[r], r))
        items.append((False, (r - 1) % p, bufs[r], r))
    comm.p2p(items)
    torch.cuda.synchronize()
    for r in range(p):
        assert torch.equal(bufs[r], snap[(r - 1) % p])


def test_unaligned_buffers(comm):
    p, n = comm.size, 1001
    bases = [rand(n + 3, torch.float32, 160 + r) for r in range(p)]
    xs = [b[1:1 + n] for b in bases]           # 4-byte aligned only
    outs_b = [torch.zeros(n + 3, device="cuda") for _ in range(p)]
    outs = [o[3:3 + n] for o in outs_b]
    comm.allreduce(xs, outs)
    torch.cuda.synchronize()
    want = ref_reduce(xs, "sum")
    for o in outs:
        torch.testing.assert_close(o, want)
