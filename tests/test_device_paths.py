"""The two data paths beside staging, on ONE GPU with emulated ranks:

* low-latency packets (kernels/ll.cu): small uniform allreduce / reduce_scatter / allgather / alltoall;
* window kernels (kernels/window.cu): reduce_scatter / allgather / alltoall / bcast straight on registered
  buffers (``comm.register`` for ordinary tensors, ``comm.symm_empty`` tensors are registered already).

Every result is compared with a plain PyTorch reference of the same operation; the communicator's counters
prove which path ran.  Real peers (NVLink stores, multimem) are covered by tests/workers/device_paths_worker.py.
"""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def al():
    import aluminum_b200 as al
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    al.init()
    old = al.get_tuning("ll_max_bytes")
    al.set_tuning("ll_max_bytes", 1 << 20)  # the largest message the packet slots hold
    yield al
    al.set_tuning("ll_max_bytes", old)


def rand(n, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    if dtype.is_floating_point:
        return (torch.randint(-16, 17, (n,), generator=g, device="cuda").float() / 8).to(dtype)
    return torch.randint(-6, 7, (n,), generator=g, device="cuda").to(dtype)


def ref_reduce(xs, op):
    st = torch.stack([x.double() for x in xs])
    return {"sum": st.sum(0), "avg": st.mean(0), "min": st.min(0).values, "max": st.max(0).values,
            "prod": st.prod(0)}[op]


# ------------------------------------------------------------------------------------------------------
# low-latency packets
# ------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("p", [2, 3, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float64, torch.int32, torch.int16])
def test_ll_allreduce_and_reduce_scatter(al, p, dtype):
    comm = al.DeviceComm(emulate=p)
    comm.set_timeout_ms(2000)
    esz = torch.empty((), dtype=dtype).element_size()
    sizes = [1, 3, 4, 5, 33, 1000, 262144 // esz, (1 << 20) // esz]
    before = comm.stats()["ll"]
    calls = 0
    for it, n in enumerate(sizes):
        for op in (("sum", "max") if dtype != torch.float64 else ("sum", "prod")):
            xs = [rand(n, dtype, 10 * it + r) for r in range(p)]
            want = ref_reduce(xs, op)
            outs = [torch.zeros(n + 2, dtype=dtype, device="cuda") for _ in range(p)]
            comm.allreduce(xs, [o[:n] for o in outs], op=op)                  # out of place
            ys = [x.clone() for x in xs]
            comm.allreduce(ys, op=op)                                         # in place, right after
            calls += 2
            torch.cuda.synchronize()
            for r in range(p):
                torch.testing.assert_close(outs[r][:n].double(), want, rtol=2e-2, atol=2e-2)
                assert torch.all(outs[r][n:] == 0)                              # nothing written past the end
                assert torch.equal(ys[r], outs[r][:n])                          # both forms, and every rank, bit-identical
            assert all(torch.equal(outs[0], o) for o in outs)
        # reduce_scatter: n elements per rank
        if n * esz <= (1 << 20):
            xs = [rand(n * p, dtype, 50 + 10 * it + r) for r in range(p)]
            want = ref_reduce(xs, "sum")
            outs = [torch.zeros(n, dtype=dtype, device="cuda") for _ in range(p)]
            comm.reduce_scatter(xs, outs)
            ys = [x.clone() for x in xs]
            comm.reduce_scatter(ys)                                           # in place: result in the first n elements
            calls += 2
            torch.cuda.synchronize()
            for r in range(p):
                torch.testing.assert_close(outs[r].double(), want[r * n:(r + 1) * n], rtol=2e-2, atol=2e-2)
                assert torch.equal(ys[r][:n], outs[r])
    assert comm.stats()["ll"] == before + calls
    assert comm.status()["code"] == 0
    comm.close()


@pytest.mark.parametrize("p", [3, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.int32])
def test_ll_two_phase_allreduce(al, p, dtype):
    """Allreduce beyond the one-phase packet limit: reduce-scatter and allgather in packets inside one kernel.
    Odd lengths, unaligned views, in place and out of place, every rank bit-identical."""
    old1, old2 = al.get_tuning("ll_max_bytes"), al.get_tuning("ar_ll2_max_bytes")
    al.set_tuning("ll_max_bytes", 64)            # everything above 64 bytes takes the two-phase form
    al.set_tuning("ar_ll2_max_bytes", 4 << 20)
    comm = al.DeviceComm(emulate=p)
    comm.set_timeout_ms(3000)
    try:
        before = comm.stats()["ll"]
        calls = 0
        for it, n in enumerate((17, 100, 1000, 70_001, 300_000)):
            for op in ("sum", "max"):
                base = [rand(n + 3, dtype, 900 + 10 * it + r) for r in range(p)]
                xs = [b[1:1 + n] for b in base]                                    # views one element into their allocations
                want = ref_reduce(xs, op)
                outs = [torch.zeros(n + 2, dtype=dtype, device="cuda") for _ in range(p)]
                comm.allreduce(xs, [o[:n] for o in outs], op=op)
                ys = [x.clone() for x in xs]
                comm.allreduce(ys, op=op)                                          # in place
                calls += 2
                torch.cuda.synchronize()
                assert comm.status()["code"] == 0, comm.status()
                for r in range(p):
                    torch.testing.assert_close(outs[r][:n].double(), want, rtol=2e-2, atol=2e-2)
                    assert torch.all(outs[r][n:] == 0)
                    assert torch.equal(ys[r], outs[r][:n])
                assert all(torch.equal(outs[0], o) for o in outs)
        assert comm.stats()["ll"] == before + calls
        # one-phase and two-phase operations alternate on the same slots
        for n in (8, 5000, 12, 90_000):
            xs = [rand(n, torch.float32, n + r) for r in range(p)]
            comm.allreduce(xs)
            torch.cuda.synchronize()
            assert all(torch.equal(xs[0], x) for x in xs)
    finally:
        comm.close()
        al.set_tuning("ll_max_bytes", old1)
        al.set_tuning("ar_ll2_max_bytes", old2)


@pytest.mark.parametrize("p", [2, 4, 8])
def test_ll_allgather_alltoall_with_scale_and_explicit_paths(al, p):
    comm = al.DeviceComm(emulate=p)
    comm.set_timeout_ms(2000)
    for it, n in enumerate([1, 2, 5, 64, 1023, 65536]):
        for dtype in (torch.float32, torch.uint8 if n % 4 == 0 else torch.int16):
            ss = [rand(n, torch.float32, 100 + r + it).to(dtype) for r in range(p)]
            outs = [torch.zeros(n * p, dtype=dtype, device="cuda") for _ in range(p)]
            comm.allgather(ss, outs, algo="ll")
            xs = [rand(n * p, torch.float32, 200 + r + it).to(dtype) for r in range(p)]
            a2 = [torch.zeros(n * p, dtype=dtype, device="cuda") for _ in range(p)]
            comm.alltoall(xs, a2, algo="ll")
            ip = [x.clone() for x in xs]
            comm.alltoall(ip)                                                 # in place (automatic path: packets too)
            gp = [torch.zeros(n * p, dtype=dtype, device="cuda") for _ in range(p)]
            for r in range(p):
                gp[r][r * n:(r + 1) * n] = ss[r]
            comm.allgather(gp)                                                # in place
            torch.cuda.synchronize()
            for r in range(p):
                assert torch.equal(outs[r], torch.cat(ss))
                assert torch.equal(gp[r], torch.cat(ss))
                want = torch.cat([xs[q][r * n:(r + 1) * n] for q in range(p)])
                assert torch.equal(a2[r], want) and torch.equal(ip[r], want)
    # fused average / scale on the packet path
    xs = [rand(777, torch.float32, 300 + r) for r in range(p)]
    comm.allreduce(xs, op="avg", algo="ll")
    ys = [rand(777, torch.float32, 300 + r) for r in range(p)]
    comm.allreduce(ys, scale=0.25, algo="ll")
    torch.cuda.synchronize()
    st = torch.stack([rand(777, torch.float32, 300 + r) for r in range(p)])
    torch.testing.assert_close(xs[0], st.mean(0))
    torch.testing.assert_close(ys[p - 1], st.sum(0) * 0.25)
    # a message that does not fit is refused when the path is forced, and staged when it is not
    big = [rand(1_200_000, torch.float32, 1) for _ in range(p)]   # beyond one slot, and beyond p half-slots (two-phase form)
    with pytest.raises(al.AlError):
        comm.allreduce(big, algo="ll")
    before = comm.stats()["ll"]
    comm.allreduce(big)
    torch.cuda.synchronize()
    assert comm.stats()["ll"] == before
    comm.close()


def test_ll_mixed_with_staged_and_rooted_operations(al):
    """Packets, staged and rooted operations interleaved on one communicator: the parities of the packet slots
    and the epochs of the flags must stay consistent whatever the sequence."""
    p = 4
    comm = al.DeviceComm(emulate=p)
    comm.set_timeout_ms(2000)
    for it in range(6):
        small = [torch.full((100,), float(r + it), device="cuda") for r in range(p)]
        comm.allreduce(small)                                                 # packets
        big = [torch.full((100_000,), float(r), device="cuda") for r in range(p)]
        comm.allreduce(big)                                                   # staged
        b = [torch.full((50,), float(r * 10 + it), device="cuda") for r in range(p)]
        comm.bcast(b, root=it % p)                                            # rooted: staged
        again = [torch.full((3,), float(r), device="cuda") for r in range(p)]
        comm.allreduce(again, op="max")                                       # packets
        comm.barrier()
        empty = [torch.zeros(0, device="cuda") for _ in range(p)]
        comm.allreduce(empty)                                                 # nothing to move: staged handshake
        torch.cuda.synchronize()
        assert all(torch.all(s == sum(range(p)) + p * it) for s in small)
        assert all(torch.all(x == sum(range(p))) for x in big)
        assert all(torch.all(x == (it % p) * 10 + it) for x in b)
        assert all(torch.all(x == p - 1) for x in again)
    assert comm.status()["code"] == 0
    comm.close()


# ------------------------------------------------------------------------------------------------------
# window kernels
# ------------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("p", [2, 8])
@pytest.mark.parametrize("symmetric", [False, True])
def test_window_allgather_alltoall_bcast(al, p, symmetric):
    comm = al.DeviceComm(emulate=p)
    comm.set_timeout_ms(2000)
    for n in (4, 1001, 300_004):  # floats per rank slice
        if symmetric:
            outs = comm.symm_empty((n * p + 8,), torch.float32)               # registered when allocated
        else:
            outs = [torch.empty(n * p + 8, device="cuda") for _ in range(p)]
            assert comm.register(outs) >= 0
        for off in (0, 3):                                                     # 3: views that are not 16-byte aligned
            before = comm.stats()["window"]
            recv = [o[off:off + n * p] for o in outs]
            for o in outs:
                o.fill_(-1.0)
            ss = [rand(n, torch.float32, 400 + r) for r in range(p)]
            comm.allgather(ss, recv, algo="window")
            torch.cuda.synchronize()
            assert comm.status()["code"] == 0, comm.status()
            for r in range(p):
                assert torch.equal(recv[r], torch.cat(ss))
                assert torch.all(outs[r][off + n * p:] == -1.0)                # nothing past the end
            xs = [rand(n * p, torch.float32, 410 + r) for r in range(p)]
            comm.alltoall(xs, recv, algo="window")
            small = [torch.full((3,), float(r), device="cuda") for r in range(p)]
            comm.allreduce(small)                                              # a packet operation right after
            a2a_want = [torch.cat([xs[q][r * n:(r + 1) * n] for q in range(p)]) for r in range(p)]
            torch.cuda.synchronize()
            for r in range(p):
                assert torch.equal(recv[r], a2a_want[r])
                assert torch.all(small[r] == sum(range(p)))
            bb = [o[off:off + n] for o in outs]
            root = p - 1
            bb[root].copy_(rand(n, torch.float32, 999))
            comm.bcast(bb, root=root, algo="window")
            torch.cuda.synchronize()
            for r in range(p):
                assert torch.equal(bb[r], rand(n, torch.float32, 999))
            assert comm.stats()["window"] == before + 3
            # in-place allgather: every rank's contribution already sits at its place
            for r in range(p):
                recv[r].zero_()
                recv[r][r * n:(r + 1) * n] = float(r + 1)
            comm.allgather([recv[r][r * n:(r + 1) * n] for r in range(p)], recv, algo="window")
            torch.cuda.synchronize()
            want = torch.cat([torch.full((n,), float(r + 1), device="cuda") for r in range(p)])
            for r in range(p):
                assert torch.equal(recv[r], want)
        # automatic selection: large enough messages on registered buffers take the window path, small ones do not
        old_min = al.get_tuning("window_min_bytes")
        al.set_tuning("window_min_bytes", 256 << 10)      # the default (16 MiB) is beyond this test's sizes
        before = comm.stats()["window"]
        comm.allgather([rand(n, torch.float32, 1 + r) for r in range(p)], [o[:n * p] for o in outs])
        torch.cuda.synchronize()
        took = comm.stats()["window"] - before
        al.set_tuning("window_min_bytes", old_min)
        assert took == (1 if n * p * 4 >= (256 << 10) else 0)
        # a private receive buffer is refused on the forced path and staged on the automatic one
        priv = [torch.zeros(n * p, device="cuda") for _ in range(p)]
        with pytest.raises(al.AlError):
            comm.allgather([rand(n, torch.float32, r) for r in range(p)], priv, algo="window")
        if symmetric:
            comm.symm_free(outs)
        else:
            comm.unregister(outs)
    comm.close()


@pytest.mark.parametrize("p", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_window_reduce_scatter(al, p, dtype):
    comm = al.DeviceComm(emulate=p)
    comm.set_timeout_ms(2000)
    esz = torch.empty((), dtype=dtype).element_size()
    for n in (16 // esz, 4096, 250_000):  # elements per rank; slices are multiples of 16 bytes
        xs = [rand(n * p + 16, dtype, 500 + r) for r in range(p)]
        assert comm.register(xs) >= 0
        for off in (0, 16 // esz, 1):      # 1: sources that are not 16-byte aligned are read element-wise
            send = [x[off:off + n * p] for x in xs]
            for op in ("sum", "max", "avg"):
                before = comm.stats()["window"]
                outs = [torch.zeros(n + 1, dtype=dtype, device="cuda") for _ in range(p)]
                comm.reduce_scatter(send, [o[:n] for o in outs], op=op, algo="window")
                torch.cuda.synchronize()
                assert comm.status()["code"] == 0, comm.status()
                assert comm.stats()["window"] == before + 1
                want = ref_reduce(send, op)
                for r in range(p):
                    torch.testing.assert_close(outs[r][:n].double(), want[r * n:(r + 1) * n], rtol=2e-2, atol=2e-2)
                    assert outs[r][n] == 0
        # in place (the result overwrites input that other ranks still read) must not take the window path
        before = comm.stats()["window"]
        ys = [x[:n * p] for x in xs]                                           # registered, but used in place
        want = ref_reduce(ys, "sum")
        comm.reduce_scatter(ys)
        torch.cuda.synchronize()
        assert comm.stats()["window"] == before
        for r in range(p):
            torch.testing.assert_close(ys[r][:n].double(), want[r * n:(r + 1) * n], rtol=2e-2, atol=2e-2)
        comm.unregister(xs)
    comm.close()


def test_registration_table_is_bounded_and_reusable(al):
    p = 2
    comm = al.DeviceComm(emulate=p)
    bufs = []
    ids = []
    for i in range(40):  # more than the table holds: the surplus is refused (-1), never an error
        t = [torch.zeros(64, device="cuda") for _ in range(p)]
        w = comm.register(t)
        bufs.append(t)
        ids.append(w)
    assert ids.count(-1) == 40 - 32 and all(w >= 0 for w in ids[:32])
    comm.unregister(bufs[5])
    t = [torch.zeros(64, device="cuda") for _ in range(p)]
    assert comm.register(t) == ids[5]      # the freed slot is taken again
    for b in bufs:
        comm.unregister(b)                  # unknown or refused buffers are ignored
    comm.close()


def test_two_rank_allreduce_is_pipelined_above_threshold(al):
    """On two ranks large allreduces run the one-shot push with half of the grid pushing while the other half
    reduces; here the threshold is lowered so that a few MB already take that schedule (several chunks)."""
    old = al.get_tuning("ar_pipeline_min_bytes")
    al.set_tuning("ar_pipeline_min_bytes", 65536)
    try:
        comm = al.DeviceComm(emulate=2)
        comm.set_timeout_ms(2000)
        for n in (3_000_001, 5_000_000):
            xs = [rand(n, torch.float32, 700 + r) for r in range(2)]
            want = torch.stack(xs).sum(0)
            outs = [torch.zeros(n, device="cuda") for _ in range(2)]
            comm.allreduce(xs, outs)
            ys = [x.clone() for x in xs]
            comm.allreduce(ys, op="avg")      # in place, fused average
            small = [torch.ones(5, device="cuda") for _ in range(2)]
            comm.allreduce(small)
            torch.cuda.synchronize()
            assert comm.status()["code"] == 0
            for r in range(2):
                torch.testing.assert_close(outs[r], want)
                torch.testing.assert_close(ys[r], want / 2)
                assert torch.all(small[r] == 2)
        comm.close()
    finally:
        al.set_tuning("ar_pipeline_min_bytes", old)


@pytest.mark.parametrize("p", [2, 4, 8])
def test_row_exchange_strided_indexed_and_chunked(al, p):
    """exchange_rows against torch indexing: strided slices (sequence <-> head), index-selected rows (expert
    dispatch / combine), uneven counts, and slices larger than a staging slot (several chunks)."""
    from aluminum_b200.parallel import ulysses
    old = al.get_tuning("dev_stage_bytes")
    al.set_tuning("dev_stage_bytes", 1 << 20)       # 1 MiB halves: slots of 128 KiB on 8 ranks
    comm = al.DeviceComm(emulate=p)
    al.set_tuning("dev_stage_bytes", old)
    comm.set_timeout_ms(2000)
    for (s, h, d, dt) in ((8, 8, 4, torch.float32), (5, 16, 3, torch.bfloat16), (600, 8, 64, torch.float32)):
        full = rand(s * p * h * d, torch.float32, s).to(dt).view(s * p, h, d)
        shards = [t.contiguous() for t in full.chunk(p, dim=0)]
        before = comm.stats()["rows"]
        heads = ulysses.seq_to_head(comm, shards)
        torch.cuda.synchronize()
        for r in range(p):
            assert torch.equal(heads[r], full[:, r * (h // p):(r + 1) * (h // p)])
        back = ulysses.head_to_seq(comm, heads)
        torch.cuda.synchronize()
        for r in range(p):
            assert torch.equal(back[r], shards[r])
        assert comm.stats()["rows"] == before + 2 and comm.status()["code"] == 0
    comm.close()


@pytest.mark.parametrize("p", [2, 4])
def test_p2p_ring_of_slots_and_rendezvous_into_registered_buffers(al, p):
    """Point-to-point: a message of many pieces through the mailbox ring (more pieces than slots), and large
    messages that wait for the receiver and go straight into its registered buffer (no mailbox, no copy-out)."""
    old = al.get_tuning("dev_mailbox_bytes")
    al.set_tuning("dev_mailbox_bytes", 1 << 20)     # 1 MiB slots: a 9 MiB message is 9 pieces through 4 slots
    comm = al.DeviceComm(emulate=p)
    al.set_tuning("dev_mailbox_bytes", old)
    comm.set_timeout_ms(3000)
    n = 9 * 256 * 1024 + 17                          # floats: 9 MiB and a ragged tail
    for registered in (False, True):
        src = [rand(n, torch.float32, 800 + r) for r in range(p)]
        dst = [torch.full((n + 4,), -1.0, device="cuda") for _ in range(p)]
        if registered:
            assert comm.register(dst) >= 0
        for it in range(2):
            items = []
            for r in range(p):
                items.append((True, (r + 1) % p, src[r], r))
                items.append((False, (r - 1) % p, dst[r][:n], r))
            comm.p2p(items)
            small = [torch.full((8,), float(r), device="cuda") for r in range(p)]
            got = [torch.zeros(8, device="cuda") for _ in range(p)]
            comm.p2p([x for r in range(p) for x in ((True, (r + 1) % p, small[r], r), (False, (r - 1) % p, got[r], r))])
            torch.cuda.synchronize()
            assert comm.status()["code"] == 0, comm.status()
            for r in range(p):
                assert torch.equal(dst[r][:n], src[(r - 1) % p])
                assert torch.all(dst[r][n:] == -1.0)
                assert torch.all(got[r] == float((r - 1) % p))
        if registered:
            comm.unregister(dst)
    comm.close()


@pytest.mark.parametrize("p", [2, 3])
def test_p2p_small_messages_travel_as_packets(al, p):
    """Messages up to p2p_ll_max_bytes use the packet slots: odd sizes, unaligned buffers, more messages in a
    row than the ring has slots, mixed with mailbox-sized messages between the same pair of ranks."""
    comm = al.DeviceComm(emulate=p)
    comm.set_timeout_ms(3000)
    seq = [1, 7, 16, 100, 4099, 3_000_000, 65_539, 2_097_152, 5, 2_097_153, 33]     # bytes; 3 000 000 and 2 097 153 go through the mailbox
    for it, nbytes in enumerate(seq):
        src = [torch.randint(0, 256, (nbytes + 3,), dtype=torch.uint8, device="cuda", generator=torch.Generator(device="cuda").manual_seed(7 * it + r)) for r in range(p)]
        dst = [torch.full((nbytes + 5,), 0xEE, dtype=torch.uint8, device="cuda") for _ in range(p)]
        items = []
        for r in range(p):
            items.append((True, (r + 1) % p, src[r][3:], r))                      # source starts 3 bytes into its allocation
            items.append((False, (r - 1) % p, dst[r][1:1 + nbytes], r))           # destination 1 byte in
        comm.p2p(items)
        torch.cuda.synchronize()
        assert comm.status()["code"] == 0, comm.status()
        for r in range(p):
            assert torch.equal(dst[r][1:1 + nbytes], src[(r - 1) % p][3:]), (nbytes, r)
            assert dst[r][0] == 0xEE and torch.all(dst[r][1 + nbytes:] == 0xEE)
    # one-directional stream of small sends, received later: the sender runs ahead by at most the ring's depth
    if p == 2:
        msgs = [torch.full((64,), float(i), device="cuda") for i in range(6)]
        got = [torch.zeros(64, device="cuda") for _ in range(6)]
        for i in range(6):
            comm.p2p([(True, 1, msgs[i], 0), (False, 0, got[i], 1)])
        torch.cuda.synchronize()
        assert all(torch.equal(got[i], msgs[i]) for i in range(6))
    comm.close()


def test_guard_regions_catch_a_write_past_the_end(al):
    """Guard mode: 4 KiB of a known pattern before and after every symmetric buffer.  Library operations leave them
    intact; a stray 4-byte store just behind a buffer (made here with the library's fill kernel, inside the block's
    own allocation) is reported by check_guards() with its position."""
    import ctypes as C
    from aluminum_b200 import _lib
    al.set_tuning("debug_guard", 1)
    try:
        p = 4
        comm = al.DeviceComm(emulate=p)
        comm.set_timeout_ms(2000)
        n = 100 * p
        ts = comm.symm_empty((n,), torch.float32)
        for r in range(p):
            ts[r].fill_(float(r))
        comm.allreduce(ts)
        outs = comm.symm_empty((n * p,), torch.float32)
        comm.allgather(ts, outs, algo="window")
        comm.reduce_scatter(outs, [t[:n] for t in ts], algo="window")
        torch.cuda.synchronize()
        comm.check_guards()                                   # nothing wrote outside
        comm.symm_free(outs)                                  # (checks again)
        stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
        assert _lib.load().al_fill_u32(C.c_void_p(ts[2].data_ptr() + n * 4), 1, 0xDEADBEEF, stream) == 0
        torch.cuda.synchronize()
        with pytest.raises(al.AlError, match="after the buffer"):
            comm.check_guards()
        comm.close()
    finally:
        al.set_tuning("debug_guard", 0)
