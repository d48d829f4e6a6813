"""Element-wise kernels, RMA / halo paths, bounded-wait failure reporting and the
host-transfer backend, all on one GPU."""
import subprocess

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def al():
    import aluminum_b200 as al
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    al.init()
    return al


def test_native_library_is_loaded(al):
    from aluminum_b200 import _lib
    assert _lib.lib_path().exists()
    maps = open("/proc/self/maps").read()
    assert "libal_b200.so" in maps, "the native library must be the code that runs"
    assert "NVIDIA" in al.info() or "devices visible" in al.info()


@pytest.mark.parametrize("src_dt,dst_dt", [(torch.float32, torch.bfloat16), (torch.bfloat16, torch.float32),
                                            (torch.float32, torch.float32), (torch.float16, torch.float32),
                                            (torch.float32, torch.float16), (torch.float64, torch.float64)])
@pytest.mark.parametrize("n", [1, 1023, 1 << 20])
def test_scale_cast(al, src_dt, dst_dt, n):
    from aluminum_b200.ops import scale_cast
    x = torch.randn(n, device="cuda", dtype=torch.float32).to(src_dt)
    out = torch.empty(n, device="cuda", dtype=dst_dt)
    scale_cast(x, out, 0.25)
    torch.cuda.synchronize()
    want = (x.double() * 0.25).to(dst_dt)
    torch.testing.assert_close(out, want, rtol=1e-2 if dst_dt != torch.float64 else 1e-12, atol=1e-3)


def test_fused_sgd_matches_torch(al):
    from aluminum_b200.ops import sgd_momentum_step
    n = 1_000_003
    p0 = torch.randn(n, device="cuda")
    ref_p = torch.nn.Parameter(p0.clone())
    opt = torch.optim.SGD([ref_p], lr=0.1, momentum=0.9, weight_decay=1e-4)
    p, m, g = p0.clone(), torch.zeros(n, device="cuda"), torch.zeros(n, device="cuda")
    for step in range(3):
        grad = torch.randn(n, device="cuda")
        ref_p.grad = grad.clone()
        opt.step()
        g.copy_(grad)
        sgd_momentum_step(p, m, g, 0.1, 0.9, 1e-4, 1.0, first_step=(step == 0), zero_grad=True)
        torch.cuda.synchronize()
        torch.testing.assert_close(p, ref_p.data, rtol=1e-5, atol=1e-6)
        assert torch.count_nonzero(g) == 0


def test_halo_exchange_emulated(al):
    from aluminum_b200.ops import HaloExchange
    for p, periodic in ((2, False), (4, False), (4, True)):
        comm = al.DeviceComm(emulate=p)
        n, c, d, h, w, depth = 1, 5, 6, 16, 24, 1
        hx = HaloExchange(comm, n, c, d, h, w, depth, periodic)
        for r, t in enumerate(hx.tensors):
            t.fill_(-1.0)
            t[:, :, depth:depth + d] = torch.randn(n, c, d, h, w, device="cuda") + 10 * r
        snap = [t.clone() for t in hx.tensors]
        hx.exchange()
        torch.cuda.synchronize()
        for r in range(p):
            has_lo = p > 1 and (periodic or r > 0)
            has_hi = p > 1 and (periodic or r < p - 1)
            lo, hi = (r - 1) % p, (r + 1) % p
            if has_lo:   # my lower halo = the lower neighbour's last interior planes
                assert torch.equal(hx.tensors[r][:, :, :depth], snap[lo][:, :, d:d + depth])
            else:
                assert torch.all(hx.tensors[r][:, :, :depth] == -1.0)
            if has_hi:   # my upper halo = the upper neighbour's first interior planes
                assert torch.equal(hx.tensors[r][:, :, depth + d:], snap[hi][:, :, depth:2 * depth])
            else:
                assert torch.all(hx.tensors[r][:, :, depth + d:] == -1.0)
            assert torch.equal(hx.tensors[r][:, :, depth:depth + d], snap[r][:, :, depth:depth + d])
        hx.exchange()  # a second round reuses the flags with a new epoch
        torch.cuda.synchronize()
        assert comm.status()["code"] == 0
        comm.close()


def test_halo_pack_unpack(al):
    from aluminum_b200.ops import halo_pack, halo_unpack
    t = torch.randn(2, 3, 8, 5, 7, device="cuda")
    packed = halo_pack(t, 2, 2)
    torch.cuda.synchronize()
    assert torch.equal(packed.view(6, 2, 35), t.view(6, 8, 35)[:, 2:4])
    u = torch.zeros_like(t)
    halo_unpack(u, packed, 5, 2)
    torch.cuda.synchronize()
    assert torch.equal(u.view(6, 8, 35)[:, 5:7], t.view(6, 8, 35)[:, 2:4])


def test_rma_put_notify_wait_emulated(al):
    comm = al.DeviceComm(emulate=2)
    bufs = comm.symm_empty((4096,), torch.float32)
    bufs[0].fill_(3.0)
    bufs[1].zero_()
    # "rank 0" puts into rank 1's buffer; in emulation the peer buffer is directly addressable
    comm.put(bufs[0], 1, bufs[1].data_ptr())
    torch.cuda.synchronize()
    assert torch.all(bufs[1] == 3.0)
    comm.symm_free(bufs)
    comm.close()


def test_bounded_wait_reports_timeout_and_gpu_stays_usable(al):
    """A wait on a flag nobody sets must give up within its budget, fill the status record and
    leave the context usable (no trap, no hang)."""
    comm = al.DeviceComm(emulate=2)
    comm.set_timeout_ms(150)
    comm.wait(1)  # no matching notify exists
    torch.cuda.synchronize()
    st = comm.status()
    assert st["code"] == 1 and st["peer"] == 1 and st["where"] == 5
    with pytest.raises(al.AlError):
        comm.allreduce([torch.ones(4, device="cuda"), torch.ones(4, device="cuda")])
    comm.close()
    # the GPU and the library are still fine: a fresh communicator works
    comm2 = al.DeviceComm(emulate=2)
    xs = [torch.ones(1000, device="cuda"), torch.ones(1000, device="cuda") * 2]
    comm2.allreduce(xs)
    torch.cuda.synchronize()
    assert torch.all(xs[0] == 3.0)
    comm2.close()


def test_data_parallel_single_gpu_matches_torch(al):
    from aluminum_b200.models import MLP
    from aluminum_b200.parallel import DataParallel, Trainer
    torch.manual_seed(0)
    model = MLP(32, 64, 10).cuda()
    ref = MLP(32, 64, 10).cuda()
    ref.load_state_dict(model.state_dict())
    dp = DataParallel(model, None, lr=0.05, momentum=0.9)
    tr = Trainer(dp, autocast_dtype=None)
    opt = torch.optim.SGD(ref.parameters(), lr=0.05, momentum=0.9)
    lossf = torch.nn.CrossEntropyLoss()
    for i in range(4):
        x = torch.randn(16, 32, device="cuda")
        y = torch.randint(0, 10, (16,), device="cuda")
        l = tr.step_device(x, y)
        opt.zero_grad()
        lr = lossf(ref(x), y)
        lr.backward()
        opt.step()
        torch.testing.assert_close(l, lr.detach(), rtol=1e-4, atol=1e-5)
    for a, b in zip(model.parameters(), ref.parameters()):
        torch.testing.assert_close(a, b, rtol=1e-4, atol=1e-5)
    # end-to-end loop with host batches
    xh = torch.randn(16, 32).pin_memory()
    yh = torch.randint(0, 10, (16,)).pin_memory()
    losses = list(tr.run((xh, yh) for _ in range(3)))
    assert len(losses) == 3 and tr.h2d_bytes > 0 and tr.d2h_bytes == 12


@pytest.mark.parametrize("op", ["allreduce", "alltoall", "bcast", "sendrecv", "gatherv", "reduce", "scatter", "send",
                                "barrier"])
def test_host_transfer_backend(al, bin_dir, op):
    """GPU buffers staged through pinned memory, ranks as two processes sharing this GPU
    (no kernel of one rank waits for the other: the stream waits are released by the host)."""
    r = subprocess.run([str(bin_dir / "alrun"), "-n", "2", "--timeout", "120", str(bin_dir / "test_ops"),
                        "--backend", "ht", "--op", op, "--max-size", "65536", "--odd-sizes", "--nonblocking"],
                       capture_output=True, text=True, timeout=180, env={**__import__("os").environ, "AL_GPU_ID": "0"})
    assert r.returncode == 0, r.stdout + r.stderr


def test_host_transfer_failure_reaches_the_caller(al, bin_dir):
    """A failed host exchange (the host communicator is aborted on the host) makes Test / Wait and later calls
    throw, releases the stream, and leaves NaN instead of stale bytes in the receive buffer."""
    r = subprocess.run([str(bin_dir / "test_ht_failure")], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "ht failure test: ok" in r.stdout, r.stdout + r.stderr


def test_single_gpu_tools(al, bin_dir):
    """Wait / event micro-benchmarks and the single-rank device examples run on this GPU."""
    for tool, needle in (("benchmark_waits", "signal-to-pass"), ("benchmark_events", "pinned flag"),
                         ("test_stream_mem_ops", "stream memory operations")):
        r = subprocess.run([str(bin_dir / tool)] + (["200"] if tool.startswith("benchmark") else []),
                           capture_output=True, text=True, timeout=120)
        assert r.returncode == 0 and needle in r.stdout, tool + r.stdout + r.stderr
    r = subprocess.run([str(bin_dir / "hello_world"), "device"], capture_output=True, text=True, timeout=120)
    assert r.returncode == 0 and "sum of ranks = 0" in r.stdout, r.stdout + r.stderr
