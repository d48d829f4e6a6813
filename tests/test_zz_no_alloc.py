"""The allocation-free allreduce entry point (include/al/noalloc.h), called through its exported
C symbol, must give the same result as the regular emulated-communicator allreduce and as a plain
fp32 sum in PyTorch - twice in a row, because the built-in scratch array keeps the previous call's
contents.  Collected last on purpose (file name), so a failure here cannot hide results of the
other tests."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _bind():
    from aluminum_b200 import _lib
    lib = _lib.load()
    fn = lib.al_noalloc_allreduce_f32
    fn.restype = C.c_int
    fn.argtypes = [C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_int, C.c_size_t, C.c_void_p]
    err = lib.al_noalloc_last_error
    err.restype = C.c_char_p
    status = lib.al_noalloc_status
    status.restype = C.c_int
    status.argtypes = [C.POINTER(C.c_int)]
    reset = lib.al_noalloc_reset
    reset.restype = C.c_int
    reset.argtypes = [C.c_void_p]
    return fn, err, status, reset


def test_no_alloc_allreduce_matches_regular_entry_point():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import aluminum_b200 as al
    fn, err, status, reset = _bind()

    al.init()
    p, n = 4, 5000
    comm = al.DeviceComm(emulate=p)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call in range(2):
        g = torch.Generator(device="cuda").manual_seed(1000 + call)
        xs = [torch.randn(n, device="cuda", generator=g) for _ in range(p)]
        want = [torch.empty(n, device="cuda") for _ in range(p)]
        comm.allreduce(xs, want)                      # existing entry point
        plain = torch.stack(xs).sum(0)                # fp32 reference of the same operation
        got = [torch.full((n,), float("nan"), device="cuda") for _ in range(p)]
        ins = (C.c_void_p * p)(*[x.data_ptr() for x in xs])
        outs = (C.c_void_p * p)(*[o.data_ptr() for o in got])
        rc = fn(ins, outs, p, n, stream)
        assert rc == 0, err().decode()
        torch.cuda.synchronize()
        for a, b in zip(got, want):
            torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-5)
            torch.testing.assert_close(a, plain, rtol=1e-5, atol=1e-5)
    code = C.c_int(-1)
    assert status(C.byref(code)) == 0 and code.value == 0, err().decode()
    # sizes beyond the built-in scratch are refused with a clear message, nothing runs
    big = 8193
    xs = [torch.zeros(big, device="cuda") for _ in range(p)]
    ins = (C.c_void_p * p)(*[x.data_ptr() for x in xs])
    assert fn(ins, ins, p, big, stream) != 0 and b"exceeds" in err()
    assert fn(ins, ins, 9, 16, stream) != 0
    comm.close()


@pytest.mark.parametrize("p,n", [(1, 100), (3, 0), (3, 1), (8, 8192), (2, 4097)])
def test_no_alloc_allreduce_edge_shapes_and_aliasing(p, n):
    """Rank counts 1 to 8, empty and full-size vectors, and outputs that alias their rank's input."""
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    fn, err, status, reset = _bind()
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    g = torch.Generator(device="cuda").manual_seed(7 * p + n)
    for call in range(2):
        xs = [torch.randn(max(n, 1), device="cuda", generator=g)[:n] for _ in range(p)]
        plain = torch.stack(xs).sum(0) if n else None
        ptrs = (C.c_void_p * p)(*[x.data_ptr() for x in xs])
        assert fn(ptrs, ptrs, p, n, stream) == 0, err().decode()   # in place: output r aliases input r
        torch.cuda.synchronize()
        for x in xs:
            if n:
                torch.testing.assert_close(x, plain, rtol=1e-5, atol=1e-5)
    code = C.c_int(-1)
    assert status(C.byref(code)) == 0 and code.value == 0, err().decode()
    # reset leaves a working entry point behind
    assert reset(stream) == 0, err().decode()
    xs = [torch.ones(16, device="cuda") for _ in range(p)]
    ptrs = (C.c_void_p * p)(*[x.data_ptr() for x in xs])
    assert fn(ptrs, ptrs, p, 16, stream) == 0, err().decode()
    torch.cuda.synchronize()
    assert all(torch.all(x == float(p)) for x in xs)
