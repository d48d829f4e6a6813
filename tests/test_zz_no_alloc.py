"""The allocation-free allreduce entry point (include/al/noalloc.h), called through its exported
C symbol, must give the same result as the regular emulated-communicator allreduce - twice in a
row, because the built-in scratch array keeps the previous call's contents.  Collected last on
purpose (file name), so a failure here cannot hide results of the other tests."""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_no_alloc_allreduce_matches_regular_entry_point():
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    import aluminum_b200 as al
    from aluminum_b200 import _lib
    lib = _lib.load()
    fn = lib.al_noalloc_allreduce_f32
    fn.restype = C.c_int
    fn.argtypes = [C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_int, C.c_size_t, C.c_void_p]
    err = lib.al_noalloc_last_error
    err.restype = C.c_char_p

    al.init()
    p, n = 4, 5000
    comm = al.DeviceComm(emulate=p)
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call in range(2):
        g = torch.Generator(device="cuda").manual_seed(1000 + call)
        xs = [torch.randn(n, device="cuda", generator=g) for _ in range(p)]
        want = [torch.empty(n, device="cuda") for _ in range(p)]
        comm.allreduce(xs, want)                      # existing entry point
        got = [torch.full((n,), float("nan"), device="cuda") for _ in range(p)]
        ins = (C.c_void_p * p)(*[x.data_ptr() for x in xs])
        outs = (C.c_void_p * p)(*[o.data_ptr() for o in got])
        rc = fn(ins, outs, p, n, stream)
        assert rc == 0, err().decode()
        torch.cuda.synchronize()
        for a, b in zip(got, want):
            torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-5)
    # sizes beyond the built-in scratch are refused with a clear message, nothing runs
    big = 8193
    xs = [torch.zeros(big, device="cuda") for _ in range(p)]
    ins = (C.c_void_p * p)(*[x.data_ptr() for x in xs])
    assert fn(ins, ins, p, big, stream) != 0 and b"exceeds" in err()
    assert fn(ins, ins, 9, 16, stream) != 0
    comm.close()
