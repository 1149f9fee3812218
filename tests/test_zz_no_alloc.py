"""The allocation-free C entry point `memarch_instinct_hs_step_noalloc` (csrc/memarch_noalloc.h), called through its
exported symbol the way a host application that may not allocate device memory would call it, against the regular
(allocating) optimizer step on the same inputs - two calls in a row, because the built-in scratch array keeps the
previous call's contents and the function has to clear what must start at zero.

Collected last on purpose (file name): a run that stops at the first failure has then already run every other test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from memarch_b200.ops import _ext
    _ext.load(required=True)
    lib = ctypes.CDLL(_ext.so_path())
    fn = lib.memarch_instinct_hs_step_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int,
                   ctypes.c_int, ctypes.c_longlong, ctypes.c_longlong, ctypes.c_float, ctypes.c_float, ctypes.c_float,
                   ctypes.c_float, ctypes.c_float, ctypes.c_void_p]
    return fn


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("bf16", [True, False])
def test_noalloc_step_matches_allocating_step_twice(bf16):
    from memarch_b200.ops import _ext
    C = _ext.C()
    fn = _lib()
    torch.manual_seed(0)
    R, Cc = 768, 1024
    dt = torch.bfloat16 if bf16 else torch.float32
    w0 = (torch.randn(R, Cc, device="cuda") * 0.05).to(dt)
    beta, wd, gain, stake, lr = 0.9, 0.1 / 0.12, 1.3, 0.6, 7.2e-5
    # regular path: device scalars, scratch from the allocator
    pa, ma = w0.clone(), torch.zeros(R, Cc, device="cuda", dtype=dt)
    wa = pa.float().clone() if bf16 else None
    gvec, st, lrt = torch.tensor([gain], device="cuda"), torch.tensor(stake, device="cuda"), torch.tensor(lr, device="cuda")
    seed = torch.zeros((), dtype=torch.int64, device="cuda")
    # allocation-free path: same inputs, caller-owned buffers only
    pb, mb = w0.clone(), torch.zeros(R, Cc, device="cuda", dtype=dt)
    wb = pb.float().clone() if bf16 else None
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        g = torch.randn(R, Cc, device="cuda").to(dt)
        C.instinct_step(pa, g, ma, wa, None, gvec, 0, st, lrt, None, beta, wd, 4, False, seed, None)
        before = torch.cuda.memory_allocated()
        rc = fn(pb.data_ptr(), g.data_ptr(), mb.data_ptr(), wb.data_ptr() if bf16 else None, int(bf16), int(bf16), int(bf16),
                R, Cc, gain, stake, lr, beta, wd, ctypes.c_void_p(stream))
        assert rc == 0
        assert torch.cuda.memory_allocated() == before          # nothing came from the caching allocator
        torch.cuda.synchronize()
        tol = 2e-2 if bf16 else 1e-4
        assert _rel(pb - w0, pa - w0) < tol, (call, _rel(pb - w0, pa - w0))
        assert _rel(mb, ma) < tol
        if bf16:
            assert _rel(wb - w0.float(), wa - w0.float()) < 1e-4


def test_noalloc_rejects_oversized_weight():
    fn = _lib()
    x = torch.zeros(8, device="cuda")
    rc = fn(x.data_ptr(), x.data_ptr(), x.data_ptr(), None, 0, 0, 0, 1 << 19, 4096, 1.0, 0.5, 1e-4, 0.9, 0.0, None)
    assert rc == 1                                              # MEMARCH_NOALLOC_TOO_LARGE, nothing launched
    torch.cuda.synchronize()
