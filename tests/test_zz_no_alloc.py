"""RMSNorm backward through ``rlb_rmsnorm_bwd_static``, the entry point for callers that may not allocate.

Some processes that embed this library own the whole device memory themselves (a server that sized its KV cache from
the free memory, a runtime with one arena reserved at start-up): a ``cudaMalloc`` made for the library can fail there
and it stalls the device. The regular ``rlb_rmsnorm_bwd`` needs a caller-provided scratch buffer; the static variant
keeps that scratch in a fixed array inside the library. This test calls the exported C symbol directly (no Python
wrapper in between) and checks that it reproduces the regular entry point on two calls in a row, which share the
array and have different shapes, and that shapes beyond the fixed maximum are refused without launching anything.

The file name sorts last on purpose: a run that stops at the first failure has then already run every other test.
"""

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def _bind(lib):
    P, I, L = C.c_void_p, C.c_int, C.c_longlong
    f = lib.rlb_rmsnorm_bwd_static
    f.argtypes = [P, P, P, P, P, P, I, L, I, L, L, P]
    f.restype = C.c_int
    s = lib.rlb_rmsnorm_bwd_static_strerror
    s.argtypes = [I]
    s.restype = C.c_char_p
    return f, s


def _regular(rows, d, dy, x, w, rstd):
    from rl_b200.ops.lib import call, lib, ptr, stream_ptr

    dx = torch.empty((rows, d), dtype=torch.bfloat16, device="cuda")
    dw = torch.empty(d, dtype=torch.float32, device="cuda")
    parts = lib().rlb_rmsnorm_bwd_parts(rows)
    scratch = torch.empty((parts, d), dtype=torch.float32, device="cuda")
    call("rlb_rmsnorm_bwd", ptr(dy), ptr(x), ptr(w), ptr(rstd), ptr(dx), ptr(scratch), ptr(dw), None, 0, rows, d, d, d, 0,
         stream_ptr())
    return dx, dw


def test_static_scratch_matches_regular_entry_point(native_lib):
    fn, strerror = _bind(native_lib)
    torch.manual_seed(0)
    stream = torch.cuda.current_stream().cuda_stream
    for rows, d in [(1000, 4096), (37, 1024)]:  # the second call reuses the array after a larger first call
        x = torch.randn(rows, d, device="cuda", dtype=torch.bfloat16)
        dy = torch.randn(rows, d, device="cuda", dtype=torch.bfloat16)
        w = (1 + 0.1 * torch.randn(d, device="cuda")).to(torch.bfloat16)
        rstd = torch.rsqrt(x.float().pow(2).mean(-1) + 1e-5)
        dx_ref, dw_ref = _regular(rows, d, dy, x, w, rstd)
        # outputs are allocated before the call; the call itself allocates nothing
        dx = torch.empty((rows, d), dtype=torch.bfloat16, device="cuda")
        dw = torch.empty(d, dtype=torch.float32, device="cuda")
        torch.cuda.synchronize()
        free_before, held_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_allocated()
        rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), 0, rows, d, d, d, stream)
        assert rc == 0, strerror(rc)
        torch.cuda.synchronize()
        # the property the entry point exists for: neither the driver nor torch's allocator handed out memory
        assert torch.cuda.memory_allocated() == held_before
        assert torch.cuda.mem_get_info()[0] >= free_before
        err_dx = (dx.float() - dx_ref.float()).abs().max().item() / (dx_ref.float().abs().max().item() + 1e-6)
        err_dw = (dw - dw_ref).abs().max().item() / (dw_ref.abs().max().item() + 1e-6)
        assert err_dx < 1e-2 and err_dw < 1e-2, (err_dx, err_dw)
        # accumulate mode adds to what dw holds
        rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), 1, rows, d, d, d, stream)
        assert rc == 0, strerror(rc)
        torch.cuda.synchronize()
        assert (dw - 2 * dw_ref).abs().max().item() / (dw_ref.abs().max().item() + 1e-6) < 1e-2


def test_static_scratch_rejects_oversize(native_lib):
    fn, strerror = _bind(native_lib)
    t = torch.zeros(8, device="cuda", dtype=torch.bfloat16)
    f = torch.zeros(8, device="cuda")
    rc = fn(t.data_ptr(), t.data_ptr(), t.data_ptr(), f.data_ptr(), t.data_ptr(), f.data_ptr(), 0, 1, 16384, 16384, 16384, 0)
    assert rc == -5 and b"8192" in strerror(rc)
    rc = fn(t.data_ptr(), t.data_ptr(), t.data_ptr(), f.data_ptr(), t.data_ptr(), f.data_ptr(), 0, 1, 12, 12, 12, 0)
    assert rc == -2


def test_static_scratch_rejects_bad_pointers(native_lib):
    """A misaligned or null operand is refused on the host: nothing reaches the 16-byte vector loads."""
    fn, strerror = _bind(native_lib)
    d = 64
    buf = torch.zeros(4 * d + 8, device="cuda", dtype=torch.bfloat16)
    good, odd = buf[:d], buf[1 : d + 1]          # odd starts 2 bytes past a 16-byte boundary
    f = torch.zeros(d, device="cuda")
    args = lambda dy, x, w, dx: (dy, x, w, f.data_ptr(), dx, f.data_ptr(), 0, 1, d, d, d, 0)
    g = good.data_ptr()
    assert fn(*args(g, g, g, g)) == 0
    for bad in (args(odd.data_ptr(), g, g, g), args(g, odd.data_ptr(), g, g), args(g, g, odd.data_ptr(), g),
                args(g, g, g, odd.data_ptr()), args(None, g, g, g)):
        assert fn(*bad) == -2
    assert fn(g, g, g, f.data_ptr(), g, f.data_ptr(), 0, 1, d, d - 8, d, 0) == -2   # stride shorter than a row
    assert fn(g, g, g, f.data_ptr(), g, f.data_ptr(), 0, 2**31, d, d, d, 0) == -2   # rows do not fit an int
    torch.cuda.synchronize()
    assert b"aligned" in strerror(-2)
