"""A device-side wait that runs out must end in a status code and a clean return, never in a hang or a fault.

Each case calls a fused compute + collective kernel with ``world = 2`` on ONE GPU: the "peer" buffers are a second
local allocation that no kernel ever signals, and the call's wait limit is a few milliseconds. The kernel therefore
times out on its first peer wait. The tests check the recorded code (``RLB_ERR_WAIT_PEER`` = 7, or ``RLB_ERR_WAIT_FLAG``
= 5 from a CTA that waited for the go-ahead of the CTA that runs the peer barrier), that the outputs were left alone,
and that the next ordinary launch on the same context works. Nothing here faults, traps or spins without a limit.
"""

import ctypes as C
import time

import pytest
import torch

pytestmark = pytest.mark.gpu

P, I, LL, F, D, U = C.c_void_p, C.c_int, C.c_longlong, C.c_float, C.c_double, C.c_uint
WAIT_S = 0.005


def _table(*tensors):
    return (P * len(tensors))(*[t.data_ptr() for t in tensors])


def _plain_gemm_ok():
    """An ordinary launch after the time-out: the context is alive and the library still computes."""
    from rl_b200.ops import functional as Fn
    from rl_b200.ops.lib import check_status

    a = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(256, 128, device="cuda", dtype=torch.bfloat16)
    y = Fn.gemm(a, w)
    ref = a.float() @ w.float().t()
    assert (y.float() - ref).abs().max().item() <= 2e-2 * ref.abs().max().item()
    assert check_status() == 0


def test_fused_optimizer_aborts_when_the_peer_never_arrives(native_lib):
    from rl_b200.ops.lib import check_status, status_word
    from rl_b200.parallel.symmetric import _bind

    lib = _bind()
    check_status()
    n = 8192   # elements per rank
    dev = "cuda"
    grads = [torch.randn(2 * n, device=dev), torch.randn(2 * n, device=dev)]
    params = [torch.randn(2 * n, device=dev).to(torch.bfloat16) for _ in range(2)]
    flags = [torch.zeros(64, dtype=torch.int32, device=dev) for _ in range(2)]
    slots = [torch.zeros(8, device=dev) for _ in range(2)]
    p_lo = torch.zeros(n, dtype=torch.int16, device=dev)
    m, v = torch.zeros(n, device=dev), torch.zeros(n, device=dev)
    scratch, norm = torch.zeros(2, device=dev), torch.full((1,), -1.0, device=dev)
    before = [t.clone() for t in (*grads, *params, p_lo, m, v)]
    t0 = time.perf_counter()
    rc = lib.rlb_fused_optim_step(_table(*grads), _table(*params), _table(*flags), _table(*slots), 0, 2, n, p_lo.data_ptr(),
                                  m.data_ptr(), v.data_ptr(), 1e-3, 0.9, 0.999, 1e-8, 0.01, 1, 1.0, 1.0, 1, WAIT_S,
                                  scratch.data_ptr(), norm.data_ptr(), status_word().data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0   # milliseconds, not the library-wide limit
    assert check_status() == 7
    for a, b in zip((*grads, *params, p_lo, m, v), before):
        assert torch.equal(a, b)            # parameters, moments, gradients and the "peer" are untouched
    assert norm.item() == -1.0
    # the same kernel with world = 1 (no peer) now completes and updates the parameters
    rc = lib.rlb_fused_optim_step(_table(grads[0]), _table(params[0]), _table(flags[0]), _table(slots[0]), 0, 1, n, p_lo.data_ptr(),
                                  m.data_ptr(), v.data_ptr(), 1e-3, 0.9, 0.999, 1e-8, 0.01, 1, 1.0, 1.0, 2, WAIT_S,
                                  scratch.data_ptr(), norm.data_ptr(), status_word().data_ptr(), torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert check_status() == 0 and norm.item() > 0 and not torch.equal(params[0][:n], before[2][:n])
    _plain_gemm_ok()


def test_tp_scatter_gemm_times_out_cleanly(native_lib):
    from rl_b200.ops.lib import check_status, status_word
    from rl_b200.parallel.tensor import _bind

    lib = _bind()
    check_status()
    M, N, K, world = 256, 256, 128, 2
    rows = M // world
    a = torch.randn(M, K, device="cuda", dtype=torch.bfloat16)
    w = torch.randn(N, K, device="cuda", dtype=torch.bfloat16)
    out = torch.full((rows, N), 7.0, device="cuda", dtype=torch.bfloat16)
    stages = [torch.zeros(world * rows * N, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    flags = [torch.zeros(64, dtype=torch.int32, device="cuda") for _ in range(world)]
    t0 = time.perf_counter()
    rc = lib.rlb_gemm_tp_scatter(a.data_ptr(), K, w.data_ptr(), K, 0, M, N, K, rows, 0, out.data_ptr(), N, None, 0, _table(*stages),
                                 _table(*flags), 0, world, 1, None, WAIT_S, status_word().data_ptr(),
                                 torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0
    assert check_status() in (5, 7)
    assert torch.all(out == 7.0)                      # the output was left alone
    assert torch.all(stages[1] == 0)                  # nothing was stored into the "peer" before it entered the call
    _plain_gemm_ok()


def test_moe_dispatch_times_out_cleanly(native_lib):
    from rl_b200.ops.lib import check_status, lib as get_lib, status_word

    lib = get_lib()
    lib.rlb_moe_push_rows.argtypes = [P, LL, P, P, P, I, I, P, P, P, I, I, I, U, D, P, LL, P]
    lib.rlb_moe_push_rows.restype = C.c_int
    check_status()
    n, d, world = 64, 256, 2
    src = torch.randn(n, d, device="cuda", dtype=torch.bfloat16)
    dst_rank = torch.zeros(n, dtype=torch.int32, device="cuda")        # every row stays on this rank
    dst_row = torch.arange(n, dtype=torch.int32, device="cuda")
    bufs = [torch.zeros(n, d, device="cuda", dtype=torch.bfloat16) for _ in range(world)]
    metas = [torch.zeros(n, 2, dtype=torch.int32, device="cuda") for _ in range(world)]
    flags = [torch.zeros(32, dtype=torch.int32, device="cuda") for _ in range(world)]
    rc = lib.rlb_moe_push_rows(src.data_ptr(), d * 2, None, dst_rank.data_ptr(), dst_row.data_ptr(), n, d * 2, _table(*bufs),
                               _table(*metas), _table(*flags), 0, world, 0, 1, WAIT_S, status_word().data_ptr(), n,
                               torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    t0 = time.perf_counter()
    torch.cuda.synchronize()
    assert time.perf_counter() - t0 < 1.0
    assert check_status() == 7                        # the closing barrier gave up on the silent peer
    assert torch.equal(bufs[0], src) and torch.all(bufs[1] == 0)   # local rows landed; the "peer" got nothing
    _plain_gemm_ok()
    # a destination row beyond the receiver's buffer is recorded and skipped, never stored (world 1: no peer to wait for)
    bad_row = dst_row.clone()
    bad_row[5] = n + 3
    one = [torch.zeros(n, d, device="cuda", dtype=torch.bfloat16)]
    rc = lib.rlb_moe_push_rows(src.data_ptr(), d * 2, None, dst_rank.data_ptr(), bad_row.data_ptr(), n, d * 2, _table(*one),
                               _table(metas[0]), _table(flags[0]), 0, 1, 0, 2, WAIT_S, status_word().data_ptr(), n,
                               torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert rc == 0 and check_status() == 8            # RLB_ERR_BOUNDS
    keep = torch.ones(n, dtype=torch.bool, device="cuda")
    keep[5] = False
    assert torch.equal(one[0][keep], src[keep]) and torch.all(one[0][5] == 0)
    _plain_gemm_ok()


def test_status_is_raised_on_the_product_path(native_lib):
    """``raise_on_status`` turns a recorded code into an exception that names it (the product paths call it where they
    synchronise anyway)."""
    from rl_b200.ops.lib import NativeLibraryError, check_status, raise_on_status, status_word

    check_status()
    status_word().fill_(7)
    with pytest.raises(NativeLibraryError, match="RLB_ERR_WAIT_PEER"):
        raise_on_status("test")
    assert check_status() == 0
    raise_on_status("test")   # clean word: no exception
