"""Symmetric (peer-mapped) device buffers for the ranks of one node, and the fused optimizer step built on them.

Every rank allocates the same buffers with ``cudaMalloc``, exports CUDA-IPC handles, and maps all peers' buffers, so
that a kernel on any GPU can load from / store to any other GPU's copy over NVLink. The handle exchange rides on the
existing ``torch.distributed`` group (control plane only). This is the NVSHMEM-free symmetric heap that the fused
compute + collective kernels use; NCCL stays the twin / fallback (and the CPU path uses gloo).
"""

from __future__ import annotations

import ctypes as C
from typing import Optional

import torch
import torch.distributed as dist

from rl_b200.ops import lib as _L

_P, _I, _LL, _F, _D, _U = C.c_void_p, C.c_int, C.c_longlong, C.c_float, C.c_double, C.c_uint
_bound = False


def _bind():
    global _bound
    lib = _L.lib()
    if not _bound:
        lib.rlb_symm_alloc.argtypes = [C.c_ulonglong, C.POINTER(_P), C.c_char_p]
        lib.rlb_symm_open.argtypes = [C.c_char_p, C.POINTER(_P)]
        lib.rlb_symm_close.argtypes = [_P]
        lib.rlb_symm_free.argtypes = [_P]
        lib.rlb_fused_optim_step.argtypes = [_P, _P, _P, _P, _I, _I, _LL, _P, _P, _P, _F, _F, _F, _F, _F, _I, _F, _F, _U, _D, _P, _P, _P, _P]
        lib.rlb_p2p_allgather.argtypes = [_P, _P, _P, _I, _I, _LL, _U, _D, _P, _P]
        for n in ("rlb_symm_alloc", "rlb_symm_open", "rlb_symm_close", "rlb_symm_free", "rlb_fused_optim_step", "rlb_p2p_allgather"):
            getattr(lib, n).restype = C.c_int
        _bound = True
    return lib


class _RawCuda:
    """Exposes a raw device pointer through ``__cuda_array_interface__`` so that torch can alias it without copying."""

    def __init__(self, ptr: int, nbytes: int, owner):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 2}
        self._owner = owner


class SymmetricBuffer:
    """``nbytes`` of device memory present on every rank of ``group`` and mapped into every rank's address space."""

    def __init__(self, nbytes: int, group=None, device: Optional[torch.device] = None):
        lib = _bind()
        self.group = group
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.nbytes = -(-int(nbytes) // 256) * 256
        ptr = _P()
        handle = C.create_string_buffer(64)
        rc = lib.rlb_symm_alloc(self.nbytes, C.byref(ptr), handle)
        if rc:
            raise RuntimeError(f"symmetric allocation of {self.nbytes} bytes failed (CUDA error {rc})")
        self.local_ptr = ptr.value
        handles = [None] * self.world
        if self.world > 1:
            dist.all_gather_object(handles, handle.raw, group=group)
        self.peer_ptrs: list[int] = []
        self._opened: list[int] = []
        for r in range(self.world):
            if r == self.rank:
                self.peer_ptrs.append(self.local_ptr)
                continue
            p = _P()
            rc = lib.rlb_symm_open(handles[r], C.byref(p))
            if rc:
                raise RuntimeError(f"mapping rank {r}'s buffer failed (CUDA error {rc}); is peer access available?")
            self.peer_ptrs.append(p.value)
            self._opened.append(p.value)
        self._table = (_P * self.world)(*self.peer_ptrs)
        self._raw = _RawCuda(self.local_ptr, self.nbytes, self)
        self.bytes = torch.as_tensor(self._raw, device=self.device)

    def tensor(self, dtype: torch.dtype, numel: Optional[int] = None, byte_offset: int = 0) -> torch.Tensor:
        """A view of the local copy as ``dtype`` (the whole buffer by default)."""
        item = torch.empty((), dtype=dtype).element_size()
        numel = (self.nbytes - byte_offset) // item if numel is None else numel
        return self.bytes[byte_offset : byte_offset + numel * item].view(dtype)

    @property
    def table(self):
        """ctypes array of the ``world`` device pointers (index = rank)."""
        return self._table

    def close(self) -> None:
        lib = _bind()
        if dist.is_initialized() and self.world > 1:
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
        for p in self._opened:
            lib.rlb_symm_close(p)
        self._opened = []
        if self.local_ptr:
            self.bytes = None
            lib.rlb_symm_free(self.local_ptr)
            self.local_ptr = 0


class FusedOptimizerComm:
    """Owns the peer-mapped parameter / gradient buffers and runs the one-kernel optimizer step."""

    def __init__(self, group=None, wait_limit_s: float = 20.0):
        self.group = group
        self.wait_limit_s = wait_limit_s
        self.epoch = 0
        self.param_buf: Optional[SymmetricBuffer] = None
        self.grad_buf: Optional[SymmetricBuffer] = None
        self.ctrl = SymmetricBuffer(4096, group)  # flags [4][8] uint32 at 0, slots [8] float at 1024
        self.rank, self.world = self.ctrl.rank, self.ctrl.world
        self._slots_table = (_P * self.world)(*[p + 1024 for p in self.ctrl.peer_ptrs])
        dev = self.ctrl.device
        self._scratch = torch.zeros(2, dtype=torch.float32, device=dev)   # partial sum of squares, abort word
        self._norm = torch.zeros(1, dtype=torch.float32, device=dev)

    # allocators handed to FlatParams so that the flat buffers live in peer-mapped memory
    def alloc_params(self, numel: int, dtype: torch.dtype, device) -> torch.Tensor:
        self.param_buf = SymmetricBuffer(numel * torch.empty((), dtype=dtype).element_size(), self.group)
        return self.param_buf.tensor(dtype, numel)

    def alloc_grads(self, numel: int, dtype: torch.dtype, device) -> torch.Tensor:
        self.grad_buf = SymmetricBuffer(numel * torch.empty((), dtype=dtype).element_size(), self.group)
        return self.grad_buf.tensor(dtype, numel)

    def usable(self, opt) -> bool:
        return (self.param_buf is not None and self.grad_buf is not None and opt.master_format == "split16"
                and opt.flat.grad is not None and opt.flat.grad.dtype == torch.float32 and opt.shard_numel % 8 == 0)

    def step(self, opt, grad_div: float = 1.0) -> torch.Tensor:
        """reduce-scatter + clip + AdamW + all-gather in one cooperative kernel (see rl_b200/csrc/comm.cu)."""
        lib = _bind()
        # No host-side rendezvous: the kernel's first flag barrier absorbs the step-time skew between the ranks (its
        # limit, wait_limit_s, is sized for that skew, not for microseconds).
        self.epoch += 1
        rc = lib.rlb_fused_optim_step(
            self.grad_buf.table, self.param_buf.table, self.ctrl.table, self._slots_table, self.rank, self.world,
            opt.shard_numel, opt.p_lo.data_ptr(), opt.m.data_ptr(), opt.v.data_ptr(), opt.lr, opt.betas[0], opt.betas[1],
            opt.eps, opt.weight_decay, opt.step_count, float(opt.max_grad_norm or 0.0), float(grad_div), self.epoch,
            float(self.wait_limit_s), self._scratch.data_ptr(), self._norm.data_ptr(), _L.status_word(self.ctrl.device).data_ptr(),
            torch.cuda.current_stream().cuda_stream)
        _L.Counters.launches += 1
        if rc:
            raise RuntimeError(f"rlb_fused_optim_step failed with code {rc}")
        opt.last_grad_norm = self._norm.clone()
        return opt.last_grad_norm

    def close(self) -> None:
        for b in (self.param_buf, self.grad_buf, self.ctrl):
            if b is not None:
                b.close()
