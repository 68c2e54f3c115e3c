"""ctypes binding of the native library ``rl_b200/_C.so`` (sm_100a kernels + C++ runtime).

The library exposes a plain C ABI (``rlb_*``). Tensors cross as raw device pointers and the current
CUDA stream as an opaque pointer, so there is no dependency on torch's C++ headers and a kernel launch
costs one foreign call. ``lib()`` loads the library once; on a machine with a GPU a missing library is
an error, never a silent fallback.
"""

from __future__ import annotations

import ctypes as C
import os
from pathlib import Path
from typing import Any

import torch

_LIB_PATH = Path(__file__).resolve().parent.parent / "_C.so"
_lib = None

P = C.c_void_p
I = C.c_int
L = C.c_longlong
F = C.c_float
U64 = C.c_ulonglong

# name -> argument types (all functions return int: 0 ok, >0 CUDA error, <0 bad argument)
_SIGS: dict[str, list[Any]] = {
    "rlb_gemm_bf16": [P, P, P, I, I, I, L, L, L, I, I, I, I, P, P, L, P, I, P],
    "rlb_gemm_num_n_tiles": [I],
    "rlb_gemm_skinny": [P, P, P, I, I, I, L, L, L, I, P, P, L, I, P, P],
    "rlb_gemm_skinny_fused": [P, P, P, I, I, I, L, L, L, I, P, P, L, I, P, I, L, F, P, L, P, P, L, I, P, P],
    "rlb_gemm_skinny_split": [I, I],
    "rlb_gemm_skinny_static_weights": [I],
    "rlb_lm_head_logprob": [P, P, I, I, I, L, L, P, F, P, P, P, P, P, P, P, P, P],
    "rlb_logprob_combine": [P, P, P, P, I, I, P, P, P, P],
    "rlb_lm_head_partials": [P, P, I, I, I, L, L, P, F, P, P, P, P, P, P],
    "rlb_lm_head_dlogits": [P, P, P, I, I, I, L, L, L, P, F, P, P, P, P, P, P],
    "rlb_rmsnorm_fwd": [P, P, P, P, P, P, L, I, L, L, F, P],
    "rlb_rmsnorm_bwd_parts": [L],
    "rlb_rmsnorm_bwd": [P, P, P, P, P, P, P, P, I, L, I, L, L, I, P],
    "rlb_rope": [P, P, P, L, I, I, L, I, P],
    "rlb_head_rmsnorm_fwd": [P, P, P, P, L, I, I, L, L, F, P],
    "rlb_head_rmsnorm_bwd": [P, P, P, P, P, P, L, I, I, L, L, L, P],
    "rlb_swiglu_fwd": [P, P, L, I, P],
    "rlb_swiglu_bwd": [P, P, P, L, I, P],
    "rlb_embedding_fwd": [P, P, P, L, I, I, P],
    "rlb_embedding_bwd": [P, P, P, L, I, I, P],
    "rlb_adamw": [P, P, P, P, I, P, P, L, F, F, F, F, F, I, P, P],
    "rlb_sumsq": [P, I, L, P, P],
    "rlb_clip_scale": [P, F, F, P, P, P],
    "rlb_clipped_pg": [P, P, P, P, P, P, L, F, F, F, F, I, F, F, I, I, F, F, I, I, I, F, P, P, P],
    "rlb_cast_f32_bf16": [P, P, L, P],
    "rlb_add_bf16": [P, P, P, L, P],
    "rlb_kv_cache_write": [P, P, P, P, L, I, I, I, I, L, L, P, P],
    "rlb_rope_kv_cache_write": [P, P, P, P, P, P, L, I, I, I, I, L, L, P, P],
    "rlb_paged_decode": [P, L, P, P, P, I, P, I, I, I, I, I, F, I, P, P, P, L, P],
    "rlb_paged_decode_tma": [P, L, P, P, I, P, I, P, I, I, I, I, I, F, I, P, P, P, L, P, P],
    "rlb_paged_decode_mma": [P, L, P, P, I, P, I, P, I, I, I, I, I, F, I, P, P, P, L, P, P],
    "rlb_sample": [P, I, L, I, I, P, P, P, F, I, F, I, U64, U64, P, P, P, P, P],
    "rlb_decode_advance": [P, P, P, P, P, P, P, P, I, P, P, P, P, I, P, P, I, I, P, I, I, P],
    "rlb_block_copy": [P, P, P, P, I, L, P],
    "rlb_gather_rows": [P, P, P, L, I, L, L, P],
}


class NativeLibraryError(RuntimeError):
    pass


def available() -> bool:
    """True when the shared object exists (it may still be unusable without a GPU)."""
    return _LIB_PATH.exists()


def _warn_if_stale() -> None:
    """The build records a hash of the native sources beside the library; when the sources have changed since, say so once
    (``RLB_STRICT_NATIVE=1``: refuse to run). The analogue of the reference's container fingerprint check at import
    (nemo_rl/__init__.py:98-229): the failure it guards against here is a library older than the code that calls it."""
    try:
        stamp = _LIB_PATH.with_name(_LIB_PATH.name + ".sources")
        if not stamp.exists():
            return
        from rl_b200.tools.fingerprint import source_hash

        built, now = stamp.read_text().strip(), source_hash()
        if built and built != now:
            msg = (f"{_LIB_PATH.name} was built from other sources (built {built}, sources now {now}): "
                   "rebuild with `python -m rl_b200.csrc.build`")
            if os.environ.get("RLB_STRICT_NATIVE", "0") == "1":
                raise NativeLibraryError(msg)
            import warnings

            warnings.warn(msg, RuntimeWarning, stacklevel=3)
    except NativeLibraryError:
        raise
    except Exception:
        pass


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise NativeLibraryError(
                f"{_LIB_PATH} is missing: build it with `python -m rl_b200.csrc.build` "
                "(the CUDA path never falls back to eager PyTorch)"
            )
        _lib = C.CDLL(str(_LIB_PATH))
        _warn_if_stale()
        for name, sig in list(_SIGS.items()):
            try:
                fn = getattr(_lib, name)
            except AttributeError:
                continue
            fn.argtypes = sig
            fn.restype = C.c_int
    return _lib


def register(name: str, sig: list[Any]) -> None:
    """Lets other modules (engine, comm) declare the entry points they bind."""
    _SIGS[name] = sig
    if _lib is not None and hasattr(_lib, name):
        fn = getattr(_lib, name)
        fn.argtypes = sig
        fn.restype = C.c_int


def ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def stream_ptr() -> int:
    return torch.cuda.current_stream().cuda_stream


_status_words: dict[int, torch.Tensor] = {}


def status_word(device: torch.device | int | None = None) -> torch.Tensor:
    """Per-device int32 that kernels with bounded waits write a code into when a wait runs out."""
    idx = torch.cuda.current_device() if device is None else torch.device(device).index or 0
    t = _status_words.get(idx)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}")
        _status_words[idx] = t
    return t


def check_status(device=None) -> int:
    """Reads (synchronously) and clears the status word. Non-zero: a kernel gave up a wait."""
    t = status_word(device)
    v = int(t.item())
    if v:
        t.zero_()
    return v


STATUS_NAMES = {1: "RLB_ERR_WAIT_FULL (a consumer waited for a TMA-filled stage)",
                2: "RLB_ERR_WAIT_EMPTY (a producer waited for a free stage)",
                3: "RLB_ERR_WAIT_TMEM_FULL (an epilogue waited for an accumulator)",
                4: "RLB_ERR_WAIT_TMEM_EMPTY (an MMA warp waited for a drained accumulator)",
                5: "RLB_ERR_WAIT_FLAG (a wait on a flag written by another CTA)",
                6: "RLB_ERR_BAD_ARG (a kernel refused its arguments)",
                7: "RLB_ERR_WAIT_PEER (a wait on a peer GPU's signal)",
                8: "RLB_ERR_BOUNDS (a debug-bounds build saw an index outside its buffer)"}


def raise_on_status(where: str, device=None) -> None:
    """Reads the status word where the host synchronises anyway (token download, gradient norm, end of a refit) and
    raises if a kernel gave up a bounded wait: its outputs are not to be trusted and the step must not continue."""
    if not torch.cuda.is_available():
        return
    code = check_status(device)
    if code:
        raise NativeLibraryError(f"{where}: a kernel reported status {code}: {STATUS_NAMES.get(code, 'unknown code')}; "
                                 "its outputs are incomplete (the CUDA context is still usable)")


class Counters:
    """Process-wide counts of native kernel launches and host<->device bytes, for benchmark reporting.

    ``launches`` counts every entry-point call that enqueues kernels; a CUDA-graph replay adds the number of calls
    that were recorded while the graph was captured (``graph_replayed``)."""

    launches = 0
    h2d_bytes = 0
    d2h_bytes = 0

    @classmethod
    def reset(cls) -> None:
        cls.launches = cls.h2d_bytes = cls.d2h_bytes = 0

    @classmethod
    def graph_replayed(cls, calls_in_graph: int) -> None:
        cls.launches += calls_in_graph


def call(name: str, *args) -> None:
    fn = getattr(lib(), name)
    rc = fn(*args)
    Counters.launches += 1
    if rc != 0:
        raise NativeLibraryError(f"{name} failed with code {rc}")


def to_device(t: torch.Tensor, device, non_blocking: bool = True) -> torch.Tensor:
    """Host -> device copy through pinned memory, counted in ``Counters.h2d_bytes``."""
    if t.device.type != "cpu" or torch.device(device).type == "cpu":
        return t.to(device)
    if not t.is_pinned():
        t = t.pin_memory()
    Counters.h2d_bytes += t.numel() * t.element_size()
    return t.to(device, non_blocking=non_blocking)


def to_host(t: torch.Tensor) -> torch.Tensor:
    """Device -> host copy, counted in ``Counters.d2h_bytes``."""
    if t.device.type == "cpu":
        return t
    Counters.d2h_bytes += t.numel() * t.element_size()
    return t.cpu()


def use_native(t: torch.Tensor) -> bool:
    """CUDA tensors run the native kernels; CPU tensors run the fp32 PyTorch restatement (the oracle)."""
    return t.is_cuda and os.environ.get("RLB_FORCE_REFERENCE_OPS", "0") != "1"
