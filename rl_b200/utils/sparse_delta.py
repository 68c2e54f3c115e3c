"""Sparse weight deltas for refit over slow links (another node, object storage): after one optimizer step most bf16
weights change in a few low bits or not at all, so ``new XOR old`` is mostly zero bytes and compresses well. The codec
is lossless: ``apply_delta(old, encode_delta(old, new)) == new`` bit for bit. Role of
nemo_rl/utils/weight_transfer_sparse_codec.py (xor-delta + zstd); zlib stands in for zstd, which this image lacks."""

from __future__ import annotations

import struct
import zlib
from typing import Iterable, Iterator

import numpy as np
import torch

_MAGIC = b"RLBD1"


def _bits(t: torch.Tensor) -> np.ndarray:
    t = t.detach().contiguous().cpu()
    return t.view(torch.uint8).numpy().reshape(-1)


def encode_delta(old: torch.Tensor, new: torch.Tensor, level: int = 1) -> bytes:
    assert old.shape == new.shape and old.dtype == new.dtype
    x = np.bitwise_xor(_bits(old), _bits(new))
    nz = int(np.count_nonzero(x))
    if nz == 0:
        return _MAGIC + struct.pack("<BQQ", 0, x.size, 0)
    if nz * 16 < x.size < 2**32:   # very sparse: gap-coded positions + values beat compressing the zero runs
        idx = np.flatnonzero(x)
        gaps = np.diff(idx, prepend=0).astype(np.uint32)
        body = zlib.compress(gaps.tobytes() + x[idx].tobytes(), level)
        return _MAGIC + struct.pack("<BQQ", 1, x.size, nz) + body
    return _MAGIC + struct.pack("<BQQ", 2, x.size, nz) + zlib.compress(x.tobytes(), level)


def apply_delta(old: torch.Tensor, blob: bytes) -> torch.Tensor:
    if blob[:5] != _MAGIC:
        raise ValueError("not a weight delta")
    mode, size, nz = struct.unpack_from("<BQQ", blob, 5)
    base = _bits(old).copy()
    if base.size != size:
        raise ValueError(f"delta is for {size} bytes, tensor has {base.size}")
    if mode == 1:
        raw = zlib.decompress(blob[22:])
        gaps = np.frombuffer(raw[: 4 * nz], dtype=np.uint32).astype(np.int64)
        vals = np.frombuffer(raw[4 * nz :], dtype=np.uint8)
        base[np.cumsum(gaps)] ^= vals
    elif mode == 2:
        base ^= np.frombuffer(zlib.decompress(blob[22:]), dtype=np.uint8)
    return torch.from_numpy(base).view(old.dtype).reshape(old.shape).to(old.device)


def encode_state_delta(old: dict, new: dict, level: int = 1) -> Iterator[tuple[str, bytes]]:
    for name, t in new.items():
        yield name, encode_delta(old[name], t, level)


def apply_state_delta(state: dict, deltas: Iterable[tuple[str, bytes]]) -> dict:
    for name, blob in deltas:
        state[name] = apply_delta(state[name], blob)
    return state


def delta_stats(old: dict, new: dict) -> dict:
    raw = sum(t.numel() * t.element_size() for t in new.values())
    enc = sum(len(b) for _, b in encode_state_delta(old, new))
    return dict(raw_bytes=raw, delta_bytes=enc, ratio=raw / max(1, enc))
