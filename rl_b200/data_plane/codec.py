"""Wire format of data-plane records and the batch <-> records conversion.

A record is a dict of named fields. Tensors are stored as (dtype, shape, raw bytes); everything else is pickled. Jagged
batches (rows of different lengths, right-padded in a ``BatchedDataDict``) are cut to their true lengths before they are
stored and padded again on the consumer, so padding never crosses the store (the reference's codec for jagged fields:
nemo_rl/data_plane/codec.py:133-250).
"""

from __future__ import annotations

import io
import pickle
import struct
from typing import Any, Optional, Sequence

import numpy as np
import torch

from rl_b200.distributed.batched_data_dict import BatchedDataDict

_MAGIC = b"RLBR1"
_NP = {torch.float32: np.float32, torch.float64: np.float64, torch.float16: np.float16, torch.int64: np.int64, torch.int32: np.int32,
       torch.int16: np.int16, torch.int8: np.int8, torch.uint8: np.uint8, torch.bool: np.bool_}


def _tensor_bytes(t: torch.Tensor) -> tuple[str, bytes]:
    t = t.detach().cpu().contiguous()
    if t.dtype == torch.bfloat16:                      # numpy has no bfloat16: ship the 16-bit patterns
        return "bfloat16", t.view(torch.int16).numpy().tobytes()
    return str(t.dtype).replace("torch.", ""), t.numpy().tobytes()


def _tensor_from(dtype: str, shape: Sequence[int], raw: bytes) -> torch.Tensor:
    if dtype == "bfloat16":
        return torch.frombuffer(bytearray(raw), dtype=torch.int16).view(torch.bfloat16).reshape(tuple(shape)).clone()
    td = getattr(torch, dtype)
    return torch.frombuffer(bytearray(raw), dtype=td).reshape(tuple(shape)).clone() if raw else torch.empty(tuple(shape), dtype=td)


def encode_record(record: dict[str, Any]) -> bytes:
    head, blobs = [], []
    for name, v in record.items():
        if isinstance(v, torch.Tensor):
            dt, raw = _tensor_bytes(v)
            head.append((name, "t", dt, tuple(v.shape), len(raw)))
        else:
            raw = pickle.dumps(v, protocol=4)
            head.append((name, "p", "", (), len(raw)))
        blobs.append(raw)
    h = pickle.dumps(head, protocol=4)
    return _MAGIC + struct.pack("<I", len(h)) + h + b"".join(blobs)


def decode_record(buf: bytes, fields: Optional[set] = None) -> dict[str, Any]:
    if buf[:5] != _MAGIC:
        raise ValueError("not a data-plane record")
    (hl,) = struct.unpack_from("<I", buf, 5)
    head = pickle.loads(buf[9 : 9 + hl])
    off, out = 9 + hl, {}
    for name, kind, dt, shape, n in head:
        if fields is None or name in fields:
            raw = buf[off : off + n]
            out[name] = _tensor_from(dt, shape, raw) if kind == "t" else pickle.loads(raw)
        off += n
    return out


def record_fields(buf: bytes) -> list[str]:
    (hl,) = struct.unpack_from("<I", buf, 5)
    return [h[0] for h in pickle.loads(buf[9 : 9 + hl])]


def batch_to_records(batch: BatchedDataDict, length_key: str = "input_lengths", jagged: Optional[Sequence[str]] = None) -> list[dict[str, Any]]:
    """One record per row. A 2-D+ tensor field whose second dimension equals the padded length is cut to the row's true
    length (or list it in ``jagged`` explicitly); other tensors are stored per row as they are."""
    n = batch.size
    lens = batch[length_key].tolist() if length_key in batch else None
    padded = int(max(lens)) if lens else 0
    recs = [dict() for _ in range(n)]
    for name, v in batch.items():
        if isinstance(v, torch.Tensor):
            is_jag = lens is not None and v.dim() >= 2 and ((jagged is not None and name in jagged) or (jagged is None and v.shape[1] >= padded > 0 and name != length_key))
            for i in range(n):
                recs[i][name] = v[i, : lens[i]].clone() if is_jag else v[i].clone()
            if is_jag:
                for i in range(n):
                    recs[i].setdefault("__jagged__", []).append(name)
        else:
            for i in range(n):
                recs[i][name] = v[i]
    return recs


def records_to_batch(records: Sequence[dict[str, Any]], pad_values: Optional[dict[str, Any]] = None) -> BatchedDataDict:
    """Stacks records into a right-padded batch (jagged fields padded with ``pad_values[name]``, default 0)."""
    pad_values = pad_values or {}
    out: dict[str, Any] = {}
    if not records:
        return BatchedDataDict(out)
    names = [k for k in records[0] if k != "__jagged__"]
    jag = set(records[0].get("__jagged__", []))
    for name in names:
        vals = [r[name] for r in records]
        if isinstance(vals[0], torch.Tensor):
            if name in jag:
                L = max(v.shape[0] for v in vals)
                buf = torch.full((len(vals), L) + tuple(vals[0].shape[1:]), pad_values.get(name, 0), dtype=vals[0].dtype)
                for i, v in enumerate(vals):
                    buf[i, : v.shape[0]] = v
                out[name] = buf
            else:
                out[name] = torch.stack(vals)
        else:
            out[name] = list(vals)
    return BatchedDataDict(out)
