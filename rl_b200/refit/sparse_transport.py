"""Sparse-delta refit over slow links: the weight update of a generation fleet that does not share NVLink with the trainer
(other nodes, another cluster, object storage in between).

The sender keeps a baseline (the weights the receivers currently hold), encodes ``new XOR baseline`` tensor by tensor with
the lossless codec of :mod:`rl_b200.utils.sparse_delta`, packs the encoded tensors into payloads of bounded size, and
streams them through a transport while later tensors are still being encoded (encode, serialise and send run in a
thread pipeline). Every payload carries a SHA-256 checksum. Receivers apply the deltas to their own copy, which then
equals the sender's bit for bit. Three transports:

* **TCP** (:class:`TcpRefitServer` / :class:`TcpRefitClient`): length-prefixed frames over sockets; servers can be arranged in
  a relay tree (each forwards what it receives to its children), and ``flush`` waits until a transfer's payloads have
  been applied on the whole subtree. Plays the role of the ZeroMQ relay of nemo_rl/utils/weight_transfer_zmq.py:68-550
  (pyzmq is not part of this image).
* **HTTP** (:func:`post_refit_endpoints`): the payloads are POSTed in parallel to the refit endpoint of every generation
  server (nemo_rl/utils/weight_transfer_http.py:45-135).
* **Object store + manifest** (:func:`stream_via_manifest`): payloads are written as objects, a manifest names them with
  their checksums, receivers download and apply (the S3 path of nemo_rl/utils/weight_transfer_stream.py:100-168, :506-606).
  :class:`FileObjectStore` keeps objects in a directory (a shared file system); an S3 client with the same three methods
  can be passed instead.

The pipeline itself follows ``stream_sparse_delta_payloads`` (weight_transfer_stream.py:266-504).
"""

from __future__ import annotations

import hashlib
import json
import os
import socket
import struct
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from dataclasses import dataclass, field
from typing import Any, Callable, Iterable, Iterator, Optional, Sequence

import torch

from rl_b200.utils.sparse_delta import apply_delta, encode_delta

_HDR = struct.Struct("<4sIQ")      # magic, header bytes, body bytes
_MAGIC = b"RLBP"


@dataclass
class SparseRefitTransport:
    """How a sparse refit travels. ``kind``: tcp | http | object_store."""

    kind: str = "tcp"
    endpoints: list = field(default_factory=list)     # tcp: (host, port) pairs of the tree roots; http: base urls
    path: str = "/refit/sparse"
    api_key_env_var: Optional[str] = None
    store_dir: Optional[str] = None
    bucket_bytes: int = 64 << 20
    encode_workers: int = 4
    send_workers: int = 4
    compression_level: int = 1


# ------------------------------------------------------------------------------------------------ payloads
def payload_checksum(body: bytes | bytearray) -> str:
    return hashlib.sha256(body).hexdigest()


def pack_payload(transfer_id: str, seq: int, items: Sequence[tuple[str, bytes]]) -> bytes:
    """One payload: a JSON header (transfer id, sequence number, names and sizes, checksum of the body) + the bodies."""
    body = b"".join(b for _, b in items)
    header = json.dumps(dict(transfer_id=transfer_id, seq=seq, names=[n for n, _ in items], sizes=[len(b) for _, b in items],
                             checksum=payload_checksum(body))).encode()
    return _HDR.pack(_MAGIC, len(header), len(body)) + header + body


def unpack_payload(buf: bytes | bytearray) -> tuple[dict, list[tuple[str, bytes]]]:
    magic, hl, bl = _HDR.unpack_from(buf, 0)
    if magic != _MAGIC or len(buf) != _HDR.size + hl + bl:
        raise ValueError("malformed refit payload")
    header = json.loads(bytes(buf[_HDR.size : _HDR.size + hl]))
    body = bytes(buf[_HDR.size + hl :])
    if payload_checksum(body) != header["checksum"]:
        raise ValueError(f"refit payload {header.get('transfer_id')}#{header.get('seq')} failed its checksum")
    items, at = [], 0
    for n, s in zip(header["names"], header["sizes"]):
        items.append((n, body[at : at + s]))
        at += s
    return header, items


def apply_payload(state: dict[str, torch.Tensor], buf: bytes | bytearray) -> dict:
    """Verifies and applies one payload to ``state`` in place; returns its header."""
    header, items = unpack_payload(buf)
    for name, blob in items:
        cur = state[name]
        new = apply_delta(cur, blob)
        if cur.data_ptr() != new.data_ptr():
            cur.copy_(new)
    return header


# ------------------------------------------------------------------------------------------------ sender pipeline
def stream_sparse_delta_payloads(named_tensors: Iterable[tuple[str, torch.Tensor]], baseline: dict[str, torch.Tensor],
                                 send: Callable[[bytes, dict], Any], transfer_id: str, bucket_bytes: int = 64 << 20,
                                 encode_workers: int = 4, send_workers: int = 4, level: int = 1, update_baseline: bool = True) -> dict:
    """Encodes every tensor against ``baseline`` (thread pool), groups the encoded tensors into payloads of about
    ``bucket_bytes`` and hands each to ``send(payload, header_info)`` on a second pool while encoding continues. After a
    tensor is encoded the baseline takes its new value, so the next refit is a delta against what the receivers hold.
    Returns counts and byte totals."""
    t0 = time.perf_counter()
    stats = dict(tensors=0, payloads=0, raw_bytes=0, sent_bytes=0, unchanged_tensors=0)
    enc_pool, send_pool = ThreadPoolExecutor(max(1, encode_workers)), ThreadPoolExecutor(max(1, send_workers))
    pending_send = []
    bucket: list[tuple[str, bytes]] = []
    size = 0

    def flush():
        nonlocal bucket, size
        if not bucket:
            return
        payload = pack_payload(transfer_id, stats["payloads"], bucket)
        info = dict(seq=stats["payloads"], tensors=len(bucket), bytes=len(payload))
        stats["payloads"] += 1
        stats["sent_bytes"] += len(payload)
        pending_send.append(send_pool.submit(send, payload, info))
        bucket, size = [], 0

    def encode(name, t):
        cpu = t.detach().to("cpu")
        blob = encode_delta(baseline[name], cpu, level)
        if update_baseline:
            baseline[name] = cpu.clone()
        return name, blob, cpu.numel() * cpu.element_size()

    window: list = []
    try:
        for name, t in named_tensors:
            window.append(enc_pool.submit(encode, name, t))
            while len(window) >= 2 * max(1, encode_workers):       # keep the pipeline shallow: encoded blobs are memory
                n, blob, raw = window.pop(0).result()
                stats["tensors"] += 1
                stats["raw_bytes"] += raw
                stats["unchanged_tensors"] += int(len(blob) <= 22)
                bucket.append((n, blob))
                size += len(blob)
                if size >= bucket_bytes:
                    flush()
        for fut in window:
            n, blob, raw = fut.result()
            stats["tensors"] += 1
            stats["raw_bytes"] += raw
            stats["unchanged_tensors"] += int(len(blob) <= 22)
            bucket.append((n, blob))
            size += len(blob)
            if size >= bucket_bytes:
                flush()
        flush()
        stats["replies"] = [f.result() for f in pending_send]
    finally:
        enc_pool.shutdown(wait=True)
        send_pool.shutdown(wait=True)
    stats["seconds"] = time.perf_counter() - t0
    stats["compression"] = stats["raw_bytes"] / max(1, stats["sent_bytes"])
    return stats


def init_baseline(named_tensors: Iterable[tuple[str, torch.Tensor]]) -> dict[str, torch.Tensor]:
    """The first refit of a fleet is a full transfer by other means; the sender records what was sent as its baseline."""
    return {n: t.detach().to("cpu").clone() for n, t in named_tensors}


# ------------------------------------------------------------------------------------------------ TCP relay
def _send_frame(sock: socket.socket, kind: bytes, body: bytes) -> None:
    sock.sendall(struct.pack("<cQ", kind, len(body)) + body)


def _recv_exact(sock: socket.socket, n: int) -> bytearray:
    buf = bytearray(n)
    view, got = memoryview(buf), 0
    while got < n:
        r = sock.recv_into(view[got:], n - got)
        if r == 0:
            raise ConnectionError("peer closed the connection")
        got += r
    return buf


def _recv_frame(sock: socket.socket) -> tuple[bytes, bytearray]:
    head = _recv_exact(sock, 9)
    kind, n = struct.unpack("<cQ", bytes(head))
    return kind, _recv_exact(sock, n)


class TcpRefitServer:
    """Receives payloads, applies them to ``state`` and forwards them to its children in the relay tree. Frames: ``D`` data
    (a payload), ``F`` flush request (JSON: transfer id, expected payload count) answered with a JSON report once this node
    and all its children have applied that many payloads of the transfer."""

    def __init__(self, state: dict[str, torch.Tensor], host: str = "127.0.0.1", port: int = 0, on_applied: Optional[Callable[[dict], None]] = None):
        self.state, self.on_applied = state, on_applied
        self._sock = socket.socket(socket.AF_INET, socket.SOCK_STREAM)
        self._sock.setsockopt(socket.SOL_SOCKET, socket.SO_REUSEADDR, 1)
        self._sock.bind((host, port))
        self._sock.listen(16)
        self.address = self._sock.getsockname()
        self.children: list[TcpRefitClient] = []
        self.applied: dict[str, int] = {}
        self.bytes_in = 0
        self.errors: list[str] = []
        self._cv = threading.Condition()
        self._stop = False
        self._thread: Optional[threading.Thread] = None

    def configure_tree(self, children: Sequence[tuple[str, int]]) -> None:
        self.children = [TcpRefitClient(h, p) for h, p in children]

    def start(self) -> tuple[str, int]:
        self._thread = threading.Thread(target=self._accept_loop, daemon=True)
        self._thread.start()
        return self.address

    def _accept_loop(self) -> None:
        self._sock.settimeout(0.2)
        while not self._stop:
            try:
                conn, _ = self._sock.accept()
            except socket.timeout:
                continue
            except OSError:
                break
            threading.Thread(target=self._serve, args=(conn,), daemon=True).start()

    def _serve(self, conn: socket.socket) -> None:
        try:
            while not self._stop:
                try:
                    kind, body = _recv_frame(conn)
                except ConnectionError:
                    return
                if kind == b"D":
                    try:
                        header = apply_payload(self.state, body)
                        for ch in self.children:
                            ch.send_payload(bytes(body))
                        with self._cv:
                            self.applied[header["transfer_id"]] = self.applied.get(header["transfer_id"], 0) + 1
                            self.bytes_in += len(body)
                            self._cv.notify_all()
                        if self.on_applied is not None:
                            self.on_applied(header)
                        _send_frame(conn, b"A", json.dumps(dict(ok=True, seq=header["seq"])).encode())
                    except Exception as e:   # a bad payload is reported to the sender, the server stays up
                        self.errors.append(f"{type(e).__name__}: {e}")
                        _send_frame(conn, b"A", json.dumps(dict(ok=False, error=str(e))).encode())
                elif kind == b"F":
                    req = json.loads(bytes(body))
                    _send_frame(conn, b"R", json.dumps(self.flush(req["transfer_id"], int(req.get("expected_payloads", 0)),
                                                                  float(req.get("timeout_s", 60.0)))).encode())
        finally:
            conn.close()

    def flush(self, transfer_id: str, expected_payloads: int = 0, timeout_s: float = 60.0) -> dict:
        deadline = time.monotonic() + timeout_s
        with self._cv:
            while self.applied.get(transfer_id, 0) < expected_payloads:
                left = deadline - time.monotonic()
                if left <= 0:
                    return dict(ok=False, applied=self.applied.get(transfer_id, 0), expected=expected_payloads, error="timeout")
                self._cv.wait(left)
            mine = self.applied.get(transfer_id, 0)
        kids = [ch.flush(transfer_id, expected_payloads, max(0.1, deadline - time.monotonic())) for ch in self.children]
        return dict(ok=all(k.get("ok") for k in kids) and not self.errors, applied=mine, bytes_in=self.bytes_in, children=kids,
                    errors=list(self.errors))

    def close(self) -> None:
        self._stop = True
        for ch in self.children:
            ch.close()
        try:
            self._sock.close()
        except OSError:
            pass


class TcpRefitClient:
    def __init__(self, host: str, port: int, timeout_s: float = 60.0):
        self.addr = (host, port)
        self.timeout_s = timeout_s
        self._sock: Optional[socket.socket] = None
        self._lock = threading.Lock()

    def _conn(self) -> socket.socket:
        if self._sock is None:
            self._sock = socket.create_connection(self.addr, timeout=self.timeout_s)
            self._sock.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        return self._sock

    def send_payload(self, payload: bytes, info: Optional[dict] = None) -> dict:
        with self._lock:
            s = self._conn()
            _send_frame(s, b"D", payload)
            _, body = _recv_frame(s)
        rep = json.loads(bytes(body))
        if not rep.get("ok"):
            raise RuntimeError(f"receiver {self.addr} rejected a refit payload: {rep.get('error')}")
        return rep

    def flush(self, transfer_id: str, expected_payloads: int, timeout_s: float = 60.0) -> dict:
        with self._lock:
            s = self._conn()
            _send_frame(s, b"F", json.dumps(dict(transfer_id=transfer_id, expected_payloads=expected_payloads, timeout_s=timeout_s)).encode())
            _, body = _recv_frame(s)
        return json.loads(bytes(body))

    def close(self) -> None:
        if self._sock is not None:
            try:
                self._sock.close()
            except OSError:
                pass
            self._sock = None


def stream_via_tcp(named_tensors, baseline, roots: Sequence[tuple[str, int]], transfer_id: str, **kw) -> dict:
    """Streams a sparse refit to the roots of one or more relay trees and waits until every tree has applied it."""
    clients = [TcpRefitClient(h, p) for h, p in roots]

    def send(payload: bytes, info: dict):
        return [c.send_payload(payload, info) for c in clients]

    try:
        stats = stream_sparse_delta_payloads(named_tensors, baseline, send, transfer_id, **kw)
        stats["flush"] = [c.flush(transfer_id, stats["payloads"]) for c in clients]
        stats["ok"] = all(f.get("ok") for f in stats["flush"])
        return stats
    finally:
        for c in clients:
            c.close()


# ------------------------------------------------------------------------------------------------ HTTP
def refit_endpoints(base_urls: Sequence[str], path: str) -> list[str]:
    return [u.rstrip("/") + "/" + path.lstrip("/") for u in base_urls]


def refit_api_key(api_key_env_var: Optional[str]) -> Optional[str]:
    if not api_key_env_var:
        return None
    key = os.environ.get(api_key_env_var)
    if not key:
        raise KeyError(f"environment variable {api_key_env_var} (the generation servers' API key) is not set")
    return key


def post_refit_endpoints(urls: Sequence[str], payload: bytes, api_key: Optional[str] = None, workers: int = 8, timeout_s: float = 120.0,
                         post: Optional[Callable] = None) -> list[dict]:
    """POSTs one payload to every endpoint in parallel; returns the servers' JSON replies. ``post(url, data, headers,
    timeout)`` can be injected (tests, other HTTP stacks); the default uses ``requests``."""
    headers = {"Content-Type": "application/octet-stream"}
    if api_key:
        headers["Authorization"] = f"Bearer {api_key}"
    if post is None:
        import requests

        session = requests.Session()

        def post(url, data, headers, timeout):
            r = session.post(url, data=data, headers=headers, timeout=timeout)
            r.raise_for_status()
            return r.json()

    with ThreadPoolExecutor(max(1, min(workers, len(urls)))) as ex:
        return list(ex.map(lambda u: post(u, payload, headers, timeout_s), urls))


def merge_refit_metrics(replies: Iterable[dict]) -> dict:
    out: dict[str, float] = {}
    n = 0
    for r in replies:
        n += 1
        for k, v in r.items():
            if isinstance(v, (int, float)) and not isinstance(v, bool):
                out[k + "_sum"] = out.get(k + "_sum", 0.0) + v
                out[k + "_max"] = max(out.get(k + "_max", float("-inf")), v)
    out["servers"] = float(n)
    return out


def stream_via_http(named_tensors, baseline, transport: SparseRefitTransport, transfer_id: str, post: Optional[Callable] = None, **kw) -> dict:
    urls = refit_endpoints(transport.endpoints, transport.path)
    key = refit_api_key(transport.api_key_env_var)
    replies: list[dict] = []

    def send(payload: bytes, info: dict):
        rs = post_refit_endpoints(urls, payload, key, transport.send_workers, post=post)
        replies.extend(rs)
        return rs

    stats = stream_sparse_delta_payloads(named_tensors, baseline, send, transfer_id, bucket_bytes=transport.bucket_bytes,
                                         encode_workers=transport.encode_workers, send_workers=transport.send_workers,
                                         level=transport.compression_level, **kw)
    stats["servers"] = merge_refit_metrics(replies)
    return stats


# ------------------------------------------------------------------------------------------------ object store + manifest
class FileObjectStore:
    """put / get / delete of named objects in a directory (a shared file system standing in for a bucket)."""

    def __init__(self, root: str):
        self.root = root
        os.makedirs(root, exist_ok=True)

    def _p(self, key: str) -> str:
        p = os.path.join(self.root, key)
        if os.path.commonpath([os.path.abspath(p), os.path.abspath(self.root)]) != os.path.abspath(self.root):
            raise ValueError(f"object key escapes the store: {key}")
        return p

    def put(self, key: str, body: bytes) -> None:
        p = self._p(key)
        os.makedirs(os.path.dirname(p), exist_ok=True)
        tmp = p + ".part"
        with open(tmp, "wb") as f:
            f.write(body)
        os.replace(tmp, p)      # readers never see a half-written object

    def get(self, key: str) -> bytearray:
        with open(self._p(key), "rb") as f:
            return bytearray(f.read())

    def delete(self, key: str) -> None:
        try:
            os.remove(self._p(key))
        except FileNotFoundError:
            pass


def stream_via_manifest(named_tensors, baseline, store, transfer_id: str, prefix: str = "refit", **kw) -> dict:
    """Writes the payloads as objects ``<prefix>/<transfer>/<seq>.bin`` and, last, the manifest
    ``<prefix>/<transfer>/manifest.json`` that names them with their checksums. Returns the stats with ``cleanup()`` under
    ``"cleanup"`` (deletes the objects once every receiver is done)."""
    entries: list[dict] = []
    lock = threading.Lock()

    def send(payload: bytes, info: dict):
        key = f"{prefix}/{transfer_id}/{info['seq']:06d}.bin"
        store.put(key, payload)
        with lock:
            entries.append(dict(key=key, seq=info["seq"], bytes=len(payload), checksum=payload_checksum(payload)))
        return key

    stats = stream_sparse_delta_payloads(named_tensors, baseline, send, transfer_id, **kw)
    entries.sort(key=lambda e: e["seq"])
    mkey = f"{prefix}/{transfer_id}/manifest.json"
    store.put(mkey, json.dumps(dict(transfer_id=transfer_id, payloads=entries)).encode())
    stats["manifest"] = mkey

    def cleanup():
        for e in entries:
            store.delete(e["key"])
        store.delete(mkey)

    stats["cleanup"] = cleanup
    return stats


def download_refit_payloads(store, manifest_key: str) -> Iterator[bytearray]:
    man = json.loads(bytes(store.get(manifest_key)))
    for e in man["payloads"]:
        body = store.get(e["key"])
        if payload_checksum(body) != e["checksum"]:
            raise ValueError(f"object {e['key']} does not match the manifest's checksum")
        yield body


def apply_manifest(state: dict[str, torch.Tensor], store, manifest_key: str) -> int:
    n = 0
    for body in download_refit_payloads(store, manifest_key):
        apply_payload(state, body)
        n += 1
    return n
