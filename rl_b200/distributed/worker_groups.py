"""Worker groups: a driver process creates one worker process per bundle of a :class:`VirtualCluster`, calls methods on all
or some of them with replicated, per-worker or sharded arguments, and collects the results. Role of
nemo_rl/distributed/worker_groups.py (``RayWorkerBuilder``, ``RayWorkerGroup`` with ``run_all_workers_single_data`` /
``run_all_workers_multiple_data`` / ``run_all_workers_sharded_data``, ``MultiWorkerFuture``) with a native control plane in
place of Ray actors:

* every worker process connects back to the driver's listener (``multiprocessing.connection`` over TCP with an
  authentication key) and then serves calls ONE AT A TIME in arrival order, like an actor; results and exceptions travel
  back tagged with the call's id and complete a ``concurrent.futures.Future`` on the driver;
* workers on the driver's node are spawned children; workers on other nodes are started there by the launcher with
  ``python -m rl_b200.distributed.worker_groups --join HOST:PORT --rank R`` and join the same listener;
* each worker gets RANK / WORLD_SIZE / LOCAL_RANK / MASTER_ADDR / MASTER_PORT of its group, so the object it hosts can form
  its ``torch.distributed`` groups (NCCL / gloo) with its peers: bulk tensors move between workers over those, the control
  plane carries arguments and results only.
"""

from __future__ import annotations

import concurrent.futures as cf
import importlib
import multiprocessing as mp
import os
import secrets
import threading
import traceback
from multiprocessing.connection import Client, Listener
from typing import Any, Optional, Sequence

from rl_b200.distributed.named_sharding import NamedSharding
from rl_b200.distributed.virtual_cluster import VirtualCluster


class WorkerError(RuntimeError):
    """A call failed inside a worker; carries the worker's traceback."""

    def __init__(self, rank: int, method: str, tb: str):
        super().__init__(f"worker {rank} failed in {method}():\n{tb}")
        self.rank, self.method, self.remote_traceback = rank, method, tb


def _resolve(fqn_or_cls):
    if not isinstance(fqn_or_cls, str):
        return fqn_or_cls
    mod, _, name = fqn_or_cls.rpartition(".")
    return getattr(importlib.import_module(mod), name)


class WorkerBuilder:
    """What to construct inside each worker process: a class (or its fully qualified name) and its arguments."""

    def __init__(self, worker_class, *init_args, **init_kwargs):
        self.worker_class, self.init_args, self.init_kwargs = worker_class, init_args, init_kwargs

    def build(self):
        return _resolve(self.worker_class)(*self.init_args, **self.init_kwargs)


# ------------------------------------------------------------------------------------------------ worker side
def _serve(conn, rank: int, builder: WorkerBuilder) -> None:
    obj, err = None, None
    try:
        obj = builder.build()
    except BaseException:
        err = traceback.format_exc()
    conn.send(("ready", rank, err))
    while err is None:
        try:
            msg = conn.recv()
        except (EOFError, OSError):
            break
        call_id, method, args, kwargs = msg
        if method == "__shutdown__":
            cleanup = args[0] if args else None
            if cleanup and hasattr(obj, cleanup):
                try:
                    getattr(obj, cleanup)()
                except BaseException:
                    pass
            conn.send((call_id, True, None))
            break
        try:
            out = getattr(obj, method)(*args, **kwargs)
            conn.send((call_id, True, out))
        except BaseException:
            conn.send((call_id, False, traceback.format_exc()))
    try:
        conn.close()
    except OSError:
        pass


def _worker_main(address, authkey: bytes, rank: int, env: dict, builder: WorkerBuilder) -> None:
    os.environ.update({k: str(v) for k, v in env.items()})
    conn = Client(address, authkey=authkey)
    conn.send(("hello", rank))
    _serve(conn, rank, builder)


# ------------------------------------------------------------------------------------------------ driver side
class _WorkerHandle:
    def __init__(self, rank: int, conn, proc, meta: dict):
        self.rank, self.conn, self.proc, self.meta = rank, conn, proc, meta
        self._pending: dict[int, tuple[cf.Future, str]] = {}
        self._lock = threading.Lock()
        self._next = 0
        self._reader = threading.Thread(target=self._read, daemon=True, name=f"worker-{rank}-reader")
        self._reader.start()

    def _read(self) -> None:
        while True:
            try:
                call_id, ok, payload = self.conn.recv()
            except (EOFError, OSError):
                with self._lock:
                    pend, self._pending = self._pending, {}
                for fut, method in pend.values():
                    if not fut.done():
                        fut.set_exception(WorkerError(self.rank, method, "the worker's connection closed before it answered"))
                return
            with self._lock:
                fut, method = self._pending.pop(call_id, (None, ""))
            if fut is None:
                continue
            if ok:
                fut.set_result(payload)
            else:
                fut.set_exception(WorkerError(self.rank, method, payload))

    def call(self, method: str, *args, **kwargs) -> cf.Future:
        fut: cf.Future = cf.Future()
        with self._lock:
            call_id = self._next
            self._next += 1
            self._pending[call_id] = (fut, method)
            self.conn.send((call_id, method, args, kwargs))     # under the lock: calls reach the worker in issue order
        return fut


class MultiWorkerFuture:
    """Futures of one group call, the workers that were called and the workers whose results count."""

    def __init__(self, futures: list, called_workers: list[int], return_from_workers: Optional[list[int]] = None):
        self.futures, self.called_workers = futures, called_workers
        self.return_from_workers = return_from_workers

    def get_results(self, group=None, timeout: Optional[float] = None) -> list[Any]:
        results = [f.result(timeout=timeout) for f in self.futures]      # wait for every call, report the first failure
        if self.return_from_workers is None:
            return results
        keep = set(self.return_from_workers)
        return [r for r, w in zip(results, self.called_workers) if w in keep]


class WorkerGroup:
    """One worker per bundle of ``cluster``; worker i is rank i of the group. ``sharding_annotations`` names the axes of the
    rank layout (e.g. pipeline / data / context / tensor parallel) for :meth:`run_all_workers_sharded_data`."""

    def __init__(self, cluster: VirtualCluster, builder: WorkerBuilder, name: str = "workers", sharding_annotations: Optional[NamedSharding] = None,
                 env_vars: Optional[dict] = None, start_timeout_s: float = 600.0, remote_nodes_join: bool = False):
        self.cluster, self.name, self.sharding_annotations = cluster, name, sharding_annotations
        cluster.claim_group()
        bundles = cluster.bundles()
        self.world = len(bundles)
        if sharding_annotations is not None and sharding_annotations.size != self.world:
            raise ValueError(f"sharding annotations cover {sharding_annotations.size} ranks, the cluster has {self.world} bundles")
        addr, port = cluster.get_master_address_and_port()
        # (multi-node jobs export RLB_WORKER_AUTHKEY, a hex string, on every node so that joining workers can authenticate)
        self._authkey = bytes.fromhex(os.environ["RLB_WORKER_AUTHKEY"]) if os.environ.get("RLB_WORKER_AUTHKEY") else secrets.token_bytes(16)
        listen_host = "127.0.0.1" if cluster.node_count() == 1 else ""
        self._listener = Listener((listen_host, 0), authkey=self._authkey)
        self.address = (cluster.node_addresses[0], self._listener.address[1])
        ctx = mp.get_context("spawn")
        procs: dict[int, Any] = {}
        metas: dict[int, dict] = {}
        # workers of one node share its cores: without a limit every worker's math library starts a thread per core
        threads = os.environ.get("OMP_NUM_THREADS") or str(max(1, (os.cpu_count() or 1) // max(1, max(cluster.bundle_ct_per_node_list))))
        for rank, b in enumerate(bundles):
            env = dict(OMP_NUM_THREADS=threads)
            env.update(env_vars or {})
            env.update(RANK=rank, WORLD_SIZE=self.world, LOCAL_RANK=max(b.gpu, 0) if cluster.use_gpus else rank, MASTER_ADDR=addr, MASTER_PORT=port,
                       RLB_WORKER_GROUP=name, RLB_NODE_RANK=b.node)
            metas[rank] = dict(rank=rank, node=b.node, gpu=b.gpu, env=env)
            if b.node == 0 or not remote_nodes_join:
                p = ctx.Process(target=_worker_main, args=(("127.0.0.1", self.address[1]), self._authkey, rank, env, builder), daemon=True,
                                name=f"{name}-{rank}")
                p.start()
                procs[rank] = p
        self._remote_builder = builder
        # every worker says hello with its rank (children and joiners alike), then reports that its object is built
        conns: dict[int, Any] = {}
        self._listener._listener._socket.settimeout(start_timeout_s)
        try:
            while len(conns) < self.world:
                c = self._listener.accept()
                kind, rank = c.recv()
                if kind == "join":       # a worker started by the launcher on another node: hand it its environment and builder
                    c.send((metas[rank]["env"], builder))
                    kind, rank = c.recv()
                assert kind == "hello"
                conns[rank] = c
            for rank, c in conns.items():
                kind, r, err = c.recv()
                if err is not None:
                    raise WorkerError(rank, "__init__", err)
        except BaseException:
            for p in procs.values():
                if p.is_alive():
                    p.terminate()
            self._listener.close()
            cluster.release_group()
            raise
        self._workers = [_WorkerHandle(r, conns[r], procs.get(r), metas[r]) for r in range(self.world)]
        self._closed = False

    # ------------------------------------------------------------------ introspection
    @property
    def workers(self) -> list[_WorkerHandle]:
        return self._workers

    @property
    def worker_metadata(self) -> list[dict]:
        return [w.meta for w in self._workers]

    @property
    def dp_size(self) -> int:
        sa = self.sharding_annotations
        return sa.get_axis_size("data_parallel") if sa is not None and "data_parallel" in sa.names else self.world

    def get_dp_leader_worker_idx(self, dp_shard_idx: int) -> int:
        """The worker at coordinate 0 of every other axis for this data-parallel index."""
        sa = self.sharding_annotations
        if sa is None:
            return dp_shard_idx
        return int(sa.get_ranks(**{n: (dp_shard_idx if n == "data_parallel" else 0) for n in sa.names}))

    # ------------------------------------------------------------------ calls
    def run_single_worker_single_data(self, method_name: str, worker_idx: int, *args, **kwargs) -> cf.Future:
        return self._workers[worker_idx].call(method_name, *args, **kwargs)

    def _rank0_only(self, worker_idx: int, axes: Optional[Sequence[str]]) -> bool:
        """Whether ``worker_idx`` is skipped because it is not at index 0 of one of ``axes``."""
        if not axes or self.sharding_annotations is None:
            return False
        c = self.sharding_annotations.get_worker_coords(worker_idx)
        return any(c.get(a, 0) != 0 for a in axes)

    def run_all_workers_single_data(self, method_name: str, *args, run_rank_0_only_axes: Optional[Sequence[str]] = None, **kwargs) -> list[cf.Future]:
        """The same arguments to every worker (or only to those at index 0 of the named axes)."""
        return [w.call(method_name, *args, **kwargs) for i, w in enumerate(self._workers) if not self._rank0_only(i, run_rank_0_only_axes)]

    def run_all_workers_multiple_data(self, method_name: str, *args, run_rank_0_only_axes: Optional[Sequence[str]] = None,
                                      common_kwargs: Optional[dict] = None, **kwargs) -> list[cf.Future]:
        """Every positional / keyword argument is a list with one entry per worker."""
        for a in list(args) + list(kwargs.values()):
            if len(a) != self.world:
                raise ValueError(f"per-worker arguments need {self.world} entries, got {len(a)}")
        futs = []
        for i, w in enumerate(self._workers):
            if self._rank0_only(i, run_rank_0_only_axes):
                continue
            futs.append(w.call(method_name, *[a[i] for a in args], **{k: v[i] for k, v in kwargs.items()}, **(common_kwargs or {})))
        return futs

    def run_all_workers_sharded_data(self, method_name: str, *, in_sharded_axes: Optional[list[str]] = None,
                                     replicate_on_axes: Optional[list[str]] = None, output_is_replicated: Optional[list[str]] = None,
                                     make_dummy_calls_to_free_axes: bool = False, common_kwargs: Optional[dict] = None, **kwargs) -> MultiWorkerFuture:
        """Keyword arguments are nested lists indexed by the coordinates along ``in_sharded_axes`` (in that order); a worker gets
        the entry at its coordinates. Along ``replicate_on_axes`` every worker gets that same entry. Along the remaining (free)
        axes only index 0 is called (the others get a call with ``None`` arguments when ``make_dummy_calls_to_free_axes``).
        Results come from the workers at index 0 of the free axes and of ``output_is_replicated``, in rank order."""
        sa = self.sharding_annotations
        if sa is None:
            raise ValueError("sharding annotations are required for sharded dispatch")
        in_sharded_axes, replicate_on_axes = list(in_sharded_axes or []), list(replicate_on_axes or [])
        output_is_replicated = list(output_is_replicated or [])
        for ax in in_sharded_axes + replicate_on_axes + output_is_replicated:
            if ax not in sa.names:
                raise ValueError(f"axis '{ax}' is not one of {sa.names}")
        both = set(in_sharded_axes) & set(replicate_on_axes)
        if both:
            raise ValueError(f"axes cannot be both sharded and replicated: {sorted(both)}")
        futures, called, returning = [], [], []
        for i, w in enumerate(self._workers):
            c = sa.get_worker_coords(i)
            free = [a for a in sa.names if a not in in_sharded_axes and a not in replicate_on_axes]
            gets_data = all(c[a] == 0 for a in free)
            if gets_data and all(c[a] == 0 for a in output_is_replicated):
                returning.append(i)
            if gets_data:
                kw = kwargs
                for ax in in_sharded_axes:
                    kw = {k: v[c[ax]] for k, v in kw.items()}
                futures.append(w.call(method_name, **kw, **(common_kwargs or {})))
                called.append(i)
            elif make_dummy_calls_to_free_axes:
                futures.append(w.call(method_name, **{k: None for k in kwargs}, **(common_kwargs or {})))
                called.append(i)
        return MultiWorkerFuture(futures, called, returning)

    def get_all_worker_results(self, future_bundle, timeout: Optional[float] = None) -> list[Any]:
        if isinstance(future_bundle, MultiWorkerFuture):
            return future_bundle.get_results(self, timeout)
        return [f.result(timeout=timeout) for f in future_bundle]

    # ------------------------------------------------------------------ end of life
    def shutdown(self, cleanup_method: Optional[str] = None, timeout: float = 30.0, force: bool = False) -> bool:
        """Asks every worker to run ``cleanup_method`` (if it has one) and leave; workers that do not leave within ``timeout``
        seconds (or all of them at once with ``force``) are terminated. Only processes this group started are touched."""
        if self._closed:
            return True
        self._closed = True
        ok = True
        futs = []
        if not force:
            for w in self._workers:
                try:
                    futs.append(w.call("__shutdown__", cleanup_method))
                except (OSError, ValueError):
                    ok = False
            for f in futs:
                try:
                    f.result(timeout=timeout)
                except Exception:
                    ok = False
        for w in self._workers:
            if w.proc is not None:
                w.proc.join(timeout=0 if force else timeout)
                if w.proc.is_alive():
                    w.proc.terminate()
                    w.proc.join(timeout=5)
                    ok = False if not force else ok
            try:
                w.conn.close()
            except OSError:
                pass
        self._listener.close()
        self.cluster.release_group()
        return ok

    def __del__(self):
        try:
            self.shutdown(force=True)
        except Exception:
            pass


def join_main(argv=None) -> int:
    """Entry point of a worker started by the launcher on a node other than the driver's: connects, receives its environment
    and what to build, then serves calls like a local worker."""
    import argparse

    ap = argparse.ArgumentParser()
    ap.add_argument("--join", required=True, help="HOST:PORT of the driver's listener")
    ap.add_argument("--rank", type=int, required=True)
    ap.add_argument("--authkey-env", default="RLB_WORKER_AUTHKEY", help="environment variable holding the hex authentication key")
    a = ap.parse_args(argv)
    host, _, port = a.join.rpartition(":")
    conn = Client((host, int(port)), authkey=bytes.fromhex(os.environ[a.authkey_env]))
    conn.send(("join", a.rank))
    env, builder = conn.recv()
    os.environ.update({k: str(v) for k, v in env.items()})
    conn.send(("hello", a.rank))
    _serve(conn, a.rank, builder)
    return 0


if __name__ == "__main__":
    raise SystemExit(join_main())
