"""Virtual cluster: which GPUs (bundles) of which nodes a job may use, how they are handed to worker groups, and where the
job's ranks meet. Role of nemo_rl/distributed/virtual_cluster.py (``RayVirtualCluster``: placement groups of GPU bundles per
node, ``max_colocated_worker_groups`` groups sharing the same GPUs, master address / port discovery, GPU sets split between
training and inference) without a cluster manager underneath: a bundle is (node index, local GPU index); workers on the
driver's node are child processes, workers on other nodes are started there by the launcher (Slurm, ssh) and join the driver
over TCP (``rl_b200/distributed/worker_groups.py``).
"""

from __future__ import annotations

import os
import socket
from dataclasses import dataclass, field
from typing import Optional, Sequence


class ResourceInsufficientError(RuntimeError):
    """The node list cannot supply the bundles that were asked for."""


@dataclass(frozen=True)
class Bundle:
    node: int          # index into the cluster's node list
    gpu: int           # local GPU index on that node (-1: a CPU-only slot)


def free_port(host: str = "127.0.0.1") -> int:
    with socket.socket() as s:
        s.bind((host, 0))
        return int(s.getsockname()[1])


def visible_gpu_count() -> int:
    try:
        import torch

        return int(torch.cuda.device_count()) if torch.cuda.is_available() else 0
    except Exception:
        return 0


@dataclass
class VirtualCluster:
    """``bundle_ct_per_node_list[i]`` slots on node i. ``use_gpus`` binds slot j of a node to its GPU j (checked against the
    driver node's GPU count for node 0); ``max_colocated_worker_groups`` worker groups may be placed on the same bundles
    (policy and generation sharing GPUs)."""

    bundle_ct_per_node_list: Sequence[int]
    use_gpus: bool = True
    num_gpus_per_node: Optional[int] = None
    max_colocated_worker_groups: int = 1
    name: str = ""
    node_addresses: Optional[Sequence[str]] = None        # host name / IP per node; node 0 is the driver's node
    _groups_placed: int = field(default=0, repr=False)
    _port: Optional[int] = field(default=None, repr=False)

    def __post_init__(self):
        self.bundle_ct_per_node_list = [int(x) for x in self.bundle_ct_per_node_list]
        if not self.bundle_ct_per_node_list or any(x <= 0 for x in self.bundle_ct_per_node_list):
            raise ValueError("every node of a virtual cluster needs at least one bundle")
        if self.node_addresses is None:
            self.node_addresses = ["127.0.0.1"] * len(self.bundle_ct_per_node_list)
        if len(self.node_addresses) != len(self.bundle_ct_per_node_list):
            raise ValueError("one address per node is required")
        per_node = self.num_gpus_per_node
        if self.use_gpus:
            if per_node is None:
                per_node = max(self.bundle_ct_per_node_list)
            if max(self.bundle_ct_per_node_list) > per_node:
                raise ResourceInsufficientError(f"{max(self.bundle_ct_per_node_list)} bundles asked of a node with {per_node} GPUs")
            have = visible_gpu_count()
            if have and self.bundle_ct_per_node_list[0] > have:
                raise ResourceInsufficientError(f"node 0 has {have} GPUs, {self.bundle_ct_per_node_list[0]} bundles were asked for")
        self.num_gpus_per_node = per_node

    # ------------------------------------------------------------------ shape
    def world_size(self) -> int:
        return sum(self.bundle_ct_per_node_list)

    def node_count(self) -> int:
        return len(self.bundle_ct_per_node_list)

    def bundles(self) -> list[Bundle]:
        """All slots in rank order: node after node, GPU after GPU."""
        return [Bundle(n, g if self.use_gpus else -1) for n, ct in enumerate(self.bundle_ct_per_node_list) for g in range(ct)]

    # ------------------------------------------------------------------ rendezvous
    def get_master_address_and_port(self) -> tuple[str, int]:
        """Where the ranks of a worker group placed on this cluster meet (``MASTER_ADDR`` / ``MASTER_PORT``): node 0, one
        fresh port per call site that asks (worker groups ask once each)."""
        addr = self.node_addresses[0]
        return addr, free_port("127.0.0.1" if addr in ("127.0.0.1", "localhost") else "")

    def get_available_address_and_port(self, node: int = 0) -> tuple[str, int]:
        return self.node_addresses[node], free_port("127.0.0.1" if self.node_addresses[node] in ("127.0.0.1", "localhost") else "")

    # ------------------------------------------------------------------ placement of worker groups
    def claim_group(self) -> int:
        """Registers one more worker group on these bundles; more than ``max_colocated_worker_groups`` is an error."""
        if self._groups_placed >= self.max_colocated_worker_groups:
            raise ResourceInsufficientError(f"cluster '{self.name}' already hosts {self._groups_placed} worker group(s) "
                                            f"(max_colocated_worker_groups={self.max_colocated_worker_groups})")
        self._groups_placed += 1
        return self._groups_placed - 1

    def release_group(self) -> None:
        self._groups_placed = max(0, self._groups_placed - 1)

    def split(self, first: int) -> tuple["VirtualCluster", "VirtualCluster"]:
        """Two disjoint clusters: the first ``first`` bundles (rank order) and the rest, e.g. training and inference GPU sets
        of a non-colocated job. The second cluster's GPU indices continue where the first one's end on a shared node."""
        b = self.bundles()
        if not 0 < first < len(b):
            raise ValueError("split point must leave bundles on both sides")
        return _SubCluster(self, b[:first], self.name + ":0"), _SubCluster(self, b[first:], self.name + ":1")

    def shutdown(self) -> bool:
        self._groups_placed = 0
        return True


class _SubCluster(VirtualCluster):
    """A cluster over an explicit subset of another cluster's bundles."""

    def __init__(self, parent: VirtualCluster, bundles: list[Bundle], name: str):
        nodes = sorted({b.node for b in bundles})
        self._bundles = [Bundle(nodes.index(b.node), b.gpu) for b in bundles]
        counts = [sum(1 for b in bundles if b.node == n) for n in nodes]
        super().__init__(counts, use_gpus=False, num_gpus_per_node=parent.num_gpus_per_node,
                         max_colocated_worker_groups=parent.max_colocated_worker_groups, name=name,
                         node_addresses=[parent.node_addresses[n] for n in nodes])
        self.use_gpus = parent.use_gpus

    def bundles(self) -> list[Bundle]:
        return list(self._bundles)


@dataclass(frozen=True)
class NodeInfo:
    """What the launcher knows about a node: address, free GPUs and the NVLink domain it sits in (GPUs of one domain -- an
    NVL72 rack, an HGX board -- reach each other without leaving NVLink; None: unknown, a domain of its own)."""

    address: str
    gpus: int
    nvlink_domain: Optional[str] = None


def place_on_nodes(nodes: Sequence[NodeInfo], num_nodes: int, gpus_per_node: int) -> list[NodeInfo]:
    """Chooses ``num_nodes`` nodes with at least ``gpus_per_node`` GPUs each so that the job spans as few NVLink domains as
    possible, and orders them domain by domain (ranks that talk most -- consecutive ranks -- then share a domain). Domains are
    taken largest first; ties and the order inside a domain follow the node addresses, so the choice is reproducible.
    Role of the topology-aware sort of nemo_rl/distributed/virtual_cluster.py."""
    ok = [n for n in nodes if n.gpus >= gpus_per_node]
    if len(ok) < num_nodes:
        raise ResourceInsufficientError(f"{num_nodes} nodes with {gpus_per_node} GPUs were asked for, {len(ok)} of {len(nodes)} qualify")
    by_domain: dict = {}
    for n in sorted(ok, key=lambda n: n.address):
        by_domain.setdefault(n.nvlink_domain if n.nvlink_domain is not None else f"\0{n.address}", []).append(n)
    whole = sorted(by_domain.items(), key=lambda kv: (-len(kv[1]), kv[0]))
    # a single domain that can hold the whole job wins (the smallest such, to leave large domains for large jobs)
    fits = [kv for kv in whole if len(kv[1]) >= num_nodes]
    if fits:
        return list(min(fits, key=lambda kv: (len(kv[1]), kv[0]))[1][:num_nodes])
    out: list[NodeInfo] = []
    for _, members in whole:
        out += members[: num_nodes - len(out)]
        if len(out) == num_nodes:
            break
    return out


def cluster_from_nodes(nodes: Sequence[NodeInfo], num_nodes: int, gpus_per_node: int, **kw) -> VirtualCluster:
    chosen = place_on_nodes(nodes, num_nodes, gpus_per_node)
    return VirtualCluster([gpus_per_node] * num_nodes, num_gpus_per_node=gpus_per_node, node_addresses=[n.address for n in chosen], **kw)


def cluster_from_config(cluster_cfg: dict, colocated_groups: int = 2, name: str = "cluster") -> VirtualCluster:
    """``cluster: {gpus_per_node, num_nodes}`` of a recipe -> the job's cluster (node addresses from ``RLB_NODE_ADDRESSES``, a
    comma-separated list the launcher exports on multi-node jobs)."""
    g, n = int(cluster_cfg.get("gpus_per_node", 1)), int(cluster_cfg.get("num_nodes", 1))
    addrs = os.environ.get("RLB_NODE_ADDRESSES")
    return VirtualCluster([g] * n, use_gpus=visible_gpu_count() > 0, num_gpus_per_node=g, max_colocated_worker_groups=colocated_groups,
                          name=name, node_addresses=addrs.split(",") if addrs else None)
