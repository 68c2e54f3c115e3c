from .adapters.local import LocalDataPlane
from .adapters.tcp_store import TCPStoreDataPlane
from .codec import batch_to_records, decode_record, encode_record, records_to_batch
from .interfaces import DataPlaneClient, SampleMeta
from .observability import ObservedDataPlane
from .preshard import preshard


def create_data_plane(cfg=None, store=None) -> DataPlaneClient:
    """``cfg.backend``: ``local`` (default) or ``tcp_store`` (needs ``store`` or ``cfg.host`` / ``cfg.port`` / ``cfg.is_server``)."""
    cfg = dict(cfg or {})
    backend = cfg.get("backend", "local")
    if cfg.pop("observe", False):
        return ObservedDataPlane(create_data_plane(cfg, store))
    if backend in ("local", "noop"):
        return LocalDataPlane(cfg.get("capacity_bytes"))
    if backend == "tcp_store":
        if store is None:
            from datetime import timedelta

            import torch.distributed as dist

            store = dist.TCPStore(cfg.get("host", "127.0.0.1"), int(cfg["port"]), None, bool(cfg.get("is_server", False)),
                                  timeout=timedelta(seconds=float(cfg.get("timeout_s", 60))), wait_for_workers=False)
        return TCPStoreDataPlane(store, cfg.get("namespace", "dp"))
    raise ValueError(f"unknown data plane backend {backend!r}")
