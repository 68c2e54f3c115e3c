"""NVML helpers against a fake library, memory tracker, sparse weight deltas, stateless process group, refit verifier,
fingerprint."""

import threading
import types

import pytest
import torch

from rl_b200.utils import nvml as N
from rl_b200.utils.memory_tracker import MemoryTracker
from rl_b200.utils.sparse_delta import apply_delta, apply_state_delta, delta_stats, encode_delta, encode_state_delta


class FakeNVML:
    NVML_CLOCK_SM = 1

    def __init__(self):
        self.inits = self.shutdowns = 0
        self.calls = []

    def nvmlInit(self):
        self.inits += 1

    def nvmlShutdown(self):
        self.shutdowns += 1

    def nvmlDeviceGetHandleByIndex(self, i):
        self.calls.append(("handle", i))
        return ("h", i)

    def nvmlDeviceGetUUID(self, h):
        return f"GPU-fake-{h[1]}".encode()

    def nvmlDeviceGetName(self, h):
        return b"NVIDIA B200"

    def nvmlDeviceGetMemoryInfo(self, h):
        return types.SimpleNamespace(free=100 << 30, used=80 << 30, total=180 << 30)

    def nvmlDeviceGetClockInfo(self, h, which):
        return 1905

    def nvmlDeviceGetMaxClockInfo(self, h, which):
        return 1965

    def nvmlDeviceGetPowerUsage(self, h):
        return 987_000

    def nvmlDeviceGetCurrentClocksEventReasons(self, h):
        return 0x4 | 0x1


def test_nvml_helpers_only_read_and_always_shut_down(monkeypatch):
    lib = FakeNVML()
    monkeypatch.setenv("CUDA_VISIBLE_DEVICES", "3,5")
    assert N.get_device_uuid(1, lib) == "GPU-fake-5" and N.get_free_memory_bytes(0, lib) == 100 << 30
    snap = N.snapshot(0, lib)
    assert snap["sm_mhz"] == 1905 and snap["sm_max_mhz"] == 1965 and snap["reasons"] == ["sw_power_cap"] and snap["power_w"] == 987.0
    assert lib.inits == lib.shutdowns == 3
    assert not [m for m in dir(lib) if "Set" in m or "Reset" in m]       # the helpers need no setter
    with pytest.raises(ValueError):
        N.device_id_to_physical(2, "0,1")
    assert N.decode_throttle_reasons(0x8 | 0x40) == ["hw_slowdown", "hw_thermal_slowdown"]

    class Broken(FakeNVML):
        def nvmlDeviceGetUUID(self, h):
            raise RuntimeError("boom")

    b = Broken()
    with pytest.raises(RuntimeError):
        N.get_device_uuid(0, b)
    assert b.shutdowns == 1


def test_memory_tracker_table():
    mt = MemoryTracker()
    mt.snapshot_start_of_stage("setup")
    blob = bytearray(64 << 20)
    mt.snapshot_start_of_stage("train")
    d = mt.deltas()
    assert [x["stage"] for x in d] == ["setup", "train"] and d[0]["host_delta_gib"] is not None and d[1]["host_delta_gib"] is None
    assert "setup" in mt.table() and len(blob)


def test_sparse_delta_is_lossless_and_small():
    torch.manual_seed(0)
    old = torch.randn(512, 256).to(torch.bfloat16)
    same = encode_delta(old, old.clone())
    assert len(same) < 32 and torch.equal(apply_delta(old, same), old)
    few = old.clone()
    few.view(-1)[::997] += 0.5
    b = encode_delta(old, few)
    assert torch.equal(apply_delta(old, b).view(torch.int16), few.view(torch.int16)) and len(b) < old.numel() * 2 // 20
    step = (old.float() * (1 + 1e-3 * torch.randn(512, 256))).to(torch.bfloat16)     # a small optimizer step: low bits change
    b2 = encode_delta(old, step)
    assert torch.equal(apply_delta(old, b2).view(torch.int16), step.view(torch.int16)) and len(b2) < old.numel() * 2
    st_old, st_new = {"a": old, "b": torch.arange(10.0)}, {"a": step, "b": torch.arange(10.0) + 1}
    got = apply_state_delta({k: v.clone() for k, v in st_old.items()}, encode_state_delta(st_old, st_new))
    assert all(torch.equal(got[k], st_new[k]) for k in st_new) and delta_stats(st_old, st_new)["ratio"] > 1.0
    with pytest.raises(ValueError):
        apply_delta(old[:1], b2)


def test_stateless_process_group_over_tcp_store():
    import socket

    from rl_b200.distributed.stateless_group import StatelessProcessGroup

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    out = {}

    def member(rank):
        g = StatelessProcessGroup("127.0.0.1", port, rank, 3, timeout_s=30)
        uid = g.unique_id()
        got = g.all_gather_obj({"rank": rank})
        t = g.broadcast_tensor(torch.arange(6.0).view(2, 3) if rank == 1 else None, src=1)
        g.barrier()
        out[rank] = (uid, got, t, g)   # the group (rank 0 hosts the store) must outlive the slowest member

    ts = [threading.Thread(target=member, args=(r,)) for r in range(3)]
    [t.start() for t in ts]
    [t.join(60) for t in ts]
    assert len(out) == 3 and len({o[0] for o in out.values()}) == 1 and len(out[0][0]) == 128
    assert all([x["rank"] for x in o[1]] == [0, 1, 2] for o in out.values())
    assert all(torch.equal(o[2], torch.arange(6.0).view(2, 3)) for o in out.values())


def test_refit_verifier_and_fingerprint(tmp_path):
    import json

    from rl_b200.tools import fingerprint as fp
    from rl_b200.tools.refit_verifier import verify

    res = verify("tiny-llama-oracle", steps=2, batch=4, prompt_len=8, new_tokens=6, device="cpu")
    assert res["ok"] and all(abs(s["token_mult_prob_error"] - 1) < 1e-3 for s in res["steps"])
    a = fp.fingerprint()
    assert a["torch"] == torch.__version__ and len(a["native_sources"]) == 16 and fp.compare(a, dict(a)) == {}
    p = tmp_path / "other.json"
    p.write_text(json.dumps(dict(a, torch="0.0")))
    assert fp.main(["--compare", str(p)]) == 1


def test_model_diagnostics(tmp_path, capsys):
    from rl_b200.models import hf_io
    from rl_b200.models.config import preset
    from rl_b200.models.transformer import build_model
    from rl_b200.tools import model_diagnostics as md

    assert md.main(["decode-vs-prefill", "--device", "cpu", "--new-tokens", "48"]) == 0
    assert md.main(["max-len", "--device", "cpu"]) == 0
    m = build_model(preset("tiny-llama-oracle", torch_dtype="float32"), dtype=torch.float32, seed=0)
    with torch.no_grad():
        m.embed_tokens[5].zero_()
    hf_io.save_pretrained(m, str(tmp_path))
    assert md.main(["embeddings", "--path", str(tmp_path)]) == 1
    out = capsys.readouterr().out
    assert '"zero_rows": [5]' in out and '"check": "max-len"' in out


def test_perf_numbers_from_a_metrics_log(tmp_path):
    import json

    from rl_b200.tools import perf_numbers as P

    with open(tmp_path / "metrics.jsonl", "w") as f:
        for step in range(1, 11):
            f.write(json.dumps({"step": step, "timing/train/total_step_time": 10.0 + step, "train/loss": 0.1}) + "\n")
            f.write(json.dumps({"step": step, "performance/tokens_per_sec_per_gpu": 1000.0 * step, "note": "text"}) + "\n")
    m = P.read_metrics(str(tmp_path))
    assert sorted(m) == list(range(1, 11)) and m[3]["performance/tokens_per_sec_per_gpu"] == 3000.0 and "note" not in m[3]
    assert list(P.window(6, 5)) == [4, 5, 6, 7, 8] and list(P.window(6, 4)) == [4, 5, 6, 7]
    s = P.summarize(m, at_step=6, average_steps=5)
    assert s["steps"] == [4, 5, 6, 7, 8] and s["averages"]["timing/train/total_step_time"] == 16.0
    assert s["averages"]["performance/tokens_per_sec_per_gpu"] == 6000.0 and "timing/train/generation" not in s["averages"]
    with pytest.raises(ValueError):
        P.summarize(m, at_step=50)
    assert P.main([str(tmp_path), "--at-step", "3", "--average-steps", "2", "--json"]) == 0


def test_model_diagnostics_sub_commands_on_cpu():
    from rl_b200.tools import model_diagnostics as D

    assert D.precision("tiny-llama-oracle", "cpu", new_tokens=16)["ok"]
    r = D.prefix_caching("tiny-llama-oracle", "cpu")
    assert r["ok"] and r["cached_prefix_tokens"] > 0
    assert D.routed_experts("cpu")["ok"]


def test_small_tools(tmp_path, capsys):
    import os

    import torch

    from rl_b200.tools import benchmark_tokenizer, check_r3_trace, code_snapshot, find_available_port_ranges

    # routing record against a capture: identical sets in any order agree; -1 rows do not count; a bent row is found
    rec = torch.tensor([[[0, 1], [2, 3]], [[4, 5], [6, 7]], [[-1, -1], [-1, -1]]], dtype=torch.int16)     # [T=3, layers=2, k=2]
    cap = torch.tensor([[[1, 0], [2, 3]], [[4, 5], [7, 1]], [[0, 1], [2, 3]]], dtype=torch.int16)
    r = check_r3_trace.compare(rec, {0: cap[:, 0], 1: cap[:, 1]})
    assert r["layers"][0]["agreement"] == 1.0 and r["layers"][1]["agreement"] == 0.5 and r["recorded_positions"] == 4
    assert abs(r["layers"][0]["unrecorded_fraction"] - 1 / 3) < 1e-9
    torch.save(rec, tmp_path / "a.pt")
    torch.save(rec, tmp_path / "b.pt")
    assert check_r3_trace.main(["--record", str(tmp_path / "a.pt"), "--capture", str(tmp_path / "b.pt")]) == 0
    # free port runs from a fake probe
    busy = {1030, 1031, 1040}
    assert find_available_port_ranges.free_ranges(1028, 1042, probe=lambda p, h: p not in busy) == [(1028, 1029), (1032, 1039), (1041, 1042)]
    # tokenizer throughput numbers
    from rl_b200.data.tokenizers import ByteTokenizer

    b = benchmark_tokenizer.benchmark(ByteTokenizer(), benchmark_tokenizer.synthetic_docs(20, 30), batch=4)
    assert b["tokens"] > 0 and b["encode_tokens_per_s"] > 0 and b["chat_templates_per_s"] > 0
    # a snapshot holds the sources and is re-used by name
    src = tmp_path / "proj"
    (src / "pkg").mkdir(parents=True)
    (src / "pkg" / "a.py").write_text("x = 1\n")
    (src / "data.bin").write_bytes(b"\0")
    snap = code_snapshot.snapshot("exp1", str(src))
    assert (tmp_path / "proj" / "code_snapshots" / "exp1" / "pkg" / "a.py").exists() and not os.path.exists(os.path.join(snap, "data.bin"))
    (src / "pkg" / "a.py").write_text("x = 2\n")
    assert code_snapshot.snapshot("exp1", str(src)) == snap and open(os.path.join(snap, "pkg", "a.py")).read() == "x = 1\n"


def test_stale_native_library_is_reported(tmp_path, monkeypatch):
    from rl_b200.ops import lib as L
    from rl_b200.tools.fingerprint import source_hash

    fake = tmp_path / "_C.so"
    fake.write_bytes(b"")
    monkeypatch.setattr(L, "_LIB_PATH", fake)
    L._warn_if_stale()                                           # no record beside the library: nothing to compare
    (tmp_path / "_C.so.sources").write_text(source_hash())
    import warnings

    with warnings.catch_warnings():
        warnings.simplefilter("error")
        L._warn_if_stale()                                       # built from the current sources: silent
    (tmp_path / "_C.so.sources").write_text("0123456789abcdef")
    with pytest.warns(RuntimeWarning, match="rebuild"):
        L._warn_if_stale()
    monkeypatch.setenv("RLB_STRICT_NATIVE", "1")
    with pytest.raises(L.NativeLibraryError):
        L._warn_if_stale()
