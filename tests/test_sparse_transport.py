"""Sparse-delta refit transports: payload format, sender pipeline, TCP relay tree, HTTP fan-out, object store + manifest."""

import json

import pytest
import torch

from rl_b200.refit import sparse_transport as ST


def _states(seed=0, n=6):
    g = torch.Generator().manual_seed(seed)
    old = {f"layers.{i}.w": torch.randn(64, 48, generator=g).to(torch.bfloat16) for i in range(n)}
    old["norm"] = torch.ones(48, dtype=torch.bfloat16)
    new = {k: v.clone() for k, v in old.items()}
    for i in range(0, n, 2):   # an optimizer step touches few low bits of some tensors and leaves others alone
        m = torch.rand(64, 48, generator=g) < 0.05
        new[f"layers.{i}.w"][m] += 0.01
    return old, new


def test_payload_round_trip_and_checksum():
    old, new = _states()
    items = [(k, ST.encode_delta(old[k], new[k])) for k in new]
    buf = ST.pack_payload("t0", 3, items)
    header, got = ST.unpack_payload(buf)
    assert header["transfer_id"] == "t0" and header["seq"] == 3 and [n for n, _ in got] == list(new)
    state = {k: v.clone() for k, v in old.items()}
    ST.apply_payload(state, buf)
    assert all(torch.equal(state[k], new[k]) for k in new)
    bad = bytearray(buf)
    bad[-1] ^= 0xFF
    with pytest.raises(ValueError, match="checksum"):
        ST.unpack_payload(bad)
    with pytest.raises(ValueError, match="malformed"):
        ST.unpack_payload(buf[:-3])


def test_pipeline_buckets_and_updates_the_baseline():
    old, new = _states()
    baseline = ST.init_baseline(old.items())
    sent = []
    stats = ST.stream_sparse_delta_payloads(new.items(), baseline, lambda p, info: sent.append((info["seq"], p)) or info["seq"], "t1",
                                            bucket_bytes=300, encode_workers=3, send_workers=2)
    assert stats["tensors"] == len(new) and stats["payloads"] == len(sent) >= 2 and stats["unchanged_tensors"] >= 4
    assert stats["compression"] > 3 and sorted(stats["replies"]) == list(range(stats["payloads"]))
    state = {k: v.clone() for k, v in old.items()}
    for _, p in sorted(sent):
        ST.apply_payload(state, p)
    assert all(torch.equal(state[k], new[k]) for k in new)
    assert all(torch.equal(baseline[k], new[k]) for k in new)       # the next refit is a delta against what was sent


def test_tcp_relay_tree_applies_on_every_node():
    old, new = _states(1)
    states = [{k: v.clone() for k, v in old.items()} for _ in range(3)]
    servers = [ST.TcpRefitServer(s) for s in states]
    addrs = [s.start() for s in servers]
    servers[0].configure_tree([addrs[1], addrs[2]])                 # root relays to two leaves
    try:
        baseline = ST.init_baseline(old.items())
        stats = ST.stream_via_tcp(new.items(), baseline, [addrs[0]], "t2", bucket_bytes=400)
        assert stats["ok"] and stats["flush"][0]["applied"] == stats["payloads"] and len(stats["flush"][0]["children"]) == 2
        for s in states:
            assert all(torch.equal(s[k], new[k]) for k in new)
        # a corrupted payload is refused and reported; the server keeps running
        c = ST.TcpRefitClient(*addrs[1])
        bad = bytearray(ST.pack_payload("t3", 0, [("norm", ST.encode_delta(new["norm"], new["norm"]))]))
        bad[-1] ^= 1
        with pytest.raises(RuntimeError, match="rejected"):
            c.send_payload(bytes(bad))
        assert c.flush("t2", stats["payloads"], 1.0)["ok"] is False   # the node remembers the error
        assert c.flush("nothing", 1, 0.2)["error"] == "timeout"
        c.close()
    finally:
        for s in servers:
            s.close()


def test_http_fan_out_and_metrics(monkeypatch):
    old, new = _states(2)
    servers = {u: {k: v.clone() for k, v in old.items()} for u in ("http://a:1", "http://b:2/")}
    seen_headers = []

    def post(url, data, headers, timeout):
        base = url.split("/refit")[0]
        state = servers[base if base in servers else base + "/"]
        h = ST.apply_payload(state, data)
        seen_headers.append(headers)
        return dict(applied=1, bytes=len(data), seq=h["seq"])

    assert ST.refit_endpoints(["http://a:1", "http://b:2/"], "/refit/sparse") == ["http://a:1/refit/sparse", "http://b:2/refit/sparse"]
    with pytest.raises(KeyError):
        ST.refit_api_key("RLB_TEST_NO_SUCH_KEY")
    monkeypatch.setenv("RLB_TEST_KEY", "secret")
    tr = ST.SparseRefitTransport(kind="http", endpoints=list(servers), api_key_env_var="RLB_TEST_KEY", bucket_bytes=500)
    stats = ST.stream_via_http(new.items(), ST.init_baseline(old.items()), tr, "t4", post=post)
    assert stats["servers"]["servers"] == 2 * stats["payloads"] and stats["servers"]["applied_sum"] == 2 * stats["payloads"]
    assert all(h["Authorization"] == "Bearer secret" for h in seen_headers)
    for s in servers.values():
        assert all(torch.equal(s[k], new[k]) for k in new)


def test_object_store_manifest(tmp_path):
    old, new = _states(3)
    store = ST.FileObjectStore(str(tmp_path / "bucket"))
    stats = ST.stream_via_manifest(new.items(), ST.init_baseline(old.items()), store, "t5", bucket_bytes=350)
    man = json.loads(bytes(store.get(stats["manifest"])))
    assert [e["seq"] for e in man["payloads"]] == list(range(stats["payloads"]))
    state = {k: v.clone() for k, v in old.items()}
    assert ST.apply_manifest(state, store, stats["manifest"]) == stats["payloads"]
    assert all(torch.equal(state[k], new[k]) for k in new)
    # a tampered object is caught by the manifest's checksum
    k0 = man["payloads"][0]["key"]
    body = store.get(k0)
    body[-1] ^= 1
    store.put(k0, bytes(body))
    with pytest.raises(ValueError, match="checksum"):
        list(ST.download_refit_payloads(store, stats["manifest"]))
    stats["cleanup"]()
    with pytest.raises(FileNotFoundError):
        store.get(stats["manifest"])
    with pytest.raises(ValueError):
        store.put("../escape", b"x")


def test_weight_synchronizer_factory_and_sparse_sender(tmp_path):
    """The factory names every way of moving weights; the sparse sender streams successive refits as deltas against what the
    receiver holds (the second refit sends only what the optimizer step changed)."""
    from rl_b200.models.config import ModelConfig
    from rl_b200.models.hf_io import iter_hf_tensors
    from rl_b200.models.transformer import build_model
    from rl_b200.refit.factory import ColocatedHandoff, SparseDeltaSynchronizer, create_weight_synchronizer

    mc = ModelConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                     head_dim=8, torch_dtype="bfloat16")
    train = build_model(mc, dtype=torch.bfloat16, seed=1)
    h = create_weight_synchronizer("colocated", train)
    assert isinstance(h, ColocatedHandoff) and h.serving_model is train and h.sync_weights() is None
    with pytest.raises(ValueError):
        create_weight_synchronizer("carrier_pigeon", train)
    receiver = {n: t.detach().clone() for n, t in iter_hf_tensors(train)}
    store = ST.FileObjectStore(str(tmp_path / "bucket"))
    sync = create_weight_synchronizer("sparse_object_store", train, store_dir=str(tmp_path / "bucket"), bucket_bytes=4096)
    assert isinstance(sync, SparseDeltaSynchronizer)
    s0 = sync.sync_weights()                       # nothing changed since the baseline: all-zero deltas
    assert s0["unchanged_tensors"] == s0["tensors"] and ST.apply_manifest(receiver, store, s0["manifest"]) == s0["payloads"]
    with torch.no_grad():
        for n, p in train.named_parameters():
            if n.endswith("down_proj"):
                p.add_(0.01)
    s1 = sync.sync_weights()
    assert 0 < s1["tensors"] - s1["unchanged_tensors"] <= 2 and s1["manifest"] != s0["manifest"]
    ST.apply_manifest(receiver, store, s1["manifest"])
    for n, t in iter_hf_tensors(train):
        assert torch.equal(receiver[n], t.detach()), n


def test_value_model_facade():
    from rl_b200.distributed.batched_data_dict import BatchedDataDict
    from rl_b200.models.config import ModelConfig
    from rl_b200.policy.value import ValueModel

    mc = ModelConfig(vocab_size=64, hidden_size=32, intermediate_size=64, num_hidden_layers=1, num_attention_heads=4, num_key_value_heads=2,
                     head_dim=8, torch_dtype="float32")
    vm = ValueModel(dict(precision="float32", train_global_batch_size=2, train_micro_batch_size=2, max_total_sequence_length=32,
                         optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=1e-3))), model_cfg=mc)
    data = BatchedDataDict(input_ids=torch.randint(0, 64, (2, 9)), input_lengths=torch.tensor([9, 5]))
    out = vm.get_values(data)
    assert out["values"].shape == (2, 9) and out["scores"].shape == (2,)
    assert not hasattr(vm, "generate") and not hasattr(vm, "get_logprobs")
