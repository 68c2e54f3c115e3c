"""Data plane (codec, adapters, pre-sharding) and the single-controller GRPO loop built on it."""

import pytest
import torch

from rl_b200.algorithms import grpo
from rl_b200.algorithms.single_controller import ControllerStalled, SingleController
from rl_b200.data.datasets.synthetic import RandomTokenPromptDataset
from rl_b200.data_plane import (LocalDataPlane, SampleMeta, TCPStoreDataPlane, batch_to_records, create_data_plane, decode_record,
                                encode_record, preshard, records_to_batch)
from rl_b200.distributed.batched_data_dict import BatchedDataDict
from rl_b200.environments.synthetic import TokenFractionEnv
from rl_b200.models.config import ModelConfig


def test_codec_round_trip_and_field_selection():
    rec = {"ids": torch.arange(7), "lp": torch.randn(7).to(torch.bfloat16), "flag": torch.tensor(True), "empty": torch.zeros(0, dtype=torch.float32),
           "text": "héllo", "obj": {"a": [1, 2]}}
    buf = encode_record(rec)
    out = decode_record(buf)
    assert out["text"] == "héllo" and out["obj"] == {"a": [1, 2]} and out["empty"].shape == (0,)
    assert torch.equal(out["ids"], rec["ids"]) and torch.equal(out["lp"], rec["lp"]) and out["lp"].dtype == torch.bfloat16
    assert set(decode_record(buf, {"ids"})) == {"ids"}
    with pytest.raises(ValueError):
        decode_record(b"garbage-bytes")


def test_jagged_batch_round_trip_drops_padding():
    lens = torch.tensor([3, 5, 1])
    ids = torch.zeros(3, 5, dtype=torch.long)
    for i, n in enumerate(lens.tolist()):
        ids[i, :n] = torch.arange(1, n + 1)
    b = BatchedDataDict(input_ids=ids, input_lengths=lens, token_mask=(ids > 0).float(), reward=torch.tensor([1.0, 0.0, 2.0]), name=["a", "b", "c"])
    recs = batch_to_records(b)
    assert [r["input_ids"].numel() for r in recs] == [3, 5, 1] and recs[2]["name"] == "c"
    back = records_to_batch(recs[:2][::-1], pad_values={"input_ids": -1})
    assert back["input_ids"].tolist() == [[1, 2, 3, 4, 5], [1, 2, 3, -1, -1]] and back["reward"].tolist() == [0.0, 1.0]
    assert back["name"] == ["b", "a"]


class _FakeStore:
    """The subset of TCPStore the adapter uses."""

    def __init__(self):
        self.d = {}

    def set(self, k, v):
        self.d[k] = bytes(v)

    def get(self, k):
        return self.d[k]

    def add(self, k, n):
        self.d[k] = int(self.d.get(k, 0)) + n
        return self.d[k]

    def check(self, ks):
        return all(k in self.d for k in ks)

    def delete_key(self, k):
        return self.d.pop(k, None) is not None


@pytest.mark.parametrize("make", [lambda: LocalDataPlane(), lambda: TCPStoreDataPlane(_FakeStore())])
def test_adapters_put_get_update_delete(make):
    dp = make()
    for i in range(4):
        dp.put(f"traj/{i}", {"ids": torch.arange(i + 1), "r": float(i)}, SampleMeta(f"traj/{i}", num_tokens=i + 1, weight_version=i // 2, group=f"g{i // 2}"))
    metas = dp.list_meta("traj/")
    assert sorted(m.key for m in metas) == [f"traj/{i}" for i in range(4)] and {m.group for m in metas} == {"g0", "g1"}
    got = dp.get(["traj/2", "traj/0"], ["ids"])
    assert [g["ids"].numel() for g in got] == [3, 1] and "r" not in got[0]
    dp.update("traj/0", {"adv": torch.ones(1)})
    assert set(dp.get(["traj/0"])[0]) >= {"ids", "r", "adv"}
    assert dp.delete(["traj/0", "traj/1", "nope"]) == 2
    assert sorted(m.key for m in dp.list_meta()) == ["traj/2", "traj/3"]
    with pytest.raises(KeyError):
        dp.get(["traj/0"])


def test_tcp_store_adapter_across_real_store():
    import socket
    from datetime import timedelta

    import torch.distributed as dist

    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    server = dist.TCPStore("127.0.0.1", port, None, True, timeout=timedelta(seconds=20), wait_for_workers=False)
    client = dist.TCPStore("127.0.0.1", port, None, False, timeout=timedelta(seconds=20))
    a, b = TCPStoreDataPlane(server), create_data_plane({"backend": "tcp_store"}, store=client)
    a.put("k", {"x": torch.arange(5, dtype=torch.float32)})
    assert b.get(["k"])[0]["x"].tolist() == [0, 1, 2, 3, 4] and [m.key for m in b.list_meta()] == ["k"]
    assert b.delete(["k"]) == 1 and a.list_meta() == []


def test_preshard_balances_tokens_and_keeps_groups():
    metas = [SampleMeta(f"k{i}", num_tokens=n, group=f"g{i // 2}") for i, n in enumerate([100, 90, 10, 20, 50, 40, 30, 60])]
    shards = preshard(metas, 2)
    assert sorted(sum(shards, [])) == sorted(m.key for m in metas)
    where = {k: r for r, ks in enumerate(shards) for k in ks}
    assert all(where[f"k{2 * g}"] == where[f"k{2 * g + 1}"] for g in range(4))
    load = [sum(m.num_tokens for m in metas if where[m.key] == r) for r in range(2)]
    assert abs(load[0] - load[1]) <= 40
    eq = preshard(metas, 4, keep_groups=False, equal_counts=True)
    assert [len(x) for x in eq] == [2, 2, 2, 2]


def _controller(tmp_path, mode, max_age=1, steps=4):
    mc = ModelConfig(vocab_size=32, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=8, torch_dtype="float32")
    ds = RandomTokenPromptDataset(256, 4, 8, 32, seed=0)
    env = {"synthetic": TokenFractionEnv({"target_token_id": 7})}
    cfg = {"grpo": dict(num_prompts_per_step=4, num_generations_per_prompt=4, max_num_steps=steps, val_period=0, seed=0),
           "loss_fn": dict(use_importance_sampling_correction=True, reference_policy_kl_penalty=0.0),
           "single_controller": dict(pump_mode=mode, max_trajectory_age_steps=max_age, rollout_ahead_batches=2, stall_timeout_s=120),
           "policy": dict(precision="float32", train_global_batch_size=16, train_micro_batch_size=8, logprob_batch_size=16,
                          max_total_sequence_length=48, max_grad_norm=1.0,
                          optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=5e-3, weight_decay=0.0)),
                          generation=dict(max_new_tokens=8, temperature=1.0, stop_token_ids=[], kv_cache_tokens=4096, block_size=8, max_running=32)),
           "logger": dict(log_dir=str(tmp_path)), "checkpointing": dict(enabled=False)}
    policy, gen, loader, _, loss_fn, logger, ck, ss, cfg = grpo.setup(cfg, None, ds, None, env, model_cfg=mc)
    hist = []
    sc = SingleController(policy, gen, loader, None, loss_fn, env, cfg, logger=logger, save_state=ss, step_callback=lambda s, m: hist.append(m["train"]))
    return sc, hist


@pytest.mark.parametrize("mode", ["interleaved", "threads"])
def test_single_controller_trains_on_age_bounded_trajectories(tmp_path, mode):
    sc, hist = _controller(tmp_path, mode)
    sc.run()
    assert len(hist) == 4 and sc.version == 4 and all(torch.isfinite(torch.tensor(h["loss"])) for h in hist)
    assert max(h["trajectory_age"] for h in hist) <= 1
    assert sc.stats["samples_trained"] == 4 * 16 and sc.stats["rollout_batches"] >= 4
    sd = sc.state_dict()
    assert sd["version"] == 4 and all(v >= 3 for _, v, _ in sd["pending"])   # what is still stored is at most one version old


def test_single_controller_drops_stale_and_reports_stall(tmp_path):
    sc, hist = _controller(tmp_path, "interleaved", max_age=0, steps=3)
    sc.sc["rollout_ahead_batches"] = 3           # runs ahead further than the age bound allows
    sc.run()
    assert len(hist) == 3 and sc.stats["dropped_stale"] > 0 and all(h["trajectory_age"] == 0 for h in hist)
    sc2, _ = _controller(tmp_path, "interleaved")
    sc2._on_stall(999.0)
    with pytest.raises(ControllerStalled):
        sc2.run()


def test_single_controller_weight_sync_and_fleet_probe_pumps(tmp_path):
    """The weight-sync pump brings the engine to the trainer's version as soon as the engine is free; the probe pump checks the
    engine between rollouts, counts failures in the same health tracker, and restarts an engine that died."""
    from rl_b200.distributed.health import ShardState

    sc, hist = _controller(tmp_path, "interleaved", steps=2)
    assert sc.engine_version == -1 and sc.sync_weights_once(blocking=True) and sc.engine_version == 0 and not sc.sync_weights_once()
    assert sc.rollout_once() > 0 and sc.train_once() is not None
    assert sc.version == 1 and sc.engine_version == 0                  # the trainer moved on, the engine has not yet
    assert sc.sync_weights_once(blocking=True) and sc.engine_version == 1 and sc.stats["weight_syncs"] == 2
    assert sc.probe_once() is None                                     # not due yet
    assert sc.probe_once(force=True) is True and sc.stats["probes"] == 1 and sc.health.state(0) == ShardState.HEALTHY
    with sc.engine_lock:
        assert sc.probe_once(force=True) is None                       # the engine is busy: the probe does not queue behind it
    # an engine that stops answering: failures add up to DEAD, the pump restarts it and rollouts go on
    calls = dict(restart=0)
    sc.generation.health_check = lambda: (_ for _ in ()).throw(RuntimeError("no answer"))
    sc.generation.restart = lambda: calls.__setitem__("restart", calls["restart"] + 1)
    for _ in range(int(sc.sc["max_generation_failures"])):
        assert sc.probe_once(force=True) is False
    assert calls["restart"] == 1 and sc.stats["engine_restarts"] == 1 and sc.stats["probe_failures"] == 3
    assert sc.health.state(0) == ShardState.HEALTHY and sc.engine_version == -1
    del sc.generation.health_check
    assert sc.probe_once(force=True) is True and sc.engine_version == 1   # the probe re-synced the restarted engine
    sc.run()
    assert sc.steps == 2 and hist[-1]["engine_version"] >= 1 and hist[-1]["weight_syncs"] >= 3


def test_observed_data_plane_counts_events():
    dp = create_data_plane({"backend": "local", "observe": True})
    dp.put("a", {"x": torch.arange(3)})
    dp.put("b", {"x": torch.arange(4)})
    assert len(dp.get(["a", "b"])) == 2 and dp.delete(["a"]) == 1
    st = dp.stats()
    assert st["put_calls"] == 2 and st["get_items"] == 2 and st["delete_calls"] == 1 and st["resident_samples"] == 1 and st["get_seconds"] >= 0


def _sync_cfg(tmp_path, steps, plane=True):
    cfg = {"grpo": dict(num_prompts_per_step=4, num_generations_per_prompt=4, max_num_steps=steps, val_period=0, seed=0),
           "loss_fn": dict(use_importance_sampling_correction=False, reference_policy_kl_penalty=0.01),
           "policy": dict(precision="float32", train_global_batch_size=16, train_micro_batch_size=8, logprob_batch_size=16,
                          max_total_sequence_length=48, max_grad_norm=1.0,
                          optimizer=dict(name="torch.optim.AdamW", kwargs=dict(lr=5e-3, weight_decay=0.0)),
                          generation=dict(max_new_tokens=8, temperature=1.0, stop_token_ids=[], kv_cache_tokens=4096, block_size=8, max_running=32)),
           "logger": dict(log_dir=str(tmp_path)), "checkpointing": dict(enabled=False)}
    if plane:
        cfg["data_plane"] = dict(enabled=True, backend="local")
    return cfg


def test_grpo_over_the_data_plane_matches_the_in_memory_trainer(tmp_path):
    """The data-plane-mediated trainer (rollout actor -> records, driver reads small fields only, policy fetches by key) takes
    the same optimizer steps as ``grpo_train`` and leaves the plane empty after every step."""
    from rl_b200.algorithms.grpo_sync import BatchMeta, PlanePolicy, grpo_train_sync

    mc = ModelConfig(vocab_size=32, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=8, torch_dtype="float32")
    env = {"synthetic": TokenFractionEnv({"target_token_id": 7})}
    hist = {}
    for mode in ("plane", "memory"):
        ds = RandomTokenPromptDataset(256, 4, 8, 32, seed=0)
        policy, gen, loader, _, loss_fn, logger, ck, ss, cfg = grpo.setup(_sync_cfg(tmp_path / mode, 3, mode == "plane"), None, ds, None, env, model_cfg=mc)
        h = []
        if mode == "plane":
            plane = LocalDataPlane()
            grpo_train_sync(policy, gen, loader, None, None, loss_fn, env, None, logger, ck, ss, cfg, data_plane=plane,
                            step_callback=lambda s, m: h.append(m["train"]))
            assert plane.stats()["resident_samples"] == 0 and plane.stats()["puts"] == 3 * 16
            assert all(x["data_plane_resident_peak"] == 16 for x in h)
        else:
            grpo.grpo_train(policy, gen, loader, None, None, loss_fn, env, None, logger, ck, ss, cfg, step_callback=lambda s, m: h.append(m["train"]))
        hist[mode] = h
    assert len(hist["plane"]) == len(hist["memory"]) == 3
    for a, b in zip(hist["plane"], hist["memory"]):
        assert a["loss"] == pytest.approx(b["loss"], rel=1e-4, abs=1e-6) and a["reward"] == pytest.approx(b["reward"], rel=1e-5)
        assert a["grad_norm"] == pytest.approx(b["grad_norm"], rel=1e-3)

    # the facade's streaming form: a step fed in two pieces equals one call
    with pytest.raises(ValueError):
        grpo_train_sync(policy, gen, loader, None, None, loss_fn, env, None, logger, ck, dict(ss), _sync_cfg(tmp_path, 1, plane=False))
    pol = PlanePolicy(policy, LocalDataPlane())
    pol.begin_train_step(loss_fn)
    with pytest.raises(AssertionError):
        pol.begin_train_step(loss_fn)
    pol.abort_train_step()
    m = BatchMeta("p", ["a", "b", "c"], [3, 4, 5], ["g0", "g0", "g1"], {"x"})
    assert m.select([0, 2]).keys == ["a", "c"] and m.size == 3 and [s.num_tokens for s in m.sample_metas()] == [3, 4, 5]


def test_prompt_group_record_to_rows_in_the_plane():
    from rl_b200.experience.payload import Completion, PromptGroupRecord, pack_payload, record_to_train_batch

    prompt = [{"role": "user", "content": "q", "token_ids": torch.tensor([5, 6, 7])}]

    def completion(gen, reward):
        return Completion([dict(prompt[0]), {"role": "assistant", "content": "a", "token_ids": torch.tensor(gen),
                                             "generation_logprobs": torch.full((len(gen),), -0.5)}], reward)

    rec = PromptGroupRecord(prompt, [completion([1, 2], 1.0), completion([3, 4, 8, 9], 0.0)], prompt_idx=3)
    td = record_to_train_batch(rec)
    assert td["input_ids"].tolist() == [[5, 6, 7, 1, 2, 0, 0], [5, 6, 7, 3, 4, 8, 9]] and td["input_lengths"].tolist() == [5, 7]
    assert td["token_mask"].tolist() == [[0, 0, 0, 1, 1, 0, 0], [0, 0, 0, 1, 1, 1, 1]] and td["total_reward"].tolist() == [1.0, 0.0]
    assert td["prompt_ids_for_adv"].tolist() == [[5, 6, 7], [5, 6, 7]] and td["generation_logprobs"][0, 3].item() == -0.5
    keys, recs, metas = pack_payload(td, weight_version=4, group_id="s7_p3")
    assert keys == ["s7_p3_g0", "s7_p3_g1"] and recs[0]["input_ids"].tolist() == [5, 6, 7, 1, 2] and recs[1]["token_mask"].numel() == 7
    assert [m.weight_version for m in metas] == [4, 4] and metas[0].num_tokens == 5 and metas[1].group == "s7_p3"
    plane = LocalDataPlane()
    plane.put_batch(keys, recs, metas)
    back = records_to_batch(plane.get(keys, ("input_ids", "input_lengths")))
    assert torch.equal(back["input_ids"], td["input_ids"])
