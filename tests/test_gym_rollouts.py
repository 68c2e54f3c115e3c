"""Gym-owned rollouts: episodes run by an agent server, streamed back per prompt group, turned into message logs."""

import time

import pytest
import torch

from rl_b200.distributed.batched_data_dict import BatchedDataDict
from rl_b200.experience import gym_rollouts as G
from rl_b200.experience.failures import DataFailure, InfraFailure


def _episode(prompt, turns):
    """turns: list of (generated ids, tool ids appended by the environment afterwards)."""
    out, seen = [], list(prompt)
    for gen, tool in turns:
        out.append(dict(role="assistant", content="x" * len(gen), prompt_token_ids=list(seen), generation_token_ids=list(gen),
                        generation_log_probs=[-0.1 * (k + 1) for k in range(len(gen))]))
        seen += list(gen)
        if tool:
            out.append(dict(type="function_call_output", content="tool says hi"))
            seen += list(tool)
    return out


class FakeGym:
    """Answers rows after a per-row delay, so that groups finish out of order."""

    def __init__(self):
        self.calls = []

    def run(self, row, sampling=None):
        self.calls.append(row["id"])
        time.sleep(row.get("delay", 0.0))
        if row.get("boom"):
            raise InfraFailure("gym down")
        if row.get("bad"):
            ep = _episode([1, 2, 3], [([4, 5], [6]), ([7], None)])
            ep[2]["prompt_token_ids"][1] = 99           # history changed under re-tokenisation
            return dict(reward=1.0, response=dict(output=ep))
        ep = _episode([1, 2, 3], [([4, 5], [6, 7]), ([8, 9, 10], None)])
        if row.get("markers"):
            ep[0]["content"] = "<tool_call> broken"
        return dict(reward=float(row["id"]), response=dict(output=ep), mask_sample=bool(row.get("flag")))


def test_episode_to_message_log_and_penalties():
    log, gen = G.episode_to_message_log(_episode([1, 2, 3], [([4, 5], [6, 7]), ([8, 9, 10], None)]))
    assert [m["role"] for m in log] == ["user", "assistant", "environment", "assistant"] and gen == 5
    assert torch.cat([m["token_ids"] for m in log]).tolist() == [1, 2, 3, 4, 5, 6, 7, 8, 9, 10]
    assert log[1]["generation_logprobs"].tolist() == pytest.approx([-0.1, -0.2]) and "generation_logprobs" not in log[2]
    with pytest.raises(DataFailure):
        G.episode_to_message_log([dict(role="assistant", prompt_token_ids=[1], generation_token_ids=[2, 3], generation_log_probs=[-1.0])])
    with pytest.raises(DataFailure):
        G.episode_to_message_log([dict(role="tool", content="only a tool")])
    cfg = dict(invalid_tool_call_penalty=0.5, thinking_penalty=0.25)
    assert G.reward_penalty([dict(role="assistant", content="<think> no end <tool_call>")], cfg) == 0.75
    assert G.reward_penalty([dict(role="assistant", content="<think>ok</think> fine")], cfg) == 0.0
    assert G.reward_penalty([dict(role="assistant", content="<tool_call>")], None) == 0.0


def test_groups_stream_in_completion_order_with_rows_in_input_order():
    rows = [dict(id=0, delay=0.25), dict(id=1, delay=0.02), dict(id=2, delay=0.0, markers=True), dict(id=3, delay=0.05, flag=True),
            dict(id=4, delay=0.1, bad=True), dict(id=5, delay=0.0)]
    gym = FakeGym()
    got = list(G.run_gym_rollout(rows, gym, num_generations=2, reward_penalty_config=dict(invalid_tool_call_penalty=0.5), max_seq_len=10))
    assert [r.group_index for r in got] == [1, 2, 0]                 # the group with the slow row comes last
    by = {r.group_index: r for r in got}
    assert by[0].rows == [0, 1] and by[0].rewards.tolist() == [0.0, 1.0]
    assert by[1].raw_rewards.tolist() == [2.0, 3.0] and by[1].rewards.tolist() == [1.5, 3.0]      # marker penalty on row 2
    assert by[1].loss_multiplier.tolist() == [1.0, 0.0]             # the gym flagged row 3
    assert by[2].loss_multiplier.tolist() == [0.0, 1.0] and by[2].metrics["data_failures"] == 1.0  # row 4: unusable history
    assert by[0].truncated.tolist() == [True, True]                 # 10 tokens reach max_seq_len
    batch = BatchedDataDict(extra_env_info=rows, idx=torch.arange(6))
    out, metrics = G.run_gym_rollout_sync(batch, FakeGym(), num_generations=2)
    assert len(out["message_log"]) == 6 and out["total_reward"].tolist() == [0.0, 1.0, 2.0, 3.0, 0.0, 5.0]
    assert out["loss_multiplier"].tolist() == [1, 1, 1, 0, 0, 1] and metrics["groups"] == 3 and metrics["generated_tokens"] == 25.0
    with pytest.raises(InfraFailure):
        list(G.run_gym_rollout([dict(id=0, boom=True)], FakeGym(), num_generations=1))


def test_client_retries_transport_errors_and_not_refusals():
    calls = []

    def post(url, body, timeout):
        calls.append(url)
        if len(calls) < 3:
            raise ConnectionError("reset")
        return dict(reward=1.0, echoed=body["policy_base_url"])

    c = G.GymClient("http://gym:9/", "http://policy:8", max_retries=2, post=post)
    assert c.run(dict(id=1))["echoed"] == "http://policy:8" and calls == ["http://gym:9/run"] * 3
    with pytest.raises(InfraFailure):
        G.GymClient("http://gym:9", "p", max_retries=1, post=lambda *a: (_ for _ in ()).throw(ConnectionError("x"))).run({})

    def refuse(*a):
        raise DataFailure("bad row")

    with pytest.raises(DataFailure):
        G.GymClient("http://gym:9", "p", max_retries=5, post=refuse).run({})
