"""OpenAI-compatible front end of the engine and the failover router, on the CPU engine path."""

import threading

import pytest
import requests
import torch

from rl_b200.data.tokenizers import ByteTokenizer
from rl_b200.distributed.health import HealthPolicy, ShardState
from rl_b200.engine.engine import GenerationEngine
from rl_b200.engine.http_server import ServerHandle, create_app
from rl_b200.engine.router import GenerationRouter, NoHealthyShardError, create_router_app
from rl_b200.models.config import ModelConfig
from rl_b200.models.transformer import CausalLM


def _server(seed=1):
    tok = ByteTokenizer(vocab_size=300)
    mc = ModelConfig(vocab_size=300, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=8, torch_dtype="float32")
    model = CausalLM(mc, dtype=torch.float32, device="cpu", seed=seed)
    eng = GenerationEngine(model, block_size=4, num_blocks=256, max_running=16, max_model_len=128, use_cuda_graphs=False)
    return ServerHandle(create_app(eng, tok, model_name="tiny")).start(), tok


def test_completions_token_in_token_out_and_batching():
    srv, tok = _server()
    try:
        base = srv.base_url
        assert requests.get(base + "/health").json()["status"] == "ok"
        assert requests.get(base + "/v1/models").json()["data"][0]["id"] == "tiny"
        ids = requests.post(base + "/tokenize", json={"prompt": "hello"}).json()
        assert ids["tokens"] == tok.encode("hello") and ids["count"] == len(ids["tokens"])
        body = dict(prompt="hello", max_tokens=5, n=3, logprobs=1, ignore_eos=True, temperature=0.7)
        out = requests.post(base + "/v1/completions", json=body).json()
        assert len(out["choices"]) == 3 and out["usage"]["completion_tokens"] == 15
        for c in out["choices"]:
            assert c["prompt_token_ids"] == tok.encode("hello") and len(c["token_ids"]) == 5
            assert len(c["logprobs"]["token_logprobs"]) == 5 and all(x <= 0 for x in c["logprobs"]["token_logprobs"])
            assert c["finish_reason"] == "length"
        # token-in prompt, greedy: the same request twice gives the same tokens
        g = dict(prompt=[5, 6, 7, 8], max_tokens=4, temperature=0, ignore_eos=True)
        a = requests.post(base + "/v1/completions", json=g).json()["choices"][0]["token_ids"]
        b = requests.post(base + "/v1/completions", json=g).json()["choices"][0]["token_ids"]
        assert a == b and len(a) == 4
        # concurrent clients share engine calls
        res = []
        ts = [threading.Thread(target=lambda: res.append(requests.post(base + "/v1/completions", json=g).json())) for _ in range(6)]
        [t.start() for t in ts]
        [t.join() for t in ts]
        assert all(r["choices"][0]["token_ids"] == a for r in res)
        chat = requests.post(base + "/v1/chat/completions", json=dict(messages=[{"role": "user", "content": "hi"}], max_tokens=3,
                                                                       ignore_eos=True)).json()
        assert chat["choices"][0]["message"]["role"] == "assistant" and len(chat["choices"][0]["token_ids"]) == 3
        assert requests.post(base + "/v1/completions", json=dict(prompt=[])).status_code == 400
    finally:
        srv.stop()


def test_weight_update_pauses_serving_and_bumps_version():
    srv, _ = _server()
    try:
        assert srv.begin_weight_update()
        got = []
        t = threading.Thread(target=lambda: got.append(requests.post(srv.base_url + "/v1/completions",
                                                                     json=dict(prompt=[1, 2], max_tokens=2, ignore_eos=True)).json()))
        t.start()
        t.join(0.5)
        assert t.is_alive() and not got          # held back while the trainer owns the engine
        srv.end_weight_update()
        t.join(30)
        assert got and got[0]["weight_version"] == 1
    finally:
        srv.stop()


def test_router_fails_over_and_recovers():
    a, _ = _server(1)
    b, _ = _server(1)
    router = GenerationRouter([a.base_url, b.base_url], HealthPolicy(suspect_after_failures=1, dead_after_failures=2),
                              request_timeout_s=20)
    body = dict(prompt=[3, 4, 5], max_tokens=3, temperature=0, ignore_eos=True)
    try:
        first = router.completions(**body)
        assert len(first["choices"][0]["token_ids"]) == 3
        a.stop()                                   # shard 0 goes away between requests
        outs = [router.completions(**body) for _ in range(4)]
        assert all(o["served_by"] == 1 for o in outs)
        assert all(o["choices"][0]["token_ids"] == first["choices"][0]["token_ids"] for o in outs)
        assert router.health.state(0) in (ShardState.SUSPECT, ShardState.DEAD) and router.stats["retries"] >= 1
        while router.health.state(0) != ShardState.DEAD:
            router.health.report_failure(0, "probe")
        assert router.probe_once() == {0: False} and router.health.state(0) == ShardState.DEAD
        # the router as a server: same API, fleet view
        rs = ServerHandle(create_router_app(router)).start()
        try:
            out = requests.post(rs.base_url + "/v1/completions", json=body).json()
            assert out["served_by"] == 1
            fleet = requests.get(rs.base_url + "/fleet").json()
            assert fleet["shards"][0]["state"] == "dead" and fleet["serviceable"]
        finally:
            rs._server.should_exit = True
        b.stop()
        with pytest.raises(NoHealthyShardError):
            router.completions(**body)
    finally:
        router.stop()


def test_remote_environment_round_trip_and_server_loss():
    from rl_b200.environments.registry import create_env
    from rl_b200.environments.remote_environment import create_env_app
    from rl_b200.environments.vlm_environment import VLMEnvironment

    srv = ServerHandle(create_env_app(VLMEnvironment({}))).start()
    env = create_env("remote", dict(url=srv.base_url, batch_size=2, max_retries=0, timeout_s=5))
    logs = [[{"role": "user", "content": "colour?", "token_ids": torch.tensor([1, 2])}, {"role": "assistant", "content": c, "token_ids": torch.tensor([3])}]
            for c in ("it is red", "blue", "maybe green")]
    try:
        out = env.step(logs, [{"ground_truth": "red"}, {"ground_truth": "red"}, {"ground_truth": "green"}])
        assert out.rewards.tolist() == [1.0, 0.0, 1.0] and out.terminateds.all() and out.answers[1] == "blue"
        assert requests.get(srv.base_url + "/health").json()["environment"] == "VLMEnvironment"
    finally:
        srv._server.should_exit = True
        srv._thread.join(5)
    with pytest.raises(ConnectionError):
        env.step(logs[:1], [{"ground_truth": "red"}])
    env.shutdown()


def test_async_sample_level_rollout_through_the_batching_frontend():
    """Every sample runs its own generate -> environment loop; samples need different numbers of turns."""
    from rl_b200.data.collate import rl_collate_fn
    from rl_b200.engine.http_server import BatchingFrontend
    from rl_b200.environments.interfaces import EnvironmentReturn
    from rl_b200.experience.rollouts import run_async_multi_turn_rollout

    class CountdownEnv:
        """Terminates a sample after ``turns`` assistant messages; reward 1 per turn."""

        def step(self, logs, metas):
            out_meta, term = [], []
            for log, m in zip(logs, metas):
                left = m["turns"] - 1
                out_meta.append({"turns": left})
                term.append(left <= 0)
            n = len(logs)
            return EnvironmentReturn([{"role": "environment", "content": "go on"}] * n, out_meta, [None] * n, torch.ones(n), torch.tensor(term), None)

    tok = ByteTokenizer(vocab_size=300)
    mc = ModelConfig(vocab_size=300, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=8, torch_dtype="float32")
    eng = GenerationEngine(CausalLM(mc, dtype=torch.float32, device="cpu", seed=2), block_size=4, num_blocks=512, max_running=16,
                           max_model_len=256, use_cuda_graphs=False)
    fe = BatchingFrontend(eng, batch_window_s=0.01)
    try:
        data = [{"message_log": [{"role": "user", "content": "x", "token_ids": torch.tensor([10 + i, 20, 30])}], "length": 3,
                 "extra_env_info": {"turns": 1 + i % 3}, "task_name": "cd", "idx": i} for i in range(6)]
        batch = rl_collate_fn(data)
        out, m = run_async_multi_turn_rollout(fe, batch, tok, {"cd": CountdownEnv()}, max_seq_len=200, max_rollout_turns=4,
                                              sampling=dict(max_new_tokens=5, temperature=1.0))
        assert out["total_reward"].tolist() == [1.0, 2.0, 3.0, 1.0, 2.0, 3.0] and m["total_turns"] == 12
        assert out["generation_lengths"].tolist() == [5, 10, 15, 5, 10, 15]
        roles = [[x["role"] for x in log] for log in out["message_log"]]
        assert roles[0] == ["user", "assistant"] and roles[2] == ["user", "assistant", "environment", "assistant", "environment", "assistant"]
        assert all(x["generation_logprobs"].numel() == 5 for log in out["message_log"] for x in log if x["role"] == "assistant")
        assert fe._calls < 12          # concurrent samples shared engine calls
    finally:
        fe.close()


def test_requests_join_the_running_engine_loop_and_leave_when_done():
    """Continuous admission: a short request that arrives while a long one is decoding joins the same engine loop at the next
    host visit and is answered first; its tokens are what the model gives for it alone (the shared batch changes nothing)."""
    import time

    from rl_b200.engine.engine import SamplingParams
    from rl_b200.engine.http_server import BatchingFrontend

    tok = ByteTokenizer(vocab_size=300)
    mc = ModelConfig(vocab_size=300, hidden_size=32, intermediate_size=64, num_hidden_layers=2, num_attention_heads=4,
                     num_key_value_heads=2, head_dim=8, torch_dtype="float32")
    model = CausalLM(mc, dtype=torch.float32, device="cpu", seed=1)
    eng = GenerationEngine(model, block_size=4, num_blocks=256, max_running=16, max_model_len=256, use_cuda_graphs=False)
    slow = []
    eng.window_hook = lambda: (time.sleep(0.01), slow.append(1))       # stretch the loop so that the second request arrives mid-way
    fe = BatchingFrontend(eng, batch_window_s=0.0)
    sp = dict(temperature=1.0, max_new_tokens=60, stop_token_ids=[], greedy=True)
    done_at, recs = {}, {}

    def ask(name, prompt, **over):
        recs[name] = fe.submit(prompt, dict(sp, **over))
        done_at[name] = time.perf_counter()

    a = threading.Thread(target=ask, args=("long", [1, 2, 3, 4, 5]))
    a.start()
    while len(slow) < 5:       # the long request is decoding
        time.sleep(0.005)
    b = threading.Thread(target=ask, args=("short", [9, 8, 7]), kwargs=dict(max_new_tokens=60))
    b.start()
    b.join(60)
    a.join(60)
    try:
        assert fe.stats["loops"] == 1 and fe.stats["joined_running_loop"] == 1 and fe.stats["answered"] == 2
        assert len(recs["long"].out_tokens) == 60 and len(recs["short"].out_tokens) == 60
        assert done_at["long"] < done_at["short"]       # same length, started earlier: each leaves when ITS tokens are done
        assert fe.pause(10)          # the frontend's loop has fully ended: the engine may be driven from this thread
        eng.window_hook = None
        alone = eng.generate([[9, 8, 7]], SamplingParams(max_new_tokens=60, stop_token_ids=[], greedy=True))[0]
        fe.resume()
        assert alone.out_tokens == recs["short"].out_tokens
        # a different sampling setting waits for a loop of its own; pausing drains the running loop
        fe.submit([4, 4], dict(sp, temperature=0.5, greedy=False, max_new_tokens=3))
        assert fe.stats["loops"] == 2 and fe.pause(10)
        fe.resume()
    finally:
        fe.close()
