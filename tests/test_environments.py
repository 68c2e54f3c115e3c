"""Environments: math verification, code execution, sliding puzzle, synthetic token rewards."""

import pytest
import torch

from rl_b200.environments.code_environment import CodeEnvironment, CodeJaccardEnvironment, extract_code
from rl_b200.environments.games.sliding_puzzle import SlidingPuzzleEnv, apply_move, make_initial_state, solved_grid
from rl_b200.environments.math_environment import MathEnvironment, answers_match, extract_answer
from rl_b200.environments.registry import create_env
from rl_b200.environments.synthetic import HashParityEnv, TokenFractionEnv


def _log(text):
    return [{"role": "user", "content": "q", "token_ids": torch.tensor([1])}, {"role": "assistant", "content": text, "token_ids": torch.tensor([2, 7, 7, 3])}]


def test_math_answers():
    assert extract_answer(r"so the answer is \boxed{\frac{3}{4}}.") == r"\frac{3}{4}"
    assert answers_match(r"\frac{3}{4}", "0.75") and answers_match("1,000", "1000") and answers_match("x = 5", "5")
    assert answers_match(r"\boxed{2}".replace("\\boxed{", "").rstrip("}"), "2.0") and not answers_match("3", "4") and not answers_match(None, "4")
    env = MathEnvironment({"num_workers": 2})
    out = env.step([_log(r"thus \boxed{42}"), _log("I think 41")], [{"ground_truth": "42"}, {"ground_truth": "42"}])
    assert out.rewards.tolist() == [1.0, 0.0] and out.terminateds.all() and out.answers[0] == "42"
    env.shutdown()


def test_code_env_executes_with_limits():
    env = CodeEnvironment({"timeout_s": 3})
    good = "```python\ndef add(a, b):\n    return a + b\n```"
    bad = "```python\ndef add(a, b):\n    return a - b\n```"
    loop = "```python\nwhile True:\n    pass\n```"
    out = env.step([_log(good), _log(bad), _log(loop), _log("no code")],
                   [{"tests": ["assert add(1, 2) == 3"]}, {"tests": ["assert add(1, 2) == 3"]}, {"tests": ["assert True"]}, {}])
    assert out.rewards.tolist() == [1.0, 0.0, 0.0, 0.0]
    assert extract_code(good).startswith("def add")
    j = CodeJaccardEnvironment().step([_log(good)], [{"ground_truth": "def add(a, b):\n    return a + b"}])
    assert j.rewards[0] > 0.9
    env.shutdown()


def test_sliding_puzzle_multi_turn():
    st = {"grid": solved_grid(3), "moves": 0, "max_moves": 5, "size": 3}
    apply_move(st["grid"], "left")  # blank moved left: solving move is "right"
    env = SlidingPuzzleEnv()
    out = env.step([_log("<action>up</action>")], [st])
    assert not out.terminateds[0] and out.rewards[0] == 0 and out.metadata[0]["moves"] == 1
    out2 = env.step([_log("<action>right</action> then <action>down</action>")], [st])
    assert out2.rewards[0] == 0  # the last action wins, and "down" leaves the board
    out3 = env.step([_log("<action>right</action>")], [st])
    assert out3.rewards[0] == 1 and out3.terminateds[0]
    s = make_initial_state(3, 8, 20, seed=1)
    assert s["grid"] != solved_grid(3) and sorted(v for r in s["grid"] for v in r) == list(range(9))


def test_synthetic_envs_and_registry():
    out = TokenFractionEnv({"target_token_id": 7}).step([_log("")], [None])
    assert out.rewards[0] == 0.5
    h = HashParityEnv().step([_log(""), _log("")], [None, None])
    assert h.rewards[0] == h.rewards[1] and 0 <= h.rewards[0] <= 1
    assert isinstance(create_env("math", {}), MathEnvironment)


def test_named_sharding_axes():
    from rl_b200.distributed.named_sharding import NamedSharding

    ns = NamedSharding.from_sizes(8, dp=2, pp=1, cp=1, tp=4)
    assert ns.size == 8 and ns.get_axis_size("tp") == 4
    assert ns.get_worker_coords(5) == {"dp": 1, "pp": 0, "cp": 0, "tp": 1}
    assert ns.get_ranks(dp=1) == [4, 5, 6, 7] and ns.get_ranks(dp=0, tp=2) == [2] and ns.get_ranks(dp=0, pp=0, cp=0, tp=2) == 2
    assert ns.axis_groups("tp") == [[0, 1, 2, 3], [4, 5, 6, 7]] and ns.axis_groups("dp") == [[0, 4], [1, 5], [2, 6], [3, 7]]
    assert ns.group_of(6, "dp") == [2, 6]


def test_tool_environment_runs_calls_and_scores_final_answers():
    import pytest as _pytest

    from rl_b200.environments.registry import create_env
    from rl_b200.environments.tool_environment import keyword_retrieve, safe_eval

    assert safe_eval("2 * (3 + 4) - 10 / 4") == 11.5 and safe_eval("-2 ** 3") == -8
    for bad in ("__import__('os')", "a + 1", "2 ** 1000", "(1).real"):
        with _pytest.raises((ValueError, SyntaxError)):
            safe_eval(bad)
    docs = ["The capital of France is Paris.", "Blackwell GPUs have tensor memory.", "Paris has the Louvre."]
    assert keyword_retrieve("capital France", docs, 1) == [docs[0]] and keyword_retrieve("zzz", docs) == []
    env = create_env("tool", {"documents": docs, "max_tool_calls": 2})
    logs = [[{"role": "user", "content": "12*12?"}, {"role": "assistant", "content": '<tool_call>{"name": "calculator", "arguments": {"expression": "12*12"}}</tool_call>'}],
            [{"role": "user", "content": "capital?"}, {"role": "assistant", "content": '<tool_call>{"name": "retrieve", "arguments": {"query": "capital of France"}}</tool_call>'}],
            [{"role": "user", "content": "q"}, {"role": "assistant", "content": r"The answer is \boxed{144}"}],
            [{"role": "user", "content": "q"}, {"role": "assistant", "content": "<tool_call>not json</tool_call>"}]]
    metas = [{"ground_truth": "144"}, {"ground_truth": "Paris"}, {"ground_truth": "144"}, {"ground_truth": "1"}]
    out = env.step(logs, metas)
    assert out.terminateds.tolist() == [False, False, True, False] and out.rewards.tolist() == [0.0, 0.0, 1.0, 0.0]
    assert '"result": 144' in out.observations[0]["content"] and "Paris" in out.observations[1]["content"] and "error" in out.observations[3]["content"]
    assert out.metadata[0]["tool_calls"] == 1 and out.answers[2] == "144"
    # second turn of sample 0: final answer after the tool response; the call budget ends sample 3
    logs[0] += [out.observations[0], {"role": "assistant", "content": r"\boxed{144}"}]
    logs[3] += [out.observations[3], {"role": "assistant", "content": "<tool_call>{}</tool_call>"}]
    out2 = env.step([logs[0], logs[3]], [out.metadata[0], dict(out.metadata[3], tool_calls=2)])
    assert out2.terminateds.tolist() == [True, True] and out2.rewards.tolist() == [1.0, 0.0]


def test_math_verifier_types_and_structured_answers():
    """Graders beyond the scalar case: tuples / sets / intervals, mixed numbers, scientific notation; the DAPO string rule;
    English and multilingual multiple choice; the multi-reward environment; a verification that runs out of time scores 0."""
    from rl_b200.environments import math_environment as M
    from rl_b200.environments.registry import create_env

    ok = M.answers_match_structured
    assert ok("(1, \\frac{1}{2})", "(1,0.5)") and ok("\\{3,1\\}", "{1,3}") and not ok("[1,2)", "(1,2)") and ok("[1,2)", "[1, 2)")
    assert ok("1 1/2", "3/2") and ok("3 \\times 10^{4}", "30000") and ok("3, 5", "3,5") and not ok("3, 5", "3, 6") and not ok("(1,2,3)", "(1,2)")
    assert M.dapo_math_verify("so the answer is \\boxed{1,000}", "1000") == (1.0, "1,000")
    assert M.dapo_math_verify("\\boxed{0.50}", "0.5")[0] == 0.0                       # no numeric leniency under this rule
    assert M.dapo_math_verify("\\boxed{7}" + " " * 400, "7") == (0.0, None)            # only the tail of the response counts
    assert M.extract_multichoice("reasoning... **Answer: (C)**") == "C" and M.extract_multichoice("答案：B", True) == "B"
    assert M.extract_multichoice("الإجابة: ب", True) == "B" and M.extract_multichoice("答案：B", False) is None

    def run(env, texts, truths):
        return env.step([[{"role": "assistant", "content": t}] for t in texts], [{"ground_truth": g} for g in truths])

    env = create_env("math", dict(math_verify_impl="dapo_math_verify"))
    assert run(env, ["\\boxed{12}", "\\boxed{13}"], ["12", "12"]).rewards.tolist() == [1.0, 0.0]
    mc = create_env("multichoice", dict(verifier_type="english_multichoice"))
    r = run(mc, ["Answer: b", "I think Answer: D", "nothing"], ["B", "A", "C"])
    assert r.rewards.tolist() == [1.0, 0.0, 0.0] and r.answers == ["B", "D", None]
    ml = create_env("multichoice", dict(verifier_type="multilingual_multichoice"))
    assert run(ml, ["정답: C", "Respuesta: A"], ["C", "B"]).rewards.tolist() == [1.0, 0.0]
    multi = create_env("math_multi_reward")
    r = run(multi, ["<think>x</think>\n<answer>42</answer>", "<answer>4.5</answer> trailing"], ["42", "4.5"])
    assert r.rewards.tolist() == [[1.0, 1.0, 1.0], [1.0, 0.0, 0.0]] and multi.REWARD_NAMES[0] == "reward/correctness"
    with pytest.raises(ValueError):
        create_env("math", dict(math_verify_impl="nope"))
    import time

    assert M._with_time_limit(lambda: time.sleep(2) or True, 0.05, False) is False
