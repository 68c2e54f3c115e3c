"""Example entrypoints run end to end on CPU with the offline recipe; tools; data registry; byte tokenizer; eval metrics."""

import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

TINY = ["policy.model_name=tiny-llama-oracle", "policy.tokenizer.name=byte", "policy.max_total_sequence_length=96",
        "policy.train_global_batch_size=8", "policy.train_micro_batch_size=4", "policy.scheduler=null", "logger.monitor_gpus=false",
        "policy.sequence_packing.sequence_length_round=1"]


def test_byte_tokenizer_roundtrip_and_chat():
    from rl_b200.data.llm_message_utils import get_formatted_message_log
    from rl_b200.data.tokenizers import ByteTokenizer

    tok = ByteTokenizer()
    s = "héllo <|user|> \\boxed{3}"
    assert tok.decode(tok.encode(s)) == s
    log = get_formatted_message_log([{"role": "user", "content": "2+2?"}, {"role": "assistant", "content": "4"}], tok)
    text = "".join(tok.decode(m["token_ids"]) for m in log)
    assert text == "<bos><|user|>2+2?<|end|><|assistant|>4<|end|><eos>"
    assert log[1]["token_ids"][0].item() == tok.encode("<|assistant|>")[0]


def test_registry_processors_and_jsonl(tmp_path):
    import json

    from rl_b200.data.datasets.registry import setup_response_data
    from rl_b200.data.tokenizers import ByteTokenizer

    p = tmp_path / "d.jsonl"
    p.write_text("\n".join(json.dumps({"q": f"{i}+1", "a": str(i + 1)}) for i in range(5)))
    tok = ByteTokenizer()
    cfg = {"train": [{"dataset_name": "jsonl", "data_path": str(p), "input_key": "q", "output_key": "a", "prompt": "Q: {}"},
                     {"dataset_name": "arithmetic", "num_samples": 3}], "max_input_seq_length": 16,
           "default": {"env_name": "math", "processor": "math_data_processor"}}
    train, val, envs, venvs = setup_response_data(tok, cfg, {"math": {"num_workers": 1}})
    assert len(train) == 8 and list(envs) == ["math"]
    it = train[1]
    assert it["extra_env_info"]["ground_truth"] == "2" and "Q: 1+1" in tok.decode(it["message_log"][0]["token_ids"])
    long_item = train[6]  # arithmetic prompt longer than 16 tokens: masked stub
    assert long_item["loss_multiplier"] == 0.0 and long_item["length"] <= 16 and long_item["idx"] == 6
    for e in envs.values():
        e.shutdown()


def test_eval_metrics():
    from rl_b200.evals.eval import eval_cons_k, eval_pass_k

    r = torch.tensor([1.0, 0, 0, 0, 0, 0, 0, 0])  # 2 prompts x 4 samples
    assert eval_pass_k(r, 4, 1) == pytest.approx(0.25) and eval_pass_k(r, 4, 4) == pytest.approx(1.0)
    assert eval_pass_k(r, 4, 2) == pytest.approx(0.5)  # 1 - C(3,2)/C(4,2)
    assert eval_cons_k(torch.tensor([1.0, 1, 0, 0]), 4, 3, ["7", "7", "8", "9"]) == 1.0
    assert eval_cons_k(torch.tensor([1.0, 0, 0, 0]), 4, 4, ["7", "8", "8", None]) == 0.0


def test_config_cli_and_refit_model(capsys):
    from rl_b200.tools import config_cli
    from rl_b200.tools.refit_bandwidth_calculator import parse_layout, refit_seconds

    assert config_cli.main(["compare", f"{ROOT}/examples/configs/grpo_math_1B.yaml", f"{ROOT}/examples/configs/grpo_math_8B.yaml"]) == 1
    assert "policy.model_name: 'llama3.2-1b' -> 'llama3.1-8b'" in capsys.readouterr().out
    assert config_cli.minimize({"a": {"b": 1, "c": 2}, "d": 3}, {"a": {"b": 1, "c": 5}, "d": 3, "e": 4}) == {"a": {"c": 5}, "e": 4}
    same = refit_seconds(16e9, parse_layout("dp8"), parse_layout("dp8"), 8)
    assert same["seconds"] == 0.0
    r = refit_seconds(64e9, parse_layout("tp4dp2"), parse_layout("tp2"), 8, bw_gbs=800.0)
    assert r["recv_bytes_per_rank"] == pytest.approx(16e9) and r["seconds"] == pytest.approx(0.02, rel=0.01)


def _recipes():
    base = os.path.join(ROOT, "examples", "configs")
    return sorted(os.path.relpath(os.path.join(d, f), base) for d, _, fs in os.walk(base) for f in fs if f.endswith(".yaml") and "evals" not in d
                  and os.path.basename(d) != "quant")      # (quant/: quantizer recipes, not training recipes)


@pytest.mark.parametrize("yaml_name", _recipes())
def test_every_recipe_loads_and_resolves(yaml_name):
    from rl_b200.utils.config import load_config

    cfg = load_config(os.path.join(ROOT, "examples", "configs", yaml_name))
    assert "policy" in cfg and "${" not in str(cfg)


def test_run_grpo_offline_recipe(capsys):
    from examples import run_grpo

    run_grpo.main(["--config", f"{ROOT}/examples/configs/grpo_arithmetic_offline.yaml", "grpo.max_num_steps=2"])
    out = capsys.readouterr().out
    assert "[grpo] step 2:" in out


def test_run_grpo_with_a_hybrid_state_space_model(capsys, tmp_path):
    """The whole loop (engine with per-sequence Mamba states, log-probabilities, training, checkpoint) on the Nemotron-H blocks."""
    from examples import run_grpo

    run_grpo.main(["--config", f"{ROOT}/examples/configs/grpo_arithmetic_offline.yaml", "grpo.max_num_steps=2", "policy.model_name=tiny-nemotron-h",
                   f"logger.log_dir={tmp_path}/logs", f"checkpointing.checkpoint_dir={tmp_path}/ckpt"])
    out = capsys.readouterr().out
    assert "[grpo] step 2:" in out
    import re

    err = [float(x) for x in re.findall(r"mult_prob_err=([0-9.]+)", out)]
    assert err and all(e < 1.05 for e in err)      # engine and trainer agree on the sampled tokens' probabilities


def test_run_grpo_from_a_single_controller_over_worker_processes(capfd, tmp_path):
    """One controller process, two policy workers behind the worker-group facade, the ordinary GRPO loop on top."""
    from examples import run_grpo_controller

    run_grpo_controller.main(["--config", f"{ROOT}/examples/configs/grpo_arithmetic_offline.yaml", "grpo.max_num_steps=2", "cluster.gpus_per_node=2",
                              "+cluster.backend=gloo", f"logger.log_dir={tmp_path}/logs", f"checkpointing.checkpoint_dir={tmp_path}/ckpt",
                              "checkpointing.save_period=2", "checkpointing.enabled=true"])
    out = capfd.readouterr().out
    assert "[grpo] step 2:" in out
    assert os.path.exists(f"{tmp_path}/ckpt/step_2/policy/weights/config.json")


def test_run_sft_dpo_rm_eval(capsys):
    from examples import run_dpo, run_eval, run_rm, run_sft

    base = TINY + ["policy.max_total_sequence_length=64"]
    run_sft.main(["--config", f"{ROOT}/examples/configs/sft.yaml", *base, "sft.max_num_steps=2", "sft.val_period=0", "sft.val_at_start=false",
                  "data.train.dataset_name=random_sft", "data.validation.dataset_name=random_sft"])
    for mod, key in ((run_dpo, "dpo"), (run_rm, "rm")):
        mod.main(["--config", f"{ROOT}/examples/configs/{key}.yaml", *base, f"{key}.max_num_steps=2", f"{key}.val_period=0",
                  f"{key}.val_at_start=false", "data.train.dataset_name=random_preference", "data.validation.dataset_name=random_preference"])
    run_eval.main([a for a in TINY if "train_" not in a and "scheduler" not in a and "logger" not in a and "sequence_packing" not in a]
                  + ["policy.generation.max_new_tokens=8", "policy.generation.temperature=1.0", "eval.num_tests_per_prompt=2",
                     "eval.k_value=2", "data.validation.dataset_name=arithmetic", "+data.validation.num_val_samples=4", "data.default.prompt_file=null"])
    out = capsys.readouterr().out
    assert "[sft] step 2:" in out and "[dpo] step 2:" in out and "[rm] step 2:" in out and "pass@2=" in out


def test_run_grpo_single_controller_recipe(capsys):
    from examples import run_grpo_single_controller

    run_grpo_single_controller.main(["--config", f"{ROOT}/examples/configs/grpo_single_controller.yaml", "grpo.max_num_steps=2"])
    assert "[single_controller] step 2:" in capsys.readouterr().out


def test_run_xtoken_distillation_recipe(capsys):
    from examples import run_xtoken_off_policy_distillation as run

    run.main(["--config", f"{ROOT}/examples/configs/xtoken_distillation_offline.yaml", "distillation.max_num_steps=2", "data.num_samples=32"])
    assert "[xtoken_distillation] step 2:" in capsys.readouterr().out


def test_run_vlm_sft_and_grpo_recipes(capsys):
    from examples import run_vlm_grpo, run_vlm_sft

    run_vlm_sft.main(["--config", f"{ROOT}/examples/configs/vlm_sft_offline.yaml", "sft.max_num_steps=2", "data.train.num_samples=32"])
    run_vlm_grpo.main(["--config", f"{ROOT}/examples/configs/vlm_grpo_offline.yaml", "grpo.max_num_steps=1", "grpo.num_prompts_per_step=4",
                       "policy.train_global_batch_size=16"])
    out = capsys.readouterr().out
    assert "[sft] step 2:" in out and "[grpo] step 1:" in out
