"""Task data processors: raw dataset record -> :class:`DatumSpec` (tokenised message log + what the environment needs).

Same role as nemo_rl/data/processors.py:140 (math), :382 (chat-template math), :882 (registry). A processor has the
signature ``(record, task_data_spec, tokenizer, max_seq_length, idx) -> DatumSpec``. Over-long prompts are truncated to a
stub and masked out with ``loss_multiplier = 0`` so batch shapes stay bounded.
"""

from __future__ import annotations

from typing import Any, Callable, Optional

import torch

from rl_b200.data.interfaces import DatumSpec, TaskDataSpec
from rl_b200.data.llm_message_utils import get_formatted_message_log


def _finish(log, extra, max_seq_length, idx, task_name, stop_strings=None) -> DatumSpec:
    length = sum(int(m["token_ids"].numel()) for m in log)
    mult = 1.0
    if max_seq_length is not None and length > max_seq_length:
        keep = max(1, min(4, max_seq_length // max(1, len(log))))
        for m in log:
            m["token_ids"] = m["token_ids"][:keep]
        length = sum(int(m["token_ids"].numel()) for m in log)
        mult = 0.0
    out: DatumSpec = {"message_log": log, "length": length, "extra_env_info": extra, "loss_multiplier": mult, "idx": idx,
                      "task_name": task_name}
    if stop_strings:
        out["stop_strings"] = stop_strings
    return out


def _chat(messages, tokenizer, generation_prompt: bool = True):
    return get_formatted_message_log(messages, tokenizer, add_eos_token=False, add_generation_prompt=generation_prompt)


def math_data_processor(rec: dict, spec: TaskDataSpec, tokenizer, max_seq_length: Optional[int], idx: int) -> DatumSpec:
    """``{problem, expected_answer}`` -> one user turn (the task prompt with ``{}`` filled by the problem)."""
    problem = rec.get("problem", rec.get("question", rec.get("prompt")))
    answer = rec.get("expected_answer", rec.get("answer", rec.get("ground_truth")))
    msgs = []
    if spec.system_prompt:
        msgs.append({"role": "system", "content": spec.system_prompt})
    msgs.append({"role": "user", "content": spec.prompt.format(problem) if spec.prompt else str(problem)})
    return _finish(_chat(msgs, tokenizer), {"ground_truth": str(answer)}, max_seq_length, idx, rec.get("task_name", spec.task_name or "math"))


def math_hf_data_processor(rec: dict, spec: TaskDataSpec, tokenizer, max_seq_length: Optional[int], idx: int) -> DatumSpec:
    """Records that already carry ``messages`` (user turn(s) then the reference answer as the last assistant turn)."""
    msgs = list(rec["messages"])
    answer = None
    if msgs and msgs[-1]["role"] == "assistant":
        answer = msgs.pop()["content"]
    if spec.prompt:
        msgs[-1] = {**msgs[-1], "content": spec.prompt.format(msgs[-1]["content"])}
    if spec.system_prompt and msgs[0]["role"] != "system":
        msgs.insert(0, {"role": "system", "content": spec.system_prompt})
    return _finish(_chat(msgs, tokenizer), {"ground_truth": str(rec.get("expected_answer", answer))}, max_seq_length, idx,
                   rec.get("task_name", spec.task_name or "math"))


def multichoice_qa_processor(rec: dict, spec: TaskDataSpec, tokenizer, max_seq_length: Optional[int], idx: int) -> DatumSpec:
    """``{question, options: {A: ..}|[..], answer}`` -> lettered multiple-choice prompt (MMLU / GPQA evaluation)."""
    opts = rec["options"]
    if isinstance(opts, (list, tuple)):
        opts = {chr(ord("A") + i): o for i, o in enumerate(opts)}
    body = str(rec["question"]) + "\n" + "\n".join(f"{k}) {v}" for k, v in opts.items())
    msgs = [{"role": "user", "content": spec.prompt.format(body) if spec.prompt else body}]
    return _finish(_chat(msgs, tokenizer), {"ground_truth": str(rec["answer"])}, max_seq_length, idx, rec.get("task_name", spec.task_name or "mcqa"))


def code_data_processor(rec: dict, spec: TaskDataSpec, tokenizer, max_seq_length: Optional[int], idx: int) -> DatumSpec:
    """``{prompt, tests | expected_output | ground_truth}`` for the code environments."""
    msgs = [{"role": "user", "content": spec.prompt.format(rec["prompt"]) if spec.prompt else rec["prompt"]}]
    extra = {k: rec[k] for k in ("tests", "expected_output", "ground_truth") if k in rec}
    return _finish(_chat(msgs, tokenizer), extra, max_seq_length, idx, rec.get("task_name", spec.task_name or "code"))


def sft_processor(rec: dict, spec: TaskDataSpec, tokenizer, max_seq_length: Optional[int], idx: int) -> DatumSpec:
    """``{messages}`` or ``{input/prompt, output/response}`` -> full conversation (trained on assistant turns)."""
    if "messages" in rec:
        msgs = list(rec["messages"])
    else:
        q = rec.get("input", rec.get("prompt", rec.get("question", rec.get("context"))))
        a = rec.get("output", rec.get("response", rec.get("answer", rec.get("answers"))))
        if isinstance(a, dict):  # squad-style {"text": [...]}
            a = a.get("text", [""])[0]
        if isinstance(a, (list, tuple)):
            a = a[0]
        msgs = [{"role": "user", "content": spec.prompt.format(q) if spec.prompt else str(q)}, {"role": "assistant", "content": str(a)}]
    if spec.system_prompt and msgs[0]["role"] != "system":
        msgs.insert(0, {"role": "system", "content": spec.system_prompt})
    log = get_formatted_message_log(msgs, tokenizer)
    return _finish(log, None, max_seq_length, idx, rec.get("task_name", spec.task_name or "sft"))


def preference_processor(rec: dict, spec: TaskDataSpec, tokenizer, max_seq_length: Optional[int], idx: int) -> dict:
    """``{prompt|context, chosen, rejected}`` (strings or message lists) or HelpSteer3-style
    ``{context, response1, response2, overall_preference}`` -> chosen / rejected message logs."""
    def as_msgs(x, role):
        return list(x) if isinstance(x, (list, tuple)) else [{"role": role, "content": str(x)}]

    if "overall_preference" in rec:
        pref = rec["overall_preference"]
        chosen, rejected = (rec["response1"], rec["response2"]) if pref < 0 or (pref == 0 and idx % 2 == 0) else (rec["response2"], rec["response1"])
    else:
        chosen, rejected = rec["chosen"], rec["rejected"]
    ctx = as_msgs(rec.get("prompt", rec.get("context", "")), "user")
    ch = get_formatted_message_log(ctx + as_msgs(chosen, "assistant"), tokenizer)
    rj = get_formatted_message_log(ctx + as_msgs(rejected, "assistant"), tokenizer)
    lc, lr = (sum(int(m["token_ids"].numel()) for m in x) for x in (ch, rj))
    mult = 1.0
    if max_seq_length is not None and max(lc, lr) > max_seq_length:
        mult = 0.0
        for log in (ch, rj):
            for m in log:
                m["token_ids"] = m["token_ids"][:2]
        lc, lr = (sum(int(m["token_ids"].numel()) for m in x) for x in (ch, rj))
    return {"message_log_chosen": ch, "message_log_rejected": rj, "length_chosen": lc, "length_rejected": lr,
            "loss_multiplier": mult, "idx": idx, "task_name": rec.get("task_name", spec.task_name or "preference")}


def token_prompt_processor(rec: dict, spec: TaskDataSpec, tokenizer, max_seq_length: Optional[int], idx: int) -> DatumSpec:
    """Records that are already token ids (``{"token_ids": [...]}``): no tokenizer involved."""
    ids = torch.as_tensor(rec["token_ids"], dtype=torch.long)
    return _finish([{"role": "user", "content": "", "token_ids": ids}], rec.get("extra_env_info"), max_seq_length, idx,
                   rec.get("task_name", spec.task_name or "synthetic"))


def nemogym_processor(rec: dict, spec: TaskDataSpec, tokenizer, max_seq_length: Optional[int], idx: int) -> DatumSpec:
    """Records of a gym-style resource server (nemo_rl/data/datasets/response_datasets/nemogym_dataset.py): the prompt is
    ``responses_create_params.input`` (or ``messages``), the whole record travels to the environment as ``extra_env_info``
    and the sample is routed by the agent that owns it (``agent_ref.name``)."""
    params = rec.get("responses_create_params") or {}
    msgs = params.get("input") or rec.get("messages") or [{"role": "user", "content": str(rec.get("question", rec.get("problem", "")))}]
    if isinstance(msgs, str):
        msgs = [{"role": "user", "content": msgs}]
    msgs = [{"role": m.get("role", "user"), "content": m.get("content", "")} for m in msgs]
    agent = (rec.get("agent_ref") or {}).get("name") or rec.get("task_name") or spec.task_name or "nemo_gym"
    out = _finish(_chat(msgs, tokenizer), dict(rec), max_seq_length, idx, agent)
    out["agent_ref"] = agent
    return out


def vlm_processor(rec: dict, spec: TaskDataSpec, tokenizer, max_seq_length: Optional[int], idx: int) -> DatumSpec:
    """Image sets need the model's patch size and image token: they are built by
    :func:`rl_b200.data.datasets.vlm.setup_vlm_data` (``examples/run_vlm_grpo.py`` / ``run_vlm_sft.py``), not by name."""
    raise RuntimeError("vision-language records are processed by rl_b200.data.datasets.vlm.make_vlm_processor (it needs the model's "
                       "patch size and image token id); use setup_vlm_data / the run_vlm_* entry points")


PROCESSOR_REGISTRY: dict[str, Callable[..., Any]] = {
    "default": math_hf_data_processor,
    "math_data_processor": math_data_processor,
    "math_hf_data_processor": math_hf_data_processor,
    "multichoice_qa_processor": multichoice_qa_processor,
    "code_data_processor": code_data_processor,
    "sft_processor": sft_processor,
    "preference_processor": preference_processor,
    "token_prompt_processor": token_prompt_processor,
    "nemogym_processor": nemogym_processor,
    "vlm_processor": vlm_processor,
}


def register_processor(name: str, fn: Callable[..., Any]) -> None:
    PROCESSOR_REGISTRY[name] = fn


def get_processor(name: Optional[str]) -> Callable[..., Any]:
    name = name or "default"
    if name not in PROCESSOR_REGISTRY:
        raise KeyError(f"unknown processor '{name}' ({sorted(PROCESSOR_REGISTRY)})")
    return PROCESSOR_REGISTRY[name]
