"""Dataset registry and ``setup_response_data`` (the role of nemo_rl/data/utils.py:107 and nemo_rl/data/datasets/).

Raw sources:
  * ``arithmetic``        -- built-in generator of integer arithmetic problems (offline; used by the examples)
  * ``jsonl`` / ``json``  -- local files, one record per line
  * ``random_tokens``     -- uniform-random token prompts (benchmarks)
  * named HuggingFace sets (``OpenMathInstruct-2``, ``DeepScaler``, ``DAPOMath17K``, ``AIME2024``, ``MATH-500``,
    ``gsm8k``, ``squad``, ``tulu3_sft_mixture``, ``HelpSteer3``, ``Tulu3Preference``...) or any ``hf:<path>`` --
    loaded through ``datasets.load_dataset`` (needs the set in the local HF cache when there is no network).
A raw source yields plain dict records; :class:`ProcessedDataset` applies a task processor lazily per item.
"""

from __future__ import annotations

import json
import random
from typing import Any, Callable, Optional

from rl_b200.data.interfaces import TaskDataSpec
from rl_b200.data.processors import get_processor

# name -> (hf path, config name, train split, val split, field renames, default processor)
HF_SETS: dict[str, tuple] = {
    "OpenMathInstruct-2": ("nvidia/OpenMathInstruct-2", None, "train_1M", None, {"problem": "problem", "expected_answer": "expected_answer"}, "math_data_processor"),
    "DeepScaler": ("agentica-org/DeepScaleR-Preview-Dataset", None, "train", None, {"problem": "problem", "answer": "expected_answer"}, "math_data_processor"),
    "DAPOMath17K": ("BytedTsinghua-SIA/DAPO-Math-17k", None, "train", None, {"prompt": "problem", "reward_model": "expected_answer"}, "math_data_processor"),
    "AIME2024": ("HuggingFaceH4/aime_2024", None, "train", None, {"problem": "problem", "answer": "expected_answer"}, "math_data_processor"),
    "AIME2025": ("opencompass/AIME2025", "AIME2025-I", "test", None, {"question": "problem", "answer": "expected_answer"}, "math_data_processor"),
    "MATH-500": ("HuggingFaceH4/MATH-500", None, "test", None, {"problem": "problem", "answer": "expected_answer"}, "math_data_processor"),
    "gsm8k": ("openai/gsm8k", "main", "train", "test", {"question": "problem", "answer": "expected_answer"}, "math_data_processor"),
    "GPQA": ("Idavidrein/gpqa", "gpqa_diamond", "train", None, {}, "multichoice_qa_processor"),
    "MMLU": ("cais/mmlu", "all", "test", None, {"choices": "options"}, "multichoice_qa_processor"),
    "MMLU-Pro": ("TIGER-Lab/MMLU-Pro", None, "test", "validation", {}, "multichoice_qa_processor"),
    "hendrycks_math": ("EleutherAI/hendrycks_math", "algebra", "train", "test", {"problem": "problem", "solution": "expected_answer"}, "math_data_processor"),
    "NuminaMath": ("AI-MO/NuminaMath-CoT", None, "train", "test", {"problem": "problem", "solution": "expected_answer"}, "math_data_processor"),
    "Nemotron-Post-Training-v1-math": ("nvidia/Nemotron-Post-Training-Dataset-v1", None, "math", None, {}, "sft_processor"),
    "squad": ("rajpurkar/squad", None, "train", "validation", {}, "sft_processor"),
    "tulu3_sft_mixture": ("allenai/tulu-3-sft-mixture", None, "train", None, {}, "sft_processor"),
    "openai_format": (None, None, "train", None, {}, "sft_processor"),
    "oasst": ("OpenAssistant/oasst1", None, "train", "validation", {}, "sft_processor"),
    "HelpSteer3": ("nvidia/HelpSteer3", "preference", "train", "validation", {}, "preference_processor"),
    "Tulu3Preference": ("allenai/llama-3.1-tulu-3-8b-preference-mixture", None, "train", None, {}, "preference_processor"),
    "OpenR1-Math-220k": ("open-r1/OpenR1-Math-220k", "default", "train", None, {"problem": "problem", "answer": "expected_answer"}, "math_data_processor"),
    "Nemotron-Cascade-2-SFT-math": ("nvidia/Nemotron-Cascade-2-SFT-Data", "math", "train", None, {}, "sft_processor"),
    "geometry3k": ("hiyouga/geometry3k", None, "train", "validation", {"problem": "problem", "answer": "expected_answer"}, "vlm_processor"),
    "clevr-cogent": ("MMInstruction/Clevr_CoGenT_TrainA_R1", None, "train", None, {"problem": "problem", "solution": "expected_answer"}, "vlm_processor"),
    "refcoco": ("jxu124/refcoco", None, "train", "validation", {}, "vlm_processor"),
    "mmpr-tiny": ("OpenGVLab/MMPR-Tiny", None, "train", None, {}, "vlm_processor"),
    "avqa": ("gijs/avqa-processed", None, "train", "validation", {"question": "problem", "answer": "expected_answer"}, "multichoice_qa_processor"),
    "MMAU": ("TwinkStart/MMAU", None, "test", None, {"question": "problem", "answer": "expected_answer", "choices": "options"}, "multichoice_qa_processor"),
    "intent": (None, None, "train", "validation", {"text": "problem", "label": "expected_answer"}, "math_data_processor"),
    "general_conversations": (None, None, "train", "validation", {}, "sft_processor"),
    "BinaryPreferenceDataset": (None, None, "train", "validation", {}, "preference_processor"),
    "arrow_text": (None, None, "train", None, {}, "sft_processor"),
    "local_math": (None, None, "train", None, {}, "math_data_processor"),
    "nemogym": (None, None, "train", "validation", {}, "nemogym_processor"),
}


class ArithmeticDataset:
    """``a op b`` problems with integer answers; deterministic in ``seed``."""

    def __init__(self, num_samples: int = 1024, max_operand: int = 99, ops: str = "+-*", seed: int = 0):
        rng = random.Random(seed)
        self.records = []
        for _ in range(num_samples):
            a, b, op = rng.randint(0, max_operand), rng.randint(0, max_operand), rng.choice(ops)
            ans = {"+": a + b, "-": a - b, "*": a * b}[op]
            self.records.append({"problem": f"What is {a} {op} {b}?", "expected_answer": str(ans)})

    def __len__(self):
        return len(self.records)

    def __getitem__(self, i):
        return self.records[i]


class JsonlRecords:
    def __init__(self, path: str, renames: Optional[dict] = None):
        self.records = []
        with open(path) as f:
            first = f.read(1)
            f.seek(0)
            rows = json.load(f) if first == "[" else (json.loads(l) for l in f if l.strip())
            for r in rows:
                for k, v in (renames or {}).items():
                    if k in r:
                        r[v] = r.pop(k)
                self.records.append(r)

    def __len__(self):
        return len(self.records)

    def __getitem__(self, i):
        return self.records[i]


class ArrowRecords:
    """Rows of a local Arrow IPC / Parquet file (the arrow_text data sets of the reference,
    nemo_rl/data/datasets/response_datasets/arrow_text_dataset.py)."""

    def __init__(self, path: str, renames: Optional[dict] = None, max_samples: Optional[int] = None):
        import pyarrow as pa
        import pyarrow.parquet as pq

        if str(path).endswith(".parquet"):
            table = pq.read_table(path)
        else:
            with pa.memory_map(path, "r") as src:
                try:
                    table = pa.ipc.open_file(src).read_all()
                except pa.ArrowInvalid:
                    table = pa.ipc.open_stream(src).read_all()
        if max_samples:
            table = table.slice(0, max_samples)
        self.rows = table.to_pylist()
        self.renames = renames or {}

    def __len__(self):
        return len(self.rows)

    def __getitem__(self, i):
        r = dict(self.rows[i])
        for a, b in self.renames.items():
            if a in r and b not in r:
                r[b] = r[a]
        return r


class HFRecords:
    def __init__(self, path: str, name: Optional[str], split: str, renames: Optional[dict] = None, max_samples: Optional[int] = None):
        try:
            import datasets
        except ImportError as e:  # pragma: no cover
            raise RuntimeError("HuggingFace `datasets` is needed for named datasets") from e
        ds = datasets.load_dataset(path, name, split=split)
        if max_samples:
            ds = ds.select(range(min(max_samples, len(ds))))
        self.ds, self.renames = ds, renames or {}

    def __len__(self):
        return len(self.ds)

    def __getitem__(self, i):
        r = dict(self.ds[int(i)])
        for k, v in self.renames.items():
            if k in r:
                val = r.pop(k)
                if k == "reward_model" and isinstance(val, dict):
                    val = val.get("ground_truth")
                if k == "prompt" and isinstance(val, list):
                    val = val[-1]["content"]
                r[v] = val
        return r


class ProcessedDataset:
    """Applies ``processor(record, task_spec, tokenizer, max_seq_length, idx)`` on access
    (nemo_rl/data/datasets/processed_dataset.py ``AllTaskProcessedDataset``). ``processor`` / ``task_spec`` may be dicts
    keyed by the record's ``task_name`` for multi-task mixtures."""

    def __init__(self, records, tokenizer, task_spec, processor, max_seq_length: Optional[int] = None, cache: bool = True):
        self.records, self.tokenizer, self.task_spec, self.processor = records, tokenizer, task_spec, processor
        self.max_seq_length = max_seq_length
        self._cache: Optional[dict[int, Any]] = {} if cache else None

    def __len__(self):
        return len(self.records)

    def __getitem__(self, i):
        i = int(i)
        if self._cache is not None and i in self._cache:
            item = self._cache[i]
        else:
            rec = self.records[i]
            task = rec.get("task_name") if isinstance(rec, dict) else None
            proc = self.processor[task] if isinstance(self.processor, dict) else self.processor
            spec = self.task_spec[task] if isinstance(self.task_spec, dict) else self.task_spec
            item = proc(rec, spec, self.tokenizer, self.max_seq_length, i)
            if self._cache is not None:
                self._cache[i] = item
        out = dict(item)
        for k in ("message_log", "message_log_chosen", "message_log_rejected"):
            if k in out:
                out[k] = [dict(m) for m in out[k]]
        return out


def load_raw_dataset(dcfg: dict, split: str = "train"):
    """``dcfg``: ``{dataset_name, data_path?, split?, max_samples?, seed?, ...}`` -> (records, default processor name)."""
    name = dcfg.get("dataset_name", "arithmetic")
    if name == "arithmetic":
        n = dcfg.get("num_samples", 1024) if split == "train" else dcfg.get("num_val_samples", 64)
        return ArithmeticDataset(n, dcfg.get("max_operand", 99), dcfg.get("ops", "+-*"), seed=dcfg.get("seed", 0) + (0 if split == "train" else 1)), "math_data_processor"
    if name in ("intent", "general_conversations", "BinaryPreferenceDataset", "arrow_text", "local_math", "nemogym") and dcfg.get("data_path"):
        # sets that live in local files (jsonl / json / arrow / parquet): the registry row supplies renames and the processor
        _, _, _, _, renames, proc = HF_SETS[name]
        path = dcfg["data_path"] if split == "train" else dcfg.get("val_data_path")
        if path is None:
            return None, None
        renames = dict(renames, **{dcfg[k]: v for k, v in (("input_key", "problem"), ("output_key", "expected_answer"),
                                                           ("problem_key", "problem"), ("solution_key", "expected_answer")) if dcfg.get(k)})
        if str(path).endswith((".arrow", ".parquet")):
            return ArrowRecords(path, renames, dcfg.get("max_samples")), proc
        return JsonlRecords(path, renames), proc
    if name in ("jsonl", "json", "ResponseDataset", "PreferenceDataset", "openai_format"):
        path = dcfg["data_path"] if split == "train" else dcfg.get("val_data_path")
        if path is None:
            return None, None
        renames = {dcfg[k]: v for k, v in (("input_key", "problem"), ("output_key", "expected_answer")) if dcfg.get(k)}
        default = {"PreferenceDataset": "preference_processor", "openai_format": "sft_processor"}.get(name, "math_data_processor")
        return JsonlRecords(path, renames), default
    if name == "random_tokens":
        from rl_b200.data.datasets.synthetic import RandomTokenPromptDataset

        return RandomTokenPromptDataset(dcfg.get("num_samples", 1024), dcfg["min_prompt_len"], dcfg["max_prompt_len"], dcfg["vocab_size"],
                                        seed=dcfg.get("seed", 0), task_name=dcfg.get("env_name", "synthetic")), None
    if name in HF_SETS or name.startswith("hf:"):
        path, cfgname, tr, va, renames, proc = HF_SETS.get(name, (name[3:], dcfg.get("subset"), "train", None, {}, "math_data_processor"))
        sp = dcfg.get("split") or (tr if split == "train" else (dcfg.get("split_validation") or va))
        if sp is None:
            return None, None
        return HFRecords(path or dcfg["data_path"], cfgname, sp, renames, dcfg.get("max_samples")), proc
    raise KeyError(f"unknown dataset '{name}'")


def setup_response_data(tokenizer, data_cfg: dict, env_cfgs: Optional[dict] = None, is_eval: bool = False):
    """Builds (train dataset, val dataset, task_to_env, val_task_to_env) from the ``data:`` and ``env:`` config trees.

    ``data.train`` / ``data.validation`` hold dataset specs (a dict or a list of dicts for mixtures); ``data.default``
    supplies shared keys (``prompt_file``, ``system_prompt_file``, ``processor``, ``env_name``)."""
    from rl_b200.environments.registry import create_env

    default = dict(data_cfg.get("default") or {})
    max_len = data_cfg.get("max_input_seq_length")

    def build(specs, split):
        if specs is None:
            return None, set()
        specs = specs if isinstance(specs, list) else [specs]
        parts, envs = [], set()
        for s in specs:
            s = {**default, **s}
            recs, proc_default = load_raw_dataset(s, split)
            if recs is None:
                continue
            env_name = s.get("env_name", "math")
            envs.add(env_name)
            if proc_default is None:  # already DatumSpecs
                parts.append(recs)
                continue
            spec = TaskDataSpec(task_name=env_name, prompt_file=s.get("prompt_file"), system_prompt_file=s.get("system_prompt_file"),
                                prompt=s.get("prompt"), system_prompt=s.get("system_prompt"))
            parts.append(ProcessedDataset(recs, tokenizer, spec, get_processor(s.get("processor") or proc_default), max_len))
        if not parts:
            return None, envs
        return (parts[0] if len(parts) == 1 else ConcatDataset(parts)), envs

    train, envs_t = build(data_cfg.get("train") or ({"dataset_name": data_cfg["dataset_name"], **data_cfg} if "dataset_name" in data_cfg else None),
                          "train")
    val_spec = data_cfg.get("validation")
    if val_spec is None and data_cfg.get("train") is not None and not is_eval:
        val_spec = data_cfg["train"]
    val, envs_v = build(val_spec, "validation")
    env_cfgs = env_cfgs or {}
    made = {n: create_env(n, env_cfgs.get(n) or {}) for n in envs_t | envs_v}
    return train, val, {n: made[n] for n in envs_t}, {n: made[n] for n in (envs_v or envs_t)}


class ConcatDataset:
    def __init__(self, parts):
        self.parts = parts
        self.offsets = [0]
        for p in parts:
            self.offsets.append(self.offsets[-1] + len(p))

    def __len__(self):
        return self.offsets[-1]

    def __getitem__(self, i):
        import bisect

        k = bisect.bisect_right(self.offsets, int(i)) - 1
        item = self.parts[k][int(i) - self.offsets[k]]
        item["idx"] = int(i)
        return item


def load_text_corpus(data_cfg: dict) -> list[dict]:
    """Plain-text corpus for off-policy distillation: ``{"text": ...}`` records.

    ``dataset_name``: ``arithmetic_text`` (synthetic, offline), ``text`` (``path``: one document per line) or ``jsonl``
    (``path``; ``text_key`` names the field, records with ``messages`` are kept as they are)."""
    name = data_cfg.get("dataset_name", "arithmetic_text")
    if name == "arithmetic_text":
        ds = ArithmeticDataset(int(data_cfg.get("num_samples", 1024)), seed=int(data_cfg.get("seed", 0)))
        return [{"text": f"{r['problem']} The answer is {r['expected_answer']}."} for r in ds.records]
    if name == "text":
        with open(data_cfg["path"]) as f:
            return [{"text": l.rstrip("\n")} for l in f if l.strip()]
    if name == "jsonl":
        key = data_cfg.get("text_key", "text")
        return [r if "messages" in r and key not in r else {"text": r[key]} for r in JsonlRecords(data_cfg["path"]).records]
    raise ValueError(f"unknown text corpus {name!r}")
