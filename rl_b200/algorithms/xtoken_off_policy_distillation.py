"""Off-policy distillation between models with different tokenizers.

A text corpus is tokenised twice; the teacher (its own tokenizer and vocabulary) scores its tokenisation, the student is
trained on its own tokenisation to match the teacher where the two can be compared (see ``x_token``). Loop and
configuration follow nemo_rl/algorithms/xtoken_off_policy_distillation.py: loader -> teacher inference -> alignment ->
``student.train`` with :class:`CrossTokenizerDistillationLossFn`.
"""

from __future__ import annotations

from typing import Callable, Optional

from rl_b200.algorithms.grpo import _ShardedPromptLoader, _aggregate_train_metrics, _is_main, _world, save_checkpoint
from rl_b200.algorithms.utils import set_seed
from rl_b200.algorithms.x_token import CrossTokenizerDistillationLossFn, TokenAligner, build_vocab_projection
from rl_b200.algorithms.x_token.loss import prepare_xtoken_batch
from rl_b200.utils.checkpoint import CheckpointManager
from rl_b200.utils.logger import Logger
from rl_b200.utils.timer import Timer

XTOKEN_DEFAULTS = dict(max_num_epochs=1, max_num_steps=1_000_000, topk_logits_k=16, seed=42, text_key="text")


def _texts(items, key: str, tokenizer) -> list[str]:
    out = []
    for it in items:
        if isinstance(it, str):
            out.append(it)
        elif key in it:
            out.append(it[key])
        elif "messages" in it:
            out.append(tokenizer.apply_chat_template(it["messages"], tokenize=False))
        else:
            raise KeyError(f"sample has neither {key!r} nor 'messages'")
    return out


def setup(cfg: dict, student_tokenizer, teacher_tokenizer, dataset, student_cfg=None, teacher_cfg=None, student=None, teacher=None):
    """Returns (student, teacher, loader, aligner, projection, loss_fn, logger, checkpointer, save_state, cfg)."""
    from rl_b200.policy.worker import PolicyWorker, ensure_parallel

    ensure_parallel(cfg["policy"])
    rank, world = _world()
    d = dict(XTOKEN_DEFAULTS)
    d.update(cfg.get("distillation") or {})
    cfg["distillation"] = d
    set_seed(d["seed"] + rank)
    logger = Logger(cfg.get("logger"), is_main=_is_main())
    checkpointer = CheckpointManager(cfg.get("checkpointing"))
    save_state = {"current_step": 0, "total_steps": 0, "current_epoch": 0}
    loader = _ShardedPromptLoader(dataset, cfg["policy"]["train_global_batch_size"], list, bool((cfg.get("data") or {}).get("shuffle", True)),
                                  d["seed"], rank, world)
    if student is None:
        student = PolicyWorker(cfg["policy"], model_cfg=student_cfg, tokenizer=student_tokenizer, init_reference_model=False, seed=d["seed"])
    if teacher is None:
        teacher = PolicyWorker(cfg.get("teacher") or cfg["policy"], model_cfg=teacher_cfg, tokenizer=teacher_tokenizer, init_optimizer=False,
                               init_reference_model=False, seed=d["seed"] + 17)
    aligner = TokenAligner(student_tokenizer, teacher_tokenizer)
    proj = build_vocab_projection(student_tokenizer, teacher_tokenizer, student.model_cfg.vocab_size, teacher.model_cfg.vocab_size)
    return student, teacher, loader, aligner, proj, CrossTokenizerDistillationLossFn(cfg.get("loss_fn")), logger, checkpointer, save_state, cfg


def xtoken_distillation_train(student, teacher, loader, aligner, proj, loss_fn, logger, checkpointer, save_state, cfg,
                              step_callback: Optional[Callable] = None) -> dict:
    d, pcfg = cfg["distillation"], cfg["policy"]
    timer = Timer()
    total_steps, epoch = save_state["total_steps"], save_state["current_epoch"]
    last: dict = {}
    while epoch < d["max_num_epochs"] and total_steps < d["max_num_steps"]:
        for items in loader:
            if total_steps >= d["max_num_steps"]:
                break
            with timer.time("total_step_time"):
                with timer.time("teacher_inference_and_alignment"):
                    data = prepare_xtoken_batch(_texts(items, d["text_key"], aligner.s_tok), aligner, proj, teacher, int(d["topk_logits_k"]),
                                                int(pcfg["max_total_sequence_length"]), pcfg.get("logprob_batch_size"))
                with timer.time("policy_training"):
                    student.prepare_for_training()
                    res = student.train(data, loss_fn, gbs=pcfg["train_global_batch_size"], mbs=pcfg["train_micro_batch_size"])
            total_steps += 1
            metrics = _aggregate_train_metrics(res)
            save_state.update(current_step=total_steps, total_steps=total_steps, current_epoch=epoch)
            timing = timer.get_timing_metrics("sum")
            ck = cfg.get("checkpointing") or {}
            if checkpointer.enabled and ck.get("save_period") and total_steps % ck["save_period"] == 0:
                save_checkpoint(student, loader, checkpointer, save_state, cfg, total_steps)
            if logger is not None:
                logger.log_metrics(metrics, total_steps, prefix="train")
                logger.log_metrics(timing, total_steps, prefix="timing/train")
            if _is_main():
                print(f"[xtoken_distillation] step {total_steps}: loss={metrics['loss']:.5f} next_token_kl={metrics.get('next_token_kl', 0):.5f} "
                      f"chunk={metrics.get('chunk_loss', 0):.5f}", flush=True)
            last = {"train": metrics, "timing": timing}
            if step_callback is not None:
                step_callback(total_steps, last)
            timer.reset()
        epoch += 1
        save_state["current_epoch"] = epoch
    return last
