"""Value model facade: a critic or reward model is a policy worker whose model ends in a scalar head.

``ValueModel`` builds such a worker from a ``value`` / ``reward_model`` config block and exposes only what a value model
does (score, train, checkpoint), so that algorithm code cannot generate from it or ask it for log-probabilities by accident
(nemo_rl/models/value/lm_value.py and its interfaces).
"""

from __future__ import annotations

from typing import Any, Optional

from rl_b200.distributed.batched_data_dict import BatchedDataDict


class ValueModel:
    def __init__(self, value_cfg: dict, model_cfg=None, tokenizer=None, device=None, seed: int = 0, worker=None, **kw):
        from rl_b200.policy.worker import PolicyWorker

        if worker is None:
            if model_cfg is not None:
                from dataclasses import replace

                model_cfg = replace(model_cfg, value_head=True)
            worker = PolicyWorker(dict(value_cfg, value_head=True), model_cfg=model_cfg, tokenizer=tokenizer, device=device,
                                  init_reference_model=False, seed=seed, **kw)
        assert worker.model_cfg.value_head, "a value model needs a scalar head (model_cfg.value_head)"
        self.worker = worker

    def get_values(self, data: BatchedDataDict, micro_batch_size: Optional[int] = None) -> BatchedDataDict:
        """``values`` [B, S] per token and ``scores`` [B] at each sequence's last token."""
        return self.worker.score(data, micro_batch_size)

    score = get_values

    def train(self, data: BatchedDataDict, loss_fn: Any, eval_mode: bool = False, *, gbs: Optional[int] = None, mbs: Optional[int] = None):
        return self.worker.train(data, loss_fn, eval_mode, gbs=gbs, mbs=mbs)

    def prepare_for_training(self, *a, **k):
        return self.worker.prepare_for_training(*a, **k)

    def prepare_for_inference(self, *a, **k):
        return self.worker.prepare_for_lp_inference(*a, **k)

    def save_checkpoint(self, *a, **k):
        return self.worker.save_checkpoint(*a, **k)

    def load_checkpoint(self, *a, **k):
        return self.worker.load_checkpoint(*a, **k)

    def shutdown(self) -> bool:
        return self.worker.shutdown()
