"""Reward-model environment: scores conversations with a trained reward model (a :class:`PolicyWorker` whose model has
a scalar head), the role of nemo_rl/environments/reward_model_environment.py. The worker is passed in (or built from
``cfg["policy"]``) and shares the GPU with the policy in the SPMD runtime."""

from __future__ import annotations

from typing import Optional

import torch

from rl_b200.data.llm_message_utils import batched_message_log_to_flat_message
from rl_b200.distributed.batched_data_dict import BatchedDataDict
from rl_b200.environments.interfaces import EnvironmentReturn


class RewardModelEnvironment:
    def __init__(self, cfg: Optional[dict] = None, worker=None):
        self.cfg = cfg or {}
        self.worker = worker
        if self.worker is None and self.cfg.get("policy") is not None:
            from rl_b200.policy.worker import PolicyWorker

            mc = self.cfg.get("model_cfg")
            if mc is not None:
                mc.value_head = True
            self.worker = PolicyWorker(self.cfg["policy"], model_cfg=mc, init_optimizer=False, init_reference_model=False)
        self.pad = int(self.cfg.get("pad_token_id", 0))

    def step(self, message_log_batch, metadata) -> EnvironmentReturn:
        assert self.worker is not None, "RewardModelEnvironment needs a reward-model worker"
        flat, lens = batched_message_log_to_flat_message(message_log_batch, {"token_ids": self.pad})
        scores = self.worker.score(BatchedDataDict(input_ids=flat["token_ids"], input_lengths=lens))["scores"].float()
        n = len(message_log_batch)
        return EnvironmentReturn([{"role": "environment", "content": ""}] * n, list(metadata), [None] * n, scores,
                                 torch.ones(n, dtype=torch.bool), [None] * n)

    def global_post_process_and_metrics(self, batch):
        return batch, {"mean_rm_score": float(batch["total_reward"].float().mean())}

    def shutdown(self):
        pass
