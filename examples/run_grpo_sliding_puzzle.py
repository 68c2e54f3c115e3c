"""Multi-turn GRPO on the sliding-puzzle game (reference: examples/run_grpo_sliding_puzzle.py).

    python examples/run_grpo_sliding_puzzle.py --config examples/configs/grpo_sliding_puzzle.yaml
"""

import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

from rl_b200.algorithms import grpo  # noqa: E402
from rl_b200.data.llm_message_utils import get_formatted_message_log  # noqa: E402
from rl_b200.distributed.launch import shutdown_distributed  # noqa: E402
from rl_b200.environments.games.sliding_puzzle import SlidingPuzzleEnv, initial_prompt, make_initial_state  # noqa: E402
from rl_b200.utils.cli import bootstrap, model_cfg_for_tokenizer  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


class PuzzleDataset:
    """A fresh, seed-determined puzzle per index: the dataset is procedural, so ``length`` only bounds an epoch."""

    def __init__(self, tokenizer, game_cfg: dict, length: int, seed: int = 0):
        self.tok, self.g, self.length, self.seed = tokenizer, game_cfg, length, seed

    def __len__(self):
        return self.length

    def __getitem__(self, i):
        st = make_initial_state(self.g.get("size", 3), self.g.get("shuffle_moves", 6), self.g.get("max_moves", 20), seed=self.seed + int(i))
        log = get_formatted_message_log([{"role": "user", "content": initial_prompt(st)}], self.tok, add_eos_token=False,
                                        add_generation_prompt=True)
        return {"message_log": log, "length": sum(int(m["token_ids"].numel()) for m in log), "extra_env_info": st, "loss_multiplier": 1.0,
                "idx": int(i), "task_name": "sliding_puzzle", "stop_strings": ["</action>"]}


def main(argv=None):
    cfg, rank, world, device, tokenizer = bootstrap(os.path.join(HERE, "configs", "grpo_sliding_puzzle.yaml"), argv)
    game = (cfg.get("env") or {}).get("sliding_puzzle_game", {}).get("cfg", {}).get("game_config", {})
    n = cfg["grpo"]["num_prompts_per_step"] * min(cfg["grpo"]["max_num_steps"], 1000)
    train = PuzzleDataset(tokenizer, game, n, seed=cfg["grpo"].get("seed", 42))
    val = PuzzleDataset(tokenizer, game, cfg["grpo"].get("max_val_samples", 32), seed=10_000_000)
    envs = {"sliding_puzzle": SlidingPuzzleEnv(game)}
    policy, generation, loader, val_loader, loss_fn, logger, ck, save_state, cfg = grpo.setup(
        cfg, tokenizer, train, val, envs, envs, model_cfg=model_cfg_for_tokenizer(cfg, tokenizer))
    try:
        grpo.grpo_train(policy, generation, loader, val_loader, tokenizer, loss_fn, envs, envs, logger, ck, save_state, cfg)
    finally:
        shutdown_distributed()


if __name__ == "__main__":
    main()
