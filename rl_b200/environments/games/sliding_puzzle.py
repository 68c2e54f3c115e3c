"""Sliding-puzzle game environment (multi-turn): the model emits moves, the environment answers with the new board
until the puzzle is solved or the move budget is spent (the game of nemo_rl/environments/games/sliding_puzzle.py).

State lives in ``extra_env_info`` (``{"grid": [[...]], "moves": n, "max_moves": m, "size": s}``); the action is parsed
from ``<action>up|down|left|right</action>`` (the blank moves in that direction). Reward 1 on the solving move.
"""

from __future__ import annotations

import random
import re
from typing import Optional

import torch

from rl_b200.environments.interfaces import EnvironmentReturn

_DIRS = {"up": (-1, 0), "down": (1, 0), "left": (0, -1), "right": (0, 1)}


def solved_grid(size: int) -> list[list[int]]:
    g = [[r * size + c + 1 for c in range(size)] for r in range(size)]
    g[-1][-1] = 0
    return g


def apply_move(grid: list[list[int]], move: str) -> bool:
    size = len(grid)
    r, c = next((i, j) for i in range(size) for j in range(size) if grid[i][j] == 0)
    dr, dc = _DIRS[move]
    nr, nc = r + dr, c + dc
    if not (0 <= nr < size and 0 <= nc < size):
        return False
    grid[r][c], grid[nr][nc] = grid[nr][nc], grid[r][c]
    return True


def generate_puzzle(size: int, shuffle_moves: int, rng: random.Random) -> list[list[int]]:
    g = solved_grid(size)
    done = 0
    while done < shuffle_moves:
        if apply_move(g, rng.choice(list(_DIRS))):
            done += 1
    if g == solved_grid(size):
        apply_move(g, "up") or apply_move(g, "left")
    return g


def render(grid: list[list[int]]) -> str:
    w = len(str(len(grid) ** 2))
    return "\n".join(" ".join((str(v) if v else "_").rjust(w) for v in row) for row in grid)


def make_initial_state(size: int = 3, shuffle_moves: int = 10, max_moves: int = 30, seed: int = 0) -> dict:
    return {"grid": generate_puzzle(size, shuffle_moves, random.Random(seed)), "moves": 0, "max_moves": max_moves, "size": size}


def initial_prompt(state: dict) -> str:
    return ("Solve the sliding puzzle by moving the blank (_). Reply with one move per turn as "
            "<action>up|down|left|right</action>.\n" + render(state["grid"]))


class SlidingPuzzleEnv:
    def __init__(self, cfg: Optional[dict] = None):
        self.cfg = cfg or {}

    def step(self, message_log_batch, metadata) -> EnvironmentReturn:
        n = len(message_log_batch)
        obs, metas, rewards, term = [], [], torch.zeros(n), torch.zeros(n, dtype=torch.bool)
        for i, (log, md) in enumerate(zip(message_log_batch, metadata)):
            md = {**md, "grid": [row[:] for row in md["grid"]]}
            text = next((str(m["content"]) for m in reversed(log) if m["role"] == "assistant"), "")
            m = re.findall(r"<action>\s*(up|down|left|right)\s*</action>", text, flags=re.I)
            md["moves"] += 1
            if not m:
                msg = "Invalid action. Use <action>up|down|left|right</action>."
            elif not apply_move(md["grid"], m[-1].lower()):
                msg = "That move leaves the board.\n" + render(md["grid"])
            else:
                msg = render(md["grid"])
            if md["grid"] == solved_grid(md["size"]):
                rewards[i] = 1.0
                term[i] = True
                msg = "Solved!\n" + msg
            elif md["moves"] >= md["max_moves"]:
                term[i] = True
                msg = "Out of moves.\n" + msg
            obs.append({"role": "environment", "content": "\n" + msg + "\n"})
            metas.append(md)
        return EnvironmentReturn(obs, metas, [["</action>"]] * n, rewards, term, [None] * n)

    def global_post_process_and_metrics(self, batch):
        r = batch["total_reward"].float()
        return batch, {"success_rate": float((r > 0).float().mean()) if len(r) else 0.0}

    def shutdown(self):
        pass
