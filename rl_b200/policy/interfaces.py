"""Contracts between the algorithm loops and the objects they drive (nemo_rl/models/policy/interfaces.py:51-262,
models/generation/interfaces.py:197-527, models/value/interfaces.py). The loops in ``rl_b200/algorithms`` use exactly these
methods, so any object that provides them (the in-tree :class:`PolicyWorker` / :class:`NativeGeneration`, a remote proxy, a
test double) can be plugged in."""

from __future__ import annotations

from typing import Any, Optional, Protocol, runtime_checkable

from rl_b200.distributed.batched_data_dict import BatchedDataDict


@runtime_checkable
class PolicyInterface(Protocol):
    def get_logprobs(self, data: BatchedDataDict, micro_batch_size: Optional[int] = None) -> BatchedDataDict:
        """``logprobs`` [B, S]: log p(token t | tokens < t) under the sampler's distribution, 0 at position 0 and on padding."""

    def get_reference_policy_logprobs(self, data: BatchedDataDict, micro_batch_size: Optional[int] = None) -> BatchedDataDict:
        """``reference_logprobs`` [B, S] under the frozen reference weights."""

    def get_topk_logits(self, data: BatchedDataDict, k: int, micro_batch_size: Optional[int] = None) -> BatchedDataDict:
        """``topk_logits`` / ``topk_indices`` [B, S-1, k] (teacher side of distillation)."""

    def train(self, data: BatchedDataDict, loss_fn: Any, eval_mode: bool = False, *, gbs: Optional[int] = None,
              mbs: Optional[int] = None) -> dict[str, Any]:
        """Optimizer steps over this rank's shard of ``data``; returns ``loss``, ``grad_norm`` and per-micro-batch metrics."""

    def prepare_for_training(self, *args, **kwargs) -> None: ...

    def prepare_for_lp_inference(self, *args, **kwargs) -> None: ...

    def finish_training(self, *args, **kwargs) -> None: ...

    def save_checkpoint(self, weights_path: str, optimizer_path: Optional[str] = None, tokenizer_path: Optional[str] = None, **kw) -> None: ...


@runtime_checkable
class ColocatablePolicyInterface(PolicyInterface, Protocol):
    """A policy that can hand its weights to a generation engine on the same devices."""

    def build_generation(self, gen_cfg: Optional[dict] = None) -> "GenerationInterface": ...

    def prepare_refit_info(self) -> dict:
        """HF name -> (shape, dtype) of every tensor a refit carries."""

    def offload_before_refit(self) -> None: ...

    def offload_after_refit(self) -> None: ...

    # an engine outside the trainer's job (nemo_rl/models/policy/interfaces.py:166-262)
    def init_collective(self, ip: str, port: int, world_size: int, *, train_world_size: int = 1) -> None: ...

    def broadcast_weights_for_collective(self, kv_scales: Any = None) -> int: ...

    def stream_weights_via_ipc_zmq(self, *args, **kwargs) -> int: ...


@runtime_checkable
class ValueInterface(Protocol):
    def score(self, data: BatchedDataDict, micro_batch_size: Optional[int] = None) -> BatchedDataDict:
        """``values`` [B, S] per token and ``scores`` [B] at each sequence's last token (critic / reward model)."""

    def train(self, data: BatchedDataDict, loss_fn: Any, eval_mode: bool = False, *, gbs: Optional[int] = None,
              mbs: Optional[int] = None) -> dict[str, Any]: ...


@runtime_checkable
class GenerationInterface(Protocol):
    def generate(self, data: BatchedDataDict, greedy: bool = False) -> BatchedDataDict:
        """Right-padded ``input_ids`` + ``input_lengths`` in; ``output_ids``, ``generation_lengths``,
        ``unpadded_sequence_lengths``, ``logprobs`` and ``truncated`` out."""

    def prepare_for_generation(self, *args, **kwargs) -> bool: ...

    def finish_generation(self, *args, **kwargs) -> bool: ...

    def invalidate_kv_cache(self) -> bool: ...

    def shutdown(self) -> bool: ...


@runtime_checkable
class RefittableGenerationInterface(GenerationInterface, Protocol):
    """The weight-receiving side (nemo_rl/models/generation/interfaces.py:392-527)."""

    def init_collective(self, rank_prefix: int, ip: str, port: int, world_size: int, *, train_world_size: int = 1) -> None: ...

    def prepare_refit_info(self, state_dict_info: Optional[dict] = None) -> None: ...

    def update_weights_from_collective(self) -> bool: ...

    def update_weights_via_ipc_zmq(self) -> bool: ...
