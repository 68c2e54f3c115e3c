"""Pipeline parallelism: contiguous layer ranges per stage, activations and their gradients exchanged with
``torch.distributed`` point-to-point calls (NCCL send/recv over NVLink on GPUs, gloo on CPU), micro-batches scheduled
one-forward-one-backward (1F1B) so that a stage holds at most ``pp - stage`` micro-batches of activations.

``PipelineRunner.train_step(microbatches, loss_fn)`` runs one accumulation window; ``forward_only`` runs inference and
returns the last stage's outputs on every stage (broadcast inside the pipeline group). The reference reaches pipeline
parallelism through Megatron's schedules (``forward_backward_func`` in nemo_rl/models/megatron/train.py) and the
``pipeline_model_parallel_size`` key of ``policy.megatron_cfg``.
"""

from __future__ import annotations

from typing import Any, Callable, Optional, Sequence

import torch
import torch.distributed as dist


class PipelineRunner:
    def __init__(self, model, pp_group, pp_rank: int, pp_size: int, hidden_size: int, dtype: torch.dtype, device,
                 rows_of: Optional[Callable[[Any], int]] = None):
        """``rows_of(batch)``: rows of the activation tensor a stage hands on for ``batch`` (token count, divided by the
        tensor-parallel size under sequence parallelism)."""
        self.model, self.group, self.rank, self.size = model, pp_group, pp_rank, pp_size
        self.hidden, self.dtype, self.device = hidden_size, dtype, torch.device(device)
        self.rows_of = rows_of or (lambda b: int(b.input_ids.numel()))
        self.first, self.last = pp_rank == 0, pp_rank == pp_size - 1
        self._prev = dist.get_global_rank(pp_group, pp_rank - 1) if not self.first else None
        self._next = dist.get_global_rank(pp_group, pp_rank + 1) if not self.last else None

    # ------------------------------------------------------------------ p2p
    def _exchange(self, send_t: Optional[torch.Tensor], recv_rows: Optional[int], peer: int) -> Optional[torch.Tensor]:
        """Sends ``send_t`` to ``peer`` and / or receives ``recv_rows`` rows from it as ONE batched operation, so that two
        neighbours that both have something for each other cannot block in opposite sends."""
        ops, got = [], None
        if send_t is not None:
            ops.append(dist.P2POp(dist.isend, send_t.contiguous(), peer, self.group))
        if recv_rows is not None:
            got = torch.empty((recv_rows, self.hidden), dtype=self.dtype, device=self.device)
            ops.append(dist.P2POp(dist.irecv, got, peer, self.group))
        for w in dist.batch_isend_irecv(ops):
            w.wait()
        return got

    # ------------------------------------------------------------------ schedules
    def train_step(self, microbatches: Sequence[Any], stage_fn: Callable[[Any, Optional[torch.Tensor]], torch.Tensor]):
        """One-forward-one-backward over ``microbatches``. ``stage_fn(batch, h_in)`` returns the tensor handed to the next
        stage or, on the last stage, the scalar loss of that micro-batch (already normalised for accumulation).
        Returns the last stage's losses (detached; empty elsewhere)."""
        n = len(microbatches)
        warm = min(n, self.size - self.rank - 1)
        pending: list[tuple[Any, Optional[torch.Tensor], torch.Tensor]] = []
        losses: list[torch.Tensor] = []
        prefetched: Optional[torch.Tensor] = None  # input of the next forward, when it came with a gradient exchange

        def forward(i: int) -> torch.Tensor:
            nonlocal prefetched
            b = microbatches[i]
            h_in = None
            if not self.first:
                h_in = prefetched if prefetched is not None else self._exchange(None, self.rows_of(b), self._prev)
                prefetched = None
                h_in.requires_grad_(True)
            out = stage_fn(b, h_in)
            pending.append((b, h_in, out))
            return out

        def backward(grad: Optional[torch.Tensor], more_forwards: bool, next_rows: Optional[int]) -> None:
            nonlocal prefetched
            pb, h_in, out = pending.pop(0)
            if self.last:
                losses.append(out.detach())
                out.backward()
            else:
                out.backward(grad)
            if not self.first:
                prefetched = self._exchange(h_in.grad, next_rows if more_forwards else None, self._prev)

        fi = 0
        for _ in range(warm):  # warm-up: forwards only
            out = forward(fi)
            fi += 1
            self._exchange(out.detach(), None, self._next)
        for _ in range(n - warm):  # steady state
            out = forward(fi)
            fi += 1
            grad = None
            if not self.last:  # hand the activation on and take the gradient of the oldest micro-batch in one exchange
                grad = self._exchange(out.detach(), pending[0][2].shape[0], self._next)
            more = fi < n
            backward(grad, more, self.rows_of(microbatches[fi]) if more else None)
        while pending:  # cool-down: backwards only
            grad = None if self.last else self._exchange(None, pending[0][2].shape[0], self._next)
            backward(grad, False, None)
        return losses

    @torch.no_grad()
    def forward_only(self, microbatches: Sequence[Any], stage_fn, out_shape_of: Callable[[Any], tuple], out_dtype=torch.float32):
        """Runs every micro-batch through the pipeline; the last stage's result of each is broadcast to all stages."""
        outs = []
        src = dist.get_global_rank(self.group, self.size - 1)
        for b in microbatches:
            h_in = None if self.first else self._exchange(None, self.rows_of(b), self._prev)
            out = stage_fn(b, h_in)
            if not self.last:
                self._exchange(out, None, self._next)
            res = out if self.last else torch.empty(out_shape_of(b), dtype=out_dtype, device=self.device)
            dist.broadcast(res, src=src, group=self.group)
            outs.append(res)
        return outs
