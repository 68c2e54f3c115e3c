"""Pipeline parallelism: contiguous layer ranges per stage, activations and their gradients exchanged with
``torch.distributed`` point-to-point calls (NCCL send/recv over NVLink on GPUs, gloo on CPU), micro-batches scheduled
one-forward-one-backward (1F1B) so that a stage holds at most ``pp - stage`` micro-batches of activations.

With ``vpp`` > 1 a rank owns ``vpp`` runs of layers instead of one (virtual stage ``c * pp + rank`` is its chunk ``c``) and
the interleaved schedule of :func:`interleaved_schedule` shortens the pipeline bubble by the same factor.

``PipelineRunner.train_step(microbatches, loss_fn)`` runs one accumulation window; ``forward_only`` runs inference and
returns the last stage's outputs on every stage (broadcast inside the pipeline group). The reference reaches pipeline
parallelism through Megatron's schedules (``forward_backward_func`` in nemo_rl/models/megatron/train.py) and the
``pipeline_model_parallel_size`` / ``virtual_pipeline_model_parallel_size`` keys of ``policy.megatron_cfg``.
"""

from __future__ import annotations

from typing import Any, Callable, Optional, Sequence

import torch
import torch.distributed as dist


def interleaved_schedule(P: int, V: int, n: int, train: bool = True, caps: Optional[Sequence[int]] = None):
    """The whole pipeline's plan for ``n`` micro-batches over ``P`` ranks with ``V`` chunks each, as a list of ticks. A tick
    is ``(ops, msgs)``: ``ops[r]`` is rank r's work in that tick -- ``None`` or ``(kind, m, c)`` with kind "F" / "B",
    micro-batch m, chunk c -- and ``msgs`` the tensors that travel when the tick's work is done: ``(src, dst, kind, m, c)``
    where (kind, m, c) names the operation at ``dst`` that consumes the tensor ("F": an activation, "B": a gradient).

    Every rank computes the same plan, so both ends of every message know about it without talking. Order of the forward
    work on a rank: micro-batches in groups of P, each group through chunk 0, then chunk 1, ... (a group's output of chunk c
    on the last rank is the input of chunk c + 1 on the first just when the first rank gets there); the backward work runs in
    the mirrored order. A rank alternates forward and backward work when both are possible, works backward when only that is, and forward
    while fewer than ``caps[r]`` of its forward results wait for their backward pass (default: the interleaved 1F1B depth
    ``2 (P - r - 1) + (V - 1) P + 1``); a cap too tight to finish is raised until the plan completes."""
    S = P * V
    f_order = [(m, c) for g in range(0, n, P) for c in range(V) for m in range(g, min(n, g + P))]
    b_order = [(m, c) for g in range(0, n, P) for c in reversed(range(V)) for m in range(g, min(n, g + P))]
    caps = list(caps) if caps is not None else [2 * (P - r - 1) + (V - 1) * P + 1 for r in range(P)]
    while True:
        have = set()            # (rank, kind, m, c): the input of that operation has arrived
        fi, bi, held, last = [0] * P, [0] * P, [0] * P, ["F"] * P
        fdone, ticks, stuck = set(), [], False
        total = (2 if train else 1) * len(f_order) * P
        done = 0
        while done < total:
            ops, msgs = [None] * P, []
            for r in range(P):
                nb = b_order[bi[r]] if (train and bi[r] < len(b_order)) else None
                nf = f_order[fi[r]] if fi[r] < len(f_order) else None
                b_ok = nb is not None and (r, nb[0], nb[1]) in fdone and (nb[1] * P + r == S - 1 or (r, "B", *nb) in have)
                f_ok = nf is not None and (not train or held[r] < caps[r]) and (nf[1] * P + r == 0 or (r, "F", *nf) in have)
                if b_ok and f_ok:       # both possible: alternate (one forward, one backward)
                    ops[r] = ("F", *nf) if last[r] == "B" else ("B", *nb)
                elif b_ok:
                    ops[r] = ("B", *nb)
                elif f_ok:
                    ops[r] = ("F", *nf)
            if all(o is None for o in ops):
                stuck = True
                break
            for r, o in enumerate(ops):
                if o is None:
                    continue
                kind, m, c = o
                s = c * P + r
                done += 1
                last[r] = kind
                if kind == "F":
                    fi[r] += 1
                    held[r] += 1
                    fdone.add((r, m, c))
                    if s < S - 1:
                        msgs.append((r, (s + 1) % P, "F", m, (s + 1) // P))
                else:
                    bi[r] += 1
                    held[r] -= 1
                    if s > 0:
                        msgs.append((r, (s - 1) % P, "B", m, (s - 1) // P))
            for (_, dst, kind, m, c) in msgs:
                have.add((dst, kind, m, c))
            ticks.append((ops, msgs))
        if not stuck:
            return ticks
        caps = [x + 1 for x in caps]


class PipelineRunner:
    def __init__(self, model, pp_group, pp_rank: int, pp_size: int, hidden_size: int, dtype: torch.dtype, device,
                 rows_of: Optional[Callable[[Any], int]] = None, vpp: int = 1):
        """``rows_of(batch)``: rows of the activation tensor a stage hands on for ``batch`` (token count, divided by the
        tensor-parallel size under sequence parallelism)."""
        self.model, self.group, self.rank, self.size = model, pp_group, pp_rank, pp_size
        self.hidden, self.dtype, self.device = hidden_size, dtype, torch.device(device)
        self.rows_of = rows_of or (lambda b: int(b.input_ids.numel()))
        self.first, self.last = pp_rank == 0, pp_rank == pp_size - 1
        self.vpp = max(1, int(vpp))
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

    # ------------------------------------------------------------------ interleaved schedule
    def _run_plan(self, microbatches: Sequence[Any], stage_fn, train: bool):
        """Executes this rank's part of :func:`interleaved_schedule`: per tick at most one chunk forward or backward, then
        ONE batched exchange of everything that tick produced for or expects from this rank (a rank with nothing to send or
        receive skips the exchange; its peers' batches do not name it). Returns {micro-batch: output of the final virtual
        stage} on the last rank ({} elsewhere)."""
        P, V, r = self.size, self.vpp, self.rank
        glob = [dist.get_global_rank(self.group, i) for i in range(P)]
        inbox: dict = {}          # (kind, m, c) -> tensor that arrived for that operation
        kept: dict = {}           # (m, c) -> (h_in, out) of a forward pass that waits for its backward pass
        final: dict = {}
        try:
            for ops, msgs in interleaved_schedule(P, V, len(microbatches), train):
                send: dict = {}
                if ops[r] is not None:
                    kind, m, c = ops[r]
                    s = c * P + r
                    self.model.active_chunk = c
                    if kind == "F":
                        h_in = inbox.pop(("F", m, c), None)
                        if h_in is not None and train:
                            h_in.requires_grad_(True)
                        out = stage_fn(microbatches[m], h_in)
                        if train:
                            kept[(m, c)] = (h_in, out)
                        if s == P * V - 1:
                            final[m] = out.detach()
                        else:
                            send[("F", m, (s + 1) // P)] = out.detach()
                    else:
                        h_in, out = kept.pop((m, c))
                        if s == P * V - 1:
                            out.backward()
                        else:
                            out.backward(inbox.pop(("B", m, c)))
                        if s > 0:
                            send[("B", m, (s - 1) // P)] = h_in.grad
                p2p, local = [], []
                for (src, dst, kind, m, c) in msgs:     # the same order on both ends of every pair
                    if src == r and dst == r:              # (P == 1 never gets here; kept for completeness)
                        local.append((kind, m, c))
                    elif src == r:
                        p2p.append(dist.P2POp(dist.isend, send[(kind, m, c)].contiguous(), glob[dst], self.group))
                    elif dst == r:
                        buf = torch.empty((self.rows_of(microbatches[m]), self.hidden), dtype=self.dtype, device=self.device)
                        inbox[(kind, m, c)] = buf
                        p2p.append(dist.P2POp(dist.irecv, buf, glob[src], self.group))
                for k in local:
                    inbox[k] = send[k]
                if p2p:
                    for w in dist.batch_isend_irecv(p2p):
                        w.wait()
        finally:
            self.model.active_chunk = None
        return final

    # ------------------------------------------------------------------ schedules
    def train_step(self, microbatches: Sequence[Any], stage_fn: Callable[[Any, Optional[torch.Tensor]], torch.Tensor]):
        """One-forward-one-backward over ``microbatches``. ``stage_fn(batch, h_in)`` returns the tensor handed to the next
        stage or, on the last stage, the scalar loss of that micro-batch (already normalised for accumulation).
        Returns the last stage's losses (detached; empty elsewhere)."""
        n = len(microbatches)
        if self.vpp > 1:
            final = self._run_plan(microbatches, stage_fn, train=True)
            return [final[m] for m in range(n)] if self.last else []
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
        if self.vpp > 1:
            final = self._run_plan(microbatches, stage_fn, train=False)
            for m, b in enumerate(microbatches):
                res = final[m] if self.last else torch.empty(out_shape_of(b), dtype=out_dtype, device=self.device)
                dist.broadcast(res, src=src, group=self.group)
                outs.append(res)
            return outs
        for b in microbatches:
            h_in = None if self.first else self._exchange(None, self.rows_of(b), self._prev)
            out = stage_fn(b, h_in)
            if not self.last:
                self._exchange(out, None, self._next)
            res = out if self.last else torch.empty(out_shape_of(b), dtype=out_dtype, device=self.device)
            dist.broadcast(res, src=src, group=self.group)
            outs.append(res)
        return outs
