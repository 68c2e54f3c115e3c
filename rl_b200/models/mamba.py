"""Mamba-2 (state-space duality) mixer for the hybrid Nemotron-H family, over packed sequences.

Per token, with heads ``h`` of width ``P``, state width ``N`` and ``G`` groups sharing the input / output maps ``B`` / ``C``:

    z, xBC, dt = in_proj(u)                       gate, conv input (x | B | C), step size
    x, B, C    = split(silu(causal_conv(xBC)))    depth-wise convolution over the last ``d_conv`` tokens
    dt         = softplus(dt + dt_bias)
    S_t        = exp(dt_t * A_h) * S_{t-1} + dt_t * x_t (outer) B_t        A_h = -exp(A_log_h)
    y_t        = S_t C_t + D_h * x_t
    out        = out_proj(group_rms_norm(y * silu(z)) * w)

Training and prefill evaluate the recurrence chunk-wise: inside a chunk of ``Q`` tokens the outputs are one masked
"attention" product ``(C B^T * decay) x``, the chunk's contribution to the state is a second product, and only the chunk
boundaries are visited one after the other. Decoding advances the state one token at a time. Packed rows are scattered to a
right-padded [sequences, max_len] grid for the scan (padding has ``dt = 0``: the state passes through unchanged) and gathered
back. The states a sequence ends in (the last ``d_conv - 1`` conv inputs and ``S``) can be returned and passed in again, which
is how the generation engine continues a prompt chunk by chunk and then token by token.

The two projections run on the framework's GEMM kernels; the scan's products are PyTorch statements in fp32 (a native
chunked-scan kernel is not written); the reference reaches the same math through the ``mamba_ssm`` package
(nemo_rl/models/dtensor/parallelize.py:465 parallelises the HuggingFace NemotronH blocks, whose mixer this module restates).
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn
import torch.nn.functional as TF

from rl_b200.ops import functional as F

from .config import ModelConfig


def packed_to_grid_index(cu_seqlens: torch.Tensor, total: int, max_len: int) -> torch.Tensor:
    """Row of the [sequences * max_len] grid each packed token lands on (device arithmetic only, no host read)."""
    t = torch.arange(total, device=cu_seqlens.device)
    cu = cu_seqlens.long()
    b = torch.searchsorted(cu[1:].contiguous(), t, right=True).clamp(max=cu.numel() - 2)
    return b * max_len + (t - cu[b])


def causal_conv(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor], lengths: torch.Tensor,
                init: Optional[torch.Tensor] = None) -> tuple[torch.Tensor, torch.Tensor]:
    """Depth-wise causal convolution over time. ``x`` [B, L, C] right-padded, ``w`` [C, K], ``init`` [B, C, K - 1] the
    inputs that preceded position 0 (zeros when absent). Returns the outputs [B, L, C] and, per sequence, the last K - 1
    valid inputs [B, C, K - 1]."""
    Bn, L, C = x.shape
    K = w.shape[1]
    pre = init.transpose(1, 2).to(x.dtype) if init is not None else x.new_zeros(Bn, K - 1, C)
    xp = torch.cat([pre, x], dim=1)                                    # [B, K - 1 + L, C]
    y = TF.conv1d(xp.transpose(1, 2), w.unsqueeze(1).to(x.dtype), b.to(x.dtype) if b is not None else None, groups=C).transpose(1, 2)
    idx = lengths.long()[:, None] + torch.arange(K - 1, device=x.device)[None, :]      # inputs len - (K - 1) .. len - 1 in xp
    last = torch.gather(xp, 1, idx[:, :, None].expand(Bn, K - 1, C)).transpose(1, 2)
    return y, last


def ssd_scan(x: torch.Tensor, dt: torch.Tensor, A: torch.Tensor, Bm: torch.Tensor, Cm: torch.Tensor, chunk: int,
             init: Optional[torch.Tensor] = None) -> tuple[torch.Tensor, torch.Tensor]:
    """Chunk-wise evaluation of the selective state-space recurrence (fp32).

    ``x`` [B, L, H, P]; ``dt`` [B, L, H] (already positive; 0 on padding); ``A`` [H] (negative); ``Bm`` / ``Cm`` [B, L, G, N];
    ``init`` [B, H, P, N]. Returns ``y`` [B, L, H, P] (without the ``D`` skip) and the final state [B, H, P, N]."""
    Bn, L, H, P = x.shape
    G, N = Bm.shape[2], Bm.shape[3]
    R = H // G
    Q = min(chunk, max(L, 1))
    pad = (-L) % Q
    if pad:
        x, dt, Bm, Cm = (TF.pad(t, (0, 0) * (t.dim() - 2) + (0, pad)) for t in (x, dt, Bm, Cm))
    nC = (L + pad) // Q
    xd = (x * dt[..., None]).view(Bn, nC, Q, G, R, P)
    a = (dt * A).view(Bn, nC, Q, G, R).permute(0, 3, 4, 1, 2)           # [B, G, R, nC, Q]: log-decay per token
    cum = a.cumsum(-1)
    Bc, Cc = Bm.view(Bn, nC, Q, G, N), Cm.view(Bn, nC, Q, G, N)
    # inside a chunk: token i reads token j <= i through exp(sum of log-decays over (j, i])
    seg = cum[..., :, None] - cum[..., None, :]
    tri = torch.ones(Q, Q, dtype=torch.bool, device=x.device).tril()
    decay = torch.where(tri, seg, seg.new_full((), float("-inf"))).exp()   # [B, G, R, nC, Q, Q]
    cb = torch.einsum("bcign,bcjgn->bgcij", Cc, Bc)                      # shared by the R heads of a group
    y = torch.einsum("bgrcij,bcjgrp->bcigrp", cb[:, :, None] * decay, xd)
    # what each chunk adds to the state by its end, and the chunk's total decay
    to_end = (cum[..., -1:] - cum).exp()                                  # [B, G, R, nC, Q]
    add = torch.einsum("bcjgn,bgrcj,bcjgrp->bcgrpn", Bc, to_end, xd)
    total = cum[..., -1].exp()                                            # [B, G, R, nC]
    S = init.view(Bn, G, R, P, N).float() if init is not None else x.new_zeros(Bn, G, R, P, N)
    starts = []
    for c in range(nC):          # the only sequential part: one step per chunk
        starts.append(S)
        S = S * total[..., c, None, None] + add[:, c]
    S0 = torch.stack(starts, dim=1)                                       # state at the start of every chunk
    y = y + torch.einsum("bcign,bcgrpn,bgrci->bcigrp", Cc, S0, cum.exp())
    y = y.reshape(Bn, nC * Q, H, P)
    return (y[:, :L] if pad else y), S.reshape(Bn, H, P, N)


def ssd_step(x: torch.Tensor, dt: torch.Tensor, A: torch.Tensor, Bm: torch.Tensor, Cm: torch.Tensor,
             S: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """One token per sequence: ``x`` [B, H, P], ``dt`` [B, H], ``Bm`` / ``Cm`` [B, G, N], ``S`` [B, H, P, N] (fp32)."""
    Bn, H, P = x.shape
    G = Bm.shape[1]
    Bh = Bm.repeat_interleave(H // G, dim=1)
    Ch = Cm.repeat_interleave(H // G, dim=1)
    S = S * (dt * A).exp()[..., None, None] + (x * dt[..., None])[..., None] * Bh[:, :, None, :]
    return torch.einsum("bhpn,bhn->bhp", S, Ch), S


def gated_group_norm(y: torch.Tensor, z: torch.Tensor, w: torch.Tensor, groups: int, eps: float) -> torch.Tensor:
    """``rms_norm`` within each of ``groups`` slices of the last dimension of ``y * silu(z)``, then the weight."""
    h = y.float() * TF.silu(z.float())
    g = h.view(*h.shape[:-1], groups, -1)
    g = g * torch.rsqrt(g.pow(2).mean(-1, keepdim=True) + eps)
    return (w.float() * g.view_as(h)).to(z.dtype)


def _proj(x: torch.Tensor, w: torch.Tensor, b: Optional[torch.Tensor]) -> torch.Tensor:
    """The two large projections run on the framework's GEMM (16-byte aligned rows); anything else on the library's."""
    if b is None and w.shape[0] % 8 == 0 and w.shape[1] % 8 == 0 and x.dim() == 2:
        return F.linear(x.contiguous(), w)
    return TF.linear(x, w, b)


class Mamba2Mixer(nn.Module):
    """Parameters in the HuggingFace layout: ``in_proj`` rows are [gate | x | B | C | dt]."""

    def __init__(self, cfg: ModelConfig, dtype, device):
        super().__init__()
        self.cfg = cfg
        d, I, C, H = cfg.hidden_size, cfg.mamba_inner, cfg.mamba_conv_dim, cfg.mamba_num_heads
        self.in_proj = nn.Parameter(torch.empty(I + C + H, d, dtype=dtype, device=device))
        self.conv_weight = nn.Parameter(torch.empty(C, 1, cfg.mamba_d_conv, dtype=dtype, device=device))   # the checkpoint's conv1d shape
        self.conv_bias = nn.Parameter(torch.zeros(C, dtype=dtype, device=device)) if cfg.mamba_conv_bias else None
        self.dt_bias = nn.Parameter(torch.ones(H, dtype=dtype, device=device))
        self.A_log = nn.Parameter(torch.zeros(H, dtype=dtype, device=device))
        self.D = nn.Parameter(torch.ones(H, dtype=dtype, device=device))
        self.norm = nn.Parameter(torch.ones(I, dtype=dtype, device=device))
        self.out_proj = nn.Parameter(torch.empty(d, I, dtype=dtype, device=device))
        if cfg.mamba_proj_bias:
            self.in_proj_bias = nn.Parameter(torch.zeros(I + C + H, dtype=dtype, device=device))
            self.out_proj_bias = nn.Parameter(torch.zeros(d, dtype=dtype, device=device))
        else:
            self.in_proj_bias = self.out_proj_bias = None

    # ------------------------------------------------------------------ pieces shared by the sequence and the step form
    def _project(self, u: torch.Tensor):
        c = self.cfg
        p = _proj(u, self.in_proj, self.in_proj_bias)
        return torch.split(p, [c.mamba_inner, c.mamba_conv_dim, c.mamba_num_heads], dim=-1)

    def _dt(self, dt: torch.Tensor) -> torch.Tensor:
        dt = TF.softplus(dt.float() + self.dt_bias.float())
        lim = self.cfg.mamba_dt_limit
        if lim is not None and (lim[0] > 0.0 or lim[1] != float("inf")):
            dt = dt.clamp(lim[0], lim[1])
        return dt

    def _finish(self, y: torch.Tensor, x: torch.Tensor, z: torch.Tensor) -> torch.Tensor:
        c = self.cfg
        y = y + self.D.float()[:, None] * x
        y = gated_group_norm(y.reshape(*y.shape[:-2], c.mamba_inner), z, self.norm, c.mamba_n_groups, c.rms_norm_eps)
        return _proj(y, self.out_proj, self.out_proj_bias)

    # ------------------------------------------------------------------ whole sequences (training, prefill)
    def forward(self, u: torch.Tensor, cu_seqlens: torch.Tensor, max_seqlen: int, state: Optional[tuple] = None,
                return_state: bool = False):
        """``u`` [T, hidden] packed; ``state`` = (conv [B, C, K - 1], ssm [B, H, P, N]) the sequences start from."""
        c = self.cfg
        T = u.shape[0]
        nseq = cu_seqlens.numel() - 1
        H, P, G, N, I = c.mamba_num_heads, c.mamba_head_dim, c.mamba_n_groups, c.ssm_state_size, c.mamba_inner
        z, xbc, dt = self._project(u)
        lengths = (cu_seqlens[1:] - cu_seqlens[:-1]).long()
        rows = packed_to_grid_index(cu_seqlens, T, max_seqlen)

        def grid(t):
            g = t.new_zeros((nseq * max_seqlen,) + tuple(t.shape[1:]))
            return g.index_copy(0, rows, t).view(nseq, max_seqlen, *t.shape[1:])

        conv, last = causal_conv(grid(xbc), self.conv_weight[:, 0], self.conv_bias, lengths, state[0] if state is not None else None)
        valid = torch.arange(max_seqlen, device=u.device)[None, :] < lengths[:, None]
        xbc_g = TF.silu(conv).float()
        dt_g = grid(self._dt(dt)) * valid[..., None]
        x, Bm, Cm = torch.split(xbc_g, [I, G * N, G * N], dim=-1)
        x = x.view(nseq, max_seqlen, H, P)
        y, S = ssd_scan(x, dt_g, -self.A_log.float().exp(), Bm.view(nseq, max_seqlen, G, N), Cm.view(nseq, max_seqlen, G, N),
                        c.mamba_chunk_size, state[1] if state is not None else None)
        y = y.reshape(nseq * max_seqlen, H, P)[rows]
        out = self._finish(y, x.reshape(nseq * max_seqlen, H, P)[rows], z)
        return (out, (last, S)) if return_state else out

    # ------------------------------------------------------------------ one token per sequence (decode)
    def step(self, u: torch.Tensor, conv_state: torch.Tensor, ssm_state: torch.Tensor):
        """``u`` [B, hidden]; returns the output [B, hidden] and the advanced (conv [B, C, K - 1], ssm [B, H, P, N])."""
        c = self.cfg
        H, P, G, N, I = c.mamba_num_heads, c.mamba_head_dim, c.mamba_n_groups, c.ssm_state_size, c.mamba_inner
        z, xbc, dt = self._project(u)
        win = torch.cat([conv_state.to(xbc.dtype), xbc[:, :, None]], dim=-1)          # [B, C, K]
        conv = (win * self.conv_weight[:, 0][None]).sum(-1)
        if self.conv_bias is not None:
            conv = conv + self.conv_bias
        x, Bm, Cm = torch.split(TF.silu(conv).float(), [I, G * N, G * N], dim=-1)
        x = x.view(-1, H, P)
        y, S = ssd_step(x, self._dt(dt), -self.A_log.float().exp(), Bm.view(-1, G, N), Cm.view(-1, G, N), ssm_state.float())
        return self._finish(y, x, z), win[:, :, 1:], S

    @torch.no_grad()
    def reset_special(self, gen: torch.Generator, dt_min: float = 1e-3, dt_max: float = 0.1, dt_floor: float = 1e-4) -> None:
        """The initial values that are not plain normal draws: decay rates 1..H, unit skip, step sizes log-uniform in
        [dt_min, dt_max] (stored through the inverse of softplus)."""
        H = self.cfg.mamba_num_heads
        self.A_log.copy_(torch.arange(1, H + 1, dtype=torch.float32).log())
        self.D.fill_(1.0)
        self.norm.fill_(1.0)
        import math

        u = torch.rand(H, generator=gen, device=self.dt_bias.device, dtype=torch.float32)
        dt = (u * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min)).exp().clamp(min=dt_floor)
        self.dt_bias.copy_(dt + torch.log(-torch.expm1(-dt)))
        if self.conv_bias is not None:
            self.conv_bias.zero_()
