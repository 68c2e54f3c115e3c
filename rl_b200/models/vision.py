"""Vision-language model: a ViT patch encoder and a projector in front of the decoder-only language model.

Images arrive as patch rows ([n_patches, C * p * p], see ``data/multimodal_utils.py::patchify``). The tower embeds them
(linear patch embedding + learned position table), runs pre-norm transformer blocks with bidirectional attention inside
each image, and the merger MLP maps the result to the language model's width. The language model's input embedding rows
at the ``image_token_id`` placeholders are replaced by these rows, in order; everything after that is the ordinary
:class:`CausalLM`. This is the structure of the Qwen2-VL / LLaVA family that the reference trains through HF AutoModel
(examples/run_vlm_grpo.py, nemo_rl/data/multimodal_utils.py); parameters are stored under ``visual.*`` names.
"""

from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

from rl_b200.ops import functional as F

from .config import ModelConfig
from .transformer import CausalLM, PackedBatch

VISION_DEFAULTS = dict(patch_size=14, channels=3, hidden_size=256, intermediate_size=1024, num_layers=4, num_heads=4, max_patches=1024,
                       norm_eps=1e-6)


def vision_config(cfg: ModelConfig) -> dict:
    v = dict(VISION_DEFAULTS)
    v.update(cfg.vision or {})
    return v


class VisionBlock(nn.Module):
    def __init__(self, d: int, f: int, heads: int, eps: float, dtype, device):
        super().__init__()
        self.heads, self.eps = heads, eps
        self.attn_norm = nn.Parameter(torch.ones(d, dtype=dtype, device=device))
        self.qkv = nn.Parameter(torch.empty(3 * d, d, dtype=dtype, device=device))
        self.proj = nn.Parameter(torch.empty(d, d, dtype=dtype, device=device))
        self.mlp_norm = nn.Parameter(torch.ones(d, dtype=dtype, device=device))
        self.fc1 = nn.Parameter(torch.empty(f, d, dtype=dtype, device=device))
        self.fc2 = nn.Parameter(torch.empty(d, f, dtype=dtype, device=device))

    def forward(self, x: torch.Tensor, sizes: list[int]) -> torch.Tensor:
        n, d = x.shape
        hd = d // self.heads
        qkv = F.linear(F.rmsnorm(x, self.attn_norm, self.eps), self.qkv).view(n, 3, self.heads, hd)
        outs, o = [], 0
        for s in sizes:  # bidirectional attention inside each image
            q, k, v = (qkv[o : o + s, j].transpose(0, 1) for j in range(3))
            outs.append(torch.nn.functional.scaled_dot_product_attention(q[None], k[None], v[None])[0].transpose(0, 1).reshape(s, d))
            o += s
        x = F.linear(torch.cat(outs), self.proj, None, x)
        h = torch.nn.functional.gelu(F.linear(F.rmsnorm(x, self.mlp_norm, self.eps), self.fc1))
        return F.linear(h, self.fc2, None, x)


class VisionTower(nn.Module):
    def __init__(self, v: dict, out_dim: int, dtype, device):
        super().__init__()
        self.v = v
        d, f = v["hidden_size"], v["intermediate_size"]
        self.patch_dim = v["channels"] * v["patch_size"] ** 2
        self.patch_dim_padded = -(-self.patch_dim // 8) * 8            # GEMM rows start on 16-byte boundaries
        self.patch_embed = nn.Parameter(torch.empty(d, self.patch_dim_padded, dtype=dtype, device=device))
        self.pos_embed = nn.Parameter(torch.empty(v["max_patches"], d, dtype=dtype, device=device))
        self.blocks = nn.ModuleList([VisionBlock(d, f, v["num_heads"], v["norm_eps"], dtype, device) for _ in range(v["num_layers"])])
        self.merger_norm = nn.Parameter(torch.ones(d, dtype=dtype, device=device))
        self.merger_fc1 = nn.Parameter(torch.empty(out_dim, d, dtype=dtype, device=device))
        self.merger_fc2 = nn.Parameter(torch.empty(out_dim, out_dim, dtype=dtype, device=device))

    def forward(self, patches: torch.Tensor, sizes: list[int]) -> torch.Tensor:
        """patches [N, patch_dim] (all images of the batch, concatenated) -> [N, out_dim]."""
        x = patches.to(self.patch_embed.dtype)
        if self.patch_dim_padded != self.patch_dim:
            x = torch.nn.functional.pad(x, (0, self.patch_dim_padded - self.patch_dim))
        pos = torch.cat([torch.arange(s, device=x.device) for s in sizes])
        x = F.linear(x.contiguous(), self.patch_embed) + self.pos_embed[pos]
        for blk in self.blocks:
            x = blk(x, sizes)
        x = F.rmsnorm(x, self.merger_norm, self.v["norm_eps"])
        return F.linear(torch.nn.functional.gelu(F.linear(x, self.merger_fc1)), self.merger_fc2)


class VLMCausalLM(CausalLM):
    """:class:`CausalLM` whose ``embed`` splices vision features into the token embeddings.

    A packed batch carries the images as ``batch.mm = {"patches": [N, patch_dim], "sizes": [patches per image]}``; the rows
    of the batch whose token is ``cfg.image_token_id`` receive the N feature rows in order."""

    def __init__(self, cfg: ModelConfig, dtype: Optional[torch.dtype] = None, device="cpu", init: bool = True, seed: int = 0, **kw):
        super().__init__(cfg, dtype=dtype, device=device, init=False, seed=seed, **kw)
        assert cfg.image_token_id is not None, "a vision-language config needs image_token_id"
        assert self.tp.world == 1 or not self.tp.sequence_parallel, "vision inputs with sequence parallelism are not supported"
        self.visual = VisionTower(vision_config(cfg), cfg.hidden_size, self.dtype, device) if self.first_stage else None
        if init:
            self.reset_parameters(seed)

    def vision_features(self, patches: torch.Tensor, sizes: list[int]) -> torch.Tensor:
        return self.visual(patches.to(self.embed_tokens.device), [int(s) for s in sizes])

    def merge_vision(self, h: torch.Tensor, input_ids: torch.Tensor, mm: Optional[dict]) -> torch.Tensor:
        if not mm or mm.get("patches") is None:
            return h
        feats = self.vision_features(mm["patches"], mm["sizes"]).to(h.dtype)
        where = (input_ids.long() == self.cfg.image_token_id).nonzero(as_tuple=True)[0]
        assert where.numel() == feats.shape[0], f"{where.numel()} image placeholder tokens for {feats.shape[0]} patch rows"
        return h.index_copy(0, where, feats)

    def embed(self, batch: PackedBatch) -> torch.Tensor:
        h = super().embed(batch)
        return self.merge_vision(h, batch.input_ids[: h.shape[0]], getattr(batch, "mm", None))
