"""Multimodal batch plumbing: ``PackedTensor`` (per-sample tensors of different sizes that travel through batch slicing,
sharding and reordering and are concatenated only where a kernel needs them) and image -> patch helpers.

Role of nemo_rl/data/multimodal_utils.py (``PackedTensor`` and its helpers). Here a PackedTensor *is* a list (one entry
per sample, ``None`` for samples without that modality), so every ``BatchedDataDict`` operation that works on per-sample
lists works on it unchanged.
"""

from __future__ import annotations

from typing import Iterable, Optional, Sequence

import torch


class PackedTensor(list):
    """One tensor (or None) per sample; ``dim_to_pack`` is the dimension along which entries are concatenated."""

    def __init__(self, tensors: Iterable[Optional[torch.Tensor]] = (), dim_to_pack: int = 0):
        super().__init__(tensors)
        self.dim_to_pack = dim_to_pack

    def as_tensor(self, device=None) -> Optional[torch.Tensor]:
        parts = [t for t in self if t is not None and t.numel() > 0]
        if not parts:
            return None
        out = torch.cat(parts, dim=self.dim_to_pack)
        return out.to(device) if device is not None else out

    def sizes(self) -> list[int]:
        return [0 if t is None else int(t.shape[self.dim_to_pack]) for t in self]

    def to(self, device) -> "PackedTensor":
        return PackedTensor([None if t is None else t.to(device) for t in self], self.dim_to_pack)

    def select(self, idx: Sequence[int]) -> "PackedTensor":
        return PackedTensor([self[i] for i in idx], self.dim_to_pack)

    def __getitem__(self, i):
        out = super().__getitem__(i)
        return PackedTensor(out, self.dim_to_pack) if isinstance(i, slice) else out

    @classmethod
    def concat(cls, items: Sequence["PackedTensor"]) -> "PackedTensor":
        dim = items[0].dim_to_pack if items else 0
        return cls([t for it in items for t in it], dim)

    @classmethod
    def empty_like(cls, n: int, dim_to_pack: int = 0) -> "PackedTensor":
        return cls([None] * n, dim_to_pack)


def patchify(image: torch.Tensor, patch: int) -> torch.Tensor:
    """[C, H, W] (H, W multiples of ``patch``) -> [H/p * W/p, C * p * p], row-major over the patch grid."""
    C, H, W = image.shape
    assert H % patch == 0 and W % patch == 0, "image size must be a multiple of the patch size"
    x = image.reshape(C, H // patch, patch, W // patch, patch).permute(1, 3, 0, 2, 4)
    return x.reshape((H // patch) * (W // patch), C * patch * patch).contiguous()


def unpatchify(patches: torch.Tensor, channels: int, height: int, width: int, patch: int) -> torch.Tensor:
    gh, gw = height // patch, width // patch
    x = patches.reshape(gh, gw, channels, patch, patch).permute(2, 0, 3, 1, 4)
    return x.reshape(channels, height, width).contiguous()


def expand_image_tokens(token_ids: Sequence[int], image_token_id: int, patches_per_image: Sequence[int]) -> list[int]:
    """Replaces the k-th single ``image_token_id`` placeholder with ``patches_per_image[k]`` copies, which is how many
    rows the vision tower will hand to the language model for that image."""
    out, k = [], 0
    for t in token_ids:
        if t == image_token_id:
            assert k < len(patches_per_image), "more image placeholders than images"
            out.extend([image_token_id] * int(patches_per_image[k]))
            k += 1
        else:
            out.append(int(t))
    assert k == len(patches_per_image), "fewer image placeholders than images"
    return out


def get_multimodal_keys(batch: dict) -> list[str]:
    return [k for k, v in batch.items() if isinstance(v, PackedTensor)]


def content_key(t: Optional[torch.Tensor]) -> int:
    """Cheap content hash of a tensor (prefix-sharing keys must tell apart equal prompts with different images)."""
    import zlib

    if t is None:
        return 0
    return zlib.crc32(t.detach().cpu().contiguous().view(torch.uint8).numpy().tobytes()) ^ (t.numel() << 32)
