"""RotaryEncoding(head_dim, theta, scaling): rotation tables for rotary position encoding.

Reference: ``apply_rope`` (fastgguf.c:3123-3145): for pair j of a head,
``angle = pos / theta^(2j / n_rot)``, divided by ``freq_factors[j]`` when the model file
carries such a vector (:3131), computed in double and rounded to float (:3130-3133); the pair
is rotated by ``(a, b) <- (a cos - b sin, a sin + b cos)`` (:3140-3141).  The pair members are
``(j, j + n_rot/2)`` (the ``neox`` branch of :3138-3139), which is the row order of model
folders; GGUF llama files permute the rows so that adjacent pairs mean the same.

The llama3 scaling divisors are what GGUF files store as ``rope_freqs.weight``
(fastgguf.c:4278); the reference has no code that computes them.  With base frequency
``f_j = theta^(-2j/hd)`` and wavelength ``l_j = 2 pi / f_j``::

    l_j < orig / high_freq_factor   -> divisor 1                   (high frequencies: untouched)
    l_j > orig / low_freq_factor    -> divisor factor              (low frequencies: slowed)
    else  s = (orig / l_j - low) / (high - low);  divisor = 1 / ((1 - s) / factor + s)

Tables are built on the host in double and stored as float32 ``[positions, hd/2]``; the
rotation kernel only multiplies.
"""
from __future__ import annotations

import math
from typing import Optional

import torch

from .base import PositionEncoding, Runtime, register_position_encoding


def rotary_divisors(head_dim: int, theta: float, scaling: Optional[dict]) -> torch.Tensor:
    """Per-pair frequency divisors (float64, [hd/2]); all ones without scaling."""
    half = head_dim // 2
    j = torch.arange(half, dtype=torch.float64)
    div = torch.ones(half, dtype=torch.float64)
    if not scaling or scaling.get("rope_type", "default") == "default":
        return div
    if scaling["rope_type"] != "llama3":
        raise ValueError(f"rotary scaling '{scaling['rope_type']}' is not known (known: default, llama3)")
    factor = float(scaling["factor"])
    low, high = float(scaling["low_freq_factor"]), float(scaling["high_freq_factor"])
    orig = float(scaling["original_max_position_embeddings"])
    freq = torch.pow(torch.tensor(float(theta), dtype=torch.float64), -2.0 * j / head_dim)
    wavelen = 2.0 * math.pi / freq
    smooth = (orig / wavelen - low) / (high - low)
    mid = 1.0 / ((1.0 - smooth) / factor + smooth)
    div = torch.where(wavelen < orig / high, div, torch.where(wavelen > orig / low, torch.full_like(div, factor), mid))
    return div


class RotaryEncoding(PositionEncoding):
    def __init__(self, runtime: Runtime, head_dim: int, theta: float, scaling: Optional[dict] = None):
        super().__init__(runtime)
        if head_dim % 2:
            raise ValueError(f"rotary encoding needs an even head_dim, got {head_dim}")
        self.head_dim, self.theta, self.scaling = int(head_dim), float(theta), scaling
        self.cos: Optional[torch.Tensor] = None
        self.sin: Optional[torch.Tensor] = None
        self.max_positions = 0

    def prepare(self, max_positions: int) -> None:
        if self.cos is not None and self.max_positions >= max_positions:
            return
        half = self.head_dim // 2
        j = torch.arange(half, dtype=torch.float64)
        inv = torch.pow(torch.tensor(self.theta, dtype=torch.float64), -2.0 * j / self.head_dim)
        inv = inv / rotary_divisors(self.head_dim, self.theta, self.scaling)
        pos = torch.arange(max_positions, dtype=torch.float64)
        ang = pos[:, None] * inv[None, :]
        self.cos = torch.cos(ang).to(torch.float32).to(self.runtime.device).contiguous()
        self.sin = torch.sin(ang).to(torch.float32).to(self.runtime.device).contiguous()
        self.max_positions = max_positions


register_position_encoding("rope", RotaryEncoding)
