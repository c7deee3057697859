"""Rotary position encoding: pair i of rotary_dim/2 turns by position * theta^(-2i/rotary_dim),
rotate-half pairing (i, i + rotary_dim/2); angles in float32 (atomserve/model.py:142-185).
Dimensions beyond rotary_dim pass through unrotated (rotary_dim = head_dim for Qwen3).
`pairing="interleaved"` pairs neighbours (2i, 2i + 1) instead, with the same frequencies; the
mixers whose fused kernels know that pairing apply it (latent attention)."""

from __future__ import annotations

import torch

from atomserve_b200 import ops
from atomserve_b200.parts.base import FusedRotary, PositionEncoding, register_part


class Rotary(PositionEncoding):
    def __init__(self, hidden_size: int, prefix: str, head_dim: int, theta: float, rotary_dim: int | None = None,
                 pairing: str = "half"):  # fmt: skip
        if pairing not in ("half", "interleaved"):
            raise ValueError(f"pairing {pairing!r} is neither 'half' nor 'interleaved'")
        self.pairing = pairing
        self.head_dim = head_dim
        self.rotary_dim = head_dim if rotary_dim is None else rotary_dim  # (0: nothing turns)
        if self.rotary_dim % 2 or self.rotary_dim > head_dim:
            raise ValueError(f"rotary_dim {self.rotary_dim} must be even and at most head_dim {head_dim}")
        self.theta = float(theta)
        self.inv_freq: torch.Tensor | None = None

    def prepare(self, device: torch.device) -> None:
        exponents = torch.arange(0, self.rotary_dim, 2, dtype=torch.float32) / self.rotary_dim
        self.inv_freq = (1.0 / (self.theta**exponents)).to(device)

    def fused_rotary(self) -> FusedRotary:
        return FusedRotary(self.inv_freq, self.rotary_dim, self.pairing)

    def apply(self, x: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """Rotate x [T, heads, head_dim] by its tokens' positions (the encoding on its own)."""
        if self.pairing != "half":
            raise NotImplementedError("the stand-alone rotary kernel pairs (i, i + rotary_dim / 2) only")
        return ops.rotary(x, positions, self.inv_freq, self.rotary_dim)


register_part("position", "rotary", Rotary)
