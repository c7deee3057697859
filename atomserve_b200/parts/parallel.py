"""Two mixers side by side as one: both read the same input, and the result is half the sum of
their outputs, each RMS-normed over the model width with a gain of its own,
(R(left(h)) gain_left + R(right(h)) gain_right) / 2. The two are given as part descriptions; what
either keeps between steps (pages, state) is this mixer's: at most one of them may keep pages.
Their input projections are stacked, so the input is multiplied once for both."""

from __future__ import annotations

import torch

from atomserve_b200 import ops
from atomserve_b200.parts.base import CacheView, Mixer, PageSpec, StateSpec, StepContext, build_part, register_part
from atomserve_b200.parts.spec import PartSpec, TensorSpec


class ParallelMixers(Mixer):
    def __init__(self, hidden_size: int, prefix: str, left: PartSpec, right: PartSpec, eps: float,
                 left_gain: str | None = None, right_gain: str | None = None):  # fmt: skip
        self.hidden_size, self.eps = hidden_size, float(eps)
        self.left, self.right = build_part("mixer", left, hidden_size), build_part("mixer", right, hidden_size)
        self.names = (left_gain or prefix + "left.out", right_gain or prefix + "right.out")
        for side in (self.left, self.right):
            if not hasattr(side, "input_weights") or not hasattr(side, "forward_from"):
                raise ValueError(f"{type(side).__name__} cannot run beside another mixer (no input_weights / forward_from)")
        if self.left.cache_spec() is not None and self.right.cache_spec() is not None:
            raise ValueError("only one of two mixers side by side may keep pages")
        names = [s.name for side in (self.left, self.right) for s in side.state_specs()]
        if len(set(names)) != len(names):
            raise ValueError(f"the two mixers' state names collide: {names}")
        self.in_proj = self.gains = None
        self.split = 0

    @property
    def state_in_graphs(self) -> bool:
        return all(getattr(side, "state_in_graphs", not side.state_specs()) for side in (self.left, self.right))

    def cache_spec(self) -> PageSpec | None:
        return self.left.cache_spec() or self.right.cache_spec()

    def state_specs(self) -> list[StateSpec]:
        return self.left.state_specs() + self.right.state_specs()

    def tensor_specs(self) -> list[TensorSpec]:
        own = [TensorSpec(n, (self.hidden_size,), kind="gain", init="gain") for n in self.names]
        return self.left.tensor_specs() + self.right.tensor_specs() + own

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        self.left.load(tensors)
        self.right.load(tensors)
        a, b = self.left.input_weights(), self.right.input_weights()
        self.split = a.shape[0]
        self.in_proj = torch.cat([a, b]).contiguous()
        self.gains = tuple(tensors[n] for n in self.names)

    def forward_halves(self, h: torch.Tensor, ctx: StepContext, cache: CacheView | None, write_cache: bool = True):
        """(left(h), (right(h), gain_left, gain_right)), float32: for a block whose norm kernel joins them."""
        proj = ops.linear(h, self.in_proj)
        takes_write = lambda side: side.cache_spec() is not None  # noqa: E731
        a = self.left.forward_from(proj, 0, ctx, cache, write_cache) if takes_write(self.left) else self.left.forward_from(proj, 0, ctx, cache)
        b = self.right.forward_from(proj, self.split, ctx, cache, write_cache) if takes_write(self.right) else self.right.forward_from(proj, self.split, ctx, cache)
        return a, (b, *self.gains)

    def forward(self, h: torch.Tensor, residual: torch.Tensor | None, ctx: StepContext,
                cache: CacheView | None, write_cache: bool = True) -> torch.Tensor:  # fmt: skip
        # (blocks that norm the sublayer's output take `forward_halves` and join in their norm's kernel)
        a, (b, ga, gb) = self.forward_halves(h, ctx, cache, write_cache)
        joined = _join(a, b, ga, gb, self.eps)
        if residual is None:
            return joined
        return residual + joined.to(residual.dtype)


def _join(a: torch.Tensor, b: torch.Tensor, ga: torch.Tensor, gb: torch.Tensor, eps: float) -> torch.Tensor:
    """(R(a) ga + R(b) gb) / 2 as float32 (two launches of the RMS form, then a sum on the device)."""
    na = ops.residual_out_norm(None, a, ga, eps, torch.float32, centred=False)[0]
    nb = ops.residual_out_norm(None, b, gb, eps, torch.float32, centred=False)[0]
    return (na + nb) * 0.5


register_part("mixer", "parallel_mixers", ParallelMixers)
