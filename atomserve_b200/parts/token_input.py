"""A per-layer token input: a second embedding table holds, for every token, `dim` values for
each layer that has such an input (this layer's in the columns from `offset`); a gate projected
from the stream, gelu_tanh(Wgate x), multiplies that slice; the product is projected to the model
width, RMS-normed with a gain, and added to the stream times `mult`:

    e = table[token, offset : offset + dim];  y = Wproj (gelu_tanh(Wgate x) * e)
    x <- x + mult * gain * y / sqrt(mean(y^2) + eps)

The table is one tensor shared by all layers (each names it; it is loaded once)."""

from __future__ import annotations

import torch

from atomserve_b200 import ops
from atomserve_b200.parts.base import StepContext, TokenInput, register_part
from atomserve_b200.parts.spec import TensorSpec


class GatedTokenSlice(TokenInput):
    def __init__(self, hidden_size: int, prefix: str, vocab_size: int, table: str, table_width: int, offset: int,
                 dim: int, eps: float, mult: float = 1.0):  # fmt: skip
        if offset < 0 or offset + dim > table_width:
            raise ValueError(f"columns {offset}..{offset + dim} lie outside a table of width {table_width}")
        self.hidden_size, self.prefix, self.vocab_size = hidden_size, prefix, vocab_size
        self.table_name, self.table_width, self.offset, self.dim = table, table_width, offset, dim
        self.eps, self.mult = float(eps), float(mult)
        self.table = self.gate = self.proj = self.gain = None
        self.dtype = torch.float32

    def tensor_specs(self) -> list[TensorSpec]:
        p = self.prefix
        return [
            TensorSpec(self.table_name, (self.vocab_size, self.table_width)),
            TensorSpec(p + "gate", (self.dim, self.hidden_size)), TensorSpec(p + "proj", (self.hidden_size, self.dim)),
            TensorSpec(p + "norm", (self.hidden_size,), kind="gain", init="gain"),
        ]  # fmt: skip

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        p = self.prefix
        self.table, self.gate, self.proj, self.gain = tensors[self.table_name], tensors[p + "gate"], tensors[p + "proj"], tensors[p + "norm"]

    def bind_dtype(self, dtype: torch.dtype) -> None:
        self.dtype = dtype

    def forward(self, x: torch.Tensor, h: torch.Tensor, ctx: StepContext) -> tuple[torch.Tensor, torch.Tensor]:
        z = ops.linear(h, self.gate, out_dtype=torch.float32)
        gated = ops.gated_token_slice(z, self.table, ctx.token_ids, self.offset)
        y = ops.linear_for_stream(gated, self.proj)  # float32, or partial sums for the norm to add up
        return ops.residual_out_norm(x, y, self.gain, self.eps, self.dtype, mult=self.mult, centred=False)


register_part("token_input", "gated_token_slice", GatedTokenSlice)
