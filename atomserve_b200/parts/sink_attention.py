"""Gated grouped-query attention with a sink, as a mixer.

Queries and keys are RMS-normed over their whole projection (all heads at once, one gain entry
per column) and carry no position; the values are the keys as projected, before that norm, so
the layer has no value projection; a query sees its last `window` positions, itself included;
each head's softmax has one more term in its denominator, exp(sink_h), a learned logit with no
key and no value; the heads side by side are multiplied by sigmoid(Wg h) and projected back.
The pages hold the normed keys as "k" and the unnormed ones as "v". Heads, sizes, the score scale,
the window and eps are parameters.
"""

from __future__ import annotations

import torch

from atomserve_b200 import ops
from atomserve_b200.parts.base import CacheView, KVCacheSpec, Mixer, PageSpec, StepContext, register_part
from atomserve_b200.parts.spec import TensorSpec


class SinkAttention(Mixer):
    def __init__(self, hidden_size: int, prefix: str, num_heads: int, num_kv_heads: int, head_dim: int, scale: float,
                 eps: float, window: int | None = None):  # fmt: skip
        if num_heads % num_kv_heads:
            raise ValueError(f"{num_heads} heads are not a multiple of {num_kv_heads} kv heads")
        self.hidden_size, self.prefix = hidden_size, prefix
        self.num_heads, self.num_kv_heads, self.head_dim = num_heads, num_kv_heads, head_dim
        self.scale, self.eps, self.window = float(scale), float(eps), window
        self.in_proj = self.o_proj = self.q_gain = self.k_gain = self.sink = None

    def cache_spec(self) -> PageSpec:
        return KVCacheSpec(self.num_kv_heads, self.head_dim, self.window)

    def tensor_specs(self) -> list[TensorSpec]:
        p, d, qw, kw = self.prefix, self.hidden_size, self.num_heads * self.head_dim, self.num_kv_heads * self.head_dim
        return [
            TensorSpec(p + "q", (qw, d)), TensorSpec(p + "k", (kw, d)), TensorSpec(p + "g", (qw, d)),
            TensorSpec(p + "o", (d, qw)),
            TensorSpec(p + "q.norm", (qw,), kind="gain", init="gain"),
            TensorSpec(p + "k.norm", (kw,), kind="gain", init="gain"),
            TensorSpec(p + "sink", (self.num_heads,), kind="gain", init="normal"),
        ]  # fmt: skip

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        p = self.prefix
        self.in_proj = torch.cat([tensors[p + n] for n in "qkg"]).contiguous()
        self.o_proj = tensors[p + "o"]
        self.q_gain, self.k_gain, self.sink = tensors[p + "q.norm"], tensors[p + "k.norm"], tensors[p + "sink"].contiguous()

    def input_weights(self) -> torch.Tensor:
        """The stacked input projection, for a mixer that runs this one beside another and
        multiplies once for both (`forward_from` then reads this one's columns of the product)."""
        return self.in_proj

    def mixed_from(self, proj: torch.Tensor, col: int, ctx: StepContext, cache: CacheView, write_cache: bool) -> torch.Tensor:
        """The gated heads side by side, [T, H * hd], from a product that holds this mixer's
        projection (queries, keys, gates) in the columns from `col`."""
        H, KV, hd = self.num_heads, self.num_kv_heads, self.head_dim
        qw, kw = H * hd, KV * hd
        q = ops.projection_norm_store(proj, col, col + qw, H, KV, hd, self.q_gain, self.k_gain, self.eps,
                                      cache.slots if write_cache else None, cache.k if write_cache else None,
                                      cache.v if write_cache else None)  # fmt: skip
        out = ops.paged_attention(q, cache.k, cache.v, cache.block_tables, ctx.req_q_start, ctx.req_pos_start,
                                  num_requests=ctx.num_requests, max_context=ctx.max_context, window=self.window,
                                  scale=self.scale, host_q_lens=ctx.host_q_lens or None, sink=self.sink)  # fmt: skip
        return ops.head_norm_gate(out.view(-1, qw), proj[:, col + qw + kw : col + 2 * qw + kw], 1)

    def forward_from(self, proj: torch.Tensor, col: int, ctx: StepContext, cache: CacheView, write_cache: bool = True) -> torch.Tensor:
        return ops.linear(self.mixed_from(proj, col, ctx, cache, write_cache), self.o_proj, out_dtype=torch.float32)

    def forward(self, h: torch.Tensor, residual: torch.Tensor | None, ctx: StepContext,
                cache: CacheView | None, write_cache: bool = True) -> torch.Tensor:  # fmt: skip
        mixed = self.mixed_from(ops.linear(h, self.in_proj), 0, ctx, cache, write_cache)
        return ops.linear(mixed, self.o_proj, residual, out_dtype=torch.float32 if residual is None else None)


register_part("mixer", "sink_attention", SinkAttention)
