"""Linear attention with a fixed decay per head ("lightning attention") as a mixer.

Per head, S_t = decay_h S_(t-1) + k_t v_t^T and o_t = S_t^T q_t, with q, k and v the activated
projections of the input; the heads' outputs side by side are RMS-normed together, multiplied by
a sigmoid gate projected from the same input, and projected back. The state S ([dim, vdim] per
head, float32) is all the mixer keeps of a request: it lives in the request's state slot, zero
at admission, and is carried from step to step. Heads, sizes, decays, eps and the activation
are parameters.
"""

from __future__ import annotations

import torch

from atomserve_b200 import ops
from atomserve_b200.parts.base import CacheView, Mixer, StateSpec, StepContext, register_part
from atomserve_b200.parts.spec import TensorSpec


class LightningAttention(Mixer):
    state_in_graphs = True  # the state is touched by this mixer's kernel alone, through ctx.state_slots

    def __init__(self, hidden_size: int, prefix: str, heads: int, dim: int, vdim: int, decay: list[float], eps: float,
                 activation: str = "silu"):  # fmt: skip
        if len(decay) != heads:
            raise ValueError(f"{len(decay)} decays for {heads} heads")
        if activation not in ("silu", "none"):
            raise ValueError(f"activation {activation!r} is neither 'silu' nor 'none'")
        self.hidden_size, self.prefix = hidden_size, prefix
        self.heads, self.dim, self.vdim, self.eps = heads, dim, vdim, float(eps)
        self.decay_values, self.activation = [float(d) for d in decay], activation
        self.in_proj = self.o_proj = self.gain = self.decay = None

    def state_specs(self) -> list[StateSpec]:
        return [StateSpec("s", (self.heads, self.dim, self.vdim), torch.float32)]

    def tensor_specs(self) -> list[TensorSpec]:
        p, d, qk, vg = self.prefix, self.hidden_size, self.heads * self.dim, self.heads * self.vdim
        return [
            TensorSpec(p + "q", (qk, d)), TensorSpec(p + "k", (qk, d)), TensorSpec(p + "v", (vg, d)),
            TensorSpec(p + "g", (vg, d)), TensorSpec(p + "o", (d, vg)),
            TensorSpec(p + "norm", (vg,), kind="gain", init="gain"),
        ]  # fmt: skip

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        p = self.prefix
        # q, k, v and the gate stacked along the output rows: one product instead of four
        self.in_proj = torch.cat([tensors[p + n] for n in "qkvg"]).contiguous()
        self.o_proj, self.gain = tensors[p + "o"], tensors[p + "norm"]
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.o_proj.device)

    def mixed(self, h: torch.Tensor, ctx: StepContext, cache: CacheView | None) -> torch.Tensor:
        """The gated, normed heads side by side, [T, heads * vdim], before the output projection."""
        qk, vg = self.heads * self.dim, self.heads * self.vdim
        proj = ops.linear(h, self.in_proj)
        # long portions are cut into segments that run side by side; the cut is made once per step
        # and shared by the step's layers
        if "lightning_segments" not in ctx.plans:
            ctx.plans["lightning_segments"] = ops.plan_segments(ctx.host_q_lens, h.device) if ctx.host_q_lens else None
        o = ops.lightning_attention(proj, 0, qk, 2 * qk, cache.state["s"], ctx.state_slots, ctx.req_q_start, self.decay,
                                    ctx.num_requests, activation=self.activation == "silu",
                                    segments=ctx.plans["lightning_segments"])  # fmt: skip
        return ops.gated_rms_norm(o, proj[:, 2 * qk + vg :], self.gain, self.eps)

    def forward(self, h: torch.Tensor, residual: torch.Tensor | None, ctx: StepContext,
                cache: CacheView | None, write_cache: bool = True) -> torch.Tensor:  # fmt: skip
        # without a residual (a block that sums in float32 itself) the product stays float32
        return ops.linear(self.mixed(h, ctx, cache), self.o_proj, residual, out_dtype=torch.float32 if residual is None else None)

    def forward_for_stream(self, h: torch.Tensor, ctx: StepContext, cache: CacheView | None, write_cache: bool = True):
        """mix(h) for a block that adds it to a float32 stream and norms the sum at once: float32, or
        the output projection's partial sums for that norm to add up (`ops.linear_for_stream`)."""
        return ops.linear_for_stream(self.mixed(h, ctx, cache), self.o_proj)


register_part("mixer", "lightning_attention", LightningAttention)
