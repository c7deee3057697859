"""A matrix memory with exponential gating (the mLSTM cell of xLSTM) as a mixer.

Per head, with q = Wq h * dim^(-1/2), k = Wk h, v = Wv h and two log gates per token,
i = cap tanh((Wi h + bi) / cap) and f = logsigmoid(cap tanh((Wf h + bf) / cap)):

    top_t = max(f_t + top_(t-1), i_t)                       (a running maximum that starts at 0)
    S_t = exp(f_t + top_(t-1) - top_t) S_(t-1) + exp(i_t - top_t) k_t v_t^T,   n_t likewise with k_t
    o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-top_t)) + floor)

Each head's o is divided by its root mean square, the heads side by side are multiplied by a
gain and by sigmoid(Wg h), and projected back. S [dim, vdim], n [dim] and top are the request's
state: float32, zero at admission, carried from step to step. The gates, their scan and everything
in the recurrence are float32; the gate pre-activations are the float32 sums of their product.
Heads, sizes, cap, eps and the floor are parameters.
"""

from __future__ import annotations

import torch

from atomserve_b200 import ops
from atomserve_b200.parts.base import CacheView, Mixer, StateSpec, StepContext, register_part
from atomserve_b200.parts.spec import TensorSpec


class MatrixMemory(Mixer):
    state_in_graphs = True  # the state is touched by this mixer's kernels alone, through ctx.state_slots

    def __init__(self, hidden_size: int, prefix: str, heads: int, dim: int, vdim: int, gate_cap: float, eps: float,
                 floor: float = 1e-6):  # fmt: skip
        if not gate_cap > 0:
            raise ValueError(f"gate_cap {gate_cap} must be positive")
        self.hidden_size, self.prefix = hidden_size, prefix
        self.heads, self.dim, self.vdim = heads, dim, vdim
        self.cap, self.eps, self.floor = float(gate_cap), float(eps), float(floor)
        self.in_proj = self.gate_proj = self.o_proj = self.gain = self.i_bias = self.f_bias = None

    def state_specs(self) -> list[StateSpec]:
        return [StateSpec("s", (self.heads, self.dim, self.vdim), torch.float32),
                StateSpec("n", (self.heads, self.dim), torch.float32),
                StateSpec("top", (self.heads,), torch.float32)]  # fmt: skip

    def tensor_specs(self) -> list[TensorSpec]:
        p, d, qk, vg, H = self.prefix, self.hidden_size, self.heads * self.dim, self.heads * self.vdim, self.heads
        return [
            TensorSpec(p + "q", (qk, d)), TensorSpec(p + "k", (qk, d)), TensorSpec(p + "v", (vg, d)),
            TensorSpec(p + "g", (vg, d)), TensorSpec(p + "o", (d, vg)),
            TensorSpec(p + "norm", (vg,), kind="gain", init="gain"),
            TensorSpec(p + "i", (H, d)), TensorSpec(p + "i.b", (H,), kind="gain", init="zeros"),
            TensorSpec(p + "f", (H, d)), TensorSpec(p + "f.b", (H,), kind="gain", init="gain"),
        ]  # fmt: skip

    def load(self, tensors: dict[str, torch.Tensor]) -> None:
        p = self.prefix
        self.in_proj = torch.cat([tensors[p + n] for n in "qkvg"]).contiguous()
        # the two gates' rows in a product of their own, whose float32 sums are never rounded
        self.gate_proj = torch.cat([tensors[p + "i"], tensors[p + "f"]]).contiguous()
        self.i_bias, self.f_bias = tensors[p + "i.b"], tensors[p + "f.b"]
        self.o_proj, self.gain = tensors[p + "o"], tensors[p + "norm"]

    def mixed(self, h: torch.Tensor, ctx: StepContext, cache: CacheView | None) -> torch.Tensor:
        """The normed, gated heads side by side, [T, heads * vdim], before the output projection."""
        H, qk, vg = self.heads, self.heads * self.dim, self.heads * self.vdim
        proj = ops.linear(h, self.in_proj)
        z = ops.linear(h, self.gate_proj, out_dtype=torch.float32)
        decay, gain, top = ops.capped_gates_scan(z, 0, H, H, self.i_bias, self.f_bias, self.cap, cache.state["top"],
                                                 ctx.state_slots, ctx.req_q_start, ctx.num_requests)  # fmt: skip
        if "lightning_segments" not in ctx.plans:  # the cut of long portions, shared by the step's recurrent layers
            ctx.plans["lightning_segments"] = ops.plan_segments(ctx.host_q_lens, h.device) if ctx.host_q_lens else None
        o, nq = ops.linear_recurrence(proj, 0, qk, 2 * qk, cache.state["s"], ctx.state_slots, ctx.req_q_start,
                                      ctx.num_requests, token_decay=decay, token_gain=gain, norm_state=cache.state["n"],
                                      q_scale=self.dim**-0.5, segments=ctx.plans["lightning_segments"])  # fmt: skip
        return ops.head_norm_gate(o, proj[:, 2 * qk + vg :], H, gain=self.gain, eps=self.eps, normaliser=(nq, top, self.floor))

    def forward(self, h: torch.Tensor, residual: torch.Tensor | None, ctx: StepContext,
                cache: CacheView | None, write_cache: bool = True) -> torch.Tensor:  # fmt: skip
        # without a residual (a block that sums in float32 itself) the product stays float32
        return ops.linear(self.mixed(h, ctx, cache), self.o_proj, residual, out_dtype=torch.float32 if residual is None else None)

    def forward_for_stream(self, h: torch.Tensor, ctx: StepContext, cache: CacheView | None, write_cache: bool = True):
        """mix(h) for a block that norms it and adds it to a float32 stream at once: float32, or the
        output projection's partial sums for that norm to add up (`ops.linear_for_stream`)."""
        return ops.linear_for_stream(self.mixed(h, ctx, cache), self.o_proj)


register_part("mixer", "matrix_memory", MatrixMemory)
