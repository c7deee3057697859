"""Gefilix as a ModelSpec: a post-norm decoder over a float32 residual stream,
x <- norm(alpha x + mixer(x)), x <- norm(alpha x + ff(x)), whose layers carry linear attention
with a decay per head or softmax attention over a cached latent, and a dense GELU feed-forward,
routed experts or none. Layer i's tensors are `l<i>.norm1`, `l<i>.mix.*`, `l<i>.norm2`,
`l<i>.mlp.*`; the embedding is `embed` (scaled), the last norm `final.norm`, the head `head`.

What the design fixes and the configuration therefore does not carry: SiLU on the recurrence's
q, k and v; neighbouring pairs in the rotation; the exact GELU in dense layers; in experts the
sigmoid's slope 1.702 and the shift 1 on the up branch; sigmoid router scores, a group scored by
its two largest, chosen weights renormalised; a sigmoid gate on the shared expert.
"""

from __future__ import annotations

from atomserve_b200.config.gefilix_config import GefilixConfig
from atomserve_b200.config.registry import register_architecture
from atomserve_b200.parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec

EXPERT_SLOPE, EXPERT_SHIFT, GROUP_TOP = 1.702, 1.0, 2


def _mixer(c: GefilixConfig, layer: dict, prefix: str) -> PartSpec:
    m = layer["mixer"]
    if layer["type"] == "lightning":
        return PartSpec("lightning_attention", dict(heads=m["heads"], dim=m["dim"], vdim=m["vdim"], decay=tuple(m["decay"]),
                                                    eps=c.norm_eps, activation="silu"), prefix)  # fmt: skip
    rot = m["rot"]
    position = PartSpec("rotary", dict(head_dim=m["rot_dim"], theta=rot["base"], rotary_dim=rot["dims"], pairing="interleaved"))
    return PartSpec("latent_attention", dict(heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"], vdim=m["vdim"],
                                             kv_rank=m["kv_rank"], scale=m["scale"], eps=c.norm_eps, position=position,
                                             reads_cache_of_another=m.get("kv_from") is not None), prefix)  # fmt: skip


def _feed_forward(mlp: dict | None, prefix: str) -> PartSpec:
    if mlp is None:
        return PartSpec("none")
    if mlp["kind"] == "dense":
        return PartSpec("gelu_mlp", dict(intermediate_size=mlp["ff"], tanh_form=False), prefix)
    router, groups, shared = mlp["router"], mlp["router"].get("groups") or {}, mlp.get("shared") or {}
    return PartSpec("routed_experts", dict(
        experts=router["experts"], top=router["top"], expert_ff=mlp["expert"]["ff"], limit=mlp["expert"]["limit"],
        groups=groups.get("count", 1), group_top=GROUP_TOP, keep=groups.get("keep", 1), scale=router["scale"],
        slope=EXPERT_SLOPE, shift=EXPERT_SHIFT, score="sigmoid", renormalise=True,
        shared_ff=shared.get("ff"), shared_limit=shared.get("limit"), shared_gated=True,
    ), prefix)  # fmt: skip


def build_spec(c: GefilixConfig) -> ModelSpec:
    layers, schedule = [], []
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        norm = dict(eps=c.norm_eps, alpha=c.postln_alpha)
        has_ff = layer.get("mlp") is not None
        layers.append(LayerSpec(
            block="post_norm",
            mixer=_mixer(c, layer, p + "mix."),
            feed_forward=_feed_forward(layer.get("mlp"), p + "mlp."),
            mixer_norm=PartSpec("stream_rms_norm", dict(norm, tensor=p + "norm1")),
            feed_forward_norm=PartSpec("stream_rms_norm", dict(norm, tensor=p + "norm2")) if has_ff else PartSpec("none"),
        ))  # fmt: skip
        # the run order is the layer order; a layer with kv_from reads the pages of that layer's entry
        schedule.append(LayerCall(i, cache_from=layer["mixer"].get("kv_from")))
    return ModelSpec(
        hidden_size=c.width,
        vocab_size=c.vocab,
        max_positions=c.max_positions,
        embedding=PartSpec("scaled_embedding", dict(vocab_size=c.vocab, scale=c.embedding_scale, tensor="embed")),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=PartSpec("stream_rms_norm", dict(eps=c.norm_eps, tensor="final.norm")),
        head=PartSpec("lm_head", dict(vocab_size=c.vocab, tied=False, tensor="head")),
    )


register_architecture(GefilixConfig.architecture, GefilixConfig, build_spec)
