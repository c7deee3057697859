"""Zogepel as a ModelSpec: a decoder over a float32 residual stream whose layers add the normed
output of each sublayer, x <- x + mult * ls1 * LN1(mixer(x)), x <- x + mult * ls2 * LN2(ff(x)),
x <- x + mult * side(x, token), with LN a centred norm with a gain and no bias and ls a layer scale
per channel. Mixers: "mlstm", a matrix memory with exponential gating, or "parallel", attention
with a sink in a sliding window beside retention. Layer i's tensors are `l<i>.norm1`, `l<i>.ls1`,
`l<i>.mix.*`, `l<i>.norm2`, `l<i>.ls2`, `l<i>.mlp.*`, `l<i>.side.*`; the embedding is `embed`
(scaled), the token inputs' table `side.embed`, the last norm `final.norm`, the head `head`.

What the design fixes and the configuration therefore does not carry: the squared ReLU in the
feed-forward; the matrix memory's query scale dim^(-1/2), its floor 1e-6 and its sigmoid gate; in
the attention the whole-projection norms, values that are the keys, no positions, the sigmoid
gate; in retention the rotate-half pairing, the key scale dim^(-1/2) after the rotation, heads
normed one by one without a gain, the SiLU gate; the token input's tanh-form GELU and RMS norm.
"""

from __future__ import annotations

from atomserve_b200.config.registry import register_architecture
from atomserve_b200.config.zogepel_config import ZogepelConfig
from atomserve_b200.parts.spec import LayerCall, LayerSpec, ModelSpec, PartSpec

MEMORY_FLOOR = 1e-6


def _mixer(c: ZogepelConfig, layer: dict, prefix: str) -> PartSpec:
    m = layer["mixer"]
    if layer["type"] == "mlstm":
        return PartSpec("matrix_memory", dict(heads=m["heads"], dim=m["dim"], vdim=m["vdim"], gate_cap=m["gate_cap"],
                                              eps=c.norm_eps, floor=MEMORY_FLOOR), prefix)  # fmt: skip
    left, right = m["left"], m["right"]
    rot = right["rot"]
    position = PartSpec("rotary", dict(head_dim=right["dim"], theta=rot["base"], rotary_dim=rot["dims"], pairing="half"))
    return PartSpec("parallel_mixers", dict(
        left=PartSpec("sink_attention", dict(num_heads=left["heads"], num_kv_heads=left["kv_heads"], head_dim=left["dim"],
                                             scale=left["scale"], eps=c.norm_eps, window=left["mask"]["size"]), prefix + "left."),
        right=PartSpec("lightning_attention", dict(heads=right["heads"], dim=right["dim"], vdim=right["vdim"],
                                                   decay=tuple(right["decay"]), eps=c.norm_eps, activation="none",
                                                   position=position if rot["dims"] else None, k_scale=right["dim"] ** -0.5,
                                                   head_norm="each", norm_gain=False, gate="silu"), prefix + "right."),
        eps=c.norm_eps,
    ), prefix)  # fmt: skip


def build_spec(c: ZogepelConfig) -> ModelSpec:
    layers, schedule, ignored = [], [], []
    side_width = (c.token_side_dim or 0) * len(c.layers)
    for i, layer in enumerate(c.layers):
        p = f"l{i}."
        norm = dict(eps=c.norm_eps, mult=c.residual_mult, centred=True)
        mlp = layer.get("mlp")
        if mlp is None:
            ignored += [p + "norm2", p + "ls2"]  # a layer without a feed-forward needs neither
        layers.append(LayerSpec(
            block="output_norm",
            mixer=_mixer(c, layer, p + "mix."),
            feed_forward=(PartSpec("activation_mlp", dict(intermediate_size=mlp["ff"], activation="relu2"), p + "mlp.")
                          if mlp is not None else PartSpec("none")),
            mixer_norm=PartSpec("output_norm", dict(norm, tensor=p + "norm1", scale_tensor=p + "ls1")),
            feed_forward_norm=(PartSpec("output_norm", dict(norm, tensor=p + "norm2", scale_tensor=p + "ls2"))
                               if mlp is not None else PartSpec("none")),
            token_input=(PartSpec("gated_token_slice", dict(vocab_size=c.vocab, table="side.embed", table_width=side_width,
                                                            offset=i * c.token_side_dim, dim=c.token_side_dim,
                                                            eps=c.norm_eps, mult=c.residual_mult), p + "side.")
                         if c.token_side_dim is not None else None),
        ))  # fmt: skip
        schedule.append(LayerCall(i))
    return ModelSpec(
        hidden_size=c.width,
        vocab_size=c.vocab,
        max_positions=c.max_positions,
        embedding=PartSpec("scaled_embedding", dict(vocab_size=c.vocab, scale=c.embedding_scale, tensor="embed")),
        layers=tuple(layers),
        schedule=tuple(schedule),
        final_norm=PartSpec("output_norm", dict(eps=c.norm_eps, centred=True, tensor="final.norm")),
        head=PartSpec("lm_head", dict(vocab_size=c.vocab, tied=False, tensor="head")),
        ignored_tensors=tuple(ignored),
    )


register_architecture(ZogepelConfig.architecture, ZogepelConfig, build_spec)
