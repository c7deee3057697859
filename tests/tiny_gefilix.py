"""Small Gefilix configurations for the tests. They differ from one another in every size and
option: heads of 1, several and odd counts; key sizes below, at and above what one thread of the
recurrence holds; value sizes other than key sizes; a latent narrower and wider than a warp;
a rotation of the whole position-encoded part and of a part of it; a layer without a feed-forward;
layers that read an earlier layer's cache; two caches of different widths in one model; experts
with and without groups, with and without a shared expert, one choice and several; K that is no
multiple of 8 (the vendor GEMM's shapes). Attention scales are larger than 1 / sqrt(size), so that
scores spread over many units and single keys matter."""

import copy


def _latent(heads, dim, rot_dim, vdim, kv_rank, scale, base=10000.0, dims=None, kv_from=None):
    m = dict(heads=heads, dim=dim, rot_dim=rot_dim, vdim=vdim, kv_rank=kv_rank, scale=scale,
             rot=dict(base=base, dims=dims or rot_dim))  # fmt: skip
    if kv_from is not None:
        m["kv_from"] = kv_from
    return dict(type="latent_attention", mixer=m)


def _lightning(heads, dim, vdim, decay):
    return dict(type="lightning", mixer=dict(heads=heads, dim=dim, vdim=vdim, decay=decay))


def _moe(experts, top, ff, limit, scale, groups=None, shared=None):
    router = dict(experts=experts, top=top, scale=scale)
    if groups:
        router["groups"] = dict(count=groups[0], keep=groups[1])
    mlp = dict(kind="moe", expert=dict(ff=ff, limit=limit), router=router)
    if shared:
        mlp["shared"] = dict(ff=shared[0], limit=shared[1])
    return mlp


GEFILIX_A = dict(
    architecture="Gefilix", vocab=300, width=96, postln_alpha=1.5, norm=dict(eps=1e-5), embedding=dict(scale=0.7),
    layers=[
        dict(_lightning(3, 24, 40, [0.5, 0.9, 1.0]), mlp=dict(kind="dense", ff=100)),
        dict(_latent(5, 24, 8, 16, 40, 0.8, base=1000.0), mlp=_moe(6, 2, 48, 1.5, 1.7, groups=(3, 2), shared=(32, 3.0))),
        dict(_lightning(2, 96, 20, [0.97, 0.8]), mlp=None),
        dict(_latent(3, 16, 8, 24, 40, 1.1, base=1000.0, kv_from=1), mlp=_moe(4, 1, 40, 0.5, 1.0)),
    ],
)  # fmt: skip
BLOCK_SIZE_A = 16

GEFILIX_B = dict(
    architecture="Gefilix", vocab=257, width=64, postln_alpha=1.0, norm=dict(eps=1e-6), embedding=dict(scale=1.0),
    layers=[
        dict(_latent(1, 32, 16, 32, 64, 0.6, dims=8), mlp=dict(kind="dense", ff=72)),
        dict(_latent(4, 16, 4, 8, 24, 1.0, base=50.0), mlp=_moe(8, 3, 24, 2.5, 2.0, groups=(2, 2))),
        dict(_latent(2, 8, 16, 40, 64, 0.9, dims=8, kv_from=0), mlp=None),
        dict(_lightning(1, 16, 16, [0.93]), mlp=_moe(5, 5, 16, 1.0, 0.5, shared=(8, 1.0))),
    ],
)  # fmt: skip
BLOCK_SIZE_B = 8

# sizes at which the bfloat16 products run this package's tensor-core GEMMs
GEFILIX_C = dict(
    architecture="Gefilix", vocab=640, width=320, postln_alpha=3.0, norm=dict(eps=2e-6), embedding=dict(scale=0.25),
    layers=[
        dict(_lightning(4, 128, 64, [0.6, 0.9, 0.99, 0.999]), mlp=_moe(8, 2, 128, 2.0, 2.5, groups=(4, 2), shared=(64, 2.0))),
        dict(_latent(4, 64, 32, 64, 96, 0.35, base=100000.0), mlp=dict(kind="dense", ff=512)),
        dict(_lightning(5, 64, 128, [0.7, 0.8, 0.9, 0.95, 1.0]), mlp=_moe(12, 3, 64, 1.0, 1.5, groups=(3, 1), shared=(128, 1.5))),
        dict(_latent(8, 32, 32, 32, 96, 0.5, base=100000.0, kv_from=1), mlp=dict(kind="dense", ff=256)),
    ],
)  # fmt: skip
BLOCK_SIZE_C = 16

GEFILIX = {"a": (GEFILIX_A, BLOCK_SIZE_A), "b": (GEFILIX_B, BLOCK_SIZE_B), "c": (GEFILIX_C, BLOCK_SIZE_C)}


def calm(cfg):
    """The same model with every allowed expert chosen (all groups kept, as many choices as
    experts): selection then has no near-ties that bfloat16 rounding of the stream could turn, so
    whole-model bfloat16 runs can be held to the float64 oracle. (Selection itself is held
    exactly by the float32 runs and, in bfloat16, at the level of the part on equal inputs.)"""
    out = copy.deepcopy(cfg)
    for layer in out["layers"]:
        mlp = layer.get("mlp")
        if mlp and mlp["kind"] == "moe":
            router = mlp["router"]
            if "groups" in router:
                router["groups"]["keep"] = router["groups"]["count"]
            router["top"] = min(router["experts"], 32)
    return out
