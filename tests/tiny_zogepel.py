"""Small Zogepel configurations for the tests. They differ from one another in every size and
option: one head, several, odd counts; as many kv heads as heads and fewer; key sizes below, at
and above what one thread of the recurrence holds; value sizes other than key sizes; windows
shorter than a page, longer than the prompts, and across page borders; a rotation of a whole head,
of a part of it, and none; decays down to 0.5 and exactly 1; layers without a feed-forward; a
model without token inputs; a token-input size that is no multiple of 8 (the vendor GEMM's
shapes); residual multipliers below, at and above 1. Score scales are larger than 1 / sqrt(size),
so that scores spread over many units and single keys matter."""


def _left(heads, kv_heads, dim, window, scale):
    return dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=dim, scale=scale, mask=dict(size=window))


def _right(heads, dim, vdim, decay, base, dims):
    return dict(heads=heads, dim=dim, vdim=vdim, decay=decay, rot=dict(base=base, dims=dims))


def _parallel(left, right, ff):
    return dict(type="parallel", mixer=dict(left=left, right=right), mlp=dict(kind="dense", ff=ff) if ff else None)


def _mlstm(heads, dim, vdim, cap, ff):
    return dict(type="mlstm", mixer=dict(heads=heads, dim=dim, vdim=vdim, gate_cap=cap), mlp=dict(kind="dense", ff=ff) if ff else None)


ZOGEPEL_A = dict(
    architecture="Zogepel", vocab=300, width=96, residual_mult=1.3, norm=dict(eps=1e-5), embedding=dict(scale=2.5),
    token_side=dict(dim=12),
    layers=[
        _parallel(_left(6, 2, 24, 20, 0.45), _right(3, 16, 40, [0.5, 0.9, 1.0], 100.0, 8), 100),
        _mlstm(3, 24, 40, 6.0, None),
        _parallel(_left(4, 4, 16, 7, 0.6), _right(1, 96, 20, [0.97], 10000.0, 96), None),
        _mlstm(2, 96, 20, 15.0, 72),
    ],
)  # fmt: skip
BLOCK_SIZE_A = 16

ZOGEPEL_B = dict(
    architecture="Zogepel", vocab=257, width=64, residual_mult=1.0, norm=dict(eps=1e-6), embedding=dict(scale=1.0),
    layers=[
        _mlstm(1, 16, 16, 10.0, 72),
        _parallel(_left(2, 1, 32, 500, 0.3), _right(5, 8, 3, [0.8, 0.7, 0.99, 1.0, 0.6], 50.0, 0), 40),
        _mlstm(5, 8, 24, 4.0, None),
        _parallel(_left(3, 3, 40, 3, 0.35), _right(2, 24, 24, [0.93, 0.999], 1000.0, 12), 64),
    ],
)  # fmt: skip
BLOCK_SIZE_B = 8

# sizes at which the bfloat16 products run this package's tensor-core GEMMs
ZOGEPEL_C = dict(
    architecture="Zogepel", vocab=640, width=256, residual_mult=0.5, norm=dict(eps=2e-6), embedding=dict(scale=8.0),
    token_side=dict(dim=24),
    layers=[
        _mlstm(4, 128, 64, 11.0, 512),
        _parallel(_left(8, 2, 64, 100, 0.2), _right(4, 64, 128, [0.9, 0.99, 0.999, 1.0], 100000.0, 32), 384),
        _parallel(_left(4, 1, 128, 33, 0.15), _right(3, 32, 64, [0.75, 0.95, 0.98], 500.0, 32), None),
        _mlstm(2, 64, 160, 8.0, 256),
    ],
)  # fmt: skip
BLOCK_SIZE_C = 16

# matrix memories only (no layer keeps pages), a width that is no multiple of 8, one head, a tiny token input
ZOGEPEL_D = dict(
    architecture="Zogepel", vocab=130, width=100, residual_mult=0.9, norm=dict(eps=1e-5), embedding=dict(scale=3.0),
    token_side=dict(dim=5),
    layers=[_mlstm(1, 40, 56, 9.0, 60), _mlstm(3, 12, 20, 5.0, None)],
)  # fmt: skip
BLOCK_SIZE_D = 16

# attention beside retention only, a window of one token in one layer
ZOGEPEL_E = dict(
    architecture="Zogepel", vocab=140, width=48, residual_mult=0.8, norm=dict(eps=1e-5), embedding=dict(scale=2.0),
    layers=[_parallel(_left(2, 2, 8, 1, 0.9), _right(2, 4, 4, [0.9, 0.5], 30.0, 2), 56),
            _parallel(_left(4, 2, 12, 37, 0.5), _right(1, 20, 36, [0.98], 300.0, 20), None)],
)  # fmt: skip
BLOCK_SIZE_E = 8

ZOGEPEL = {"a": (ZOGEPEL_A, BLOCK_SIZE_A), "b": (ZOGEPEL_B, BLOCK_SIZE_B), "c": (ZOGEPEL_C, BLOCK_SIZE_C),
           "d": (ZOGEPEL_D, BLOCK_SIZE_D), "e": (ZOGEPEL_E, BLOCK_SIZE_E)}
