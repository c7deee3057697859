"""A plain, slow implementation of the Zogepel design, one function per mechanism, written from
the design's equations and sharing nothing with the package. Everything is float64 on the CPU,
token by token where the design is a recurrence; the tests hold the engine to it.

Notation: x is the residual stream [T, width] of one sequence, h a sublayer's input, positions
count from 0. A weight W is stored [out, in] and applied as h @ W.T.
"""

from __future__ import annotations

import math

import torch

F64 = torch.float64


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z**3)))


def rms_unit(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x divided by its root mean square over the last axis (eps inside the root)."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def layer_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """Centred norm with a weight and no bias; the variance is the mean squared deviation."""
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w


def rotate_half_pairs(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """x [T, heads, dim]: entry i < dims / 2 is paired with entry i + dims / 2 and the pair turned by
    position * base^(-2 i / dims); entries from `dims` on pass unchanged."""
    half = dims // 2
    out = x.clone()
    for i in range(half):
        a = positions.to(F64) * (base ** (-2.0 * i / dims))
        c, s = torch.cos(a)[:, None], torch.sin(a)[:, None]
        u, v = x[..., i], x[..., i + half]
        out[..., i] = u * c - v * s
        out[..., i + half] = v * c + u * s
    return out


def windowed_sink_softmax(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int, scale: float,
                          sink: torch.Tensor, first: int = 0) -> torch.Tensor:
    """q [Tq, H, d] are the queries of positions first .. first + Tq - 1; k, v [T, G, d] the keys and
    values of positions 0 .. T - 1. Position i sees j with 0 <= i - j < window; the denominator of
    head h also holds exp(sink[h])."""
    Tq, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(Tq, H, v.shape[2], dtype=F64)
    for t in range(Tq):
        i = first + t
        lo = max(0, i - window + 1)
        for head in range(H):
            g = head // (H // G)
            s = (k[lo : i + 1, g] @ q[t, head]) * scale
            top = torch.maximum(s.max(), sink[head])
            e = torch.exp(s - top)
            out[t, head] = (e[:, None] * v[lo : i + 1, g]).sum(0) / (e.sum() + torch.exp(sink[head] - top))
    return out


def sink_window_attention(h: torch.Tensor, w: dict, m: dict, eps: float, stored=lambda t: t) -> torch.Tensor:
    """Softmax attention in a sliding window with a sink; the values are the keys as projected;
    queries and keys are RMS-normed over their whole projection; no positions enter the scores;
    the heads are gated by sigmoid(W_g h) before W_o."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    q_raw, k_raw = stored(h @ w["q"].T), stored(h @ w["k"].T)
    q = stored(rms_unit(q_raw, eps) * w["q.norm"]).view(T, H, d)
    k = stored(rms_unit(k_raw, eps) * w["k.norm"]).view(T, G, d)
    out = stored(windowed_sink_softmax(q, k, k_raw.view(T, G, d), m["mask"]["size"], m["scale"], w["sink"]))
    return stored(out.reshape(T, H * d) * torch.sigmoid(stored(h @ w["g"].T))) @ w["o"].T


def retention(h: torch.Tensor, w: dict, m: dict, eps: float, positions: torch.Tensor, stored=lambda t: t) -> torch.Tensor:
    """Linear attention with a fixed decay per head: S <- decay S + k v^T, o = S^T q; q and k are
    rotated, k then scaled by dim^(-1/2); each head's o is made unit-RMS, the heads gated by
    silu(W_g h), then W_o."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = rotate_half_pairs(stored(h @ w["q"].T).view(T, H, d), positions, m["rot"]["base"], m["rot"]["dims"])
    k = rotate_half_pairs(stored(h @ w["k"].T).view(T, H, d), positions, m["rot"]["base"], m["rot"]["dims"]) * d**-0.5
    v = stored(h @ w["v"].T).view(T, H, dv)
    o = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        S = torch.zeros(d, dv, dtype=F64)
        for t in range(T):
            S = m["decay"][head] * S + torch.outer(k[t, head], v[t, head])
            o[t, head] = S.T @ q[t, head]
    o = rms_unit(o, eps).reshape(T, H * dv)
    z = stored(h @ w["g"].T)
    return stored(o * (z * torch.sigmoid(z))) @ w["o"].T


def parallel_mixer(h: torch.Tensor, w: dict, m: dict, eps: float, positions: torch.Tensor, stored=lambda t: t) -> torch.Tensor:
    """Half the sum of the two mixers' outputs, each RMS-normed over the width with its weight."""
    left = sink_window_attention(h, {k[5:]: v for k, v in w.items() if k.startswith("left.")}, m["left"], eps, stored)
    right = retention(h, {k[6:]: v for k, v in w.items() if k.startswith("right.")}, m["right"], eps, positions, stored)
    return 0.5 * (rms_unit(left, eps) * w["left.out"] + rms_unit(right, eps) * w["right.out"])


def mlstm(h: torch.Tensor, w: dict, m: dict, eps: float, stored=lambda t: t) -> torch.Tensor:
    """Matrix memory with exponential gates and a running maximum that starts at 0. `stored` is
    applied to what an implementation may keep in a 16-bit type (the q, k, v and gate projections
    and the gated heads); the tests use it to measure what such rounding alone does."""
    T = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = stored(h @ w["q"].T).view(T, H, d) * d**-0.5
    k = stored(h @ w["k"].T).view(T, H, d)
    v = stored(h @ w["v"].T).view(T, H, dv)
    gi = cap * torch.tanh((h @ w["i"].T + w["i.b"]) / cap)
    gf = torch.nn.functional.logsigmoid(cap * torch.tanh((h @ w["f"].T + w["f.b"]) / cap))
    o = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        S, n, top = torch.zeros(d, dv, dtype=F64), torch.zeros(d, dtype=F64), torch.zeros((), dtype=F64)
        for t in range(T):
            new_top = torch.maximum(gf[t, head] + top, gi[t, head])
            keep, take = torch.exp(gf[t, head] + top - new_top), torch.exp(gi[t, head] - new_top)
            S = keep * S + take * torch.outer(k[t, head], v[t, head])
            n = keep * n + take * k[t, head]
            top = new_top
            o[t, head] = (S.T @ q[t, head]) / (torch.maximum((n @ q[t, head]).abs(), torch.exp(-top)) + 1e-6)
    o = rms_unit(o, eps).reshape(T, H * dv) * w["norm"]
    return stored(o * torch.sigmoid(stored(h @ w["g"].T))) @ w["o"].T


def relu2_mlp(h: torch.Tensor, w: dict, stored=lambda t: t) -> torch.Tensor:
    return stored(torch.relu(stored(h @ w["up"].T)) ** 2) @ w["down"].T


def token_side(x: torch.Tensor, tokens: torch.Tensor, table: torch.Tensor, w: dict, layer: int, dim: int, eps: float,
               stored=lambda t: t) -> torch.Tensor:
    """The per-layer token input, before its residual multiplier: a gated slice of a second
    embedding projected to the width and RMS-normed with a weight."""
    e = table[tokens][:, layer * dim : (layer + 1) * dim]
    y = stored(gelu_tanh(x @ w["gate"].T) * e) @ w["proj"].T
    return rms_unit(y, eps) * w["norm"]


def _sub(tensors: dict, prefix: str) -> dict:
    return {k[len(prefix) :]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config: dict, tensors: dict, tokens: list[int], return_layers: bool = False, stored=lambda t: t):
    """Logits [T, vocab] of one whole sequence (and the stream after every layer). `stored` is
    applied to what an implementation may keep in a 16-bit type (the copy of the stream that the
    sublayers read, projections, activations between products); the tests use it to measure what
    such rounding alone does to the logits."""
    t = {k: v.to(F64) for k, v in tensors.items()}
    ids = torch.tensor(tokens, dtype=torch.long)
    positions = torch.arange(len(tokens))
    eps, mult = config["norm"]["eps"], config["residual_mult"]
    side = config.get("token_side")
    x = t["embed"][ids] * config["embedding"]["scale"]
    streams = []
    for i, layer in enumerate(config["layers"]):
        p = f"l{i}."
        if layer["type"] == "mlstm":
            y = mlstm(stored(x), _sub(t, p + "mix."), layer["mixer"], eps, stored)
        elif layer["type"] == "parallel":
            y = parallel_mixer(stored(x), _sub(t, p + "mix."), layer["mixer"], eps, positions, stored)
        else:
            raise ValueError(layer["type"])
        x = x + mult * layer_norm(y, t[p + "norm1"], eps) * t[p + "ls1"]
        if layer.get("mlp") is not None:
            y = relu2_mlp(stored(x), _sub(t, p + "mlp."), stored)
            x = x + mult * layer_norm(y, t[p + "norm2"], eps) * t[p + "ls2"]
        if side:
            x = x + mult * token_side(stored(x), ids, t["side.embed"], _sub(t, p + "side."), i, side["dim"], eps, stored)
        streams.append(x)
    logits = stored(layer_norm(x, t["final.norm"], eps)) @ t["head"].T
    return (logits, torch.stack(streams)) if return_layers else logits


def tensor_shapes(config: dict) -> dict[str, tuple[int, ...]]:
    """Every tensor of a model of this configuration, by name."""
    d, V, L = config["width"], config["vocab"], len(config["layers"])
    side = config.get("token_side")
    shapes = {"embed": (V, d), "final.norm": (d,), "head": (V, d)}
    if side:
        shapes["side.embed"] = (V, L * side["dim"])
    for i, layer in enumerate(config["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = shapes[p + "ls1"] = (d,)
        if layer["type"] == "mlstm":
            H, dk, dv = m["heads"], m["dim"], m["vdim"]
            shapes.update({p + "mix.q": (H * dk, d), p + "mix.k": (H * dk, d), p + "mix.v": (H * dv, d), p + "mix.g": (H * dv, d),
                           p + "mix.o": (d, H * dv), p + "mix.norm": (H * dv,), p + "mix.i": (H, d), p + "mix.i.b": (H,),
                           p + "mix.f": (H, d), p + "mix.f.b": (H,)})  # fmt: skip
        else:
            a, b = m["left"], m["right"]
            qw, kw = a["heads"] * a["dim"], a["kv_heads"] * a["dim"]
            shapes.update({p + "mix.left.q": (qw, d), p + "mix.left.k": (kw, d), p + "mix.left.q.norm": (qw,),
                           p + "mix.left.k.norm": (kw,), p + "mix.left.sink": (a["heads"],), p + "mix.left.g": (qw, d),
                           p + "mix.left.o": (d, qw), p + "mix.left.out": (d,), p + "mix.right.out": (d,)})  # fmt: skip
            H, dk, dv = b["heads"], b["dim"], b["vdim"]
            shapes.update({p + "mix.right.q": (H * dk, d), p + "mix.right.k": (H * dk, d), p + "mix.right.v": (H * dv, d),
                           p + "mix.right.g": (H * dv, d), p + "mix.right.o": (d, H * dv)})  # fmt: skip
        if layer.get("mlp") is not None:
            ff = layer["mlp"]["ff"]
            shapes.update({p + "mlp.up": (ff, d), p + "mlp.down": (d, ff), p + "norm2": (d,), p + "ls2": (d,)})
        if side:
            shapes.update({p + "side.gate": (side["dim"], d), p + "side.proj": (d, side["dim"]), p + "side.norm": (d,)})
    return shapes


def random_checkpoint(config: dict, seed: int) -> dict[str, torch.Tensor]:
    """Random float32 weights whose matrices are exact in bfloat16: matrices N(0, 1 / fan_in), gains
    1 + N(0, 0.1), sinks N(0, 2^2) (so that they weigh in the denominator), gate biases N(1, 1)."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(config).items():
        if name.endswith(".sink"):
            w[name] = 2.0 * torch.randn(shape, generator=g)
        elif name.endswith(".b"):
            w[name] = 1.0 + torch.randn(shape, generator=g)
        elif len(shape) == 1:
            w[name] = 1.0 + 0.1 * torch.randn(shape, generator=g)
        else:
            std = 1.0 if name in ("embed", "side.embed") else shape[1] ** -0.5
            w[name] = (torch.randn(shape, generator=g) * std).bfloat16().float()
    return w


def greedy_generate(config: dict, tensors: dict, prompt: list[int], n: int) -> list[int]:
    """The n tokens that follow `prompt` when the largest logit is taken each time (the whole
    sequence is run again for every token: slow and stateless)."""
    tokens = list(prompt)
    for _ in range(n):
        tokens.append(int(forward(config, tensors, tokens)[-1].argmax()))
    return tokens[len(prompt) :]
