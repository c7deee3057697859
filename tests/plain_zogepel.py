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


def sink_window_attention(h: torch.Tensor, w: dict, m: dict, eps: float) -> torch.Tensor:
    """Softmax attention in a sliding window whose denominator also holds exp(sink) per head; the
    values are the keys as projected; queries and keys are RMS-normed over their whole projection;
    no positions enter the scores; the heads are gated by sigmoid(W_g h) before W_o."""
    T = h.shape[0]
    H, G, d, window, scale = m["heads"], m["kv_heads"], m["dim"], m["mask"]["size"], m["scale"]
    q_raw, k_raw = h @ w["q"].T, h @ w["k"].T
    v = k_raw.view(T, G, d)
    q = (rms_unit(q_raw, eps) * w["q.norm"]).view(T, H, d)
    k = (rms_unit(k_raw, eps) * w["k.norm"]).view(T, G, d)
    out = torch.zeros(T, H, d, dtype=F64)
    for t in range(T):
        lo = max(0, t - window + 1)
        for head in range(H):
            g = head // (H // G)
            s = (k[lo : t + 1, g] @ q[t, head]) * scale
            top = torch.maximum(s.max(), w["sink"][head])
            e = torch.exp(s - top)
            denom = e.sum() + torch.exp(w["sink"][head] - top)
            out[t, head] = (e[:, None] * v[lo : t + 1, g]).sum(0) / denom
    gate = torch.sigmoid(h @ w["g"].T)
    return (out.reshape(T, H * d) * gate) @ w["o"].T


def retention(h: torch.Tensor, w: dict, m: dict, eps: float, positions: torch.Tensor) -> torch.Tensor:
    """Linear attention with a fixed decay per head: S <- decay S + k v^T, o = S^T q; q and k are
    rotated, k then scaled by dim^(-1/2); each head's o is made unit-RMS, the heads gated by
    silu(W_g h), then W_o."""
    T = h.shape[0]
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    q = rotate_half_pairs((h @ w["q"].T).view(T, H, d), positions, m["rot"]["base"], m["rot"]["dims"])
    k = rotate_half_pairs((h @ w["k"].T).view(T, H, d), positions, m["rot"]["base"], m["rot"]["dims"]) * d**-0.5
    v = (h @ w["v"].T).view(T, H, dv)
    o = torch.zeros(T, H, dv, dtype=F64)
    for head in range(H):
        S = torch.zeros(d, dv, dtype=F64)
        for t in range(T):
            S = m["decay"][head] * S + torch.outer(k[t, head], v[t, head])
            o[t, head] = S.T @ q[t, head]
    o = rms_unit(o, eps).reshape(T, H * dv)
    z = h @ w["g"].T
    return (o * (z * torch.sigmoid(z))) @ w["o"].T


def parallel_mixer(h: torch.Tensor, w: dict, m: dict, eps: float, positions: torch.Tensor) -> torch.Tensor:
    """Half the sum of the two mixers' outputs, each RMS-normed over the width with its weight."""
    left = sink_window_attention(h, {k[5:]: v for k, v in w.items() if k.startswith("left.")}, m["left"], eps)
    right = retention(h, {k[6:]: v for k, v in w.items() if k.startswith("right.")}, m["right"], eps, positions)
    return 0.5 * (rms_unit(left, eps) * w["left.out"] + rms_unit(right, eps) * w["right.out"])


def mlstm(h: torch.Tensor, w: dict, m: dict, eps: float) -> torch.Tensor:
    """Matrix memory with exponential gates and a running maximum that starts at 0."""
    T = h.shape[0]
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    q = (h @ w["q"].T).view(T, H, d) * d**-0.5
    k = (h @ w["k"].T).view(T, H, d)
    v = (h @ w["v"].T).view(T, H, dv)
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
    return (o * torch.sigmoid(h @ w["g"].T)) @ w["o"].T


def relu2_mlp(h: torch.Tensor, w: dict) -> torch.Tensor:
    return (torch.relu(h @ w["up"].T) ** 2) @ w["down"].T


def token_side(x: torch.Tensor, tokens: torch.Tensor, table: torch.Tensor, w: dict, layer: int, dim: int, eps: float) -> torch.Tensor:
    """The per-layer token input, before its residual multiplier: a gated slice of a second
    embedding projected to the width and RMS-normed with a weight."""
    e = table[tokens][:, layer * dim : (layer + 1) * dim]
    y = (gelu_tanh(x @ w["gate"].T) * e) @ w["proj"].T
    return rms_unit(y, eps) * w["norm"]


def _sub(tensors: dict, prefix: str) -> dict:
    return {k[len(prefix) :]: v for k, v in tensors.items() if k.startswith(prefix)}


def forward(config: dict, tensors: dict, tokens: list[int], return_layers: bool = False):
    """Logits [T, vocab] of one whole sequence (and the stream after every layer)."""
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
            y = mlstm(x, _sub(t, p + "mix."), layer["mixer"], eps)
        elif layer["type"] == "parallel":
            y = parallel_mixer(x, _sub(t, p + "mix."), layer["mixer"], eps, positions)
        else:
            raise ValueError(layer["type"])
        x = x + mult * layer_norm(y, t[p + "norm1"], eps) * t[p + "ls1"]
        if layer.get("mlp") is not None:
            y = relu2_mlp(x, _sub(t, p + "mlp."))
            x = x + mult * layer_norm(y, t[p + "norm2"], eps) * t[p + "ls2"]
        if side:
            x = x + mult * token_side(x, ids, t["side.embed"], _sub(t, p + "side."), i, side["dim"], eps)
        streams.append(x)
    logits = layer_norm(x, t["final.norm"], eps) @ t["head"].T
    return (logits, torch.stack(streams)) if return_layers else logits
