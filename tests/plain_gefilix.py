"""A plain, slow implementation of the Gefilix design, one function per mechanism, written from
the design's equations and sharing nothing with the package: the oracle of the tests.

The design: a post-norm decoder, x <- norm(alpha x + sublayer(x)), whose layers carry one of
two mixers, a linear-attention recurrence with a fixed decay per head ("lightning") or softmax
attention over a cached low-rank latent ("latent_attention", optionally reading the latent an
earlier layer cached), and one of two feed-forwards, a dense erf-GELU one or routed experts with
grouped selection and a gated shared expert. Everything is computed in the dtype asked for
(float64 for reference values) token by token or with whole-prompt matrices, whichever is
plainer. `cfg` is the parsed config.json; `w` maps tensor names to tensors.
"""

from __future__ import annotations

import math

import torch


def rms_norm(x, gain, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * gain


def embed(w, cfg, tokens, dtype):
    return w["embed"][torch.as_tensor(tokens, dtype=torch.long)].to(dtype) * cfg["embedding"]["scale"]


def rotate_pairs(x, positions, base, dims):
    """x [T, ..., n]: of the first `dims` entries, (2i, 2i + 1) turns by position * base^(-2i/dims)."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims)
    angle = positions.to(x.dtype)[:, None] * freq[None, :]
    shape = (x.shape[0],) + (1,) * (x.dim() - 2) + (dims // 2,)
    cos, sin = torch.cos(angle).view(shape), torch.sin(angle).view(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def lightning_mixer(w, p, m, eps, h, state=None):
    """Linear attention with a decay per head. Returns (output [T, width], final state [H, D, V])."""
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    silu = torch.nn.functional.silu
    q = silu(h @ w[p + "q"].to(h.dtype).T).view(T, H, D)
    k = silu(h @ w[p + "k"].to(h.dtype).T).view(T, H, D)
    v = silu(h @ w[p + "v"].to(h.dtype).T).view(T, H, V)
    decay = torch.tensor(m["decay"], dtype=h.dtype).view(H, 1, 1)
    S = torch.zeros(H, D, V, dtype=h.dtype) if state is None else state.clone()
    outs = []
    for t in range(T):
        S = decay * S + k[t][:, :, None] * v[t][:, None, :]
        outs.append(torch.einsum("hdv,hd->hv", S, q[t]))
    o = torch.stack(outs).reshape(T, H * V)
    o = rms_norm(o, w[p + "norm"].to(h.dtype), eps) * torch.sigmoid(h @ w[p + "g"].to(h.dtype).T)
    return o @ w[p + "o"].to(h.dtype).T, S


def latent_keys(w, p, m, eps, h, positions):
    """What a latent-attention layer caches per token: the normed latent and the turned shared key part."""
    R = m["kv_rank"]
    d = h @ w[p + "dkv"].to(h.dtype).T
    c = rms_norm(d[:, :R], w[p + "dkv.norm"].to(h.dtype), eps)
    kr = rotate_pairs(d[:, R:], positions, m["rot"]["base"], m["rot"]["dims"])
    return c, kr


def latent_attention_mixer(w, p, m, eps, h, positions, cached, past=None):
    """Softmax attention whose keys and values are up-projections of the cached latent.
    `cached` = (c, kr) of this step's tokens (the layer's own or an earlier layer's), `past` the
    same for the tokens before them. Returns output [T, width]."""
    T = h.shape[0]
    H, D, Rt, V = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, kr = cached
    if past is not None:
        c, kr = torch.cat([past[0], c]), torch.cat([past[1], kr])
    S = c.shape[0]
    q = (h @ w[p + "q"].to(h.dtype).T).view(T, H, D + Rt)
    q_plain = q[..., :D]
    q_turn = rotate_pairs(q[..., D:], positions, m["rot"]["base"], m["rot"]["dims"])
    k_plain = (c @ w[p + "uk"].to(h.dtype).T).view(S, H, D)
    value = (c @ w[p + "uv"].to(h.dtype).T).view(S, H, V)
    scores = (torch.einsum("thd,shd->hts", q_plain, k_plain) + torch.einsum("thr,sr->hts", q_turn, kr)) * m["scale"]
    key_pos = torch.arange(S)
    visible = key_pos[None, :] <= positions[:, None]
    scores = scores.masked_fill(~visible[None], -math.inf)
    out = torch.einsum("hts,shv->thv", torch.softmax(scores, -1), value)
    out = out * torch.sigmoid(h @ w[p + "g"].to(h.dtype).T)[:, :, None]
    return out.reshape(T, H * V) @ w[p + "o"].to(h.dtype).T


def dense_feed_forward(w, p, h):
    up = h @ w[p + "up"].to(h.dtype).T
    return (0.5 * up * (1.0 + torch.erf(up / math.sqrt(2.0)))) @ w[p + "down"].to(h.dtype).T


def clamped_expert(w, p, h, limit):
    g = torch.clamp(h @ w[p + "gate"].to(h.dtype).T, max=limit)
    u = torch.clamp(h @ w[p + "up"].to(h.dtype).T, -limit, limit)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].to(h.dtype).T


def route(scores, router):
    """scores [T, E] -> (chosen [T, top], weights [T, top])."""
    E, top = router["experts"], router["top"]
    allowed = torch.ones_like(scores, dtype=torch.bool)
    groups = router.get("groups")
    if groups:
        per = E // groups["count"]
        grouped = scores.view(-1, groups["count"], per)
        group_score = grouped.topk(min(2, per), -1).values.sum(-1)
        best = group_score.topk(groups["keep"], -1).indices
        keep = torch.zeros_like(group_score, dtype=torch.bool).scatter_(1, best, True)
        allowed = keep[:, :, None].expand(-1, -1, per).reshape(-1, E)
    chosen = scores.masked_fill(~allowed, -math.inf).topk(top, -1).indices
    s = scores.gather(1, chosen)
    return chosen, s / (s.sum(-1, keepdim=True) + 1e-20) * router["scale"]


def expert_feed_forward(w, p, mlp, h):
    router = mlp["router"]
    scores = torch.sigmoid(h @ w[p + "router"].to(h.dtype).T)
    chosen, weights = route(scores, router)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t].tolist(), weights[t]):
            out[t] += a * clamped_expert(w, f"{p}e{e}.", h[t : t + 1], mlp["expert"]["limit"])[0]
    if mlp.get("shared"):
        gate = torch.sigmoid(h @ w[p + "shared.sg"].to(h.dtype).T)
        out = out + gate * clamped_expert(w, p + "shared.", h, mlp["shared"]["limit"])
    return out


def feed_forward(w, p, mlp, h):
    return dense_feed_forward(w, p, h) if mlp["kind"] == "dense" else expert_feed_forward(w, p, mlp, h)


def forward(w, cfg, tokens, dtype=torch.float64, start=0, carried=None, residuals=None):
    """Logits [T, vocab] of `tokens` at positions start, start + 1, ... `carried` (a dict this
    function fills and reads) holds what earlier calls for the same sequence left: the latent
    caches and recurrent states per layer, so a sequence may be fed in pieces. `residuals`, a
    list, receives the residual stream after every layer."""
    eps, alpha = cfg["norm"]["eps"], cfg["postln_alpha"]
    carried = {} if carried is None else carried
    positions = torch.arange(start, start + len(tokens))
    x = embed(w, cfg, tokens, dtype)
    now = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        if layer["type"] == "lightning":
            y, carried[i] = lightning_mixer(w, p + "mix.", m, eps, x, carried.get(i))
        else:
            src = m.get("kv_from")
            if src is None:
                now[i] = latent_keys(w, p + "mix.", m, eps, x, positions)
                src = i
            y = latent_attention_mixer(w, p + "mix.", m, eps, x, positions, now[src], carried.get(("kv", src)))
        x = rms_norm(alpha * x + y, w[p + "norm1"].to(dtype), eps)
        if layer.get("mlp"):
            x = rms_norm(alpha * x + feed_forward(w, p + "mlp.", layer["mlp"], x), w[p + "norm2"].to(dtype), eps)
        if residuals is not None:
            residuals.append(x.clone())
    for i, (c, kr) in now.items():
        past = carried.get(("kv", i))
        carried[("kv", i)] = (c, kr) if past is None else (torch.cat([past[0], c]), torch.cat([past[1], kr]))
    x = rms_norm(x, w["final.norm"].to(dtype), eps)
    return x @ w["head"].to(dtype).T


def tensor_shapes(cfg):
    """Every tensor name of a model of `cfg` with its shape."""
    d, out = cfg["width"], {"embed": (cfg["vocab"], cfg["width"])}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out[p + "norm1"] = (d,)
        if layer["type"] == "lightning":
            H, D, V = m["heads"], m["dim"], m["vdim"]
            out.update({p + "mix.q": (H * D, d), p + "mix.k": (H * D, d), p + "mix.v": (H * V, d),
                        p + "mix.g": (H * V, d), p + "mix.o": (d, H * V), p + "mix.norm": (H * V,)})  # fmt: skip
        else:
            H, D, Rt, V, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            out.update({p + "mix.q": (H * (D + Rt), d), p + "mix.uk": (H * D, R), p + "mix.uv": (H * V, R),
                        p + "mix.g": (H, d), p + "mix.o": (d, H * V)})  # fmt: skip
            if m.get("kv_from") is None:
                out.update({p + "mix.dkv": (R + Rt, d), p + "mix.dkv.norm": (R,)})
        mlp = layer.get("mlp")
        if not mlp:
            continue
        out[p + "norm2"] = (d,)
        if mlp["kind"] == "dense":
            out.update({p + "mlp.up": (mlp["ff"], d), p + "mlp.down": (d, mlp["ff"])})
        else:
            names = [f"e{e}" for e in range(mlp["router"]["experts"])]
            sizes = [mlp["expert"]["ff"]] * len(names)
            if mlp.get("shared"):
                names.append("shared")
                sizes.append(mlp["shared"]["ff"])
                out[p + "mlp.shared.sg"] = (1, d)
            for n, ff in zip(names, sizes):
                out.update({f"{p}mlp.{n}.gate": (ff, d), f"{p}mlp.{n}.up": (ff, d), f"{p}mlp.{n}.down": (d, ff)})
            out[p + "mlp.router"] = (mlp["router"]["experts"], d)
    out["final.norm"] = (d,)
    out["head"] = (cfg["vocab"], d)
    return out


def random_checkpoint(cfg, seed, matrix_std=None, bf16_exact=True):
    """Random float32 weights: matrices N(0, 1/fan_in) (so activations keep their size through
    the layers and scores, routers and gates are not all alike), vectors 1 + N(0, 0.1)."""
    g = torch.Generator().manual_seed(seed)
    w = {}
    for name, shape in tensor_shapes(cfg).items():
        if len(shape) == 1:
            w[name] = 1.0 + 0.1 * torch.randn(shape, generator=g)
        else:
            std = matrix_std if matrix_std is not None else shape[1] ** -0.5
            w[name] = torch.randn(shape, generator=g) * (1.0 if name == "embed" else std)
            if bf16_exact:
                w[name] = w[name].bfloat16().float()
    return w


def greedy_generate(w, cfg, prompt, n, dtype=torch.float64):
    """The n tokens that follow `prompt` when the largest logit is taken each time."""
    w = {k: v.to(dtype) for k, v in w.items()}
    carried, out = {}, []
    logits = forward(w, cfg, prompt, dtype, 0, carried)
    for i in range(n):
        out.append(int(logits[-1].argmax()))
        if i + 1 < n:
            logits = forward(w, cfg, out[-1:], dtype, len(prompt) + i, carried)
    return out
