"""Operations of blocks whose norm sits on the sublayer's output, x <- x + mult * norm(f(x)), and of
the mixers such blocks carry: the Python faces of csrc/out_norm.cu."""

from __future__ import annotations

import torch

from atomserve_b200.ops.library import KernelLibraryError, check, dtype_code, lib, ptr, require_cuda, stream
from atomserve_b200.ops.linear import PartialSums


def _f32_rows(x: torch.Tensor | None, name: str, shape: tuple | None = None) -> None:
    if x is None:
        return
    if x.dtype != torch.float32 or not x.is_contiguous() or (shape is not None and tuple(x.shape) != shape):
        raise KernelLibraryError(f"{name} must be contiguous float32{'' if shape is None else ' ' + str(list(shape))}, got {x.dtype} {tuple(x.shape)}")


def residual_out_norm(x: torch.Tensor | None, y: torch.Tensor | PartialSums, gain: torch.Tensor, eps: float, dtype: torch.dtype, *,
                      mult: float = 1.0, scale: torch.Tensor | None = None, centred: bool = True,
                      halves: tuple[torch.Tensor, torch.Tensor, torch.Tensor] | None = None,
                      rows: torch.Tensor | None = None, want_stream: bool = True) -> tuple[torch.Tensor | None, torch.Tensor]:  # fmt: skip
    """out = x + mult * N(y) * gain * scale, with N the centred norm (y - mean) / sqrt(var + eps) or,
    `centred=False`, y / sqrt(mean(y^2) + eps). x (float32 [N, width]) absent: the norm alone.
    `halves=(b, gain_a, gain_b)`: y stands for (R(y) gain_a + R(b) gain_b) / 2, R the unit-RMS norm.
    `rows` (int32) picks source rows. y may also be the partial sums of a product
    (`linear_for_stream`), which the kernel then adds up itself. Returns (out as float32 or None, out
    in `dtype`); with dtype float32 both are one tensor."""
    if isinstance(y, PartialSums):
        require_cuda(x, gain, scale)
        _f32_rows(x, "x", (y.tokens, y.columns))
        _f32_rows(gain, "gain", (y.columns,))
        _f32_rows(scale, "scale", (y.columns,))
        if x is None or rows is not None or halves is not None or dtype != torch.bfloat16:
            raise KernelLibraryError("partial sums are normed and added to all rows of a stream of their shape, for bfloat16 products")
        out32 = torch.empty_like(x)
        out_c = torch.empty_like(x, dtype=dtype)
        check(lib().asb_partial_residual_out_norm(ptr(out32), ptr(out_c), ptr(y.workspace), *y.layout(), ptr(x), ptr(gain),
                                                  ptr(scale), x.shape[0], x.shape[1], float(mult), float(eps), int(centred), stream()))  # fmt: skip
        return out32, out_c
    b, gain_a, gain_b = halves if halves is not None else (None, None, None)
    require_cuda(x, y, gain, scale, rows, b, gain_a, gain_b)
    if y.dim() != 2:
        raise KernelLibraryError("residual_out_norm: y must be [rows, width]")
    width = y.shape[1]
    _f32_rows(y, "y")
    _f32_rows(x, "x", tuple(y.shape))
    _f32_rows(b, "the second half", tuple(y.shape))
    for t, name in ((gain, "gain"), (scale, "scale"), (gain_a, "gain_a"), (gain_b, "gain_b")):
        _f32_rows(t, name, (width,))
    n = y.shape[0] if rows is None else rows.shape[0]
    out32 = torch.empty(n, width, device=y.device, dtype=torch.float32) if (want_stream or dtype == torch.float32) else None
    out_c = None if dtype == torch.float32 else torch.empty(n, width, device=y.device, dtype=dtype)
    check(lib().asb_residual_out_norm(ptr(out32), ptr(out_c), ptr(x), ptr(y), ptr(b), ptr(gain_a), ptr(gain_b), ptr(gain),
                                      ptr(scale), ptr(rows), n, width, float(mult), float(eps), int(centred),
                                      dtype_code(out_c) if out_c is not None else 0, stream()))  # fmt: skip
    return out32, (out32 if out_c is None else out_c)


def head_norm_gate(o: torch.Tensor, gate: torch.Tensor, heads: int, *, gain: torch.Tensor | None = None,
                   eps: float | None = None, gate_activation: str = "sigmoid",
                   normaliser: tuple[torch.Tensor, torch.Tensor, float] | None = None) -> torch.Tensor:  # fmt: skip
    """Per head of o [N, heads * width] (float32 or the gate's dtype): divided by its root mean
    square (`eps` None: not normed), times `gain` [heads * width] if given, times sigmoid or SiLU of
    `gate` [N, heads * width] (rows may be strided: a column range of a projection), in the gate's
    dtype. `normaliser=(nq, top, floor)`, float32 [N, heads] each: o is first divided by
    max(|nq|, exp(-top)) + floor."""
    nq, top, floor = normaliser if normaliser is not None else (None, None, 0.0)
    require_cuda(o, gate, gain, nq, top)
    if gate_activation not in ("sigmoid", "silu"):
        raise KernelLibraryError(f"gate activation {gate_activation!r} is neither 'sigmoid' nor 'silu'")
    if o.dim() != 2 or not o.is_contiguous() or o.shape[1] % heads or o.dtype not in (torch.float32, gate.dtype):
        raise KernelLibraryError("head_norm_gate: o must be contiguous [N, heads * width], float32 or the gate's dtype")
    if gate.shape != o.shape or gate.stride(1) != 1:
        raise KernelLibraryError("head_norm_gate: gate must have o's shape with unit column stride")
    _f32_rows(gain, "gain", (o.shape[1],))
    _f32_rows(nq, "nq", (o.shape[0], heads))
    _f32_rows(top, "top", (o.shape[0], heads))
    out = torch.empty(o.shape, device=o.device, dtype=gate.dtype)
    check(lib().asb_head_norm_gate(ptr(out), ptr(o), 0 if o.dtype == torch.float32 else 1, ptr(gate), gate.stride(0),
                                   ptr(gain), ptr(nq), ptr(top), o.shape[0], heads, o.shape[1] // heads,
                                   int(eps is not None), float(eps or 0.0), float(floor),
                                   int(gate_activation == "silu"), dtype_code(gate), stream()))  # fmt: skip
    return out


def projection_norm_store(proj: torch.Tensor, q_off: int, k_off: int, heads: int, kv_heads: int, head_dim: int,
                          q_gain: torch.Tensor, k_gain: torch.Tensor, eps: float, slots: torch.Tensor | None,
                          k_cache: torch.Tensor | None, v_cache: torch.Tensor | None) -> torch.Tensor:  # fmt: skip
    """From a projection [T, columns] holding queries (heads * head_dim columns from q_off) and
    keys (kv_heads * head_dim from k_off): both RMS-normed over all their columns at once, times
    their gains; returns the queries [T, heads, head_dim], writes the normed keys to `k_cache` and
    the keys as projected to `v_cache` at `slots` (pages [blocks, kv_heads, block_size, head_dim];
    slot -1 or no slots: nothing is written)."""
    require_cuda(proj, q_gain, k_gain, slots, k_cache, v_cache)
    if proj.dim() != 2 or proj.stride(1) != 1:
        raise KernelLibraryError("projection_norm_store: proj must be [tokens, columns] with unit column stride")
    qw, kw = heads * head_dim, kv_heads * head_dim
    if q_off + qw > proj.shape[1] or k_off + kw > proj.shape[1]:
        raise KernelLibraryError("projection_norm_store: the column ranges lie outside proj")
    _f32_rows(q_gain, "q_gain", (qw,))
    _f32_rows(k_gain, "k_gain", (kw,))
    bs = 1
    if slots is not None:
        if k_cache is None or v_cache is None or k_cache.shape != v_cache.shape or k_cache.dtype != proj.dtype or v_cache.dtype != proj.dtype:
            raise KernelLibraryError("projection_norm_store: pages of keys and values of proj's dtype and one shape are needed")
        if k_cache.shape[1] != kv_heads or k_cache.shape[3] != head_dim or slots.dtype != torch.int32:
            raise KernelLibraryError("projection_norm_store: pages must be [blocks, kv_heads, block_size, head_dim], slots int32")
        bs = k_cache.shape[2]
    q = torch.empty(proj.shape[0], heads, head_dim, device=proj.device, dtype=proj.dtype)
    check(lib().asb_projection_norm_store(ptr(q), ptr(proj), proj.stride(0), q_off, k_off, ptr(q_gain), ptr(k_gain), ptr(slots),
                                          ptr(k_cache), ptr(v_cache), proj.shape[0], heads, kv_heads, head_dim, bs,
                                          float(eps), dtype_code(proj), stream()))  # fmt: skip
    return q


def capped_gates_scan(z: torch.Tensor, i_off: int, f_off: int, heads: int, i_bias: torch.Tensor, f_bias: torch.Tensor,
                      cap: float, top_state: torch.Tensor, state_slots: torch.Tensor, req_q_start: torch.Tensor,
                      num_requests: int) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:  # fmt: skip
    """The gates of a matrix memory with exponential gating. z: float32 [T, columns] with the input
    gate's pre-activations in `heads` columns from i_off and the forget gate's from f_off. Log gates
    i = cap tanh((zi + bi) / cap), f = logsigmoid(cap tanh((zf + bf) / cap)); per request and head, in
    token order, top_t = max(f_t + top_(t-1), i_t), carried in `top_state` [slots, heads]. Returns
    (decay, gain, top), float32 [T, heads]: exp(f_t + top_(t-1) - top_t), exp(i_t - top_t), top_t."""
    require_cuda(z, i_bias, f_bias, top_state, state_slots, req_q_start)
    if z.dtype != torch.float32 or z.dim() != 2 or z.stride(1) != 1 or max(i_off, f_off) + heads > z.shape[1]:
        raise KernelLibraryError("capped_gates_scan: z must be float32 [T, columns] holding both gates' columns")
    _f32_rows(i_bias, "i_bias", (heads,))
    _f32_rows(f_bias, "f_bias", (heads,))
    if top_state.dtype != torch.float32 or top_state.dim() != 2 or top_state.shape[1] != heads or not top_state.is_contiguous():
        raise KernelLibraryError(f"capped_gates_scan: the running maxima must be contiguous float32 [slots, {heads}]")
    decay = torch.empty(z.shape[0], heads, device=z.device, dtype=torch.float32)
    gain, top = torch.empty_like(decay), torch.empty_like(decay)
    check(lib().asb_capped_gates_scan(ptr(decay), ptr(gain), ptr(top), ptr(z), z.stride(0), i_off, f_off, ptr(i_bias),
                                      ptr(f_bias), ptr(top_state), ptr(state_slots), ptr(req_q_start), num_requests, heads,
                                      float(cap), stream()))  # fmt: skip
    return decay, gain, top


def gated_token_slice(z: torch.Tensor, table: torch.Tensor, ids: torch.Tensor, offset: int) -> torch.Tensor:
    """gelu_tanh(z) * table[ids, offset : offset + dim] in the table's dtype; z: float32 [T, dim]."""
    require_cuda(z, table, ids)
    if z.dtype != torch.float32 or z.dim() != 2 or not z.is_contiguous() or ids.dtype != torch.int32 or not table.is_contiguous():
        raise KernelLibraryError("gated_token_slice takes float32 z [T, dim], int32 ids and a contiguous table")
    out = torch.empty(z.shape, device=z.device, dtype=table.dtype)
    check(lib().asb_gated_token_slice(ptr(out), ptr(z), ptr(table), ptr(ids), z.shape[0], table.shape[1], offset, z.shape[1],
                                      table.shape[0], dtype_code(table), stream()))  # fmt: skip
    return out
