"""Operations of a float32 residual stream whose norm comes after the sum, and the further
feed-forward activations: the Python faces of csrc/stream_norm.cu and csrc/activation_more.cu."""

from __future__ import annotations

import torch

from atomserve_b200.ops.library import KernelLibraryError, check, dtype_code, lib, ptr, require_cuda, stream
from atomserve_b200.ops.linear import PartialSums, linear, linear_partial


def _stream(x: torch.Tensor, name: str) -> None:
    if x.dtype != torch.float32 or x.dim() != 2 or not x.is_contiguous():
        raise KernelLibraryError(f"{name} must be a contiguous float32 [rows, width] tensor, got {x.dtype} {tuple(x.shape)}")


def embedding_scaled(ids: torch.Tensor, table: torch.Tensor, scale: float, status: torch.Tensor) -> torch.Tensor:
    """float32 out[t] = table[ids[t]] * scale; an id outside the table sets `status` and gives zeros."""
    require_cuda(ids, table, status)
    if ids.dtype != torch.int32 or table.dim() != 2 or not table.is_contiguous():
        raise KernelLibraryError("embedding_scaled takes int32 ids and a contiguous table")
    out = torch.empty(ids.shape[0], table.shape[1], device=table.device, dtype=torch.float32)
    check(lib().asb_embedding_scaled(ptr(out), ptr(table), ptr(ids), ids.shape[0], table.shape[1], table.shape[0],
                                     float(scale), dtype_code(table), ptr(status), stream()))  # fmt: skip
    return out


def cast_rows(x: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """The float32 stream in the compute dtype (itself where that is float32)."""
    if dtype == torch.float32:
        return x
    require_cuda(x)
    _stream(x, "x")
    out = torch.empty_like(x, dtype=dtype)
    check(lib().asb_cast_rows(ptr(out), ptr(x), x.numel(), dtype_code(out), stream()))
    return out


def scaled_add_rms_norm(x: torch.Tensor, y: torch.Tensor | PartialSums | None, alpha: float, gain: torch.Tensor, eps: float,
                        dtype: torch.dtype, rows: torch.Tensor | None = None,
                        want_stream: bool = True) -> tuple[torch.Tensor | None, torch.Tensor]:  # fmt: skip
    """s = alpha x + y (y absent: alpha x); n = gain * s / sqrt(mean(s^2) + eps). x: float32
    [N, width]; y: float32 or bfloat16, or the partial sums of a product (`linear_for_stream`),
    which the kernel then adds up itself; `rows` (int32) picks source rows. Returns (n as float32 or
    None, n in `dtype`); with dtype float32 both are one tensor."""
    if isinstance(y, PartialSums):
        require_cuda(x, gain)
        _stream(x, "x")
        if rows is not None or dtype != torch.bfloat16 or (y.tokens, y.columns) != tuple(x.shape) or gain.shape != (x.shape[1],):
            raise KernelLibraryError("partial sums are added to all rows of a stream of their shape, for bfloat16 products")
        out32 = torch.empty_like(x)
        out_c = torch.empty_like(x, dtype=dtype)
        check(lib().asb_partial_scaled_add_rmsnorm(ptr(out32), ptr(out_c), ptr(y.workspace), *y.layout(), ptr(x), ptr(gain),
                                                   x.shape[0], x.shape[1], float(alpha), float(eps), stream()))  # fmt: skip
        return out32, out_c
    require_cuda(x, y, gain, rows)
    _stream(x, "x")
    width = x.shape[1]
    if gain.dtype != torch.float32 or gain.shape != (width,):
        raise KernelLibraryError(f"gain must be float32 [{width}]")
    if y is not None and (y.shape != x.shape or not y.is_contiguous() or y.dtype not in (torch.float32, torch.bfloat16)):
        raise KernelLibraryError("y must match x in shape, contiguous, float32 or bfloat16")
    n = x.shape[0] if rows is None else rows.shape[0]
    out32 = torch.empty(n, width, device=x.device, dtype=torch.float32) if (want_stream or dtype == torch.float32) else None
    out_c = None if dtype == torch.float32 else torch.empty(n, width, device=x.device, dtype=dtype)
    check(lib().asb_scaled_add_rmsnorm(ptr(out32), ptr(out_c), ptr(x), ptr(y), 0 if y is None else dtype_code(y), ptr(gain),
                                       ptr(rows), n, width, float(alpha), float(eps),
                                       dtype_code(out_c) if out_c is not None else 0, stream()))  # fmt: skip
    return out32, (out32 if out_c is None else out_c)


def linear_for_stream(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor | PartialSums:
    """x . w^T for a block that adds it to a float32 stream and norms the sum: float32, or, where
    the tensor-core GEMM runs with partial sums (few tokens) and `scaled_add_rms_norm` can read
    them, those partial sums. They live in the GEMMs' shared workspace, so the sum and norm must
    follow at once."""
    if w.shape[0] % 8 == 0 and w.shape[0] <= 8192:
        product = linear_partial(x, w)
        if product is not None:
            return product
    return linear(x, w, out_dtype=torch.float32)


def gated_rms_norm(o: torch.Tensor, gate: torch.Tensor, gain: torch.Tensor, eps: float) -> torch.Tensor:
    """gain * o / sqrt(mean(o^2) + eps) * sigmoid(gate) in gate's dtype. o: float32 [N, width];
    gate: [N, width] in the compute dtype, rows may be strided (a column range of a projection)."""
    require_cuda(o, gate, gain)
    _stream(o, "o")
    if gate.shape != o.shape or gate.stride(1) != 1:
        raise KernelLibraryError("gate must have o's shape with unit column stride")
    out = torch.empty(o.shape, device=o.device, dtype=gate.dtype)
    check(lib().asb_gated_rmsnorm(ptr(out), ptr(o), ptr(gate), gate.stride(0), ptr(gain), o.shape[0], o.shape[1],
                                  float(eps), dtype_code(gate), stream()))  # fmt: skip
    return out


ACTIVATIONS = {"gelu": 0, "gelu_tanh": 1, "relu2": 2}


def activation(x: torch.Tensor, kind: str) -> torch.Tensor:
    """Elementwise, float32 inside: "gelu" 0.5 z (1 + erf(z / sqrt 2)), "gelu_tanh" its tanh form,
    "relu2" max(z, 0)^2."""
    require_cuda(x)
    if kind not in ACTIVATIONS:
        raise KernelLibraryError(f"activation {kind!r} is not one of {sorted(ACTIVATIONS)}")
    if not x.is_contiguous():
        raise KernelLibraryError("activation takes a contiguous tensor")
    out = torch.empty_like(x)
    check(lib().asb_gelu(ptr(out), ptr(x), x.numel(), ACTIVATIONS[kind], dtype_code(x), stream()))
    return out


def gelu(x: torch.Tensor, tanh_form: bool = False) -> torch.Tensor:
    """The exact GELU 0.5 z (1 + erf(z / sqrt 2)), or its tanh form."""
    return activation(x, "gelu_tanh" if tanh_form else "gelu")


def clamped_glu(gate_up: torch.Tensor, limit: float, slope: float = 1.0, shift: float = 0.0) -> torch.Tensor:
    """[T, 2F] (gate columns first) -> g sigmoid(slope g) (u + shift) with g = min(gate, limit),
    u = clamp(up, -limit, limit); limit <= 0 clamps nothing."""
    require_cuda(gate_up)
    if gate_up.dim() != 2 or gate_up.shape[1] % 2 or not gate_up.is_contiguous():
        raise KernelLibraryError("clamped_glu takes a contiguous [tokens, 2 * intermediate] tensor")
    inter = gate_up.shape[1] // 2
    out = torch.empty(gate_up.shape[0], inter, device=gate_up.device, dtype=gate_up.dtype)
    check(lib().asb_clamped_glu(ptr(out), ptr(gate_up), gate_up.shape[0], inter, float(limit), float(slope), float(shift),
                                dtype_code(gate_up), stream()))  # fmt: skip
    return out
