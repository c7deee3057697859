"""Linear attention with a decay per head over per-request state (csrc/lightning.cu)."""

from __future__ import annotations

import dataclasses

import torch

from atomserve_b200.ops.library import KernelLibraryError, check, dtype_code, lib, ptr, require_cuda, stream


SEGMENT_TOKENS = 64  # tokens of a segment when a long portion is cut to run side by side
SEGMENT_FROM = 256  # a request bringing at least this many tokens is cut


@dataclasses.dataclass
class Segments:
    """A step's requests cut into segments of consecutive rows: `bounds` int32 [S + 1] (rows),
    `req_start` int32 [R + 1] (the segments of each request), `index` int32 [S] = 0..S-1."""

    bounds: torch.Tensor
    req_start: torch.Tensor
    index: torch.Tensor
    count: int


def plan_segments(q_lens: list[int], device: torch.device) -> Segments | None:
    """The segments of a step whose requests bring `q_lens` tokens, or None when no request is
    long enough to be worth cutting (decode steps, short portions)."""
    if not q_lens or max(q_lens) < SEGMENT_FROM:
        return None
    bounds, req_start, row = [0], [0], 0
    for n in q_lens:
        pieces = -(-n // SEGMENT_TOKENS) if n >= SEGMENT_FROM else 1
        for i in range(pieces):
            bounds.append(row + min(n, (i + 1) * SEGMENT_TOKENS) if n >= SEGMENT_FROM else row + n)
        row += n
        req_start.append(len(bounds) - 1)
    count = len(bounds) - 1
    packed = torch.tensor(bounds + req_start + list(range(count)), dtype=torch.int32).to(device, non_blocking=True)
    a, b = len(bounds), len(bounds) + len(req_start)
    return Segments(packed[:a], packed[a:b], packed[b:], count)


def lightning_attention(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, state: torch.Tensor,
                        state_slots: torch.Tensor, req_q_start: torch.Tensor, decay: torch.Tensor,
                        num_requests: int, activation: bool = True, segments: Segments | None = None) -> torch.Tensor:  # fmt: skip
    """S <- decay_h S + k v^T, o = S^T q for every new token of every request, in order; the
    state [slots, H, D, V] (float32) is read and left updated in each request's slot.

    proj: [T, W] in the compute dtype, holding q (H * D columns from q_off), k (from k_off) and v
    (H * V columns from v_off), head by head; `activation`: SiLU on all three. Returns float32
    [T, H * V]. With `segments` (`plan_segments`) long portions run as segments side by side: each
    from a zero state, then a walk over each request's segments that hands every segment the
    state it starts from, then that state's share added to the segment's tokens."""
    require_cuda(proj, state, state_slots, req_q_start, decay)
    if proj.dim() != 2 or not proj.is_contiguous():
        raise KernelLibraryError("lightning_attention: proj must be a contiguous [tokens, columns] tensor")
    if state.dtype != torch.float32 or state.dim() != 4 or not state.is_contiguous():
        raise KernelLibraryError("lightning_attention: state must be contiguous float32 [slots, H, D, V]")
    _, H, D, V = state.shape
    if decay.dtype != torch.float32 or decay.shape != (H,):
        raise KernelLibraryError(f"lightning_attention: decay must be float32 [{H}]")
    for t in (state_slots, req_q_start):
        if t.dtype != torch.int32 or not t.is_contiguous():
            raise KernelLibraryError("lightning_attention: index tensors must be contiguous int32")
    if max(q_off, k_off) + H * D > proj.shape[1] or v_off + H * V > proj.shape[1]:
        raise KernelLibraryError("lightning_attention: the column ranges lie outside proj")
    out = torch.empty(proj.shape[0], H * V, device=proj.device, dtype=torch.float32)
    if segments is None:
        check(lib().asb_lightning_attention(ptr(out), ptr(proj), proj.shape[1], q_off, k_off, v_off, ptr(state),
                                            ptr(state_slots), ptr(req_q_start), ptr(decay), num_requests, H, D, V,
                                            int(activation), 0, dtype_code(proj), stream()))  # fmt: skip
        return out
    local = torch.empty(segments.count, H, D, V, device=proj.device, dtype=torch.float32)
    for mode in (1, 2):
        if mode == 2:
            check(lib().asb_lightning_scan(ptr(local), ptr(state), ptr(state_slots), ptr(segments.req_start),
                                           ptr(segments.bounds), ptr(decay), num_requests, H, D, V, stream()))  # fmt: skip
        check(lib().asb_lightning_attention(ptr(out), ptr(proj), proj.shape[1], q_off, k_off, v_off, ptr(local),
                                            ptr(segments.index), ptr(segments.bounds), ptr(decay), segments.count, H, D, V,
                                            int(activation), mode, dtype_code(proj), stream()))  # fmt: skip
    return out
