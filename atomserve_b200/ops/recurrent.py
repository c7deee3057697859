"""Linear attention with a decay per head over per-request state (csrc/lightning.cu)."""

from __future__ import annotations

import torch

from atomserve_b200.ops.library import KernelLibraryError, check, dtype_code, lib, ptr, require_cuda, stream


def lightning_attention(proj: torch.Tensor, q_off: int, k_off: int, v_off: int, state: torch.Tensor,
                        state_slots: torch.Tensor, req_q_start: torch.Tensor, decay: torch.Tensor,
                        num_requests: int, activation: bool = True) -> torch.Tensor:  # fmt: skip
    """S <- decay_h S + k v^T, o = S^T q for every new token of every request, in order; the
    state [slots, H, D, V] (float32) is read and left updated in each request's slot.

    proj: [T, W] in the compute dtype, holding q (H * D columns from q_off), k (from k_off) and v
    (H * V columns from v_off), head by head; `activation`: SiLU on all three. Returns float32
    [T, H * V]."""
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
    check(lib().asb_lightning_attention(ptr(out), ptr(proj), proj.shape[1], q_off, k_off, v_off, ptr(state),
                                        ptr(state_slots), ptr(req_q_start), ptr(decay), num_requests, H, D, V,
                                        int(activation), dtype_code(proj), stream()))  # fmt: skip
    return out
