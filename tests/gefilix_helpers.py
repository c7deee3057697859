"""Test-side helpers for the Gefilix tests: model folders from the plain implementation's
random weights, oracles, and the comparison rule."""

from __future__ import annotations

import json
import pathlib

import torch
from safetensors.torch import save_file

import plain_gefilix as plain

FLOAT32_TOLERANCE = 2e-5  # largest difference over the largest reference magnitude
BFLOAT16_TOLERANCE = 0.04  # per row: rms of the difference (mean taken off) over the rms of the reference (mean taken off)


def write_folder(cfg: dict, w: dict, folder: pathlib.Path) -> pathlib.Path:
    folder.mkdir(parents=True, exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    save_file({k: v.contiguous() for k, v in w.items()}, str(folder / "model.safetensors"))
    return folder


def prompts(cfg: dict, lengths: list[int], seed: int) -> list[list[int]]:
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in lengths]


def oracle(w: dict, cfg: dict, prompt: list[int]) -> torch.Tensor:
    """float64 logits of the whole prompt, kept as float32."""
    return plain.forward({k: v.double() for k, v in w.items()}, cfg, prompt).float()


def check(got: torch.Tensor, ref: torch.Tensor, dtype, what: str, bf16_tolerance: float = BFLOAT16_TOLERANCE) -> None:
    got = got.float().cpu()
    assert got.shape == ref.shape, f"{what}: shape {tuple(got.shape)} for {tuple(ref.shape)}"
    assert torch.isfinite(got).all(), f"{what}: not finite"
    if dtype in ("float32", torch.float32):
        err = float((got.double() - ref.double()).abs().max() / ref.double().abs().max())
        assert err < FLOAT32_TOLERANCE, f"{what}: relative error {err:.3g}"
    else:
        d = (got - ref).double()
        if got.dim() == 2 and got.shape[1] > 1:
            d = d - d.mean(-1, keepdim=True)
            scale = (ref.double() - ref.double().mean(-1, keepdim=True)).pow(2).mean().sqrt()
        else:
            scale = ref.double().pow(2).mean().sqrt()
        err = float(d.pow(2).mean(-1).sqrt().max() / scale)
        assert err < bf16_tolerance, f"{what}: error {err:.3g} of the reference's spread, allowed {bf16_tolerance}"
