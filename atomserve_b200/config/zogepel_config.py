"""Typed configuration of the Zogepel design, read from its own config.json keys.

A Zogepel model is a list of layers around a float32 residual stream, each adding the normed,
layer-scaled output of its mixer, then of its feed-forward (if it has one), then a per-layer
token input (if the model has one), every time multiplied by `residual_mult`. A layer's mixer is
"mlstm" (a matrix memory with exponential gating) or "parallel" (attention with a sink in a sliding
window beside retention with a decay per head). Every size and every constant that may differ
between models is a key; what the design fixes is written in `models/zogepel.py`.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any

from atomserve_b200.config.gefilix_config import _need
from atomserve_b200.config.model_config import ModelConfigError

MIXERS = ("mlstm", "parallel")


@dataclass(frozen=True)
class ZogepelConfig:
    vocab: int
    width: int
    layers: tuple[dict[str, Any], ...]
    norm_eps: float
    residual_mult: float
    embedding_scale: float
    token_side_dim: int | None = None  # None: the model has no per-layer token input
    max_positions: int = 1 << 20  # no learned or tabulated positions: no limit of the design's own

    architecture = "Zogepel"

    @classmethod
    def from_dict(cls, raw: dict) -> "ZogepelConfig":
        name = raw.get("architecture") or (raw.get("architectures") or [None])[0]
        if name != cls.architecture:
            raise ModelConfigError(f"expected architecture {cls.architecture!r}, got {name!r}")
        _need(raw, ("vocab", "width", "layers", "norm", "residual_mult", "embedding"), "config.json")
        _need(raw["norm"], ("eps",), "config.json norm")
        _need(raw["embedding"], ("scale",), "config.json embedding")
        side = raw.get("token_side")
        if side is not None:
            _need(side, ("dim",), "config.json token_side")
        config = cls(
            vocab=int(raw["vocab"]),
            width=int(raw["width"]),
            layers=tuple(copy.deepcopy(layer) for layer in raw["layers"]),
            norm_eps=float(raw["norm"]["eps"]),
            residual_mult=float(raw["residual_mult"]),
            embedding_scale=float(raw["embedding"]["scale"]),
            token_side_dim=int(side["dim"]) if side is not None else None,
            max_positions=int(raw.get("max_positions", 1 << 20)),
        )
        config.validate()
        return config

    def validate(self) -> None:
        if self.vocab < 1 or self.width < 1 or not self.layers:
            raise ModelConfigError("vocab, width and the number of layers must be positive")
        if not self.norm_eps >= 0:
            raise ModelConfigError("norm.eps must be >= 0")
        if self.token_side_dim is not None and self.token_side_dim < 1:
            raise ModelConfigError("token_side.dim must be positive")
        for i, layer in enumerate(self.layers):
            where = f"layer {i}"
            _need(layer, ("type", "mixer"), where)
            m = layer["mixer"]
            if layer["type"] == "mlstm":
                _need(m, ("heads", "dim", "vdim", "gate_cap"), where + " mixer")
                if not m["gate_cap"] > 0:
                    raise ModelConfigError(f"{where}: gate_cap must be positive")
            elif layer["type"] == "parallel":
                _need(m, ("left", "right"), where + " mixer")
                left, right = m["left"], m["right"]
                _need(left, ("heads", "kv_heads", "dim", "vdim", "scale", "mask"), where + " mixer left")
                _need(left["mask"], ("size",), where + " mixer left mask")
                if left["heads"] % left["kv_heads"]:
                    raise ModelConfigError(f"{where}: {left['heads']} heads are not a multiple of {left['kv_heads']} kv heads")
                if left["vdim"] != left["dim"]:
                    raise ModelConfigError(f"{where}: the values are the keys, so vdim {left['vdim']} must equal dim {left['dim']}")
                if left["mask"]["size"] < 1:
                    raise ModelConfigError(f"{where}: mask.size must be positive")
                _need(right, ("heads", "dim", "vdim", "decay", "rot"), where + " mixer right")
                _need(right["rot"], ("base", "dims"), where + " mixer right rot")
                if len(right["decay"]) != right["heads"]:
                    raise ModelConfigError(f"{where}: {len(right['decay'])} decays for {right['heads']} heads")
                if right["rot"]["dims"] % 2 or not 0 <= right["rot"]["dims"] <= right["dim"]:
                    raise ModelConfigError(f"{where}: rot.dims {right['rot']['dims']} must be even and at most dim {right['dim']}")
            else:
                raise ModelConfigError(f"{where}: mixer type {layer['type']!r} is not one of {MIXERS}")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            _need(mlp, ("kind", "ff"), where + " mlp")
            if mlp["kind"] != "dense":
                raise ModelConfigError(f"{where}: mlp kind {mlp['kind']!r} is not 'dense'")

    def to_dict(self) -> dict:
        """The config.json this configuration round-trips through."""
        out = {
            "architecture": self.architecture,
            "embedding": {"scale": self.embedding_scale},
            "layers": [copy.deepcopy(layer) for layer in self.layers],
            "norm": {"eps": self.norm_eps},
            "residual_mult": self.residual_mult,
            "vocab": self.vocab,
            "width": self.width,
        }
        if self.token_side_dim is not None:
            out["token_side"] = {"dim": self.token_side_dim}
        return out
