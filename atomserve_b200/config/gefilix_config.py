"""Typed configuration of the Gefilix design, read from its own config.json keys.

A Gefilix model is a list of layers, each naming its mixer ("lightning": linear attention with
a decay per head; "latent_attention": softmax attention over a cached low-rank latent, which a
layer with `kv_from` reads from an earlier layer's cache instead of making its own) and its
feed-forward (dense, routed experts, or none), around a residual stream that is normed after
every sum. Every size and every constant that may differ between models is a key; what the
design fixes (activations, the experts' slope and shift, which of a group's scores count) is
written in `models/gefilix.py`.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any

from atomserve_b200.config.model_config import ModelConfigError

MIXERS = ("lightning", "latent_attention")


def _need(raw: dict, keys: tuple[str, ...], where: str) -> None:
    missing = [k for k in keys if k not in raw]
    if missing:
        raise ModelConfigError(f"{where} lacks required keys: {missing}")


@dataclass(frozen=True)
class GefilixConfig:
    vocab: int
    width: int
    layers: tuple[dict[str, Any], ...]
    norm_eps: float
    postln_alpha: float
    embedding_scale: float
    max_positions: int = 1 << 20  # the design has no learned or tabulated positions: no limit of its own

    architecture = "Gefilix"

    @classmethod
    def from_dict(cls, raw: dict) -> "GefilixConfig":
        name = raw.get("architecture") or (raw.get("architectures") or [None])[0]
        if name != cls.architecture:
            raise ModelConfigError(f"expected architecture {cls.architecture!r}, got {name!r}")
        _need(raw, ("vocab", "width", "layers", "norm", "postln_alpha", "embedding"), "config.json")
        _need(raw["norm"], ("eps",), "config.json norm")
        _need(raw["embedding"], ("scale",), "config.json embedding")
        config = cls(
            vocab=int(raw["vocab"]),
            width=int(raw["width"]),
            layers=tuple(copy.deepcopy(layer) for layer in raw["layers"]),
            norm_eps=float(raw["norm"]["eps"]),
            postln_alpha=float(raw["postln_alpha"]),
            embedding_scale=float(raw["embedding"]["scale"]),
            max_positions=int(raw.get("max_positions", 1 << 20)),
        )
        config.validate()
        return config

    def validate(self) -> None:
        if self.vocab < 1 or self.width < 1 or not self.layers:
            raise ModelConfigError("vocab, width and the number of layers must be positive")
        if not self.norm_eps >= 0:
            raise ModelConfigError("norm.eps must be >= 0")
        for i, layer in enumerate(self.layers):
            where = f"layer {i}"
            _need(layer, ("type", "mixer"), where)
            m = layer["mixer"]
            if layer["type"] == "lightning":
                _need(m, ("heads", "dim", "vdim", "decay"), where + " mixer")
                if len(m["decay"]) != m["heads"]:
                    raise ModelConfigError(f"{where}: {len(m['decay'])} decays for {m['heads']} heads")
            elif layer["type"] == "latent_attention":
                _need(m, ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot"), where + " mixer")
                _need(m["rot"], ("base", "dims"), where + " mixer rot")
                if m["rot"]["dims"] % 2 or m["rot"]["dims"] > m["rot_dim"]:
                    raise ModelConfigError(f"{where}: rot.dims {m['rot']['dims']} must be even and at most rot_dim {m['rot_dim']}")
                src = m.get("kv_from")
                if src is not None:
                    if not 0 <= src < i or self.layers[src]["type"] != "latent_attention" or self.layers[src]["mixer"].get("kv_from") is not None:
                        raise ModelConfigError(f"{where}: kv_from {src} must name an earlier latent_attention layer with a cache of its own")
                    other = self.layers[src]["mixer"]
                    if any(other[k] != m[k] for k in ("kv_rank", "rot_dim", "rot")):
                        raise ModelConfigError(f"{where}: kv_rank, rot_dim and rot must equal those of layer {src}")
            else:
                raise ModelConfigError(f"{where}: mixer type {layer['type']!r} is not one of {MIXERS}")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            _need(mlp, ("kind",), where + " mlp")
            if mlp["kind"] == "dense":
                _need(mlp, ("ff",), where + " mlp")
            elif mlp["kind"] == "moe":
                _need(mlp, ("expert", "router"), where + " mlp")
                _need(mlp["expert"], ("ff", "limit"), where + " mlp expert")
                _need(mlp["router"], ("experts", "top", "scale"), where + " mlp router")
                groups = mlp["router"].get("groups")
                if groups:
                    _need(groups, ("count", "keep"), where + " mlp router groups")
                    if mlp["router"]["experts"] % groups["count"]:
                        raise ModelConfigError(f"{where}: {mlp['router']['experts']} experts do not form {groups['count']} equal groups")
                if mlp.get("shared"):
                    _need(mlp["shared"], ("ff", "limit"), where + " mlp shared")
            else:
                raise ModelConfigError(f"{where}: mlp kind {mlp['kind']!r} is neither 'dense' nor 'moe'")

    def to_dict(self) -> dict:
        """The config.json this configuration round-trips through."""
        return {
            "architecture": self.architecture,
            "embedding": {"scale": self.embedding_scale},
            "layers": [copy.deepcopy(layer) for layer in self.layers],
            "norm": {"eps": self.norm_eps},
            "postln_alpha": self.postln_alpha,
            "vocab": self.vocab,
            "width": self.width,
        }
