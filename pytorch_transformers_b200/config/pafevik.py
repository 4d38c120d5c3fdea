"""Configuration of the Pafevik design: a decoder whose layers are listed one by one, each with a
mixer (latent attention or a gated linear recurrence) and an optional routed feed-forward.

config.json keys: ``architecture`` ("Pafevik"), ``vocab``, ``width``, ``norm.eps``, ``logit_scale`` and
``layers``: a list of ``{"type", "mixer": {...}, "mlp": {...} | null}``. A ``latent_attention`` mixer gives
``heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, rot: {base, dims}`` and optionally ``kv_from`` (the
index of the layer whose cache entry it reads); an ``rglru`` mixer gives ``width, blocks, conv``; an
``mlp`` of kind ``moe`` gives ``expert.ff`` and ``router: {experts, top, identity, scale, groups: {count, keep}}``.
"""
from __future__ import annotations

import dataclasses
from typing import Any, ClassVar, Dict, List, Optional

from .base import ModelConfig, _require

MIXERS = ("latent_attention", "rglru")


def _positive_int(value, what: str) -> int:
    _require(isinstance(value, int) and not isinstance(value, bool) and value > 0, f"{what} must be a positive integer, got {value!r}")
    return value


@dataclasses.dataclass
class PafevikConfig(ModelConfig):
    model_type: ClassVar[str] = "pafevik"

    architecture: str = "Pafevik"
    vocab: int = 0
    width: int = 0
    layers: List[Dict[str, Any]] = dataclasses.field(default_factory=list)
    norm: Dict[str, Any] = dataclasses.field(default_factory=lambda: {"eps": 1e-6})
    logit_scale: float = 1.0
    tie_word_embeddings: bool = False        # the head is a tensor of its own

    def __post_init__(self) -> None:
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        _require(isinstance(self.layers, list) and len(self.layers) > 0, "layers must be a non-empty list")
        _require(isinstance(self.norm, dict) and float(self.norm.get("eps", 0)) > 0, "norm.eps must be positive")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            _require(isinstance(layer, dict) and layer.get("type") in MIXERS,
                     f"{where}.type must be one of {', '.join(MIXERS)}, got {layer.get('type') if isinstance(layer, dict) else layer!r}")
            m = layer.get("mixer")
            _require(isinstance(m, dict), f"{where}.mixer must be an object")
            if layer["type"] == "latent_attention":
                for key in ("heads", "dim", "vdim", "q_rank", "kv_rank"):
                    _positive_int(m.get(key), f"{where}.mixer.{key}")
                rot_dim = m.get("rot_dim")
                _require(isinstance(rot_dim, int) and rot_dim >= 0 and rot_dim % 2 == 0, f"{where}.mixer.rot_dim must be even and >= 0")
                rot = m.get("rot") or {}
                dims = rot.get("dims", rot_dim)
                _require(isinstance(dims, int) and 0 <= dims <= rot_dim and dims % 2 == 0,
                         f"{where}.mixer.rot.dims must be even and at most rot_dim")
                _require(dims == 0 or float(rot.get("base", 0)) > 0, f"{where}.mixer.rot.base must be positive")
                _require(float(m.get("scale", 0)) > 0, f"{where}.mixer.scale must be positive")
                src = m.get("kv_from")
                if src is not None:
                    _require(isinstance(src, int) and 0 <= src < i and self.layers[src].get("type") == "latent_attention"
                             and self.layers[src]["mixer"].get("kv_from") is None,
                             f"{where}.mixer.kv_from must name an earlier latent_attention layer with a projection of its own")
                    s = self.layers[src]["mixer"]
                    _require(s.get("kv_rank") == m["kv_rank"] and s.get("rot_dim") == rot_dim and s.get("rot") == m.get("rot"),
                             f"{where}.mixer: kv_rank, rot_dim and rot must equal those of layer {src}, whose cache entry it reads")
            else:
                _positive_int(m.get("width"), f"{where}.mixer.width")
                _positive_int(m.get("blocks"), f"{where}.mixer.blocks")
                _positive_int(m.get("conv"), f"{where}.mixer.conv")
                _require(m["width"] % m["blocks"] == 0, f"{where}.mixer.width must be a multiple of blocks")
            mlp = layer.get("mlp")
            if mlp is not None:
                _require(isinstance(mlp, dict) and mlp.get("kind", "moe") == "moe", f"{where}.mlp.kind must be 'moe'")
                _positive_int((mlp.get("expert") or {}).get("ff"), f"{where}.mlp.expert.ff")
                r = mlp.get("router")
                _require(isinstance(r, dict), f"{where}.mlp.router must be an object")
                _positive_int(r.get("experts"), f"{where}.mlp.router.experts")
                _positive_int(r.get("top"), f"{where}.mlp.router.top")

    # the names that the rest of the library uses for the two sizes every decoder has
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)
