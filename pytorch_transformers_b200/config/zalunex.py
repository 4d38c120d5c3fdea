"""Configuration of the Zalunex design: a decoder with learned positions whose layers are listed one by
one; every layer's mixer is a pair of an attention with window, sink and output gate and a linear attention
with fixed decays, and its feed-forward is a clamped gated unit or a mixture of plain experts; a stretch of
the layers may run several times with the same weights.

config.json keys: ``architecture`` ("Zalunex"), ``vocab``, ``width``, ``max_positions``, ``norm.eps``,
``residual_mult``, ``logit_softcap``, ``loop: {start, stop, times}`` and ``layers``: a list of
``{"type": "parallel", "mixer": {...}, "mlp": {...} | null}``. The mixer gives ``left: {heads, kv_heads, dim,
vdim, scale, mask: {size}}``, ``right: {heads, dim, vdim, decay: [per head]}``, ``left_scale``,
``right_scale``; an ``mlp`` of kind ``dense`` gives ``ff, limit``, one of kind ``moe`` gives ``expert.ff`` and
``router: {experts, top}``.
"""
from __future__ import annotations

import dataclasses
from typing import Any, ClassVar, Dict, List, Optional

from .base import ModelConfig, _require
from .pafevik import _positive_int

MIXERS = ("parallel",)


@dataclasses.dataclass
class ZalunexConfig(ModelConfig):
    model_type: ClassVar[str] = "zalunex"

    architecture: str = "Zalunex"
    vocab: int = 0
    width: int = 0
    max_positions: int = 0
    layers: List[Dict[str, Any]] = dataclasses.field(default_factory=list)
    loop: Optional[Dict[str, Any]] = None
    norm: Dict[str, Any] = dataclasses.field(default_factory=lambda: {"eps": 1e-6})
    residual_mult: float = 1.0
    logit_softcap: Optional[float] = None
    tie_word_embeddings: bool = False        # the head is a tensor of its own

    def __post_init__(self) -> None:
        _positive_int(self.vocab, "vocab")
        _positive_int(self.width, "width")
        _positive_int(self.max_positions, "max_positions")
        _require(isinstance(self.layers, list) and len(self.layers) > 0, "layers must be a non-empty list")
        _require(isinstance(self.norm, dict) and float(self.norm.get("eps", 0)) > 0, "norm.eps must be positive")
        _require(self.logit_softcap is None or float(self.logit_softcap) >= 0, "logit_softcap must not be negative")
        if self.loop is not None:
            _require(isinstance(self.loop, dict), "loop must be an object")
            a, b, times = self.loop.get("start"), self.loop.get("stop"), self.loop.get("times")
            _require(all(isinstance(v, int) and not isinstance(v, bool) for v in (a, b, times))
                     and 0 <= a <= b <= len(self.layers) and times >= 1,
                     f"loop must give 0 <= start <= stop <= {len(self.layers)} and times >= 1, got {self.loop!r}")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            _require(isinstance(layer, dict) and layer.get("type") in MIXERS,
                     f"{where}.type must be one of {', '.join(MIXERS)}, got {layer.get('type') if isinstance(layer, dict) else layer!r}")
            m = layer.get("mixer")
            _require(isinstance(m, dict) and isinstance(m.get("left"), dict) and isinstance(m.get("right"), dict),
                     f"{where}.mixer must be an object with left and right")
            left, right = m["left"], m["right"]
            for key in ("heads", "kv_heads", "dim", "vdim"):
                _positive_int(left.get(key), f"{where}.mixer.left.{key}")
            _require(left["heads"] % left["kv_heads"] == 0, f"{where}.mixer.left.heads must be a multiple of kv_heads")
            _require(float(left.get("scale", 0)) > 0, f"{where}.mixer.left.scale must be positive")
            _require(isinstance(left.get("mask"), dict), f"{where}.mixer.left.mask must be an object")
            _positive_int(left["mask"].get("size"), f"{where}.mixer.left.mask.size")
            for key in ("heads", "dim", "vdim"):
                _positive_int(right.get(key), f"{where}.mixer.right.{key}")
            decay = right.get("decay")
            _require(isinstance(decay, list) and len(decay) == right["heads"] and all(0.0 <= float(a) <= 1.0 for a in decay),
                     f"{where}.mixer.right.decay must list one number in [0, 1] per head")
            mlp = layer.get("mlp")
            if mlp is not None:
                _require(isinstance(mlp, dict) and mlp.get("kind") in ("dense", "moe"), f"{where}.mlp.kind must be 'dense' or 'moe'")
                if mlp["kind"] == "dense":
                    _positive_int(mlp.get("ff"), f"{where}.mlp.ff")
                    _require(float(mlp.get("limit", 0)) > 0, f"{where}.mlp.limit must be positive")
                else:
                    _positive_int((mlp.get("expert") or {}).get("ff"), f"{where}.mlp.expert.ff")
                    r = mlp.get("router")
                    _require(isinstance(r, dict), f"{where}.mlp.router must be an object")
                    _positive_int(r.get("experts"), f"{where}.mlp.router.experts")
                    _positive_int(r.get("top"), f"{where}.mlp.router.top")
                    _require(r["top"] <= r["experts"], f"{where}.mlp.router.top must not exceed experts")

    def layer_runs(self) -> List[int]:
        """The layers' indices in the order they run."""
        n = len(self.layers)
        if not self.loop:
            return list(range(n))
        a, b, times = self.loop["start"], self.loop["stop"], self.loop["times"]
        return list(range(a)) + list(range(a, b)) * times + list(range(b, n))

    # the names that the rest of the library uses for the sizes every decoder has
    @property
    def vocab_size(self) -> int:
        return self.vocab

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @property
    def max_position_embeddings(self) -> int:
        return self.max_positions
