"""Pafevik as an assembly of parts: PafevikConfig -> ModelSpec, with the checkpoint's tensor names.

Every layer is a pre-norm ``sequential`` block of RMS norms around a mixer (``latent_attention`` or
``rglru``) and, unless its ``mlp`` is null, a ``routed_experts`` feed-forward. The residual stream is
float32. Tensor names: ``embed``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.*``, ``l<i>.mlp.*``,
``final.norm``, ``head``. A latent-attention layer with ``kv_from: j`` has no key/value down-projection;
its schedule entry reads the cache entry that layer j writes.
"""
from __future__ import annotations

from ..config.pafevik import PafevikConfig
from ..parts.base import ModelSpec, PartSpec, ScheduleEntry

RGLRU_DECAY = 8.0     # log a = -8 * r * softplus(lam): fixed by the design


def _norm(cfg: PafevikConfig, name: str) -> PartSpec:
    return PartSpec("norm", "rmsnorm", {"size": cfg.width, "eps": float(cfg.norm["eps"])}, names={"weight": name})


def _mixer(cfg: PafevikConfig, i: int) -> PartSpec:
    layer = cfg.layers[i]
    m, p = layer["mixer"], f"l{i}.mix."
    if layer["type"] == "latent_attention":
        own = m.get("kv_from") is None
        rot = m.get("rot") or {}
        dims = int(rot.get("dims", m["rot_dim"]))
        children = {}
        if dims > 0:
            children["position"] = PartSpec("position", "rotary", {"head_dim": m["rot_dim"], "theta": float(rot["base"]),
                                                                   "rotary_dim": dims, "interleaved": True})
        names = {"dq": p + "dq", "dq_norm": p + "dq.norm", "uq": p + "uq", "uk": p + "uk", "uv": p + "uv",
                 "g": p + "g", "o": p + "o"}
        if own:
            names.update({"dkv": p + "dkv", "dkv_norm": p + "dkv.norm"})
        return PartSpec("mixer", "latent_attention",
                        {"hidden": cfg.width, "heads": m["heads"], "dim": m["dim"], "rot_dim": m["rot_dim"],
                         "vdim": m["vdim"], "q_rank": m["q_rank"], "kv_rank": m["kv_rank"], "scale": float(m["scale"]),
                         "eps": float(cfg.norm["eps"]), "own_kv": own}, children=children, names=names)
    names = {"y": p + "y", "y_b": p + "y.b", "x": p + "x", "x_b": p + "x.b", "conv": p + "conv", "conv_b": p + "conv.b",
             "ra": p + "ra", "ra_b": p + "ra.b", "ri": p + "ri", "ri_b": p + "ri.b", "lam": p + "lam", "o": p + "o"}
    return PartSpec("mixer", "rglru", {"hidden": cfg.width, "width": m["width"], "blocks": m["blocks"], "taps": m["conv"],
                                       "decay": RGLRU_DECAY}, names=names)


def _feed_forward(cfg: PafevikConfig, i: int) -> PartSpec:
    mlp, p = cfg.layers[i]["mlp"], f"l{i}.mlp."
    r = mlp["router"]
    groups = r.get("groups") or {}
    names = {"router": p + "router", "correction": p + "correction"}
    for e in range(r["experts"]):
        for t in ("gate", "up", "down"):
            names[f"e{e}.{t}"] = f"{p}e{e}.{t}"
    return PartSpec("feed_forward", "routed_experts",
                    {"hidden": cfg.width, "inner": mlp["expert"]["ff"], "experts": r["experts"], "top": r["top"],
                     "identity": int(r.get("identity", 0)), "groups": int(groups.get("count", 1)),
                     "keep": int(groups.get("keep", groups.get("count", 1))), "scale": float(r.get("scale", 1.0))},
                    names=names)


def pafevik_block(cfg: PafevikConfig, i: int) -> PartSpec:
    children = {"norm_mixer": _norm(cfg, f"l{i}.norm1"), "mixer": _mixer(cfg, i)}
    if cfg.layers[i].get("mlp") is not None:
        children["norm_ff"] = _norm(cfg, f"l{i}.norm2")
        children["feed_forward"] = _feed_forward(cfg, i)
    return PartSpec("block", "sequential", children=children)


def pafevik_spec(cfg: PafevikConfig) -> ModelSpec:
    schedule = []
    for i, layer in enumerate(cfg.layers):
        src = layer["mixer"].get("kv_from") if layer["type"] == "latent_attention" else None
        schedule.append(ScheduleEntry(block=i, cache_entry=i if src is None else int(src), writes_cache=src is None))
    return ModelSpec(vocab_size=cfg.vocab, hidden_size=cfg.width, embedding_name="embed",
                     blocks=[pafevik_block(cfg, i) for i in range(len(cfg.layers))],
                     final_norm=_norm(cfg, "final.norm"), head_name="head", schedule=schedule,
                     logit_scale=float(cfg.logit_scale), stream_float32=True)
