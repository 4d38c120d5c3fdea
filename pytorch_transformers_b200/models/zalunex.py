"""Zalunex as an assembly of parts: ZalunexConfig -> ModelSpec, with the checkpoint's tensor names.

Every layer is a ``sandwich`` block (an RMS norm before and after each sublayer, weights stored as the
gain's distance from one, a fixed multiplier on what a sublayer adds) around a ``pair`` mixer, a
``sink_attention`` beside a ``linear_attention``, and a ``clamped_glu`` feed-forward or ``routed_experts``
with sigmoid scores, plain erf-GELU experts and the weight on the expert's input. Learned position vectors
are added to the embeddings; the residual stream is float32; the logits are soft-capped. A stretch of layers
that runs several times appears several times in the schedule, each run with a cache entry of its own.
Tensor names: ``embed``, ``pos``, ``l<i>.norm1|norm1b|norm2|norm2b``, ``l<i>.mix.left.*``, ``l<i>.mix.right.*``,
``l<i>.mlp.*``, ``final.norm``, ``head``.
"""
from __future__ import annotations

from ..config.zalunex import ZalunexConfig
from ..parts.base import ModelSpec, PartSpec, ScheduleEntry

GLU_ALPHA = 1.702     # g * sigmoid(1.702 g): fixed by the design


def _norm(cfg: ZalunexConfig, name: str) -> PartSpec:
    return PartSpec("norm", "rmsnorm", {"size": cfg.width, "eps": float(cfg.norm["eps"]), "one_plus": True},
                    names={"weight": name})


def _mixer(cfg: ZalunexConfig, i: int) -> PartSpec:
    m, p, eps = cfg.layers[i]["mixer"], f"l{i}.mix.", float(cfg.norm["eps"])
    l, r = m["left"], m["right"]
    left = PartSpec("mixer", "sink_attention",
                    {"hidden": cfg.width, "heads": l["heads"], "kv_heads": l["kv_heads"], "dim": l["dim"], "vdim": l["vdim"],
                     "scale": float(l["scale"]), "window": int(l["mask"]["size"]), "eps": eps},
                    names={n: f"{p}left.{t}" for n, t in (("q", "q"), ("k", "k"), ("v", "v"), ("g", "g"), ("o", "o"),
                                                          ("q_norm", "q.norm"), ("k_norm", "k.norm"), ("sink", "sink"))})
    right = PartSpec("mixer", "linear_attention",
                     {"hidden": cfg.width, "heads": r["heads"], "dim": r["dim"], "vdim": r["vdim"],
                      "decay": [float(a) for a in r["decay"]], "eps": eps},
                     names={n: f"{p}right.{n}" for n in ("q", "k", "v", "g", "o", "norm")})
    return PartSpec("mixer", "pair", {"left_scale": float(m.get("left_scale", 1.0)), "right_scale": float(m.get("right_scale", 1.0))},
                    children={"left": left, "right": right})


def _feed_forward(cfg: ZalunexConfig, i: int) -> PartSpec:
    mlp, p = cfg.layers[i]["mlp"], f"l{i}.mlp."
    if mlp["kind"] == "dense":
        return PartSpec("feed_forward", "clamped_glu",
                        {"hidden": cfg.width, "inner": mlp["ff"], "limit": float(mlp["limit"]), "alpha": GLU_ALPHA,
                         "wide_out": True}, names={n: p + n for n in ("gate", "up", "down")})
    r = mlp["router"]
    names = {"router": p + "router"}
    for e in range(r["experts"]):
        for t in ("up", "down"):
            names[f"e{e}.{t}"] = f"{p}e{e}.{t}"
    return PartSpec("feed_forward", "routed_experts",
                    {"hidden": cfg.width, "inner": mlp["expert"]["ff"], "experts": r["experts"], "top": r["top"],
                     "score": "sigmoid", "correction": False, "expert": "plain", "activation": "gelu", "weight_on": "input"},
                    names=names)


def zalunex_block(cfg: ZalunexConfig, i: int) -> PartSpec:
    children = {"norm_mixer": _norm(cfg, f"l{i}.norm1"), "post_mixer": _norm(cfg, f"l{i}.norm1b"), "mixer": _mixer(cfg, i)}
    if cfg.layers[i].get("mlp") is not None:
        children["norm_ff"] = _norm(cfg, f"l{i}.norm2")
        children["post_ff"] = _norm(cfg, f"l{i}.norm2b")
        children["feed_forward"] = _feed_forward(cfg, i)
    return PartSpec("block", "sandwich", {"mult": float(cfg.residual_mult)}, children=children)


def zalunex_spec(cfg: ZalunexConfig) -> ModelSpec:
    # every run of a layer has a cache entry (pages and state) of its own
    schedule = [ScheduleEntry(block=i, cache_entry=run) for run, i in enumerate(cfg.layer_runs())]
    return ModelSpec(vocab_size=cfg.vocab, hidden_size=cfg.width, embedding_name="embed",
                     blocks=[zalunex_block(cfg, i) for i in range(len(cfg.layers))],
                     final_norm=_norm(cfg, "final.norm"), head_name="head", schedule=schedule, stream_float32=True,
                     position_table_name="pos", max_positions=cfg.max_positions,
                     logit_softcap=float(cfg.logit_softcap or 0.0))
