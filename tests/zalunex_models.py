"""Small Zalunex configurations and seeded weights for the tests (test-side code only).

The configurations differ from one another in every size: head counts and groupings, key and value sizes
that differ from each other and are no multiple of 8, windows shorter than a page, longer than a page and
longer than any prompt, decays from 0 to 1, layer order, which stretch of layers runs again and how often,
layers without a feed-forward, router shapes. "ones" sets to 1 what can be 1 (heads, window, experts, top,
the loop's times, the residual multiplier). Weights are drawn so that every tensor matters: the layers' norm weights are
near 0 (their gain is 1 + weight), sinks are as large as scores are, plain gains lie around 1.
"""
from __future__ import annotations

import os

import numpy as np
import torch

import tiny_models as tm


def left(heads, kv_heads, dim, vdim, window, scale=None):
    return {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "mask": {"size": window},
            "scale": scale if scale is not None else 2.0 * dim ** -0.5}


def right(heads, dim, vdim, decay):
    assert len(decay) == heads
    return {"heads": heads, "dim": dim, "vdim": vdim, "decay": list(decay)}


def pair(l, r, left_scale=1.0, right_scale=1.0):
    return {"left": l, "right": r, "left_scale": left_scale, "right_scale": right_scale}


def dense(ff, limit):
    return {"kind": "dense", "ff": ff, "limit": limit}


def moe(ff, experts, top):
    return {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}


def _cfg(vocab, width, positions, layers, mult, eps, softcap, loop=None):
    cfg = {"architecture": "Zalunex", "vocab": vocab, "width": width, "max_positions": positions, "norm": {"eps": eps},
           "residual_mult": mult, "logit_softcap": softcap,
           "layers": [{"type": "parallel", "mixer": m, "mlp": f} for m, f in layers]}
    if loop is not None:
        cfg["loop"] = dict(zip(("start", "stop", "times"), loop))
    return cfg


CONFIGS = {
    # grouped heads, values shorter than keys, a window shorter than a page; the last two layers run twice; one without feed-forward
    "mixed": _cfg(211, 96, 700, [
        (pair(left(6, 2, 24, 20, 33), right(3, 16, 24, [0.5, 0.9, 0.999]), 1.3, 0.8), dense(80, 2.0)),
        (pair(left(4, 4, 16, 16, 70), right(2, 24, 8, [1.0, 0.7]), 0.6, 1.4), moe(24, 6, 2)),
        (pair(left(2, 1, 32, 40, 5), right(4, 8, 12, [0.0, 0.3, 0.95, 0.99]), 1.0, 1.0), None),
    ], 0.4, 1e-5, 20.0, loop=(1, 3, 2)),
    # sizes that are no multiple of 8 or of a warp; no loop, no soft cap; three of five experts
    "odd": _cfg(97, 52, 400, [
        (pair(left(5, 5, 10, 14, 7), right(2, 6, 10, [0.8, 0.97]), 0.9, 1.1), moe(18, 5, 3)),
        (pair(left(3, 1, 18, 6, 129), right(3, 10, 6, [0.6, 0.9, 0.999]), 1.5, 0.5), dense(30, 0.7)),
    ], 0.25, 1e-6, None),
    # whatever can be 1 is 1
    "ones": _cfg(64, 32, 400, [
        (pair(left(1, 1, 16, 16, 1), right(1, 8, 8, [0.9])), moe(16, 1, 1)),
        (pair(left(1, 1, 8, 8, 2), right(1, 16, 16, [1.0])), dense(16, 1.0)),
    ], 1.0, 1e-6, 1.0, loop=(0, 1, 1)),
    # windows longer than a page and longer than every prompt; the first layer alone runs three times; tensor-core shapes
    "wide": _cfg(300, 128, 600, [
        (pair(left(8, 2, 64, 64, 130), right(4, 32, 64, [0.9, 0.99, 0.999, 0.97]), 1.1, 0.9), moe(48, 10, 3)),
        (pair(left(4, 1, 64, 64, 1000), right(2, 64, 32, [0.95, 0.999]), 0.7, 1.2), dense(200, 3.0)),
    ], 0.5, 1e-5, 30.0, loop=(0, 1, 3)),
}


def tensor_shapes(cfg):
    W = cfg["width"]
    shapes = {"embed": (cfg["vocab"], W), "pos": (cfg["max_positions"], W), "final.norm": (W,), "head": (cfg["vocab"], W)}
    for i, layer in enumerate(cfg["layers"]):
        p, l, r = f"l{i}.", layer["mixer"]["left"], layer["mixer"]["right"]
        shapes.update({p + "norm1": (W,), p + "norm1b": (W,)})
        shapes.update({p + "mix.left.q": (l["heads"] * l["dim"], W), p + "mix.left.k": (l["kv_heads"] * l["dim"], W),
                       p + "mix.left.v": (l["kv_heads"] * l["vdim"], W), p + "mix.left.q.norm": (l["dim"],),
                       p + "mix.left.k.norm": (l["dim"],), p + "mix.left.sink": (l["heads"],),
                       p + "mix.left.g": (l["heads"], W), p + "mix.left.o": (W, l["heads"] * l["vdim"])})
        shapes.update({p + "mix.right.q": (r["heads"] * r["dim"], W), p + "mix.right.k": (r["heads"] * r["dim"], W),
                       p + "mix.right.v": (r["heads"] * r["vdim"], W), p + "mix.right.g": (r["heads"] * r["vdim"], W),
                       p + "mix.right.o": (W, r["heads"] * r["vdim"]), p + "mix.right.norm": (r["heads"] * r["vdim"],)})
        mlp = layer.get("mlp")
        if mlp is None:
            continue
        shapes.update({p + "norm2": (W,), p + "norm2b": (W,)})
        if mlp["kind"] == "dense":
            shapes.update({p + "mlp.gate": (mlp["ff"], W), p + "mlp.up": (mlp["ff"], W), p + "mlp.down": (W, mlp["ff"])})
        else:
            shapes[p + "mlp.router"] = (mlp["router"]["experts"], W)
            for e in range(mlp["router"]["experts"]):
                shapes.update({f"{p}mlp.e{e}.up": (mlp["expert"]["ff"], W), f"{p}mlp.e{e}.down": (W, mlp["expert"]["ff"])})
    return shapes


def bf16_exact(w):
    """float32 values that a bfloat16 file holds exactly (so both dtypes see one model)."""
    w = np.asarray(w, dtype=np.float32)
    return (tm.to_bf16_bits(w).astype(np.uint32) << 16).view(np.float32).reshape(w.shape)


def make_weights(cfg, seed):
    rng = np.random.Generator(np.random.PCG64(seed))
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        z = rng.standard_normal(shape).astype(np.float32)
        fan_in = shape[-1]
        last = name.split(".")[-1]
        if name.endswith("q.norm") or name.endswith("k.norm") or name.endswith("right.norm"):
            w = 1.0 + 0.2 * z              # plain gains
        elif last in ("norm1", "norm1b", "norm2", "norm2b") or name == "final.norm":
            w = 0.2 * z                    # the gain is one plus this
        elif last == "sink":
            w = 1.5 * z
        elif name == "embed":
            w = z
        elif name == "pos":
            w = 0.5 * z
        elif last == "router":
            w = 2.0 * z / np.sqrt(fan_in)
        else:
            w = 1.2 * z / np.sqrt(fan_in)
        out[name] = bf16_exact(w)
    return out


def write_folder(tmp, name, seed=0, bf16=False, cfg=None):
    cfg = cfg or CONFIGS[name]
    folder = os.path.join(str(tmp), f"zalunex_{name}")
    return tm.write_model_folder(folder, cfg, make_weights(cfg, seed), bf16=bf16)


def torch_weights(cfg, seed, dtype=torch.float64):
    return {k: torch.from_numpy(v).to(dtype) for k, v in make_weights(cfg, seed).items()}


def prompts(cfg, lengths, seed=0):
    rng = np.random.Generator(np.random.PCG64(700 + seed))
    return [rng.integers(0, cfg["vocab"], size=n).tolist() for n in lengths]
