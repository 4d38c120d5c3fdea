"""Small Pafevik configurations and seeded weights for the tests (test-side code only).

The configurations differ from one another in every size: head counts, sizes that are no multiple of
8, ranks, layer order, which layer reads whose cache entry, layers without a feed-forward, router
shapes; "recurrent" has no attention layer and "shared" three attention layers on one cache entry; "ones" sets to 1 what can be 1 (heads, blocks, taps, top, groups) and has no identity
expert. Weights are drawn so that every tensor matters: norm gains around 1, router corrections
large enough to change choices (and negative), decays spread over (0, 1).
"""
from __future__ import annotations

import os

import numpy as np
import torch

import tiny_models as tm


def latent(heads, dim, rot_dim, vdim, q_rank, kv_rank, base=10000.0, kv_from=None, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
         "rot": {"base": base, "dims": rot_dim}, "scale": scale if scale is not None else (dim + rot_dim) ** -0.5}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return {"type": "latent_attention", "mixer": m}


def rglru(width, blocks, conv):
    return {"type": "rglru", "mixer": {"width": width, "blocks": blocks, "conv": conv}}


def moe(ff, experts, top, identity=0, count=1, keep=1, scale=1.0):
    return {"kind": "moe", "expert": {"ff": ff},
            "router": {"experts": experts, "top": top, "identity": identity, "scale": scale,
                       "groups": {"count": count, "keep": keep}}}


def _cfg(vocab, width, layers, logit_scale, eps):
    return {"architecture": "Pafevik", "vocab": vocab, "width": width, "norm": {"eps": eps}, "logit_scale": logit_scale,
            "layers": [dict(l, mlp=m) for l, m in layers]}


CONFIGS = {
    # attention first and last, the last reading the first's cache entry; a layer without feed-forward
    "mixed": _cfg(211, 96, [
        (latent(3, 24, 8, 20, 40, 48), moe(40, 6, 3, identity=2, count=4, keep=2, scale=2.0)),
        (rglru(64, 2, 4), None),
        (rglru(128, 8, 2), moe(24, 5, 2, identity=1, count=3, keep=2, scale=0.7)),
        (latent(3, 24, 8, 20, 40, 48, kv_from=0), moe(40, 6, 3, identity=2, count=4, keep=2, scale=2.0)),
    ], 0.25, 1e-5),
    # sizes that are no multiple of 8 or of a warp; recurrence first; two attention layers of their own
    "odd": _cfg(97, 52, [
        (rglru(42, 3, 3), moe(18, 3, 1, identity=1, count=2, keep=1, scale=1.3)),
        (latent(5, 10, 6, 14, 18, 22, base=500.0), moe(18, 4, 2)),
        (latent(2, 12, 2, 6, 9, 30, base=77.0, scale=0.4), None),
    ], 2.0, 1e-6),
    # whatever can be 1 is 1; no identity expert, one group
    "ones": _cfg(64, 32, [
        (latent(1, 16, 4, 16, 8, 8), moe(16, 2, 1)),
        (rglru(32, 1, 1), moe(16, 1, 1)),
    ], 1.0, 1e-6),
    # no attention at all: no paged cache entry, state only
    "recurrent": _cfg(50, 40, [
        (rglru(48, 4, 2), moe(8, 2, 1, identity=1, count=1, keep=1, scale=1.0)),
        (rglru(24, 2, 5), None),
    ], 1.0, 1e-5),
    # two later layers read the first layer's cache entry, one of them right after it
    "shared": _cfg(80, 48, [
        (latent(2, 8, 4, 12, 16, 24, base=300.0), None),
        (latent(4, 6, 4, 8, 12, 24, base=300.0, kv_from=0), moe(12, 3, 2, identity=0, count=3, keep=2, scale=1.0)),
        (rglru(32, 2, 3), None),
        (latent(1, 20, 4, 24, 8, 24, base=300.0, kv_from=0, scale=0.3), None),
    ], 0.7, 1e-6),
    # 18 heads in two chunks of 16, tensor-core shapes (latent 128, rotated part 32), keys of 64 and values of 40
    "wide": _cfg(300, 192, [
        (latent(18, 32, 32, 40, 72, 128, base=5e5), moe(48, 10, 3, identity=0, count=5, keep=2, scale=1.2)),
        (rglru(192, 6, 4), moe(48, 10, 3, identity=0, count=5, keep=2, scale=1.2)),
    ], 0.8, 1e-5),
}


def tensor_shapes(cfg):
    W = cfg["width"]
    shapes = {"embed": (cfg["vocab"], W), "final.norm": (W,), "head": (cfg["vocab"], W)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = (W,)
        if layer["type"] == "latent_attention":
            H = m["heads"]
            shapes.update({p + "mix.dq": (m["q_rank"], W), p + "mix.dq.norm": (m["q_rank"],),
                           p + "mix.uq": (H * (m["dim"] + m["rot_dim"]), m["q_rank"]),
                           p + "mix.uk": (H * m["dim"], m["kv_rank"]), p + "mix.uv": (H * m["vdim"], m["kv_rank"]),
                           p + "mix.g": (H * m["vdim"], W), p + "mix.o": (W, H * m["vdim"])})
            if m.get("kv_from") is None:
                shapes.update({p + "mix.dkv": (m["kv_rank"] + m["rot_dim"], W), p + "mix.dkv.norm": (m["kv_rank"],)})
        else:
            R, B = m["width"], m["blocks"]
            shapes.update({p + "mix.y": (R, W), p + "mix.y.b": (R,), p + "mix.x": (R, W), p + "mix.x.b": (R,),
                           p + "mix.conv": (R, m["conv"]), p + "mix.conv.b": (R,),
                           p + "mix.ra": (B, R // B, R // B), p + "mix.ra.b": (B, R // B),
                           p + "mix.ri": (B, R // B, R // B), p + "mix.ri.b": (B, R // B),
                           p + "mix.lam": (R,), p + "mix.o": (W, R)})
        mlp = layer.get("mlp")
        if mlp is not None:
            shapes[p + "norm2"] = (W,)
            r = mlp["router"]
            n = r["experts"] + r.get("identity", 0)
            shapes.update({p + "mlp.router": (n, W), p + "mlp.correction": (n,)})
            for e in range(r["experts"]):
                shapes.update({f"{p}mlp.e{e}.gate": (mlp["expert"]["ff"], W), f"{p}mlp.e{e}.up": (mlp["expert"]["ff"], W),
                               f"{p}mlp.e{e}.down": (W, mlp["expert"]["ff"])})
    return shapes


def make_weights(cfg, seed):
    """float32 arrays whose values a bfloat16 file holds exactly (so both dtypes see one model)."""
    rng = np.random.Generator(np.random.PCG64(seed))
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        z = rng.standard_normal(shape).astype(np.float32)
        fan_in = shape[-1]
        if name.endswith("norm") or name.endswith("norm1") or name.endswith("norm2"):
            w = 1.0 + 0.2 * z
        elif name.endswith(".correction"):
            w = 0.3 * z - 0.2
        elif name.endswith(".lam"):
            w = 1.5 * z - 1.0
        elif name.endswith(".conv"):
            w = 0.5 * z
        elif name.endswith(".b"):
            w = 0.3 * z
        elif name == "embed":
            w = z
        elif name.endswith(".router"):
            w = 2.0 * z / np.sqrt(fan_in)
        else:
            w = 1.2 * z / np.sqrt(fan_in)
        bits = tm.to_bf16_bits(w.astype(np.float32))
        out[name] = (bits.astype(np.uint32) << 16).view(np.float32).reshape(shape)
    return out


def write_folder(tmp, name, seed=0, bf16=False, cfg=None):
    cfg = cfg or CONFIGS[name]
    folder = os.path.join(str(tmp), f"pafevik_{name}")
    return tm.write_model_folder(folder, cfg, make_weights(cfg, seed), bf16=bf16)


def torch_weights(cfg, seed, dtype=torch.float64):
    return {k: torch.from_numpy(v).to(dtype) for k, v in make_weights(cfg, seed).items()}


def prompts(cfg, lengths, seed=0):
    rng = np.random.Generator(np.random.PCG64(500 + seed))
    return [rng.integers(0, cfg["vocab"], size=n).tolist() for n in lengths]
