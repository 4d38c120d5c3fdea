"""A plain, slow implementation of the Zalunex design for the tests: one function per mechanism,
whole sequences at a time, torch on the CPU in a working dtype of the caller's choice (float64
for an oracle). It shares no code with the package.

Notation: ``h`` [tokens, width] is a mixer's or feed-forward's input (already normed), ``w`` a
dict of tensors by checkpoint name, ``p`` the prefix of a tensor group (``"l3.mix.left."``).
Linear weights are [out, in] and applied as ``h @ W.T``.
"""
from __future__ import annotations

import math

import torch


def rms(x, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def norm_one_plus(x, weight, eps):
    """RMS norm whose stored weight is the gain's distance from one."""
    return rms(x, eps) * (1.0 + weight)


def sink_window_attention(h, w, p, m, eps):
    """Grouped-query attention without positions in the scores: per-head RMS norm of queries and keys
    (one gain for all heads), a sliding window, a per-head sink in the softmax's denominator, and a
    per-head sigmoid gate on the head's output. One whole sequence."""
    H, G, d, vd, win = m["heads"], m["kv_heads"], m["dim"], m["vdim"], m["mask"]["size"]
    T = h.shape[0]
    q = rms((h @ w[p + "q"].T).reshape(T, H, d), eps) * w[p + "q.norm"]
    k = rms((h @ w[p + "k"].T).reshape(T, G, d), eps) * w[p + "k.norm"]
    v = (h @ w[p + "v"].T).reshape(T, G, vd)
    gate = torch.sigmoid(h @ w[p + "g"].T)                          # [T, H]
    out = torch.zeros(T, H, vd, dtype=h.dtype)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"]                   # [T, T]: query i, key j
        i = torch.arange(T)[:, None]
        j = torch.arange(T)[None, :]
        seen = (i - j >= 0) & (i - j < win)
        s = s.masked_fill(~seen, -math.inf)
        sink = w[p + "sink"][head]
        top = torch.maximum(s.max(-1, keepdim=True).values, sink)
        e = torch.exp(s - top)
        denom = e.sum(-1, keepdim=True) + torch.exp(sink - top)     # the sink has no value
        out[:, head] = (e / denom) @ v[:, g]
    out = out * gate[:, :, None]
    return out.reshape(T, H * vd) @ w[p + "o"].T


def lightning_attention(h, w, p, m, eps, state=None):
    """Linear attention with a fixed decay per head: S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t.
    All heads' outputs form one row that is RMS-normed as a whole, then gated and projected. ``state`` [heads, dim, vdim]
    continues an earlier part of the sequence; returns (output, state after the last token)."""
    H, d, vd = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    silu = torch.nn.functional.silu
    q = silu(h @ w[p + "q"].T).reshape(T, H, d)
    k = silu(h @ w[p + "k"].T).reshape(T, H, d)
    v = silu(h @ w[p + "v"].T).reshape(T, H, vd)
    decay = torch.tensor(m["decay"], dtype=h.dtype)
    S = torch.zeros(H, d, vd, dtype=h.dtype) if state is None else state.clone()
    o = torch.zeros(T, H, vd, dtype=h.dtype)
    for t in range(T):
        S = decay[:, None, None] * S + k[t][:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = rms(o.reshape(T, H * vd), eps) * w[p + "norm"]
    o = o * torch.sigmoid(h @ w[p + "g"].T)
    return o @ w[p + "o"].T, S


def pair_mixer(h, w, p, m, eps):
    left = sink_window_attention(h, w, p + "left.", m["left"], eps)
    right, _ = lightning_attention(h, w, p + "right.", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


def clamped_glu(h, w, p, mlp):
    g = torch.clamp(h @ w[p + "gate"].T, max=mlp["limit"])
    u = torch.clamp(h @ w[p + "up"].T, -mlp["limit"], mlp["limit"])
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def gelu_erf(z):
    return 0.5 * z * (1.0 + torch.erf(z / math.sqrt(2.0)))


def route_sigmoid(h, w, p, router):
    """(ids [tokens, top], weights [tokens, top]): the ``top`` largest sigmoid scores, as they are."""
    s = torch.sigmoid(h @ w[p + "router"].to(h.dtype).T)
    weights, ids = torch.topk(s, router["top"], dim=-1)
    return ids, weights


def moe_scaled_input(h, w, p, mlp):
    """Each chosen expert sees the token's row times the expert's weight."""
    ids, weights = route_sigmoid(h, w, p, mlp["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(ids[t].tolist(), weights[t]):
            x = s * h[t]
            out[t] += gelu_erf(x @ w[f"{p}e{e}.up"].T) @ w[f"{p}e{e}.down"].T
    return out


def layer_order(cfg):
    """The layer indices in running order: the stretch [start, stop) of the list is gone through ``times`` times
    before the layers after it follow."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return list(range(n))
    a, b, times = loop["start"], loop["stop"], loop["times"]
    return list(range(a)) + list(range(a, b)) * times + list(range(b, n))


def forward(cfg, w, tokens, dtype=torch.float64, layers_out=None):
    """Logits [tokens, vocab] of one whole sequence. ``layers_out``: a list that receives the residual
    stream after every layer run."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps, mult = cfg["norm"]["eps"], cfg["residual_mult"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    x = w["embed"][tokens] + w["pos"][: len(tokens)]
    for i in layer_order(cfg):
        layer, p = cfg["layers"][i], f"l{i}."
        assert layer["type"] == "parallel"
        y = pair_mixer(norm_one_plus(x, w[p + "norm1"], eps), w, p + "mix.", layer["mixer"], eps)
        x = x + mult * norm_one_plus(y, w[p + "norm1b"], eps)
        mlp = layer.get("mlp")
        if mlp is not None:
            hin = norm_one_plus(x, w[p + "norm2"], eps)
            y = clamped_glu(hin, w, p + "mlp.", mlp) if mlp["kind"] == "dense" else moe_scaled_input(hin, w, p + "mlp.", mlp)
            x = x + mult * norm_one_plus(y, w[p + "norm2b"], eps)
        if layers_out is not None:
            layers_out.append(x.clone())
    x = norm_one_plus(x, w["final.norm"], eps)
    logits = x @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * torch.tanh(logits / cap)
    return logits
