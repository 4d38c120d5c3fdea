"""A plain, slow implementation of the Pafevik design for the tests: one function per mechanism,
whole sequences at a time, torch on the CPU in a working dtype of the caller's choice (float64
for an oracle). It shares no code with the package.

Notation: ``h`` [tokens, width] is a mixer's or feed-forward's input (already normed), ``w`` a
dict of tensors by checkpoint name, ``p`` the prefix of a layer's tensors (``"l3."``).
Linear weights are [out, in] and applied as ``h @ W.T``.
"""
from __future__ import annotations

import math

import torch


def rms_norm(x, weight, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def rotate_interleaved(x, positions, base, dims):
    """Pairs (2i, 2i+1) of the last axis' first ``dims`` entries turn by positions * base^(-2i/dims).
    x: [tokens, ..., d]; positions: [tokens]."""
    out = x.clone()
    i = torch.arange(dims // 2, dtype=x.dtype)
    freq = base ** (-2.0 * i / dims)
    ang = positions.to(x.dtype)[:, None] * freq[None, :]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = torch.cos(ang).reshape(shape), torch.sin(ang).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def latent_kv(h, w, p, m, eps, positions):
    """The cached part of a latent-attention layer: (latent c [tokens, kv_rank], rotated shared key
    [tokens, rot_dim])."""
    r = m["kv_rank"]
    dkv = h @ w[p + "mix.dkv"].T
    c = rms_norm(dkv[:, :r], w[p + "mix.dkv.norm"], eps)
    kr = rotate_interleaved(dkv[:, r:], positions, m["rot"]["base"], m["rot"]["dims"])
    return c, kr


def latent_attention(h, w, p, m, eps, positions, shared=None):
    """Latent attention over one whole sequence. ``shared``: (c, kr) of the layer named by kv_from."""
    H, d, rd, vd = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    T = h.shape[0]
    cq = rms_norm(h @ w[p + "mix.dq"].T, w[p + "mix.dq.norm"], eps)
    q = (cq @ w[p + "mix.uq"].T).reshape(T, H, d + rd)
    q_plain, q_rot = q[..., :d], rotate_interleaved(q[..., d:], positions, m["rot"]["base"], m["rot"]["dims"])
    c, kr = shared if shared is not None else latent_kv(h, w, p, m, eps, positions)
    k = (c @ w[p + "mix.uk"].T).reshape(T, H, d)
    v = (c @ w[p + "mix.uv"].T).reshape(T, H, vd)
    scores = (torch.einsum("thd,shd->hts", q_plain, k) + torch.einsum("thr,sr->hts", q_rot, kr)) * m["scale"]
    i = torch.arange(T)
    scores = scores.masked_fill(~(i[None, :] <= i[:, None])[None], float("-inf"))
    o = torch.einsum("hts,shv->thv", torch.softmax(scores, -1), v).reshape(T, H * vd)
    o = o * torch.sigmoid(h @ w[p + "mix.g"].T)
    return o @ w[p + "mix.o"].T, (c, kr)


def causal_conv(x, taps_w, bias):
    """Per-channel causal convolution: out[t, c] = bias[c] + sum_k taps_w[c, k] * x[t - (K-1) + k, c]."""
    T, K = x.shape[0], taps_w.shape[1]
    padded = torch.cat([torch.zeros(K - 1, x.shape[1], dtype=x.dtype), x])
    out = bias[None, :].expand(T, -1).clone()
    for k in range(K):
        out = out + taps_w[:, k][None, :] * padded[k:k + T]
    return out


def rglru(h, w, p, m):
    """The recurrent block over one whole sequence."""
    R, B = m["width"], m["blocks"]
    y = gelu_tanh(h @ w[p + "mix.y"].T + w[p + "mix.y.b"])
    u = causal_conv(h @ w[p + "mix.x"].T + w[p + "mix.x.b"], w[p + "mix.conv"], w[p + "mix.conv.b"])
    T = h.shape[0]
    ub = u.reshape(T, B, R // B)
    r = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + "mix.ra"]) + w[p + "mix.ra.b"]).reshape(T, R)
    i = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, w[p + "mix.ri"]) + w[p + "mix.ri.b"]).reshape(T, R)
    log_a = -8.0 * r * torch.nn.functional.softplus(w[p + "mix.lam"])
    a = torch.exp(log_a)
    drive = torch.sqrt(1.0 - a * a) * i * u
    S = torch.zeros(R, dtype=h.dtype)
    out = torch.empty_like(u)
    for t in range(T):
        S = a[t] * S + drive[t]
        out[t] = S
    return (out * y) @ w[p + "mix.o"].T


def route(h, w, p, router):
    """(chosen [tokens, top] of expert ids, weights [tokens, top])."""
    E, I = router["experts"], router.get("identity", 0)
    n = E + I
    s = torch.softmax(h @ w[p + "mlp.router"].T, -1)
    choice = s + w[p + "mlp.correction"]
    groups = router.get("groups") or {"count": 1, "keep": 1}
    G, keep = groups["count"], groups["keep"]
    per = n // G
    best = choice.reshape(-1, G, per).max(-1).values
    kept = torch.zeros_like(best, dtype=torch.bool)
    kept.scatter_(1, best.topk(keep, dim=-1).indices, True)
    masked = choice.masked_fill(~kept.repeat_interleave(per, dim=1), float("-inf"))
    chosen = masked.topk(router["top"], dim=-1).indices
    return chosen, s.gather(1, chosen) * router["scale"]


def moe(h, w, p, mlp):
    router = mlp["router"]
    E = router["experts"]
    chosen, weights = route(h, w, p, router)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t].tolist(), weights[t]):
            if e >= E:
                out[t] += g * h[t]
            else:
                q = p + f"mlp.e{e}."
                z = h[t] @ w[q + "gate"].T
                out[t] += g * ((z * torch.sigmoid(z) * (h[t] @ w[q + "up"].T)) @ w[q + "down"].T)
    return out


def forward(cfg, w, tokens, dtype=torch.float64, layers_out=None):
    """Logits [tokens, vocab] of one whole sequence; ``layers_out`` collects the residual stream
    after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.as_tensor(tokens)]
    pos = torch.arange(len(tokens))
    kept = {}
    for li, layer in enumerate(cfg["layers"]):
        p = f"l{li}."
        h = rms_norm(x, w[p + "norm1"], eps)
        m = layer["mixer"]
        if layer["type"] == "latent_attention":
            src = m.get("kv_from")
            y, kept[li] = latent_attention(h, w, p, m, eps, pos, kept[src] if src is not None else None)
        elif layer["type"] == "rglru":
            y = rglru(h, w, p, m)
        else:
            raise ValueError(layer["type"])
        x = x + y
        if layer.get("mlp") is not None:
            x = x + moe(rms_norm(x, w[p + "norm2"], eps), w, p, layer["mlp"])
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms_norm(x, w["final.norm"], eps) @ w["head"].T) * cfg["logit_scale"]
