"""Zalunex on the GPU against the plain implementation (tests/plain_zalunex.py), in float32 and bfloat16.

First every mechanism alone: the small kernels (embeddings plus positions, the closing norm with the
stream's sum, the clamped gated unit, the soft cap), then each mixer as a part on a cache of its own
(the attention with window, sink and gate; the decaying sum; the pair of both), the sigmoid router with
plain experts. Inputs are made so that a fault shows: one key that a query is aligned with, placed just
inside and just outside the window, at a page's border, far back; a key far back that only a decay close
to one still carries; a sink that takes nearly all the weight. Then whole models of several shapes: each
request alone, a prompt and then single tokens, prompts in portions down to two tokens, batches of unequal
requests on a small cache whose slots and pages are used again, long decoding through replayed graphs,
greedy generation through ``generate``, and the trace runner as a child process.
"""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_zalunex as plain
import zalunex_models as zm

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
DTYPES = ["float32", "bfloat16"]


def K():
    from pytorch_transformers_b200 import kernels
    return kernels


def tdtype(name):
    return getattr(torch, name)


def row_errors(got, ref):
    got, ref = got.double().cpu().reshape(-1, got.shape[-1]), ref.double().cpu().reshape(-1, ref.shape[-1])
    return (got - ref).norm(dim=1) / ref.norm(dim=1).clamp_min(1e-30)


def close(got, ref, dtype, what="", f32=3e-5, bf16=3e-2):
    """float32: every row within rounding of float32 sums. bfloat16: the rows' median within a bfloat16
    model's rounding and 85 rows in 100 within twice that (a router's close call moves a row, and through the
    decaying sum the rows after it)."""
    e = row_errors(got, ref)
    if dtype == "float32":
        assert e.max() < f32, f"{what}: worst row error {e.max():.3g}"
    else:
        assert e.median() < bf16 and (e < 2 * bf16).double().mean() >= 0.85, \
            f"{what}: median row error {e.median():.3g}, worst {e.max():.3g}"


def rounded(t, dtype):
    """The values a tensor of ``dtype`` holds, as float64."""
    return t.to(tdtype(dtype)).double()


# ------------------------------------------------------------------------------------------------ small kernels
@pytest.mark.parametrize("width", [52, 256, 3000])
@pytest.mark.parametrize("ydtype", DTYPES)
def test_closing_norm_sum_and_next_norm(width, ydtype):
    k = K()
    g = torch.Generator().manual_seed(width)
    x, y = torch.randn(7, width, generator=g) * 3, (torch.randn(7, width, generator=g) * 2).to(tdtype(ydtype))
    g1, g2 = 1 + 0.2 * torch.randn(width, generator=g), 1 + 0.2 * torch.randn(width, generator=g)
    out = k.post_norm_add(x.cuda(), y.cuda(), g1.cuda(), 1e-5, 0.3)
    ref = x.double() + 0.3 * plain.rms(y.double(), 1e-5) * g1.double()
    torch.testing.assert_close(out.double().cpu(), ref, atol=1e-5, rtol=1e-5)
    for nd in DTYPES:
        out2, nxt = k.post_norm_add(x.cuda(), y.cuda(), g1.cuda(), 1e-5, 0.3, gain_next=g2.cuda(), eps_next=1e-3, next_dtype=tdtype(nd))
        torch.testing.assert_close(out2, out, atol=0, rtol=0)
        close(nxt, plain.rms(ref, 1e-3) * g2.double(), nd, "next norm", f32=1e-5, bf16=6e-3)


@pytest.mark.parametrize("dtype", DTYPES)
def test_embeddings_plus_positions_and_soft_cap_and_gated_unit(dtype):
    k = K()
    g = torch.Generator().manual_seed(1)
    table, pos = torch.randn(50, 36, generator=g).to(tdtype(dtype)), torch.randn(20, 36, generator=g).to(tdtype(dtype))
    ids, at = torch.tensor([3, 49, 0, 7], dtype=torch.int32), torch.tensor([0, 19, 5, 5], dtype=torch.int32)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    out = k.embed_sum(ids.cuda(), at.cuda(), table.cuda(), pos.cuda(), status)
    assert out.dtype == torch.float32 and int(status.item()) == 0
    torch.testing.assert_close(out.cpu(), table[ids.long()].float() + pos[at.long()].float(), atol=0, rtol=0)
    k.embed_sum(ids.cuda(), torch.tensor([0, 20, 5, 5], dtype=torch.int32).cuda(), table.cuda(), pos.cuda(), status)
    assert int(status.item()) == 2          # a position beyond the table is reported, not read
    z = torch.randn(5, 70, generator=g) * 40
    torch.testing.assert_close(k.softcap_(z.clone().cuda(), 30.0).cpu(), 30.0 * torch.tanh(z / 30.0), atol=1e-5, rtol=1e-5)
    gu = (torch.randn(9, 2 * 23, generator=g) * 2).to(tdtype(dtype))
    got = k.glu_clamp(gu.cuda(), 1.5, 1.702)
    gg, uu = gu[:, :23].double().clamp(max=1.5), gu[:, 23:].double().clamp(-1.5, 1.5)
    close(got, gg * torch.sigmoid(1.702 * gg) * (uu + 1), dtype, "gated unit", f32=1e-6, bf16=6e-3)
    assert (gu[:, :23] > 1.5).any() and (gu[:, 23:] < -1.5).any() and (gu[:, :23] < -1.5).any()   # both clamps bite; the gate has no floor


# ------------------------------------------------------------------------------------------------ mixers as parts
class Mixer:
    """A mixer part alone on a cache of its own, fed rows directly."""

    def __init__(self, spec, weights, dtype):
        from pytorch_transformers_b200.parts.base import BuildContext, make_part
        self.k, self.dt = K(), tdtype(dtype)
        self.part = make_part(BuildContext(torch.device("cuda"), self.dt, self.k), spec)
        for part in self.part.walk():
            decls = part.param_decls()
            if decls:
                part.bind({n: weights[part.spec.names[n]].to(device="cuda", dtype=torch.float32 if d.role == "vector" else self.dt)
                           for n, d in decls.items()})
        for part in self.part.walk():
            if hasattr(part, "after_bind"):
                part.after_bind()
        planners = self.part.planner()
        self.planners = list(planners) if isinstance(planners, (list, tuple)) else [planners]

    def cache(self, max_tokens, max_slots=None):
        from pytorch_transformers_b200.cache.paged import Cache
        return Cache([(0, self.part.cache_need(), self.part.state_need())], max_tokens, self.dt, "cuda", max_slots=max_slots)

    def step(self, cache, slots, rows):
        """``rows``: per sequence a [n, width] tensor of its next inputs; returns the mixer's output per sequence."""
        from pytorch_transformers_b200.engine.batch import StepContext
        from pytorch_transformers_b200.parts.base import ScheduleEntry
        ctx = StepContext(cache, slots, [[0] * r.shape[0] for r in rows], 1, [[] for _ in rows], self.planners)
        x = torch.cat(rows).to(self.dt).cuda().contiguous()
        y = self.part.forward(x, ctx, ScheduleEntry(0, 0))
        ctx.commit()
        return list(y.double().cpu().split([r.shape[0] for r in rows]))


def left_spec(m, width, eps=1e-5, p="mix.left."):
    from pytorch_transformers_b200.parts.base import PartSpec
    return PartSpec("mixer", "sink_attention",
                    dict(hidden=width, heads=m["heads"], kv_heads=m["kv_heads"], dim=m["dim"], vdim=m["vdim"], scale=m["scale"],
                         window=m["mask"]["size"], eps=eps),
                    names={n: p + t for n, t in (("q", "q"), ("k", "k"), ("v", "v"), ("g", "g"), ("o", "o"), ("q_norm", "q.norm"),
                                                 ("k_norm", "k.norm"), ("sink", "sink"))})


def right_spec(m, width, eps=1e-5, p="mix.right."):
    from pytorch_transformers_b200.parts.base import PartSpec
    return PartSpec("mixer", "linear_attention", dict(hidden=width, heads=m["heads"], dim=m["dim"], vdim=m["vdim"], decay=m["decay"], eps=eps),
                    names={n: p + n for n in ("q", "k", "v", "g", "o", "norm")})


def left_weights(m, width, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    H, G, d, vd = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    r = lambda *s: torch.randn(*s, generator=g)
    w = {"q": r(H * d, width) / width ** 0.5, "k": r(G * d, width) / width ** 0.5, "v": r(G * vd, width) / width ** 0.5,
         "g": r(H, width) / width ** 0.5, "o": r(width, H * vd) / (H * vd) ** 0.5, "q.norm": 1 + 0.2 * r(d), "k.norm": 1 + 0.2 * r(d),
         "sink": 1.5 * r(H)}
    return {"mix.left." + n: rounded(t, dtype) for n, t in w.items()}


def right_weights(m, width, seed, dtype):
    g = torch.Generator().manual_seed(seed)
    H, d, vd = m["heads"], m["dim"], m["vdim"]
    r = lambda *s: torch.randn(*s, generator=g)
    w = {"q": r(H * d, width) / width ** 0.5, "k": r(H * d, width) / width ** 0.5, "v": r(H * vd, width) / width ** 0.5,
         "g": r(H * vd, width) / width ** 0.5, "o": r(width, H * vd) / (H * vd) ** 0.5, "norm": 1 + 0.2 * r(H * vd)}
    return {"mix.right." + n: rounded(t, dtype) for n, t in w.items()}


LEFTS = [zm.left(6, 2, 24, 20, 33), zm.left(5, 5, 10, 14, 7), zm.left(1, 1, 16, 16, 1), zm.left(3, 1, 18, 6, 129),
         zm.left(8, 2, 64, 64, 130), zm.left(2, 2, 128, 128, 64), zm.left(4, 1, 64, 64, 1000), zm.left(2, 1, 40, 72, 65)]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m", LEFTS, ids=lambda m: f"{m['heads']}x{m['kv_heads']}x{m['dim']}x{m['vdim']}w{m['mask']['size']}")
def test_attention_with_window_sink_and_gate(dtype, m):
    """Two sequences: whole prompts, a prompt in portions, then single tokens (past the window and across pages)."""
    width = 48
    w = left_weights(m, width, m["dim"], dtype)
    mix = Mixer(left_spec(m, width), w, dtype)
    g = torch.Generator().manual_seed(7)
    hs = [rounded(torch.randn(n, width, generator=g), dtype) for n in (210, 75)]
    refs = [plain.sink_window_attention(h, w, "mix.left.", m, 1e-5) for h in hs]
    cache = mix.cache(64 * 6)
    slots = [cache.open(), cache.open()]
    got = [[], []]
    for cuts in (((0, 100), (0, 3)), ((100, 163), (3, 70)), ((163, 165), (70, 71))):
        outs = mix.step(cache, slots, [h[a:b] for h, (a, b) in zip(hs, cuts)])
        for i in range(2):
            got[i].append(outs[i])
    for t in range(4):                      # the second sequence ends
        outs = mix.step(cache, slots, [hs[0][165 + t:166 + t], hs[1][71 + t:72 + t]])
        for i in range(2):
            got[i].append(outs[i])
    cache.close(slots[1])
    for t in range(169, 210):
        got[0].append(mix.step(cache, slots[:1], [hs[0][t:t + 1]])[0])
    cache.check()
    for i in range(2):
        close(torch.cat(got[i]), refs[i], dtype, f"sequence {i}", bf16=2e-2)


def needle_case(dtype, window, query_pos, key_pos, past, d=32, vd=24):
    """One head on one K/V head with unit gains, and W_q = W_k P for a permutation P of the input's entries: a query
    whose input is P^T times an earlier token's input has that token's key as its query, score = scale * dim, while
    all other keys (its own too) score far lower. The sequence runs as a prompt of ``past`` tokens and the rest in
    one step (or token by token when the rest is short). Returns (the mixer's rows, the plain rows, the needle's value
    row times the query's gate through W_o)."""
    width = 40
    m = zm.left(1, 1, d, vd, window, scale=48.0 / d)      # an aligned key scores 48, others about 48 / sqrt(d) * N(0, 1)
    w = left_weights(m, width, 11, dtype)
    P = torch.eye(width, dtype=torch.float64)[torch.roll(torch.arange(width), 7)]
    w["mix.left.q"] = w["mix.left.k"] @ P
    w["mix.left.q.norm"] = torch.ones(d, dtype=torch.float64)
    w["mix.left.k.norm"] = torch.ones(d, dtype=torch.float64)
    w["mix.left.sink"] = torch.zeros(1, dtype=torch.float64)
    g = torch.Generator().manual_seed(query_pos * 1000 + key_pos)
    h = rounded(torch.randn(query_pos + 1, width, generator=g), dtype)
    if key_pos != query_pos:
        h[query_pos] = P.T @ h[key_pos]
    ref = plain.sink_window_attention(h, w, "mix.left.", m, 1e-5)
    mix = Mixer(left_spec(m, width), w, dtype)
    cache = mix.cache(64 * ((query_pos + 64) // 64))
    s = cache.open()
    got = []
    if past:
        got.append(mix.step(cache, [s], [h[:past]])[0])
    rest = query_pos + 1 - past
    if rest <= 8:
        for t in range(past, query_pos + 1):
            got.append(mix.step(cache, [s], [h[t:t + 1]])[0])
    else:
        got.append(mix.step(cache, [s], [h[past:]])[0])
    v = h[key_pos:key_pos + 1] @ w["mix.left.v"].T
    gate = torch.sigmoid(h[query_pos:query_pos + 1] @ w["mix.left.g"].T)
    return torch.cat(got), ref, ((v * gate) @ w["mix.left.o"].T)[0]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,vd", [(32, 24), (64, 64)])        # the general kernel; the tensor-core kernel (bfloat16)
@pytest.mark.parametrize("window,query_pos,past", [(33, 200, 0), (33, 200, 150), (33, 200, 200), (64, 191, 0), (64, 192, 192),
                                                   (65, 130, 128), (130, 400, 399), (130, 400, 0), (1, 70, 70), (2, 64, 64),
                                                   (500, 450, 449), (500, 450, 0), (7, 6, 0), (7, 7, 4)])
def test_attention_sees_the_window_and_not_one_key_more(dtype, window, query_pos, past, d, vd):
    """The aligned key sits at the window's last place (distance window - 1: seen) and one further (distance
    window: not seen), or at the first token when the window is longer than the sequence; as part of a prompt
    and as a single token; across page borders."""
    tol = 1e-4 if dtype == "float32" else 3e-2
    inside = max(0, query_pos - (window - 1))
    got, ref, needle = needle_case(dtype, window, query_pos, inside, past, d, vd)
    close(got, ref, dtype, "key at the window's edge", bf16=2e-2)
    if inside < query_pos:          # the needle is not the query itself: the row is the needle's value
        assert row_errors(got[-1:], needle[None]).max() < tol
    outside = query_pos - window
    if outside >= 0:
        got, ref, needle = needle_case(dtype, window, query_pos, outside, past, d, vd)
        close(got, ref, dtype, "key just outside the window", bf16=2e-2)
        assert row_errors(got[-1:], needle[None]).max() > 0.2


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_heavy_sink_takes_the_weight(dtype):
    m = zm.left(3, 1, 16, 16, 50)
    w = left_weights(m, 32, 5, dtype)
    w["mix.left.sink"] = torch.tensor([30.0, -30.0, 0.5], dtype=torch.float64)
    g = torch.Generator().manual_seed(3)
    h = rounded(torch.randn(90, 32, generator=g), dtype)
    mix = Mixer(left_spec(m, 32), w, dtype)
    cache = mix.cache(128)
    s = cache.open()
    got = torch.cat([mix.step(cache, [s], [h[:80]])[0]] + [mix.step(cache, [s], [h[t:t + 1]])[0] for t in range(80, 90)])
    close(got, plain.sink_window_attention(h, w, "mix.left.", m, 1e-5), dtype, "sinks of 30, -30 and 0.5", bf16=2e-2)


RIGHTS = [zm.right(3, 16, 24, [0.5, 0.9, 0.999]), zm.right(2, 6, 10, [1.0, 0.0]), zm.right(1, 8, 8, [0.97]),
          zm.right(4, 32, 64, [0.9, 0.99, 0.999, 0.6]), zm.right(2, 128, 128, [0.999, 0.95]), zm.right(2, 72, 40, [0.98, 0.8]),
          zm.right(2, 64, 128, [1.0, 0.5]), zm.right(3, 128, 64, [0.9, 0.0, 0.999]), zm.right(1, 64, 64, [0.99])]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m", RIGHTS, ids=lambda m: f"{m['heads']}x{m['dim']}x{m['vdim']}")
def test_decaying_sum_whole_in_portions_in_chunks_and_token_by_token(dtype, m):
    """Two sequences: a prompt long enough for the chunked form (a last chunk that is not full), a portion that
    continues it token by token, a portion that continues it in chunks, then single tokens; the other sequence
    short, beside it. A slot that is used again starts from an empty state."""
    width = 48
    w = right_weights(m, width, m["dim"], dtype)
    mix = Mixer(right_spec(m, width), w, dtype)
    g = torch.Generator().manual_seed(9)
    hs = [rounded(torch.randn(n, width, generator=g), dtype) for n in (700, 40)]
    refs = [plain.lightning_attention(h, w, "mix.right.", m, 1e-5)[0] for h in hs]
    cache = mix.cache(64, max_slots=2)      # no pages are needed
    slots = [cache.open(), cache.open()]
    got = [[], []]
    for cuts in (((0, 300), (0, 2)), ((300, 317), (2, 30)), ((317, 690), (30, 31))):
        outs = mix.step(cache, slots, [h[a:b] for h, (a, b) in zip(hs, cuts)])
        for i in range(2):
            got[i].append(outs[i])
    for t in range(9):
        outs = mix.step(cache, slots, [hs[0][690 + t:691 + t], hs[1][31 + t:32 + t]])
        for i in range(2):
            got[i].append(outs[i])
    got[0].append(mix.step(cache, slots[:1], [hs[0][699:]])[0])
    for i in range(2):
        close(torch.cat(got[i]), refs[i], dtype, f"sequence {i}", f32=1e-4, bf16=2e-2)
    cache.close(slots[1])
    again = cache.open()
    assert again == slots[1]
    close(mix.step(cache, [again], [hs[1][:25]])[0], refs[1][:25], dtype, "a slot used again", f32=1e-4, bf16=2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("far,steps", [(0, "prompt"), (3, "tokens"), (63, "prompt"), (64, "tokens")])
def test_decaying_sum_carries_a_far_key_only_where_the_decay_allows(dtype, far, steps):
    """One early token has a key and value 30 times the others'. 600 tokens later the head whose decay is 1 still
    answers with it, the head with decay 0.9 has forgotten it: the rows follow the plain implementation either way,
    and without the early token the first head's row is another one."""
    width, m = 32, zm.right(2, 8, 8, [1.0, 0.9])
    w = right_weights(m, width, 2, dtype)
    g = torch.Generator().manual_seed(far)
    h = rounded(torch.randn(601 + far, width, generator=g), dtype)
    h[far] *= 30.0
    mix = Mixer(right_spec(m, width), w, dtype)

    def run(rows):
        cache = mix.cache(64, max_slots=1)
        s = cache.open()
        if steps == "prompt":
            return torch.cat([mix.step(cache, [s], [rows[:-1]])[0], mix.step(cache, [s], [rows[-1:]])[0]])
        out = [mix.step(cache, [s], [rows[:far + 1]])[0], mix.step(cache, [s], [rows[far + 1:-5]])[0]]
        return torch.cat(out + [mix.step(cache, [s], [rows[t:t + 1]])[0] for t in range(len(rows) - 5, len(rows))])

    got = run(h)
    close(got, plain.lightning_attention(h, w, "mix.right.", m, 1e-5)[0], dtype, "with the far key", f32=1e-4, bf16=2e-2)
    calm = h.clone()
    calm[far] /= 30.0
    assert row_errors(run(calm)[-1:], got[-1:]).max() > 0.05


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name,layer", [("mixed", 0), ("mixed", 2), ("odd", 1), ("ones", 0), ("wide", 0)])
def test_pair_of_mixers_is_the_weighted_sum(dtype, name, layer):
    from pytorch_transformers_b200.parts.base import PartSpec
    cfg = zm.CONFIGS[name]
    m, width = cfg["layers"][layer]["mixer"], cfg["width"]
    w = {**left_weights(m["left"], width, 1, dtype), **right_weights(m["right"], width, 2, dtype)}
    spec = PartSpec("mixer", "pair", dict(left_scale=m["left_scale"], right_scale=m["right_scale"]),
                    children={"left": left_spec(m["left"], width), "right": right_spec(m["right"], width)})
    mix = Mixer(spec, w, dtype)
    assert mix.part.cache_need().window == m["left"]["mask"]["size"] and mix.part.state_need().numel > 0
    g = torch.Generator().manual_seed(4)
    h = rounded(torch.randn(300, width, generator=g), dtype)
    cache = mix.cache(64 * 5)
    s = cache.open()
    got = torch.cat([mix.step(cache, [s], [h[:270]])[0], mix.step(cache, [s], [h[270:298]])[0]] +
                    [mix.step(cache, [s], [h[t:t + 1]])[0] for t in (298, 299)])
    close(got, plain.pair_mixer(h, w, "mix.", m, 1e-5), dtype, "pair", f32=1e-4, bf16=2e-2)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("experts,top,ff,tokens", [(6, 2, 24, 40), (5, 3, 18, 1), (1, 1, 16, 9), (10, 3, 48, 700), (12, 1, 40, 130)])
def test_sigmoid_router_and_plain_experts(dtype, experts, top, ff, tokens):
    from pytorch_transformers_b200.parts.base import BuildContext, PartSpec, make_part
    k, width = K(), 56
    g = torch.Generator().manual_seed(experts)
    w = {"router": rounded(2.0 * torch.randn(experts, width, generator=g) / width ** 0.5, dtype)}
    for e in range(experts):
        w[f"e{e}.up"] = rounded(1.2 * torch.randn(ff, width, generator=g) / width ** 0.5, dtype)
        w[f"e{e}.down"] = rounded(1.2 * torch.randn(width, ff, generator=g) / ff ** 0.5, dtype)
    h = rounded(torch.randn(tokens, width, generator=g), dtype)
    mlp = zm.moe(ff, experts, top)
    ids, weights = k.route(h.to(tdtype(dtype)).cuda(), w["router"].float().cuda(), None, 1, 1, top, 1.0, "sigmoid")
    ref_ids, ref_weights = plain.route_sigmoid(h, w, "", mlp["router"])
    assert (ids.cpu().long() == ref_ids).double().mean() > 0.99           # a close call may fall the other way
    same = (ids.cpu().long() == ref_ids).all(-1)
    torch.testing.assert_close(weights.cpu().double()[same], ref_weights[same], atol=1e-5, rtol=1e-5)
    spec = PartSpec("feed_forward", "routed_experts",
                    dict(hidden=width, inner=ff, experts=experts, top=top, score="sigmoid", correction=False, expert="plain",
                         activation="gelu", weight_on="input"), names={n: n for n in w})
    part = make_part(BuildContext(torch.device("cuda"), tdtype(dtype), k), spec)
    part.bind({n: t.to(device="cuda", dtype=torch.float32 if n == "router" else tdtype(dtype)) for n, t in w.items()})
    got = part.forward(h.to(tdtype(dtype)).cuda(), None)
    assert got.dtype == torch.float32
    ref = plain.moe_scaled_input(h, w, "", mlp)
    close(got[same.cuda()], ref[same], dtype, "experts", f32=2e-5, bf16=2e-2)


# ------------------------------------------------------------------------------------------------ whole models
class Loaded:
    def __init__(self, tmp, name, dtype):
        import pytorch_transformers_b200 as ptb
        self.cfg = zm.CONFIGS[name]
        self.folder = zm.write_folder(tmp, name, seed=len(name), bf16=(dtype == "bfloat16"))
        self.model = ptb.AutoModelForCausalLM.from_pretrained(self.folder, dtype=dtype)
        self.w = zm.torch_weights(self.cfg, len(name))
        self._ref = {}

    def plain_logits(self, ids):
        key = tuple(ids)
        if key not in self._ref:
            self._ref[key] = plain.forward(self.cfg, self.w, ids)
        return self._ref[key]


@pytest.fixture(scope="module")
def loaded(tmp_path_factory):
    made = {}

    def get(name, dtype):
        if (name, dtype) not in made:
            made[(name, dtype)] = Loaded(tmp_path_factory.mktemp(f"{name}_{dtype}"), name, dtype)
        return made[(name, dtype)]
    return get


NAMES = sorted(zm.CONFIGS)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_each_request_alone_and_whole(loaded, name, dtype):
    L = loaded(name, dtype)
    assert L.model.spec.stream_float32 and L.model.use_graphs
    cache = L.model.new_cache(320)
    for ids in zm.prompts(L.cfg, (1, 2, 5, 70, 129, 300), seed=1):
        s = cache.open()
        close(L.model.step(cache, [s], [ids], want="all"), L.plain_logits(ids), dtype, f"{name} {len(ids)} tokens")
        cache.close(s)
    L.model.check_errors()
    cache.check()


def test_residual_stream_after_every_layer_run(loaded):
    """The float32 model's stream after every run of a layer (a layer that runs again counts each time)."""
    L = loaded("mixed", "float32")
    ids = zm.prompts(L.cfg, (50,), seed=2)[0]
    want = []
    plain.forward(L.cfg, L.w, ids, layers_out=want)
    got = []
    blocks = L.model.blocks
    originals = [b.forward for b in blocks]
    try:
        for b, orig in zip(blocks, originals):
            b.forward = (lambda x, ctx, entry, orig=orig: (got.append(orig(x, ctx, entry)), got[-1])[1])     # a tensor, or a stream with the next norm
        cache = L.model.new_cache(64)
        L.model.step(cache, [cache.open()], [ids], want="last")
    finally:
        for b in blocks:
            del b.forward
    assert len(got) == len(want) == 5
    from pytorch_transformers_b200.parts.base import resolve
    assert sum(not torch.is_tensor(a) for a in got) == 4        # every run but the last hands its successor the opening norm
    for i, (a, b) in enumerate(zip(got, want)):
        assert row_errors(resolve(K(), a), b).max() < 1e-5, f"layer run {i}"


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_single_tokens(loaded, name, dtype):
    L = loaded(name, dtype)
    cache = L.model.new_cache(256)
    for n, head in ((100, 60), (34, 1), (200, 62)):        # the single tokens cross a page's border and pass the windows
        ids = zm.prompts(L.cfg, (n,), seed=n)[0]
        ref = L.plain_logits(ids)
        s = cache.open()
        rows = [L.model.step(cache, [s], [ids[:head]], want="all")]
        rows += [L.model.step(cache, [s], [[t]], want="last") for t in ids[head:]]
        close(torch.cat(rows), ref, dtype, f"{name} prompt of {head} then {n - head} single tokens")
        cache.close(s)
    L.model.check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
@pytest.mark.parametrize("portion", [2, 3, 17, 64])
def test_prompts_in_portions(loaded, name, dtype, portion):
    L = loaded(name, dtype)
    cache = L.model.new_cache(192)
    ids = zm.prompts(L.cfg, (150,), seed=portion)[0]
    s = cache.open()
    rows = [L.model.step(cache, [s], [ids[i:i + portion]], want="all") for i in range(0, len(ids), portion)]
    close(torch.cat(rows), L.plain_logits(ids), dtype, f"{name} in portions of {portion}")
    cache.close(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_long_prompt_in_chunks_then_a_long_portion(loaded, name, dtype):
    """Prompts long enough for the chunked decaying sum, the second portion continuing the first one's state."""
    L = loaded(name, dtype)
    cache = L.model.new_cache(64 * 9)
    ids = zm.prompts(L.cfg, (390,), seed=12)[0]        # with the model of 400 positions: nearly all of them
    s = cache.open()
    got = torch.cat([L.model.step(cache, [s], [ids[:290]], want="all"), L.model.step(cache, [s], [ids[290:]], want="all")])
    close(got, L.plain_logits(ids), dtype, f"{name} 290 + 100 tokens")
    with pytest.raises(Exception):                      # beyond the learned positions
        L.model.step(cache, [s], [ids[:L.cfg["max_positions"] - 390 + 1]], want="last")
    cache.close(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_batches_of_unequal_requests_on_a_small_cache(loaded, name, dtype):
    """Two batches one after the other on a cache that holds just one of them: slots and pages of the first
    are used again by the second, whose sequences must start from empty state. Shorter requests end earlier."""
    L = loaded(name, dtype)
    runs = len(plain.layer_order(L.cfg))
    cache = L.model.new_cache(64 * 5, max_slots=3)
    for seed, (lengths, heads) in enumerate([((130, 7, 66), (120, 2, 64)), ((3, 90, 65), (1, 64, 33))]):
        reqs = zm.prompts(L.cfg, lengths, seed=10 + seed)
        refs = [L.plain_logits(r) for r in reqs]
        slots = [cache.open() for _ in reqs]
        assert sorted(slots) == [0, 1, 2]
        out = L.model.step(cache, slots, [r[:h] for r, h in zip(reqs, heads)], want="last")
        live, t, got, want = [0, 1, 2], 0, [], []
        while True:
            for row, i in enumerate(live):
                got.append(out[row])
                want.append(refs[i][heads[i] + t - 1])
            for i in [i for i in live if heads[i] + t >= lengths[i]]:
                cache.close(slots[i])
            live = [i for i in live if heads[i] + t < lengths[i]]
            if not live:
                break
            out = L.model.step(cache, [slots[i] for i in live], [[reqs[i][heads[i] + t]] for i in live], want="last")
            t += 1
        close(torch.stack(got), torch.stack(want), dtype, f"{name} batch {seed}")
        cache.check()
        assert not cache.records
    assert len(cache.state_offsets) == runs         # a state per run of a layer
    L.model.check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "ones", "wide"])
def test_long_decoding(loaded, name, dtype):
    L = loaded(name, dtype)
    cache = L.model.new_cache(64 * 12)
    reqs = zm.prompts(L.cfg, (330, 290), seed=5)
    refs = [L.plain_logits(r) for r in reqs]
    slots = [cache.open(), cache.open()]
    heads = (3, 1)
    out = [L.model.step(cache, slots, [r[:h] for r, h in zip(reqs, heads)], want="last")]
    L.model.record_steps(True)
    for t in range(289):
        out.append(L.model.step(cache, slots, [[reqs[0][3 + t]], [reqs[1][1 + t]]], want="last"))
    kinds = [r["kind"] for r in L.model.step_timings()]
    L.model.record_steps(False)
    assert kinds.count("graph") > 250            # the single-token steps were replayed graphs
    got = torch.stack(out)
    close(got[:, 0], refs[0][2:2 + 290], dtype, f"{name} long decoding, first")
    close(got[:, 1], refs[1][0:290], dtype, f"{name} long decoding, second")
    L.model.check_errors()
    cache.check()


@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_generate(loaded, name):
    L = loaded(name, "float32")
    prompts = zm.prompts(L.cfg, (9, 1, 30), seed=3)
    out = L.model.generate(prompts, max_new_tokens=12, do_sample=False, eos_token_id=None)
    for p, seq in zip(prompts, out):
        assert seq[:len(p)] == p and len(seq) == len(p) + 12
        ids = list(p)
        for tok in seq[len(p):]:
            logits = L.plain_logits(ids)[-1]
            top2 = logits.topk(2).values
            if float(top2[0] - top2[1]) > 1e-4:          # no test on a tie within float32 rounding
                assert int(logits.argmax()) == tok
            ids.append(tok)


def test_generation_with_sampling_and_stop_tokens_runs(loaded):
    L = loaded("mixed", "bfloat16")
    prompts = zm.prompts(L.cfg, (5, 40), seed=8)
    out = L.model.generate(prompts, max_new_tokens=20, do_sample=True, top_k=20, temperature=0.8, seed=1, eos_token_id=7)
    assert all(len(o) <= len(p) + 20 for o, p in zip(out, prompts))
    again = L.model.generate(prompts, max_new_tokens=20, do_sample=True, top_k=20, temperature=0.8, seed=1, eos_token_id=7)
    assert out == again


@pytest.mark.parametrize("dtype", DTYPES)
def test_random_model_from_config_and_from_folder_are_one_model(tmp_path, dtype):
    import pytorch_transformers_b200 as ptb
    cfg = ptb.ZalunexConfig.from_dict(zm.CONFIGS["odd"])
    folder = ptb.write_random_model(cfg, seed=4, folder=str(tmp_path / "m"), dtype=tdtype(dtype))
    a = ptb.AutoModelForCausalLM.from_pretrained(folder, dtype=dtype)
    b = ptb.AutoModelForCausalLM.from_config(cfg, seed=4, dtype=dtype)
    ids = zm.prompts(zm.CONFIGS["odd"], (20,), seed=0)
    ca, cb = a.new_cache(64), b.new_cache(64)
    la, lb = a.step(ca, [ca.open()], ids, want="all"), b.step(cb, [cb.open()], ids, want="all")
    torch.testing.assert_close(la, lb, atol=0, rtol=0)
    assert torch.isfinite(la).all() and float(la.std()) > 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_runner_as_a_child_process(tmp_path, dtype):
    name = "mixed"
    cfg = zm.CONFIGS[name]
    folder = zm.write_folder(tmp_path, name, seed=2, bf16=(dtype == "bfloat16"))
    w = zm.torch_weights(cfg, 2)
    reqs = dict(zip("abc", zm.prompts(cfg, (70, 9, 40), seed=4)))
    refs = {kk: plain.forward(cfg, w, v) for kk, v in reqs.items()}
    heads = {"a": 64, "b": 6, "c": 40}
    steps = [{"step": 0, "entries": [{"id": i, "tokens": reqs[i][:heads[i]], "want": [0, heads[i] - 1]} for i in "abc"], "end": ["c"]}]
    expect = {0: [(i, p) for i in "abc" for p in (0, heads[i] - 1)]}
    for t in range(6):
        live = [i for i in "ab" if heads[i] + t < len(reqs[i])]
        steps.append({"step": t + 1, "entries": [{"id": i, "tokens": [reqs[i][heads[i] + t]], "want": [0]} for i in live],
                      "end": [i for i in live if heads[i] + t + 1 == len(reqs[i])]})
        expect[t + 1] = [(i, heads[i] + t) for i in live]
    out = str(tmp_path / "out")
    proc = subprocess.run([sys.executable, os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out", out,
                           "--max-tokens", "192"], input="\n".join(json.dumps(s) for s in steps) + "\n", capture_output=True,
                          text=True, timeout=900)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert [l for l in proc.stdout.splitlines() if l.startswith("done")] == [f"done {s['step']}" for s in steps]
    got, want = [], []
    for step, rows in expect.items():
        arr = np.fromfile(os.path.join(out, f"{step}.f32"), dtype="<f4").reshape(-1, cfg["vocab"])
        assert arr.shape[0] == len(rows)
        got.append(torch.from_numpy(arr.copy()))
        want += [refs[i][p] for i, p in rows]
    close(torch.cat(got), torch.stack(want), dtype, "trace runner")
