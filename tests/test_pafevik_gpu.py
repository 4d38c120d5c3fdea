"""Pafevik on the GPU against the plain implementation (tests/plain_pafevik.py), in float32 and bfloat16.

First every mechanism alone on its kernels (the float32 stream's norm and sum, block-diagonal products,
the latent cache rows and attention, the recurrence, the router, the grouped experts), with inputs made
so that a fault shows: a far key that one query is aligned with, keys on both sides of a page border,
the first tokens, all-negative choice scores. Then whole models of several shapes: each request alone,
a prompt and then single tokens, prompts in portions down to two tokens, batches of unequal requests
on a small cache whose slots and pages are used again, long decoding through replayed graphs, greedy
generation through ``generate``, and the trace runner as a child process.
"""
import json
import math
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import pafevik_models as pm
import plain_pafevik as plain

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


def close(got, ref, dtype, what="", f32=2e-5, bf16=3e-2):
    """float32: every row within rounding of float32 sums. bfloat16: the rows' median within a bfloat16
    model's rounding and 85 rows in 100 within twice that: a router's close call moves a row, and through a
    recurrence's state the few rows after it."""
    e = row_errors(got, ref)
    if dtype == "float32":
        assert e.max() < f32, f"{what}: worst row error {e.max():.3g}"
    else:
        assert e.median() < bf16 and (e < 2 * bf16).double().mean() >= 0.85, \
            f"{what}: median row error {e.median():.3g}, worst {e.max():.3g}"


# ------------------------------------------------------------------------------------------------ mechanisms alone
@pytest.mark.parametrize("width", [52, 256, 3000])
def test_stream_norm_and_sum(width):
    k = K()
    g = torch.Generator().manual_seed(width)
    x = torch.randn(7, width, generator=g) * 3
    a = torch.randn(7, width, generator=g)
    gain = 1 + 0.1 * torch.randn(width, generator=g)
    for out in (torch.float32, torch.bfloat16):
        for addend in (None, a, a.bfloat16()):
            res = k.norm_stream(x.cuda(), gain.cuda(), None, 1e-6, "rmsnorm", out, None if addend is None else addend.cuda())
            total = x.double() if addend is None else x.double() + addend.double()
            ref = plain.rms_norm(total, gain.double(), 1e-6)
            y = res if addend is None else res[1]
            assert y.dtype == out
            torch.testing.assert_close(y.double().cpu(), ref, atol=1e-5 if out == torch.float32 else 3e-2, rtol=1e-5 if out == torch.float32 else 1e-2)
            if addend is not None:
                assert res[0].dtype == torch.float32
                torch.testing.assert_close(res[0].cpu(), (x + addend.float()), atol=0, rtol=0)
    torch.testing.assert_close(k.add_stream(x.cuda(), a.bfloat16().cuda()).cpu(), x + a.bfloat16().float(), atol=0, rtol=0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,groups,n,kk", [(1, 3, 20, 24), (70, 5, 14, 10), (130, 1, 80, 80), (9, 18, 64, 32), (300, 4, 40, 24)])
def test_block_linear(dtype, m, groups, n, kk):
    k = K()
    dt = tdtype(dtype)
    g = torch.Generator().manual_seed(m)
    wide = torch.randn(m, groups, kk + 6, generator=g).to(dt)      # rows wider than what is read: strides
    w = (torch.randn(groups, n, kk, generator=g) / math.sqrt(kk)).to(dt)
    bias = torch.randn(groups, n, generator=g)
    gate = torch.randn(m, groups * n + 5, generator=g).to(dt)
    x = wide.cuda()[:, :, 3:3 + kk]
    ref = torch.einsum("tgk,gnk->tgn", wide[:, :, 3:3 + kk].double(), w.double())
    tol = dict(atol=1e-5, rtol=1e-5) if dtype == "float32" else dict(atol=2e-2, rtol=2e-2)
    y = k.block_linear(x, w.cuda(), out_dtype=torch.float32)
    torch.testing.assert_close(y.double().cpu(), ref, atol=1e-5, rtol=1e-5)      # float32 out: only the sums round
    y = k.block_linear(x, w.cuda(), bias.cuda(), act="sigmoid", out_dtype=torch.float32)
    torch.testing.assert_close(y.double().cpu(), torch.sigmoid(ref + bias.double()), atol=1e-5, rtol=1e-5)
    y = k.block_linear(x, w.cuda(), gate=gate.cuda()[:, :groups * n])
    want = ref * torch.sigmoid(gate[:, :groups * n].double()).reshape(m, groups, n)
    assert y.dtype == dt
    torch.testing.assert_close(y.double().cpu(), want, **tol)


def latent_case(dtype, heads, rank, rot, pasts, news, needle=None, base=10000.0, scale=0.2, seed=0):
    """Cache rows from random down-projections in two steps (``pasts``, then ``news`` tokens per sequence), then
    the latent attention of the second step; returns (kernel output, plain output) for the second step's rows.
    needle=(b, key position): the last query of sequence b is aligned with that key's latent, in all heads."""
    from pytorch_transformers_b200.cache.paged import Cache
    from pytorch_transformers_b200.engine.batch import StepContext
    from pytorch_transformers_b200.parts.attention import AttentionTiles
    from pytorch_transformers_b200.parts.base import CacheNeed
    k = K()
    dt = tdtype(dtype)
    g = torch.Generator().manual_seed(seed)
    totals = [p + n for p, n in zip(pasts, news)]
    dkv = [torch.randn(t, rank + rot, generator=g) for t in totals]
    q_abs = [torch.randn(t, heads, rank, generator=g) for t in totals]
    q_rot = [torch.randn(t, heads, 5 + rot, generator=g) for t in totals]       # the rotated part sits at offset 5
    norm_w = 1 + 0.2 * torch.randn(rank, generator=g)
    if needle is not None:
        b, pos = needle
        direction = torch.randn(rank, generator=g)
        dkv[b][pos, :rank] = 3.0 * direction
        q_abs[b][-1] = (40.0 / scale) * (direction / direction.norm() / math.sqrt(rank))[None, :]
        q_rot[b][-1] = 0.0
    cache = Cache([(0, CacheNeed("full", 1, rank + rot, 0, v_head_dim=0), None)], sum((t + 63) // 64 * 64 for t in totals), dt, "cuda")
    assert cache.groups[0].v.numel() == 0
    slots = [cache.open() for _ in totals]
    pool, _, gi = cache.entry_storage(0)
    inv_freq = (1.0 / (base ** (torch.arange(0, rot, 2).float() / rot))).cuda() if rot else None

    def step(ranges, attend):
        live = [i for i, r in enumerate(ranges) if r[1] > r[0]]
        ctx = StepContext(cache, [slots[i] for i in live], [[0] * (ranges[i][1] - ranges[i][0]) for i in live], 1,
                          [[] for _ in live], [AttentionTiles(k)])
        rope = k.rope_table(ctx.dev["tok_pos"], inv_freq) if rot else None
        cat = lambda xs: torch.cat([xs[i][ranges[i][0]:ranges[i][1]] for i in live])
        src = torch.cat([torch.zeros(ctx.n_tokens, 3), cat(dkv)], dim=1).to(dt).cuda()     # rows wider than the latent
        k.latent_store(src[:, 3:], norm_w.cuda(), 1e-6, pool, ctx.batch_c[gi], rope, rank, rot, True)
        out = None
        if attend:
            tiles = ctx.plan(AttentionTiles.plan_key)
            qa, qr = cat(q_abs).cuda().contiguous(), cat(q_rot).to(dt).cuda().contiguous()
            if tiles.facts["mma_tokens"] == 1:
                outs = [k.latent_attention(qa, qr, 5, pool, ctx.batch_c[gi], tiles.dev["mtile_seq"], tiles.dev["mtile_q0"],
                                           tiles.facts["n_mma_tiles"], 1, rope, rank, rot, scale, True, n_splits=s)
                        for s in (1, 2, 5)]
                for o in outs[1:]:      # the splits of the key pages only change the order of float32 sums
                    torch.testing.assert_close(o.float(), outs[0].float(), atol=2e-2 if dtype == "bfloat16" else 1e-5, rtol=1e-2 if dtype == "bfloat16" else 1e-5)
                out = outs[-1]
            else:
                out = k.latent_attention(qa, qr, 5, pool, ctx.batch_c[gi], tiles.dev["tile_seq"], tiles.dev["tile_q0"],
                                         tiles.facts["n_tiles"], k.generic_tile_rows(), rope, rank, rot, scale, True)
        ctx.commit()
        return out, live

    if any(pasts):
        step([(0, p) for p in pasts], False)
    out, live = step([(p, t) for p, t in zip(pasts, totals)], True)
    cache.check()
    refs = []
    for i in live:
        pos = torch.arange(totals[i])
        raw = dkv[i].to(dt).double()
        c = plain.rms_norm(raw[:, :rank], norm_w.double(), 1e-6)
        kr = plain.rotate_interleaved(raw[:, rank:], pos, base, rot) if rot else raw[:, rank:]
        c, kr = c.to(dt).double(), kr.to(dt).double()          # as the cache holds them
        qr = q_rot[i].to(dt).double()[..., 5:]
        qr = plain.rotate_interleaved(qr, pos, base, rot) if rot else qr
        sc = (torch.einsum("thr,sr->hts", q_abs[i].double(), c) + torch.einsum("thr,sr->hts", qr, kr)) * scale
        idx = torch.arange(totals[i])
        sc = sc.masked_fill(~(idx[None, :] <= idx[:, None])[None], float("-inf"))
        refs.append(torch.einsum("hts,sr->thr", torch.softmax(sc, -1), c)[pasts[i]:])
    return out.double().cpu(), torch.cat(refs)


LATENT_TOL = {"float32": dict(atol=2e-5, rtol=1e-4), "bfloat16": dict(atol=3e-2, rtol=2e-2)}


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,rank,rot", [(3, 48, 8), (5, 22, 6), (1, 8, 0), (18, 128, 32), (20, 64, 48), (2, 130, 4)])
def test_latent_attention_prompts_chunks_and_single_tokens(dtype, heads, rank, rot):
    for pasts, news in [((0, 0, 0), (1, 5, 70)), ((63, 64, 65, 0), (1, 1, 1, 1)), ((130, 2), (3, 129)), ((200,), (1,))]:
        got, ref = latent_case(dtype, heads, rank, rot, pasts, news, seed=heads)
        torch.testing.assert_close(got, ref, **LATENT_TOL[dtype])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("past,new,pos", [(900, 1, 3), (900, 1, 0), (449, 1, 63), (449, 1, 64), (100, 350, 1), (0, 300, 127),
                                          (0, 300, 128), (320, 1, 320), (320, 1, 319)])
def test_latent_attention_finds_one_far_key(dtype, past, new, pos):
    """The last query is aligned with one key (far back, at a page's last or first place, the first token, the
    token itself): its output must be that key's latent."""
    got, ref = latent_case(dtype, 4, 32, 8, (past, 17), (new, 2), needle=(0, pos), seed=pos)
    last = new - 1
    torch.testing.assert_close(got[last], ref[last], **LATENT_TOL[dtype])
    # and the plain output of that row is the needle's latent itself: nothing else has weight
    assert row_errors(got[last], ref[last]).max() < (1e-4 if dtype == "float32" else 2e-2)
    off = latent_case(dtype, 4, 32, 8, (past, 17), (new, 2), needle=(0, pos), seed=pos + 1)[0][last]
    assert (off - got[last]).abs().max() > 0.1      # another needle gives another row


def rglru_case(dtype, R, blocks, taps, pasts, news, seed=0, chunk=0):
    """The recurrence's kernels from random branch projections in two steps; (kernel output, plain) for the
    second step, and the state rows of the slots."""
    from pytorch_transformers_b200.cache.paged import Cache
    from pytorch_transformers_b200.engine.batch import StepContext
    from pytorch_transformers_b200.parts.base import StateNeed
    k = K()
    dt = tdtype(dtype)
    g = torch.Generator().manual_seed(seed)
    bw = R // blocks
    totals = [p + n for p, n in zip(pasts, news)]
    proj = [torch.randn(t, 2 * R, generator=g).to(dt) for t in totals]
    by, bx, conv_b = (0.3 * torch.randn(R, generator=g) for _ in range(3))
    conv_w = 0.5 * torch.randn(R, taps, generator=g)
    gates_w = (torch.randn(blocks, 2 * bw, bw, generator=g) / math.sqrt(bw)).to(dt)
    gates_b = 0.3 * torch.randn(blocks, 2 * bw, generator=g)
    lam = 1.5 * torch.randn(R, generator=g) - 1
    cache = Cache([(0, None, StateNeed(3)), (1, None, StateNeed(R * taps))], 64 * len(totals), dt, "cuda",
                  max_slots=len(totals) + 1)   # another entry's state beside it
    cache.open()                                    # slot 0 is somebody else's
    slots = [cache.open() for _ in totals]
    state = cache.entry_state(1)
    state[:] = 7.0                                   # opening a slot zeroes it; a stale value must not survive that
    cache.close(slots.pop())
    slots.append(cache.open())
    for s in slots[:-1]:
        state[s].zero_()

    def step(ranges):
        live = [i for i, r in enumerate(ranges) if r[1] > r[0]]
        ctx = StepContext(cache, [slots[i] for i in live], [[0] * (ranges[i][1] - ranges[i][0]) for i in live], 1, [[] for _ in live])
        p = torch.cat([proj[i][ranges[i][0]:ranges[i][1]] for i in live]).cuda()
        y_act, u = k.rglru_conv(p, by.cuda(), bx.cuda(), conv_w.cuda(), conv_b.cuda(), state, ctx.dev["slots"], ctx.batch_c[0])
        gates = k.block_linear(u.view(-1, blocks, bw), gates_w.cuda(), gates_b.cuda(), act="sigmoid", out_dtype=torch.float32)
        if chunk:       # the chunked scan: chunks side by side, joined in order
            seqs, firsts = ctx.tiles(chunk)
            first_of = [sum((n + chunk - 1) // chunk for n in ctx.new[:b]) for b in range(ctx.n_seqs)]
            ints = lambda v: torch.tensor(v, dtype=torch.int32, device="cuda")
            out = k.rglru_scan_chunks(gates, u, y_act, lam.cuda(), p, bx.cuda(), state, ctx.dev["slots"], ctx.batch_c[0], blocks,
                                      taps, 8.0, ints(seqs), ints(firsts), ints(first_of), len(seqs), chunk)
        else:
            out = k.rglru_scan(gates, u, y_act, lam.cuda(), p, bx.cuda(), state, ctx.dev["slots"], ctx.batch_c[0], blocks, taps, 8.0)
        ctx.commit()
        return out, live

    if any(pasts):
        step([(0, p) for p in pasts])
    out, live = step([(p, t) for p, t in zip(pasts, totals)])
    refs = []
    for i in live:
        p = proj[i].double()
        y = plain.gelu_tanh(p[:, :R] + by.double())
        u = plain.causal_conv(p[:, R:] + bx.double(), conv_w.double(), conv_b.double())
        if dtype == "bfloat16":
            u, y = u.to(dt).double(), y.to(dt).double()      # the branches leave their kernels in the model dtype
        ub = u.reshape(-1, blocks, bw)
        gt = torch.sigmoid(torch.einsum("tbi,boi->tbo", ub, gates_w.double()) + gates_b.double())
        r, inp = gt[..., :bw].reshape(-1, R), gt[..., bw:].reshape(-1, R)
        a = torch.exp(-8.0 * r * torch.nn.functional.softplus(lam.double()))
        S = torch.zeros(R, dtype=torch.float64)
        rows = []
        for t in range(totals[i]):
            S = a[t] * S + torch.sqrt(1 - a[t] ** 2) * inp[t] * u[t]
            rows.append(S * y[t])
        refs.append(torch.stack(rows)[pasts[i]:])
    assert float(state[0].abs().max()) == 7.0           # nobody wrote into the other sequence's rows
    return out.double().cpu(), torch.cat(refs)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("R,blocks,taps", [(64, 2, 4), (42, 3, 3), (32, 1, 1), (320, 4, 8)])
def test_recurrence_in_two_steps_equals_whole(dtype, R, blocks, taps):
    for pasts, news in [((0, 0), (1, 40)), ((1, 2, 3, 7), (1, 1, 1, 1)), ((5, 1), (2, 30)), ((90,), (1,))]:
        got, ref = rglru_case(dtype, R, blocks, taps, pasts, news, seed=R + taps)
        torch.testing.assert_close(got, ref, **({"atol": 2e-5, "rtol": 1e-4} if dtype == "float32" else {"atol": 3e-2, "rtol": 3e-2}))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("chunk", [1, 7, 64])
def test_recurrence_scanned_in_chunks(dtype, chunk):
    """Chunks of 1, of 7 (a ragged last chunk) and of 64 tokens, from an empty state and from a carried one,
    and the state they leave: a third step of single tokens goes on from it."""
    for pasts, news in [((0, 0, 0), (130, 1, 64)), ((5, 70), (129, 3))]:
        got, ref = rglru_case(dtype, 96, 3, 4, pasts, news, seed=chunk, chunk=chunk)
        torch.testing.assert_close(got, ref, **({"atol": 2e-5, "rtol": 1e-4} if dtype == "float32" else {"atol": 3e-2, "rtol": 3e-2}))


def test_recurrence_keeps_a_slow_decay_exact():
    """a close to 1: 1 - a^2 must not be formed from a rounded a^2."""
    k = K()
    from pytorch_transformers_b200.cache.paged import Cache
    from pytorch_transformers_b200.engine.batch import StepContext
    from pytorch_transformers_b200.parts.base import StateNeed
    R, T = 32, 1500      # a decay rounded to float32 and used 1,500 times alike would be off by 4e-5 of the state
    cache = Cache([(0, None, StateNeed(R))], 64, torch.float32, "cuda")
    slot = cache.open()
    ctx = StepContext(cache, [slot], [[0] * T], 1, [[]])
    g = torch.Generator().manual_seed(0)
    u, y = torch.randn(T, R, generator=g), torch.ones(T, R)
    gates = torch.cat([torch.full((T, 1, R), 1e-4), torch.ones(T, 1, R)], dim=2)      # r tiny: log a = -8e-4 * softplus(lam)
    lam = torch.zeros(R)
    proj = torch.zeros(T, 2 * R)
    out = k.rglru_scan(gates.cuda(), u.cuda(), y.cuda(), lam.cuda(), proj.cuda(), torch.zeros(R).cuda(), cache.entry_state(0),
                       ctx.dev["slots"], ctx.batch_c[0], 1, 1, 8.0)
    log_a = torch.tensor(-8.0 * 1e-4 * math.log(2.0), dtype=torch.float64)
    a, S, rows = torch.exp(log_a), torch.zeros(R, dtype=torch.float64), []
    for t in range(T):
        S = a * S + torch.sqrt(-torch.expm1(2 * log_a)) * u[t].double()
        rows.append(S.clone())
    torch.testing.assert_close(out.double().cpu(), torch.stack(rows), atol=2e-6, rtol=2e-6)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("n,identity,count,keep,top", [(8, 2, 4, 2, 3), (6, 0, 3, 1, 2), (1, 0, 1, 1, 1), (20, 4, 2, 1, 3),
                                                      (70, 5, 5, 2, 6), (256, 0, 8, 4, 8)])
def test_router_and_experts(dtype, n, identity, count, keep, top):
    k = K()
    dt = tdtype(dtype)
    width, ff, experts = 40, 24, n - identity
    g = torch.Generator().manual_seed(n)
    w = {"l0.mlp.router": 2.0 * torch.randn(n, width, generator=g) / math.sqrt(width),
         "l0.mlp.correction": 0.3 * torch.randn(n, generator=g) - 2.0}         # every choice score is negative
    for e in range(experts):
        w[f"l0.mlp.e{e}.gate"] = (torch.randn(ff, width, generator=g) / math.sqrt(width)).to(dt).float()
        w[f"l0.mlp.e{e}.up"] = (torch.randn(ff, width, generator=g) / math.sqrt(width)).to(dt).float()
        w[f"l0.mlp.e{e}.down"] = (torch.randn(width, ff, generator=g) / math.sqrt(ff)).to(dt).float()
    w64 = {kk: v.double() for kk, v in w.items()}
    mlp = {"expert": {"ff": ff}, "router": {"experts": experts, "identity": identity, "top": top, "scale": 1.7,
                                            "groups": {"count": count, "keep": keep}}}
    gate_up = torch.stack([torch.cat([w[f"l0.mlp.e{e}.gate"], w[f"l0.mlp.e{e}.up"]]) for e in range(experts)]).to(dt).cuda()
    down = torch.stack([w[f"l0.mlp.e{e}.down"] for e in range(experts)]).to(dt).cuda()
    for tokens in (1, 3, 50, 700):       # few pairs: tiles of 16 rows; many: tiles of 64
        h = torch.randn(tokens, width, generator=g).to(dt)
        base = torch.randn(tokens, width, generator=g)
        ids, weights = k.route(h.cuda(), w["l0.mlp.router"].cuda(), w["l0.mlp.correction"].cuda(), count, keep, top, 1.7)
        chosen, ref_w = plain.route(h.double(), w64, "l0.", mlp["router"])
        order = ids.cpu().long().sort(dim=1)
        ref_order = chosen.sort(dim=1)
        same = (order.values == ref_order.values).all(dim=1)
        assert same.double().mean() >= (1.0 if dtype == "float32" else 0.97), "the router chose other experts"
        torch.testing.assert_close(weights.cpu().double().gather(1, order.indices)[same], ref_w.gather(1, ref_order.indices)[same],
                                   atol=1e-6 if dtype == "float32" else 2e-3, rtol=1e-5 if dtype == "float32" else 2e-2)
        out = k.routed_experts(h.cuda(), ids, weights, gate_up, down, base=base.cuda())
        assert out.dtype == torch.float32
        ref = base.double() + plain.moe(h.double(), w64, "l0.", mlp)
        e = row_errors(out[same.cuda()], ref[same])
        assert e.max() < (2e-5 if dtype == "float32" else 2e-2)
        if dtype == "bfloat16":           # a stream of the model dtype takes the sum in its own dtype
            out16 = k.routed_experts(h.cuda(), ids, weights, gate_up, down, base=base.bfloat16().cuda())
            assert out16.dtype == torch.bfloat16
            wide = k.routed_experts(h.cuda(), ids, weights, gate_up, down, base=base.cuda(), mma_tile_rows=128)
            assert row_errors(wide[same.cuda()], ref[same]).max() < 2e-2      # the tensor-core kernel's tiles of 128 rows


# ------------------------------------------------------------------------------------------------ whole models
class Loaded:
    def __init__(self, tmp, name, dtype):
        import pytorch_transformers_b200 as ptb
        self.cfg = pm.CONFIGS[name]
        self.folder = pm.write_folder(tmp, name, seed=len(name), bf16=(dtype == "bfloat16"))
        self.model = ptb.AutoModelForCausalLM.from_pretrained(self.folder, dtype=dtype)
        self.w = pm.torch_weights(self.cfg, len(name))
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


NAMES = sorted(pm.CONFIGS)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_each_request_alone_and_whole(loaded, name, dtype):
    L = loaded(name, dtype)
    assert L.model.spec.stream_float32 and L.model.use_graphs
    cache = L.model.new_cache(320)
    for ids in pm.prompts(L.cfg, (1, 2, 5, 70, 129, 300), seed=1):
        s = cache.open()
        close(L.model.step(cache, [s], [ids], want="all"), L.plain_logits(ids), dtype, f"{name} {len(ids)} tokens")
        cache.close(s)
    L.model.check_errors()
    cache.check()


@pytest.mark.parametrize("name", ["wide", "shared"])
def test_long_prompts_unfolded_and_folded_agree(loaded, name):
    """Long prompts of a bfloat16 model go through the tcgen05 prompt kernel on unfolded keys and values, also a
    portion that continues cached tokens; with that path switched off the folded kernel gives the same rows."""
    L = loaded(name, "bfloat16")
    k = K()
    ids = pm.prompts(L.cfg, (400,), seed=9)[0]
    ref = L.plain_logits(ids)
    calls, orig = [], k.latent_unfolded_attention

    def spy(*a, **kw):
        calls.append(1)
        return orig(*a, **kw)

    def run():
        cache = L.model.new_cache(448)
        s = cache.open()
        return torch.cat([L.model.step(cache, [s], [ids[:300]], want="all"), L.model.step(cache, [s], [ids[300:]], want="all")])

    layers = [m for m in L.model._mixers if hasattr(m, "_unfold_size")]
    k.latent_unfolded_attention = spy
    try:
        unfolded = run()
        assert len(calls) == 2 * len(layers)
        for m in layers:
            m._unfold_size = lambda: 0
        folded = run()
        assert len(calls) == 2 * len(layers)
    finally:
        k.latent_unfolded_attention = orig
        for m in layers:
            m.__dict__.pop("_unfold_size", None)
    close(unfolded, ref, "bfloat16", f"{name} unfolded")
    close(folded, ref, "bfloat16", f"{name} folded")
    close(unfolded, folded, "bfloat16", f"{name} unfolded against folded")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_prompt_then_single_tokens(loaded, name, dtype):
    L = loaded(name, dtype)
    cache = L.model.new_cache(256)
    for n, head in ((100, 60), (34, 1), (70, 62)):        # the single tokens cross a page's border
        ids = pm.prompts(L.cfg, (n,), seed=n)[0]
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
    ids = pm.prompts(L.cfg, (150,), seed=portion)[0]
    s = cache.open()
    rows = [L.model.step(cache, [s], [ids[i:i + portion]], want="all") for i in range(0, len(ids), portion)]
    close(torch.cat(rows), L.plain_logits(ids), dtype, f"{name} in portions of {portion}")
    cache.close(s)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", NAMES)
def test_batches_of_unequal_requests_on_a_small_cache(loaded, name, dtype):
    """Two batches one after the other on a cache that holds just one of them: slots and pages of the first
    are used again by the second, whose sequences must start from empty state. Shorter requests end earlier."""
    L = loaded(name, dtype)
    cache = L.model.new_cache(64 * 5, max_slots=3)
    for seed, (lengths, heads) in enumerate([((130, 7, 66), (120, 2, 64)), ((3, 90, 65), (1, 64, 33))]):
        reqs = pm.prompts(L.cfg, lengths, seed=10 + seed)
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
    L.model.check_errors()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["mixed", "ones"])
def test_long_decoding(loaded, name, dtype):
    L = loaded(name, dtype)
    cache = L.model.new_cache(64 * 12)
    reqs = pm.prompts(L.cfg, (330, 290), seed=5)
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


@pytest.mark.parametrize("name", NAMES)
def test_greedy_generation_through_generate(loaded, name):
    L = loaded(name, "float32")
    prompts = pm.prompts(L.cfg, (9, 1, 30), seed=3)
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
    prompts = pm.prompts(L.cfg, (5, 40), seed=8)
    out = L.model.generate(prompts, max_new_tokens=20, do_sample=True, top_k=20, temperature=0.8, seed=1, eos_token_id=7)
    assert all(len(o) <= len(p) + 20 for o, p in zip(out, prompts))
    again = L.model.generate(prompts, max_new_tokens=20, do_sample=True, top_k=20, temperature=0.8, seed=1, eos_token_id=7)
    assert out == again


@pytest.mark.parametrize("dtype", DTYPES)
def test_random_model_from_config_and_from_folder_are_one_model(tmp_path, dtype):
    import pytorch_transformers_b200 as ptb
    cfg = ptb.PafevikConfig.from_dict(pm.CONFIGS["odd"])
    folder = ptb.write_random_model(cfg, seed=4, folder=str(tmp_path / "m"), dtype=tdtype(dtype))
    a = ptb.AutoModelForCausalLM.from_pretrained(folder, dtype=dtype)
    b = ptb.AutoModelForCausalLM.from_config(cfg, seed=4, dtype=dtype)
    ids = pm.prompts(pm.CONFIGS["odd"], (20,), seed=0)
    ca, cb = a.new_cache(64), b.new_cache(64)
    la, lb = a.step(ca, [ca.open()], ids, want="all"), b.step(cb, [cb.open()], ids, want="all")
    torch.testing.assert_close(la, lb, atol=0, rtol=0)
    assert torch.isfinite(la).all() and float(la.std()) > 0


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_runner_as_a_child_process(tmp_path, dtype):
    name = "mixed"
    cfg = pm.CONFIGS[name]
    folder = pm.write_folder(tmp_path, name, seed=2, bf16=(dtype == "bfloat16"))
    w = pm.torch_weights(cfg, 2)
    reqs = dict(zip("abc", pm.prompts(cfg, (70, 9, 40), seed=4)))
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
