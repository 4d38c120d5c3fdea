"""The latent-attention mixer: queries and keys/values both go through a low-rank latent, and only the
key/value latent (RMS-normed) and one rotated key part shared by all heads are cached per token.

With ``h`` the mixer's input, H heads, per head ``dim`` plain and ``rot_dim`` rotated query/key
entries, values of size ``vdim``, latent sizes ``q_rank`` and ``kv_rank``:

    c_q = rmsnorm(W_dq h) * w_qn        q = W_uq c_q      laid out per head as [dim plain | rot_dim to rotate]
    [c_raw | kr_raw] = W_dkv h          c = rmsnorm(c_raw) * w_kvn,   kr = rotate(kr_raw, position)
    k_h = W_uk[h] c,  v_h = W_uv[h] c
    score_h(i, j) = (q_plain_h(i) . k_h(j) + rotate(q_rot_h(i)) . kr(j)) * scale,   j <= i
    out = W_o (concat_h softmax(score_h) v_h  *  sigmoid(W_g h))

The cache row of a token is [c | kr] (one row for all heads, no value pool). The kernels use
``q_plain_h . (W_uk[h] c) = (W_uk[h]^T q_plain_h) . c``: the key up-projection is folded into the query,
every head scores against the cached rows themselves, and the softmax-weighted sum of the latents
goes through W_uv[h] afterwards. Long prompts of a bfloat16 model whose per-head sizes fit the tcgen05
prompt kernel (64 or 128) take the unfolded way instead: the cached latents of the step's sequences go
through [W_uk; W_uv] in one library product into per-head keys and values in scratch pools, and that
kernel runs on them. A layer built with ``own_kv=False`` has no W_dkv: its schedule
entry reads the cache entry that another latent-attention layer writes.
"""
from __future__ import annotations

from typing import Dict

import torch

from .attention import AttentionTiles
from .base import BuildContext, CacheNeed, ParamDecl, Part, PartSpec, register_part
from .linear import linear


UNFOLD_MAX_BYTES = 8 << 30      # most scratch (per-head keys and values of every page) that the unfolded prompt path may hold


class LatentContext:
    """For prompts that the unfolded path takes: (sequence, position) of every cached row that the step's
    sequences will hold after it, in the order of the sequences. Steps of few tokens get an empty plan."""
    plan_key = "latent_context"

    def __init__(self, kernels):
        self.kernels = kernels

    def plan(self, ctx):
        from ..engine.batch import StepPlan
        if max(ctx.new) <= self.kernels.TC_TILE_TOKENS // 2:      # the tile lists hold 128 tokens a tile only beyond this
            return StepPlan(arrays={}, facts={"n_ctx": 0})
        seqs, poss = [], []
        for b, (p, n) in enumerate(zip(ctx.past, ctx.new)):
            seqs += [b] * (p + n)
            poss += range(p + n)
        return StepPlan(arrays={"ctx_seq": seqs, "ctx_pos": poss}, facts={"n_ctx": len(seqs)})


@register_part("mixer", "latent_attention")
class LatentAttention(Part):
    graph_safe = True
    fuses_add = True

    def __init__(self, build: BuildContext, spec: PartSpec, hidden: int, heads: int, dim: int, rot_dim: int, vdim: int,
                 q_rank: int, kv_rank: int, scale: float, eps: float, own_kv: bool = True):
        super().__init__(build, spec)
        self.hidden, self.heads, self.dim, self.rot_dim, self.vdim = int(hidden), int(heads), int(dim), int(rot_dim), int(vdim)
        self.q_rank, self.kv_rank, self.scale, self.eps, self.own_kv = int(q_rank), int(kv_rank), float(scale), float(eps), bool(own_kv)
        if min(self.heads, self.dim, self.vdim, self.q_rank, self.kv_rank) <= 0 or self.rot_dim < 0:
            raise ValueError("latent attention needs positive head count, sizes and ranks")
        if self.kv_rank > 512:
            raise ValueError(f"the latent attention kernel keeps a row's sums in registers up to kv_rank 512, got {self.kv_rank}")
        self.position = self.children.get("position")
        self.interleaved = bool(getattr(self.position, "interleaved", False))
        self.p_dq = self.p_dq_norm = self.p_uq = self.p_side = self.p_dkv_norm = self.p_uk_t = self.p_uv = self.p_o = None
        self.p_ukv = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        H = self.heads
        d = {"dq": ParamDecl((self.q_rank, self.hidden)),
             "dq_norm": ParamDecl((self.q_rank,), role="vector", init="one_plus_normal"),
             "uq": ParamDecl((H * (self.dim + self.rot_dim), self.q_rank)),
             "uk": ParamDecl((H * self.dim, self.kv_rank)),
             "uv": ParamDecl((H * self.vdim, self.kv_rank)),
             "g": ParamDecl((H * self.vdim, self.hidden)),
             "o": ParamDecl((self.hidden, H * self.vdim))}
        if self.own_kv:
            d["dkv"] = ParamDecl((self.kv_rank + self.rot_dim, self.hidden))
            d["dkv_norm"] = ParamDecl((self.kv_rank,), role="vector", init="one_plus_normal")
        return d

    def bind(self, tensors: Dict[str, torch.Tensor]) -> None:
        H = self.heads
        self.p_dq, self.p_dq_norm, self.p_uq, self.p_o = tensors["dq"], tensors["dq_norm"], tensors["uq"], tensors["o"]
        # the gate and the key/value down-projection read the same input: one product
        self.p_side = torch.cat([tensors["g"], tensors["dkv"]]) if self.own_kv else tensors["g"]
        self.p_dkv_norm = tensors.get("dkv_norm")
        # W_uk per head, transposed: [H, kv_rank, dim] maps a head's plain query part into latent space
        self.p_uk_t = tensors["uk"].view(H, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.p_uv = tensors["uv"].view(H, self.vdim, self.kv_rank)
        # for prompts through the unfolded path: keys and values of all heads from one product
        self.p_ukv = torch.cat([tensors["uk"], tensors["uv"]]) if self._unfold_size() else None

    def cache_need(self):
        return CacheNeed("full", 1, self.kv_rank + self.rot_dim, 0, v_head_dim=0) if self.own_kv else None

    def state_need(self):
        return None

    def planner(self):
        return [AttentionTiles(self.build.kernels), LatentContext(self.build.kernels)]

    def _unfold_size(self):
        """Per-head size of the tcgen05 prompt kernel that holds this layer's keys and values, or 0."""
        k = self.build.kernels
        if self.build.dtype != torch.bfloat16:
            return 0
        need = max(self.dim + self.rot_dim, self.vdim)
        for hd in (64, 128):
            if need <= hd and k.attention_tc_supports(hd):
                return hd
        return 0

    def _unfold_pools(self, cache, group, hd):
        """Scratch pools for the unfolded keys and values, laid out like the group's pages; kept on the cache.
        Layers of equal sizes share them (a layer rewrites every row that it reads)."""
        pages = cache.groups[group].k.shape[1]
        key = (group, self.heads, hd, self.dim, self.rot_dim, self.vdim)
        pools = cache.__dict__.setdefault("_latent_unfold", {})
        if key not in pools:
            if 2 * pages * self.heads * 64 * hd * 2 > UNFOLD_MAX_BYTES:
                pools[key] = None
            else:
                shape = (pages, self.heads, 64, hd)     # zeroed: what lies beyond a head's entries must stay zero
                pools[key] = (torch.zeros(shape, dtype=torch.bfloat16, device=self.build.device),
                              torch.zeros(shape, dtype=torch.bfloat16, device=self.build.device))
        return pools[key]

    def _splits(self, ctx) -> int:
        """Blocks that share the key pages of a (token, 16 heads) tile in a step of single tokens: up to
        two blocks an SM, each with two pages at least."""
        k = self.build.kernels
        blocks = ctx.n_seqs * ((self.heads + k.LATENT_ROWS - 1) // k.LATENT_ROWS)
        return max(1, min((2 * k.sm_count(self.build.device)) // blocks, ctx.pages_hint // 2, 64))

    def forward(self, x, ctx, entry, add=None):
        k = self.build.kernels
        t, H = x.shape[0], self.heads
        cq = k.norm(linear(k, x, self.p_dq), self.p_dq_norm, None, self.eps, "rmsnorm")
        q = linear(k, cq, self.p_uq).view(t, H, self.dim + self.rot_dim)
        side = linear(k, x, self.p_side)
        gate = side[:, :H * self.vdim]
        pool, _, group = ctx.cache.entry_storage(entry.cache_entry)
        batch = ctx.batch_c[group]
        rope = ctx.rope(self.position)
        if entry.writes_cache:
            if not self.own_kv:
                raise ValueError("a latent attention layer without a key/value projection cannot write a cache entry")
            k.latent_store(side[:, H * self.vdim:], self.p_dkv_norm, self.eps, pool, batch, rope, self.kv_rank,
                           self.rot_dim, self.interleaved)
        tiles = ctx.plan(AttentionTiles.plan_key)
        rows = ctx.plan(LatentContext.plan_key)
        hd = self._unfold_size()
        if hd and rows.facts["n_ctx"] and tiles.facts["mma_tokens"] == k.TC_TILE_TOKENS:
            pools = self._unfold_pools(ctx.cache, group, hd)
            if pools is not None:
                # long prompts in bfloat16: per-head keys and values unfolded from the cached latents, and the
                # tcgen05 prompt kernel on them
                o = k.latent_unfolded_attention(q, pool, pools[0], pools[1], self.p_ukv, gate, batch, rows.dev["ctx_seq"],
                                                rows.dev["ctx_pos"], rows.facts["n_ctx"], tiles.dev["mtile_seq"],
                                                tiles.dev["mtile_q0"], tiles.facts["n_mma_tiles"], rope, self.dim,
                                                self.rot_dim, self.vdim, self.kv_rank, self.scale, self.interleaved)
                return linear(k, o, self.p_o, add=add)
        q_abs = k.block_linear(q[:, :, :self.dim], self.p_uk_t, out_dtype=torch.float32)
        if tiles.facts["mma_tokens"] == 1:     # a step of single tokens: a tile is one token's heads
            o_lat = k.latent_attention(q_abs, q, self.dim, pool, batch, tiles.dev["mtile_seq"], tiles.dev["mtile_q0"],
                                       tiles.facts["n_mma_tiles"], 1, rope, self.kv_rank, self.rot_dim, self.scale,
                                       self.interleaved, n_splits=self._splits(ctx))
        else:
            o_lat = k.latent_attention(q_abs, q, self.dim, pool, batch, tiles.dev["tile_seq"], tiles.dev["tile_q0"],
                                       tiles.facts["n_tiles"], k.generic_tile_rows(), rope, self.kv_rank, self.rot_dim,
                                       self.scale, self.interleaved)
        o = k.block_linear(o_lat, self.p_uv, gate=gate)       # values up, times sigmoid(gate)
        return linear(k, o.view(t, H * self.vdim), self.p_o, add=add)
