"""Attention with separate query, key and value projections, and what some designs put around the softmax:

* a norm of queries and keys per head (RMS over the head's ``dim`` entries, one gain [dim] for all heads);
* no position in the scores, or a rotation from a ``position`` child (not built here: the scores of this
  mixer carry no position);
* a sliding window: position i sees j with 0 <= i - j < window (0: all earlier positions);
* a sink: one learned logit per head that takes part in the softmax's normalisation only: ``exp(sink)`` is one
  more term of the denominator, used as stored (``scale`` does not touch it), and nothing is read for it;
* an output gate: head h's result times sigmoid(W_g x)_h, one number per head, read from the mixer's input;
* values of a size of their own (``vdim``).

score = (q . k) * scale. Query head h reads K/V head h // (heads / kv_heads). Scores, softmax and the
norms' statistics are float32. The four input projections are one matrix [q | k | v | g] and one product;
``forward_projected`` lets a ``pair`` mixer run that product together with another mixer's.
"""
from __future__ import annotations

from typing import Dict

import torch

from .attention import MAX_HEAD_DIM, AttentionTiles
from .base import BuildContext, CacheNeed, ParamDecl, Part, PartSpec, register_part
from .linear import linear


@register_part("mixer", "sink_attention")
class SinkAttention(Part):
    graph_safe = True

    def __init__(self, build: BuildContext, spec: PartSpec, hidden: int, heads: int, kv_heads: int, dim: int, vdim: int,
                 scale: float, window: int = 0, eps: float = 1e-6, qk_norm: bool = True, sink: bool = True,
                 gate: bool = True):
        super().__init__(build, spec)
        if heads % kv_heads:
            raise ValueError(f"heads ({heads}) must be a multiple of kv_heads ({kv_heads})")
        if not (0 < dim <= MAX_HEAD_DIM and 0 < vdim <= MAX_HEAD_DIM):
            raise ValueError(f"the attention kernels take head sizes from 1 to {MAX_HEAD_DIM}, got {dim} and {vdim}")
        self.hidden, self.heads, self.kv_heads, self.dim, self.vdim = int(hidden), int(heads), int(kv_heads), int(dim), int(vdim)
        self.scale, self.window, self.eps = float(scale), int(window), float(eps)
        self.qk_norm, self.has_sink, self.has_gate = bool(qk_norm), bool(sink), bool(gate)
        self.p_in = self.p_o = self.p_q_norm = self.p_k_norm = self.p_sink = None

    def param_decls(self) -> Dict[str, ParamDecl]:
        H, G, d, vd = self.heads, self.kv_heads, self.dim, self.vdim
        decls = {"q": ParamDecl((H * d, self.hidden)), "k": ParamDecl((G * d, self.hidden)),
                 "v": ParamDecl((G * vd, self.hidden)), "o": ParamDecl((self.hidden, H * vd))}
        if self.qk_norm:
            decls["q_norm"] = ParamDecl((d,), role="vector", init="one_plus_normal", std=0.1)
            decls["k_norm"] = ParamDecl((d,), role="vector", init="one_plus_normal", std=0.1)
        if self.has_sink:
            decls["sink"] = ParamDecl((H,), role="vector", std=1.0)
        if self.has_gate:
            decls["g"] = ParamDecl((H, self.hidden))
        return decls

    def bind(self, t: Dict[str, torch.Tensor]) -> None:
        rows = [t["q"], t["k"], t["v"]] + ([t["g"]] if self.has_gate else [])
        self.p_in = torch.cat(rows).contiguous()
        self.p_o = t["o"]
        self.p_q_norm, self.p_k_norm, self.p_sink = t.get("q_norm"), t.get("k_norm"), t.get("sink")

    # ---- the projected protocol (parts/pair.py)
    def in_rows(self) -> int:
        return (self.heads + self.kv_heads) * self.dim + self.kv_heads * self.vdim + (self.heads if self.has_gate else 0)

    def out_columns(self) -> int:
        return self.heads * self.vdim

    def in_weight(self):
        return self.p_in

    def out_weight(self):
        return self.p_o

    def release_projections(self) -> None:
        self.p_in = self.p_o = None

    def cache_need(self):
        return CacheNeed("window" if self.window > 0 else "full", self.kv_heads, self.dim, self.window, v_head_dim=self.vdim)

    def state_need(self):
        return None

    def planner(self):
        return AttentionTiles(self.build.kernels)

    def forward_projected(self, proj, ctx, entry, out, out_scale: float = 1.0) -> None:
        """``proj`` [tokens, in_rows()] -> the gated heads [tokens, heads * vdim] times ``out_scale`` into ``out``."""
        k = self.build.kernels
        k_pool, v_pool, group = ctx.cache.entry_storage(entry.cache_entry)
        batch = ctx.batch_c[group]
        q = k.qk_norm_store(proj, k_pool, v_pool, batch, self.p_q_norm, self.p_k_norm, self.heads, self.kv_heads, self.dim,
                            self.vdim, self.eps, write_cache=entry.writes_cache)
        gate = proj[:, self.in_rows() - self.heads:] if self.has_gate else None
        tiles = ctx.plan(AttentionTiles.plan_key)
        if (q.dtype == torch.bfloat16 and self.dim == self.vdim and k.attention_mma_supports(self.dim)
                and out.stride(0) % 2 == 0 and out.data_ptr() % 4 == 0):
            # bfloat16 with a head size of the tensor-core kernel: tiles of tokens x heads of a K/V group; a step of
            # single tokens divides each sequence's visible pages among blocks that a second kernel joins
            tokens = tiles.facts["mma_tokens"]
            q_per_kv = self.heads // self.kv_heads
            if tokens == 1:
                hpk = min(q_per_kv, 128)
                warps, splits = (hpk + 15) // 16, self._decode_splits(ctx, hpk)
            else:
                warps, splits = 8, 1
                hpk = max(1, min(q_per_kv, 128 // tokens))
            k.attention_mma(q, k_pool, v_pool, batch, tiles.dev["mtile_seq"], tiles.dev["mtile_q0"], tiles.facts["n_mma_tiles"],
                            None, self.kv_heads, self.scale, self.window, tokens, hpk, warps, splits, sinks=self.p_sink,
                            gate=gate, out_scale=out_scale, out=out, wide_weights=True)
            return
        k.attention_generic(q, k_pool, v_pool, batch, tiles.dev["tile_seq"], tiles.dev["tile_q0"], tiles.facts["n_tiles"],
                            None, self.kv_heads, self.scale, self.window, sinks=self.p_sink, gate=gate, out_scale=out_scale,
                            out=out)

    def _decode_splits(self, ctx, hpk: int) -> int:
        """Blocks per (sequence, K/V head) in a step of single tokens: enough to fill the device, each with two
        pages of visible keys at least."""
        k = self.build.kernels
        q_per_kv = self.heads // self.kv_heads
        blocks = ctx.n_seqs * self.kv_heads * ((q_per_kv + hpk - 1) // hpk)
        pages = ctx.pages_hint
        if self.window > 0:
            pages = min(pages, self.window // k.PAGE + 2)
        return max(1, min((2 * k.sm_count(self.build.device)) // blocks, pages // 2, 64))

    def forward(self, x, ctx, entry):
        k = self.build.kernels
        proj = linear(k, x, self.p_in)
        heads = torch.empty((x.shape[0], self.out_columns()), dtype=x.dtype, device=x.device)
        self.forward_projected(proj, ctx, entry, heads)
        return linear(k, heads, self.p_o)
