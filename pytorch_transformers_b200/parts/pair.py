"""A mixer made of two: both children read the pair's input ``h`` and the result is ``left_scale * left(h) + right_scale * right(h)``.

Each child is a mixer that can run in two halves around its own projections (the *projected* protocol):

* ``in_weight()``: its input projections stacked into one matrix [rows, hidden];
* ``forward_projected(proj, ctx, entry, out, out_scale)``: from its rows of the projection (a view whose rows
  lie wider apart) to its heads' results times ``out_scale``, written into ``out`` (a view of columns);
* ``out_weight()``: its output projection [hidden, columns of ``out``].

The pair then does one product for all input projections of both children, lets each child work on its
columns, and one product over the concatenated heads with the output matrices side by side: the
weighted sum of the two mixers is that product's own sum over k (the scales go into the heads' values
in float32, before they are rounded for the product). At most one child may keep pages and at most
one a per-sequence state: both use the pair's one cache entry.
"""
from __future__ import annotations

import torch

from .base import BuildContext, Part, PartSpec, register_part
from .linear import linear


@register_part("mixer", "pair")
class MixerPair(Part):
    graph_safe = True

    def __init__(self, build: BuildContext, spec: PartSpec, left_scale: float = 1.0, right_scale: float = 1.0):
        super().__init__(build, spec)
        self.left, self.right = self.children["left"], self.children["right"]
        self.scales = (float(left_scale), float(right_scale))
        for child in (self.left, self.right):
            for method in ("in_weight", "forward_projected", "out_weight", "out_columns"):
                if not hasattr(child, method):
                    raise ValueError(f"mixer {child.spec.kind!r} cannot be one of a pair: it lacks {method}()")
        if self.left.cache_need() is not None and self.right.cache_need() is not None:
            raise ValueError("both mixers of a pair want pages of the one cache entry")
        if self.left.state_need() is not None and self.right.state_need() is not None:
            raise ValueError("both mixers of a pair want the state of the one cache entry")
        self.p_in = self.p_out = None

    def cache_need(self):
        return self.left.cache_need() or self.right.cache_need()

    def state_need(self):
        return self.left.state_need() or self.right.state_need()

    def planner(self):
        out = []
        for child in (self.left, self.right):
            p = child.planner()
            out += list(p) if isinstance(p, (list, tuple)) else ([p] if p is not None else [])
        return out

    def after_bind(self) -> None:
        """Both children's input projections in one matrix, their output projections side by side."""
        rows = [self.left.in_weight(), self.right.in_weight()]
        # the right child's part of the projection starts at a whole 16-byte word (kernels that load 16 bytes at a time)
        self.pad = (-self.left.in_rows()) % 8
        if self.pad:
            rows.insert(1, torch.zeros((self.pad, rows[0].shape[1]), dtype=rows[0].dtype, device=rows[0].device))
        self.p_in = torch.cat(rows).contiguous()
        self.p_out = torch.cat([self.left.out_weight(), self.right.out_weight()], dim=1).contiguous()
        self.left.release_projections()
        self.right.release_projections()

    def forward(self, x, ctx, entry):
        """float32 [tokens, hidden] (the product's sums, unrounded): a float32 norm or sum follows."""
        k = self.build.kernels
        w_in, w_out = self.p_in, self.p_out
        proj = linear(k, x, w_in)
        rows_l = self.left.in_rows()
        cols_l, cols_r = self.left.out_columns(), self.right.out_columns()
        heads = torch.empty((x.shape[0], cols_l + cols_r), dtype=x.dtype, device=x.device)
        self.left.forward_projected(proj[:, :rows_l], ctx, entry, heads[:, :cols_l], self.scales[0])
        self.right.forward_projected(proj[:, rows_l + self.pad:], ctx, entry, heads[:, cols_l:], self.scales[1])
        return linear(k, heads, w_out, wide_out=True)
