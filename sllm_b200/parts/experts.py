"""A mixture of experts as a feed-forward: a sigmoid router that narrows its choice to the best groups of experts, small
two-matrix experts, and optionally one expert every token uses.

    z = W_router x (float32);  s = sigmoid(z);  choice = s + correction
    the experts form ``groups`` equal groups of neighbours; a group's score is the sum of its two largest choice scores;
    only experts of the ``keep`` best groups can be chosen; the ``top`` largest choice scores among them win;
    out = sum over the winners of (s_e * scale) * W_down,e gelu(W_up,e x)   (weights not renormalized)   + shared(x)

All experts' up projections are ONE matrix (expert e's rows at e * ff, the shared expert's after them) and their down
projections one matrix side by side: a token's activation row carries its routing weights (zero for an expert not
chosen), so the second product adds up the weighted experts by itself, in float32, in one order whatever else the batch
holds.  Every expert's product is computed for every token: with E experts of which ``top`` are used that is E/top times
the arithmetic of a sorted, grouped product, and none of its bookkeeping; a decode step reads every expert's matrix
either way once the batch holds a few tokens.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import FEED_FORWARDS, FeedForward, TensorSpec
from .standard import Linear


@FEED_FORWARDS.register("routed_experts")
class RoutedExperts(FeedForward):
    """Parameters: ``hidden_size``, ``experts``, ``top``, ``groups`` and ``keep`` (1 and 1: no narrowing), ``scale``,
    ``expert_ff``, ``shared_ff`` (0: no shared expert).  The activation is the exact (erf) gelu; no biases."""

    def __init__(self, params, **kw):
        super().__init__(params, **kw)
        p = params
        self.hidden = int(p["hidden_size"])
        self.E, self.top = int(p["experts"]), int(p["top"])
        self.groups, self.keep = int(p.get("groups", 1)), int(p.get("keep", 1))
        self.scale = float(p["scale"])
        self.ff, self.shared_ff = int(p["expert_ff"]), int(p.get("shared_ff") or 0)
        if self.E % self.groups or not 1 <= self.keep <= self.groups:
            raise ValueError(f"routed_experts: {self.groups} groups (keep {self.keep}) do not fit {self.E} experts")
        if not 1 <= self.top <= self.keep * (self.E // self.groups):
            raise ValueError(f"routed_experts: top={self.top} experts cannot come from {self.keep} groups of {self.E // self.groups}")

    def tensor_specs(self):
        W = self.hidden
        specs = []
        for e in range(self.E):
            specs += [TensorSpec(f"e{e}.up", (self.ff, W)), TensorSpec(f"e{e}.down", (W, self.ff))]
        specs += [TensorSpec("router", (self.E, W)), TensorSpec("correction", (self.E,), role="bias")]
        if self.shared_ff:
            specs += [TensorSpec("shared.up", (self.shared_ff, W)), TensorSpec("shared.down", (W, self.shared_ff))]
        return specs

    def bind(self, fetch):
        names = [f"e{e}" for e in range(self.E)] + (["shared"] if self.shared_ff else [])
        self.up = Linear(self._matrix(torch.cat([fetch(f"{n}.up") for n in names], dim=0)))          # [E ff + shared, W]
        self.down = Linear(self._matrix(torch.cat([fetch(f"{n}.down") for n in names], dim=1)))      # [W, E ff + shared]
        self.router = Linear(self._matrix(fetch("router")))
        self.correction = self._f32(fetch("correction"))

    accepts_residual = True

    def route(self, x):
        """(dense weights [T, E], indices [T, top], weights [T, top]) of the normed rows ``x``."""
        return ops.moe_route(self.router(x, torch.float32), self.correction, self.groups, self.keep, self.top, self.scale)

    def forward(self, x, step, residual=None):
        dense, _, _ = self.route(x)
        act = ops.moe_act(self.up(x, self.dtype), dense, self.ff, self.dtype)        # [T, E ff + shared]
        return self.down.into(act, residual)

    def weight_bytes(self):
        return self.up.nbytes() + self.down.nbytes() + self.router.nbytes() + 4 * self.E
