"""Latent attention: keys and values of every head are up-projections of one small vector per token, and only that
vector is cached.

    q = W_q x  [heads, dim];   c = rmsnorm(W_dkv x) * gain  [rank]  (the latent, cached);
    k_h = W_uk,h c,  v_h = W_uv,h c;   score = (q_h . k_h) * scale;   causal softmax;
    head h's output times sigmoid(W_g x)_h;   W_o on the concatenated heads.

No positions enter.  The score of a query against a key is computed in the latent space: q_h . (W_uk,h c) =
(W_uk,h^T q_h) . c, so each head's query is carried through its key up-projection once per token, the attention
kernels read the cached latents as ONE shared key-and-value head of size ``rank`` (the cache holds each latent
once: `PagedKV(values=False)`), and each head's weighted sum of latents goes through its value up-projection
afterwards.  Nothing per head is ever stored per cached token.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import MIXERS, LayerCache, Mixer, PagedKV, StepContext, TensorSpec
from .standard import Linear


@MIXERS.register("latent_attention")
class LatentAttention(Mixer):
    """Parameters: ``hidden_size``, ``heads``, ``dim`` (query/key size of a head), ``vdim`` (value size), ``kv_rank``,
    ``scale``, ``eps`` (of the latent's norm), ``gate`` (a sigmoid gate per head on the output; default true).
    q, the down-projection and the gate are one matrix; its product stays float32 (the latent's norm is float32)."""

    MAX_RANK = 256      # the attention kernels' largest head

    def __init__(self, params, **kw):
        super().__init__(params, **kw)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["heads"])
        self.dim = int(params["dim"])
        self.vdim = int(params["vdim"])
        self.rank = int(params["kv_rank"])
        self.scale = float(params["scale"])
        self.eps = float(params["eps"])
        self.gate = bool(params.get("gate", True))
        if not 1 <= self.rank <= self.MAX_RANK:
            raise ValueError(f"latent_attention: kv_rank={self.rank} is outside 1..{self.MAX_RANK}, the largest head the "
                             f"attention kernels take")

    def cache_need(self):
        return PagedKV(1, self.rank, None, values=False)

    def tensor_specs(self):
        H, W, r = self.heads, self.hidden, self.rank
        specs = [TensorSpec("q", (H * self.dim, W)), TensorSpec("dkv", (r, W)), TensorSpec("dkv.norm", (r,), role="gain"),
                 TensorSpec("uk", (H * self.dim, r)), TensorSpec("uv", (H * self.vdim, r))]
        if self.gate:
            specs.append(TensorSpec("g", (H, W)))
        specs.append(TensorSpec("o", (W, H * self.vdim)))
        return specs

    def bind(self, fetch):
        H, r = self.heads, self.rank
        names = ("q", "dkv", "g") if self.gate else ("q", "dkv")
        self.inp = Linear(self._matrix(torch.cat([fetch(n) for n in names], dim=0)))
        self.off_c, self.off_g = H * self.dim, H * self.dim + r
        self.c_gain = self._f32(fetch("dkv.norm"))
        # [H, rank, dim]: carries a head's query into the latent space;  [H, vdim, rank]: a head's latent sum out of it
        self.uk_t = self._matrix(fetch("uk").reshape(H, self.dim, r).transpose(1, 2))
        self.uv = self._matrix(fetch("uv").reshape(H, self.vdim, r))
        self.out = Linear(self._matrix(fetch("o")))

    accepts_residual = True

    def forward(self, x, step: StepContext, cache: LayerCache, position, write_cache=True, residual=None):
        g = step.groups[cache.group]
        proj = self.inp(x, torch.float32)                                           # [T, H*dim + rank (+ H)] float32
        if write_cache:
            ops.latent_write(proj, self.off_c, self.rank, self.c_gain, self.eps, g.slot_mapping, cache.k)
        ql = ops.head_linear(proj, 0, self.uk_t, self.dtype)                        # [T, H*rank] queries in the latent space
        al = ops.paged_attention(ql, cache.k, cache.v, step, cache.group, self.heads, 1, self.rank, self.scale, None)
        y = ops.head_linear(al, 0, self.uv, self.dtype, gate=proj if self.gate else None, goff=self.off_g)   # [T, H*vdim]
        return self.out.into(y, residual)

    def weight_bytes(self):
        n = self.inp.nbytes() + self.out.nbytes() + 4 * self.rank
        return n + (self.uk_t.numel() + self.uv.numel()) * self.uk_t.element_size()
