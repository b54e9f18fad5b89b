"""A recurrent mixer: the generalized delta rule.

Per head a float32 matrix state S [key channel, value channel] that every token decays per key channel, frees along
its unit key at a per-channel rate, and writes its key-value product into:

    S <- diag(d) S - (a * u) (u^T S) + k v^T        (S on the right is the state before the token),        o = S^T r

with r, k, v = W_r x, W_k x, W_v x; d = exp(-exp(-1/2) * sigmoid(W_w2 tanh(W_w1 x) + w0)) (a low-rank decay);
a = sigmoid(W_a x + b_a); u = k / sqrt(sum(k^2) + 1e-6) per head.  Each head's o over its root mean square, times a
gain over all heads, times sigmoid(W_g x), then W_o.  The state starts at zero and is carried from token to token;
it lives in the request's state slot, so a prompt's portions and single decoded tokens continue one another.
"""

from __future__ import annotations

import torch

from .. import ops
from .base import MIXERS, LayerCache, Mixer, SlotState, StepContext, TensorSpec
from .standard import Linear


@MIXERS.register("general_delta")
class GeneralDelta(Mixer):
    """Parameters: ``hidden_size``, ``heads``, ``dim`` (key and value channels of a head), ``eps`` (of the output's
    unit norm), ``decay_rank`` (None: read from the checkpoint's ``w1``).  r, k, v, g, a and w1 are one matrix, so the
    mixer's input is read once; the product stays float32, as everything that enters the recurrence does."""

    NAMES = ("r", "k", "v", "g", "a", "w1")

    def __init__(self, params, **kw):
        super().__init__(params, **kw)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["heads"])
        self.dim = int(params["dim"])
        self.eps = float(params["eps"])
        self.rank = params.get("decay_rank")
        self.C = self.heads * self.dim
        if not ops.delta_rule_supports(self.dim, self.dim):
            raise ValueError(f"general_delta: a head of {self.dim} channels is outside what the recurrence kernel keeps in registers (1..256)")
        self.inp = self.w2 = self.out = None

    def cache_need(self):
        return SlotState((self.heads, self.dim, self.dim), "delta")

    def tensor_specs(self):
        C, W, R = self.C, self.hidden, self.rank
        default = max(8, min(64, W // 16))
        return [TensorSpec("r", (C, W)), TensorSpec("k", (C, W)), TensorSpec("v", (C, W)), TensorSpec("g", (C, W)),
                TensorSpec("a", (C, W)), TensorSpec("a.b", (C,), role="bias"),
                TensorSpec("w1", (R, W), shape_default=(R or default, W)), TensorSpec("w2", (C, R), shape_default=(C, R or default)),
                TensorSpec("w0", (C,), role="bias"), TensorSpec("norm", (C,), role="gain"), TensorSpec("o", (W, C))]

    def bind(self, fetch):
        w1 = fetch("w1")
        self.rank = int(w1.shape[0])
        if tuple(fetch("w2").shape) != (self.C, self.rank):
            raise ValueError(f"general_delta: w2 {tuple(fetch('w2').shape)} does not fit w1's {self.rank} rows")
        C = self.C
        self.inp = Linear(self._matrix(torch.cat([fetch(n) for n in self.NAMES], dim=0)))
        self.offs = {"r": 0, "k": C, "v": 2 * C, "g": 3 * C, "a": 4 * C, "w1": 5 * C}
        self.a_bias = self._f32(fetch("a.b"))
        self.w2 = Linear(self._matrix(fetch("w2")), self._f32(fetch("w0")))
        self.gain = self._f32(fetch("norm"))
        self.out = Linear(self._matrix(fetch("o")))

    accepts_residual = True

    def forward(self, x, step: StepContext, cache: LayerCache, position, write_cache=True, residual=None):
        o = self.offs
        proj = self.inp(x, torch.float32)                                            # [T, 5C + R] float32
        lora = ops.tanh_cols(proj, o["w1"], self.rank, self.dtype)                   # [T, R]
        decay = self.w2(lora, torch.float32)                                         # [T, C] decay logits, float32
        out = ops.delta_rule(proj, (o["r"], o["k"], o["v"], o["a"]), decay, self.a_bias, cache.states["delta"], step,
                             self.heads, self.dim, self.dim)                         # [T, C] float32
        y = ops.delta_out(out, self.gain, proj, o["g"], self.eps, self.heads, self.dim, self.dtype)
        return self.out.into(y, residual)

    def weight_bytes(self):
        return self.inp.nbytes() + self.w2.nbytes() + self.out.nbytes() + 8 * self.C
