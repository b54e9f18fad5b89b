"""Recurrent mixers of the delta-rule family: the generalized delta rule, and the gated delta rule behind short
convolutions (`GatedDelta`, at the end of the file).

The generalized delta rule:

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


@MIXERS.register("gated_delta")
class GatedDelta(Mixer):
    """The gated delta rule.  Per head a float32 matrix state S [key channel, value channel]:

        S <- g S;    w = beta (v - S^T k);    S <- S + k w^T;    o = S^T q      (the read-out sees the token's own write)

    q = W_q x and k = W_k x (``kv_heads`` heads of ``dim``), v = W_v x (``heads`` heads of ``vdim``; head h reads q/k head
    h // (heads / kv_heads)); each passes a causal convolution over ``conv`` taps per channel and silu; q and k become unit
    vectors per head (x / sqrt(sum(x^2) + 1e-6)), q also times dim^(-1/2); beta = sigmoid(W_b x) and the decay g =
    exp(-exp(A_log) softplus(W_a x + dt_bias)), one number per head.  Each head's o over its root mean square (``eps``) times
    a gain shared by the heads, times silu(W_g x), then W_o.  Two states per request: the matrix, and the convolution's
    last ``conv`` - 1 inputs.  All six projections are one matrix whose product stays float32."""

    NAMES = ("q", "k", "v", "b", "a", "g")

    def __init__(self, params, **kw):
        super().__init__(params, **kw)
        self.hidden = int(params["hidden_size"])
        self.heads = int(params["heads"])
        self.kv_heads = int(params.get("kv_heads", self.heads))
        self.dim = int(params["dim"])
        self.vdim = int(params["vdim"])
        self.taps = int(params.get("conv", 1))
        self.eps = float(params["eps"])
        if self.heads % self.kv_heads:
            raise ValueError(f"gated_delta: {self.heads} heads are no multiple of {self.kv_heads} query/key heads")
        if self.taps < 1:
            raise ValueError(f"gated_delta: conv={self.taps} must be at least 1")
        if not ops.delta_rule_supports(self.dim, self.vdim):
            raise ValueError(f"gated_delta: a head of {self.dim} key channels is outside what the recurrence kernel keeps in registers (1..256)")
        self.K, self.V = self.kv_heads * self.dim, self.heads * self.vdim
        self.C = 2 * self.K + self.V            # channels that pass the convolution

    def cache_need(self):
        needs = [SlotState((self.heads, self.dim, self.vdim), "delta")]
        if self.taps > 1:
            needs.append(SlotState((self.C, self.taps - 1), "conv"))
        return tuple(needs)

    def tensor_specs(self):
        H, W, K, V, t = self.heads, self.hidden, self.K, self.V, self.taps
        return [TensorSpec("q", (K, W)), TensorSpec("q.conv", (K, t), role="bias"), TensorSpec("k", (K, W)),
                TensorSpec("k.conv", (K, t), role="bias"), TensorSpec("v", (V, W)), TensorSpec("v.conv", (V, t), role="bias"),
                TensorSpec("b", (H, W)), TensorSpec("A_log", (H,), role="bias"), TensorSpec("norm", (self.vdim,), role="gain"),
                TensorSpec("a", (H, W)), TensorSpec("dt_bias", (H,), role="bias"), TensorSpec("g", (V, W)), TensorSpec("o", (W, V))]

    def bind(self, fetch):
        H = self.heads
        self.inp = Linear(self._matrix(torch.cat([fetch(n) for n in self.NAMES], dim=0)))
        self.offs = (0, self.K, 2 * self.K)
        self.off_b, self.off_a, self.off_g = self.C, self.C + H, self.C + 2 * H
        self.conv_w = self._f32(torch.cat([fetch(f"{n}.conv").float() for n in ("q", "k", "v")], dim=0))
        self.a_log = self._f32(fetch("A_log"))
        self.dt_bias = self._f32(fetch("dt_bias"))
        self.gain = self._f32(fetch("norm").float().repeat(H))
        self.out = Linear(self._matrix(fetch("o")))

    accepts_residual = True

    def mix(self, x, step: StepContext, cache: LayerCache, position=None, write_cache=True):
        proj = self.inp(x, torch.float32)                                            # [T, C + 2H + V] float32
        cv = ops.short_conv_silu(proj, 0, self.conv_w, cache.states.get("conv"), step)      # [T, C] float32
        o = ops.gated_delta_rule(cv, self.offs, proj, self.off_b, self.off_a, self.a_log, self.dt_bias, cache.states["delta"],
                                 step, self.heads, self.kv_heads, self.dim, self.vdim, self.dim ** -0.5)
        return ops.delta_out(o, self.gain, proj, self.off_g, self.eps, self.heads, self.vdim, self.dtype, "silu")

    def forward(self, x, step, cache, position, write_cache=True, residual=None):
        return self.out.into(self.mix(x, step, cache, position, write_cache), residual)

    def weight_bytes(self):
        return self.inp.nbytes() + self.out.nbytes() + 4 * (self.conv_w.numel() + self.gain.numel() + 2 * self.heads)
