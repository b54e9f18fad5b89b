"""Plain, slow, whole-sequence statement of the Nutopel design, one function per mechanism.

A decoder-only model of pre-norm layers, x <- x + mixer(norm(x)), x <- x + ff(norm(x)), whose norms carry
their gain as an offset from one.  A layer's mixer is either gated linear attention (a matrix state per head
with a decay per key channel) or a pair of mixers side by side, softmax attention restricted to the query's own
block of positions next to a gated delta rule behind short convolutions, whose outputs are normed and averaged.
The feed-forward is a mixture of small experts behind a sigmoid router that first narrows the choice to the
best groups of experts, plus one expert every token uses.

Everything is numpy in one floating type (float64 by default), no cache, no batching, token by token where a
recurrence is stated token by token.  Shares no code with the package.
"""

from __future__ import annotations

import json
import math
import struct

import numpy as np


# ---- model folder ---------------------------------------------------------------------------

def read_safetensors(path: str, dtype=np.float64) -> dict:
    with open(path, "rb") as f:
        (n,) = struct.unpack("<Q", f.read(8))
        header = json.loads(f.read(n))
        blob = f.read()
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        raw = blob[lo:hi]
        if meta["dtype"] == "BF16":
            arr = (np.frombuffer(raw, dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(dtype)
        elif meta["dtype"] == "F32":
            arr = np.frombuffer(raw, dtype="<f4").astype(dtype)
        elif meta["dtype"] == "I32":
            arr = np.frombuffer(raw, dtype="<i4")
        else:
            raise ValueError(f"{name}: dtype {meta['dtype']}")
        out[name] = arr.reshape(meta["shape"]).copy()
    return out


def load_model(model_dir: str, dtype=np.float64):
    with open(f"{model_dir}/config.json") as f:
        cfg = json.load(f)
    return cfg, read_safetensors(f"{model_dir}/model.safetensors", dtype)


# ---- small pieces ---------------------------------------------------------------------------

def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def gelu_erf(z):
    return 0.5 * z * (1.0 + np.vectorize(math.erf)(z / math.sqrt(2.0)))


def unit_rms(x, eps):
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def norm_one_plus(x, w, eps):
    """The layers' and the model's norm: the stored gain is an offset from one."""
    return unit_rms(x, eps) * (1.0 + w)


def norm_plain(x, w, eps):
    return unit_rms(x, eps) * w


# ---- rotary positions with a two-regime frequency scaling --------------------------------------

def rotary_frequencies(rot: dict):
    """(frequencies [dims/2], the factor cos and sin are multiplied by)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def dim_of(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x, positions, rot: dict):
    """x [T, heads, dim]: the first dims channels of each head turn by position * frequency, channel i paired with i + dims/2."""
    dims = int(rot["dims"])
    f, mag = rotary_frequencies(rot)
    ang = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = (np.cos(ang) * mag)[:, None, :], (np.sin(ang) * mag)[:, None, :]
    half = dims // 2
    u, v = x[..., :half], x[..., half:dims]
    out = x.copy()
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


# ---- mixers ------------------------------------------------------------------------------------

def block_attention(h, w, p, m, eps, positions):
    """Softmax attention in which position i sees j <= i of its own block of ``mask.size`` positions only."""
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(T, H, D)
    k = (h @ w[p + "k"].T).reshape(T, G, D)
    v = (h @ w[p + "v"].T).reshape(T, G, V)
    q = norm_plain(q, w[p + "q.norm"], eps)
    k = norm_plain(k, w[p + "k.norm"], eps)
    q, k = rotate(q, positions, m["rot"]), rotate(k, positions, m["rot"])
    size = int(m["mask"]["size"])
    pos = np.asarray(positions)
    seen = (pos[None, :] <= pos[:, None]) & (pos[None, :] // size == pos[:, None] // size)
    out = np.zeros((T, H, V), dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        s = (q[:, hh] @ k[:, g].T) * m["scale"]
        s = np.where(seen, s, -np.inf)
        e = np.exp(s - s.max(-1, keepdims=True))
        out[:, hh] = (e / e.sum(-1, keepdims=True)) @ v[:, g]
    return out.reshape(T, H * V) @ w[p + "o"].T


def short_convolution(x, taps_w):
    """x [T, C], taps_w [C, taps]: y_t = sum_j taps_w[:, taps-1-j] * x_(t-j), zeros before the start."""
    T, C = x.shape
    taps = taps_w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, C), dtype=x.dtype), x], axis=0)
    y = np.zeros_like(x)
    for j in range(taps):
        y += padded[j:j + T] * taps_w[:, j][None, :]
    return y


def gated_delta(h, w, p, m, eps):
    T = h.shape[0]
    H, G, D, V = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_convolution(h @ w[p + "q"].T, w[p + "q.conv"])).reshape(T, G, D)
    k = silu(short_convolution(h @ w[p + "k"].T, w[p + "k.conv"])).reshape(T, G, D)
    v = silu(short_convolution(h @ w[p + "v"].T, w[p + "v.conv"])).reshape(T, H, V)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * D ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w[p + "b"].T)
    decay = np.exp(-np.exp(w[p + "A_log"])[None, :] * softplus(h @ w[p + "a"].T + w[p + "dt_bias"][None, :]))
    gate = silu(h @ w[p + "g"].T).reshape(T, H, V)
    out = np.zeros((T, H, V), dtype=h.dtype)
    for hh in range(H):
        g = hh // (H // G)
        S = np.zeros((D, V), dtype=h.dtype)
        for t in range(T):
            S = decay[t, hh] * S
            u = beta[t, hh] * (v[t, hh] - S.T @ k[t, g])
            S = S + np.outer(k[t, g], u)
            out[t, hh] = S.T @ q[t, g]
    out = norm_plain(out, w[p + "norm"], eps) * gate
    return out.reshape(T, H * V) @ w[p + "o"].T


def side_by_side(h, w, p, m, eps, positions):
    left = block_attention(h, w, p + "left.", m["left"], eps, positions)
    right = gated_delta(h, w, p + "right.", m["right"], eps)
    return 0.5 * (norm_plain(left, w[p + "left.out"], eps) + norm_plain(right, w[p + "right.out"], eps))


def gated_linear_attention(h, w, p, m, eps):
    T = h.shape[0]
    H, D, V = m["heads"], m["dim"], m["vdim"]
    q = (h @ w[p + "q"].T).reshape(T, H, D) * D ** -0.5
    k = (h @ w[p + "k"].T).reshape(T, H, D)
    v = (h @ w[p + "v"].T).reshape(T, H, V)
    z = (h @ w[p + "a1"].T) @ w[p + "a2"].T + w[p + "a2.b"][None, :]
    alpha = (sigmoid(z) ** (1.0 / m["tau"])).reshape(T, H, D)
    out = np.zeros((T, H, V), dtype=h.dtype)
    for hh in range(H):
        S = np.zeros((D, V), dtype=h.dtype)
        for t in range(T):
            S = alpha[t, hh][:, None] * S + np.outer(k[t, hh], v[t, hh])
            out[t, hh] = S.T @ q[t, hh]
    out = norm_plain(out, w[p + "norm"], eps).reshape(T, H * V) * silu(h @ w[p + "g"].T)
    return out @ w[p + "o"].T


# ---- feed-forward ------------------------------------------------------------------------------------

def route(h, w, p, r, margins=None):
    """(chosen experts [T, top], their weights [T, top]).  ``margins`` (a list) receives, per token, how far the choice
    was from going another way: the smaller of the gaps between the last group kept and the first one left out, and
    between the last expert chosen and the first one not."""
    E, top = int(r["experts"]), int(r["top"])
    s = sigmoid(h @ w[p + "router"].T)
    choice = s + w[p + "correction"][None, :]
    gr = r.get("groups")
    if gr:
        count, keep = int(gr["count"]), int(gr["keep"])
        per = E // count
        grouped = choice.reshape(-1, count, per)
        score = np.sort(grouped, axis=-1)[..., -2:].sum(-1)
        best = np.argsort(-score, axis=-1, kind="stable")[:, :keep]
        ranked = -np.sort(-score, axis=-1)
        group_gap = ranked[:, keep - 1] - ranked[:, keep] if keep < count else np.full(h.shape[0], np.inf)
        allowed = np.zeros((h.shape[0], count), dtype=bool)
        np.put_along_axis(allowed, best, True, axis=1)
        choice = np.where(np.repeat(allowed, per, axis=1), choice, -np.inf)
    else:
        group_gap = np.full(h.shape[0], np.inf)
    chosen = np.argsort(-choice, axis=-1, kind="stable")[:, :top]
    if margins is not None:
        ranked = -np.sort(-choice, axis=-1)
        gap = ranked[:, top - 1] - ranked[:, top] if top < E else np.full(h.shape[0], np.inf)
        margins.append(np.minimum(gap, group_gap))
    return chosen, np.take_along_axis(s, chosen, axis=1) * float(r["scale"])


def expert(h, w, p):
    return gelu_erf(h @ w[p + "up"].T) @ w[p + "down"].T


def mixture(h, w, p, mlp, margins=None):
    chosen, weight = route(h, w, p, mlp["router"], margins)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, g in zip(chosen[t], weight[t]):
            out[t] += g * expert(h[t:t + 1], w, f"{p}e{e}.")[0]
    if mlp.get("shared"):
        out += expert(h, w, p + "shared.")
    return out


# ---- the model ------------------------------------------------------------------------------------

def forward(ids, cfg, w, dtype=np.float64, layers_out=None, margins=None):
    """Logits [T, vocab] of one sequence; ``layers_out`` (a list) receives the stream after every layer, ``margins`` (a
    list) every router's margins per token (see `route`)."""
    eps = float(cfg["norm"]["eps"])
    positions = np.arange(len(ids))
    x = w["embed"][np.asarray(ids, dtype=np.int64)].astype(dtype)
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        h = norm_one_plus(x, w[p + "norm1"], eps)
        if layer["type"] == "parallel":
            x = x + side_by_side(h, w, p + "mix.", layer["mixer"], eps, positions)
        elif layer["type"] == "gla":
            x = x + gated_linear_attention(h, w, p + "mix.", layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            x = x + mixture(norm_one_plus(x, w[p + "norm2"], eps), w, p + "mlp.", layer["mlp"], margins)
        if layers_out is not None:
            layers_out.append(x.copy())
    return (norm_one_plus(x, w["final.norm"], eps) @ w["head"].T) * float(cfg["logit_scale"])
