"""Plain, slow, whole-sequence statement of the Rososun design, one function per mechanism.

A decoder-only model whose layers are "parallel" blocks: one grouped RMS norm, whose output both the
mixer and the feed-forward read, and one addition of both terms to the stream.  The mixer's input is
first blended with the previous token's normed vector (token shift).  Two mixers exist: a generalized
delta rule (a matrix state per head, decayed per key channel, with a rank-one removal along the unit
key) and latent attention (keys and values of all heads are up-projections of one small normed latent
vector per token; no positions; a sigmoid gate per head).  The feed-forward is gated, with the tanh
form of GELU and biases everywhere.  Positions enter once, as a sinusoidal vector added to the scaled
embedding.  A layer may use another layer's tensors (with a state of its own).

Everything is numpy in one floating type (float64 by default), no cache, no batching: the whole
sequence is recomputed for every question.  Shares no code with the package.
"""

from __future__ import annotations

import json
import struct

import numpy as np


# ---- model folder ---------------------------------------------------------------------------

def read_safetensors(path: str, dtype=np.float64) -> dict:
    """8-byte little-endian header length, a JSON header name -> dtype/shape/data_offsets, raw bytes."""
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


def gelu_tanh(z):
    return 0.5 * z * (1.0 + np.tanh(np.sqrt(2.0 / np.pi) * (z + 0.044715 * z ** 3)))


def unit_rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt((x * x).mean(-1, keepdims=True) + eps)


def embedding(ids, table, scale):
    return table[np.asarray(ids, dtype=np.int64)] * scale


def sinusoid(positions, width, dtype=np.float64):
    """Pairs (sin, cos) of the angle p * f_i, f_i = 10000^(-2i/width), at channels (2i, 2i+1) of position p."""
    i = np.arange(width // 2, dtype=np.float64)
    ang = (np.asarray(positions, dtype=np.float64)[:, None] * 10000.0 ** (-2.0 * i / width)[None, :]).astype(dtype)
    out = np.empty((len(positions), width), dtype=dtype)
    out[:, 0::2] = np.sin(ang)
    out[:, 1::2] = np.cos(ang)
    return out


def group_norm(x, gain, groups, eps):
    """The vector in `groups` equal consecutive parts, each over its own root mean square; then times the gain."""
    T, W = x.shape
    return unit_rms(x.reshape(T, groups, W // groups), eps).reshape(T, W) * gain


def token_shift(h, mix, before=None):
    """h + (previous token's h - h) * mix; the first token's predecessor is `before` (zeros at a sequence's start)."""
    prev = np.concatenate([np.zeros_like(h[:1]) if before is None else before[None], h[:-1]], axis=0)
    return h + (prev - h) * mix


# ---- mixers ---------------------------------------------------------------------------------

def general_delta(h, w, p, heads, dim, eps, state=None):
    """The generalized delta rule, token by token.  Per head a state S [key channel, value channel]:

        S <- diag(d) S - (a * u) (u^T S) + k v^T,     o = S^T r

    d = exp(-exp(-1/2) * sigmoid(W_w2 tanh(W_w1 h) + w0)) the decay, a = sigmoid(W_a h + b_a) the removal
    rate, u the key of the head over its Euclidean length (1e-6 inside the root); S on the right is the state
    before the token.  Each head's o over its root mean square, times a gain over all heads, times
    sigmoid(W_g h), then W_o.  Returns (term, final state)."""
    T = h.shape[0]
    r, k, v = h @ w[f"{p}.r"].T, h @ w[f"{p}.k"].T, h @ w[f"{p}.v"].T
    d = np.exp(-np.exp(-0.5) * sigmoid(np.tanh(h @ w[f"{p}.w1"].T) @ w[f"{p}.w2"].T + w[f"{p}.w0"]))
    a = sigmoid(h @ w[f"{p}.a"].T + w[f"{p}.a.b"])
    shp = (T, heads, dim)
    r, k, v, d, a = (z.reshape(shp) for z in (r, k, v, d, a))
    u = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    S = np.zeros((heads, dim, dim), dtype=h.dtype) if state is None else state.copy()
    o = np.empty(shp, dtype=h.dtype)
    for t in range(T):
        uS = np.einsum("hi,hij->hj", u[t], S)
        S = d[t][:, :, None] * S - (a[t] * u[t])[:, :, None] * uS[:, None, :] + k[t][:, :, None] * v[t][:, None, :]
        o[t] = np.einsum("hij,hi->hj", S, r[t])
    o = unit_rms(o, eps).reshape(T, heads * dim) * w[f"{p}.norm"]
    o = o * sigmoid(h @ w[f"{p}.g"].T)
    return o @ w[f"{p}.o"].T, S


def latent_attention(h, w, p, heads, dim, vdim, rank, scale, eps):
    """Keys and values of every head are up-projections of one latent vector per token, c = the normed
    W_dkv h (plain gain).  No positions; causal; ordinary softmax; head i's output times sigmoid(W_g h)_i."""
    T = h.shape[0]
    q = (h @ w[f"{p}.q"].T).reshape(T, heads, dim)
    c = unit_rms(h @ w[f"{p}.dkv"].T, eps) * w[f"{p}.dkv.norm"]
    k = (c @ w[f"{p}.uk"].T).reshape(T, heads, dim)
    v = (c @ w[f"{p}.uv"].T).reshape(T, heads, vdim)
    s = np.einsum("thd,jhd->htj", q, k) * scale
    s = np.where(np.tril(np.ones((T, T), dtype=bool))[None], s, -np.inf)
    s = np.exp(s - s.max(-1, keepdims=True))
    s = s / s.sum(-1, keepdims=True)
    o = np.einsum("htj,jhd->thd", s, v)
    o = o * sigmoid(h @ w[f"{p}.g"].T)[:, :, None]
    return o.reshape(T, heads * vdim) @ w[f"{p}.o"].T, c


# ---- feed-forward ---------------------------------------------------------------------------

def dense_ffn(h, w, p):
    g = h @ w[f"{p}.gate"].T + w[f"{p}.gate.b"]
    u = h @ w[f"{p}.up"].T + w[f"{p}.up.b"]
    return (gelu_tanh(g) * u) @ w[f"{p}.down"].T + w[f"{p}.down.b"]


# ---- the model ------------------------------------------------------------------------------

def forward(ids, cfg, w, return_layers=False):
    """Logits [T, vocab] of one sequence (and the stream after every layer run, if asked)."""
    dtype = w["embed"].dtype
    W = cfg["width"]
    eps, groups = cfg["norm"]["eps"], cfg["norm"]["groups"]
    x = embedding(ids, w["embed"], cfg["embedding"]["scale"]) + sinusoid(np.arange(len(ids)), W, dtype)
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{layer.get('weights_of', i)}"
        m = layer["mixer"]
        h = group_norm(x, w[f"{p}.norm1"], groups, eps)
        hs = token_shift(h, w[f"{p}.shift"])
        if layer["type"] == "general_delta":
            term, _ = general_delta(hs, w, f"{p}.mix", m["heads"], m["dim"], eps)
        elif layer["type"] == "latent_attention":
            term, _ = latent_attention(hs, w, f"{p}.mix", m["heads"], m["dim"], m["vdim"], m["kv_rank"], m["scale"], eps)
        else:
            raise ValueError(layer["type"])
        if layer.get("mlp") is not None:
            term = term + dense_ffn(h, w, f"{p}.mlp")
        x = x + term
        streams.append(x)
    x = group_norm(x, w["final.norm"], groups, eps)
    logits = x @ w["head"].T
    return (logits, np.stack(streams)) if return_layers else logits
