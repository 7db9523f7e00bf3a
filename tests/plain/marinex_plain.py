"""Plain, slow implementation of the Marinex decoder: whole sequences, no cache, no batching.

One function per mechanism, numpy float64 throughout, written from the design's equations and
sharing no code with the product package (model folders are read with the `safetensors` package).

Notation: x is the residual stream [T, D]; a sublayer reads x itself, and what it returns is RMS-normed
before it joins the stream.  H query heads, G key/value heads, dk the query/key size of a head, dv its value
size, R the size of the latent of the latent attention.
"""
from __future__ import annotations

import json
import math
import os

import numpy as np


def read_model_folder(folder):
    """config.json as a dict and every tensor as float64 (integer tables as int64), by stored name."""
    import torch
    from safetensors.torch import load_file

    with open(os.path.join(folder, "config.json")) as f:
        cfg = json.load(f)
    raw = load_file(os.path.join(folder, "model.safetensors"))
    tensors = {k: (v.to(torch.float64).numpy() if v.is_floating_point() else v.to(torch.int64).numpy())
               for k, v in raw.items()}
    return cfg, tensors


# --------------------------------------------------------------------------------------------
# small functions
# --------------------------------------------------------------------------------------------
def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def gelu_erf(z):
    return 0.5 * z * (1.0 + np.vectorize(math.erf)(z / math.sqrt(2.0)))


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def rms_norm(x, weight, eps):
    return rms(x, eps) * weight


def frequencies(dims, base):
    return np.array([base ** (-2.0 * i / dims) for i in range(dims // 2)])


def rotate_neighbours(x, positions, dims, base):
    """x [T, ..., d]: the lanes (2i, 2i + 1), i < dims / 2, of the last axis turn by position * base^(-2i / dims);
    lanes from `dims` on stay."""
    if dims == 0:
        return x.copy()
    ang = positions[:, None] * frequencies(dims, base)[None, :]            # [T, dims / 2]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (dims // 2,)
    c, s = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    out = x.copy()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def rotate_halves(x, positions, dims, base):
    """The same turn with lane i paired with lane i + dims / 2, i < dims / 2."""
    if dims == 0:
        return x.copy()
    half = dims // 2
    ang = positions[:, None] * frequencies(dims, base)[None, :]
    shape = (x.shape[0],) + (1,) * (x.ndim - 2) + (half,)
    c, s = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    out = x.copy()
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def softmax_with_sink(scores, visible, sink):
    """scores [T, T], visible [T, T] bool, sink a number: p_ij = e^(s_ij) / (e^sink + sum_visible e^(s_ij))."""
    s = np.where(visible, scores, -np.inf)
    m = np.maximum(s.max(axis=-1, keepdims=True), sink)
    e = np.exp(s - m)
    return e / (np.exp(sink - m) + e.sum(axis=-1, keepdims=True))


def causal(T):
    i = np.arange(T)
    return i[None, :] <= i[:, None]


def window(T, size):
    i = np.arange(T)
    d = i[:, None] - i[None, :]
    return (d >= 0) & (d < size)


# --------------------------------------------------------------------------------------------
# mixers
# --------------------------------------------------------------------------------------------
def attention(h, w, m, eps, prefix):
    """Grouped-query attention with normed queries, keys and values, a number per head on the scores, capped scores
    and a sink of score 0.  h [T, D]; m the mixer's configuration; w the tensors by stored name."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = np.arange(T, dtype=np.float64)
    q = (h @ w[prefix + "q"].T).reshape(T, H, dk)
    k = (h @ w[prefix + "k"].T).reshape(T, G, dk)
    v = (h @ w[prefix + "v"].T).reshape(T, G, dv)
    q = rms_norm(q, w[prefix + "q.norm"], eps)
    k = rms_norm(k, w[prefix + "k.norm"], eps)
    q = rotate_neighbours(q, pos, m["rot"]["dims"], m["rot"]["base"])
    k = rotate_neighbours(k, pos, m["rot"]["dims"], m["rot"]["base"])
    v = rms(v, eps)
    cap = m["softcap"]
    out = np.zeros((T, H, dv))
    see = causal(T)
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * m["scale"] * w[prefix + "temp"][head]
        s = cap * np.tanh(s / cap)
        out[:, head] = softmax_with_sink(s, see, 0.0) @ v[:, g]
    return out.reshape(T, H * dv) @ w[prefix + "o"].T


def latent_attention(h, w, m, eps, prefix):
    """Attention over a latent: queries through a normed latent of their own; keys and values of all heads from one
    normed latent per position plus one turned key part that the heads share; a window; a learned sink per head; a
    sigmoid gate per head."""
    T = h.shape[0]
    H, dk, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = np.arange(T, dtype=np.float64)
    cq = rms_norm(h @ w[prefix + "dq"].T, w[prefix + "dq.norm"], eps)
    q = (cq @ w[prefix + "uq"].T).reshape(T, H, dk + dr)
    q_plain, q_turn = q[..., :dk], q[..., dk:]
    down = h @ w[prefix + "dkv"].T
    c = rms_norm(down[:, :R], w[prefix + "dkv.norm"], eps)
    k_turn = rotate_halves(down[:, R:], pos, m["rot"]["dims"], m["rot"]["base"])      # [T, dr]
    q_turn = rotate_halves(q_turn, pos, m["rot"]["dims"], m["rot"]["base"])
    k_plain = (c @ w[prefix + "uk"].T).reshape(T, H, dk)
    v = (c @ w[prefix + "uv"].T).reshape(T, H, dv)
    gate = sigmoid(h @ w[prefix + "g"].T)                                              # [T, H]
    see = window(T, m["mask"]["size"])
    out = np.zeros((T, H, dv))
    for head in range(H):
        s = (q_plain[:, head] @ k_plain[:, head].T + q_turn[:, head] @ k_turn.T) * m["scale"]
        out[:, head] = softmax_with_sink(s, see, w[prefix + "sink"][head]) @ v[:, head] * gate[:, head:head + 1]
    return out.reshape(T, H * dv) @ w[prefix + "o"].T


# --------------------------------------------------------------------------------------------
# feed-forward
# --------------------------------------------------------------------------------------------
def route(h, w, f, prefix):
    """(chosen [T, top] expert numbers, weights [T, top]): sigmoid scores; the choice adds a stored correction and is
    limited to the experts of the best groups (a group's mark: the sum of its two largest corrected scores); the
    weights are the scores themselves."""
    r = f["router"]
    E, top, n_groups, keep = r["experts"], r["top"], r["groups"]["count"], r["groups"]["keep"]
    s = sigmoid(h @ w[prefix + "router"].T)                     # [T, E]
    choice = s + w[prefix + "correction"]
    per = E // n_groups
    chosen = np.zeros((h.shape[0], top), dtype=np.int64)
    weights = np.zeros((h.shape[0], top))
    for t in range(h.shape[0]):
        grouped = choice[t].reshape(n_groups, per)
        marks = np.sort(grouped, axis=-1)[:, ::-1][:, :2].sum(axis=-1)
        best = np.argsort(-marks, kind="stable")[:keep]
        masked = np.full(E, -np.inf)
        for g in best:
            masked[g * per:(g + 1) * per] = choice[t, g * per:(g + 1) * per]
        ids = np.argsort(-masked, kind="stable")[:top]
        chosen[t], weights[t] = ids, s[t, ids]
    return chosen, weights


def experts(h, w, f, prefix):
    chosen, weights = route(h, w, f, prefix)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(chosen[t], weights[t]):
            inner = gelu_erf(w[f"{prefix}e{e}.up"] @ h[t])
            out[t] += a * (w[f"{prefix}e{e}.down"] @ inner)
    return out


# --------------------------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------------------------
MIXERS = {"attention": attention, "latent_attention": latent_attention}


def layer(x, w, entry, eps, i):
    p = f"l{i}."
    x = x + rms_norm(MIXERS[entry["type"]](x, w, entry["mixer"], eps, p + "mix."), w[p + "norm1"], eps)
    if entry.get("mlp") is not None:
        x = x + rms_norm(experts(x, w, entry["mlp"], p + "mlp."), w[p + "norm2"], eps)
    return x


def forward(cfg, w, tokens, collect=None):
    """Logits [T, vocab] of one sequence; `collect` (a list) receives the stream after every layer."""
    eps = cfg["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)]
    for i, entry in enumerate(cfg["layers"]):
        x = layer(x, w, entry, eps, i)
        if collect is not None:
            collect.append(x.copy())
    return rms_norm(x, w["final.norm"], eps) @ w["head"].T


def greedy(cfg, w, prompt, n):
    """n tokens after the prompt, each the argmax of the last position's logits (the lowest index on a tie)."""
    tokens, out = list(prompt), []
    for _ in range(n):
        out.append(int(np.argmax(forward(cfg, w, tokens)[-1])))
        tokens.append(out[-1])
    return out
