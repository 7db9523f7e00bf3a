"""Plain, slow implementation of the Ridopel decoder: whole sequences, no cache, no batching.

One function per mechanism, numpy float64 throughout, written from the design's equations and
sharing no code with the product package (model folders are read with the `safetensors` package).

Notation: x is the residual stream [T, D]; h the input of a mixer (normed, then passed through the
layer's input convolution); H heads, dk the query/key size of a head, dv its value size, R the size of
the latent of the latent attention.
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


def silu(z):
    return z * sigmoid(z)


def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def rms_norm(x, weight, eps):
    return rms(x, eps) * weight


def input_convolution(h, taps):
    """h [T, C], taps [C, K]: h_t + sum_j taps[:, j] h_(t - (K - 1) + j), zeros before the start."""
    T, C = h.shape
    K = taps.shape[1]
    padded = np.concatenate([np.zeros((K - 1, C)), h], axis=0)
    y = h.copy()
    for j in range(K):
        y += padded[j:j + T] * taps[:, j]
    return y


def softmax(z):
    z = z - z.max(axis=-1, keepdims=True)
    e = np.exp(z)
    return e / e.sum(axis=-1, keepdims=True)


# --------------------------------------------------------------------------------------------
# the diagonal-decay recurrences
# --------------------------------------------------------------------------------------------
def wkv_scan(r, k, v, w, u):
    """One head.  r, k, w [T, dk], v [T, dv], u [dk]: o_t = (S + diag(u) k_t v_t^T)^T r_t with the state before
    the token, then S <- diag(w_t) S + k_t v_t^T."""
    T, dk = k.shape
    S = np.zeros((dk, v.shape[1]))
    out = np.zeros((T, v.shape[1]))
    for t in range(T):
        kv = np.outer(k[t], v[t])
        out[t] = (S + u[:, None] * kv).T @ r[t]
        S = w[t][:, None] * S + kv
    return out


def wkv_mixer(h, w, m, eps):
    """w: the mixer's tensors by their short names."""
    H, dk = m["heads"], m["dim"]
    T = h.shape[0]
    prev = np.concatenate([np.zeros((1, h.shape[1])), h[:-1]], axis=0)
    mix = {s: h + (prev - h) * w["mu." + s] for s in "rkvgw"}
    r = (mix["r"] @ w["r"].T).reshape(T, H, dk)
    k = (mix["k"] @ w["k"].T).reshape(T, H, dk)
    v = (mix["v"] @ w["v"].T).reshape(T, H, dk)
    gate = silu(mix["g"] @ w["g"].T)
    decay = np.exp(-np.exp(np.tanh(mix["w"] @ w["w1"].T) @ w["w2"].T + w["w0"])).reshape(T, H, dk)
    u = w["u"].reshape(H, dk)
    o = np.stack([rms(wkv_scan(r[:, i], k[:, i], v[:, i], decay[:, i], u[i]), eps) for i in range(H)], axis=1)
    return (o.reshape(T, H * dk) * w["norm"] * gate) @ w["o"].T


def hgrn2_scan(q, f, v):
    """One head.  q, f [T, dk], v [T, dv]: S <- diag(f_t) S + (1 - f_t) v_t^T, o_t = S^T q_t (after the write)."""
    T, dk = q.shape
    S = np.zeros((dk, v.shape[1]))
    out = np.zeros((T, v.shape[1]))
    for t in range(T):
        S = f[t][:, None] * S + np.outer(1.0 - f[t], v[t])
        out[t] = S.T @ q[t]
    return out


def hgrn2_mixer(h, w, m, eps):
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = silu(h @ w["q"].T).reshape(T, H, dk)
    v = (h @ w["v"].T).reshape(T, H, dv)
    low = w["lower"]
    f = (low + (1.0 - low) * sigmoid(h @ w["f"].T + w["f.b"])).reshape(T, H, dk)
    o = np.stack([rms_norm(hgrn2_scan(q[:, i], f[:, i], v[:, i]), w["norm"], eps) for i in range(H)], axis=1)
    return o.reshape(T, H * dv) @ w["o"].T


# --------------------------------------------------------------------------------------------
# latent attention
# --------------------------------------------------------------------------------------------
def rotate_pairs(x, positions, dims, base):
    """x [T, ..., d]: lanes 2i and 2i + 1 (i < dims / 2) turn by position * base^(-2i / dims)."""
    out = x.copy()
    half = dims // 2
    freq = np.array([base ** (-2.0 * i / dims) for i in range(half)])
    ang = np.asarray(positions, dtype=np.float64)[:, None] * freq
    shape = (len(positions),) + (1,) * (x.ndim - 2) + (half,)
    c, s = np.cos(ang).reshape(shape), np.sin(ang).reshape(shape)
    a, b = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = a * c - b * s
    out[..., 1:dims:2] = b * c + a * s
    return out


def latent_attention(h, w, m, eps, positions=None):
    H, dk, dr, dv, R = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    T = h.shape[0]
    positions = list(range(T)) if positions is None else positions
    q = (h @ w["q"].T).reshape(T, H, dk + dr)
    down = h @ w["dkv"].T
    c = rms_norm(down[:, :R], w["dkv.norm"], eps)
    k_rot = rotate_pairs(down[:, R:], positions, m["rot"]["dims"], m["rot"]["base"])           # [T, dr], one for all heads
    q_rot = rotate_pairs(q[:, :, dk:], positions, m["rot"]["dims"], m["rot"]["base"])
    k = (c @ w["uk"].T).reshape(T, H, dk)
    v = (c @ w["uv"].T).reshape(T, H, dv)
    scores = (np.einsum("thd,shd->hts", q[:, :, :dk], k) + np.einsum("thd,sd->hts", q_rot, k_rot)) * m["scale"]
    mask = np.asarray(positions)[None, :] > np.asarray(positions)[:, None]
    scores = np.where(mask[None], -np.inf, scores)
    p = softmax(scores)
    o = np.einsum("hts,shd->thd", p, v).reshape(T, H * dv)
    return (o * sigmoid(h @ w["g"].T)) @ w["o"].T


# --------------------------------------------------------------------------------------------
# feed-forward
# --------------------------------------------------------------------------------------------
def expert(h, gate, up, down, limit):
    g = np.minimum(h @ gate.T, limit)
    u = np.clip(h @ up.T, -limit, limit)
    return (g * sigmoid(1.702 * g) * (u + 1.0)) @ down.T


def route(h, router, correction, top):
    """(chosen experts [T, top], their weights [T, top])."""
    s = softmax(h @ router.T)
    order = np.argsort(-(s + correction), axis=-1, kind="stable")[:, :top]
    chosen = np.take_along_axis(s, order, axis=-1)
    return order, chosen / (chosen.sum(axis=-1, keepdims=True) + 1e-20)


def experts_feed_forward(h, w, f):
    ids, weights = route(h, w["router"], w["correction"], f["router"]["top"])
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t], weights[t]):
            out[t] += a * expert(h[t], w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"], f["expert"]["limit"])
    return out


# --------------------------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------------------------
def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def mixer(h, layer, tensors, prefix, eps):
    w, m = sub(tensors, prefix + "mix."), layer["mixer"]
    if layer["type"] == "wkv":
        return wkv_mixer(h, w, m, eps)
    if layer["type"] == "hgrn2":
        return hgrn2_mixer(h, w, m, eps)
    if layer["type"] == "latent_attention":
        return latent_attention(h, w, m, eps)
    raise ValueError(layer["type"])


def run_order(cfg):
    """[(layer, first of a pass)]: the looped layers `times` times in a row, the others once."""
    n = len(cfg["layers"])
    loop = cfg.get("loop") or {"start": 0, "stop": 0, "times": 1}
    order = [(i, False) for i in range(loop["start"])]
    for _ in range(loop["times"]):
        order += [(i, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return order + [(i, False) for i in range(loop["stop"], n)]


def forward(cfg, tensors, tokens, return_layers=False):
    """Logits [T, vocab] of a whole sequence (and the stream after every layer run)."""
    eps = cfg["norm"]["eps"]
    x0 = rms_norm(tensors["embed"][np.asarray(tokens)], tensors["embed.norm"], eps)
    x = x0.copy()
    layers_out = []
    for i, first in run_order(cfg):
        layer, p = cfg["layers"][i], f"l{i}."
        if first:
            x = np.concatenate([x, x0], axis=-1) @ tensors["loop.in"].T
        h = input_convolution(rms_norm(x, tensors[p + "norm1"], eps), tensors[p + "canon1"])
        x = x + mixer(h, layer, tensors, p, eps)
        if layer["mlp"] is not None:
            x = x + experts_feed_forward(rms_norm(x, tensors[p + "norm2"], eps), sub(tensors, p + "mlp."), layer["mlp"])
        layers_out.append(x.copy())
    logits = rms_norm(x, tensors["final.norm"], eps) @ tensors["head"].T
    cap = cfg.get("logit_softcap")
    if cap:
        logits = cap * np.tanh(logits / cap)
    return (logits, np.stack(layers_out)) if return_layers else logits


def greedy(cfg, tensors, prompt, n_new):
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(np.argmax(forward(cfg, tensors, tokens)[-1])))
    return tokens[len(prompt):]
