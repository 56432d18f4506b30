"""Plain, slow implementation of the Nufolix decoder: whole sequences, no cache, no batching.

One function per mechanism, numpy float64 throughout, written from the design's equations and
sharing no code with the product package (model folders are read with the `safetensors` package).

Notation: x is the residual stream [T, D]; h the normed input of a sublayer; H heads, G key/value (or
query/key) heads, dk the query/key size of a head, dv its value size, N the state size of a state-space head.
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


def softplus(z):
    return np.logaddexp(0.0, z)


def rms_norm(x, weight, eps):
    """x / sqrt(mean(x^2) + eps) * weight over the last axis."""
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * weight


def causal_conv(x, taps, bias=None):
    """x [T, C], taps [C, K]: y_t = sum_k taps[:, k] x_(t - (K-1) + k), zeros before the start."""
    T, C = x.shape
    K = taps.shape[1]
    padded = np.concatenate([np.zeros((K - 1, C)), x], axis=0)
    y = np.zeros((T, C))
    for k in range(K):
        y += padded[k:k + T] * taps[:, k]
    if bias is not None:
        y = y + bias
    return y


def xielu(z, p, q):
    """z > 0: softplus(p) z^2 + z/2;  z <= 0: (1/2 + softplus(q)) (exp(z) - 1 - z) + z/2."""
    ap, an = softplus(p), 0.5 + softplus(q)
    zn = np.minimum(z, 0.0)
    return np.where(z > 0, ap * z * z + 0.5 * z, an * (np.expm1(zn) - zn) + 0.5 * z)


# --------------------------------------------------------------------------------------------
# the state-space mixer
# --------------------------------------------------------------------------------------------
def mamba2_scan(xs, B, C, dt, A_log, D, heads, groups):
    """xs [T, heads, dv], B and C [T, groups, N], dt [T, heads] (after its softplus): per head
    S <- exp(-exp(A_log) dt) S + dt B x^T (S is N x dv), y = S^T C + D x."""
    T, _, dv = xs.shape
    N = B.shape[2]
    per = heads // groups
    y = np.zeros((T, heads, dv))
    for h in range(heads):
        g = h // per
        S = np.zeros((N, dv))
        a = -math.exp(A_log[h])
        for t in range(T):
            S = math.exp(a * dt[t, h]) * S + dt[t, h] * np.outer(B[t, g], xs[t, h])
            y[t, h] = S.T @ C[t, g] + D[h] * xs[t, h]
    return y


def mamba2_mixer(h, w, m, eps):
    """w: this mixer's tensors by their short names ('in', 'conv', 'conv.b', 'dt_bias', 'A_log', 'D', 'norm', 'o')."""
    heads, dv, N, G = m["heads"], m["vdim"], m["state"], m["groups"]
    inner = heads * dv
    p = h @ w["in"].T
    z, xbc, dt = p[:, :inner], p[:, inner:2 * inner + 2 * G * N], p[:, 2 * inner + 2 * G * N:]
    xbc = silu(causal_conv(xbc, w["conv"], w["conv.b"]))
    xs = xbc[:, :inner].reshape(-1, heads, dv)
    B = xbc[:, inner:inner + G * N].reshape(-1, G, N)
    C = xbc[:, inner + G * N:].reshape(-1, G, N)
    dt = softplus(dt + w["dt_bias"])
    y = mamba2_scan(xs, B, C, dt, w["A_log"], w["D"], heads, G).reshape(-1, inner)
    y = y * silu(z)
    parts = m["norm_groups"]
    y = y.reshape(y.shape[0], parts, inner // parts)
    y = (y / np.sqrt((y * y).mean(axis=-1, keepdims=True) + eps)).reshape(-1, inner) * w["norm"]
    return y @ w["o"].T


# --------------------------------------------------------------------------------------------
# the attention without a softmax
# --------------------------------------------------------------------------------------------
def rotate(x, positions, dims, base):
    """x [T, heads, d]: the first `dims` lanes of every head rotate, lane i with lane i + dims/2, by the angle
    position * base^(-2i/dims); the other lanes pass."""
    half = dims // 2
    out = x.copy()
    if half == 0:
        return out
    f = np.asarray([base ** (-2.0 * i / dims) for i in range(half)])
    a = np.asarray(positions, dtype=np.float64)[:, None] * f[None, :]
    c, s = np.cos(a)[:, None, :], np.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    out[..., :half] = u * c - v * s
    out[..., half:dims] = v * c + u * s
    return out


def sigmoid_attention_weights(q, k, scale, softcap, head_bias):
    """q [T, H, dk], k [T, G, dk]: w[h, i, j] = sigmoid(cap(scale q_hi . k_gj) + bias_h) for j <= i, else 0."""
    T, H, _ = q.shape
    G = k.shape[1]
    per = H // G
    w = np.zeros((H, T, T))
    mask = np.tril(np.ones((T, T), dtype=bool))
    for h in range(H):
        s = (q[:, h] @ k[:, h // per].T) * scale
        s = softcap * np.tanh(s / softcap)
        w[h] = np.where(mask, sigmoid(s + head_bias[h]), 0.0)
    return w


def mix_heads(w, talk):
    """w [H, T, T], talk [H, H]: w'_h = sum_g talk[h, g] w_g."""
    return np.einsum("hg,gij->hij", talk, w)


def sigmoid_attention(h, w, m, positions=None):
    """w: the tensors 'q', 'q.b', 'k', 'k.b', 'v', 'v.b', 'talk', 'pb', 'o'."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    positions = list(range(T)) if positions is None else positions
    q = (h @ w["q"].T + w["q.b"]).reshape(T, H, dk)
    k = (h @ w["k"].T + w["k.b"]).reshape(T, G, dk)
    v = (h @ w["v"].T + w["v.b"]).reshape(T, G, dv)
    q = rotate(q, positions, m["rot"]["dims"], m["rot"]["base"])
    k = rotate(k, positions, m["rot"]["dims"], m["rot"]["base"])
    wt = sigmoid_attention_weights(q, k, m["scale"], m["softcap"], w["pb"])
    wt = mix_heads(wt, w["talk"])
    per = H // G
    out = np.zeros((T, H, dv))
    for hd in range(H):
        out[:, hd] = wt[hd] @ v[:, hd // per]
    return out.reshape(T, H * dv) @ w["o"].T


# --------------------------------------------------------------------------------------------
# the gated delta rule
# --------------------------------------------------------------------------------------------
def unit(x):
    return x / np.sqrt((x * x).sum(axis=-1, keepdims=True) + 1e-6)


def delta_rule_scan(q, k, v, beta, g):
    """q, k [T, G, dk]; v [T, H, dv]; beta [T, H]; g [T, H, dk].  Per head, S [dk, dv] from zero:
    S <- g[:, None] S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q."""
    T, H, dv = v.shape
    G, dk = q.shape[1], q.shape[2]
    per = H // G
    o = np.zeros((T, H, dv))
    for h in range(H):
        S = np.zeros((dk, dv))
        c = h // per
        for t in range(T):
            S = g[t, h][:, None] * S
            u = beta[t, h] * (v[t, h] - S.T @ k[t, c])
            S = S + np.outer(k[t, c], u)
            o[t, h] = S.T @ q[t, c]
    return o


def delta_rule_mixer(h, w, m, eps):
    """w: 'q', 'q.conv', 'k', 'k.conv', 'v', 'v.conv', 'b', 'A_log', 'norm', 'a1', 'a2', 'dt_bias', 'g1', 'g2', 'o'."""
    T = h.shape[0]
    H, G, dk, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(causal_conv(h @ w["q"].T, w["q.conv"])).reshape(T, G, dk)
    k = silu(causal_conv(h @ w["k"].T, w["k.conv"])).reshape(T, G, dk)
    v = silu(causal_conv(h @ w["v"].T, w["v.conv"])).reshape(T, H, dv)
    q = unit(q) * dk ** -0.5
    k = unit(k)
    beta = sigmoid(h @ w["b"].T)
    rate = softplus((h @ w["a1"].T) @ w["a2"].T + w["dt_bias"]).reshape(T, H, dk)
    g = np.exp(-np.exp(w["A_log"])[None, :, None] * rate)
    o = delta_rule_scan(q, k, v, beta, g)
    o = o / np.sqrt((o * o).mean(axis=-1, keepdims=True) + eps) * w["norm"]
    o = o * sigmoid((h @ w["g1"].T) @ w["g2"].T).reshape(T, H, dv)
    return o.reshape(T, H * dv) @ w["o"].T


# --------------------------------------------------------------------------------------------
# the whole model
# --------------------------------------------------------------------------------------------
def sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def feed_forward(h, w):
    z = h @ w["up"].T + w["up.b"]
    return xielu(z, w["act"][0], w["act"][1]) @ w["down"].T + w["down.b"]


def mixer(h, layer, tensors, prefix, eps):
    m = layer["mixer"]
    if layer["type"] == "mamba2":
        return mamba2_mixer(h, sub(tensors, prefix + "mix."), m, eps)
    if layer["type"] == "parallel":
        left = sigmoid_attention(h, sub(tensors, prefix + "mix.left."), m["left"])
        right = delta_rule_mixer(h, sub(tensors, prefix + "mix.right."), m["right"], eps)
        return m["left_scale"] * left + m["right_scale"] * right
    raise ValueError(layer["type"])


def forward(cfg, tensors, tokens, return_layers=False):
    """Logits [T, vocab] of one sequence from position 0 (and the stream after every layer)."""
    eps = cfg["norm"]["eps"]
    mult = cfg["residual_mult"]
    x = tensors["embed"][np.asarray(tokens)] * cfg["embedding"]["scale"]
    after = []
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        a = mixer(rms_norm(x, tensors[p + "norm1"], eps), layer, tensors, p, eps)
        x = x + mult * rms_norm(a, tensors[p + "norm1b"], eps)
        if layer["mlp"] is not None:
            f = feed_forward(rms_norm(x, tensors[p + "norm2"], eps), sub(tensors, p + "mlp."))
            x = x + mult * rms_norm(f, tensors[p + "norm2b"], eps)
        after.append(x.copy())
    logits = rms_norm(x, tensors["final.norm"], eps) @ tensors["embed"].T
    return (logits, after) if return_layers else logits


def greedy(cfg, tensors, prompt, n_new):
    """The prompt's greedy continuation, recomputing the whole sequence for every token."""
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(np.argmax(forward(cfg, tensors, tokens)[-1])))
    return tokens[len(prompt):]
