"""Plain, slow implementation of the Fobilorn decoder: whole sequences, no cache, no batching.

One function per mechanism, numpy float64 throughout, written from the design's equations and
sharing no code with the product package (model folders are read with the `safetensors` package).

Notation: x is the residual stream [T, D]; h the normed input of a layer's two sublayers; H query
heads, G key/value heads, dk the query/key size of a head and dv its value size.
"""
from __future__ import annotations

import json
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


def rms_unit(x, eps):
    """x divided by its root mean square over the last axis, eps inside the root."""
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)


def dynamic_tanh(x, weight, bias, alpha):
    """The norm without statistics: tanh(alpha x) * weight + bias, alpha a scalar."""
    return np.tanh(float(alpha) * x) * weight + bias


# --------------------------------------------------------------------------------------------
# embedding
# --------------------------------------------------------------------------------------------
def bigram_rows(tokens, buckets, mul_prev, mul_cur):
    """Row of the bigram table for every token: a hash of (previous token, token); the first token of a
    sequence takes the table's last row (number `buckets`)."""
    rows = []
    for t, tok in enumerate(tokens):
        rows.append(buckets if t == 0 else (int(tokens[t - 1]) * mul_prev + int(tok) * mul_cur) % buckets)
    return np.asarray(rows, dtype=np.int64)


def embedding(tokens, table, bigram, buckets, mul_prev, mul_cur):
    tokens = np.asarray(tokens, dtype=np.int64)
    return table[tokens] + bigram[bigram_rows(tokens, buckets, mul_prev, mul_cur)]


# --------------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------------
def visible(i, j, window, keep_first):
    """Whether the query at position i sees the key at position j: causal, and either inside the window of
    the latest `window` positions or among the first `keep_first` of the sequence."""
    return j <= i and (i - j < window or j < keep_first)


def sink_softmax(scores, mask):
    """p_j = exp(s_j) / (1 + sum_visible exp(s_j)): a softmax with one more entry of score 0 whose value is
    nothing.  scores, mask [T, T]."""
    s = np.where(mask, scores, -np.inf)
    m = np.maximum(s.max(axis=-1, keepdims=True), 0.0)
    e = np.where(mask, np.exp(s - m), 0.0)
    return e / (np.exp(-m) + e.sum(axis=-1, keepdims=True))


def attend(q, k, v, scale, window, keep_first, sink=True):
    """One head: q [T, dk], k [T, dk], v [T, dv], the row t at position t.  Returns [T, dv]."""
    T = q.shape[0]
    mask = np.array([[visible(i, j, window, keep_first) for j in range(T)] for i in range(T)])
    s = (q @ k.T) * scale
    if sink:
        return sink_softmax(s, mask) @ v
    s = np.where(mask, s, -np.inf)
    e = np.exp(s - s.max(axis=-1, keepdims=True))
    return (e / e.sum(axis=-1, keepdims=True)) @ v


def attention(h, w, spec, eps, v_first=None, mixes=False):
    """The attention mixer on the normed input h [T, D].  `w`: the layer's tensors by short name (q, k, v,
    q.norm, k.norm, vmix, g, o).  `spec`: heads, kv_heads, dim, vdim, scale, mask.size, mask.keep_first.
    `mixes` with `v_first` [T, G dv]: the values are blended with the first blending layer's values of the same
    tokens.  Returns (output [T, D], the values this layer keeps [T, G dv])."""
    T = h.shape[0]
    H, G, dk, dv = spec["heads"], spec["kv_heads"], spec["dim"], spec["vdim"]
    q = h @ w["q"].T
    k = h @ w["k"].T
    v = h @ w["v"].T
    # one root mean square over the whole projection, all heads at once
    q = rms_unit(q, eps) * w["q.norm"]
    k = rms_unit(k, eps) * w["k.norm"]
    if mixes and v_first is not None:
        lam = float(w["vmix"])
        v = (1.0 - lam) * v + lam * v_first
    q = q.reshape(T, H, dk)
    k = k.reshape(T, G, dk)
    vh = v.reshape(T, G, dv)
    window, keep = spec["mask"]["size"], spec["mask"]["keep_first"]
    gate = sigmoid(h @ w["g"].T)                      # [T, H]
    out = np.zeros((T, H, dv))
    for head in range(H):
        kv = head // (H // G)
        out[:, head] = attend(q[:, head], k[:, kv], vh[:, kv], spec["scale"], window, keep) * gate[:, head:head + 1]
    return out.reshape(T, H * dv) @ w["o"].T, v


# --------------------------------------------------------------------------------------------
# feed-forward
# --------------------------------------------------------------------------------------------
def gated_ff(h, gate, up, down):
    return (silu(h @ gate.T) * (h @ up.T)) @ down.T


def route(h, router, top):
    """Chosen experts and their weights: the `top` largest of sigmoid(router h), the weights being those scores
    as they are."""
    s = sigmoid(h @ router.T)
    order = np.argsort(-s, axis=-1, kind="stable")[:, :top]
    return order, np.take_along_axis(s, order, axis=-1)


def moe_ff(h, w, n_experts, top, has_shared, on_input=True):
    """Sum over a token's chosen experts of expert(weight * h), plus the shared expert on h.  (`on_input` False: the
    weight multiplies the expert's output instead, which the design does not do; the product's part has both.)"""
    chosen, weight = route(h, w["router"], top)
    out = np.zeros_like(h)
    for t in range(h.shape[0]):
        for e, s in zip(chosen[t], weight[t]):
            x = s * h[t:t + 1] if on_input else h[t:t + 1]
            y = gated_ff(x, w[f"e{e}.gate"], w[f"e{e}.up"], w[f"e{e}.down"])[0]
            out[t] += y if on_input else s * y
    if has_shared:
        out = out + gated_ff(h, w["shared.gate"], w["shared.up"], w["shared.down"])
    return out


# --------------------------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------------------------
def _sub(tensors, prefix):
    return {k[len(prefix):]: v for k, v in tensors.items() if k.startswith(prefix)}


def _norm(x, tensors, name):
    return dynamic_tanh(x, tensors[name], tensors[name + ".b"], tensors[name + ".alpha"])


def forward(cfg, tensors, tokens, return_layers=False):
    """Logits [T, vocab] of one whole sequence (and the stream after every layer on request)."""
    big = cfg["embedding"]["bigram"]
    x = embedding(tokens, tensors["embed"], tensors["bigram"], big["buckets"], big["mul_prev"], big["mul_cur"])
    x = _norm(x, tensors, "embed.norm")
    eps = cfg["norm"]["eps"]
    v_first = None
    streams = []
    for i, layer in enumerate(cfg["layers"]):
        if layer["type"] != "attention":
            raise ValueError(f"layer {i}: unknown mixer {layer['type']!r}")
        h = _norm(x, tensors, f"l{i}.norm1")
        spec = layer["mixer"]
        mixes = bool(spec.get("v_mix"))
        a, v = attention(h, _sub(tensors, f"l{i}.mix."), spec, eps, v_first, mixes)
        if mixes and v_first is None:
            v_first = v
        mlp = layer.get("mlp")
        f = 0.0
        if mlp is not None:
            w = _sub(tensors, f"l{i}.mlp.")
            if mlp["kind"] == "dense":
                f = gated_ff(h, w["gate"], w["up"], w["down"])
            elif mlp["kind"] == "moe":
                f = moe_ff(h, w, mlp["router"]["experts"], mlp["router"]["top"], mlp.get("shared") is not None)
            else:
                raise ValueError(f"layer {i}: unknown feed-forward {mlp['kind']!r}")
        x = x + (a + f)
        streams.append(x.copy())
    logits = _norm(x, tensors, "final.norm") @ tensors["head"].T
    return (logits, np.stack(streams)) if return_layers else logits
