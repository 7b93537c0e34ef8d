"""A plain, slow Fuvolix in numpy: whole sequences, no cache, one function per mechanism.

Fuvolix is a decoder-only stack whose layers each pick one of three token mixers (attention
over a low-rank latent with a shared rotated key part, a gated matrix memory with a
stabilised exponential input gate, a matrix memory with a fixed decay per head), optionally
followed by a squared-relu feed-forward.  Every sublayer is normed on the way in and on the
way out, the mixer's input first passes a short causal convolution over time, and what a
layer hands on is a learned weighted sum of the embedding output and of all layer results so
far.

This file is the yardstick of the tests and shares no code with ``mini_llm_b200``: its own
reader of the weights file (``plain_gpt2.read_safetensors``, also test code) and its own
formulas, in float64.  Sequences are run token by token where the mechanism is a recurrence.
"""

from __future__ import annotations

import json
import math
import os

import numpy as np

from plain_gpt2 import read_safetensors


def load_model(folder):
    with open(os.path.join(folder, "config.json")) as handle:
        config = json.load(handle)
    return config, read_safetensors(os.path.join(folder, "model.safetensors"))


# ---- small pieces ----------------------------------------------------------------------------

def rms(x, eps):
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)


def grouped_rms_norm(x, weight, groups, eps):
    """The width is cut into ``groups`` equal consecutive pieces; each piece is divided by its
    own root mean square; the gain spans the whole width."""
    rows, width = x.shape
    pieces = x.reshape(rows, groups, width // groups)
    return rms(pieces, eps).reshape(rows, width) * weight


def causal_taps(h, weight):
    """h + conv(h): per channel c, conv_t = sum_j weight[c, j] * h[t - (taps - 1) + j, c], with
    zeros before the first token."""
    n, width = h.shape
    taps = weight.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, width)), h])
    out = h.copy()
    for j in range(taps):
        out += padded[j:j + n] * weight[:, j]
    return out


def rotate_pairs(x, positions, base, dims):
    """Rotary positions, interleaved layout: within the first ``dims`` entries of the last axis,
    (x[2i], x[2i+1]) turns by the angle position * base^(-2i/dims)."""
    out = x.copy()
    half = dims // 2
    freq = base ** (-2.0 * np.arange(half) / dims)
    angle = np.asarray(positions, dtype=np.float64)[:, None] * freq[None, :]
    shape = [len(positions)] + [1] * (x.ndim - 2) + [half]
    cos, sin = np.cos(angle).reshape(shape), np.sin(angle).reshape(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def log_sigmoid(z):
    return -np.logaddexp(0.0, -z)


def silu(z):
    return z * sigmoid(z)


# ---- the mixers ------------------------------------------------------------------------------

def latent_attention(h, t, p, sizes, eps):
    """Attention whose keys and values are expanded from a normed latent of rank ``kv_rank``;
    every head's key also has ``rot_dim`` rotated entries that all heads share."""
    n = h.shape[0]
    heads, dim, rot, vdim, rank = sizes["heads"], sizes["dim"], sizes["rot_dim"], sizes["vdim"], sizes["kv_rank"]
    positions = np.arange(n)
    q = (h @ t[p + "q"].T).reshape(n, heads, dim + rot)
    down = h @ t[p + "dkv"].T
    latent = rms(down[:, :rank], eps) * t[p + "dkv.norm"]
    shared = rotate_pairs(down[:, rank:], positions, sizes["rot"]["base"], sizes["rot"]["dims"])
    q_plain = q[:, :, :dim]
    q_turned = rotate_pairs(q[:, :, dim:], positions, sizes["rot"]["base"], sizes["rot"]["dims"])
    keys = (latent @ t[p + "uk"].T).reshape(n, heads, dim)
    values = (latent @ t[p + "uv"].T).reshape(n, heads, vdim)
    mixed = np.zeros((n, heads, vdim))
    for head in range(heads):
        scores = (q_plain[:, head] @ keys[:, head].T + q_turned[:, head] @ shared.T) * sizes["scale"]
        scores = np.where(np.tril(np.ones((n, n), dtype=bool)), scores, -np.inf)
        scores -= scores.max(axis=1, keepdims=True)
        weights = np.exp(scores)
        weights /= weights.sum(axis=1, keepdims=True)
        mixed[:, head] = weights @ values[:, head]
    return mixed.reshape(n, heads * vdim) @ t[p + "o"].T


def gated_matrix_memory(h, t, p, sizes, eps):
    """mLSTM: per head a matrix S and a vector n, both scaled down by a running maximum m of
    the log gates (m starts at 0)."""
    n_tok = h.shape[0]
    heads, dim, vdim, cap = sizes["heads"], sizes["dim"], sizes["vdim"], sizes["gate_cap"]
    q = (h @ t[p + "q"].T).reshape(n_tok, heads, dim) * dim ** -0.5
    k = (h @ t[p + "k"].T).reshape(n_tok, heads, dim)
    v = (h @ t[p + "v"].T).reshape(n_tok, heads, vdim)
    log_in = cap * np.tanh((h @ t[p + "i"].T + t[p + "i.b"]) / cap)
    log_keep = log_sigmoid(cap * np.tanh((h @ t[p + "f"].T + t[p + "f.b"]) / cap))
    out = np.zeros((n_tok, heads, vdim))
    for head in range(heads):
        S = np.zeros((dim, vdim))
        norm = np.zeros(dim)
        m = 0.0
        for step in range(n_tok):
            m_new = max(log_keep[step, head] + m, log_in[step, head])
            keep = math.exp(log_keep[step, head] + m - m_new)
            take = math.exp(log_in[step, head] - m_new)
            S = keep * S + take * np.outer(k[step, head], v[step, head])
            norm = keep * norm + take * k[step, head]
            m = m_new
            bottom = max(abs(norm @ q[step, head]), math.exp(-m)) + 1e-6
            out[step, head] = (S.T @ q[step, head]) / bottom
    out = rms(out, eps).reshape(n_tok, heads * vdim) * t[p + "norm"]
    return (out * sigmoid(h @ t[p + "g"].T)) @ t[p + "o"].T


def decaying_matrix_memory(h, t, p, sizes, eps):
    """Lightning attention as a recurrence: S <- decay_head * S + k v^T, out = S^T q."""
    n_tok = h.shape[0]
    heads, dim, vdim = sizes["heads"], sizes["dim"], sizes["vdim"]
    q = silu(h @ t[p + "q"].T).reshape(n_tok, heads, dim)
    k = silu(h @ t[p + "k"].T).reshape(n_tok, heads, dim)
    v = silu(h @ t[p + "v"].T).reshape(n_tok, heads, vdim)
    out = np.zeros((n_tok, heads, vdim))
    for head in range(heads):
        S = np.zeros((dim, vdim))
        for step in range(n_tok):
            S = sizes["decay"][head] * S + np.outer(k[step, head], v[step, head])
            out[step, head] = S.T @ q[step, head]
    out = rms(out.reshape(n_tok, heads * vdim), eps) * t[p + "norm"]
    return (out * sigmoid(h @ t[p + "g"].T)) @ t[p + "o"].T


MIXERS = {"latent_attention": latent_attention, "mlstm": gated_matrix_memory, "lightning": decaying_matrix_memory}


def squared_relu_mlp(h, t, p):
    up = np.maximum(h @ t[p + "up"].T, 0.0)
    return (up * up) @ t[p + "down"].T


# ---- the model -------------------------------------------------------------------------------

def forward(config, t, tokens, streams=None):
    """Logits [len, vocab].  ``streams`` (a list) receives what each layer hands on."""
    eps, groups = config["norm"]["eps"], config["norm"]["groups"]
    norm = lambda x, name: grouped_rms_norm(x, t[name], groups, eps)
    x = norm(t["embed"][np.asarray(tokens)], "embed.norm")
    results = [x]
    for index, layer in enumerate(config["layers"]):
        p = f"l{index}."
        h = causal_taps(norm(x, p + "norm1"), t[p + "canon1"])
        x = x + norm(MIXERS[layer["type"]](h, t, p + "mix.", layer["mixer"], eps), p + "norm1b")
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError(f"feed-forward kind {layer['mlp']['kind']!r} is not part of the plain model")
            x = x + norm(squared_relu_mlp(norm(x, p + "norm2"), t, p + "mlp."), p + "norm2b")
        results.append(x)
        x = sum(w * r for w, r in zip(t[p + "dwa"], results))
        if streams is not None:
            streams.append(x)
    return norm(x, "final.norm") @ t["embed"].T
