"""A plain, slow Sumozen in numpy float64: one function per mechanism, token by token where the
mechanism is a recurrence.  It shares nothing with the package: the tests compare the engine
with it.  ``config`` is the nested dictionary of the model's ``config.json``; ``weights`` maps
tensor names to float64 arrays."""

from __future__ import annotations

import math

import numpy as np


def sigmoid(z):
    return 1.0 / (1.0 + np.exp(-z))


def silu(z):
    return z * sigmoid(z)


def softplus(z):
    return np.logaddexp(0.0, z)


def offset_rms_norm(x, w, eps):
    """Rows over their root mean square, times (1 + w)."""
    return x / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps) * (1.0 + w)


def causal_taps(u, w, bias=None):
    """u [T, C], w [C, taps]: y_t = sum_j w[:, j] u_(t - taps + 1 + j), zeros before the start."""
    n, taps = u.shape[0], w.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, u.shape[1])), u])
    y = np.zeros_like(u)
    for j in range(taps):
        y += padded[j:j + n] * w[:, j]
    return y if bias is None else y + bias


def yarn_frequencies(rot):
    """The per-pair frequencies and the factor both cos and sin are multiplied by."""
    dims, base = rot["dims"], rot["base"]
    i = np.arange(dims // 2, dtype=np.float64)
    f = base ** (-2.0 * i / dims)
    scaling = rot.get("scaling")
    if not scaling:
        return f, 1.0
    factor, original = scaling["factor"], scaling["original"]

    def at(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(at(scaling["fast"])), 0)
    hi = min(math.ceil(at(scaling["slow"])), dims - 1)
    ramp = np.clip((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_interleaved(x, positions, rot):
    """x [T, heads, size]: pairs (2i, 2i+1) among the first rot.dims entries turn by position * f_i."""
    f, amplitude = yarn_frequencies(rot)
    dims = rot["dims"]
    angle = positions[:, None].astype(np.float64) * f[None, :]
    cos, sin = np.cos(angle)[:, None, :] * amplitude, np.sin(angle)[:, None, :] * amplitude
    out = x.copy()
    even, odd = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = even * cos - odd * sin
    out[..., 1:dims:2] = odd * cos + even * sin
    return out


def capped_attention(h, sizes, w, prefix):
    """The softmax side: projections with biases, taps, rotation, capped scores, all earlier keys."""
    n = h.shape[0]
    heads, groups, dim, vdim = sizes["heads"], sizes["kv_heads"], sizes["dim"], sizes["vdim"]
    streams = {}
    for name in ("q", "k", "v"):
        projected = h @ w[f"{prefix}.{name}"].T + w[f"{prefix}.{name}.b"]
        streams[name] = causal_taps(projected, w[f"{prefix}.{name}.conv"])
    positions = np.arange(n)
    q = rotate_interleaved(streams["q"].reshape(n, heads, dim), positions, sizes["rot"])
    k = rotate_interleaved(streams["k"].reshape(n, groups, dim), positions, sizes["rot"])
    v = streams["v"].reshape(n, groups, vdim)
    out = np.zeros((n, heads, vdim))
    cap = sizes.get("softcap")
    visible = np.tril(np.ones((n, n), dtype=bool))
    for head in range(heads):
        g = head // (heads // groups)
        score = (q[:, head] @ k[:, g].T) * sizes["scale"]
        if cap:
            score = cap * np.tanh(score / cap)
        score = np.where(visible, score, -np.inf)
        p = np.exp(score - score.max(axis=1, keepdims=True))
        out[:, head] = (p / p.sum(axis=1, keepdims=True)) @ v[:, g]
    return out.reshape(n, heads * vdim) @ w[f"{prefix}.o"].T + w[f"{prefix}.o.b"]


def gated_delta(h, sizes, w, prefix, eps):
    """The delta-rule side: S <- g S; u = beta (v - S^T k); S <- S + k u^T; o = S^T q."""
    n = h.shape[0]
    heads, groups, dim, vdim = sizes["heads"], sizes["kv_heads"], sizes["dim"], sizes["vdim"]
    q = silu(causal_taps(h @ w[f"{prefix}.q"].T, w[f"{prefix}.q.conv"])).reshape(n, groups, dim)
    k = silu(causal_taps(h @ w[f"{prefix}.k"].T, w[f"{prefix}.k.conv"])).reshape(n, groups, dim)
    v = silu(causal_taps(h @ w[f"{prefix}.v"].T, w[f"{prefix}.v.conv"])).reshape(n, heads, vdim)
    q = q / np.sqrt((q * q).sum(-1, keepdims=True) + 1e-6) * dim ** -0.5
    k = k / np.sqrt((k * k).sum(-1, keepdims=True) + 1e-6)
    beta = sigmoid(h @ w[f"{prefix}.b"].T)
    decay = np.exp(-np.exp(w[f"{prefix}.A_log"]) * softplus(h @ w[f"{prefix}.a"].T + w[f"{prefix}.dt_bias"]))
    gate = silu(h @ w[f"{prefix}.g"].T).reshape(n, heads, vdim)
    state = np.zeros((heads, dim, vdim))
    out = np.zeros((n, heads, vdim))
    for t in range(n):
        for head in range(heads):
            g = head // (heads // groups)
            s = state[head] * decay[t, head]
            u = beta[t, head] * (v[t, head] - s.T @ k[t, g])
            s = s + np.outer(k[t, g], u)
            state[head] = s
            out[t, head] = s.T @ q[t, g]
    out = out / np.sqrt((out * out).mean(-1, keepdims=True) + eps) * w[f"{prefix}.norm"] * gate
    return out.reshape(n, heads * vdim) @ w[f"{prefix}.o"].T


def parallel_mixer(h, mixer, w, prefix, eps):
    left = capped_attention(h, mixer["left"], w, f"{prefix}.left")
    right = gated_delta(h, mixer["right"], w, f"{prefix}.right", eps)
    return mixer["left_scale"] * left + mixer["right_scale"] * right


def state_space(h, sizes, w, prefix, eps):
    """S_t = exp(-exp(A_log) dt) S_(t-1) + dt B_t x_t^T; y_t = S_t^T C_t + D x_t; gate, norm in parts, W_o."""
    n = h.shape[0]
    heads, vdim, state_size, groups = sizes["heads"], sizes["vdim"], sizes["state"], sizes["groups"]
    inner, bc = heads * vdim, groups * state_size
    projected = h @ w[f"{prefix}.in"].T
    z, xbc, dt = projected[:, :inner], projected[:, inner:2 * inner + 2 * bc], projected[:, 2 * inner + 2 * bc:]
    xbc = silu(causal_taps(xbc, w[f"{prefix}.conv"], w[f"{prefix}.conv.b"]))
    x = xbc[:, :inner].reshape(n, heads, vdim)
    b = xbc[:, inner:inner + bc].reshape(n, groups, state_size)
    c = xbc[:, inner + bc:].reshape(n, groups, state_size)
    dt = softplus(dt + w[f"{prefix}.dt_bias"])
    decay = np.exp(-np.exp(w[f"{prefix}.A_log"]) * dt)
    state = np.zeros((heads, state_size, vdim))
    y = np.zeros((n, heads, vdim))
    for t in range(n):
        for head in range(heads):
            g = head // (heads // groups)
            state[head] = decay[t, head] * state[head] + dt[t, head] * np.outer(b[t, g], x[t, head])
            y[t, head] = state[head].T @ c[t, g] + w[f"{prefix}.D"][head] * x[t, head]
    y = y.reshape(n, inner) * silu(z)
    parts = y.reshape(n, sizes["norm_groups"], -1)
    parts = parts / np.sqrt((parts * parts).mean(-1, keepdims=True) + eps)
    return (parts.reshape(n, inner) * w[f"{prefix}.norm"]) @ w[f"{prefix}.o"].T


def gated_expert(x, w, prefix):
    return (silu(x @ w[f"{prefix}.gate"].T) * (x @ w[f"{prefix}.up"].T)) @ w[f"{prefix}.down"].T


def routed_experts(h, mlp, w, prefix):
    """Sigmoid scores, the `top` largest, each expert fed its score times the token."""
    scores = sigmoid(h @ w[f"{prefix}.router"].T)
    out = np.zeros_like(h)
    top = mlp["router"]["top"]
    for t in range(h.shape[0]):
        chosen = np.argsort(-scores[t], kind="stable")[:top]
        for e in chosen:
            out[t] += gated_expert(scores[t, e] * h[t:t + 1], w, f"{prefix}.e{e}")[0]
    if mlp.get("shared"):
        out += gated_expert(h, w, f"{prefix}.shared") * sigmoid(h @ w[f"{prefix}.shared.sg"].T)
    return out


def forward(config, w, tokens, layers_out=None):
    """Logits [T, vocab] of one sequence from its first token on."""
    eps = config["norm"]["eps"]
    x = w["embed"][np.asarray(tokens)]
    for index, layer in enumerate(config["layers"]):
        prefix = f"l{index}"
        h = offset_rms_norm(x, w[f"{prefix}.norm1"], eps)
        if layer["type"] == "parallel":
            x = x + parallel_mixer(h, layer["mixer"], w, f"{prefix}.mix", eps)
        elif layer["type"] == "mamba2":
            x = x + state_space(h, layer["mixer"], w, f"{prefix}.mix", eps)
        else:
            raise ValueError(layer["type"])
        if layer["mlp"] is not None:
            x = x + routed_experts(offset_rms_norm(x, w[f"{prefix}.norm2"], eps), layer["mlp"], w, f"{prefix}.mlp")
        if layers_out is not None:
            layers_out.append(x.copy())
    return offset_rms_norm(x, w["final.norm"], eps) @ w["head"].T


def load_model(folder):
    """(config dictionary, {name: float64 array}) of a model folder; its own small safetensors reader."""
    import json
    import os
    import struct

    with open(os.path.join(folder, "config.json")) as handle:
        config = json.load(handle)
    with open(os.path.join(folder, "model.safetensors"), "rb") as handle:
        data = handle.read()
    (length,) = struct.unpack("<Q", data[:8])
    header = json.loads(data[8:8 + length])
    body = data[8 + length:]
    tensors = {}
    for name, info in header.items():
        if name == "__metadata__":
            continue
        begin, end = info["data_offsets"]
        if info["dtype"] == "F32":
            values = np.frombuffer(body[begin:end], dtype="<f4").astype(np.float64)
        elif info["dtype"] == "BF16":
            values = (np.frombuffer(body[begin:end], dtype="<u2").astype(np.uint32) << 16).view(np.float32).astype(np.float64)
        else:
            raise ValueError(f"{name}: element type {info['dtype']}")
        tensors[name] = values.reshape(info["shape"])
    return config, tensors
