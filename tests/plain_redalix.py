"""A plain, slow implementation of the Redalix design in float64, one function per mechanism.

It shares nothing with the engine: dense masks, explicit loops over tokens for every recurrence,
weights in a dict by checkpoint name, the configuration as the nested dict of config.json.
Everything works on one whole sequence [T, width]; there is no cache and no state to carry.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import numpy as np


def rms_norm(x: np.ndarray, weight: Optional[np.ndarray], eps: float) -> np.ndarray:
    y = x / np.sqrt(np.mean(x * x, axis=-1, keepdims=True) + eps)
    return y if weight is None else y * weight


def gelu_tanh(z: np.ndarray) -> np.ndarray:
    return 0.5 * z * (1.0 + np.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def relu_squared(z: np.ndarray) -> np.ndarray:
    return np.square(np.maximum(z, 0.0))


def sigmoid(z: np.ndarray) -> np.ndarray:
    return 1.0 / (1.0 + np.exp(-z))


def softplus(z: np.ndarray) -> np.ndarray:
    return np.maximum(z, 0.0) + np.log1p(np.exp(-np.abs(z)))


def silu(z: np.ndarray) -> np.ndarray:
    return z * sigmoid(z)


def visible(num_tokens: int, size: int, keep_first: int = 0) -> np.ndarray:
    """mask[i, j]: query i sees key j (causal, a window of ``size`` keys, the first
    ``keep_first`` keys always)."""
    i = np.arange(num_tokens)[:, None]
    j = np.arange(num_tokens)[None, :]
    return (j <= i) & ((i - j < size) | (j < keep_first))


def yarn_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """(frequency per pair, factor on cos and sin)."""
    half = dims // 2
    freq = np.array([base ** (-2.0 * i / dims) for i in range(half)], dtype=np.float64)
    if not scaling:
        return freq, 1.0
    factor, original = float(scaling["factor"]), float(scaling["original"])

    def turn_dim(turns: float) -> float:
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(scaling["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(scaling["slow"]))), dims - 1)
    ramp = np.clip((np.arange(half) - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return freq / factor * ramp + freq * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x: np.ndarray, positions: np.ndarray, rot: Optional[dict]) -> np.ndarray:
    """x [T, heads, dim]: neighbouring pairs of the first rot.dims dims turn by position * f_i."""
    if not rot:
        return x
    dims = int(rot["dims"])
    freq, mscale = yarn_frequencies(dims, float(rot["base"]), rot.get("scaling"))
    angle = positions[:, None].astype(np.float64) * freq[None, :]
    cos, sin = np.cos(angle)[:, None, :] * mscale, np.sin(angle)[:, None, :] * mscale
    out = x.copy()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * cos - v * sin
    out[..., 1:dims:2] = v * cos + u * sin
    return out


def causal_conv(x: np.ndarray, weight: np.ndarray, bias: np.ndarray) -> np.ndarray:
    """x [T, C]; weight [C, taps], the last column is the current token's; zeros before the start."""
    T, taps = x.shape[0], weight.shape[1]
    padded = np.concatenate([np.zeros((taps - 1, x.shape[1])), x])
    out = np.tile(bias, (T, 1)).astype(np.float64)
    for k in range(taps):
        out += padded[k : k + T] * weight[:, k]
    return out


def attention(h, W, prefix, cfg, positions) -> np.ndarray:
    """Softmax attention with grouped heads over a windowed causal mask; optional biases,
    pair rotation, sink in the denominator and per-head output gate."""
    T = h.shape[0]
    H, G, dim, vdim = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]

    def proj(name):
        y = h @ W[prefix + name].T
        if prefix + name + ".b" in W:
            y = y + W[prefix + name + ".b"]
        return y

    q = proj("q").reshape(T, H, dim)
    k = proj("k").reshape(T, G, dim)
    v = proj("v").reshape(T, G, vdim)
    q = rotate_pairs(q, positions, cfg.get("rot"))
    k = rotate_pairs(k, positions, cfg.get("rot"))
    mask = visible(T, int(cfg["mask"]["size"]), int(cfg["mask"].get("keep_first", 0)))
    sink = W.get(prefix + "sink")
    out = np.zeros((T, H, vdim))
    for head in range(H):
        g = head // (H // G)
        s = (q[:, head] @ k[:, g].T) * cfg["scale"]
        s = np.where(mask, s, -np.inf)
        m = s.max(axis=-1, keepdims=True)
        if sink is not None:
            m = np.maximum(m, sink[head])
        p = np.exp(s - m)
        denom = p.sum(axis=-1, keepdims=True)
        if sink is not None:
            denom = denom + np.exp(sink[head] - m)
        out[:, head] = (p / denom) @ v[:, g]
    if prefix + "g" in W:
        out = out * sigmoid(h @ W[prefix + "g"].T)[:, :, None]
    return out.reshape(T, H * vdim) @ W[prefix + "o"].T


def gated_recurrence(h, W, prefix, cfg) -> np.ndarray:
    """Two branches; the second goes through a short convolution and a linear recurrence whose
    decay and input gate come from block-diagonal matrices."""
    T = h.shape[0]
    width, blocks = cfg["width"], cfg["blocks"]
    y = gelu_tanh(h @ W[prefix + "y"].T + W[prefix + "y.b"])
    u = causal_conv(h @ W[prefix + "x"].T + W[prefix + "x.b"], W[prefix + "conv"], W[prefix + "conv.b"])
    part = width // blocks
    ub = u.reshape(T, blocks, part)
    r = sigmoid(np.einsum("boi,tbi->tbo", W[prefix + "ra"], ub) + W[prefix + "ra.b"]).reshape(T, width)
    i = sigmoid(np.einsum("boi,tbi->tbo", W[prefix + "ri"], ub) + W[prefix + "ri.b"]).reshape(T, width)
    log_a = -8.0 * r * softplus(W[prefix + "lam"])
    a = np.exp(log_a)
    state = np.zeros(width)
    out = np.zeros((T, width))
    for t in range(T):
        state = a[t] * state + np.sqrt(1.0 - a[t] ** 2) * i[t] * u[t]
        out[t] = state
    return (out * y) @ W[prefix + "o"].T


def state_space(h, W, prefix, cfg, eps) -> np.ndarray:
    """Selective state-space mixer with scalar decay per head."""
    T = h.shape[0]
    heads, P, N, groups = cfg["heads"], cfg["vdim"], cfg["state"], cfg["groups"]
    inner = heads * P
    zxbcdt = h @ W[prefix + "in"].T
    z = zxbcdt[:, :inner]
    xbc = zxbcdt[:, inner : 2 * inner + 2 * groups * N]
    dt = zxbcdt[:, 2 * inner + 2 * groups * N :]
    xbc = silu(causal_conv(xbc, W[prefix + "conv"], W[prefix + "conv.b"]))
    x = xbc[:, :inner].reshape(T, heads, P)
    B = xbc[:, inner : inner + groups * N].reshape(T, groups, N)
    C = xbc[:, inner + groups * N :].reshape(T, groups, N)
    dt = softplus(dt + W[prefix + "dt_bias"])
    A = -np.exp(W[prefix + "A_log"])
    y = np.zeros((T, heads, P))
    for head in range(heads):
        g = head // (heads // groups)
        S = np.zeros((N, P))
        for t in range(T):
            S = math.exp(A[head] * dt[t, head]) * S + dt[t, head] * np.outer(B[t, g], x[t, head])
            y[t, head] = S.T @ C[t, g] + W[prefix + "D"][head] * x[t, head]
    y = y.reshape(T, inner) * silu(z)
    parts = cfg["norm_groups"]
    y = rms_norm(y.reshape(T, parts, inner // parts), None, eps).reshape(T, inner) * W[prefix + "norm"]
    return y @ W[prefix + "o"].T


def side_by_side(h, W, prefix, cfg, eps, positions) -> np.ndarray:
    left = attention(h, W, prefix + "left.", cfg["left"], positions)
    right = gated_recurrence(h, W, prefix + "right.", cfg["right"])
    return 0.5 * (rms_norm(left, W[prefix + "left.out"], eps) + rms_norm(right, W[prefix + "right.out"], eps))


def expert(h, W, prefix, act) -> np.ndarray:
    return act(h @ W[prefix + "up"].T) @ W[prefix + "down"].T


def feed_forward(h, W, prefix, cfg, tokens) -> np.ndarray:
    if cfg["kind"] == "dense":
        return expert(h, W, prefix, gelu_tanh)
    top = int(cfg["router"]["top"])
    table = W[prefix + "table"].astype(np.int64)
    out = np.zeros_like(h)
    for t, token in enumerate(tokens):
        for e in table[token]:
            out[t] += expert(h[t : t + 1], W, f"{prefix}e{int(e)}.", relu_squared)[0] / top
    if cfg.get("shared"):
        gate = sigmoid(h @ W[prefix + "shared.sg"].T)
        out += gate * expert(h, W, prefix + "shared.", relu_squared)
    return out


def forward(config: dict, weights: Dict[str, np.ndarray], tokens: List[int], collect: Optional[list] = None) -> np.ndarray:
    """Logits [T, vocab] of one whole sequence; ``collect`` receives the stream after every layer."""
    W = {name: np.asarray(value, dtype=np.float64) for name, value in weights.items()}
    eps = float(config["norm"]["eps"])
    tokens = [int(t) for t in tokens]
    positions = np.arange(len(tokens))
    x = W["embed"][tokens]
    for index, layer in enumerate(config["layers"]):
        p = f"l{index}."
        h = rms_norm(x, W[p + "norm1"], eps)
        kind, cfg = layer["type"], layer["mixer"]
        if kind == "parallel":
            mixed = side_by_side(h, W, p + "mix.", cfg, eps, positions)
        elif kind == "attention":
            mixed = attention(h, W, p + "mix.", cfg, positions)
        elif kind == "mamba2":
            mixed = state_space(h, W, p + "mix.", cfg, eps)
        else:
            raise ValueError(f"unknown layer type {kind!r}")
        if layer.get("mlp"):
            mixed = mixed + feed_forward(h, W, p + "mlp.", layer["mlp"], tokens)
        x = x + mixed
        if collect is not None:
            collect.append(x.copy())
    return rms_norm(x, W["final.norm"], eps) @ W["head"].T
