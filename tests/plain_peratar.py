"""A plain, slow implementation of the Peratar design in float64, one function per mechanism.

It shares no code with the engine: it reads the checkpoint's tensors by their names, runs a whole
sequence at once with a dense causal mask, expands every head's keys and values from the latent
(the engine never does) and keeps every layer's result in a Python list.  The tests compare the
engine with it.

Notation: x [T, E] the stream, H heads, d unrotated and r rotated query/key dims, v value dims,
k the latent's rank.
"""
from __future__ import annotations

import math
from typing import Any, Dict, List, Optional, Sequence

import torch

DT = torch.float64


def layer_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    mean = x.mean(-1, keepdim=True)
    var = ((x - mean) ** 2).mean(-1, keepdim=True)
    return (x - mean) / torch.sqrt(var + eps) * weight


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * weight


def rotate_pairs(x: torch.Tensor, positions: torch.Tensor, base: float, dims: int) -> torch.Tensor:
    """x [T, ..., n]: dims 2i, 2i+1 (i < dims/2) turn by positions * base^(-2i/dims); the rest pass."""
    out = x.clone()
    shape = [x.shape[0]] + [1] * (x.dim() - 2)
    for i in range(dims // 2):
        angle = positions.to(DT) * base ** (-2.0 * i / dims)
        c, s = torch.cos(angle).view(shape), torch.sin(angle).view(shape)
        u, w = x[..., 2 * i], x[..., 2 * i + 1]
        out[..., 2 * i] = u * c - w * s
        out[..., 2 * i + 1] = w * c + u * s
    return out


def softplus(z: float) -> float:
    return math.log1p(math.exp(-abs(z))) + max(z, 0.0)


def xielu(z: torch.Tensor, p: float, q: float) -> torch.Tensor:
    positive = softplus(p) * z * z + z / 2
    negative = (0.5 + softplus(q)) * (torch.exp(z) - 1 - z) + z / 2
    return torch.where(z > 0, positive, negative)


def latent_of(h: torch.Tensor, w: Dict[str, torch.Tensor], p: str, m: Dict[str, Any], eps: float,
              positions: torch.Tensor):
    """What a layer with a down projection caches: (normalised latent [T, k], rotated key part [T, r])."""
    down = h @ w[p + "mix.dkv"].T
    k = m["kv_rank"]
    latent = rms_norm(down[:, :k], w[p + "mix.dkv.norm"], eps)
    key_rot = rotate_pairs(down[:, k:], positions, m["rot"]["base"], m["rot"]["dims"])
    return latent, key_rot


def latent_attention(h, w, p, m, latent, key_rot, positions):
    T = h.shape[0]
    H, d, r, v = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    q = (h @ w[p + "mix.q"].T).view(T, H, d + r)
    q_plain = q[..., :d]
    q_rot = rotate_pairs(q[..., d:], positions, m["rot"]["base"], m["rot"]["dims"])
    keys = (latent @ w[p + "mix.uk"].T).view(T, H, d)
    values = (latent @ w[p + "mix.uv"].T).view(T, H, v)
    out = torch.zeros(T, H, v, dtype=DT)
    for head in range(H):
        scores = (q_plain[:, head] @ keys[:, head].T + q_rot[:, head] @ key_rot.T) * m["scale"]
        mask = torch.ones(T, T, dtype=torch.bool).tril()
        scores = scores.masked_fill(~mask, float("-inf"))
        out[:, head] = torch.softmax(scores, dim=-1) @ values[:, head]
    head_gate = torch.sigmoid(h @ w[p + "mix.g"].T)
    return (out * head_gate[..., None]).reshape(T, H * v) @ w[p + "mix.o"].T


def dense_feed_forward(h, w, p):
    a, b = (float(t) for t in w[p + "mlp.act"])
    inner = xielu(h @ w[p + "mlp.up"].T + w[p + "mlp.up.b"], a, b)
    return inner @ w[p + "mlp.down"].T + w[p + "mlp.down.b"]


def gate(h, w, name):
    return torch.sigmoid(h @ w[name].T + w[name + ".b"])


def depth_mix(results: Sequence[torch.Tensor], weights: torch.Tensor) -> torch.Tensor:
    assert len(results) == weights.numel()
    return sum(weights[j] * results[j] for j in range(len(results)))


def forward_states(tensors: Dict[str, torch.Tensor], cfg: Dict[str, Any], tokens: Sequence[int]):
    """(logits [T, V], the stream after every layer's mix [L, T, E], the results X_0 .. X_L)."""
    w = {name: t.to(DT) for name, t in tensors.items()}
    eps = cfg["norm"]["eps"]
    positions = torch.arange(len(tokens))
    x = w["embed"][torch.tensor(list(tokens), dtype=torch.long)]
    results: List[torch.Tensor] = [x]
    cached: Dict[int, Any] = {}
    after = []
    for index, layer in enumerate(cfg["layers"]):
        p = f"l{index}."
        m = layer["mixer"]
        source: Optional[int] = m.get("kv_from")
        if source is None:
            cached[index] = latent_of(x, w, p, m, eps, positions)
            source = index
        latent, key_rot = cached[source]
        mixed = latent_attention(x, w, p, m, latent, key_rot, positions) * gate(x, w, p + "rg1")
        x = x + layer_norm(mixed, w[p + "norm1"], eps)
        if layer.get("mlp") is not None:
            product = dense_feed_forward(x, w, p) * gate(x, w, p + "rg2")
            x = x + layer_norm(product, w[p + "norm2"], eps)
        results.append(x)
        x = depth_mix(results, w[p + "dwa"])
        after.append(x)
    logits = layer_norm(x, w["final.norm"], eps) @ w["head"].T
    cap = cfg.get("logit_softcap")
    if cap is not None:
        logits = cap * torch.tanh(logits / cap)
    return logits, torch.stack(after), results


def forward_logits(tensors, cfg, tokens, dtype=None) -> torch.Tensor:
    return forward_states(tensors, cfg, tokens)[0]
