"""``Redalix`` as a model spec.

Every layer has one RMS norm whose output both of its sublayers read:

    h = norm1(x);   x <- x + mixer(h) + feed_forward(h)          (a layer may have no feed-forward)

with one of three mixers, listed layer by layer in the configuration: ``attention`` (windowed
softmax attention with biases, pair rotation with stretched slow pairs, and a gate per head),
``mamba2`` (a state-space layer) and ``parallel`` (windowed attention without rotation, with a
learned sink per head and the first keys kept behind the window, beside a gated linear
recurrence; each result RMS-normed, half their sum).  The feed-forward is dense (tanh GELU) or a
set of squared-ReLU experts chosen by a table over token ids, plus a shared expert behind a
sigmoid gate.  After the last layer: RMS norm and the head.

This module only maps configuration keys to part parameters and checkpoint names to part
weights.  It has no forward pass.
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

from ..config.model_config import ModelConfig, RedalixConfig, RedalixFeedForwardConfig, WindowAttentionConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSource, WeightSpec

ARCHITECTURE = "Redalix"

# The recurrence's decay is exp(-8 * r * softplus(lam)): a constant of the design.
DECAY_SCALE = 8.0


def _matrix(*sources: TensorSource) -> WeightSpec:
    return WeightSpec(sources=tuple(sources), role="matrix")


def _vector(*sources: TensorSource) -> WeightSpec:
    return WeightSpec(sources=tuple(sources), role="vector")


def _rms(name: str, size: int, eps: float) -> PartSpec:
    return PartSpec(kind="rms", params={"size": size, "eps": eps},
                    weights={"weight": _vector(TensorSource(name, (size,), init="one_plus_normal"))})


def padded_head_dim(attention: WindowAttentionConfig) -> int:
    """The head size the attention kernels run: both of the mixer's sizes fit, in steps of 16."""
    return -(-max(attention.dim, attention.vdim) // 16) * 16


def _attention(prefix: str, a: WindowAttentionConfig, width: int) -> Tuple[dict, Dict[str, WeightSpec]]:
    params = {
        "hidden_size": width, "num_heads": a.heads, "num_kv_heads": a.kv_heads, "head_dim": padded_head_dim(a),
        "key_dim": a.dim, "value_dim": a.vdim, "window": a.window, "keep_first": a.keep_first,
        "softmax_scale": a.scale, "qkv_bias": a.biases, "sink": a.sink, "head_gate": a.head_gate,
    }
    weights = {
        "q.weight": _matrix(TensorSource(prefix + "q", (a.heads * a.dim, width))),
        "k.weight": _matrix(TensorSource(prefix + "k", (a.kv_heads * a.dim, width))),
        "v.weight": _matrix(TensorSource(prefix + "v", (a.kv_heads * a.vdim, width))),
        "out.weight": _matrix(TensorSource(prefix + "o", (width, a.heads * a.vdim))),
    }
    if a.biases:
        weights["q.bias"] = _vector(TensorSource(prefix + "q.b", (a.heads * a.dim,)))
        weights["k.bias"] = _vector(TensorSource(prefix + "k.b", (a.kv_heads * a.dim,)))
        weights["v.bias"] = _vector(TensorSource(prefix + "v.b", (a.kv_heads * a.vdim,)))
    if a.sink:
        weights["sink"] = _vector(TensorSource(prefix + "sink", (a.heads,)))
    if a.head_gate:
        weights["gate.weight"] = _matrix(TensorSource(prefix + "g", (a.heads, width)))
    return params, weights


def _feed_forward(prefix: str, f: RedalixFeedForwardConfig, width: int, vocab: int) -> PartSpec:
    if f.kind == "dense":
        return PartSpec(
            kind="dense_act",
            params={"hidden_size": width, "intermediate_size": f.ff, "activation": "gelu_tanh"},
            weights={"up.weight": _matrix(TensorSource(prefix + "up", (f.ff, width))),
                     "down.weight": _matrix(TensorSource(prefix + "down", (width, f.ff)))},
        )
    X, F = f.experts, f.expert_ff
    params = {"hidden_size": width, "experts": X, "top": f.top, "expert_ff": F, "vocab_size": vocab}
    weights = {
        "up.weight": _matrix(*(TensorSource(f"{prefix}e{e}.up", (F, width)) for e in range(X))),
        "down.weight": _matrix(*(TensorSource(f"{prefix}e{e}.down", (width, F)) for e in range(X))),
        "table": WeightSpec(sources=(TensorSource(prefix + "table", (vocab, f.top), init=f"distinct_below:{X}"),),
                            role="table"),
    }
    if f.shared_ff is not None:
        params["shared"] = {"hidden_size": width, "intermediate_size": f.shared_ff, "activation": "relu_squared",
                            "gate_rows": 1}
        weights["shared.up.weight"] = _matrix(TensorSource(prefix + "shared.up", (f.shared_ff, width)),
                                              TensorSource(prefix + "shared.sg", (1, width)))
        weights["shared.down.weight"] = _matrix(TensorSource(prefix + "shared.down", (width, f.shared_ff)))
    return PartSpec(kind="table_experts", params=params, weights=weights)


def build_redalix_spec(config: ModelConfig) -> ModelSpec:
    if not isinstance(config, RedalixConfig):
        raise TypeError(f"expected a RedalixConfig, got {type(config).__name__}")
    c = config
    E, V = c.hidden_size, c.vocab_size
    positions: Dict[tuple, PartSpec] = {}

    def position(key: tuple, make) -> PartSpec:
        if key not in positions:
            positions[key] = make()
        return positions[key]

    layers = []
    for index, layer in enumerate(c.layers):
        p = f"l{index}.mix."
        pos: Optional[PartSpec] = None
        if layer.type == "attention":
            a = layer.left
            base, dims, scaling = a.rot
            params, weights = _attention(p, a, E)
            mixer = PartSpec(kind="attention", params=params, weights=weights)
            D = padded_head_dim(a)
            pos = position(("rot", base, dims, scaling, D), lambda: PartSpec(
                kind="rotary_interleaved",
                params={"rotary_dim": dims, "base": base, "max_position": c.max_position_embeddings, "head_dim": D,
                        "scaling": None if scaling is None else dict(zip(("factor", "original", "fast", "slow"), scaling))}))
        elif layer.type == "mamba2":
            s = layer.state_space
            inner, C = s.heads * s.vdim, s.heads * s.vdim + 2 * s.groups * s.state
            mixer = PartSpec(
                kind="state_space",
                params={"hidden_size": E, "heads": s.heads, "value_dim": s.vdim, "state_size": s.state,
                        "groups": s.groups, "norm_groups": s.norm_groups, "conv_taps": s.conv, "eps": c.norm_eps},
                weights={
                    "in.weight": _matrix(TensorSource(p + "in", (inner + C + s.heads, E))),
                    "conv.weight": _vector(TensorSource(p + "conv", (C, s.conv), init="normal_wide")),
                    "conv.bias": _vector(TensorSource(p + "conv.b", (C,))),
                    "dt_bias": _vector(TensorSource(p + "dt_bias", (s.heads,))),
                    "a_log": _vector(TensorSource(p + "A_log", (s.heads,))),
                    "d": _vector(TensorSource(p + "D", (s.heads,), init="one_plus_normal")),
                    "norm.weight": _vector(TensorSource(p + "norm", (inner,), init="one_plus_normal")),
                    "out.weight": _matrix(TensorSource(p + "o", (E, inner))),
                },
            )
        else:
            a, r = layer.left, layer.right
            left_params, left_weights = _attention(p + "left.", a, E)
            part = r.width // r.blocks
            W = r.width
            right_weights = {
                "in.weight": _matrix(TensorSource(p + "right.y", (W, E)), TensorSource(p + "right.x", (W, E))),
                "in.bias": _vector(TensorSource(p + "right.y.b", (W,)), TensorSource(p + "right.x.b", (W,))),
                "conv.weight": _vector(TensorSource(p + "right.conv", (W, r.conv), init="normal_wide")),
                "conv.bias": _vector(TensorSource(p + "right.conv.b", (W,))),
                "gate_a.weight": _vector(TensorSource(p + "right.ra", (r.blocks, part, part), init="normal_wide")),
                "gate_a.bias": _vector(TensorSource(p + "right.ra.b", (r.blocks, part))),
                "gate_i.weight": _vector(TensorSource(p + "right.ri", (r.blocks, part, part), init="normal_wide")),
                "gate_i.bias": _vector(TensorSource(p + "right.ri.b", (r.blocks, part))),
                "lam": _vector(TensorSource(p + "right.lam", (W,))),
                "out.weight": _matrix(TensorSource(p + "right.o", (E, W))),
            }
            weights = {"left." + k: v for k, v in left_weights.items()}
            weights.update({"right." + k: v for k, v in right_weights.items()})
            weights["left.out_norm"] = _vector(TensorSource(p + "left.out", (E,), init="one_plus_normal"))
            weights["right.out_norm"] = _vector(TensorSource(p + "right.out", (E,), init="one_plus_normal"))
            mixer = PartSpec(
                kind="side_by_side",
                params={
                    "hidden_size": E, "eps": c.norm_eps, "scale": 0.5,
                    "left": {"kind": "attention", "params": left_params},
                    "right": {"kind": "gated_linear_recurrence",
                              "params": {"hidden_size": E, "width": W, "blocks": r.blocks, "conv_taps": r.conv,
                                         "decay_scale": DECAY_SCALE, "branch_activation": "gelu_tanh"}},
                },
                weights=weights,
            )
            D = padded_head_dim(a)
            pos = position(("none", D), lambda: PartSpec(kind="none", params={"head_dim": D}))
        feed_forward = None if layer.mlp is None else _feed_forward(f"l{index}.mlp.", layer.mlp, E, V)
        layers.append(LayerSpec(block="parallel", mixer=mixer, feed_forward=feed_forward,
                                norms={"input": _rms(f"l{index}.norm1", E, c.norm_eps)}, position=pos))
    spec = ModelSpec(
        architecture=c.architecture,
        hidden_size=E,
        vocab_size=V,
        max_position=c.max_position_embeddings,
        embedding=PartSpec(kind="token_embedding", params={"vocab_size": V, "hidden_size": E},
                           weights={"weight": _matrix(TensorSource("embed", (V, E)))}),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(layer=i) for i in range(len(layers))),
        final_norm=_rms("final.norm", E, c.norm_eps),
        lm_head=PartSpec(kind="linear_head", params={"hidden_size": E, "vocab_size": V},
                         weights={"weight": _matrix(TensorSource("head", (V, E)))}),
        eos_token_ids=tuple(c.eos_token_ids),
    )
    spec.validate()
    return spec


register_architecture(ARCHITECTURE, RedalixConfig.from_dict, build_redalix_spec)
