"""``Peratar`` as a model spec.

A decoder-only model whose every layer is

    x <- x + norm1(sigmoid(W_rg1 x + b) * latent_attention(x))
    x <- x + norm2(sigmoid(W_rg2 x + b) * dense_xielu(x))          (a layer may have no feed-forward)

with weight-only layer norms on the sublayers' results, and whose layer e + 1 reads
``sum_{j <= e+1} dwa_e[j] X_j`` over the results X_j of all layers so far (X_0 the embedding
output) instead of the last result alone.  The mixer caches a normalised latent and one rotated
key part per token; a layer with ``kv_from`` reads the cache of that earlier layer.  After the
last layer: layer norm, the head, and ``cap * tanh(logits / cap)``.

The gates read the same rows as the sublayer they gate, so their matrices ride along as the
first rows of that sublayer's first projection (``side_rows``): ``in.weight`` of the mixer is
rg1 | q | dkv | g and ``up.weight`` of the feed-forward is rg2 | up, concatenated in that order.

This module only maps configuration keys to part parameters and checkpoint names to part
weights.  It has no forward pass.
"""
from __future__ import annotations

from typing import Dict, Tuple

from ..config.model_config import ModelConfig, PeratarConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry, TensorSource, WeightSpec

ARCHITECTURE = "Peratar"


def _matrix(*sources: TensorSource) -> WeightSpec:
    return WeightSpec(sources=tuple(sources), role="matrix")


def _vector(*sources: TensorSource) -> WeightSpec:
    return WeightSpec(sources=tuple(sources), role="vector")


def _layer_norm(name: str, size: int, eps: float) -> PartSpec:
    return PartSpec(
        kind="layer_norm",
        params={"size": size, "eps": eps},
        weights={"weight": _vector(TensorSource(name, (size,), init="one_plus_normal"))},
    )


def build_peratar_spec(config: ModelConfig) -> ModelSpec:
    if not isinstance(config, PeratarConfig):
        raise TypeError(f"expected a PeratarConfig, got {type(config).__name__}")
    c = config
    E, V, L = c.hidden_size, c.vocab_size, len(c.layers)
    positions: Dict[Tuple[int, float], PartSpec] = {}
    layers = []
    for index, layer in enumerate(c.layers):
        p = f"l{index}."
        m = layer.mixer
        H = m.heads
        own = m.kv_from is None
        position = positions.get((m.rot_dims, m.rot_base))
        if position is None:
            position = PartSpec(
                kind="rotary_interleaved",
                params={"rotary_dim": m.rot_dims, "base": m.rot_base, "max_position": c.max_position_embeddings},
            )
            positions[(m.rot_dims, m.rot_base)] = position
        sources = [TensorSource(p + "rg1", (E, E)), TensorSource(p + "mix.q", (H * (m.dim + m.rot_dim), E))]
        if own:
            sources.append(TensorSource(p + "mix.dkv", (m.kv_rank + m.rot_dim, E)))
        sources.append(TensorSource(p + "mix.g", (H, E)))
        mixer_weights = {
            "in.weight": _matrix(*sources),
            "side.bias": _vector(TensorSource(p + "rg1.b", (E,))),
            "uk.weight": _matrix(TensorSource(p + "mix.uk", (H * m.dim, m.kv_rank))),
            "uv.weight": _matrix(TensorSource(p + "mix.uv", (H * m.vdim, m.kv_rank))),
            "out.weight": _matrix(TensorSource(p + "mix.o", (E, H * m.vdim))),
        }
        if own:
            mixer_weights["latent_norm.weight"] = _vector(
                TensorSource(p + "mix.dkv.norm", (m.kv_rank,), init="one_plus_normal"))
        mixer = PartSpec(
            kind="latent_attention",
            params={
                "hidden_size": E, "num_heads": H, "dim": m.dim, "rot_dim": m.rot_dim, "value_dim": m.vdim,
                "kv_rank": m.kv_rank, "softmax_scale": m.scale, "eps": c.norm_eps, "own_latent": own,
                "output_gate": True, "side_rows": E,
            },
            weights=mixer_weights,
        )
        norms = {"mixer": _layer_norm(p + "norm1", E, c.norm_eps)}
        feed_forward = None
        if layer.ff is not None:
            F = layer.ff
            feed_forward = PartSpec(
                kind="dense_xielu",
                params={"hidden_size": E, "intermediate_size": F, "side_rows": E},
                weights={
                    "up.weight": _matrix(TensorSource(p + "rg2", (E, E)), TensorSource(p + "mlp.up", (F, E))),
                    "up.bias": _vector(TensorSource(p + "rg2.b", (E,)), TensorSource(p + "mlp.up.b", (F,))),
                    "down.weight": _matrix(TensorSource(p + "mlp.down", (E, F))),
                    "down.bias": _vector(TensorSource(p + "mlp.down.b", (E,))),
                    "act": _vector(TensorSource(p + "mlp.act", (2,))),
                },
            )
            norms["feed_forward"] = _layer_norm(p + "norm2", E, c.norm_eps)
        layers.append(
            LayerSpec(
                block="post_norm",
                mixer=mixer,
                feed_forward=feed_forward,
                norms=norms,
                position=position,
                block_params={"depth_mix": True, "num_entries": L},
                block_weights={
                    "depth_mix.weight": _vector(TensorSource(p + "dwa", (index + 2,), init="average_plus_normal")),
                },
            )
        )
    spec = ModelSpec(
        architecture=c.architecture,
        hidden_size=E,
        vocab_size=V,
        max_position=c.max_position_embeddings,
        embedding=PartSpec(
            kind="token_embedding",
            params={"vocab_size": V, "hidden_size": E},
            weights={"weight": _matrix(TensorSource("embed", (V, E)))},
        ),
        layers=tuple(layers),
        schedule=tuple(ScheduleEntry(layer=i, cache_of=layer.mixer.kv_from) for i, layer in enumerate(c.layers)),
        final_norm=_layer_norm("final.norm", E, c.norm_eps),
        lm_head=PartSpec(
            kind="linear_head",
            params={"hidden_size": E, "vocab_size": V, "softcap": c.logit_softcap},
            weights={"weight": _matrix(TensorSource("head", (V, E)))},
        ),
        eos_token_ids=tuple(c.eos_token_ids),
    )
    spec.validate()
    return spec


register_architecture(ARCHITECTURE, PeratarConfig.from_dict, build_peratar_spec)
