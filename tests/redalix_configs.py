"""Small Redalix configurations and weights for the tests.

The configurations differ in every size and make sizes differ that a model may happen to make
equal or 1: query/key and value sizes of a head, heads per KV head (1, 2, 3, 4), experts per
token (1, 2, 3), parts of the recurrence (1, 3, 4), groups of the state-space layer and of its
norm, taps of the two convolutions (1 to 5), a shared expert or none, a feed-forward or none,
kept first keys (none, a few, more than the window, more than a page), rotation of all or some
dims with and without stretched pairs, widths that are no multiples of eight.  ``make_weights``
draws weights at a scale at which every mechanism does something: a unit-variance stream, gates
away from 1/2, decays spread between 0 and 1, sinks that take a visible share of the softmax.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Optional

import torch


def attention(heads, kv_heads, dim, vdim, scale, size, keep_first=None, rot=None) -> Dict[str, Any]:
    mask: Dict[str, Any] = {"size": size}
    if keep_first is not None:
        mask["keep_first"] = keep_first
    out = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": vdim, "scale": scale, "mask": mask}
    if rot is not None:
        out["rot"] = rot
    return out


def rotation(base, dims, factor=None, original=None, fast=None, slow=None) -> Dict[str, Any]:
    out: Dict[str, Any] = {"base": base, "dims": dims}
    if factor is not None:
        out["scaling"] = {"factor": factor, "original": original, "fast": fast, "slow": slow}
    return out


def recurrence(width, blocks, conv) -> Dict[str, Any]:
    return {"width": width, "blocks": blocks, "conv": conv}


def state_space(heads, vdim, state, groups, norm_groups, conv) -> Dict[str, Any]:
    return {"heads": heads, "vdim": vdim, "state": state, "groups": groups, "norm_groups": norm_groups, "conv": conv}


def dense(ff) -> Dict[str, Any]:
    return {"kind": "dense", "ff": ff}


def moe(experts, top, ff, shared=None) -> Dict[str, Any]:
    out: Dict[str, Any] = {"kind": "moe", "expert": {"ff": ff}, "router": {"experts": experts, "top": top}}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


def parallel(left, right, mlp) -> Dict[str, Any]:
    return {"type": "parallel", "mixer": {"left": left, "right": right}, "mlp": mlp}


def attn_layer(mix, mlp) -> Dict[str, Any]:
    return {"type": "attention", "mixer": mix, "mlp": mlp}


def mamba_layer(mix, mlp) -> Dict[str, Any]:
    return {"type": "mamba2", "mixer": mix, "mlp": mlp}


def config(width, vocab, layers, eps=1e-5) -> Dict[str, Any]:
    return {"architecture": "Redalix", "vocab": vocab, "width": width, "norm": {"eps": eps}, "layers": layers}


# One layer of each kind; value size above and below the query/key size; three heads on one KV
# head; a layer without feed-forward; stretched pairs on some of the rotating dims.
SMALL = config(64, 120, [
    parallel(attention(4, 2, 16, 24, 0.25, 12, keep_first=3), recurrence(48, 3, 3), dense(40)),
    attn_layer(attention(3, 1, 24, 8, 0.2, 9, rot=rotation(100.0, 16, factor=4.0, original=16, fast=8.0, slow=1.0)),
               moe(5, 2, 24, shared=16)),
    mamba_layer(state_space(4, 8, 12, 2, 4, 2), None),
], eps=1e-6)

# Sizes of one and widths that are no multiples of eight: one expert per token and no shared
# expert, a recurrence in one part with five taps, one group and one norm group, a convolution of
# one tap, no grouping of heads, no kept keys in one parallel layer and more kept keys than the
# window in the other, a window of one key, rotation without stretching.
ODD = config(100, 331, [
    mamba_layer(state_space(3, 20, 7, 1, 1, 1), moe(3, 1, 17)),
    parallel(attention(2, 2, 20, 12, 0.3, 7, keep_first=0), recurrence(36, 1, 5), moe(4, 3, 12, shared=9)),
    attn_layer(attention(5, 5, 12, 20, 0.3, 1, rot=rotation(50.0, 8)), dense(52)),
    parallel(attention(3, 1, 8, 8, 0.4, 5, keep_first=11), recurrence(44, 4, 2), None),
    attn_layer(attention(4, 2, 16, 16, 0.2, 30, rot=rotation(10000.0, 16, factor=2.0, original=8, fast=4.0, slow=0.5)),
               moe(6, 2, 20, shared=24)),
], eps=1e-5)

# Heads of 64 and 128: prompt portions on the tensor-memory attention kernels; windows and kept
# keys longer than a page and a key tile; a state of 64 x 32 per head.
WIDE = config(256, 500, [
    parallel(attention(8, 2, 64, 64, 0.125, 150, keep_first=70), recurrence(256, 4, 4), moe(8, 2, 64, shared=128)),
    attn_layer(attention(4, 1, 128, 96, 0.09, 200, rot=rotation(1000000.0, 64, factor=8.0, original=128, fast=32.0,
                                                                  slow=1.0)), dense(384)),
    mamba_layer(state_space(8, 32, 64, 2, 2, 4), moe(8, 2, 64)),
    parallel(attention(4, 4, 64, 32, 0.125, 64, keep_first=64), recurrence(128, 2, 4), dense(256)),
], eps=2e-5)

ALL = {"small": SMALL, "odd": ODD, "wide": WIDE}


def make_weights(cfg: Dict[str, Any], seed: int, sharp: float = 1.0) -> Dict[str, torch.Tensor]:
    """Tensors under the checkpoint's names, bfloat16 (tables int32).  ``sharp`` scales the query
    projections: at 3 or more the softmax puts most of its weight on a few keys."""
    from velox_b200.config.registry import architecture_of

    arch = architecture_of(cfg)
    spec = arch.build_spec(arch.parse_config(cfg))
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, source in sorted(spec.checkpoint_tensors().items()):
        shape = tuple(source.shape)
        last = name.rsplit(".", 1)[-1]
        if last == "table":
            bound = int(source.init.split(":")[1])
            out[name] = torch.rand((shape[0], bound), generator=gen).argsort(dim=1)[:, : shape[1]].to(torch.int32).contiguous()
            continue
        if name == "embed":
            t = torch.randn(shape, generator=gen)
        elif last in ("norm1", "norm", "out") and len(shape) == 1:
            t = 1.0 + 0.3 * torch.randn(shape, generator=gen)
        elif last in ("ra", "ri"):
            t = 1.5 * torch.randn(shape, generator=gen) / shape[-1] ** 0.5
        elif last == "conv":
            t = torch.randn(shape, generator=gen) / shape[-1] ** 0.5
        elif last == "lam":
            t = 1.5 * torch.randn(shape, generator=gen) - 1.0
        elif last == "A_log":
            t = 0.7 * torch.randn(shape, generator=gen) - 0.5
        elif last == "dt_bias":
            t = torch.randn(shape, generator=gen) - 1.0
        elif last == "D":
            t = 1.0 + 0.3 * torch.randn(shape, generator=gen)
        elif last == "sink":
            t = 1.0 + torch.randn(shape, generator=gen)
        elif len(shape) == 1 or last == "b":
            t = 0.5 * torch.randn(shape, generator=gen)
        else:
            t = torch.randn(shape, generator=gen) / shape[-1] ** 0.5
            if last == "q":
                t = t * sharp
            if last == "sg":
                t = t * 2.0
        out[name] = t.to(torch.bfloat16)
    return out


def write_folder(folder: str, cfg: Dict[str, Any], tensors: Dict[str, torch.Tensor]) -> None:
    from safetensors.torch import save_file

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as handle:
        json.dump(cfg, handle)
    save_file({k: v.contiguous() for k, v in tensors.items()}, os.path.join(folder, "model.safetensors"))


def as_numpy(tensors: Dict[str, torch.Tensor]):
    return {k: (v.numpy() if v.dtype == torch.int32 else v.float().numpy()) for k, v in tensors.items()}
