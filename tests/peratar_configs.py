"""Small Peratar configurations and weights for the tests.

The configurations differ in every size; some make sizes differ that a model may happen to make
equal (the rotated width and the number of dims that rotate, the sizes of different layers), have
a layer without feed-forward, a single head, cached rows that need padding, inner sizes that
are no multiple of eight.  ``make_weights`` draws weights at a scale at which the model does
something (a unit-variance stream, gates away from 1/2) and can sharpen the attention so that a
key that is lost or wrongly seen changes the logits visibly.
"""
from __future__ import annotations

import json
import os
from typing import Any, Dict, Optional

import torch


def mixer(heads, dim, rot_dim, vdim, kv_rank, scale, base=10000.0, rot_dims=None, kv_from=None) -> Dict[str, Any]:
    out = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank, "scale": scale,
           "rot": {"base": base, "dims": rot_dim if rot_dims is None else rot_dims}}
    if kv_from is not None:
        out["kv_from"] = kv_from
    return out


def layer(mix, ff: Optional[int]) -> Dict[str, Any]:
    return {"type": "latent_attention", "mixer": mix, "mlp": None if ff is None else {"kind": "dense", "ff": ff}}


def config(width, vocab, layers, eps=1e-5, cap=12.0) -> Dict[str, Any]:
    return {"architecture": "Peratar", "vocab": vocab, "width": width, "norm": {"eps": eps},
            "logit_softcap": cap, "layers": layers}


# Three layers, the middle one without feed-forward, the last one on the first one's cache.
SMALL = config(96, 200, [
    layer(mixer(3, 16, 8, 24, 40, 0.21, base=500.0), 72),
    layer(mixer(3, 16, 8, 24, 40, 0.21, base=500.0), None),
    layer(mixer(2, 24, 8, 16, 40, 0.18, base=500.0, kv_from=0), 56),
], eps=1e-6, cap=9.0)

# Every layer another size: one head; a rotated part of which only some dims rotate; cached rows
# of 32, 39 (padded to 48) and 16 values; a rank and inner widths that are no multiple of eight;
# two layers reading other layers' caches.
ODD = config(128, 331, [
    layer(mixer(1, 8, 12, 8, 20, 0.3, base=10000.0, rot_dims=8), 100),
    layer(mixer(5, 24, 6, 16, 33, 0.17, base=77.0), 132),
    layer(mixer(2, 16, 6, 40, 33, 0.25, base=77.0, kv_from=1), None),
    layer(mixer(4, 8, 4, 8, 12, 0.35, base=3.0e5), 64),
    layer(mixer(3, 40, 12, 8, 20, 0.11, base=10000.0, rot_dims=8, kv_from=0), 60),
], eps=1e-5, cap=30.0)

# Cached rows of 128 values and eight heads: the shapes for which prompt portions run on the
# tensor-memory attention kernel and decoded tokens on clusters; unrotated, rotated and value
# widths all equal.
WIDE = config(256, 500, [
    layer(mixer(8, 32, 32, 32, 96, 0.125, base=1000000.0), 512),
    layer(mixer(8, 32, 32, 32, 96, 0.125, base=1000000.0, kv_from=0), 512),
], eps=2e-5, cap=25.0)

# More heads than an attention tile has rows (20 and 17 on one cached row), so a token's heads
# are cut across tiles.
MANY_HEADS = config(160, 300, [
    layer(mixer(20, 8, 8, 8, 40, 0.3), 96),
    layer(mixer(17, 16, 8, 12, 40, 0.2, kv_from=0), 64),
])

# A width that is no multiple of four, an odd vocabulary, odd inner widths, an odd rotated width of
# which four dims rotate, cached rows of 24 and 11 values; the largest row the attention kernels
# take (224 + 32 = 256) in a model of its own.
RAGGED = config(90, 1001, [
    layer(mixer(3, 10, 5, 7, 19, 0.3, rot_dims=4), 77),
    layer(mixer(2, 6, 5, 9, 19, 0.3, rot_dims=4, kv_from=0), 33),
    layer(mixer(5, 12, 2, 3, 9, 0.3), None),
], cap=5.0)
LARGEST_ROW = config(192, 257, [
    layer(mixer(3, 32, 32, 48, 224, 0.1), 200),
    layer(mixer(2, 64, 32, 16, 224, 0.1, kv_from=0), None),
])

ALL = {"small": SMALL, "odd": ODD, "wide": WIDE, "many_heads": MANY_HEADS, "ragged": RAGGED, "largest_row": LARGEST_ROW}


def make_weights(cfg: Dict[str, Any], seed: int, sharp: float = 1.0) -> Dict[str, torch.Tensor]:
    """bfloat16 tensors under the checkpoint's names.  ``sharp`` scales the query projections: at
    4 or more the softmax puts most of its weight on a few keys, wherever they are."""
    from velox_b200.config.registry import architecture_of

    arch = architecture_of(cfg)
    spec = arch.build_spec(arch.parse_config(cfg))
    gen = torch.Generator().manual_seed(seed)
    out = {}
    for name, source in sorted(spec.checkpoint_tensors().items()):
        shape = tuple(source.shape)
        if name == "embed":
            t = torch.randn(shape, generator=gen)
        elif name.endswith("norm") or name.endswith("norm1") or name.endswith("norm2"):
            t = 1.0 + 0.3 * torch.randn(shape, generator=gen)
        elif name.endswith(".dwa"):
            t = torch.full(shape, 1.0 / shape[0]) + 0.3 * torch.randn(shape, generator=gen)
        elif name.endswith(".act"):
            t = torch.randn(shape, generator=gen)
        elif len(shape) == 1:
            t = 0.5 * torch.randn(shape, generator=gen)
        else:
            t = torch.randn(shape, generator=gen) / shape[1] ** 0.5
            if name.endswith("mix.q"):
                t = t * sharp
            if name.endswith("mix.uk"):
                t = t * 2.0
        out[name] = t.to(torch.bfloat16)
    return out


def write_folder(folder: str, cfg: Dict[str, Any], tensors: Dict[str, torch.Tensor]) -> None:
    from safetensors.torch import save_file

    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w", encoding="utf-8") as handle:
        json.dump(cfg, handle)
    save_file({k: v.contiguous() for k, v in tensors.items()}, os.path.join(folder, "model.safetensors"))
