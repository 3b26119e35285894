"""Small Rulunex configurations for the tests, as raw config.json dicts, and a writer that draws their weights
here (not through the engine's random-weights mode), tensor by tensor under the names the design gives them.

The configurations differ in every size and option: with and without a repeated stretch (from the first layer,
from the middle, once, three times), layers without a feed-forward, grouped / multi-query / one head per key
head, windows shorter and longer than a page, with and without a window and wavelength scaling, rotary parts
narrower than the head, sizes that are no multiple of 8, feed-forward widths that do and do not allow the
interleaved weight layout, head widths that the tensor-core kernels take and ones they do not."""

from __future__ import annotations

import json
import math
import os

import torch
from safetensors.torch import save_file


def _latent(heads, dim, rot_dim, vdim, rank, scale, base=10000.0, dims=None):
    return {"type": "latent_attention",
            "mixer": {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
                      "rot": {"base": base, "dims": rot_dim if dims is None else dims}}}


def _window(heads, kv_heads, dim, scale, dims, window=None, base=10000.0, scaling=None):
    rot = {"base": base, "dims": dims}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "low", "high", "original"), scaling))
    mixer = {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "scale": scale, "rot": rot}
    if window is not None:
        mixer["mask"] = {"size": window}
    return {"type": "attention", "mixer": mixer}


def _layer(mixer, ff, limit=1.5):
    return {**mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}


# a stretch of two layers run three times, grouped heads, a window shorter than two pages, one layer without a
# feed-forward, one feed-forward width that is no multiple of 64
RULUNEX_A = {
    "architecture": "Rulunex", "vocab": 200, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 1.7},
    "loop": {"start": 1, "stop": 3, "times": 3},
    "layers": [
        _layer(_window(4, 2, 32, 0.2, 16, window=20, scaling=(8.0, 1.0, 4.0, 64)), 96),
        _layer(_latent(3, 16, 8, 24, 40, 0.22), 128, limit=0.8),
        _layer(_latent(2, 32, 16, 16, 24, 0.15, base=500.0), None),
        _layer(_window(2, 1, 48, 0.15, 48), 64, limit=3.0),
    ],
}
# no repeated stretch; sizes that are no multiple of 8; a rotation narrower than the rotated part; one head per
# key head; a window of 7
RULUNEX_B = {
    "architecture": "Rulunex", "vocab": 131, "width": 48, "norm": {"eps": 3e-6}, "embedding": {"scale": 0.9},
    "layers": [
        _layer(_latent(3, 12, 6, 10, 20, 0.3, base=100.0, dims=4), 50),
        _layer(_window(3, 3, 16, 0.25, 8, window=7, base=50.0), 36),
        _layer(_latent(1, 20, 4, 12, 36, 0.2), None),
    ],
}
# the whole model is the repeated stretch (twice); head widths the tensor-core kernels take; windows that end
# inside and beyond a block of keys
RULUNEX_C = {
    "architecture": "Rulunex", "vocab": 160, "width": 128, "norm": {"eps": 1e-6}, "embedding": {"scale": 11.3},
    "loop": {"start": 0, "stop": 3, "times": 2},
    "layers": [
        _layer(_window(4, 2, 64, 0.125, 32, window=33, scaling=(4.0, 1.0, 2.0, 32)), 192),
        _layer(_latent(4, 32, 32, 32, 64, 0.125, base=250000.0), 128),
        _layer(_window(2, 1, 128, 0.09, 128, window=100), 64),
    ],
}
# one pass of a "repeated" stretch (the projection at its start still runs), no feed-forward anywhere
RULUNEX_D = {
    "architecture": "Rulunex", "vocab": 150, "width": 32, "norm": {"eps": 1e-5}, "embedding": {"scale": 5.0},
    "loop": {"start": 1, "stop": 2, "times": 1},
    "layers": [_layer(_latent(2, 8, 8, 8, 16, 0.25), None), _layer(_window(2, 2, 16, 0.25, 16, window=5), None)],
}
RULUNEX = {"A": RULUNEX_A, "B": RULUNEX_B, "C": RULUNEX_C, "D": RULUNEX_D}


def single_mixer(kind: str, mlp: bool = True) -> dict:
    """One layer with the given mixer (and a feed-forward), no repeated stretch."""
    mixer = {"latent": _latent(2, 16, 8, 16, 24, 0.2),
             "latent_wide": _latent(5, 16, 32, 24, 64, 0.2),        # widths the tensor-core kernel takes
             "latent_many": _latent(8, 32, 64, 16, 128, 0.12),
             "window": _window(4, 2, 16, 0.25, 8, window=24, scaling=(2.0, 1.0, 4.0, 16)),
             "causal": _window(2, 2, 32, 0.18, 32),
             "odd": _window(3, 1, 20, 0.2, 10, window=9)}[kind]
    return {"architecture": "Rulunex", "vocab": 120, "width": 64, "norm": {"eps": 1e-5}, "embedding": {"scale": 2.0},
            "layers": [_layer(mixer, 64 if mlp else None)]}


def tensor_shapes(cfg: dict) -> dict[str, tuple[int, ...]]:
    w = cfg["width"]
    out = {"embed": (cfg["vocab"], w), "final.norm": (w,)}
    if cfg.get("loop"):
        out["loop.in"] = (w, 2 * w)
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}", layer["mixer"]
        out[f"{p}.norm1"] = (w,)
        if layer["type"] == "latent_attention":
            h, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            out.update({f"{p}.mix.q": (h * (d + r), w), f"{p}.mix.dkv": (rank + r, w), f"{p}.mix.dkv.norm": (rank,),
                        f"{p}.mix.uk": (h * d, rank), f"{p}.mix.uv": (h * dv, rank), f"{p}.mix.g": (h, w),
                        f"{p}.mix.o": (w, h * dv)})
        else:
            h, g, d = m["heads"], m["kv_heads"], m["dim"]
            out.update({f"{p}.mix.q": (h * d, w), f"{p}.mix.k": (g * d, w), f"{p}.mix.q.norm": (h * d,),
                        f"{p}.mix.k.norm": (g * d,), f"{p}.mix.o": (w, h * d)})
        if layer["mlp"] is not None:
            ff = layer["mlp"]["ff"]
            out.update({f"{p}.mlp.gate": (ff, w), f"{p}.mlp.up": (ff, w), f"{p}.mlp.down": (w, ff)})
    return out


def draw_weights(cfg: dict, seed: int, sharp: float = 1.0) -> dict[str, torch.Tensor]:
    """float32 tensors whose values are bfloat16 numbers.  ``sharp`` multiplies the query projections, so that
    the softmax has a few large weights and a key that is lost or one too many shows."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith("norm1") or name == "final.norm":
            t = torch.randn(shape, generator=g) * 0.15                       # offsets from one
        elif name.endswith(".norm"):
            t = 1.0 + torch.randn(shape, generator=g) * 0.15                 # plain weights
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            t = torch.randn(shape, generator=g) / math.sqrt(shape[1])
            if name.endswith(".mix.q"):
                t = t * sharp
            if name.endswith(".mlp.gate") or name.endswith(".mlp.up"):
                t = t * 1.5                                                  # so that the clamps bite
            if name.endswith(".mix.g"):
                t = t * 2.0
        out[name] = t.to(torch.bfloat16).to(torch.float32)
    return out


def write_model(cfg: dict, weights: dict[str, torch.Tensor], folder: str) -> str:
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f, indent=1)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in weights.items()},
              os.path.join(folder, "model.safetensors"))
    return folder
