"""Small Guvetar configurations for the tests, as raw config.json dicts, and a writer that draws their
weights here (not through the engine's random-weights mode), tensor by tensor under the names the design
gives them, with values that keep every mechanism alive: decays spread between fast and slow, gates
that move, stream matrices near the identity, sharp attention scores.

The configurations differ in every size and option: streams (3, absent, 1, 4), layer order and kinds,
layers without a feed-forward, grouped / multi-query / one head per key head, equal and unequal key and
value widths, one head, one convolution tap, sizes that are no multiple of 8 (so that products fall to
the engine's paths for odd shapes), with and without the query multiplier."""

from __future__ import annotations

import json
import math
import os

import torch
from safetensors.torch import save_file


def _mamba(inner, state, dt_rank, conv):
    return {"type": "mamba1", "mixer": {"inner": inner, "state": state, "dt_rank": dt_rank, "conv": conv}}


def _mlstm(heads, dim, vdim, cap):
    return {"type": "mlstm", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "gate_cap": cap}}


def _parallel(left, right, ls, rs):
    return {"type": "parallel", "mixer": {"left": left, "right": right, "left_scale": ls, "right_scale": rs}}


def _ff(n):
    return None if n is None else {"kind": "dense", "ff": n}


def _layer(mixer, ff):
    return {**mixer, "mlp": _ff(ff)}


GUVETAR_A = {
    "architecture": "Guvetar", "vocab": 200, "width": 64, "streams": 3, "norm": {"eps": 1e-5},
    "layers": [
        _layer(_parallel({"heads": 4, "kv_heads": 2, "dim": 16, "vdim": 24, "scale": 0.3,
                          "q_temp": {"coef": 0.7, "every": 5}},
                         {"heads": 2, "dim": 8, "vdim": 16}, 0.7, 1.2), 96),
        _layer(_mlstm(2, 16, 8, 10.0), None),
        _layer(_mamba(96, 8, 4, 3), 80),
        _layer(_mamba(72, 16, 8, 5), None),
    ],
}
# a plain residual (no streams), sizes that are no multiple of 8, one head per key head, no query multiplier
GUVETAR_B = {
    "architecture": "Guvetar", "vocab": 131, "width": 48, "norm": {"eps": 3e-6},
    "layers": [
        _layer(_mlstm(3, 10, 12, 6.0), 50),
        _layer(_mamba(50, 5, 3, 2), 36),
        _layer(_parallel({"heads": 3, "kv_heads": 3, "dim": 20, "vdim": 12, "scale": 0.25},
                         {"heads": 1, "dim": 24, "vdim": 40}, 1.0, 0.4), None),
    ],
}
# one stream, one head everywhere, one tap (no convolution memory), multi-query attention, wider heads
GUVETAR_C = {
    "architecture": "Guvetar", "vocab": 97, "width": 96, "streams": 1, "norm": {"eps": 1e-6},
    "layers": [
        _layer(_mamba(128, 40, 16, 1), 64),
        _layer(_parallel({"heads": 4, "kv_heads": 1, "dim": 40, "vdim": 72, "scale": 0.16,
                          "q_temp": {"coef": 0.25, "every": 16}},
                         {"heads": 3, "dim": 40, "vdim": 8}, 0.6, 0.45), 128),
        _layer(_mlstm(1, 64, 40, 9.0), 72),
    ],
}
# no attention at all (no cache pages, only states), four streams
GUVETAR_D = {
    "architecture": "Guvetar", "vocab": 150, "width": 32, "streams": 4, "norm": {"eps": 1e-5},
    "layers": [_layer(_mlstm(4, 8, 8, 8.0), 48), _layer(_mamba(64, 4, 2, 4), None)],
}
# head widths the tensor-core attention kernel of bfloat16 runs takes (32, 64, 96, 128), with groups of two and
# of three query heads per key head, beside a scan
GUVETAR_E = {
    "architecture": "Guvetar", "vocab": 120, "width": 64, "streams": 2, "norm": {"eps": 1e-5},
    "layers": [
        _layer(_parallel({"heads": 4, "kv_heads": 2, "dim": 32, "vdim": 64, "scale": 0.2,
                          "q_temp": {"coef": 0.3, "every": 7}},
                         {"heads": 2, "dim": 16, "vdim": 16}, 1.0, 1.0), 64),
        _layer(_mamba(64, 8, 8, 4), None),
        _layer(_parallel({"heads": 3, "kv_heads": 1, "dim": 96, "vdim": 32, "scale": 0.12},
                         {"heads": 1, "dim": 32, "vdim": 32}, 0.6, 0.9), 96),
        _layer(_parallel({"heads": 2, "kv_heads": 2, "dim": 128, "vdim": 128, "scale": 0.1},
                         {"heads": 2, "dim": 8, "vdim": 8}, 1.1, 0.3), None),
    ],
}
GUVETAR = {"A": GUVETAR_A, "B": GUVETAR_B, "C": GUVETAR_C, "D": GUVETAR_D, "E": GUVETAR_E}


def single_mixer(kind: str, streams=None) -> dict:
    """A one-layer model whose only sublayer is a mixer of ``kind``: the mechanism alone."""
    mixers = {
        "mamba1": _mamba(40, 6, 5, 4),
        "mlstm": _mlstm(2, 12, 20, 12.0),
        "parallel": _parallel({"heads": 2, "kv_heads": 1, "dim": 12, "vdim": 20, "scale": 0.4,
                               "q_temp": {"coef": 0.4, "every": 3}}, {"heads": 2, "dim": 6, "vdim": 10}, 0.9, 0.6),
        "sigmoid_only": _parallel({"heads": 2, "kv_heads": 2, "dim": 32, "vdim": 32, "scale": 0.35},
                                  {"heads": 1, "dim": 4, "vdim": 4}, 1.0, 0.0),
        "hgrn2_only": _parallel({"heads": 1, "kv_heads": 1, "dim": 8, "vdim": 8, "scale": 0.3},
                                {"heads": 3, "dim": 10, "vdim": 14}, 0.0, 1.0),
    }
    cfg = {"architecture": "Guvetar", "vocab": 90, "width": 40, "norm": {"eps": 1e-5},
           "layers": [_layer(mixers[kind], None)]}
    if streams:
        cfg["streams"] = streams
    return cfg


def draw_weights(cfg: dict, seed: int, sharp: float = 1.0) -> dict[str, torch.Tensor]:
    """Every tensor of ``cfg`` in fp32 with bfloat16-representable values.  ``sharp`` scales the query
    and key norm weights (scores grow with its square)."""
    g = torch.Generator().manual_seed(seed)
    W = cfg["width"]

    def normal(*shape, std=1.0):
        return torch.randn(*shape, generator=g) * std

    def uniform(*shape, lo=0.0, hi=1.0):
        return lo + (hi - lo) * torch.rand(*shape, generator=g)

    def lin(out, inp, gain=1.0):
        return normal(out, inp, std=gain / math.sqrt(inp))

    t: dict[str, torch.Tensor] = {"embed": normal(cfg["vocab"], W, std=1.0), "final.norm": uniform(W, lo=0.7, hi=1.3)}
    S = cfg.get("streams")
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}", layer["mixer"]
        subs = [1] + ([2] if layer["mlp"] is not None else [])
        for q in subs:
            t[f"{p}.norm{q}"] = uniform(W, lo=0.7, hi=1.3)
            if S:
                t[f"{p}.hc{q}.in"] = uniform(S, lo=0.3, hi=1.0)
                t[f"{p}.hc{q}.out"] = uniform(S, lo=-1.0, hi=1.0)
                t[f"{p}.hc{q}.mix"] = torch.eye(S) * 0.8 + normal(S, S, std=0.15)
        x = f"{p}.mix"
        if layer["type"] == "mamba1":
            I, N, R, K = m["inner"], m["state"], m["dt_rank"], m["conv"]
            t[f"{x}.in"] = lin(2 * I, W)
            t[f"{x}.conv"] = normal(I, K, std=0.6)
            t[f"{x}.conv.b"] = normal(I, std=0.2)
            t[f"{x}.x"] = lin(R + 2 * N, I)
            t[f"{x}.dt"] = lin(I, R, gain=1.5)
            t[f"{x}.dt.b"] = uniform(I, lo=-3.0, hi=0.5)
            t[f"{x}.A_log"] = torch.log(uniform(I, N, lo=0.05, hi=4.0))
            t[f"{x}.D"] = uniform(I, lo=0.5, hi=1.5)
            t[f"{x}.o"] = lin(W, I)
        elif layer["type"] == "mlstm":
            H, d, dv = m["heads"], m["dim"], m["vdim"]
            t[f"{x}.q"], t[f"{x}.k"] = lin(H * d, W, gain=2.0), lin(H * d, W, gain=2.0)
            t[f"{x}.v"], t[f"{x}.g"] = lin(H * dv, W), lin(H * dv, W, gain=2.0)
            t[f"{x}.o"] = lin(W, H * dv)
            t[f"{x}.norm"] = uniform(H * dv, lo=0.7, hi=1.3)
            t[f"{x}.i"], t[f"{x}.f"] = lin(H, W, gain=3.0), lin(H, W, gain=3.0)
            t[f"{x}.i.b"], t[f"{x}.f.b"] = normal(H, std=1.0), uniform(H, lo=1.0, hi=5.0)
        else:
            lm, rm = m["left"], m["right"]
            H, G, d, dv = lm["heads"], lm["kv_heads"], lm["dim"], lm["vdim"]
            t[f"{x}.left.q"], t[f"{x}.left.k"], t[f"{x}.left.v"] = lin(H * d, W), lin(G * d, W), lin(G * dv, W)
            t[f"{x}.left.q.norm"] = uniform(d, lo=0.8, hi=1.6) * sharp
            t[f"{x}.left.k.norm"] = uniform(d, lo=0.8, hi=1.6) * sharp
            t[f"{x}.left.pb"] = uniform(H, lo=-4.0, hi=-1.0)
            t[f"{x}.left.o"] = lin(W, H * dv, gain=0.5)
            H, d, dv = rm["heads"], rm["dim"], rm["vdim"]
            t[f"{x}.right.q"], t[f"{x}.right.f"], t[f"{x}.right.v"] = lin(H * d, W), lin(H * d, W, gain=2.0), lin(H * dv, W)
            t[f"{x}.right.f.b"] = normal(H * d, std=1.0)
            t[f"{x}.right.lower"] = uniform(H * d, lo=0.0, hi=0.9)
            t[f"{x}.right.norm"] = uniform(dv, lo=0.7, hi=1.3)
            t[f"{x}.right.o"] = lin(W, H * dv)
        if layer["mlp"] is not None:
            t[f"{p}.mlp.up"], t[f"{p}.mlp.down"] = lin(layer["mlp"]["ff"], W, gain=1.5), lin(W, layer["mlp"]["ff"])
    return {k: v.to(torch.bfloat16).to(torch.float32).contiguous() for k, v in t.items()}


def write_model(cfg: dict, weights: dict[str, torch.Tensor], folder: str) -> str:
    """config.json and model.safetensors (bfloat16) in ``folder``."""
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    save_file({k: v.to(torch.bfloat16).contiguous() for k, v in weights.items()}, os.path.join(folder, "model.safetensors"))
    return folder
