"""A plain, slow implementation of the Rulunex decoder for the tests to compare the engine with:
whole sequences, no cache, no batching, one function per mechanism.  It shares no code with
``gllm_b200``: it reads the raw config.json dict and the raw tensors by name.

Notation.  ``T`` tokens of one sequence at positions ``0 .. T-1``; ``W`` the model width; linear
weights are stored ``[out, in]`` and applied as ``x @ W.T``.  Every function computes in the dtype of
its inputs (float64 in the tests).

The design: scaled token embedding; layers with ONE norm whose output feeds the mixer and the
feed-forward side by side, ``x += mixer(n(x)) + ff(n(x))``; a stretch of layers that is run several times
with the same weights, each pass beginning with a projection of ``[x ; embedding]`` back to the width;
two mixers: softmax attention over a latent vector per token (keys and values are up-projections of the
latent, plus one rotated key part shared by the heads, plus a sigmoid gate on every head's output), and
grouped-query attention inside a sliding window whose values are the un-normed, un-rotated keys; a
gated feed-forward with clamped inputs; logits through the embedding table.
"""

from __future__ import annotations

import math

import torch

SIGMOID_SLOPE = 1.702        # the feed-forward's gate is g * sigmoid(1.702 g)


# ------------------------------------------------------------------ pieces
def plain_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def plain_layer_norm(x, weight, eps):
    """The layers' and the model's norm: the stored weight is an offset from one."""
    return plain_rms(x, eps) * (1.0 + weight)


def plain_frequencies(rot: dict) -> torch.Tensor:
    """``base^(-2i/dims)`` for i < dims/2, float64; with ``scaling`` the long wavelengths are slowed down:
    untouched below ``original/high``, divided by ``factor`` above ``original/low``, blended between."""
    dims = rot["dims"]
    f = torch.tensor([float(rot["base"]) ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=torch.float64)
    sc = rot.get("scaling")
    if not sc:
        return f
    out = []
    for fi in f.tolist():
        wavelength = 2.0 * math.pi / fi
        if wavelength < sc["original"] / sc["high"]:
            out.append(fi)
        elif wavelength > sc["original"] / sc["low"]:
            out.append(fi / sc["factor"])
        else:
            s = (sc["original"] / wavelength - sc["low"]) / (sc["high"] - sc["low"])
            out.append((1.0 - s) * fi / sc["factor"] + s * fi)
    return torch.tensor(out, dtype=torch.float64)


def plain_rotate(x: torch.Tensor, positions: torch.Tensor, freqs: torch.Tensor, interleaved: bool) -> torch.Tensor:
    """``x`` [T, heads, d]: the first ``2 * len(freqs)`` columns of every head are rotated, pair i by the
    angle ``p * f_i``; pairs are columns (2i, 2i+1) when ``interleaved``, (i, i + dims/2) otherwise."""
    half = freqs.numel()
    dims = 2 * half
    ang = positions.to(torch.float64)[:, None] * freqs[None, :]            # [T, half]
    cos, sin = ang.cos().to(x.dtype)[:, None, :], ang.sin().to(x.dtype)[:, None, :]
    out = x.clone()
    if interleaved:
        u, v = x[..., 0:dims:2], x[..., 1:dims:2]
        out[..., 0:dims:2] = u * cos - v * sin
        out[..., 1:dims:2] = v * cos + u * sin
    else:
        u, v = x[..., :half], x[..., half:dims]
        out[..., :half] = u * cos - v * sin
        out[..., half:dims] = v * cos + u * sin
    return out


def plain_softmax_attention(q, k, v, scale: float, window: int | None) -> torch.Tensor:
    """``q`` [T, H, dk], ``k`` [T, G, dk], ``v`` [T, G, dv]; query head h uses key head h // (H/G); position i
    sees j <= i, and with a window only i - j < window.  Returns [T, H, dv]."""
    T, H, _ = q.shape
    G = k.shape[1]
    rep = H // G
    i = torch.arange(T)
    seen = i[None, :] <= i[:, None]
    if window:
        seen &= (i[:, None] - i[None, :]) < window
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        s = (q[:, h] @ k[:, h // rep].T) * scale
        s = s.masked_fill(~seen, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ v[:, h // rep]
    return out


# ------------------------------------------------------------------ mixers
def plain_latent_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, d, r, dv, rank = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
    pos = torch.arange(T)
    freqs = plain_frequencies(m["rot"])
    q = (h @ w[p + ".q"].T).view(T, H, d + r)
    down = h @ w[p + ".dkv"].T
    c = plain_rms(down[:, :rank], eps) * w[p + ".dkv.norm"]
    k_rot = plain_rotate(down[:, None, rank:], pos, freqs, interleaved=True)            # [T, 1, r]
    q_rot = plain_rotate(q[:, :, d:], pos, freqs, interleaved=True)
    k_plain = (c @ w[p + ".uk"].T).view(T, H, d)
    v = (c @ w[p + ".uv"].T).view(T, H, dv)
    keys = torch.cat([k_plain, k_rot.expand(T, H, r)], dim=-1)
    queries = torch.cat([q[:, :, :d], q_rot], dim=-1)
    a = plain_softmax_attention(queries, keys, v, m["scale"], None)
    gate = torch.sigmoid(h @ w[p + ".g"].T)                                             # [T, H]
    return (a * gate[:, :, None]).reshape(T, H * dv) @ w[p + ".o"].T


def plain_window_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    pos = torch.arange(T)
    freqs = plain_frequencies(m["rot"])
    q_raw, k_raw = h @ w[p + ".q"].T, h @ w[p + ".k"].T
    q = (plain_rms(q_raw, eps) * w[p + ".q.norm"]).view(T, H, d)
    k = (plain_rms(k_raw, eps) * w[p + ".k.norm"]).view(T, G, d)
    q, k = plain_rotate(q, pos, freqs, False), plain_rotate(k, pos, freqs, False)
    v = k_raw.view(T, G, d)
    window = (m.get("mask") or {}).get("size")
    a = plain_softmax_attention(q, k, v, m["scale"], window)
    return a.reshape(T, H * d) @ w[p + ".o"].T


def plain_feed_forward(h: torch.Tensor, w: dict, p: str, mlp: dict) -> torch.Tensor:
    limit = mlp["limit"]
    g = torch.clamp(h @ w[p + ".gate"].T, max=limit)
    u = torch.clamp(h @ w[p + ".up"].T, min=-limit, max=limit)
    return (g * torch.sigmoid(SIGMOID_SLOPE * g) * (u + 1.0)) @ w[p + ".down"].T


MIXERS = {"latent_attention": plain_latent_attention, "attention": plain_window_attention}


# ------------------------------------------------------------------ the model
def plain_layer_order(cfg: dict) -> list[tuple[int, bool]]:
    """(layer, begins a pass) in the order the layers run."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, False) for i in range(n)]
    order = [(i, False) for i in range(loop["start"])]
    for _ in range(loop["times"]):
        order += [(i, i == loop["start"]) for i in range(loop["start"], loop["stop"])]
    return order + [(i, False) for i in range(loop["stop"], n)]


def plain_forward(cfg: dict, w: dict, tokens, dtype=torch.float64, return_layers: bool = False):
    """Logits [T, vocab] of one whole sequence (and the residual after every layer run)."""
    w = {k: v.to(dtype) for k, v in w.items()}
    eps = cfg["norm"]["eps"]
    x0 = w["embed"][torch.as_tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    x = x0
    after = []
    for i, begins in plain_layer_order(cfg):
        layer = cfg["layers"][i]
        if begins:
            x = torch.cat([x, x0], dim=-1) @ w["loop.in"].T
        h = plain_layer_norm(x, w[f"l{i}.norm1"], eps)
        y = MIXERS[layer["type"]](h, w, f"l{i}.mix", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            y = y + plain_feed_forward(h, w, f"l{i}.mlp", layer["mlp"])
        x = x + y
        after.append(x)
    logits = plain_layer_norm(x, w["final.norm"], eps) @ w["embed"].T
    return (logits, torch.stack(after)) if return_layers else logits
