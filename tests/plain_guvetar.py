"""A plain, slow implementation of the Guvetar decoder for the tests to compare the engine with:
whole sequences, token by token, no cache, no batching, one function per mechanism.  It shares no
code with ``gllm_b200``: it reads the raw config.json dict and the raw tensors by name.

Notation.  ``T`` tokens of one sequence at positions ``0 .. T-1``; ``W`` the model width; linear
weights are stored ``[out, in]`` and applied as ``x @ W.T``.  Every function computes in the dtype of
its inputs (float64 in the tests).

The design: token embedding plus a sinusoid of the position; ``streams`` copies of the residual
(hyper-connections: a learnt read vector, a learnt stream-to-stream matrix and a learnt write vector
per sublayer); per layer a mixer (one of ``mamba1``: selective state-space scan; ``mlstm``: matrix
memory with exponential gates and a running maximum; ``parallel``: sigmoid-weighted attention beside a
gated linear-attention head whose forget gate also scales what is written) and an optional dense
feed-forward with a squared-ReLU activation; RMS norm; logits through the embedding table.
"""

from __future__ import annotations

import math

import torch
import torch.nn.functional as F


# ------------------------------------------------------------------ pieces
def plain_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) over the last axis."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def plain_sinusoid(positions: torch.Tensor, width: int, dtype=torch.float64) -> torch.Tensor:
    """[T, W]: column 2i = sin(p * 10000^(-2i/W)), column 2i+1 = cos of the same angle."""
    i = torch.arange((width + 1) // 2, dtype=torch.float64)
    freq = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * i / width)
    ang = positions.to(torch.float64)[:, None] * freq[None, :]
    out = torch.zeros(positions.numel(), 2 * freq.numel(), dtype=torch.float64)
    out[:, 0::2] = ang.sin()
    out[:, 1::2] = ang.cos()
    return out[:, :width].to(dtype)


def plain_gelu_tanh(z):
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def plain_dense_ff(h: torch.Tensor, w: dict, p: str) -> torch.Tensor:
    """down(relu(up h)^2)."""
    a = torch.relu(h @ w[p + ".up"].T)
    return (a * a) @ w[p + ".down"].T


# ------------------------------------------------------------------ mamba1
def plain_mamba1(h: torch.Tensor, w: dict, p: str, m: dict) -> torch.Tensor:
    """Selective scan, token by token.  ``h`` [T, W]."""
    inner, n_state, rank, taps = m["inner"], m["state"], m["dt_rank"], m["conv"]
    T = h.shape[0]
    xz = h @ w[p + ".in"].T
    x, z = xz[:, :inner], xz[:, inner:]
    conv_w, conv_b = w[p + ".conv"], w[p + ".conv.b"]
    padded = torch.cat([torch.zeros(taps - 1, inner, dtype=h.dtype), x], 0)
    xc = torch.zeros_like(x)
    for t in range(T):
        window = padded[t:t + taps]                      # inputs t-taps+1 .. t, the last is the current token
        xc[t] = (window * conv_w.T).sum(0) + conv_b
    xc = F.silu(xc)
    proj = xc @ w[p + ".x"].T
    dt_in, B, C = proj[:, :rank], proj[:, rank:rank + n_state], proj[:, rank + n_state:]
    dt = F.softplus(dt_in @ w[p + ".dt"].T + w[p + ".dt.b"])
    A = -torch.exp(w[p + ".A_log"])
    S = torch.zeros(inner, n_state, dtype=h.dtype)
    y = torch.zeros_like(x)
    for t in range(T):
        S = torch.exp(dt[t][:, None] * A) * S + (dt[t] * xc[t])[:, None] * B[t][None, :]
        y[t] = S @ C[t] + w[p + ".D"] * xc[t]
    return (y * F.silu(z)) @ w[p + ".o"].T


# ------------------------------------------------------- sigmoid attention
def plain_sigmoid_attention(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """Causal attention whose weights are sigmoid(score + head bias), not normalised over the keys;
    per-head RMS norm of queries and keys; a query multiplier that grows with the logarithm of the
    position; grouped key/value heads; no rotation."""
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = (h @ w[p + ".q"].T).view(T, H, d)
    k = (h @ w[p + ".k"].T).view(T, G, d)
    v = (h @ w[p + ".v"].T).view(T, G, dv)
    q = plain_rms(q, eps) * w[p + ".q.norm"]
    k = plain_rms(k, eps) * w[p + ".k.norm"]
    pos = torch.arange(T)
    temp = m.get("q_temp")
    if temp is not None:
        mult = 1.0 + temp["coef"] * torch.log(torch.floor((pos + 1).to(h.dtype) / temp["every"]) + 1.0)
        q = q * mult[:, None, None]
    out = torch.zeros(T, H, dv, dtype=h.dtype)
    visible = pos[None, :] <= pos[:, None]
    for head in range(H):
        g = head // (H // G)
        score = (q[:, head] @ k[:, g].T) * m["scale"] + w[p + ".pb"][head]
        weight = torch.sigmoid(score) * visible
        out[:, head] = weight @ v[:, g]
    return out.reshape(T, H * dv) @ w[p + ".o"].T


# ------------------------------------------------------------------ hgrn2
def plain_hgrn2(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """Gated linear attention: forget gate f in [lower, 1) per (head, key channel); the state row of
    a channel decays by f and takes (1 - f) v."""
    H, d, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = F.silu(h @ w[p + ".q"].T).view(T, H, d)
    v = (h @ w[p + ".v"].T).view(T, H, dv)
    low = w[p + ".lower"]
    f = (low + (1.0 - low) * torch.sigmoid(h @ w[p + ".f"].T + w[p + ".f.b"])).view(T, H, d)
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hdv,hd->hv", S, q[t])
    o = plain_rms(o, eps) * w[p + ".norm"]
    return o.reshape(T, H * dv) @ w[p + ".o"].T


def plain_parallel(h, w, p, m, eps):
    left = plain_sigmoid_attention(h, w, p + ".left", m["left"], eps)
    right = plain_hgrn2(h, w, p + ".right", m["right"], eps)
    return m["left_scale"] * left + m["right_scale"] * right


# ------------------------------------------------------------------ mlstm
def plain_mlstm(h: torch.Tensor, w: dict, p: str, m: dict, eps: float) -> torch.Tensor:
    """Matrix memory with a log-space input gate, a log-sigmoid forget gate (both soft-capped) and a
    running maximum that starts at zero."""
    H, d, dv, cap = m["heads"], m["dim"], m["vdim"], m["gate_cap"]
    T = h.shape[0]
    q = (h @ w[p + ".q"].T).view(T, H, d) * d ** -0.5
    k = (h @ w[p + ".k"].T).view(T, H, d)
    v = (h @ w[p + ".v"].T).view(T, H, dv)
    ig = cap * torch.tanh((h @ w[p + ".i"].T + w[p + ".i.b"]) / cap)                  # [T, H]
    fg = F.logsigmoid(cap * torch.tanh((h @ w[p + ".f"].T + w[p + ".f.b"]) / cap))
    S = torch.zeros(H, d, dv, dtype=h.dtype)
    n = torch.zeros(H, d, dtype=h.dtype)
    mx = torch.zeros(H, dtype=h.dtype)
    o = torch.zeros(T, H, dv, dtype=h.dtype)
    for t in range(T):
        new = torch.maximum(fg[t] + mx, ig[t])
        keep = torch.exp(fg[t] + mx - new)
        take = torch.exp(ig[t] - new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        mx = new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        o[t] = num / den[:, None]
    o = plain_rms(o, eps).reshape(T, H * dv) * w[p + ".norm"]
    o = o * torch.sigmoid(h @ w[p + ".g"].T)
    return o @ w[p + ".o"].T


MIXERS = {
    "mamba1": lambda h, w, p, m, eps: plain_mamba1(h, w, p, m),
    "parallel": plain_parallel,
    "mlstm": plain_mlstm,
}


# ------------------------------------------------------------------ the model
def plain_forward(cfg: dict, weights: dict, tokens, dtype=torch.float64, return_layers: bool = False):
    """Logits [T, vocab] of one whole sequence (and, with ``return_layers``, the sum of the streams
    after every layer, [layers, T, W])."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    T, W = tokens.numel(), cfg["width"]
    x0 = w["embed"][tokens] + plain_sinusoid(torch.arange(T), W, dtype)
    streams = cfg.get("streams")
    xs = x0[None].repeat(streams, 1, 1) if streams else x0
    after = []

    def sublayer(xs, layer, q, fn):
        if streams:
            hc = f"l{layer}.hc{q}"
            u = torch.einsum("s,stw->tw", w[hc + ".in"], xs)
        else:
            u = xs
        y = fn(plain_rms(u, eps) * w[f"l{layer}.norm{q}"])
        if streams:
            # new stream t = sum_s mix[s, t] * old stream s + out[t] * y
            return torch.einsum("st,snw->tnw", w[hc + ".mix"], xs) + w[hc + ".out"][:, None, None] * y[None]
        return xs + y

    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}"
        mixer = MIXERS[layer["type"]]
        xs = sublayer(xs, i, 1, lambda hh: mixer(hh, w, p + ".mix", layer["mixer"], eps))
        if layer.get("mlp") is not None:
            if layer["mlp"]["kind"] != "dense":
                raise ValueError("unknown feed-forward kind")
            xs = sublayer(xs, i, 2, lambda hh: plain_dense_ff(hh, w, p + ".mlp"))
        after.append(xs.sum(0) if streams else xs)
    x = xs.sum(0) if streams else xs
    logits = (plain_rms(x, eps) * w["final.norm"]) @ w["embed"].T
    if return_layers:
        return logits, torch.stack(after)
    return logits
