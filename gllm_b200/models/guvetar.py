"""``Guvetar`` as a ModelSpec: token embedding plus a sinusoid of the position (base 10000), a residual
of ``streams`` parallel streams (or one plain residual), layers whose mixer is a selective scan
("mamba1"), a matrix memory with exponential gates ("mlstm") or sigmoid attention beside gated linear
attention ("parallel"), each followed by an optional dense feed-forward with a squared ReLU, RMS norm
with the weight multiplying directly, and the embedding table as the output head.

Tensor names: ``embed``, ``final.norm``; layer ``i``: ``l<i>.norm1|norm2``, ``l<i>.mix.*`` (the mixer),
``l<i>.mlp.up|down``, ``l<i>.hc1|hc2.in|out|mix`` (how the mixer / the feed-forward reads and writes the
streams).
"""

from __future__ import annotations

from gllm_b200.config.guvetar_config import GuvetarConfig
from gllm_b200.config.registry import register_architecture
from gllm_b200.models.spec import LayerSpec, ModelSpec, PartSpec, PlanEntry

SINUSOID_BASE = 10000.0


def _mixer_spec(cfg: GuvetarConfig, kind: str, m: dict, p: str) -> PartSpec:
    width, eps = cfg.hidden_size, cfg.norm_eps
    if kind == "mamba1":
        return PartSpec(
            "selective_scan",
            dict(hidden_size=width, inner=m["inner"], states=m["state"], dt_rank=m["dt_rank"], taps=m["conv"]),
            {"in": f"{p}.in", "conv": f"{p}.conv", "conv_bias": f"{p}.conv.b", "x": f"{p}.x", "dt": f"{p}.dt",
             "dt_bias": f"{p}.dt.b", "A_log": f"{p}.A_log", "D": f"{p}.D", "o": f"{p}.o"},
        )
    if kind == "mlstm":
        return PartSpec(
            "exp_gated_memory",
            dict(hidden_size=width, heads=m["heads"], dk=m["dim"], dv=m["vdim"], gate_cap=m["gate_cap"], eps=eps),
            {**{n: f"{p}.{n}" for n in ("q", "k", "v", "g", "o", "norm", "i", "f")},
             "i_bias": f"{p}.i.b", "f_bias": f"{p}.f.b"},
        )
    if kind == "parallel":
        lm, rm = m["left"], m["right"]
        left = PartSpec(
            "sigmoid_attention",
            dict(hidden_size=width, heads=lm["heads"], kv_heads=lm["kv_heads"], dk=lm["dim"], dv=lm["vdim"],
                 scale=lm["scale"], eps=eps, query_temperature=lm.get("q_temp")),
            {**{n: f"{p}.left.{n}" for n in ("q", "k", "v", "o")}, "q_norm": f"{p}.left.q.norm",
             "k_norm": f"{p}.left.k.norm", "head_bias": f"{p}.left.pb"},
        )
        right = PartSpec(
            "gated_linear_attention",
            dict(hidden_size=width, heads=rm["heads"], dk=rm["dim"], dv=rm["vdim"], eps=eps),
            {**{n: f"{p}.right.{n}" for n in ("q", "f", "v", "norm", "o", "lower")}, "f_bias": f"{p}.right.f.b"},
        )
        return PartSpec("parallel", dict(left=left, right=right, left_scale=m["left_scale"],
                                         right_scale=m["right_scale"]))
    raise ValueError(f"unknown layer type {kind!r}")


def build_guvetar_spec(cfg: GuvetarConfig) -> ModelSpec:
    width, eps, streams = cfg.hidden_size, cfg.norm_eps, cfg.streams

    def norm(weight: str, connection: str | None) -> PartSpec:
        if streams is None:
            return PartSpec("rmsnorm", dict(size=width, eps=eps), {"weight": weight})
        names = {"weight": weight}
        if connection is not None:
            names.update(read=f"{connection}.in", write=f"{connection}.out", mix=f"{connection}.mix")
        return PartSpec("stream_rmsnorm", dict(size=width, streams=streams, eps=eps, connected=connection is not None),
                        names)

    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}"
        parts = {"mixer_norm": norm(f"{p}.norm1", f"{p}.hc1"), "mixer": _mixer_spec(cfg, layer.type, layer.mixer, f"{p}.mix")}
        if layer.mlp is not None:
            parts["feed_forward_norm"] = norm(f"{p}.norm2", f"{p}.hc2")
            parts["feed_forward"] = PartSpec(
                "dense", dict(hidden_size=width, intermediate_size=layer.mlp["ff"], activation="relu_squared"),
                {"up": f"{p}.mlp.up", "down": f"{p}.mlp.down"})
        layers.append(LayerSpec("prenorm" if streams is None else "stream_prenorm", parts))
    return ModelSpec(
        hidden_size=width,
        vocab_size=cfg.vocab_size,
        layers=tuple(layers),
        plan=tuple(PlanEntry(i) for i in range(len(layers))),
        final_norm=norm("final.norm", None),
        embedding_name="embed",
        head_name=None,
        eos_token_ids=cfg.eos_token_ids,
        position_sinusoid_base=SINUSOID_BASE,
        residual_streams=streams or 1,
    )


register_architecture("Guvetar", GuvetarConfig, build_guvetar_spec)
