"""``Rulunex`` as a ModelSpec: a scaled token embedding; layers of the ``shared_norm`` block (one RMS norm whose
weight is stored as an offset from one, read by the mixer and the feed-forward side by side); the mixer is
``latent_attention`` (softmax attention over one cached latent per token, rotated key part shared by the heads,
neighbouring rotary pairs, a sigmoid gate per head) or ``attention`` (grouped-query attention in a sliding
window, q and k RMS-normed over their whole projections, values = the keys as projected, rotary pairs of the two
halves with optional long-wavelength scaling); the feed-forward is ``clamped_glu``; layers ``loop.start ..
loop.stop-1`` run ``loop.times`` times with the same weights (every pass with caches of its own, and beginning
with the ``loop.in`` projection of ``[x ; embedding output]``); the embedding table is the output head.

Tensor names: ``embed``, ``final.norm``, ``loop.in``; layer ``i``: ``l<i>.norm1``, ``l<i>.mix.*`` (the mixer),
``l<i>.mlp.gate|up|down``.
"""

from __future__ import annotations

from gllm_b200.config.registry import register_architecture
from gllm_b200.config.rulunex_config import RulunexConfig
from gllm_b200.models.spec import LayerSpec, ModelSpec, PartSpec, PlanEntry

# the design's fixed constants: the feed-forward's gate is g * sigmoid(1.702 g), its up branch is u + 1
GATE_SIGMOID_SLOPE = 1.702
UP_OFFSET = 1.0


def _rotary(rot: dict, head_dim: int, interleaved: bool) -> PartSpec:
    scaling = rot.get("scaling")
    if scaling is not None:
        scaling = {"rope_type": "llama3", "factor": scaling["factor"], "low_freq_factor": scaling["low"],
                   "high_freq_factor": scaling["high"], "original_max_position_embeddings": scaling["original"]}
    return PartSpec("rotary", dict(head_dim=head_dim, rotary_dim=int(rot["dims"]), theta=float(rot["base"]),
                                   scaling=scaling, interleaved=interleaved))


def _mixer_spec(cfg: RulunexConfig, kind: str, m: dict, p: str) -> PartSpec:
    width, eps = cfg.hidden_size, cfg.norm_eps
    if kind == "latent_attention":
        return PartSpec(
            "latent_attention",
            dict(hidden_size=width, heads=m["heads"], dim=m["dim"], rot_dim=m["rot_dim"], vdim=m["vdim"],
                 kv_rank=m["kv_rank"], scale=m["scale"], eps=eps, gated=True,
                 position=_rotary(m["rot"], m["rot_dim"], interleaved=True)),
            {**{n: f"{p}.{n}" for n in ("q", "dkv", "uk", "uv", "g", "o")}, "dkv_norm": f"{p}.dkv.norm"},
        )
    if kind == "attention":
        mask = m.get("mask")
        return PartSpec(
            "attention",
            dict(hidden_size=width, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                 scale=m["scale"], window=None if mask is None else int(mask["size"]), qk_norm_eps=eps,
                 qk_norm_whole=True, values_from_keys=True,
                 position=_rotary(m["rot"], m["dim"], interleaved=False) if int(m["rot"]["dims"]) > 0 else None),
            {"q": f"{p}.q", "k": f"{p}.k", "o": f"{p}.o", "q_norm": f"{p}.q.norm", "k_norm": f"{p}.k.norm"},
        )
    raise ValueError(f"unknown layer type {kind!r}")


def layer_order(cfg: RulunexConfig) -> list[tuple[int, bool]]:
    """(layer, begins a pass of the repeated stretch) in running order."""
    n = len(cfg.layers)
    if cfg.loop is None:
        return [(i, False) for i in range(n)]
    start, stop, times = cfg.loop
    order = [(i, False) for i in range(start)]
    for _ in range(times):
        order += [(i, i == start) for i in range(start, stop)]
    return order + [(i, False) for i in range(stop, n)]


def build_rulunex_spec(cfg: RulunexConfig) -> ModelSpec:
    width, eps = cfg.hidden_size, cfg.norm_eps

    def norm(weight: str) -> PartSpec:
        return PartSpec("rmsnorm", dict(size=width, eps=eps, unit_offset=True), {"weight": weight})

    layers = []
    for i, layer in enumerate(cfg.layers):
        p = f"l{i}"
        parts = {"norm": norm(f"{p}.norm1"), "mixer": _mixer_spec(cfg, layer.type, layer.mixer, f"{p}.mix")}
        if layer.mlp is not None:
            parts["feed_forward"] = PartSpec(
                "clamped_glu",
                dict(hidden_size=width, intermediate_size=layer.mlp["ff"], limit=layer.mlp["limit"],
                     slope=GATE_SIGMOID_SLOPE, up_offset=UP_OFFSET),
                {n: f"{p}.mlp.{n}" for n in ("gate", "up", "down")})
        layers.append(LayerSpec("shared_norm", parts))
    return ModelSpec(
        hidden_size=width,
        vocab_size=cfg.vocab_size,
        layers=tuple(layers),
        plan=tuple(PlanEntry(i, rejoins_embedding=begins) for i, begins in layer_order(cfg)),
        final_norm=norm("final.norm"),
        embedding_name="embed",
        head_name=None,
        eos_token_ids=cfg.eos_token_ids,
        embedding_scale=cfg.embedding_scale,
        rejoin_name="loop.in" if cfg.loop is not None else None,
    )


register_architecture("Rulunex", RulunexConfig, build_rulunex_spec)
