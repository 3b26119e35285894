"""``Rulunex``'s own config.json keys as a typed configuration.

config.json names ``architecture`` (a string), ``vocab``, ``width``, ``norm.eps``, ``embedding.scale``,
``layers``: one entry per layer with ``type`` (which mixer: "latent_attention" | "attention"), ``mixer`` (that
mixer's sizes and constants) and ``mlp`` (``{"kind": "dense", "ff": n, "limit": x}``, or null for a layer
without a feed-forward), and optionally ``loop`` (``start``, ``stop``, ``times``: layers ``start .. stop-1`` run
``times`` times in a row with the same weights).  Every size and constant the model uses comes from here or
from a tensor's shape.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any

from gllm_b200.config.model_config import DTYPE_NAMES, ConfigError, ModelConfig, as_eos, require

MIXER_KEYS = {
    "latent_attention": ("heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot"),
    "attention": ("heads", "kv_heads", "dim", "vdim", "scale", "rot"),
}
FEED_FORWARD_KINDS = ("dense",)
SCALING_KEYS = ("factor", "low", "high", "original")


@dataclass(frozen=True)
class RulunexLayer:
    type: str
    mixer: dict[str, Any]
    mlp: dict[str, Any] | None

    @classmethod
    def from_dict(cls, index: int, d: dict) -> "RulunexLayer":
        where = f"layers[{index}]"
        kind = require(d, "type")
        if kind not in MIXER_KEYS:
            raise ConfigError(f"{where}: unknown layer type {kind!r}; known: {sorted(MIXER_KEYS)}")
        mixer = require(d, "mixer")
        for key in MIXER_KEYS[kind]:
            if key not in mixer:
                raise ConfigError(f"{where}.mixer lacks {key!r}")
        rot = mixer["rot"]
        if "base" not in rot or "dims" not in rot:
            raise ConfigError(f"{where}.mixer.rot needs 'base' and 'dims'")
        if int(rot["dims"]) % 2 or int(rot["dims"]) < 0:
            raise ConfigError(f"{where}.mixer.rot.dims must be even")
        scaling = rot.get("scaling")
        if scaling is not None:
            for key in SCALING_KEYS:
                if key not in scaling:
                    raise ConfigError(f"{where}.mixer.rot.scaling lacks {key!r}")
        if kind == "attention":
            if int(mixer["heads"]) % int(mixer["kv_heads"]):
                raise ConfigError(f"{where}.mixer: heads is not a multiple of kv_heads")
            if int(mixer["vdim"]) != int(mixer["dim"]):
                raise ConfigError(f"{where}.mixer: the values are the keys, so vdim must equal dim")
            if int(rot["dims"]) > int(mixer["dim"]):
                raise ConfigError(f"{where}.mixer.rot.dims exceeds dim")
            mask = mixer.get("mask")
            if mask is not None and int(require(mask, "size")) <= 0:
                raise ConfigError(f"{where}.mixer.mask.size must be positive")
        else:
            if int(rot["dims"]) > int(mixer["rot_dim"]):
                raise ConfigError(f"{where}.mixer.rot.dims exceeds rot_dim")
        mlp = d.get("mlp")
        if mlp is not None:
            if mlp.get("kind") not in FEED_FORWARD_KINDS:
                raise ConfigError(f"{where}.mlp: unknown kind {mlp.get('kind')!r}; known: {list(FEED_FORWARD_KINDS)}")
            if int(require(mlp, "ff")) <= 0:
                raise ConfigError(f"{where}.mlp.ff must be positive")
            if not float(require(mlp, "limit")) > 0:
                raise ConfigError(f"{where}.mlp.limit must be positive")
        return cls(kind, copy.deepcopy(mixer), copy.deepcopy(mlp))

    def to_dict(self) -> dict:
        return {"type": self.type, "mixer": copy.deepcopy(self.mixer), "mlp": copy.deepcopy(self.mlp)}


@dataclass(frozen=True)
class RulunexConfig(ModelConfig):
    """A decoder whose layers put a mixer (latent attention, or windowed attention whose values are its keys)
    and a clamped gated feed-forward side by side behind one norm, with a stretch of layers that may run
    several times, and the embedding table as output head."""

    layers: tuple[RulunexLayer, ...] = field(default_factory=tuple)
    norm_eps: float = 0.0
    embedding_scale: float = 1.0
    # (start, stop, times) or None
    loop: tuple[int, int, int] | None = None

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "RulunexConfig":
        arch = d.get("architecture") or (d.get("architectures") or [None])[0]
        layers = require(d, "layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("'layers' must be a non-empty list")
        dtype = d.get("torch_dtype", d.get("dtype", "bfloat16"))
        if dtype not in DTYPE_NAMES:
            raise ConfigError(f"unsupported dtype {dtype!r}")
        vocab, width = int(require(d, "vocab")), int(require(d, "width"))
        if vocab <= 0 or width <= 0:
            raise ConfigError("'vocab' and 'width' must be positive")
        loop = d.get("loop")
        if loop is not None:
            start, stop, times = (int(require(loop, k)) for k in ("start", "stop", "times"))
            if not 0 <= start < stop <= len(layers) or times < 0:
                raise ConfigError("'loop' needs 0 <= start < stop <= number of layers and times >= 0")
            loop = (start, stop, times)
        return cls(
            architecture=str(arch), vocab_size=vocab, hidden_size=width, dtype=DTYPE_NAMES[dtype],
            eos_token_ids=as_eos(d.get("eos_token_id")),
            layers=tuple(RulunexLayer.from_dict(i, layer) for i, layer in enumerate(layers)),
            norm_eps=float(require(require(d, "norm"), "eps")),
            embedding_scale=float(require(require(d, "embedding"), "scale")),
            loop=loop,
        )

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {
            "architecture": self.architecture,
            "embedding": {"scale": self.embedding_scale},
            "layers": [layer.to_dict() for layer in self.layers],
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab_size,
            "width": self.hidden_size,
            "torch_dtype": self.dtype,
        }
        if self.loop is not None:
            out["loop"] = dict(zip(("start", "stop", "times"), self.loop))
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
