"""``Guvetar``'s own config.json keys as a typed configuration.

config.json names ``architecture`` (a string), ``vocab``, ``width``, ``norm.eps``, optionally
``streams`` (the number of residual streams; absent: one plain residual), and ``layers``: one entry
per layer with ``type`` (which mixer: "mamba1" | "mlstm" | "parallel"), ``mixer`` (that mixer's
sizes and constants) and ``mlp`` (``{"kind": "dense", "ff": n}``, or null for a layer without a
feed-forward).  Every size and constant the model uses comes from here or from a tensor's shape.
"""

from __future__ import annotations

import copy
from dataclasses import dataclass, field
from typing import Any

from gllm_b200.config.model_config import DTYPE_NAMES, ConfigError, ModelConfig, as_eos, require

MIXER_KEYS = {
    "mamba1": ("conv", "dt_rank", "inner", "state"),
    "mlstm": ("dim", "heads", "vdim", "gate_cap"),
    "parallel": ("left", "right", "left_scale", "right_scale"),
}
LEFT_KEYS = ("dim", "heads", "kv_heads", "vdim", "scale")
RIGHT_KEYS = ("dim", "heads", "vdim")
FEED_FORWARD_KINDS = ("dense",)


@dataclass(frozen=True)
class GuvetarLayer:
    type: str
    mixer: dict[str, Any]
    mlp: dict[str, Any] | None

    @classmethod
    def from_dict(cls, index: int, d: dict) -> "GuvetarLayer":
        where = f"layers[{index}]"
        kind = require(d, "type")
        if kind not in MIXER_KEYS:
            raise ConfigError(f"{where}: unknown layer type {kind!r}; known: {sorted(MIXER_KEYS)}")
        mixer = require(d, "mixer")
        for key in MIXER_KEYS[kind]:
            if key not in mixer:
                raise ConfigError(f"{where}.mixer lacks {key!r}")
        if kind == "parallel":
            for side, keys in (("left", LEFT_KEYS), ("right", RIGHT_KEYS)):
                for key in keys:
                    if key not in mixer[side]:
                        raise ConfigError(f"{where}.mixer.{side} lacks {key!r}")
            temp = mixer["left"].get("q_temp")
            if temp is not None and ("coef" not in temp or "every" not in temp or not temp["every"] > 0):
                raise ConfigError(f"{where}.mixer.left.q_temp needs 'coef' and a positive 'every'")
            if mixer["left"]["heads"] % mixer["left"]["kv_heads"]:
                raise ConfigError(f"{where}.mixer.left: heads is not a multiple of kv_heads")
        mlp = d.get("mlp")
        if mlp is not None:
            if mlp.get("kind") not in FEED_FORWARD_KINDS:
                raise ConfigError(f"{where}.mlp: unknown kind {mlp.get('kind')!r}; known: {list(FEED_FORWARD_KINDS)}")
            if int(require(mlp, "ff")) <= 0:
                raise ConfigError(f"{where}.mlp.ff must be positive")
        return cls(kind, copy.deepcopy(mixer), copy.deepcopy(mlp))

    def to_dict(self) -> dict:
        return {"type": self.type, "mixer": copy.deepcopy(self.mixer), "mlp": copy.deepcopy(self.mlp)}


@dataclass(frozen=True)
class GuvetarConfig(ModelConfig):
    """A decoder of mixed layers (selective scan, matrix memory, sigmoid attention beside gated linear
    attention) over a residual of one or several streams, with sinusoidal positions added to the
    embedding and the embedding table as output head."""

    layers: tuple[GuvetarLayer, ...] = field(default_factory=tuple)
    norm_eps: float = 0.0
    streams: int | None = None

    @classmethod
    def from_dict(cls, d: dict[str, Any]) -> "GuvetarConfig":
        arch = d.get("architecture") or (d.get("architectures") or [None])[0]
        layers = require(d, "layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("'layers' must be a non-empty list")
        dtype = d.get("torch_dtype", d.get("dtype", "bfloat16"))
        if dtype not in DTYPE_NAMES:
            raise ConfigError(f"unsupported dtype {dtype!r}")
        streams = d.get("streams")
        if streams is not None and not 1 <= int(streams) <= 16:
            raise ConfigError("'streams' must be between 1 and 16")
        vocab, width = int(require(d, "vocab")), int(require(d, "width"))
        if vocab <= 0 or width <= 0:
            raise ConfigError("'vocab' and 'width' must be positive")
        return cls(
            architecture=str(arch), vocab_size=vocab, hidden_size=width, dtype=DTYPE_NAMES[dtype],
            eos_token_ids=as_eos(d.get("eos_token_id")),
            layers=tuple(GuvetarLayer.from_dict(i, layer) for i, layer in enumerate(layers)),
            norm_eps=float(require(require(d, "norm"), "eps")),
            streams=None if streams is None else int(streams),
        )

    def to_dict(self) -> dict[str, Any]:
        out: dict[str, Any] = {
            "architecture": self.architecture,
            "layers": [layer.to_dict() for layer in self.layers],
            "norm": {"eps": self.norm_eps},
            "vocab": self.vocab_size,
            "width": self.hidden_size,
            "torch_dtype": self.dtype,
        }
        if self.streams is not None:
            out["streams"] = self.streams
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out
