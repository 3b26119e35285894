"""A residual kept as several streams (hyper-connections), as a norm kind and a block kind.

Instead of one residual ``x`` there are ``streams`` copies, all equal to the embedding at the start.
A sublayer reads ``u = sum_s read[s] x_s``, runs on the RMS norm of ``u``, and its result ``y`` is
written back to all streams at once from the old ones: ``x_t <- sum_s mix[s, t] x_s + write[t] y``
(``mix`` is indexed [from, to]).  After the last layer the streams are summed.

The single-stream block defers each add to the norm kernel that follows it; the same protocol is kept
here.  ``StreamNorm`` owns a sublayer's three connection tensors beside its norm weight; the block
hands the sublayer's result on as a ``StreamWrite`` (the result with the ``mix`` and ``write`` it is
to be written with), and the next ``StreamNorm`` (the next sublayer's, the next layer's, or the
model's final norm, which reads the plain sum) does that write and its own read + norm in one kernel.
"""

from __future__ import annotations

from dataclasses import dataclass

import torch

from gllm_b200 import ops
from gllm_b200.ops import stateful
from gllm_b200.parts.base import Block, Norm, TensorExpectation, register_block, register_norm


@dataclass
class StreamWrite:
    """A sublayer's result that has not been written into the streams yet."""

    y: torch.Tensor
    mix: torch.Tensor       # [streams, streams] fp32, [from, to]
    write: torch.Tensor     # [streams] fp32


@register_norm("stream_rmsnorm")
class StreamNorm(Norm):
    """RMS norm of a weighted sum of the residual streams.  ``connected`` False: it has no connection
    tensors of its own and reads the plain sum of the streams (a model's final norm)."""

    graph_safe_portions = True

    def __init__(self, names, size: int, streams: int, eps: float, connected: bool = True):
        super().__init__(names)
        self.size, self.streams, self.eps, self.connected = int(size), int(streams), float(eps), bool(connected)
        self.weight = self.read = self.mix = self.write = None

    def kernel_needs(self):
        return {"modules": {"hyper_streams"}}

    def expected_tensors(self):
        exp = {self.names["weight"]: TensorExpectation((self.size,), "vector")}
        if self.connected:
            exp[self.names["read"]] = TensorExpectation((self.streams,), "vector")
            exp[self.names["write"]] = TensorExpectation((self.streams,), "vector")
            exp[self.names["mix"]] = TensorExpectation((self.streams, self.streams), "mixing")
        return exp

    def load(self, get, dtype, device):
        self.weight = get(self.names["weight"], "vector")
        if self.connected:
            self.read = get(self.names["read"], "vector")
            self.write = get(self.names["write"], "vector")
            self.mix = get(self.names["mix"], "mixing")

    def pending(self, y) -> StreamWrite:
        """``y``, the result of the sublayer this norm fed, with the tensors it is written back with."""
        return StreamWrite(ops.as_tensor(y), self.mix, self.write)

    def forward(self, branch, resid, dtype, rows=None):
        if branch is not None and not isinstance(branch, StreamWrite):
            raise TypeError("a stream norm takes the result of a sublayer as a StreamWrite")
        y, mix, write = (branch.y, branch.mix, branch.write) if branch is not None else (None, None, None)
        return stateful.stream_mix_norm(y, resid, mix, write, self.read, self.weight, self.eps, dtype, self.streams,
                                        rows=rows)


@register_block("stream_prenorm")
class StreamPreNormBlock(Block):
    """``mixer`` then (optionally) ``feed_forward``, each on the norm of its read of the streams."""

    graph_safe_portions = True
    part_kinds = {"mixer_norm": "norm", "mixer": "mixer", "feed_forward_norm": "norm", "feed_forward": "feed_forward"}
    optional_parts = frozenset({"feed_forward_norm", "feed_forward"})

    def forward(self, branch, resid, ctx, cache):
        ctx.residual_sink = None          # a write into the streams is not a plain add: no product adds itself
        x = self.mixer_norm.forward(branch, resid, ctx.dtype)
        branch = self.mixer_norm.pending(self.mixer.forward(x, ctx, cache))
        if self.feed_forward is not None:
            x = self.feed_forward_norm.forward(branch, resid, ctx.dtype)
            branch = self.feed_forward_norm.pending(self.feed_forward.forward(x, ctx))
        return branch, resid
