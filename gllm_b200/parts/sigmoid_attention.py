"""Causal attention without a softmax over the paged cache: the weight of a visible key is
``sigmoid(q . k * scale + bias[head])`` and the weights are not normalised over the keys.

``q = W_q h`` (heads x dk), ``k = W_k h`` (kv_heads x dk), ``v = W_v h`` (kv_heads x dv), query head
``h`` using key/value head ``h // (heads / kv_heads)``; queries and keys are RMS-normed per head with
one weight each, shared by the heads; no rotation: positions enter only through an optional query
multiplier ``1 + coef * ln(floor((p + 1) / every) + 1)``.  Keys (normed) and values are cached in pages
whose key and value widths may differ; norms, scores, weights and the sum over the keys are fp32.
"""

from __future__ import annotations

import torch

from gllm_b200 import ops
from gllm_b200.ops import stateful
from gllm_b200.parts.base import KVPageRequirement, Mixer, TensorExpectation, register_mixer


@register_mixer("sigmoid_attention")
class SigmoidAttention(Mixer):
    graph_safe_portions = True

    def __init__(self, names, hidden_size: int, heads: int, kv_heads: int, dk: int, dv: int, scale: float, eps: float,
                 query_temperature: dict | None = None):
        super().__init__(names)
        if heads % kv_heads:
            raise ValueError("heads must be a multiple of kv_heads")
        if dk > 256 or dv > 256:
            raise ValueError("the sigmoid-attention kernel takes key and value widths up to 256")
        self.hidden_size, self.heads, self.kv_heads = int(hidden_size), int(heads), int(kv_heads)
        self.dk, self.dv, self.scale, self.eps = int(dk), int(dv), float(scale), float(eps)
        self.temp_coef = float(query_temperature["coef"]) if query_temperature else 0.0
        self.temp_every = float(query_temperature["every"]) if query_temperature else 1.0
        self.w_qkv = self.w_o = self.q_norm = self.k_norm = self.head_bias = None

    def kernel_needs(self):
        return {"modules": {"attention_sigmoid", "attention_sigmoid_mma"}}

    def kv_requirement(self):
        return KVPageRequirement(((self.kv_heads, self.dk), (self.kv_heads, self.dv)), None)

    def expected_tensors(self):
        n = self.names
        return {
            n["q"]: TensorExpectation((self.heads * self.dk, self.hidden_size)),
            n["k"]: TensorExpectation((self.kv_heads * self.dk, self.hidden_size)),
            n["v"]: TensorExpectation((self.kv_heads * self.dv, self.hidden_size)),
            n["q_norm"]: TensorExpectation((self.dk,), "vector"),
            n["k_norm"]: TensorExpectation((self.dk,), "vector"),
            n["head_bias"]: TensorExpectation((self.heads,), "bias"),
            n["o"]: TensorExpectation((self.hidden_size, self.heads * self.dv)),
        }

    def load(self, get, dtype, device):
        n = self.names
        self.w_qkv = torch.cat([get(n[k], "matrix") for k in ("q", "k", "v")], 0).contiguous()
        self.w_o = get(n["o"], "matrix")
        self.q_norm, self.k_norm = get(n["q_norm"], "vector"), get(n["k_norm"], "vector")
        self.head_bias = get(n["head_bias"], "bias")

    def forward(self, x, ctx, cache):
        view = ctx.groups[cache.group]
        qkv = ops.as_tensor(ops.linear(x, self.w_qkv))
        stateful.qk_norm_store(qkv, self.q_norm, self.k_norm, self.eps, self.temp_coef, self.temp_every, ctx.positions,
                               view.slot_mapping if cache.writes else None, cache.pages, self.heads, self.kv_heads,
                               self.dk, self.dv, cache.block_size)
        attn = stateful.sigmoid_attention(qkv, cache.pages, view.block_table, ctx.positions, ctx.token_row,
                                          self.head_bias, self.heads, self.kv_heads, self.dk, self.dv, cache.block_size,
                                          self.scale, batch=ctx)
        return ops.linear(attn, self.w_o, split_ok=True, add_into=getattr(ctx, "residual_sink", None))
