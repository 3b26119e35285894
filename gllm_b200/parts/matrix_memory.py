"""Mixers whose state is a matrix per head, ``S <- diag(a) S + b v^T``, ``o = S^T q``
(``csrc/recurrent.cu``), kept in fp32 per request.

``gated_linear_attention``: the forget gate also decides what is written.  ``q = silu(W_q h)``,
``v = W_v h``, ``f = lower + (1 - lower) * sigmoid(W_f h + b_f)`` per (head, key channel), ``a = f``,
``b = 1 - f``; there is no key and no other scale.  Each head's output is RMS-normed with one weight
shared by the heads, then ``W_o``.

``exp_gated_memory``: a matrix memory with exponential gates.  ``q = W_q h / sqrt(dk)``, ``k = W_k h``,
``v = W_v h``; per head a log input gate ``i = cap * tanh((W_i h + b_i) / cap)`` and a log forget gate
``f = logsigmoid(cap * tanh((W_f h + b_f) / cap))``; a running maximum ``m`` (from 0) keeps the
exponentials bounded: ``m' = max(f + m, i)``, ``S <- exp(f + m - m') S + exp(i - m') k v^T``, a
normaliser ``n`` likewise with ``k`` alone, ``o = S^T q / (max(|n . q|, exp(-m')) + 1e-6)``.  Each
head's ``o`` is divided by its root mean square, the concatenation is multiplied by a weight of its
whole size and by ``sigmoid(W_g h)``, then ``W_o``.
"""

from __future__ import annotations

import torch

from gllm_b200 import ops
from gllm_b200.ops import stateful
from gllm_b200.parts.base import Mixer, StateRequirement, TensorExpectation, register_mixer


def _check_sizes(dk: int, dv: int) -> None:
    if not (1 <= dk <= 512 and dv >= 1):
        raise ValueError("the matrix recurrence takes up to 512 key channels per head")


@register_mixer("gated_linear_attention")
class GatedLinearAttention(Mixer):
    graph_safe_portions = True

    def __init__(self, names, hidden_size: int, heads: int, dk: int, dv: int, eps: float):
        super().__init__(names)
        self.hidden_size, self.heads, self.dk, self.dv, self.eps = int(hidden_size), int(heads), int(dk), int(dv), float(eps)
        _check_sizes(self.dk, self.dv)
        self.w_qv = self.w_f = self.w_o = self.f_bias = self.lower = self.norm = None

    def kernel_needs(self):
        return {"modules": {"recurrent"}}

    def state_requirement(self):
        return StateRequirement((self.heads, self.dv, self.dk), torch.float32)

    def expected_tensors(self):
        n, hk, hv = self.names, self.heads * self.dk, self.heads * self.dv
        return {
            n["q"]: TensorExpectation((hk, self.hidden_size)),
            n["f"]: TensorExpectation((hk, self.hidden_size)),
            n["f_bias"]: TensorExpectation((hk,), "bias"),
            n["lower"]: TensorExpectation((hk,), "bias"),
            n["v"]: TensorExpectation((hv, self.hidden_size)),
            n["norm"]: TensorExpectation((self.dv,), "vector"),
            n["o"]: TensorExpectation((self.hidden_size, hv)),
        }

    def load(self, get, dtype, device):
        n = self.names
        self.w_qv = torch.cat([get(n["q"], "matrix"), get(n["v"], "matrix")], 0).contiguous()
        self.w_f, self.w_o = get(n["f"], "matrix"), get(n["o"], "matrix")
        self.f_bias, self.lower, self.norm = get(n["f_bias"], "bias"), get(n["lower"], "bias"), get(n["norm"], "vector")

    def forward(self, x, ctx, cache):
        hk = self.heads * self.dk
        qv = ops.linear(x, self.w_qv)
        gates = ops.linear(x, self.w_f, out_dtype=torch.float32)      # the gate of the recurrence stays fp32
        o = stateful.matrix_recurrence(stateful.GATED_LINEAR, qv[:, :hk], None, qv[:, hk:], gates, self.f_bias,
                                       self.lower, 0.0, 1.0, cache.states[0], None, ctx.cu_q, ctx.state_slots,
                                       ctx.num_requests, self.heads, self.dk, self.dv, max_q_len=ctx.max_q_len)
        normed = stateful.head_norm(o, self.heads, self.dv, self.norm, self.eps, x.dtype)
        return ops.linear(normed, self.w_o, split_ok=True, add_into=getattr(ctx, "residual_sink", None))


@register_mixer("exp_gated_memory")
class ExpGatedMemory(Mixer):
    graph_safe_portions = True
    DENOMINATOR_EPS = 1e-6

    def __init__(self, names, hidden_size: int, heads: int, dk: int, dv: int, gate_cap: float, eps: float):
        super().__init__(names)
        self.hidden_size, self.heads, self.dk, self.dv = int(hidden_size), int(heads), int(dk), int(dv)
        self.gate_cap, self.eps = float(gate_cap), float(eps)
        _check_sizes(self.dk, self.dv)
        self.w_qkvg = self.w_if = self.w_o = self.if_bias = self.norm = None

    def kernel_needs(self):
        return {"modules": {"recurrent"}}

    def state_requirement(self):
        # the memory, column by column, with its normaliser as one more column, and the running maximum
        return (StateRequirement((self.heads, self.dv + 1, self.dk), torch.float32),
                StateRequirement((self.heads,), torch.float32))

    def expected_tensors(self):
        n, hk, hv = self.names, self.heads * self.dk, self.heads * self.dv
        return {
            n["q"]: TensorExpectation((hk, self.hidden_size)),
            n["k"]: TensorExpectation((hk, self.hidden_size)),
            n["v"]: TensorExpectation((hv, self.hidden_size)),
            n["g"]: TensorExpectation((hv, self.hidden_size)),
            n["o"]: TensorExpectation((self.hidden_size, hv)),
            n["norm"]: TensorExpectation((hv,), "vector"),
            n["i"]: TensorExpectation((self.heads, self.hidden_size)),
            n["i_bias"]: TensorExpectation((self.heads,), "bias"),
            n["f"]: TensorExpectation((self.heads, self.hidden_size)),
            n["f_bias"]: TensorExpectation((self.heads,), "bias"),
        }

    def load(self, get, dtype, device):
        n = self.names
        self.w_qkvg = torch.cat([get(n[k], "matrix") for k in ("q", "k", "v", "g")], 0).contiguous()
        self.w_if = torch.cat([get(n["i"], "matrix"), get(n["f"], "matrix")], 0).contiguous()
        self.if_bias = torch.cat([get(n["i_bias"], "bias"), get(n["f_bias"], "bias")]).contiguous()
        self.w_o, self.norm = get(n["o"], "matrix"), get(n["norm"], "vector")

    def forward(self, x, ctx, cache):
        hk, hv = self.heads * self.dk, self.heads * self.dv
        qkvg = ops.linear(x, self.w_qkvg)
        gates = ops.linear(x, self.w_if, out_dtype=torch.float32)     # the gates of the recurrence stay fp32
        memory, maximum = cache.states
        o = stateful.matrix_recurrence(stateful.EXP_GATED, qkvg[:, :hk], qkvg[:, hk:2 * hk], qkvg[:, 2 * hk:2 * hk + hv],
                                       gates, self.if_bias, None, self.gate_cap, self.dk ** -0.5, memory, maximum,
                                       ctx.cu_q, ctx.state_slots, ctx.num_requests, self.heads, self.dk, self.dv, max_q_len=ctx.max_q_len)
        normed = stateful.head_norm(o, self.heads, self.dv, self.norm, self.eps, x.dtype, with_denominator=True,
                                    denominator_eps=self.DENOMINATOR_EPS, gate=qkvg[:, 2 * hk + hv:])
        return ops.linear(normed, self.w_o, split_ok=True, add_into=getattr(ctx, "residual_sink", None))
