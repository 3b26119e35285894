"""Softmax attention over one cached latent vector per token (multi-head latent attention).

``q = W_q h`` is laid out head by head as ``[plain (dim) ; rotated (rot_dim)]``.  ``W_dkv h`` has
``kv_rank + rot_dim`` rows: the first ``kv_rank``, RMS-normed, are the latent ``c``; the last ``rot_dim``,
rotated by the position, are one key part ``kr`` shared by all heads.  Head ``n``'s key is
``[W_uk[n] c ; kr]`` and its value ``W_uv[n] c``; the score is ``(q_plain . k_plain + q_rot . kr) * scale``,
causal softmax; optionally every head's result is multiplied by ``sigmoid(W_g h)[n]``; then ``W_o``.

Only ``[c ; kr]`` is cached (one "head" of ``kv_rank + rot_dim`` numbers per token).  Both up-projections act
on the query's side: ``qa = W_uk[n]^T q_plain`` is scored against the cached ``c`` directly, the weighted sum of
the ``c`` is taken, and ``W_uv[n]`` maps that sum to the head's value width.  One product gives q, the
down-projection and the gate logits; norms, angles, scores and the softmax are fp32.
"""

from __future__ import annotations

import torch

from gllm_b200 import ops
from gllm_b200.ops import latent
from gllm_b200.parts.base import (POSITION_ENCODINGS, KVPageRequirement, Mixer, TensorExpectation, build_part,
                                  register_mixer)


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    graph_safe_portions = True

    def __init__(self, names, hidden_size: int, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int,
                 scale: float, eps: float, position, gated: bool = False):
        """``position``: a PartSpec of the rotary family over ``rot_dim`` columns (pairs of neighbours);
        ``gated``: the per-head sigmoid gate on the result (tensor name ``g``)."""
        super().__init__(names)
        self.hidden_size, self.heads, self.dim, self.rot_dim = int(hidden_size), int(heads), int(dim), int(rot_dim)
        self.vdim, self.kv_rank, self.scale, self.eps = int(vdim), int(kv_rank), float(scale), float(eps)
        self.gated = bool(gated)
        if self.kv_rank > 512 or self.kv_rank + self.rot_dim > 640:
            raise ValueError("the latent attention kernels take a latent of up to 512 numbers and 640 with the rotated part")
        self.position = build_part(POSITION_ENCODINGS, position)
        self.q_head = self.dim + self.rot_dim
        self.down_col = self.heads * self.q_head
        self.gate_col = self.down_col + self.kv_rank + self.rot_dim
        self.w_in = self.w_uk_t = self.w_uv = self.w_o = self.c_norm = None

    def kernel_needs(self):
        # the second module holds the tensor-core kernels of bfloat16 runs
        return {"modules": {"attention_latent", "attention_latent_mma"}}

    def kv_requirement(self):
        return KVPageRequirement(((1, self.kv_rank + self.rot_dim),), None)

    def expected_tensors(self):
        n, w = self.names, self.hidden_size
        exp = {
            n["q"]: TensorExpectation((self.heads * self.q_head, w)),
            n["dkv"]: TensorExpectation((self.kv_rank + self.rot_dim, w)),
            n["dkv_norm"]: TensorExpectation((self.kv_rank,), "vector"),
            n["uk"]: TensorExpectation((self.heads * self.dim, self.kv_rank)),
            n["uv"]: TensorExpectation((self.heads * self.vdim, self.kv_rank)),
        }
        if self.gated:
            exp[n["g"]] = TensorExpectation((self.heads, w))
        exp[n["o"]] = TensorExpectation((w, self.heads * self.vdim))
        return exp

    def load(self, get, dtype, device):
        n = self.names
        stacked = [get(n["q"], "matrix"), get(n["dkv"], "matrix")] + ([get(n["g"], "matrix")] if self.gated else [])
        rows = sum(t.shape[0] for t in stacked)
        if rows % 8:            # rows of the product's result stay 16-byte aligned
            stacked.append(torch.zeros((8 - rows % 8, self.hidden_size), dtype=stacked[0].dtype, device=device))
        self.w_in = torch.cat(stacked, 0).contiguous()
        self.c_norm = get(n["dkv_norm"], "vector")
        # [heads, kv_rank, dim]: qa = W_uk[h]^T q_plain
        self.w_uk_t = get(n["uk"], "matrix").view(self.heads, self.dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = get(n["uv"], "matrix").view(self.heads, self.vdim, self.kv_rank).contiguous()
        self.w_o = get(n["o"], "matrix").contiguous()
        self.position.load(get, dtype, device)

    def forward(self, x, ctx, cache):
        view = ctx.groups[cache.group]
        inv_freq, rotary_dim, interleaved = self.position.rotary()
        if not interleaved or rotary_dim > self.rot_dim:
            raise ValueError("latent attention rotates neighbouring pairs of at most rot_dim columns")
        # (the projection is summed by the product's own, row-parallel kernel: handing its unsummed splits to
        # latent_prep, one block a token, made a step of one token 5 % slower)
        rows = latent.latent_prep(ops.as_tensor(ops.linear(x, self.w_in)), self.c_norm, self.eps, ctx.positions, inv_freq,
                                  view.slot_mapping if cache.writes else None, cache.pages, self.heads, self.dim,
                                  self.rot_dim, self.kv_rank, self.down_col, cache.block_size)
        qa = latent.head_linear(rows, self.q_head, self.w_uk_t)
        summed = latent.attention_latent(qa, rows, self.q_head, self.dim, self.gate_col if self.gated else None,
                                         cache.pages, view.block_table, ctx.positions, ctx.token_row, self.heads,
                                         self.kv_rank, self.rot_dim, cache.block_size, self.scale, batch=ctx)
        values = latent.head_linear(summed, self.kv_rank, self.w_uv)
        return ops.linear(values, self.w_o, split_ok=True, add_into=getattr(ctx, "residual_sink", None))
