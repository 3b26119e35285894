"""Python entry points of ``csrc/attention_latent.cu``: attention over one cached latent vector per
token.  As everywhere in ``gllm_b200.ops``: CUDA tensors only, no CPU path."""

from __future__ import annotations

import os
from ctypes import c_float, c_int, c_int64, c_void_p

import torch

from gllm_b200.ops import _check, _cuda, _fn, _ptr, _stream, _suffix, status_word
from gllm_b200.ops.build import load_module

# GLLM_B200_LATENT_MMA=0: the latent attention of bf16 models stays on the CUDA-core kernel (for measurements)
USE_TENSOR_CORES = os.environ.get("GLLM_B200_LATENT_MMA", "1") != "0"
SPLIT_KEYS = 128          # a range of keys is at least this long (measured: 64 and 128 equal at batch 1, 128 quicker at batch 8)
MAX_SPLITS = 64
KEY_TILE = 32
_mma = None


def _mma_fns():
    global _mma
    if _mma is None:
        lib = load_module("attention_latent_mma")
        f = lib.gllm_attention_latent_mma
        P = c_void_p
        f.argtypes = [P, c_int64, P, c_int64, c_int, P, c_int64, P, c_int64, P, P, P, P, c_int, P, P, P, c_int, c_int,
                      c_int, c_int, c_int, c_int, c_int, c_int, c_float, c_int, c_int, P, P]
        f.restype = c_int
        lib.gllm_attention_latent_mma_supports.argtypes = [c_int, c_int]
        lib.gllm_attention_latent_mma_supports.restype = c_int
        lib.gllm_attention_latent_mma_tokens_per_tile.argtypes = [c_int]
        lib.gllm_attention_latent_mma_tokens_per_tile.restype = c_int
        hl = lib.gllm_head_linear_mma
        hl.argtypes = [P, c_int64, c_int, P, P, c_int64, c_int, c_int, c_int, c_int, c_int, P]
        hl.restype = c_int
        _mma = (f, lib.gllm_attention_latent_mma_supports, lib.gllm_attention_latent_mma_tokens_per_tile, hl)
    return _mma


MMA_SIZES = {(64, 32), (64, 64), (96, 32), (128, 32), (128, 64), (256, 32), (256, 64), (512, 64)}


def tensor_core_kernel_takes(dtype: torch.dtype, rank: int, rot: int) -> bool:
    """True for the (latent, rotated part) widths the tensor-core kernel is built for, in bfloat16."""
    return dtype == torch.bfloat16 and (rank, rot) in MMA_SIZES and USE_TENSOR_CORES


def _attention_latent_mma(qa, rows, q_head, q_plain, gate_col, pages, block_table, heads, rank, rot, block_size, scale,
                          batch, out):
    """The tensor-core kernel.  Steps whose tiles do not fill the GPU (single tokens over long contexts) cut every
    request's keys into ranges of at least ``SPLIT_KEYS`` keys, one CTA each, merged by a second kernel."""
    f, _, tokens_per_tile = _mma_fns()[:3]
    n = qa.shape[0]
    qt = tokens_per_tile(heads)
    tiles = -(-batch.max_q_len // qt) * (1 if heads <= 64 else heads) * batch.num_requests
    sms = torch.cuda.get_device_properties(qa.device).multi_processor_count
    splits, tiles_per_split = 1, 0
    # (with more than half as many tiles as SMs the ranges cost more than they win: 512 tokens over 1,536 cached ones
    # 255 us in three ranges against 217 us in one; 128 tokens: 73 against 174 us)
    # The ranges have to cover the longest sequence of every step this launch serves.  A captured prompt portion
    # is replayed for other contexts (the step's own longest sequence is then only that of the captured step), so
    # under capture the bound is what a block-table row can hold; single tokens are captured per sequence bucket.
    longest = batch.max_seq_len
    if batch.max_q_len > 1 and torch.cuda.is_current_stream_capturing():
        longest = max(longest, block_table.shape[1] * block_size)
    if 2 * tiles <= sms and longest > 2 * SPLIT_KEYS:
        want = min(MAX_SPLITS, -(-2 * sms // tiles))
        key_tiles = -(-longest // KEY_TILE)
        tiles_per_split = max(SPLIT_KEYS // KEY_TILE, -(-key_tiles // want))
        splits = -(-key_tiles // tiles_per_split)
    part_o = part_ml = None
    if splits > 1:
        part_o = batch.workspace.get("latent_attention_partial_out", splits * n * heads * rank, torch.float32)
        part_ml = batch.workspace.get("latent_attention_partial_max_sum", splits * n * heads * 2, torch.float32)
    item = qa.element_size()
    gate_ptr = None if gate_col is None else rows.data_ptr() + gate_col * item
    code = f(qa.data_ptr(), qa.stride(0), rows.data_ptr() + q_plain * item, rows.stride(0), int(q_head), gate_ptr,
             rows.stride(0), out.data_ptr(), out.stride(0), _ptr(part_o), _ptr(part_ml), pages.data_ptr(),
             block_table.data_ptr(), block_table.stride(0), batch.cu_q.data_ptr(), batch.context_lens.data_ptr(),
             batch.state_slots.data_ptr(), batch.num_requests, batch.max_q_len, n, int(heads), int(rank), int(rot),
             int(block_size), pages.shape[0], float(scale), splits, tiles_per_split,
             status_word(qa.device).data_ptr(), _stream())
    _check(code, "attention_latent_mma")
    return out


def _rows(t: torch.Tensor, name: str, dtype=None) -> None:
    _cuda(t, name, dtype, contiguous=False)
    if t.dim() != 2 or t.stride(1) != 1:
        raise ValueError(f"{name} must be [tokens, columns] with contiguous columns")


def latent_prep(rows, norm_weight: torch.Tensor, eps: float, positions: torch.Tensor,
                inv_freq: torch.Tensor, slot_mapping: torch.Tensor | None, pages: torch.Tensor, heads: int,
                q_plain: int, rot: int, rank: int, down_col: int, block_size: int) -> torch.Tensor:
    """On the projection rows ``[n, >= heads * (q_plain + rot) + rank + rot]`` (a tensor, or a SplitSum that is
    summed into a new tensor first, in the same kernel): rotate the last ``rot`` columns of every query head in
    place (neighbouring pairs, ``2 * len(inv_freq)`` columns of them), and store
    ``[rms(down[:rank]) * norm_weight ; rotate(down[rank:])]`` of the down-projection at column ``down_col``
    into the token's cache slot.  ``pages`` is the pool layer ``[pages, block_size * (rank + rot)]``.  Returns the
    rows."""
    from gllm_b200.ops import SplitSum, _parts_args

    parts_ptr, n_parts, part_stride = _parts_args(rows)
    if isinstance(rows, SplitSum):
        if n_parts > 16:
            rows = rows.tensor()
            parts_ptr, n_parts, part_stride = None, 0, 0
        else:
            rows = torch.empty(tuple(rows.shape), dtype=rows.dtype, device=rows.device)
    _rows(rows, "rows")
    _cuda(norm_weight, "norm_weight", torch.float32)
    _cuda(inv_freq, "inv_freq", torch.float32)
    _cuda(positions, "positions", torch.int32)
    _cuda(pages, "pages", rows.dtype, contiguous=False)
    if norm_weight.numel() != rank:
        raise ValueError("the latent's norm needs one weight per column")
    if pages.stride(0) != block_size * (rank + rot):
        raise ValueError("the cache layer's pages are not block_size * (rank + rot) wide")
    if down_col + rank + rot > rows.shape[1] or heads * (q_plain + rot) > down_col:
        raise ValueError("the projection rows are narrower than the heads and the down-projection need")
    if slot_mapping is not None:
        _cuda(slot_mapping, "slot_mapping", torch.int32)
    f = _fn("attention_latent", f"gllm_latent_prep_{_suffix(rows.dtype)}")
    _check(f(rows.data_ptr(), rows.stride(0), parts_ptr, n_parts, part_stride, rows.shape[1], norm_weight.data_ptr(),
             float(eps), positions.data_ptr(), inv_freq.data_ptr(), _ptr(slot_mapping), pages.data_ptr(), rows.shape[0],
             int(heads), int(q_plain + rot), int(q_plain), int(down_col), int(rank), int(rot), 2 * inv_freq.numel(),
             int(block_size), pages.shape[0], status_word(rows.device).data_ptr(), _stream()), "latent_prep")
    return rows


def head_linear(x: torch.Tensor, x_head: int, weight: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """``out[n, h, :] = weight[h] @ x[n, h * x_head : h * x_head + I]`` for ``weight [heads, J, I]``: one small
    product per head in one launch; ``out`` is ``[n, heads * J]``."""
    _rows(x, "x")
    _cuda(weight, "weight", x.dtype)
    heads, j, i = weight.shape
    if (heads - 1) * x_head + i > x.shape[1]:
        raise ValueError("the heads do not lie inside the rows of x")
    n = x.shape[0]
    if out is None:
        out = torch.empty((n, heads * j), dtype=x.dtype, device=x.device)
    if (x.dtype == torch.bfloat16 and USE_TENSOR_CORES and i % 8 == 0 and x.stride(0) % 8 == 0 and x_head % 8 == 0
            and j % 2 == 0 and out.stride(0) % 2 == 0 and x.data_ptr() % 16 == 0 and weight.data_ptr() % 16 == 0
            and out.data_ptr() % 4 == 0):
        _check(_mma_fns()[3](x.data_ptr(), x.stride(0), int(x_head), weight.data_ptr(), out.data_ptr(), out.stride(0), j,
                             n, heads, i, j, _stream()), "head_linear_mma")
        return out
    f = _fn("attention_latent", f"gllm_head_linear_{_suffix(x.dtype)}")
    _check(f(x.data_ptr(), x.stride(0), int(x_head), weight.data_ptr(), out.data_ptr(), out.stride(0), j, n, heads, i,
             j, _stream()), "head_linear")
    return out


def attention_latent(qa: torch.Tensor, rows: torch.Tensor, q_head: int, q_plain: int, gate_col: int | None,
                     pages: torch.Tensor, block_table: torch.Tensor, positions: torch.Tensor, token_row: torch.Tensor,
                     heads: int, rank: int, rot: int, block_size: int, scale: float, window: int | None = None,
                     batch=None) -> torch.Tensor:
    """Softmax attention of every (token, head) over its request's cached ``[c ; kr]`` vectors: scores
    ``(qa . c + qr . kr) * scale`` with ``qa [n, heads * rank]`` and ``qr`` the rotated part of every query head
    inside ``rows``; the result ``[n, heads * rank]`` is the weighted sum of the ``c`` (times
    ``sigmoid(rows[n, gate_col + h])`` with ``gate_col``)."""
    _rows(qa, "qa")
    _rows(rows, "rows", qa.dtype)
    _cuda(pages, "pages", qa.dtype, contiguous=False)
    _cuda(block_table, "block_table", torch.int32, contiguous=False)
    _cuda(positions, "positions", torch.int32)
    _cuda(token_row, "token_row", torch.int32)
    n = qa.shape[0]
    if qa.shape[1] != heads * rank or pages.stride(0) != block_size * (rank + rot):
        raise ValueError("qa or the cache layer does not match heads, rank and rot")
    out = torch.empty((n, heads * rank), dtype=qa.dtype, device=qa.device)
    if (batch is not None and not window and tensor_core_kernel_takes(qa.dtype, rank, rot) and qa.stride(0) % 8 == 0
            and rows.stride(0) % 8 == 0 and q_head % 8 == 0 and q_plain % 8 == 0
            and rows.data_ptr() % 16 == 0 and qa.data_ptr() % 16 == 0):
        return _attention_latent_mma(qa, rows, q_head, q_plain, gate_col, pages, block_table, heads, rank, rot,
                                     block_size, scale, batch, out)
    t = _suffix(qa.dtype)
    item = qa.element_size()
    f = _fn("attention_latent", f"gllm_attention_latent_{t}")
    gate_ptr = None if gate_col is None else rows.data_ptr() + gate_col * item
    _check(f(qa.data_ptr(), qa.stride(0), rank, rows.data_ptr() + q_plain * item, rows.stride(0), int(q_head),
             gate_ptr, rows.stride(0), out.data_ptr(), out.stride(0), rank, pages.data_ptr(), block_table.data_ptr(),
             block_table.stride(0), positions.data_ptr(), token_row.data_ptr(), n, int(heads), int(rank), int(rot),
             int(block_size), pages.shape[0], float(scale), int(window or 0), status_word(qa.device).data_ptr(),
             _stream()), "attention_latent")
    return out
