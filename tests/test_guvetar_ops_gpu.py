"""The kernels of the Guvetar parts one by one against plain fp32 PyTorch formulas of the same operation."""

import math

import pytest
import torch
import torch.nn.functional as F

from plain_guvetar import plain_rms, plain_sinusoid

pytestmark = pytest.mark.gpu


def close(got, want, tol):
    scale = max(1.0, float(want.abs().max()))
    assert float((got.float().cpu() - want.float()).abs().max()) <= tol * scale


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("streams,width", [(1, 40), (3, 72), (4, 256), (8, 100), (16, 64)])
def test_embed_streams(dtype, streams, width):
    from gllm_b200.ops import stateful

    g = torch.Generator().manual_seed(0)
    table = torch.randn(50, width, generator=g).to(dtype)
    tokens = torch.randint(0, 50, (37,), generator=g, dtype=torch.int32)
    positions = torch.randint(0, 3000, (37,), generator=g, dtype=torch.int32)
    i = torch.arange((width + 1) // 2, dtype=torch.float64)
    freq = torch.pow(torch.tensor(10000.0, dtype=torch.float64), -2.0 * i / width).float()
    out = stateful.embed_streams(tokens.cuda(), table.cuda(), positions.cuda(), freq.cuda(), streams=streams)
    want = table[tokens.long()].float() + plain_sinusoid(positions, width, torch.float64).float()
    assert out.shape == (37, streams * width)
    for s in range(streams):
        close(out[:, s * width:(s + 1) * width], want, 2e-4)      # fp32 angles of positions up to 3,000
    plain = stateful.embed_streams(tokens.cuda(), table.cuda(), None, None, streams=1)
    close(plain, table[tokens.long()].float(), 0.0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("streams,width", [(1, 48), (2, 64), (4, 200), (7, 96), (8, 1024), (11, 72), (16, 128)])
def test_stream_mix_norm(dtype, streams, width):
    from gllm_b200.ops import stateful

    g = torch.Generator().manual_seed(1)
    n = 21
    x = torch.randn(n, streams, width, generator=g)
    y = torch.randn(n, width, generator=g).to(dtype)
    mix = torch.eye(streams) + 0.2 * torch.randn(streams, streams, generator=g)
    write, read = torch.randn(streams, generator=g), torch.randn(streams, generator=g)
    weight = 1 + 0.1 * torch.randn(width, generator=g)
    new = torch.einsum("st,nsw->ntw", mix, x) + write[None, :, None] * y.float()[:, None, :]
    want = plain_rms(torch.einsum("t,ntw->nw", read, new), 1e-5) * weight
    resid = x.reshape(n, -1).cuda().contiguous()
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    # at chosen rows the streams stay as they are
    rows = torch.tensor([3, 0, 20], dtype=torch.int32)
    some = stateful.stream_mix_norm(y.cuda(), resid, mix.cuda(), write.cuda(), read.cuda(), weight.cuda(), 1e-5, dtype,
                                    streams, rows=rows.cuda())
    close(some, want[rows.long()], tol)
    close(resid, x.reshape(n, -1), 0.0)
    out = stateful.stream_mix_norm(y.cuda(), resid, mix.cuda(), write.cuda(), read.cuda(), weight.cuda(), 1e-5, dtype, streams)
    close(out, want, tol)
    close(resid, new.reshape(n, -1), 1e-5)
    # no result to write, plain sum of the streams (a final norm right after the embedding)
    out, total = stateful.stream_mix_norm(None, resid, None, None, None, weight.cuda(), 1e-5, dtype, streams, want_sum=True)
    close(total, new.sum(1), 1e-5)
    close(out, plain_rms(new.sum(1), 1e-5) * weight, tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_pointwise(dtype):
    from gllm_b200 import ops

    g = torch.Generator().manual_seed(2)
    x, y = torch.randn(33, 70, generator=g).to(dtype), torch.randn(33, 70, generator=g).to(dtype)
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    close(ops.relu_sq(x.cuda()), torch.relu(x.float()) ** 2, tol)
    close(ops.scaled_sum(x.cuda(), y.cuda(), 0.8, -0.5), 0.8 * x.float() - 0.5 * y.float(), tol)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("taps", [1, 2, 4, 7])
def test_conv_silu_with_its_state(dtype, taps):
    """Two requests in one batch, one of them continuing from a state, against a convolution over the whole history."""
    from gllm_b200.ops import stateful

    g = torch.Generator().manual_seed(3)
    ch = 50
    w, bias = torch.randn(ch, taps, generator=g), torch.randn(ch, generator=g)
    hist = torch.randn(9, ch, generator=g).to(dtype)             # request 0: 4 tokens before this step, 5 in it
    other = torch.randn(3, ch, generator=g).to(dtype)            # request 1: new, 3 tokens
    batch = torch.cat([hist[4:], other], 0)
    wide = torch.cat([batch, torch.zeros(8, 6, dtype=dtype)], 1)  # rows are a slice of wider rows
    state = torch.zeros(3, max(taps - 1, 0), ch)
    for k in range(taps - 1):
        src = 4 - (taps - 1) + k
        if src >= 0:
            state[0, k] = hist[src].float()
    positions = torch.tensor([4, 5, 6, 7, 8, 0, 1, 2], dtype=torch.int32)
    token_row = torch.tensor([0] * 5 + [1] * 3, dtype=torch.int32)
    out = stateful.conv_silu(wide.cuda()[:, :ch], w.cuda(), bias.cuda(), state.cuda(), positions.cuda(), token_row.cuda())

    def whole(seq):
        padded = torch.cat([torch.zeros(taps - 1, ch), seq.float()], 0)
        return torch.stack([F.silu((padded[t:t + taps] * w.T).sum(0) + bias) for t in range(seq.shape[0])])

    want = torch.cat([whole(hist)[4:], whole(other)], 0)
    close(out, want, 1e-5 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_head_norm(dtype):
    from gllm_b200.ops import stateful

    g = torch.Generator().manual_seed(4)
    n, heads, dv = 11, 3, 20
    o = torch.randn(n, heads, dv + 2, generator=g)
    o[:, :, dv + 1] = o[:, :, dv + 1].abs()
    gate = torch.randn(n, heads * dv, generator=g).to(dtype)
    tol = 1e-5 if dtype == torch.float32 else 1e-2
    shared = 1 + 0.1 * torch.randn(dv, generator=g)
    got = stateful.head_norm(o[:, :, :dv].reshape(n, -1).contiguous().cuda(), heads, dv, shared.cuda(), 1e-5, dtype)
    close(got, (plain_rms(o[:, :, :dv], 1e-5) * shared).reshape(n, -1), tol)
    each = 1 + 0.1 * torch.randn(heads * dv, generator=g)
    den = torch.maximum(o[:, :, dv].abs(), o[:, :, dv + 1]) + 1e-6
    want = plain_rms(o[:, :, :dv] / den[:, :, None], 1e-5).reshape(n, -1) * each * torch.sigmoid(gate.float())
    got = stateful.head_norm(o.reshape(n, -1).contiguous().cuda(), heads, dv, each.cuda(), 1e-5, dtype, with_denominator=True,
                             denominator_eps=1e-6, gate=gate.cuda())
    close(got, want, tol)
