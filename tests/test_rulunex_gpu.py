"""Rulunex on the GPU against the plain implementation: each mixer alone, whole prompts against token by token
decoding and portions of every size, mixed batches over a pool so small that pages and slots are used again, one
decisive key far away, at page borders and just inside and outside the window, the first tokens, long decoding
through the decode graphs, other sizes, the kernels one by one, and greedy generation through the engine."""

import copy
import math
import os

import numpy as np
import pytest
import torch

from plain_rulunex import (plain_feed_forward, plain_forward, plain_latent_attention, plain_rms,
                           plain_window_attention)
from replay_helpers import (BF16_TOL_MAX, BF16_TOL_MEAN, FP32_TOL, LENGTHS, compare, mixed_steps, replay, rounded,
                            run_steps, sequences, single_request_steps)
from tiny_rulunex import RULUNEX, draw_weights, single_mixer, write_model

pytestmark = pytest.mark.gpu

PAGE = {"A": 4, "B": 8, "C": 16, "D": 16}


def tolerance(dtype):
    return (FP32_TOL, None) if dtype == "float32" else (BF16_TOL_MAX, BF16_TOL_MEAN)


def make(cfg, tmp_path, dtype, seed=7, max_tokens=512, block_size=16, max_live=4, sharp=None):
    from gllm_b200.engine.replay import build_runner

    sharp = (3.0 if dtype == "float32" else 1.5) if sharp is None else sharp
    weights = draw_weights(cfg, seed=seed, sharp=sharp)
    folder = write_model(cfg, weights, str(tmp_path / "model"))
    _, runner = build_runner(folder, dtype, max_tokens, block_size=block_size, max_live=max_live)
    return weights, folder, runner


def steps_of(tokens, cuts, rid="r", first_step=0, end=True):
    """One request fed in portions of the given sizes; every logit is wanted."""
    steps, index, p = [], [], 0
    for i, n in enumerate(cuts):
        last = p + n == len(tokens)
        steps.append({"step": first_step + i, "entries": [{"id": rid, "tokens": tokens[p:p + n], "want": list(range(n))}],
                      "end": [rid] if (last and end) else []})
        index += [(first_step + i, k, rid, p + k) for k in range(n)]
        p += n
    assert p == len(tokens)
    return steps, index


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("mlp", [True, False])
@pytest.mark.parametrize("kind", ["latent", "latent_wide", "latent_many", "window", "causal", "odd"])
def test_each_mixer_alone(kind, mlp, dtype, tmp_path):
    cfg = single_mixer(kind, mlp)
    weights, _, runner = make(cfg, tmp_path, dtype)
    toks = torch.randint(0, cfg["vocab"], (75,), generator=torch.Generator().manual_seed(2)).tolist()
    plain = {"r": plain_forward(cfg, weights, toks)}
    steps, index = steps_of(toks, [40] + [1] * 35)
    compare(run_steps(runner, steps), index, plain, *tolerance(dtype))
    steps, index = steps_of(toks, [75])
    compare(run_steps(runner, steps), index, plain, *tolerance(dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_all_cuts_and_mixed_batches(name, dtype, tmp_path):
    cfg = RULUNEX[name]
    weights, _, runner = make(cfg, tmp_path, dtype, max_tokens=rounded(max(LENGTHS.values())), block_size=PAGE[name])
    seqs = sequences(cfg["vocab"], seed=5)
    plain = {k: plain_forward(cfg, weights, v) for k, v in seqs.items()}
    steps, index = single_request_steps(seqs)
    compare(run_steps(runner, steps), index, plain, *tolerance(dtype))
    runner.cache.check_invariants()
    # four live requests at most over 448 tokens of pages: pages and slots are used again
    from gllm_b200.engine.replay import build_runner

    _, small = build_runner(str(tmp_path / "model"), dtype, 448, block_size=PAGE[name])
    steps, index = mixed_steps(seqs, max_tokens=448, seed=9)
    compare(run_steps(small, steps), index, plain, *tolerance(dtype))
    small.cache.check_invariants()
    assert all(g.allocator.total_reused > 0 for g in small.cache.groups)
    assert small.graph_replays > 0


def test_every_pass_of_the_repeated_stretch_has_a_cache_of_its_own(tmp_path):
    cfg = RULUNEX["A"]
    _, _, runner = make(cfg, tmp_path, "float32")
    # 1 + 3 * 2 + 1 layer runs: the windowed group holds layer 0 alone, the latent layers of the stretch one
    # pool layer per pass, the last layer a group of its own (no window)
    layers_per_group = sorted(len(g.owner_entries) for g in runner.cache.groups)
    assert sum(layers_per_group) == 8 and len(runner.model.spec.plan) == 8
    assert [e.rejoins_embedding for e in runner.model.spec.plan] == [False, True, False, True, False, True, False, False]


def test_replay_through_the_command(tmp_path):
    cfg = RULUNEX["A"]
    weights = draw_weights(cfg, seed=7, sharp=3.0)
    folder = write_model(cfg, weights, str(tmp_path / "model"))
    seqs = sequences(cfg["vocab"], seed=6)
    plain = {k: plain_forward(cfg, weights, v) for k, v in seqs.items()}
    steps, index = mixed_steps(seqs, max_tokens=448, seed=3)
    results = replay(folder, "float32", steps, str(tmp_path / "out"), max_tokens=448, vocab=cfg["vocab"])
    compare(results, index, plain, FP32_TOL)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "C"])
def test_portions_at_every_edge(name, dtype, tmp_path):
    """Portions that end just before, at and just after the edges the kernels have: pages of 16, the windows,
    the attention kernels' blocks of 32 and 64 keys."""
    cfg = RULUNEX[name]
    weights, _, runner = make(cfg, tmp_path, dtype, max_tokens=256)
    toks = torch.randint(0, cfg["vocab"], (200,), generator=torch.Generator().manual_seed(8)).tolist()
    plain = {"r": plain_forward(cfg, weights, toks)}
    for cuts in ([7, 1, 1, 7, 15, 2, 31, 1, 33, 16, 17, 9, 8, 2, 2, 3, 45],
                 [2, 2, 2, 2, 8, 16, 32, 64, 63, 9],
                 [1, 1, 1, 1, 1, 3, 24, 31, 33, 104]):
        steps, index = steps_of(toks, cuts)
        compare(run_steps(runner, steps), index, plain, *tolerance(dtype))


# ------------------------------------------------------------------------------------------------
# One decisive key.  Token 1 (the key) and token 2 (the query) have one-hot embeddings, so the norm in front of the
# mixer maps them to fixed vectors whatever else is in the sequence; head 0's query for token 2 is made to point
# along head 0's key for token 1 in the part of the head that the rotation leaves alone, and token 1's value is
# made large.  Every other key scores far lower, so the logits after token 2 say whether token 1's key was seen.
def decisive_latent_model(kind="latent"):
    cfg = single_mixer(kind, mlp=False)
    m = cfg["layers"][0]["mixer"]
    w = draw_weights(cfg, seed=11, sharp=1.0)
    W, d, r, rank, eps = cfg["width"], m["dim"], m["rot_dim"], m["kv_rank"], cfg["norm"]["eps"]
    ca, cb = 5, 9
    w["embed"][1], w["embed"][2] = 0.0, 0.0
    w["embed"][1, ca], w["embed"][2, cb] = 3.0, 3.0
    w["embed"][3:, [ca, cb]] = 0.0                       # the other tokens have nothing in the two marker columns
    w["l0.norm1"][[ca, cb]] = 0.0
    h_key = torch.zeros(W, dtype=torch.float64)
    h_key[ca] = math.sqrt(W)                             # what the layer's norm makes of token 1
    c = plain_rms(w["l0.mix.dkv"].double()[:rank] @ h_key, eps) * w["l0.mix.dkv.norm"].double()
    k0 = w["l0.mix.uk"].double()[:d] @ c                 # head 0's un-rotated key for token 1
    w["l0.mix.q"][:, cb] *= 0.05
    w["l0.mix.q"][:d, cb] = (k0 / k0.norm() * 2.5).float()
    w["l0.mix.uv"] *= 3.0
    w["l0.mix.g"][0, cb] = 0.5                           # head 0's gate is open for token 2
    return cfg, {k: v.to(torch.bfloat16).to(torch.float32) for k, v in w.items()}


def decisive_window_model(window):
    cfg = single_mixer("window", mlp=False)
    m = cfg["layers"][0]["mixer"]
    m["mask"]["size"] = window
    m["scale"] = 0.12
    w = draw_weights(cfg, seed=13, sharp=1.0)
    d, dims = m["dim"], m["rot"]["dims"]
    ca, cb = 5, 9
    w["embed"][1], w["embed"][2] = 0.0, 0.0
    w["embed"][1, ca], w["embed"][2, cb] = 3.0, 3.0
    w["embed"][3:, [ca, cb]] = 0.0
    w["l0.norm1"][[ca, cb]] = 0.0
    # token 1's key and token 2's query live in the un-rotated columns of head 0 alone
    w["l0.mix.k"][:, ca], w["l0.mix.q"][:, cb] = 0.0, 0.0
    w["l0.mix.k"][dims:d, ca] = 1.0
    w["l0.mix.q"][dims:d, cb] = 1.0
    w["l0.mix.q.norm"][:], w["l0.mix.k.norm"][:] = 1.0, 1.0
    return cfg, {k: v.to(torch.bfloat16).to(torch.float32) for k, v in w.items()}


def check_decisive(cfg, weights, runner, toks, key_at, dtype, seen=True):
    n = len(toks)
    tol_max, _ = tolerance(dtype)
    plain = plain_forward(cfg, weights, toks)
    without = list(toks)
    without[key_at] = 3
    blind = plain_forward(cfg, weights, without)
    scale = max(1.0, float(plain.abs().max()))
    moved = float((plain[-1] - blind[-1]).abs().max())
    if seen:        # the test is sharp: losing that one key moves the last logits by far more than the tolerance
        assert moved > (20 if dtype == "float32" else 3) * tol_max * scale, moved / scale
    else:           # a key outside the window changes nothing
        assert moved < 1e-9
    for cuts in ([n], [n - 1, 1], [key_at + 1, n - key_at - 3, 2] if key_at + 3 < n else [n - 2, 2]):
        steps, index = steps_of(toks, cuts)
        compare(run_steps(runner, steps), [i for i in index if i[3] >= n - 2], {"r": plain}, tol_max, None)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("kind", ["latent", "latent_wide"])
def test_a_far_key_at_page_and_block_edges(kind, dtype, tmp_path):
    from gllm_b200.engine.replay import build_runner

    cfg, weights = decisive_latent_model(kind)
    folder = write_model(cfg, weights, str(tmp_path / "model"))
    _, runner = build_runner(folder, dtype, 1024, block_size=16)
    g = torch.Generator().manual_seed(5)
    n = 600
    if dtype == "bfloat16":
        from gllm_b200.ops import latent

        m = cfg["layers"][0]["mixer"]
        assert latent.tensor_core_kernel_takes(torch.bfloat16, m["kv_rank"], m["rot_dim"]) == (kind == "latent_wide")
    for far in (0, 15, 16, 17, 31, 32, 33, 63, 64, 255, 256, 511):
        toks = torch.randint(3, cfg["vocab"], (n,), generator=g).tolist()
        toks[far], toks[-1] = 1, 2
        check_decisive(cfg, weights, runner, toks, far, dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("window", [5, 16, 24, 33, 70])
def test_a_key_just_inside_and_just_outside_the_window(window, dtype, tmp_path):
    from gllm_b200.engine.replay import build_runner

    cfg, weights = decisive_window_model(window)
    folder = write_model(cfg, weights, str(tmp_path / "model"))
    _, runner = build_runner(folder, dtype, 512, block_size=16)
    g = torch.Generator().manual_seed(6)
    for n in (window + 1, 97, 128, 131, 200):
        if n <= window:
            continue
        toks = torch.randint(3, cfg["vocab"], (n,), generator=g).tolist()
        toks[-1] = 2
        inside, outside = list(toks), list(toks)
        inside[n - window] = 1                           # the oldest key the last token still sees
        outside[n - window - 1] = 1                      # the newest it does not
        check_decisive(cfg, weights, runner, inside, n - window, dtype, seen=True)
        check_decisive(cfg, weights, runner, outside, n - window - 1, dtype, seen=False)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decoding(dtype, tmp_path):
    """Prompts of one, two and three tokens, then hundreds of tokens decoded one by one (replays of the decode
    graph), past the windows and over many pages."""
    cfg = RULUNEX["A"]
    weights, _, runner = make(cfg, tmp_path, dtype, max_tokens=512)
    g = torch.Generator().manual_seed(12)
    for first in (1, 2, 3):
        n = first + (330 if first == 2 else 20)
        toks = torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()
        plain = {"r": plain_forward(cfg, weights, toks)}
        steps, index = steps_of(toks, [first] + [1] * (n - first))
        compare(run_steps(runner, steps), index, plain, *tolerance(dtype))
    assert runner.graph_replays > 300


def test_single_tokens_over_a_long_context(tmp_path):
    """bfloat16 with the head widths of the tensor-core kernels: a context of 900 tokens, then single tokens,
    alone and two requests at once."""
    cfg = RULUNEX["C"]
    weights, folder, runner = make(cfg, tmp_path, "bfloat16", max_tokens=2048)
    g = torch.Generator().manual_seed(31)
    a = torch.randint(0, cfg["vocab"], (930,), generator=g).tolist()
    b = torch.randint(0, cfg["vocab"], (700,), generator=g).tolist()
    plain = {"a": plain_forward(cfg, weights, a), "b": plain_forward(cfg, weights, b)}
    steps = [{"step": 0, "entries": [{"id": "a", "tokens": a[:900], "want": [899]}], "end": []},
             {"step": 1, "entries": [{"id": "b", "tokens": b[:690], "want": [689]}], "end": []}]
    index = [(0, 0, "a", 899), (1, 0, "b", 689)]
    for i in range(10):
        steps.append({"step": 2 + i, "entries": [{"id": "a", "tokens": [a[900 + i]], "want": [0]},
                                                  {"id": "b", "tokens": [b[690 + i]], "want": [0]}], "end": []})
        index += [(2 + i, 0, "a", 900 + i), (2 + i, 1, "b", 690 + i)]
    for i in range(10, 30):
        steps.append({"step": 2 + i, "entries": [{"id": "a", "tokens": [a[900 + i]], "want": [0]}], "end": []})
        index.append((2 + i, 0, "a", 900 + i))
    compare(run_steps(runner, steps), index, plain, BF16_TOL_MAX, BF16_TOL_MEAN)


def test_a_captured_portion_replayed_over_a_longer_context(tmp_path):
    """Portions of one size run as a CUDA graph captured on the first of them; the later ones replay it over a
    context the captured step did not have.  With keys cut into ranges (few tiles, tensor-core latent kernel) the
    ranges must cover those contexts too: the one decisive key lies beyond the captured step's longest sequence."""
    from gllm_b200.engine.replay import build_runner
    from gllm_b200.engine.step import StepRunner

    cfg, weights = decisive_latent_model("latent_wide")
    folder = write_model(cfg, weights, str(tmp_path / "model"))
    _, runner = build_runner(folder, "bfloat16", 1024, block_size=16)
    graphed = StepRunner(runner.model, runner.cache, max_tokens_per_step=1024, prefill_graph_tokens=(320,))
    toks = torch.randint(3, cfg["vocab"], (960,), generator=torch.Generator().manual_seed(17)).tolist()
    toks[500], toks[-1] = 1, 2
    plain = plain_forward(cfg, weights, toks)
    without = list(toks)
    without[500] = 3
    blind = plain_forward(cfg, weights, without)
    tol_max, _ = tolerance("bfloat16")
    scale = max(1.0, float(plain.abs().max()))
    assert float((plain[-1] - blind[-1]).abs().max()) > 3 * tol_max * scale
    steps, index = steps_of(toks, [320, 320, 320])
    compare(run_steps(graphed, steps), [i for i in index if i[3] >= 958], {"r": plain}, tol_max, None)
    assert graphed.graph_replays == 2


def test_a_slot_and_its_pages_used_again_start_clean(tmp_path):
    """One state slot and a pool of four pages: the second request gets the first one's slot and pages."""
    cfg = RULUNEX["A"]
    weights, _, runner = make(cfg, tmp_path, "float32", max_tokens=64, max_live=1)
    g = torch.Generator().manual_seed(13)
    a = torch.randint(0, cfg["vocab"], (60,), generator=g).tolist()
    b = torch.randint(0, cfg["vocab"], (50,), generator=g).tolist()
    for rid, toks, cuts in (("a", a, [33, 20, 7]), ("b", b, [3, 40] + [1] * 7), ("c", a, [60])):
        steps, index = steps_of(toks, cuts, rid=rid)
        compare(run_steps(runner, steps), index, {rid: plain_forward(cfg, weights, toks)}, FP32_TOL)
    assert all(g.allocator.total_reused > 0 for g in runner.cache.groups)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_through_the_entry_point(name, dtype, tmp_path):
    from gllm_b200 import GenerationRequest, GeneratorParams, LLMEngine

    cfg = RULUNEX[name]
    weights = draw_weights(cfg, seed=21, sharp=1.5)
    folder = write_model(cfg, weights, str(tmp_path / "m"))
    g = torch.Generator().manual_seed(4)
    prompts = [torch.randint(0, cfg["vocab"], (n,), generator=g).tolist() for n in (1, 7, 16, 23, 40)]
    # few pages, small portions: chunked prefill, continuous batching and (with pages) preemption happen
    params = GeneratorParams(block_size=8, max_batch_size=3, max_seq_len=64, num_blocks=10, model_dtype=dtype,
                             max_num_batched_tokens=24, prefill_chunk=8)
    engine = LLMEngine(folder, params, device="cuda:0")
    reqs = [GenerationRequest(prompt_token_ids=p, max_new_tokens=12, temperature=0.0, ignore_eos=True) for p in prompts]
    results = engine.generate(reqs)
    slack = 1e-5 if dtype == "float32" else 0.05
    for p, r in zip(prompts, results):
        assert len(r.token_ids) == 12 and r.finish_reason == "length"
        tokens = list(p)
        for t in r.token_ids:
            logits = plain_forward(cfg, weights, tokens)[-1]
            best = int(logits.argmax())
            if t != best:
                assert float(logits[best] - logits[t]) <= slack * float(logits.abs().max()), (len(tokens), t, best)
            tokens.append(t)
    engine.cache.check_invariants()
    assert not engine.scheduler.has_work
    if dtype == "float32":
        for req, r in zip(reqs, results):
            assert engine.generate([req])[0].token_ids == r.token_ids


def test_random_weights_mode_writes_a_model_that_runs(tmp_path):
    from gllm_b200.config import load_config
    from gllm_b200.engine.replay import build_runner
    from gllm_b200.weights import write_random_model

    folder = write_random_model(str(tmp_path / "m"), load_config(copy.deepcopy(RULUNEX["C"])), seed=3)
    assert os.path.isfile(os.path.join(folder, "model.safetensors"))
    _, runner = build_runner(folder, "bfloat16", 128)
    steps, _ = steps_of(list(range(40)), [30, 1, 9])
    out = run_steps(runner, steps)
    assert all(np.isfinite(v).all() for v in out.values())


# ------------------------------------------------------------------------------------------------ kernels one by one
def _t(x, dtype):
    return x.to(dtype).cuda()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("block", [0, 64])
def test_gated_activation_with_clamps(dtype, block):
    from gllm_b200 import ops

    g = torch.Generator().manual_seed(1)
    n, inter = 37, 192
    gate, up = torch.randn(n, inter, generator=g) * 2, torch.randn(n, inter, generator=g) * 2
    gate, up = gate.to(dtype).float(), up.to(dtype).float()
    for slope, limit, offset in ((1.702, 1.25, 1.0), (1.0, None, 0.0), (0.5, 3.0, -0.5)):
        gc = gate.clamp(max=limit) if limit else gate
        uc = up.clamp(-limit, limit) if limit else up
        want = gc * torch.sigmoid(slope * gc) * (uc + offset)
        if block:
            stacked = torch.stack([gate.view(n, inter // block, block), up.view(n, inter // block, block)], 2).reshape(n, -1)
        else:
            stacked = torch.cat([gate, up], 1)
        got = ops.gated_activation(_t(stacked, dtype), slope=slope, limit=limit, up_offset=offset, block=block)
        torch.testing.assert_close(got.float().cpu(), want, rtol=1e-2 if dtype == torch.bfloat16 else 1e-5,
                                   atol=1e-2 if dtype == torch.bfloat16 else 1e-5)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_whole_projection_norm_and_values_from_keys(dtype):
    from gllm_b200 import ops

    g = torch.Generator().manual_seed(2)
    n, qc, kc, eps = 19, 96, 40, 1e-5
    qk = (torch.randn(n, qc + kc, generator=g) * 3).to(dtype).float()
    wq, wk = 1 + 0.2 * torch.randn(qc, generator=g), 1 + 0.2 * torch.randn(kc, generator=g)
    got = ops.qk_rownorm(_t(qk, dtype), wq.cuda(), wk.cuda(), eps, qc, kc).float().cpu()
    q, k = qk[:, :qc], qk[:, qc:]
    want = torch.cat([plain_rms(q, eps) * wq, plain_rms(k, eps) * wk, k], 1)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    torch.testing.assert_close(got, want, rtol=tol, atol=tol)
    assert torch.equal(got[:, qc + kc:], k)              # the values are the projection itself


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_residual_add_and_join(dtype):
    from gllm_b200 import ops

    g = torch.Generator().manual_seed(3)
    n, w = 21, 72
    resid, other = torch.randn(n, w, generator=g), torch.randn(n, w, generator=g)
    branch = torch.randn(n, w, generator=g).to(dtype)
    r = resid.clone().cuda()
    joined = ops.join_rows(branch.cuda(), r, other.cuda(), dtype).float().cpu()
    assert torch.equal(r.cpu(), resid)                   # the join leaves the residual alone
    want = torch.cat([resid + branch.float(), other], 1).to(dtype).float()
    torch.testing.assert_close(joined, want, rtol=0, atol=0)
    ops.residual_add(r, branch.cuda())
    torch.testing.assert_close(r.cpu(), resid + branch.float(), rtol=0, atol=0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,heads,i,j,stride", [(70, 3, 20, 37, 29), (1, 4, 64, 24, 96), (150, 3, 136, 70, 144)])
def test_one_product_per_head(dtype, n, heads, i, j, stride):
    from gllm_b200.ops import latent

    g = torch.Generator().manual_seed(4)
    x = torch.randn(n, heads * stride + 8, generator=g).to(dtype)
    w = torch.randn(heads, j, i, generator=g).to(dtype)
    got = latent.head_linear(x.cuda(), stride, w.cuda()).float().cpu().view(n, heads, j)
    want = torch.stack([x[:, h * stride:h * stride + i].double() @ w[h].double().T for h in range(heads)], 1)
    tol = 3e-2 if dtype == torch.bfloat16 else 1e-4
    torch.testing.assert_close(got.double(), want, rtol=tol, atol=tol)


@pytest.mark.parametrize("single", [False, True])
@pytest.mark.parametrize("heads,rank,rot", [(5, 64, 32), (16, 128, 64), (70, 96, 32), (3, 512, 64)])
def test_latent_attention_on_the_tensor_cores_against_the_cuda_cores(heads, rank, rot, single):
    """Both kernels over the same pages: prompt portions beside single tokens over long contexts (whose keys are cut
    into ranges), with a gate; and both against a plain fp64 softmax."""
    from types import SimpleNamespace

    from gllm_b200.engine.step import Workspace
    from gllm_b200.ops import latent

    g = torch.Generator().manual_seed(heads)
    block, dk = 16, rank + rot
    q_lens, ctx_lens = ([1, 1, 1], [900, 0, 333]) if single else ([37, 1, 1, 5], [70, 900, 0, 333])
    n, nreq = sum(q_lens), len(q_lens)
    pages_per = [-(-(c + q) // block) for c, q in zip(ctx_lens, q_lens)]
    num_pages = sum(pages_per) + 1
    perm = torch.randperm(num_pages - 1, generator=g).tolist()
    table = torch.full((nreq + 1, max(pages_per)), -1, dtype=torch.int32)
    it = iter(perm)
    for r, k in enumerate(pages_per):
        table[r, :k] = torch.tensor([next(it) for _ in range(k)], dtype=torch.int32)
    pool = (torch.randn(num_pages, block * dk, generator=g) * 0.5).to(torch.bfloat16)
    q_head = 8 + rot
    width = heads * q_head + heads + 6
    width += -width % 8
    rows = torch.randn(n, width, generator=g).to(torch.bfloat16)
    qa = (torch.randn(n, heads * rank, generator=g) * 0.3).to(torch.bfloat16)
    gate_col = heads * q_head
    cu = [0]
    for q in q_lens:
        cu.append(cu[-1] + q)
    positions = torch.tensor([c + i for c, q in zip(ctx_lens, q_lens) for i in range(q)], dtype=torch.int32)
    token_row = torch.tensor([r for r, q in enumerate(q_lens) for _ in range(q)], dtype=torch.int32)
    batch = SimpleNamespace(max_q_len=max(q_lens), num_requests=nreq, max_seq_len=max(c + q for c, q in zip(ctx_lens, q_lens)),
                            cu_q=torch.tensor(cu, dtype=torch.int32).cuda(), context_lens=torch.tensor(ctx_lens, dtype=torch.int32).cuda(),
                            state_slots=torch.arange(nreq, dtype=torch.int32).cuda(), workspace=Workspace("cuda:0"))
    scale = 0.5 / math.sqrt(dk)
    args = (qa.cuda(), rows.cuda(), q_head, 8, gate_col, pool.cuda(), table.cuda(), positions.cuda(), token_row.cuda(),
            heads, rank, rot, block, scale)
    fast = latent.attention_latent(*args, batch=batch).float().cpu()
    slow = latent.attention_latent(*args, batch=None).float().cpu()
    keys = pool.view(num_pages, block, dk).double()
    want = torch.zeros(n, heads, rank, dtype=torch.float64)
    for i in range(n):
        r, p = int(token_row[i]), int(positions[i])
        k = torch.cat([keys[int(table[r, b])] for b in range(p // block + 1)])[:p + 1]
        for h in range(heads):
            q = torch.cat([qa[i, h * rank:(h + 1) * rank], rows[i, h * q_head + 8:(h + 1) * q_head]]).double()
            w = torch.softmax(k @ q * scale, 0)
            want[i, h] = (w[:, None] * k[:, :rank]).sum(0) * torch.sigmoid(rows[i, gate_col + h].double())
    want = want.view(n, heads * rank)
    torch.testing.assert_close(slow.double(), want, rtol=2e-2, atol=4e-3)
    torch.testing.assert_close(fast.double(), want, rtol=2e-2, atol=6e-3)
