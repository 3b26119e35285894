"""Guvetar on the GPU against the plain implementation: each mixer alone, whole prompts against token
by token decoding and portions of every size, mixed batches over a pool so small that pages and state
slots are used again, keys far away and at the edges of pages and key blocks, the first tokens, long
decoding through the decode graphs, other sizes, and greedy generation through the engine."""

import copy
import os

import numpy as np
import pytest
import torch

from plain_guvetar import plain_forward
from replay_helpers import (BF16_TOL_MAX, BF16_TOL_MEAN, FP32_TOL, LENGTHS, compare, mixed_steps, replay, rounded,
                            run_steps, sequences, single_request_steps)
from tiny_guvetar import GUVETAR, draw_weights, single_mixer, write_model

pytestmark = pytest.mark.gpu

PAGE = {"A": 4, "B": 8, "C": 16, "D": 16, "E": 16}


def tolerance(dtype):
    return (FP32_TOL, None) if dtype == "float32" else (BF16_TOL_MAX, BF16_TOL_MEAN)


def make(cfg, tmp_path, dtype, seed=7, max_tokens=512, block_size=16, max_live=4, sharp=None):
    from gllm_b200.engine.replay import build_runner

    sharp = (1.5 if dtype == "float32" else 1.0) if sharp is None else sharp
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
@pytest.mark.parametrize("streams", [None, 2])
@pytest.mark.parametrize("kind", ["mamba1", "mlstm", "parallel", "sigmoid_only", "hgrn2_only"])
def test_each_mixer_alone(kind, streams, dtype, tmp_path):
    cfg = single_mixer(kind, streams)
    weights, _, runner = make(cfg, tmp_path, dtype)
    toks = torch.randint(0, cfg["vocab"], (75,), generator=torch.Generator().manual_seed(2)).tolist()
    plain = {"r": plain_forward(cfg, weights, toks)}
    steps, index = steps_of(toks, [40] + [1] * 35)
    compare(run_steps(runner, steps), index, plain, *tolerance(dtype))
    steps, index = steps_of(toks, [75])
    compare(run_steps(runner, steps), index, plain, *tolerance(dtype))


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_all_cuts_and_mixed_batches(name, dtype, tmp_path):
    cfg = GUVETAR[name]
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


def test_replay_through_the_command(tmp_path):
    cfg = GUVETAR["A"]
    weights = draw_weights(cfg, seed=7, sharp=1.5)
    folder = write_model(cfg, weights, str(tmp_path / "model"))
    seqs = sequences(cfg["vocab"], seed=6)
    plain = {k: plain_forward(cfg, weights, v) for k, v in seqs.items()}
    steps, index = mixed_steps(seqs, max_tokens=448, seed=3)
    results = replay(folder, "float32", steps, str(tmp_path / "out"), max_tokens=448, vocab=cfg["vocab"])
    compare(results, index, plain, FP32_TOL)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_portions_at_every_edge(dtype, tmp_path):
    """Portions that end just before, at and just after the edges the kernels have: pages of 16, the
    recurrences' chunks of 8 tokens, the attention's blocks of 32 keys, the convolution's taps."""
    cfg = GUVETAR["A"]
    weights, _, runner = make(cfg, tmp_path, dtype, max_tokens=256)
    toks = torch.randint(0, cfg["vocab"], (200,), generator=torch.Generator().manual_seed(8)).tolist()
    plain = {"r": plain_forward(cfg, weights, toks)}
    for cuts in ([7, 1, 1, 7, 15, 2, 31, 1, 33, 16, 17, 9, 8, 2, 2, 3, 45],
                 [2, 2, 2, 2, 8, 16, 32, 64, 63, 9],
                 [1, 1, 1, 1, 1, 3, 24, 31, 33, 104]):
        steps, index = steps_of(toks, cuts)
        compare(run_steps(runner, steps), index, plain, *tolerance(dtype))


def far_key_model():
    """Sigmoid attention alone, built so that one far key decides the last token's logits: token 1's
    key and token 2's query point the same way in head 0, every other score is far below the head's
    (very negative) bias."""
    cfg = single_mixer("sigmoid_only")
    cfg = copy.deepcopy(cfg)
    left = cfg["layers"][0]["mixer"]["left"]
    left["scale"], left["heads"], left["kv_heads"] = 0.5, 1, 1
    w = draw_weights(cfg, seed=11, sharp=1.0)
    W, d = cfg["width"], left["dim"]
    ca, cb = W - 2, W - 4                       # two slow sine columns: the position adds next to nothing there
    w["embed"][:, [ca, cb]] = 0.0
    w["embed"][1] *= 0.1
    w["embed"][2] *= 0.1
    w["embed"][1, ca] = 6.0
    w["embed"][2, cb] = 6.0
    direction = torch.zeros(d)
    direction[:4] = 1.0
    w["l0.mix.left.k"][:4] *= 0.05            # the other keys have next to nothing along that direction
    w["l0.mix.left.q"][:4] *= 0.05
    w["l0.mix.left.k"][:d, ca] = direction * 3.0
    w["l0.mix.left.q"][:d, cb] = direction * 3.0
    w["l0.mix.left.q.norm"][:] = 1.75
    w["l0.mix.left.k.norm"][:] = 1.5
    w["l0.mix.left.pb"][:] = -12.0
    w["l0.mix.left.v"] *= 3.0
    w["l0.mix.left.o"] *= 2.0
    w["final.norm"][[ca, cb]] = 0.0           # the two marker columns do not reach the logits themselves
    return cfg, {k: v.to(torch.bfloat16).to(torch.float32) for k, v in w.items()}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_far_key_at_page_and_block_edges(dtype, tmp_path):
    from gllm_b200.engine.replay import build_runner

    cfg, weights = far_key_model()
    folder = write_model(cfg, weights, str(tmp_path / "model"))
    _, runner = build_runner(folder, dtype, 1024, block_size=16)
    g = torch.Generator().manual_seed(5)
    n = 600
    tol_max, tol_mean = tolerance(dtype)
    for far in (0, 15, 16, 17, 31, 32, 33, 255, 256, 511):
        toks = torch.randint(3, cfg["vocab"], (n,), generator=g).tolist()
        toks[far], toks[-1] = 1, 2
        plain = plain_forward(cfg, weights, toks)
        without = list(toks)
        without[far] = 3
        blind = plain_forward(cfg, weights, without)
        scale = max(1.0, float(plain.abs().max()))
        # the test is sharp: losing that one key moves the last logits by far more than the tolerance
        assert float((plain[-1] - blind[-1]).abs().max()) > (20 if dtype == "float32" else 4) * tol_max * scale
        # the last token in a portion, and decoded alone
        for cuts in ([n], [n - 1, 1], [far + 1, n - far - 3, 2] if far + 3 < n else [n]):
            steps, index = steps_of(toks, cuts)
            compare(run_steps(runner, steps), [i for i in index if i[3] >= n - 2], {"r": plain}, tol_max, None)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_first_tokens_and_long_decoding(dtype, tmp_path):
    """Prompts of one, two and three tokens, then hundreds of tokens decoded one by one (replays of the
    decode graph): state that is lost, doubled or started wrong shows at once or adds up."""
    cfg = GUVETAR["C"]
    weights, _, runner = make(cfg, tmp_path, dtype, max_tokens=512)
    g = torch.Generator().manual_seed(12)
    for first in (1, 2, 3):
        n = first + (330 if first == 2 else 20)
        toks = torch.randint(0, cfg["vocab"], (n,), generator=g).tolist()
        plain = {"r": plain_forward(cfg, weights, toks)}
        steps, index = steps_of(toks, [first] + [1] * (n - first))
        compare(run_steps(runner, steps), index, plain, *tolerance(dtype))
    assert runner.graph_replays > 300


def test_single_tokens_over_a_long_context_on_the_tensor_cores(tmp_path):
    """bfloat16 with head widths the tensor-core attention takes: a context of 900 tokens, then single tokens
    whose keys are cut into ranges with one CTA each (the partial results are added afterwards), alone and two
    requests at once; then the same tokens through the CUDA-core kernel agree with them."""
    cfg = GUVETAR["E"]
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


def test_a_slot_and_its_pages_used_again_start_clean(tmp_path):
    """One state slot and a pool of four pages: the second request gets the first one's slot and pages."""
    cfg = GUVETAR["A"]
    weights, _, runner = make(cfg, tmp_path, "float32", max_tokens=64, max_live=1)
    g = torch.Generator().manual_seed(13)
    a = torch.randint(0, cfg["vocab"], (60,), generator=g).tolist()
    b = torch.randint(0, cfg["vocab"], (50,), generator=g).tolist()
    for rid, toks, cuts in (("a", a, [33, 20, 7]), ("b", b, [3, 40] + [1] * 7), ("c", a, [60])):
        steps, index = steps_of(toks, cuts, rid=rid)
        compare(run_steps(runner, steps), index, {rid: plain_forward(cfg, weights, toks)}, FP32_TOL)
    assert runner.cache.groups[0].allocator.total_reused > 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "D"])
def test_greedy_generation_through_the_entry_point(name, dtype, tmp_path):
    from gllm_b200 import GenerationRequest, GeneratorParams, LLMEngine

    cfg = GUVETAR[name]
    weights = draw_weights(cfg, seed=21, sharp=1.0)
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
    if name == "A":
        assert engine.counters["preemptions"] >= 1
    if dtype == "float32":
        for req, r in zip(reqs, results):
            assert engine.generate([req])[0].token_ids == r.token_ids


def test_random_weights_mode_writes_a_model_that_runs(tmp_path):
    from gllm_b200.config import load_config
    from gllm_b200.engine.replay import build_runner
    from gllm_b200.weights import write_random_model

    folder = write_random_model(str(tmp_path / "m"), load_config(copy.deepcopy(GUVETAR["C"])), seed=3)
    assert os.path.isfile(os.path.join(folder, "model.safetensors"))
    _, runner = build_runner(folder, "bfloat16", 128)
    steps, _ = steps_of(list(range(40)), [30, 1, 9])
    out = run_steps(runner, steps)
    assert all(np.isfinite(v).all() for v in out.values())
