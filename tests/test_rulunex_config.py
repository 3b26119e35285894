"""Rulunex without a GPU: the configuration, the spec's tensor list against the names and shapes the tests' own
writer uses, the order in which layers run, the cache the plan asks for, and the plain implementation's masks."""

import copy

import pytest
import torch

from plain_rulunex import (plain_forward, plain_frequencies, plain_layer_order, plain_rotate,
                           plain_softmax_attention)
from tiny_rulunex import RULUNEX, draw_weights, single_mixer, tensor_shapes


def spec_of(raw):
    from gllm_b200.config import load_config
    from gllm_b200.config.registry import architecture_for

    cfg = load_config(copy.deepcopy(raw))
    return cfg, architecture_for(cfg.architecture).build_spec(cfg)


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_the_spec_expects_the_designs_tensors(name):
    from gllm_b200.models.decoder import expected_tensors_of_spec

    cfg, spec = spec_of(RULUNEX[name])
    expected = {k: tuple(v.shape) for k, v in expected_tensors_of_spec(spec).items()}
    assert expected == tensor_shapes(RULUNEX[name])
    assert cfg.to_dict()["layers"] == RULUNEX[name]["layers"]
    assert type(cfg).from_dict(cfg.to_dict()) == cfg


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_the_plan_follows_the_repeated_stretch(name):
    _, spec = spec_of(RULUNEX[name])
    assert [(e.layer, e.rejoins_embedding) for e in spec.plan] == plain_layer_order(RULUNEX[name])
    assert (spec.rejoin_name is not None) == ("loop" in RULUNEX[name])


def test_a_pass_of_no_layers_and_a_stretch_that_never_runs():
    raw = copy.deepcopy(RULUNEX["A"])
    raw["loop"]["times"] = 0
    _, spec = spec_of(raw)
    assert [e.layer for e in spec.plan] == [0, 3]
    assert not any(e.rejoins_embedding for e in spec.plan)


def test_configuration_errors_name_the_place():
    from gllm_b200.config.model_config import ConfigError

    for edit, message in (
        (lambda d: d["layers"][0]["mixer"].pop("scale"), "lacks 'scale'"),
        (lambda d: d["layers"][0].update(type="conv"), "unknown layer type"),
        (lambda d: d["layers"][0]["mixer"].update(vdim=8), "vdim must equal dim"),
        (lambda d: d["layers"][0]["mixer"].update(kv_heads=3), "multiple of kv_heads"),
        (lambda d: d["layers"][1]["mlp"].pop("limit"), "limit"),
        (lambda d: d["loop"].update(stop=9), "'loop' needs"),
        (lambda d: d.pop("embedding"), "embedding"),
    ):
        raw = copy.deepcopy(RULUNEX["A"])
        edit(raw)
        with pytest.raises(ConfigError, match=message):
            spec_of(raw)


def test_the_cache_manager_gets_one_layer_per_run():
    from gllm_b200.cache.manager import CacheManager
    from gllm_b200.models.decoder import DecoderModel

    _, spec = spec_of(RULUNEX["A"])
    model = DecoderModel(spec, torch.float32, "cpu")
    cache = CacheManager(model.cache_requirements(), block_size=8, num_blocks=6, max_batch_size=2, max_seq_len=48,
                         dtype=torch.float32, device="cpu", allocate_pools=False)
    groups = {(g.requirement.tensors, g.window): len(g.owner_entries) for g in cache.groups}
    # layer 0: keys and values of 2 heads of 32 inside a window of 20; the stretch: three runs each of a latent of
    # 40 + 8 and of 24 + 16 (equal widths, one group); the last layer: keys and values of one head of 48
    assert groups == {(((2, 32), (2, 32)), 20): 1, (((1, 48),), None): 3, (((1, 40),), None): 3,
                      (((1, 48), (1, 48)), None): 1}


def test_plain_masks_and_rotations():
    q = torch.zeros(6, 1, 2, dtype=torch.float64)
    k = torch.zeros(6, 1, 2, dtype=torch.float64)
    v = torch.eye(6, dtype=torch.float64)[:, None, :]
    seen = plain_softmax_attention(q, k, v, 1.0, 3)[:, 0]
    want = torch.tensor([[1, 0, 0, 0, 0, 0], [.5, .5, 0, 0, 0, 0], [1 / 3] * 3 + [0] * 3, [0] + [1 / 3] * 3 + [0, 0],
                         [0, 0] + [1 / 3] * 3 + [0], [0, 0, 0] + [1 / 3] * 3], dtype=torch.float64)
    torch.testing.assert_close(seen, want)
    f = plain_frequencies({"base": 100.0, "dims": 4})
    torch.testing.assert_close(f, torch.tensor([1.0, 0.1], dtype=torch.float64))
    x = torch.tensor([[[1.0, 0.0, 0.0, 1.0, 7.0]]], dtype=torch.float64)
    pos = torch.tensor([2])
    near = plain_rotate(x, pos, f, interleaved=True)[0, 0]
    far = plain_rotate(x, pos, f, interleaved=False)[0, 0]
    c2, s2, c02, s02 = (torch.cos(torch.tensor(2.0)), torch.sin(torch.tensor(2.0)), torch.cos(torch.tensor(0.2)),
                        torch.sin(torch.tensor(0.2)))
    torch.testing.assert_close(near, torch.tensor([c2, s2, -s02, c02, 7.0], dtype=torch.float64))
    torch.testing.assert_close(far, torch.tensor([c2, -s02, s2, c02, 7.0], dtype=torch.float64))
    # scaling: short wavelengths stay, long ones are slowed by the factor
    scaled = plain_frequencies({"base": 10000.0, "dims": 8, "scaling": {"factor": 4.0, "low": 1.0, "high": 4.0,
                                                                         "original": 64}})
    plain = plain_frequencies({"base": 10000.0, "dims": 8})
    assert scaled[0] == plain[0] and abs(float(scaled[-1] / plain[-1]) - 0.25) < 1e-12
    assert plain[1] / 4 < scaled[1] < plain[1]


def test_the_plain_model_is_causal_and_windowed():
    cfg = single_mixer("window")
    w = draw_weights(cfg, seed=3, sharp=2.0)
    g = torch.Generator().manual_seed(1)
    toks = torch.randint(0, cfg["vocab"], (60,), generator=g).tolist()
    base = plain_forward(cfg, w, toks)
    later = list(toks)
    later[20] = (later[20] + 1) % cfg["vocab"]
    moved = plain_forward(cfg, w, later)
    assert torch.equal(base[:20], moved[:20])                       # nothing before the change moves
    window = cfg["layers"][0]["mixer"]["mask"]["size"]
    assert not torch.equal(base[20 + window - 1], moved[20 + window - 1])
    assert torch.equal(base[20 + window:], moved[20 + window:])     # and nothing once the window has passed it
