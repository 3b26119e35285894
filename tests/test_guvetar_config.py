"""Guvetar without a GPU: its configuration, the tensors its spec expects, the cache manager's state
tensors, and the plain implementation's own consistency (whole sequence against a longer one)."""

import copy

import pytest
import torch

from plain_guvetar import plain_forward
from tiny_guvetar import GUVETAR, draw_weights, single_mixer


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_the_spec_expects_exactly_the_tensors_the_design_names(name):
    from gllm_b200.config import load_config
    from gllm_b200.weights.random_init import expected_tensors_of

    cfg = GUVETAR[name]
    weights = draw_weights(cfg, seed=1)
    expected = expected_tensors_of(load_config(copy.deepcopy(cfg)))
    assert set(expected) == set(weights)
    for key, exp in expected.items():
        assert tuple(exp.shape) == tuple(weights[key].shape), key


def test_config_round_trip_and_errors():
    from gllm_b200.config import ConfigError, GuvetarConfig, load_config

    cfg = load_config(copy.deepcopy(GUVETAR["A"]))
    assert isinstance(cfg, GuvetarConfig) and cfg.streams == 3 and cfg.hidden_size == 64 and cfg.vocab_size == 200
    again = load_config(cfg.to_dict())
    assert again.layers == cfg.layers and again.norm_eps == cfg.norm_eps and again.streams == 3
    assert load_config(copy.deepcopy(GUVETAR["B"])).streams is None
    bad = copy.deepcopy(GUVETAR["A"])
    bad["layers"][1]["type"] = "other"
    with pytest.raises(ConfigError):
        load_config(bad)
    bad = copy.deepcopy(GUVETAR["A"])
    del bad["layers"][2]["mixer"]["dt_rank"]
    with pytest.raises(ConfigError):
        load_config(bad)
    bad = copy.deepcopy(GUVETAR["A"])
    bad["layers"][0]["mixer"]["left"]["kv_heads"] = 3
    with pytest.raises(ConfigError):
        load_config(bad)
    bad = copy.deepcopy(GUVETAR["A"])
    bad["layers"][0]["mlp"] = {"kind": "routed", "ff": 8}
    with pytest.raises(ConfigError):
        load_config(bad)


def test_spec_layers_follow_the_config():
    from gllm_b200.config import load_config
    from gllm_b200.config.registry import architecture_for

    spec = architecture_for("Guvetar").build_spec(load_config(copy.deepcopy(GUVETAR["A"])))
    assert [layer.parts["mixer"].kind for layer in spec.layers] == ["parallel", "exp_gated_memory", "selective_scan",
                                                                    "selective_scan"]
    assert ["feed_forward" in layer.parts for layer in spec.layers] == [True, False, True, False]
    assert spec.residual_streams == 3 and spec.head_name is None and spec.position_sinusoid_base == 10000.0
    plain = architecture_for("Guvetar").build_spec(load_config(copy.deepcopy(GUVETAR["B"])))
    assert plain.residual_streams == 1 and {layer.block for layer in plain.layers} == {"prenorm"}


def test_cache_manager_gives_every_state_tensor_and_zeroes_a_reused_slot():
    from gllm_b200.cache.manager import CacheManager
    from gllm_b200.parts.base import KVPageRequirement, StateRequirement

    two = (StateRequirement((3, 2)), StateRequirement((5,)))
    reqs = [(None, two, None), (KVPageRequirement(((2, 4), (2, 6))), StateRequirement((7,)), None), (None, None, None)]
    cache = CacheManager(reqs, block_size=4, num_blocks=6, max_batch_size=2, max_seq_len=24, dtype=torch.float32,
                         device="cpu")
    caches = cache.mixer_caches()
    assert [len(c.states) for c in caches] == [2, 1, 0]
    assert caches[0].states[0].shape == (3, 3, 2) and caches[0].states[1].shape == (3, 5)
    assert caches[1].state is caches[1].states[0] and caches[1].tensor(1).shape == (7, 2, 4, 6)
    slot = cache.add_request("a").slot
    for c in caches:
        for s in c.states:
            s[slot] = 9.0
    cache.free_request("a")
    assert cache.add_request("b").slot == slot
    assert all(float(s[slot].abs().sum()) == 0.0 for c in caches for s in c.states)


@pytest.mark.parametrize("kind", ["mamba1", "mlstm", "parallel"])
def test_plain_implementation_is_causal(kind):
    """The plain implementation is the tests' measure: the logits of a prefix do not change when
    tokens are appended."""
    cfg = single_mixer(kind, streams=2)
    w = draw_weights(cfg, seed=3)
    toks = torch.randint(0, cfg["vocab"], (19,), generator=torch.Generator().manual_seed(0)).tolist()
    full = plain_forward(cfg, w, toks)
    part = plain_forward(cfg, w, toks[:11])
    assert torch.allclose(full[:11], part, atol=1e-12, rtol=0)
