"""Typed configuration and the architecture registry."""

import json

import pytest
import torch

from socrates_b200.config import (ConfigError, Qwen3Config, config_from_dict, known_architectures,
                                  load_config, register_architecture, unregister_architecture)
from tiny_configs import TINY_A, TINY_B


def test_reads_every_size_from_config():
    a, b = config_from_dict(TINY_A), config_from_dict(TINY_B)
    assert (a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (64, 4, 2, 16)
    assert (b.hidden_size, b.num_attention_heads, b.num_key_value_heads, b.head_dim) == (96, 8, 2, 32)
    assert a.tie_word_embeddings and not b.tie_word_embeddings
    assert a.rms_norm_eps == 1e-6 and b.rms_norm_eps == 1e-5
    assert a.rope_theta == 1e4 and b.rope_theta == 1e6
    assert a.layer_windows == (None, None)
    assert b.layer_windows == (None, 37, 37)


def test_head_dim_defaults_to_hidden_over_heads():
    d = dict(TINY_A)
    del d["head_dim"]
    assert config_from_dict(d).head_dim == 16


def test_missing_keys_are_named():
    d = dict(TINY_A)
    del d["rope_theta"], d["rms_norm_eps"]
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert "rope_theta" in str(e.value) and "rms_norm_eps" in str(e.value)


@pytest.mark.parametrize("key,value", [("attention_bias", True), ("hidden_act", "gelu"),
                                       ("rope_scaling", {"type": "yarn"}), ("num_key_value_heads", 3)])
def test_unsupported_options_are_refused(key, value):
    d = dict(TINY_A)
    d[key] = value
    with pytest.raises(ConfigError):
        config_from_dict(d)


def test_unknown_architecture_lists_known():
    d = dict(TINY_A, architectures=["LlamaForCausalLM"])
    with pytest.raises(ConfigError) as e:
        config_from_dict(d)
    assert "Qwen3ForCausalLM" in str(e.value)
    assert "Qwen3ForCausalLM" in known_architectures()


def test_round_trip_through_json(tmp_path):
    for src in (TINY_A, TINY_B):
        cfg = config_from_dict(src)
        (tmp_path / "config.json").write_text(json.dumps(cfg.to_dict()))
        assert load_config(tmp_path) == cfg


def test_layer_types_select_windows():
    d = dict(TINY_B, layer_types=["sliding_attention", "full_attention", "sliding_attention"])
    assert config_from_dict(d).layer_windows == (37, None, 37)


def test_plan_is_data():
    plan = config_from_dict(TINY_B).plan()
    assert len(plan.layers) == 3 and [e.layer for e in plan.order] == [0, 1, 2]
    assert plan.layers[0].mixer.params["window"] is None
    assert plan.layers[2].mixer.params["window"] == 37
    assert plan.layers[1].mixer.params["num_kv_heads"] == 2
    assert plan.head.params["tied_to"] is None
    assert config_from_dict(TINY_A).plan().head.params["tied_to"] == "model.embed_tokens.weight"


def test_register_another_architecture():
    class Other(Qwen3Config):
        architecture = "OtherForCausalLM"
    register_architecture("OtherForCausalLM", Other)
    try:
        cfg = config_from_dict(dict(TINY_A, architectures=["OtherForCausalLM"]))
        assert isinstance(cfg, Other)
        with pytest.raises(ValueError):
            register_architecture("OtherForCausalLM", Other)
    finally:
        unregister_architecture("OtherForCausalLM")


def test_page_pool_from_memory():
    """`num_blocks=None`: pages from the memory that is free after the weights, never more than
    every row at full length, never fewer than one row needs; an explicit number is kept."""
    from socrates_b200.cache import CacheManager, CacheNeeds, PagedKVSpec
    from socrates_b200.config import EngineConfig
    cfg = EngineConfig(max_batch=64, max_len=8192, block_size=16)
    full = 64 * 512
    # the 32B shape: 64 layers of 8 KV heads of 128, bfloat16 -> 256 KiB a token, 4 MiB a page
    needs = [CacheNeeds(PagedKVSpec(8, 128, None)) for _ in range(64)]
    per_page = CacheManager.bytes_per_page(needs, 16, torch.bfloat16)
    assert per_page == 64 * 2 * 8 * 16 * 128 * 2
    assert cfg.pages_from_memory(10 ** 15, per_page) == full               # memory is no limit: the worst case
    got = cfg.pages_from_memory(110 * 2 ** 30, per_page)                   # 110 GiB free beside the weights
    assert got == int(110 * 2 ** 30 * 0.9) // per_page and 512 <= got < full
    assert cfg.pages_from_memory(1, per_page) == 512                       # at least one row
    assert EngineConfig(num_blocks=77).pages_from_memory(10 ** 15, per_page) == 77
    with pytest.raises(ValueError):
        EngineConfig(kv_memory_fraction=0.0).validate()
