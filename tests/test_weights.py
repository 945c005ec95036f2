"""Weights by name: dtype rules, the one error that lists everything, random folders."""

import json

import pytest
import torch
from safetensors.torch import load_file, save_file

from socrates_b200.config import config_from_dict
from socrates_b200.engine.model import Model
from socrates_b200.weights import WeightsError, load_weights, random_tensors, write_model_folder
from tiny_configs import TINY_A, TINY_B, make_folder


def expected(cfg_dict):
    return Model(config_from_dict(cfg_dict).plan()).parameters()


def test_expected_names_follow_the_checkpoint():
    names = set(expected(TINY_A))
    assert "model.embed_tokens.weight" in names and "model.norm.weight" in names
    assert "lm_head.weight" not in names                      # tied
    assert "lm_head.weight" in set(expected(TINY_B))          # untied
    for leaf in ("input_layernorm.weight", "post_attention_layernorm.weight",
                 "self_attn.q_proj.weight", "self_attn.k_proj.weight", "self_attn.v_proj.weight",
                 "self_attn.o_proj.weight", "self_attn.q_norm.weight", "self_attn.k_norm.weight",
                 "mlp.gate_proj.weight", "mlp.up_proj.weight", "mlp.down_proj.weight"):
        assert f"model.layers.1.{leaf}" in names
    assert len(names) == 2 * 11 + 2


def test_random_folder_is_seeded_and_loads(tmp_path):
    f1 = make_folder(tmp_path / "x", "A")
    f2 = make_folder(tmp_path / "y", "A")
    a, b = load_file(str(f1 / "model.safetensors")), load_file(str(f2 / "model.safetensors"))
    assert set(a) == set(b) and all(torch.equal(a[k], b[k]) for k in a)
    assert a["model.embed_tokens.weight"].dtype == torch.bfloat16
    assert a["model.norm.weight"].dtype == torch.float32
    assert json.loads((f1 / "config.json").read_text())["architectures"] == ["Qwen3ForCausalLM"]
    w = load_weights(f1, expected(TINY_A), torch.bfloat16, "cpu")
    assert w["model.layers.0.mlp.up_proj.weight"].dtype == torch.bfloat16
    assert w["model.norm.weight"].dtype == torch.float32      # stored in 32-bit: stays so
    w32 = load_weights(f1, expected(TINY_A), torch.float32, "cpu")
    assert w32["model.layers.0.mlp.up_proj.weight"].dtype == torch.float32
    assert torch.equal(w32["model.layers.0.mlp.up_proj.weight"],
                       w["model.layers.0.mlp.up_proj.weight"].float())
    other = random_tensors(expected(TINY_A), seed=5)
    assert not torch.equal(other["model.embed_tokens.weight"], a["model.embed_tokens.weight"])


def test_matrix_stored_in_float32_stays_float32(tmp_path):
    folder = make_folder(tmp_path, "A")
    t = load_file(str(folder / "model.safetensors"))
    t["model.layers.0.mlp.up_proj.weight"] = t["model.layers.0.mlp.up_proj.weight"].float()
    save_file(t, str(folder / "model.safetensors"))
    w = load_weights(folder, expected(TINY_A), torch.bfloat16, "cpu")
    assert w["model.layers.0.mlp.up_proj.weight"].dtype == torch.float32
    assert w["model.layers.0.mlp.down_proj.weight"].dtype == torch.bfloat16


def test_one_error_lists_missing_unexpected_and_shapes(tmp_path):
    folder = make_folder(tmp_path, "A")
    t = load_file(str(folder / "model.safetensors"))
    del t["model.layers.1.self_attn.k_norm.weight"]
    del t["model.norm.weight"]
    t["model.layers.0.extra.weight"] = torch.zeros(3)
    t["lm_head.weight"] = torch.zeros(256, 64, dtype=torch.bfloat16)   # tied config: not asked for
    t["model.layers.0.mlp.down_proj.weight"] = torch.zeros(64, 127, dtype=torch.bfloat16)
    save_file(t, str(folder / "model.safetensors"))
    with pytest.raises(WeightsError) as e:
        load_weights(folder, expected(TINY_A), torch.bfloat16, "cpu")
    err = e.value
    assert set(err.missing) == {"model.layers.1.self_attn.k_norm.weight", "model.norm.weight"}
    assert set(err.unexpected) == {"model.layers.0.extra.weight", "lm_head.weight"}
    assert len(err.wrong_shape) == 1 and "down_proj" in err.wrong_shape[0]
    msg = str(err)
    for needle in ("k_norm", "model.norm.weight", "extra", "lm_head", "(64, 127)", "(64, 128)"):
        assert needle in msg


def test_missing_file_is_an_error(tmp_path):
    with pytest.raises(WeightsError):
        load_weights(tmp_path, expected(TINY_A), torch.bfloat16, "cpu")


def test_sharded_folder_with_index(tmp_path):
    folder = make_folder(tmp_path, "A")
    t = load_file(str(folder / "model.safetensors"))
    names = sorted(t)
    half = len(names) // 2
    save_file({k: t[k] for k in names[:half]}, str(folder / "model-00001-of-00002.safetensors"))
    save_file({k: t[k] for k in names[half:]}, str(folder / "model-00002-of-00002.safetensors"))
    (folder / "model.safetensors").unlink()
    wm = {k: ("model-00001-of-00002.safetensors" if i < half else "model-00002-of-00002.safetensors")
          for i, k in enumerate(names)}
    (folder / "model.safetensors.index.json").write_text(json.dumps({"weight_map": wm}))
    w = load_weights(folder, expected(TINY_A), torch.bfloat16, "cpu")
    assert set(w) == set(names)


def test_copy_of_a_tied_head_is_accepted_only_if_faithful(tmp_path):
    """A tied configuration whose file also carries lm_head.weight: accepted when it repeats
    the embedding bit for bit, reported when it differs (the file and config.json would then
    disagree about what the head is)."""
    from socrates_b200.config import config_from_dict
    from socrates_b200.engine.model import Model
    folder = make_folder(tmp_path, "A")
    model = Model(config_from_dict(TINY_A).plan())
    assert model.duplicates() == {"lm_head.weight": "model.embed_tokens.weight"}
    t = load_file(str(folder / "model.safetensors"))
    t["lm_head.weight"] = t["model.embed_tokens.weight"].clone()
    save_file(t, str(folder / "model.safetensors"))
    w = load_weights(folder, model.parameters(), torch.bfloat16, "cpu", model.duplicates())
    assert "lm_head.weight" not in w and "model.embed_tokens.weight" in w
    t["lm_head.weight"][3, 5] += 1
    save_file(t, str(folder / "model.safetensors"))
    with pytest.raises(WeightsError) as e:
        load_weights(folder, model.parameters(), torch.bfloat16, "cpu", model.duplicates())
    assert len(e.value.unexpected) == 1 and "differs from model.embed_tokens.weight" in e.value.unexpected[0]
    # an untied configuration declares no such copy
    from tiny_configs import TINY_B
    assert Model(config_from_dict(TINY_B).plan()).duplicates() == {}
