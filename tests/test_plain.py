"""The plain implementation itself: against the reference's stored outputs, and its parts."""

import hashlib
from pathlib import Path

import pytest
import torch

import plain_qwen3 as plain
from tiny_configs import make_folder

GOLDEN = Path(__file__).resolve().parent / "golden"


def _checksum(w):
    h = hashlib.sha256()
    for k in sorted(w):
        h.update(k.encode())
        h.update(w[k].to(torch.float32).numpy().tobytes())
    return h.hexdigest()


@pytest.mark.parametrize("name", ["A", "B0"])
def test_plain_matches_reference_golden(tmp_path, name):
    """Logits of the reference's own model classes (stored by tests/golden/make_golden.py)."""
    from safetensors import safe_open
    gold = torch.load(GOLDEN / f"golden_{name}.pt")
    cfg, w = gold["config"], {}
    with safe_open(str(GOLDEN / f"golden_{name}.safetensors"), framework="pt") as f:
        for k in f.keys():
            w[k] = f.get_tensor(k)
    assert _checksum(w) == gold["weights_sha256"]              # the weights the reference ran
    mine = plain.logits(w, cfg, gold["ids"], torch.float32)[gold["positions"]]
    assert torch.allclose(mine, gold["logits"], atol=2e-6, rtol=1e-5)
    # and the framework's seeded writer still makes these weights on this machine, or says so
    _, fresh = plain.load_folder(make_folder(tmp_path, name))
    if _checksum(fresh) != gold["weights_sha256"]:
        import warnings
        warnings.warn("this torch draws other random weights than the one that made the golden files")


def test_rms_norm_formula():
    x = torch.tensor([[3.0, 4.0]])
    w = torch.tensor([2.0, 0.5])
    y = plain.rms_norm(x, w, 0.0)
    r = (12.5) ** 0.5
    assert torch.allclose(y, torch.tensor([[3 / r * 2, 4 / r * 0.5]]))


def test_rope_is_a_rotation_and_pairs_halves():
    pos = torch.tensor([0, 3])
    cos, sin = plain.rope_tables(pos, 8, 10000.0)
    x = torch.randn(2, 1, 8, dtype=torch.float64)
    y = plain.apply_rope(x, cos, sin)
    assert torch.allclose(y[0], x[0])                                  # position 0: identity
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1))
    a = 3.0                                                            # dim 0 pairs with dim 4, freq 1
    assert torch.allclose(y[1, 0, 0], x[1, 0, 0] * torch.cos(torch.tensor(a, dtype=torch.float64))
                          - x[1, 0, 4] * torch.sin(torch.tensor(a, dtype=torch.float64)), atol=1e-6)


def test_mask_causal_and_window():
    p = torch.arange(6)
    full = plain.attention_mask(p, p, None)
    assert full[3].tolist() == [True, True, True, True, False, False]
    win = plain.attention_mask(p, p, 2)
    assert win[3].tolist() == [False, False, True, True, False, False]
    assert win[0].tolist() == [True, False, False, False, False, False]


def test_attention_core_gqa_and_uniform_weights():
    T, Hq, Hkv, D = 4, 4, 2, 8
    q = torch.zeros(T, Hq, D, dtype=torch.float64)                     # zero queries: uniform weights
    k = torch.randn(T, Hkv, D, dtype=torch.float64)
    v = torch.randn(T, Hkv, D, dtype=torch.float64)
    keep = plain.attention_mask(torch.arange(T), torch.arange(T), None)
    o = plain.attention_core(q, k, v, D ** -0.5, keep)
    assert torch.allclose(o[2, 0], v[:3, 0].mean(0)) and torch.allclose(o[2, 1], v[:3, 0].mean(0))
    assert torch.allclose(o[2, 2], v[:3, 1].mean(0)) and torch.allclose(o[2, 3], v[:3, 1].mean(0))


def test_logits_are_causal(tmp_path):
    cfg, w = plain.load_folder(make_folder(tmp_path, "B"))
    ids = list(range(3, 60))
    whole = plain.logits(w, cfg, ids)
    part = plain.logits(w, cfg, ids[:20])
    assert torch.allclose(whole[:20], part, atol=1e-12)


def test_window_changes_far_positions_only(tmp_path):
    cfg, w = plain.load_folder(make_folder(tmp_path, "B"))
    cfg0 = dict(cfg, use_sliding_window=False, sliding_window=None)
    cfg0.pop("layer_types", None)
    ids = [(7 * i + 3) % cfg["vocab_size"] for i in range(80)]
    a, b = plain.logits(w, cfg, ids), plain.logits(w, cfg0, ids)
    assert torch.allclose(a[:37], b[:37], atol=1e-12)                  # the window is not yet full
    assert (a[60:] - b[60:]).abs().max() > 1e-6


def test_sampling_reference_is_seeded():
    l = torch.randn(300)
    assert plain.greedy(l) == int(l.argmax())
    a = plain.sample_temperature(l, 0.8, seed=3, counter=5)
    assert a == plain.sample_temperature(l, 0.8, seed=3, counter=5)
    draws = {plain.sample_temperature(l, 0.8, seed=3, counter=c) for c in range(40)}
    assert len(draws) > 5
    u = plain.uniform_for(1, 2, torch.arange(100000))
    assert 0 < float(u.min()) and float(u.max()) < 1 and abs(float(u.mean()) - 0.5) < 0.01
