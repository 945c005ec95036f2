"""Each part alone on the GPU against the plain implementation's function for it."""

import pytest
import torch

import plain_qwen3 as plain
from tiny_configs import TINY_B, make_folder

pytestmark = pytest.mark.gpu
DEV = "cuda"


def setup(tmp_path, dtype):
    from socrates_b200.cache import CacheManager
    from socrates_b200.engine.engine import build_model
    from socrates_b200.engine.runner import ModelRunner
    folder = make_folder(tmp_path, "B")
    cfg, w = plain.load_folder(folder)
    config, model = build_model(folder, dtype, DEV)
    cache = CacheManager(model.cache_needs(), 4, 256, 16, 40, dtype, DEV)
    runner = ModelRunner(model, cache, dtype, DEV, max_tokens=256, max_seqs=4, use_graphs=False)
    return cfg, {k: v.double() for k, v in w.items()}, model, cache, runner


def tol(dtype):
    return dict(atol=2e-5, rtol=2e-4) if dtype == torch.float32 else dict(atol=1e-2, rtol=3e-2)


def feed(runner, cache, row, tokens, start):
    from socrates_b200.engine.runner import StepEntry
    if not cache.active[row]:
        cache.assign(row)
    assert cache.reserve(row, start + len(tokens))
    return runner.prepare([StepEntry(row, tokens, start, [len(tokens) - 1])])


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_norm_part(tmp_path, dtype):
    from socrates_b200.parts import Branch, ResidualStream
    cfg, w, model, cache, runner = setup(tmp_path, dtype)
    ctx = feed(runner, cache, 0, [1, 2, 3, 4, 5], 0)
    norm = model.layers[1].norms[0]
    res = torch.randn(5, 96, device=DEV)
    delta = torch.randn(2, 5, 96, device=DEV)
    stream = ResidualStream(res.clone())
    stream.pending = Branch(delta)
    out = norm.apply(ctx, stream)
    total = (res + delta[0] + delta[1]).double().cpu()
    want = plain.rms_norm(total, w["model.layers.1.input_layernorm.weight"], cfg["rms_norm_eps"])
    assert stream.pending is None
    assert torch.allclose(stream.residual.cpu().double(), total, atol=1e-6)
    assert torch.allclose(out.double().cpu(), want, **tol(dtype))


def test_position_part():
    from socrates_b200.config import PartSpec
    from socrates_b200.parts import build_part
    rot = build_part("position", PartSpec("rotary", {"head_dim": 32, "rotary_dim": 32, "theta": 1e6}), "")
    table, r = rot.tables(DEV)
    want = 1.0 / (1e6 ** (torch.arange(0, 32, 2).float() / 32))
    assert r == 32 and torch.equal(table.cpu(), want)
    none = build_part("position", PartSpec("none", {}), "")
    assert none.tables(DEV)[1] == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_feed_forward_part(tmp_path, dtype):
    cfg, w, model, cache, runner = setup(tmp_path, dtype)
    ctx = feed(runner, cache, 0, [1, 2, 3, 4, 5, 6, 7], 0)
    x = torch.randn(7, 96, device=DEV).to(dtype)
    branch = model.layers[2].feed_forward.forward(ctx, x)
    want = plain.swiglu(x.double().cpu(), w, "model.layers.2.mlp.")
    assert branch.partial.dtype == torch.float32
    assert torch.allclose(branch.partial.sum(0).double().cpu(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("layer", [0, 1])          # 0: all keys; 1: a window of 37
def test_mixer_part_in_portions(tmp_path, dtype, layer):
    """The attention part fed a sequence in three portions equals plain attention on the whole."""
    from socrates_b200.engine.context import CacheView
    cfg, w, model, cache, runner = setup(tmp_path, dtype)
    n = 90
    x = (torch.randn(n, 96) * 2).to(dtype)
    positions = torch.arange(n)
    window = plain.layer_windows(cfg)[layer]
    want = plain.attention(x.double(), w, f"model.layers.{layer}.self_attn.", cfg, positions, window)
    mixer = model.layers[layer].mixer
    got, start = [], 0
    for count in (50, 2, 38):
        ctx = feed(runner, cache, 1, [0] * count, start)
        branch = mixer.forward(ctx, x[start:start + count].to(DEV).contiguous(), CacheView(cache, layer, True))
        got.append(branch.partial.sum(0).double().cpu())
        cache.commit(1, start + count)
        start += count
    assert torch.allclose(torch.cat(got), want, **tol(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_embedding_and_head(tmp_path, dtype):
    from socrates_b200.engine.context import CacheView
    from socrates_b200.parts import ResidualStream
    cfg, w, model, cache, runner = setup(tmp_path, dtype)
    ids = [5, 9, 200, 383, 0, 17, 17, 42, 300, 1, 2]
    ctx = feed(runner, cache, 2, ids, 0)
    x = model.embedding.forward(ctx)
    want_x = w["model.embed_tokens.weight"][torch.tensor(ids)]
    assert torch.equal(x.double().cpu(), want_x)
    stream = ResidualStream(x)
    model.layers[0].forward(ctx, stream, CacheView(cache, 0, True))
    total = stream.residual.double().cpu() + stream.pending.partial.sum(0).double().cpu()
    want = plain.block(want_x, w, 0, dict(cfg), torch.arange(len(ids)), None)
    assert torch.allclose(total, want, **tol(dtype))
    h = model.final_norm.apply(ctx, stream, row_index=ctx.logit_index, buffer="normed_out")
    logits = model.head.forward(ctx, h)
    want_l = plain.rms_norm(want[-1:], w["model.norm.weight"], cfg["rms_norm_eps"]) @ w["lm_head.weight"].T
    assert logits.dtype == torch.float32 and logits.shape == (1, cfg["vocab_size"])
    assert torch.allclose(logits.double().cpu(), want_l, **tol(dtype))
