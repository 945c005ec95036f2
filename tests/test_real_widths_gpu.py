"""One layer at the widths of real checkpoints through bin/trace_run against the plain
implementation, in bfloat16 and (W4) in float32: the tiny configurations never reach the tile
sizes, K cuts and group sizes that the kernels meet there.

W4:  hidden 2560, 32 query heads over 8 KV heads, head_dim 128, intermediate 9728 (groups of 4).
W14: hidden 5120, 40 query heads over 8 KV heads, head_dim 128, intermediate 17408 (groups of
     5, which do not divide a 128-row tile), a window of 100 keys, untied head.
Each sequence is replayed whole, with its last 32 tokens one by one, in portions of changing
size, and mixed: up to four live requests, portions of some beside decoded tokens of others, in a
pool so small that pages are used again.  Every position's logits are compared.
"""

import pytest
import torch

import plain_qwen3 as plain
from traces import Trace, compare, first_wrong, last_decoded, mixed, portions, run_trace, whole

pytestmark = pytest.mark.gpu

BASE = {
    "architectures": ["Qwen3ForCausalLM"], "model_type": "qwen3", "num_hidden_layers": 1, "head_dim": 128,
    "rms_norm_eps": 1e-6, "rope_theta": 1000000.0, "attention_bias": False, "hidden_act": "silu",
    "rope_scaling": None, "max_position_embeddings": 4096,
}
WIDE = {
    "W4": dict(BASE, vocab_size=2048, hidden_size=2560, intermediate_size=9728, num_attention_heads=32,
               num_key_value_heads=8, tie_word_embeddings=True, sliding_window=None, use_sliding_window=False),
    "W14": dict(BASE, vocab_size=1000, hidden_size=5120, intermediate_size=17408, num_attention_heads=40,
                num_key_value_heads=8, tie_word_embeddings=False, sliding_window=100, use_sliding_window=True,
                max_window_layers=0),
}
TOL = {"bfloat16": 2e-2, "float32": 1e-4}     # as for the tiny configurations (tests/test_replay_gpu.py)


@pytest.fixture(scope="module", params=[("W4", "bfloat16"), ("W14", "bfloat16"), ("W4", "float32")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def replayed(request, tmp_path_factory):
    from socrates_b200.config import config_from_dict
    from socrates_b200.weights import write_model_folder
    name, dtype = request.param
    tmp = tmp_path_factory.mktemp(f"wide_{name}_{dtype}")
    folder = write_model_folder(config_from_dict(WIDE[name]), 3, tmp / name)
    cfg, w = plain.load_folder(folder)
    g = torch.Generator().manual_seed(5)
    seqs = {f"s{i}": torch.randint(0, WIDE[name]["vocab_size"], (n,), generator=g).tolist()
            for i, n in enumerate((140, 333))}
    reference = {k: plain.logits(w, cfg, ids).numpy() for k, ids in seqs.items()}
    trace = Trace()
    for kind, build in (("whole", whole), ("last32", last_decoded), ("portions", portions)):
        for k, ids in seqs.items():
            build(trace, f"{kind}:{k}", ids)
    mixed(trace, {f"mixed{j}:{k}": ids for j in range(2) for k, ids in seqs.items()}, seed=11)
    result = run_trace(folder, dtype, trace, trace.most_held, tmp / "out")
    return dict(name=name, dtype=dtype, trace=trace, result=result, reference=reference)


def test_every_position_matches_the_plain_implementation(replayed):
    r = replayed
    key = lambda rid: rid.split(":")[1]
    worst, where = compare(r["trace"], r["result"], r["reference"], key)
    tol = TOL[r["dtype"]]
    bad = first_wrong(r["trace"], r["result"], r["reference"], tol, key)
    assert bad is None, (f"{r['name']} {r['dtype']}: first wrong logits at step {bad[0]}, request {bad[1]}, "
                         f"position {bad[2]} (error {bad[3]:.3g} > {tol}); worst {worst:.3g} at {where}")


def test_the_benchmarks_decode_configuration_bfloat16_against_float32():
    """What bench.py times, checked for once: two layers at the Qwen3-4B widths, batch 8,
    2,048-token prompts, then 64 decode steps replayed from the recorded CUDA graph, the same
    tokens fed to the bfloat16 engine and to the float32 engine (same weights, true 32-bit
    kernels) on the GPU; the logits of every decode step agree within the bfloat16 tolerance."""
    from socrates_b200 import Engine
    from socrates_b200.config import config_from_dict
    from socrates_b200.engine.model import Model
    from socrates_b200.engine.runner import SamplingArgs, StepEntry
    from socrates_b200.weights import random_tensors_on_device

    dev = torch.device("cuda:0")
    cfg = dict(WIDE["W4"], num_hidden_layers=2, vocab_size=8192)
    config = config_from_dict(cfg)
    drawn = random_tensors_on_device(Model(config.plan()).parameters(), 0, torch.bfloat16, dev)
    B, T, steps = 8, 2048, 64
    g = torch.Generator().manual_seed(2)
    prompts = torch.randint(0, 8192, (B, T), generator=g).tolist()
    fed = torch.randint(0, 8192, (steps, B), generator=g).tolist()
    logits = {}
    for dtype in (torch.float32, torch.bfloat16):
        model = Model(config.plan())
        model.bind({k: (v.to(dtype) if v.dtype == torch.bfloat16 else v) for k, v in drawn.items()}, dtype)
        eng = Engine((config, model), device="cuda:0", dtype=dtype, max_batch=B, max_len=8192, block_size=16,
                     num_blocks=B * (T + steps + 16) // 16 + 8, token_budget=T, max_new_tokens=steps + 8)
        cache, runner = eng.cache, eng.runner
        for r in range(B):
            cache.assign(r)
            assert cache.reserve(r, T)
            runner.step([StepEntry(r, prompts[r], 0, [])])
            cache.commit(r, T)
        rows = []
        for i in range(steps):
            for r in range(B):
                assert cache.reserve(r, T + i + 1)
            out = runner.step([StepEntry(r, [fed[i][r]], T + i, [0]) for r in range(B)], [SamplingArgs()] * B)
            rows.append(out.logits.float().clone())
            for r in range(B):
                cache.commit(r, T + i + 1)
        runner.check_status()
        assert runner.graph_replays >= steps - 2
        logits[dtype] = torch.stack(rows)
        del eng, model, cache, runner
        torch.cuda.empty_cache()
    ref, got = logits[torch.float32], logits[torch.bfloat16]
    assert torch.isfinite(got).all()
    err = float((got - ref).abs().max() / ref.abs().max())
    assert err < TOL["bfloat16"], err
