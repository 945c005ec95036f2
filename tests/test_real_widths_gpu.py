"""One layer at the widths of real checkpoints through bin/trace_run against the plain
implementation, in bfloat16: the tiny configurations never reach the tile sizes, K cuts and
group sizes that the tensor-core kernels meet there.

W4:  hidden 2560, 32 query heads over 8 KV heads, head_dim 128, intermediate 9728 (groups of 4).
W14: hidden 5120, 40 query heads over 8 KV heads, head_dim 128, intermediate 17408 (groups of
     5, which do not divide a 128-row tile), a window of 100 keys, untied head.
Each sequence is replayed whole, with its last 32 tokens one by one, and in portions of
changing size; every position's logits are compared.
"""

import pytest
import torch

import plain_qwen3 as plain
from traces import Trace, compare, first_wrong, last_decoded, portions, run_trace, whole

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
TOL = 2e-2          # as for the tiny configurations in bfloat16 (tests/test_replay_gpu.py)


@pytest.fixture(scope="module", params=sorted(WIDE))
def replayed(request, tmp_path_factory):
    from socrates_b200.config import config_from_dict
    from socrates_b200.weights import write_model_folder
    name = request.param
    tmp = tmp_path_factory.mktemp(f"wide_{name}")
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
    result = run_trace(folder, "bfloat16", trace, trace.most_held, tmp / "out")
    return dict(name=name, trace=trace, result=result, reference=reference)


def test_every_position_matches_the_plain_implementation(replayed):
    r = replayed
    key = lambda rid: rid.split(":")[1]
    worst, where = compare(r["trace"], r["result"], r["reference"], key)
    bad = first_wrong(r["trace"], r["result"], r["reference"], TOL, key)
    assert bad is None, (f"{r['name']}: first wrong logits at step {bad[0]}, request {bad[1]}, position {bad[2]} "
                         f"(error {bad[3]:.3g} > {TOL}); worst {worst:.3g} at {where}")
