"""Replay through bin/trace_run against the plain implementation.

The same sequences are replayed whole; most of them in one step and the last 32 tokens
one by one; in portions of changing size down to two tokens; and mixed, up to four
live requests with portions of some beside decoded tokens of others, in a pool so
small that pages are used again.  Both tiny configurations and B without its window (the
shape on which the plain implementation is checked against the reference's own output),
float32 and bfloat16.  Every position's logits are compared.
"""

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
from tiny_configs import ALL_CONFIGS as CONFIGS, make_folder
from traces import Trace, compare, first_wrong, last_decoded, mixed, portions, run_trace, whole

pytestmark = pytest.mark.gpu

# Error of a logits row, relative to the largest logit of its sequence.  float32: the
# reference's own model-level tolerance is 1e-4 (tests/test_paged_model.py:35-76).
# bfloat16: activations are rounded to 8 bits of mantissa about ten times a layer.
TOL = {"float32": 1e-4, "bfloat16": 2e-2}
LENGTHS = {"A": [70, 131, 203], "B": [65, 150, 301], "B0": [65, 150, 301]}


def sequences(name):
    vocab = CONFIGS[name][0]["vocab_size"]
    g = torch.Generator().manual_seed(100 + len(name) + CONFIGS[name][1])
    return {f"s{i}": torch.randint(0, vocab, (n,), generator=g).tolist()
            for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module", params=[(c, d) for c in ("A", "B", "B0") for d in ("float32", "bfloat16")],
                ids=lambda p: f"{p[0]}-{p[1]}")
def replayed(request, tmp_path_factory):
    name, dtype = request.param
    tmp = tmp_path_factory.mktemp(f"replay_{name}_{dtype}")
    folder = make_folder(tmp, name)
    cfg, w = plain.load_folder(folder)
    seqs = sequences(name)
    reference = {k: plain.logits(w, cfg, ids).numpy() for k, ids in seqs.items()}

    trace = Trace()
    spans = {}
    for kind, build in (("whole", whole), ("last32", last_decoded), ("portions", portions)):
        a = len(trace.steps)
        for k, ids in seqs.items():
            build(trace, f"{kind}:{k}", ids)
        spans[kind] = (a, len(trace.steps))
    a = len(trace.steps)
    reqs = {f"mixed{j}:{k}": ids for j in range(2) for k, ids in seqs.items()}
    mixed(trace, reqs, seed=7)
    spans["mixed"] = (a, len(trace.steps))
    # The pool holds exactly what the live requests of the busiest step hold (each
    # rounded up to 64 tokens): far fewer pages than the trace touches, so freed pages
    # are handed out again.
    result = run_trace(folder, dtype, trace, trace.most_held, tmp / "out")
    return dict(name=name, dtype=dtype, trace=trace, result=result, reference=reference, spans=spans)


def _check(r, kind):
    lo, hi = r["spans"][kind]
    sub = Trace()
    sub.expect = {s: rows for s, rows in r["trace"].expect.items() if lo <= s < hi}
    assert sub.expect, "the schedule wrote no logits"
    key = lambda rid: rid.split(":")[1]
    tol = TOL[r["dtype"]]
    worst, where = compare(sub, r["result"], r["reference"], key)
    bad = first_wrong(sub, r["result"], r["reference"], tol, key)
    assert bad is None, (f"{r['name']} {r['dtype']} {kind}: first wrong logits at step {bad[0]}, request "
                         f"{bad[1]}, position {bad[2]} (error {bad[3]:.3g} > {tol}); worst {worst:.3g} at {where}")


def test_whole(replayed):
    _check(replayed, "whole")


def test_last_32_one_by_one(replayed):
    _check(replayed, "last32")


def test_portions_of_changing_size(replayed):
    _check(replayed, "portions")


def test_mixed_with_pages_used_again(replayed):
    _check(replayed, "mixed")


def test_schedules_agree_with_each_other(replayed):
    """In float32 the way of cutting must not matter beyond rounding: whole against the
    other three, position by position, much tighter than against the oracle."""
    r = replayed
    if r["dtype"] != "float32":
        pytest.skip("bfloat16 rounds differently per schedule; covered against the oracle")
    by_pos = {}
    for step, rows in r["trace"].expect.items():
        for i, (rid, pos) in enumerate(rows):
            by_pos.setdefault((rid.split(":")[1], pos), []).append(r["result"][step][i])
    worst = 0.0
    for (seq, pos), rows in by_pos.items():
        scale = float(np.abs(r["reference"][seq]).max())
        for other in rows[1:]:
            worst = max(worst, float(np.abs(other - rows[0]).max()) / scale)
    assert worst <= 2e-5, worst
