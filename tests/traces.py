"""Builders of replay traces and the bookkeeping to compare their logits.

A trace is a list of steps in the format of bin/trace_run.  `Trace.add` also records,
for every row of logits a step will write, which request and which position it
belongs to, so that the output files can be compared with the plain implementation's
whole-sequence logits.
"""

from __future__ import annotations

import json
import random
import subprocess
import sys
from pathlib import Path
from typing import Dict, List, Sequence, Tuple

import numpy as np

ROOT = Path(__file__).resolve().parent.parent


class Trace:
    def __init__(self):
        self.steps: List[dict] = []
        self.expect: Dict[int, List[Tuple[str, int]]] = {}     # step -> [(request, position)]
        self.fed: Dict[str, int] = {}
        self.most_held = 0        # most tokens live requests hold at any time, each rounded up to 64

    def add(self, entries: Sequence[Tuple[str, Sequence[int], Sequence[int]]], end: Sequence[str] = ()):
        """entries: (request id, its next tokens, wanted places among them)."""
        n = len(self.steps)
        rows = []
        out = []
        for rid, tokens, want in entries:
            start = self.fed.get(rid, 0)
            out.append({"id": rid, "tokens": [int(t) for t in tokens], "want": [int(w) for w in want]})
            rows += [(rid, start + w) for w in want]
            self.fed[rid] = start + len(tokens)
        self.steps.append({"step": n, "entries": out, "end": list(end)})
        self.most_held = max(self.most_held, sum(-(-v // 64) * 64 for v in self.fed.values()))
        if rows:
            self.expect[n] = rows
        for rid in end:
            self.fed.pop(rid, None)
        return n

    def text(self) -> str:
        return "".join(json.dumps(s) + "\n" for s in self.steps)


def whole(trace: Trace, rid: str, ids: Sequence[int]):
    trace.add([(rid, ids, range(len(ids)))], end=[rid])


def last_decoded(trace: Trace, rid: str, ids: Sequence[int], tail: int = 32):
    n = len(ids)
    head = n - tail
    trace.add([(rid, ids[:head], range(head))])
    for i in range(head, n):
        trace.add([(rid, ids[i:i + 1], [0])], end=[rid] if i == n - 1 else [])


def portions(trace: Trace, rid: str, ids: Sequence[int], sizes=(7, 2, 16, 3, 2, 33, 5, 17, 2, 64)):
    i, k, n = 0, 0, len(ids)
    while i < n:
        c = min(sizes[k % len(sizes)], n - i)
        if n - i - c == 1:          # never leave a single token: portions go down to two
            c += 1
        trace.add([(rid, ids[i:i + c], range(c))], end=[rid] if i + c == n else [])
        i += c
        k += 1


def mixed(trace: Trace, requests: Dict[str, Sequence[int]], seed: int, live_limit: int = 4, tail: int = 32):
    """Up to `live_limit` requests at a time: portions (2..24 tokens) of prompts beside
    single decoded tokens of requests that are in their last `tail` tokens; some
    requests sit a step out.  A finished request makes room for the next."""
    rng = random.Random(seed)
    waiting = list(requests.items())
    live: Dict[str, int] = {}
    while waiting or live:
        while waiting and len(live) < live_limit and (not live or rng.random() < 0.6):
            rid, _ = waiting.pop(0)
            live[rid] = 0
        entries, ended = [], []
        for rid in list(live):
            ids = requests[rid]
            done, n = live[rid], len(ids)
            if len(live) > 1 and rng.random() < 0.2:
                continue                                     # left out of this step
            if n - done <= tail and done > 0:
                c = 1
            else:
                c = min(rng.randint(2, 24), n - done)
            entries.append((rid, ids[done:done + c], range(c)))
            live[rid] = done + c
            if live[rid] == n:
                ended.append(rid)
                del live[rid]
        if entries:
            trace.add(entries, end=ended)


def run_trace(model_dir, dtype: str, trace: Trace, max_tokens: int, out_dir, env=None, timeout=900):
    """Run bin/trace_run on the trace; returns {step: float32 array [wanted, vocab]}."""
    out_dir = Path(out_dir)
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model_dir), "--dtype", dtype,
           "--out", str(out_dir), "--max-tokens", str(max_tokens)]
    proc = subprocess.run(cmd, input=trace.text(), capture_output=True, text=True, timeout=timeout, env=env)
    if proc.returncode != 0:
        raise RuntimeError(f"trace_run exited with {proc.returncode}\nstdout:\n{proc.stdout[-2000:]}\n"
                           f"stderr:\n{proc.stderr[-4000:]}")
    done = [l for l in proc.stdout.splitlines() if l.startswith("done ")]
    assert [int(l.split()[1]) for l in done] == list(range(len(trace.steps))), "a step was not acknowledged"
    cfg = json.loads((Path(model_dir) / "config.json").read_text())
    V = cfg["vocab_size"]
    result = {}
    for step, rows in trace.expect.items():
        arr = np.fromfile(str(out_dir / f"{step}.f32"), dtype="<f4")
        assert arr.size == len(rows) * V, f"step {step}: {arr.size} floats for {len(rows)} rows of {V}"
        result[step] = arr.reshape(len(rows), V)
    return result


def compare(trace: Trace, result, reference: Dict[str, "np.ndarray"], key=lambda rid: rid):
    """Worst error of every logits row against `reference[key(request)][position]`,
    relative to the largest reference logit of that request; also where it occurred.
    Returns (worst, (step, request, position))."""
    worst, where = 0.0, None
    for step, rows in trace.expect.items():
        got = result[step]
        for i, (rid, pos) in enumerate(rows):
            ref = reference[key(rid)]
            scale = float(np.abs(ref).max())
            err = float(np.abs(got[i] - ref[pos]).max()) / scale
            if not np.isfinite(err):
                err = float("inf")
            if err > worst:
                worst, where = err, (step, rid, pos)
    return worst, where


def first_wrong(trace: Trace, result, reference, tol, key=lambda rid: rid):
    """The first (step, request, position) whose error exceeds `tol`, or None."""
    for step in sorted(trace.expect):
        for i, (rid, pos) in enumerate(trace.expect[step]):
            ref = reference[key(rid)]
            err = float(np.abs(result[step][i] - ref[pos]).max()) / float(np.abs(ref).max())
            if not err <= tol:
                return step, rid, pos, err
    return None
