"""Trace replay: feed given token ids through a model step by step and write logits.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps are read from standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

Every entry brings the next tokens of request `id`; all entries of a step run as one
batch through the engine's own model, step function, cache manager and kernels (the
ones generation uses: this program has no forward pass, cache or loader of its own).
Nothing is sampled.  For a step in which something is wanted, `<out>/<step>.f32` holds
the logits at the wanted places in the order of the entries and of `want`, as
little-endian float32 `[wanted, vocab]`.  After every step a line `done <step>` is
printed and flushed.  Requests named in `end` give their pages back after the step.
The page pool holds `--max-tokens` slots (rounded up to whole pages), so pages are
used again once requests end.

The nearest thing in the reference is its teacher-forced comparison
(bench/day_8/equivalence.py:68-84) and the hand-driven scenario of
tests/test_paged_model.py:35-76; it has no such program.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
from pathlib import Path
from typing import Dict, List

MAX_LIVE = 8


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run", description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=("bfloat16", "float32"), default="bfloat16")
    ap.add_argument("--out", required=True, help="folder the logits are written to")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time")
    ap.add_argument("--device", default=os.environ.get("DEVICE", "cuda:0"))
    args = ap.parse_args(argv)

    import numpy as np
    import torch

    from ..cache import CacheManager, pages_for
    from ..kernels import require_kernels
    from .engine import build_model, resolve_dtype
    from .runner import ModelRunner, StepEntry

    if not torch.cuda.is_available():
        print("trace_run: no CUDA device; the engine has no CPU path", file=sys.stderr)
        return 2
    require_kernels()
    device = torch.device(args.device)
    torch.cuda.set_device(device)
    dtype = resolve_dtype(args.dtype)
    page = int(os.environ.get("KV_BLOCK", "16"))
    use_graphs = os.environ.get("COMPILE", "1") not in ("0", "false", "False")
    out_dir = Path(args.out)
    out_dir.mkdir(parents=True, exist_ok=True)

    config, model = build_model(args.model, dtype, device)
    num_pages = max(1, pages_for(args.max_tokens, page))
    max_len = num_pages * page
    cache = CacheManager(model.cache_needs(), max_rows=MAX_LIVE, max_len=max_len, page_size=page,
                         num_pages=num_pages, dtype=dtype, device=device)
    runner = ModelRunner(model, cache, dtype, device, max_tokens=max_len, max_seqs=MAX_LIVE,
                         use_graphs=use_graphs)
    rows: Dict[str, int] = {}
    free_rows: List[int] = list(range(MAX_LIVE - 1, -1, -1))

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        step = json.loads(line)
        number = step["step"]
        entries: List[StepEntry] = []
        for e in step.get("entries", []):
            rid = str(e["id"])
            tokens = [int(t) for t in e["tokens"]]
            if rid not in rows:
                if not free_rows:
                    print(f"trace_run: step {number}: more than {MAX_LIVE} live requests", file=sys.stderr)
                    return 3
                rows[rid] = free_rows.pop()
                cache.assign(rows[rid])
            row = rows[rid]
            start = cache.lengths[row]
            if not cache.reserve(row, start + len(tokens)):
                print(f"trace_run: step {number}: request {rid} needs more pages than --max-tokens "
                      f"{args.max_tokens} leaves free", file=sys.stderr)
                return 3
            entries.append(StepEntry(row, tokens, start, [int(w) for w in e.get("want", [])]))
        if entries:
            result = runner.step(entries)
            for e in entries:
                cache.commit(e.row, e.start + len(e.tokens))
            if result.logits is not None:
                arr = result.logits.to("cpu", torch.float32).numpy().astype("<f4", copy=False)
                arr.tofile(str(out_dir / f"{number}.f32"))
            else:
                torch.cuda.current_stream().synchronize()
            runner.check_status()
        for rid in step.get("end", []):
            rid = str(rid)
            if rid in rows:
                row = rows.pop(rid)
                cache.release(row)
                free_rows.append(row)
        print(f"done {number}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
