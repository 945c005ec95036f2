"""Command line of the engine, in the manner of the reference's

    ENGINE=paged uv run -m model.inference_paged        (model/inference_paged.py:1-4, 240-255)

which builds an Engine, submits a list of prompts, runs, and prints each output and a
line `wall | tokens | tok/s`.  Here:

    MODEL_ID=/path/to/folder python -m socrates_b200.inference_paged
    python -m socrates_b200.inference_paged --model DIR --prompt "how to make pizza?"
    python -m socrates_b200.inference_paged --model DIR --prompt-ids 5,17,3 --max-new-tokens 32
    python -m socrates_b200.inference_paged --random-config config.json --seed 0 --num-prompts 16

Environment variables keep the reference's names and meanings where it has them and
are overridden by the flags:

    MODEL_ID         the model (there: a hub id picking a pinned config; here: a folder with
                     config.json and safetensors)            model/qwen/qwen_kv_cont.py:26
    DEVICE           device, default cuda:0                  model/inference_cont.py:29
    COMPILE          0 disables the CUDA graphs of the decode step (there: torch.compile)
                                                             model/inference_cont.py:43
    KV_BLOCK         slots per page, default 16              model/inference_paged.py:51
    ENGINE           only "paged" exists here                model/server.py:79-85
    ATTN_IMPL        auto or cuda (there also ref, the PyTorch fallback: refused here, there is
                     no path beside the CUDA kernels)        model/kernels/__init__.py:23-35
    PAGED_PARTITION  auto, or keys per partition of the split-key decode attention, 0 = one
                     pass                                    model/kernels/__init__.py:36-41
    MAX_BATCH, MAX_LEN, MAX_NEW_TOKENS   the reference's module constants
                                                             model/inference_cont.py:21-23

A folder that holds tokenizer.json is tokenised with its own tokenizer and chat template and
its outputs are printed as text, as the reference prints them (model/inference_paged.py:67-70,
139-143, 242-251); a folder without one (random weights) gets a byte tokenizer.  `--num-blocks`
not given: the page pool is sized from the memory that is free after the weights.

There is no server.
"""

from __future__ import annotations

import argparse
import json
import os
import sys
import tempfile
import time
from pathlib import Path


def _env_flag(name: str, default: str = "1") -> bool:
    return os.environ.get(name, default) not in ("0", "false", "False")


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m socrates_b200.inference_paged",
                                 description="Generate with the paged engine on one GPU.")
    ap.add_argument("--model", default=os.environ.get("MODEL_ID"),
                    help="folder with config.json and model.safetensors (env MODEL_ID)")
    ap.add_argument("--random-config", help="a config.json; a model folder with random weights is made from it")
    ap.add_argument("--seed", type=int, default=0, help="seed of the random weights and of sampling")
    ap.add_argument("--device", default=os.environ.get("DEVICE", "cuda:0"))
    ap.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
    ap.add_argument("--max-batch", type=int, default=int(os.environ.get("MAX_BATCH", "18")))
    ap.add_argument("--max-len", type=int, default=int(os.environ.get("MAX_LEN", "2048")))
    ap.add_argument("--max-new-tokens", type=int, default=int(os.environ.get("MAX_NEW_TOKENS", "64")))
    ap.add_argument("--block-size", type=int, default=int(os.environ.get("KV_BLOCK", "16")))
    ap.add_argument("--num-blocks", type=int, default=None, help="pages in the pool (default: from free memory, at most max_batch rows of max_len)")
    ap.add_argument("--token-budget", type=int, default=2048, help="most tokens one step runs")
    ap.add_argument("--temperature", type=float, default=0.0, help="0 = greedy")
    ap.add_argument("--no-compile", action="store_true", help="no CUDA graphs (same as COMPILE=0)")
    ap.add_argument("--no-warmup", action="store_true",
                    help="record each decode graph at the first step of its width instead of at start-up")
    ap.add_argument("--prompt", action="append", default=[], help="a text prompt (the folder's tokenizer and chat template, else bytes); repeatable")
    ap.add_argument("--prompt-ids", action="append", default=[], help="a prompt as comma-separated token ids; repeatable")
    ap.add_argument("--num-prompts", type=int, default=0, help="this many random prompts")
    ap.add_argument("--prompt-len", type=int, default=32, help="length of the random prompts")
    args = ap.parse_args(argv)

    if os.environ.get("ENGINE", "paged") != "paged":
        print(f"ENGINE={os.environ['ENGINE']!r}: only the paged engine exists here", file=sys.stderr)
        return 2
    if os.environ.get("ATTN_IMPL", "auto") not in ("auto", "cuda"):
        print(f"ATTN_IMPL={os.environ['ATTN_IMPL']!r}: this engine has the CUDA kernels only (auto or cuda)",
              file=sys.stderr)
        return 2

    import torch

    from .config import config_from_dict, load_config
    from .engine.engine import Engine
    from .engine.tokenizer import load_tokenizer
    from .weights import write_model_folder

    tmp = None
    model_dir = args.model
    if args.random_config:
        tmp = tempfile.TemporaryDirectory()
        cfg = config_from_dict(json.loads(Path(args.random_config).read_text()))
        model_dir = str(write_model_folder(cfg, args.seed, Path(tmp.name) / "model"))
    if not model_dir:
        ap.error("give --model DIR (or MODEL_ID=DIR), or --random-config CONFIG.json")

    vocab = load_config(model_dir).plan().vocab_size
    tok = load_tokenizer(model_dir, vocab)      # the folder's own tokenizer, else bytes
    compile_ = _env_flag("COMPILE") and not args.no_compile
    engine = Engine(model_dir, tok=tok, device=args.device, dtype=args.dtype, compile=compile_,
                    max_batch=args.max_batch, max_len=args.max_len, max_new_tokens=args.max_new_tokens,
                    block_size=args.block_size, num_blocks=args.num_blocks, token_budget=args.token_budget,
                    warmup=not args.no_warmup)

    prompts = list(args.prompt)
    prompts += [[int(t) for t in p.split(",") if t.strip()] for p in args.prompt_ids]
    if args.num_prompts or not prompts:
        g = torch.Generator().manual_seed(args.seed)
        n = args.num_prompts or 4
        prompts += [torch.randint(1, vocab, (args.prompt_len,), generator=g).tolist() for _ in range(n)]

    reqs = [engine.submit(p, temperature=args.temperature, seed=args.seed + i) for i, p in enumerate(prompts)]
    pages = engine.cache.groups[0].allocator.num_pages if engine.cache.groups else 0
    print(f"{len(reqs)} requests, {engine.max_batch} rows, {pages} blocks of {args.block_size}\n")
    t0 = time.perf_counter()
    engine.run()
    torch.cuda.synchronize()
    wall = time.perf_counter() - t0
    for p, r in zip(prompts, reqs):
        shown = p if isinstance(p, str) else " ".join(str(t) for t in p[:16]) + (" ..." if len(p) > 16 else "")
        print(f"> {shown}\n{tok.decode(r.output)}\n")
    total = sum(len(r.output) for r in reqs)
    print(f"{wall:.2f}s | {total} tok | {total / wall:.2f} tok/s")
    if tmp is not None:
        tmp.cleanup()
    return 0


if __name__ == "__main__":
    sys.exit(main())
