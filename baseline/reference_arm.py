"""The reference arm of bench.py: the unmodified reference engine, timed on the same workload.

Nothing of socrates_b200 is imported here.  The reference lives as a plain copy of its
`model` package under baseline/_ref (see install_reference.py beside this file), with
its own paged-attention extension built by its own setup.py for compute capability 10.0
(model/kernels/setup.py:8-9,20 of the reference names that switch).  The arm drives the
reference's stock path:

  * `Qwen3Paged(cfg)` (model/qwen/qwen_kv_paged.py:191-224) at the benchmark's shape with
    random weights, matrices N(0, 0.02) and gains 1 + N(0, 0.1), in bfloat16;
  * `model.inference_paged.Engine(model=..., tok=<stub>, device="cuda", compile=<default>)`
    (model/inference_paged.py:55-108): the constructor arguments exist so that the engine
    can run without hub weights or a tokenizer;
  * its own `submit` / `admit` (whole-prompt eager prefill) and then `decode_step()`
    (model/inference_paged.py:181-194), which copies the step's ids and positions to the
    device, replays its compiled decode graph and reads the argmax tokens back.

`value` is timed with CUDA events around K calls of decode_step(); `e2e` is the wall
clock around K more calls (each call already holds the host-to-device copies and the
read-back of the tokens).

Two settings are not the reference's defaults, both through its own switches:

  * PAGED_PARTITION=128.  Its "auto" rule (model/kernels/__init__.py:36-41) takes one pass
    over the whole row from 64 (row, KV head) blocks on, and the one-pass kernel keeps
    group x row-length floats in shared memory and refuses more than 47 KB
    (model/kernels/csrc/paged_attention.cu:301-315): 8,192-token rows at batch 8 are
    refused.  128 is the split size its auto rule uses whenever it splits.
  * COMPILE.  The measurement runs in a child process.  If the child dies with
    torch.compile on (the reference's default), the parent records how, and runs it once
    more with the reference's COMPILE=0; the printed line says which one it is.
"""

import json
import os
import subprocess
import sys
import time
from pathlib import Path
from types import SimpleNamespace

HERE = Path(__file__).resolve().parent
REF_ROOT = HERE / "_ref"


def unavailable(why):
    print(json.dumps({"impl": "reference", "unavailable": " ".join(str(why).split())[:400]}))
    return 0


class PromptTable:
    """Stands where the tokenizer stands: a prompt is a key into a table of token ids.

    Engine.submit calls apply_chat_template, then the tokenizer itself, and record()
    looks at all_special_ids (model/inference_paged.py:139-143, 204); nothing else."""

    all_special_ids = []

    def __init__(self):
        self.table = {}

    def add(self, key, ids):
        self.table[key] = ids

    def apply_chat_template(self, messages, **_):
        return messages[0]["content"]

    def __call__(self, text, return_tensors="pt"):
        return SimpleNamespace(input_ids=self.table[text])

    def decode(self, ids):
        return " ".join(str(i) for i in ids)


def run(args, argv):
    """Parent: runs the measurement in a child process (`bench.py --impl reference` with
    SOCRATES_REFERENCE_CHILD set), first as the reference ships (COMPILE=1), then, if that child
    dies, with the reference's own COMPILE=0.  Prints the child's line, or why there is none."""
    if not (REF_ROOT / "model" / "inference_paged.py").exists():
        return unavailable("baseline/_ref holds no copy of the reference (baseline/install_reference.py "
                           "makes it where the reference's source tree is present)")
    import torch
    if not torch.cuda.is_available():
        return unavailable("no CUDA device")
    failures = []
    for compile_flag in ("1", "0"):
        env = dict(os.environ, SOCRATES_REFERENCE_CHILD="1", COMPILE=compile_flag, DEVICE="cuda",
                   HF_HUB_OFFLINE="1", PYTHONFAULTHANDLER="1")
        env.setdefault("PAGED_PARTITION", "128")
        proc = subprocess.run([sys.executable, *argv], env=env, capture_output=True, text=True)
        lines = [l for l in proc.stdout.splitlines() if l.startswith("{")]
        if proc.returncode == 0 and lines:
            line = json.loads(lines[-1])
            if failures:
                line.setdefault("notes", {})["earlier_attempts"] = failures
            print(json.dumps(line))
            return 0
        tail = " | ".join(proc.stderr.strip().splitlines()[-6:])
        failures.append(f"COMPILE={compile_flag}: exit code {proc.returncode}: {tail}"[:600])
        sys.stderr.write(proc.stderr[-4000:])
    return unavailable("the reference engine did not finish the workload: " + " || ".join(failures))


def measure(args, cfg_dict, shape_name, layers_full, ClockSampler, peaks, arithmetic):
    """Child: builds the reference's engine and times it (see the module docstring)."""
    os.environ.setdefault("HF_HUB_OFFLINE", "1")
    os.environ["DEVICE"] = "cuda"
    sys.path.insert(0, str(REF_ROOT))
    import torch

    torch.cuda.set_device(0)
    notes = {"paged_partition": os.environ.get("PAGED_PARTITION", "auto")}
    import glob
    built = glob.glob(str(REF_ROOT / "model" / "kernels" / "_C*.so"))
    if not built:
        # The reference's own switch for running without its extension.
        os.environ["ATTN_IMPL"] = "ref"
        notes["attn_impl"] = "ref (the reference's _C extension is not built under baseline/_ref)"
    try:
        from model.inference_paged import Engine
        from model.qwen.qwen_kv_paged import Qwen3Paged
    except Exception as e:                                   # noqa: BLE001
        return unavailable(f"import of the reference failed: {type(e).__name__}: {e}")

    K, W, B, ctx = args.steps, max(args.warmup, 3), args.batch, args.context
    max_len, page = 8192, 16
    cfg = {k: cfg_dict[k] for k in ("hidden_size", "intermediate_size", "num_hidden_layers",
                                    "num_attention_heads", "num_key_value_heads", "head_dim",
                                    "vocab_size", "rms_norm_eps", "rope_theta")}
    V = cfg["vocab_size"]
    gen = torch.Generator().manual_seed(0)

    with torch.device("meta"):
        model = Qwen3Paged(cfg)
    model = model.to(torch.bfloat16).to_empty(device="cuda")
    dgen = torch.Generator(device="cuda").manual_seed(0)
    with torch.no_grad():
        for p in model.parameters():
            if p.dim() > 1:
                p.normal_(0.0, 0.02, generator=dgen)
            else:
                p.copy_(1.0 + 0.1 * torch.randn(p.shape, device="cuda", generator=dgen))
    model = model.eval()

    max_new = min(max_len - ctx, 3 * (K + W) + 64)
    tok = PromptTable()

    def make(compile_flag):
        return Engine(model=model, tok=tok, device="cuda", compile=compile_flag, max_batch=B,
                      max_len=max_len, max_new_tokens=max_new, block_size=page)

    from model.inference_cont import COMPILE
    t_build = time.perf_counter()
    engine = make(COMPILE)
    notes["compile"] = bool(COMPILE)
    notes["startup_s"] = round(time.perf_counter() - t_build, 1)

    decode_bytes, prefill_flops = arithmetic(cfg_dict, cfg["num_hidden_layers"])
    pk = peaks()

    # Prefill through the engine's own admission: one whole prompt per request, eager.
    for i in range(B):
        tok.add(f"p{i}", torch.randint(1, V, (1, ctx), generator=gen))
    reqs, prefill_times = [], []
    for i in range(B):
        reqs.append(engine.submit(f"p{i}"))
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        engine.admit()                       # the queue holds this one request: its prefill
        torch.cuda.synchronize()
        prefill_times.append((time.perf_counter() - t0) * 1e3)
    prefill_ms = sorted(prefill_times)[len(prefill_times) // 2]
    assert engine.n_active == B

    sampler = ClockSampler()
    sampler.start()
    time.sleep(0.3)
    for _ in range(W):
        engine.decode_step()
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    start.record()
    for _ in range(K):
        engine.decode_step()
    end.record()
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    ms = start.elapsed_time(end) / K
    clocks = sampler.summary(t0, t1)

    t0 = time.perf_counter()
    for _ in range(K):
        engine.decode_step()
    torch.cuda.synchronize()
    e2e_dt = time.perf_counter() - t0
    assert all(not r.done for r in reqs), "a request finished inside the timed region"

    # batch 1 with the same engine: the other rows are cancelled and retired
    points = {}
    if not args.skip_points:
        for r in reqs[1:]:
            r.cancelled = True
        engine.sweep()
        for _ in range(W):
            engine.decode_step()
        torch.cuda.synchronize()
        s1, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        n1 = max(8, K // 2)
        s1.record()
        for _ in range(n1):
            engine.decode_step()
        e1.record()
        torch.cuda.synchronize()
        points["decode_b1"] = round(1000.0 * n1 / s1.elapsed_time(e1), 1)
    sampler.stop()

    value = B * 1000.0 / ms
    achieved = decode_bytes(B, ctx) / (ms * 1e-3) / 1e9
    T = ctx
    line = {
        "metric": f"decode tokens/s ({shape_name} shape, batch {B}, {ctx}-token contexts)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), token ids uniform over the vocabulary",
        "impl": "reference", "same_config": True,
        "config": {"model": f"{shape_name} shape", "layers": cfg["num_hidden_layers"],
                   "layers_full": layers_full, "hidden": cfg["hidden_size"],
                   "heads": cfg["num_attention_heads"], "kv_heads": cfg["num_key_value_heads"],
                   "head_dim": cfg["head_dim"], "intermediate": cfg["intermediate_size"], "vocab": V,
                   "tied_head": True, "global_batch": B, "seq_len": ctx, "max_len": max_len,
                   "page_size": page, "parallelism": "single GPU",
                   "torch_compile": notes["compile"], "attn_impl": os.environ.get("ATTN_IMPL", "auto"),
                   "paged_partition": notes["paged_partition"],
                   "l2": "inputs larger than L2 (weights 8 GB per step)", "peaks": pk["source"]},
        "clocks": clocks,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "prefill": {"value": round(T * 1000.0 / prefill_ms, 1), "tokens": T, "ms": round(prefill_ms, 3),
                    "frac": round(prefill_flops(T) / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4),
                    "how": f"median of {B} whole-prompt eager prefills in Engine.admit(), wall clock"},
        "e2e": {"value": round(B * K / e2e_dt, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": 2 * B * 8, "d2h_bytes_per_step": B * 8},
        "notes": notes,
    }
    if points:
        line["points"] = points
    print(json.dumps(line))
    return 0
