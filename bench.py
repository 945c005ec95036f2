#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference] [--shape 4b|8b|32b]

Default run: the layer sizes of the Qwen3-4B shape (36 layers, hidden 2560, 32 query
heads over 8 KV heads, head_dim 128, intermediate 9728, vocabulary 151936, tied head),
random weights, bfloat16, batch 8, 2,048-token contexts in 8,192-token rows, 16-slot
pages.  One "step" is one decode step of the whole batch.  `--shape 32b` runs the same
points on the Qwen3-32B shape at 4,096-token contexts; `--shape 8b` runs continuous
batching through the scheduler (64 requests, Poisson arrivals) on the Qwen3-8B shape.
`--impl reference` runs the unmodified reference engine on the same workload
(baseline/reference_arm.py).  It prints ONE JSON line:

  value      decoded tokens a second, K steps timed on the device with CUDA events;
  e2e        the same through the Python entry point (Engine.step), host tokens in and out;
  prefill    one 2,048-token prompt in one step: tokens a second and fraction of the
             bfloat16 tensor peak;
  roofline   bytes a decode step has to read (every weight once, the live KV) / its time,
             against the measured copy bandwidth;
  points     decode tokens a second at batch 1 and 64.

Peaks come from MEASURED_PEAKS.json beside this file when present, else from the
fallback figures 6.65 TB/s and 1.59 PFLOP/s.
"""

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

def _qwen3(hidden, inter, layers, heads, tied):
    return {"architectures": ["Qwen3ForCausalLM"], "vocab_size": 151936, "hidden_size": hidden,
            "intermediate_size": inter, "num_hidden_layers": layers, "num_attention_heads": heads,
            "num_key_value_heads": 8, "head_dim": 128, "rms_norm_eps": 1e-6, "rope_theta": 1e6,
            "tie_word_embeddings": tied, "max_position_embeddings": 40960}


# The three real shapes of the benchmark: (name, config.json keys, context of the decode points)
SHAPES = {
    "4b": ("Qwen3-4B", _qwen3(2560, 9728, 36, 32, True), 2048),
    "8b": ("Qwen3-8B", _qwen3(4096, 12288, 36, 32, False), 2048),
    "32b": ("Qwen3-32B", _qwen3(5120, 25600, 64, 64, False), 4096),
}


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    out = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}
    if p.exists():
        try:
            d = json.loads(p.read_text())
            out["hbm_gbs"] = float(d.get("hbm_gbs", out["hbm_gbs"]))
            out["bf16_tflops"] = float(d.get("bf16_tflops", out["bf16_tflops"]))
            if "bf16_tflops_sustained" in d:
                out["bf16_tflops_sustained"] = float(d["bf16_tflops_sustained"])
            out["source"] = "measured"
        except Exception:
            pass
    return out


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index=0):
        self.proc, self.lines, self.index = None, [], index

    def start(self):
        if os.environ.get("BENCH_NO_CLOCKS") == "1":      # to see what the sampling itself costs
            return
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()

    def summary(self, t0, t1):
        mhz, mx, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for t, line in self.lines:
            if not (t0 <= t <= t1 + 0.2):
                continue
            f = [x.strip() for x in line.split(",")]
            try:
                mhz.append(int(float(f[0])))
                mx = max(mx, int(float(f[1])))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, f[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


def arithmetic(cfg, layers):
    """Bytes a decode step reads and flops a prefill does (analysis/arithmetic.py:84-143
    of the reference states the same formulas)."""
    d, F, V = cfg["hidden_size"], cfg["intermediate_size"], cfg["vocab_size"]
    Hq, Hkv, D = cfg["num_attention_heads"], cfg["num_key_value_heads"], cfg["head_dim"]
    linear = layers * ((Hq + 2 * Hkv) * D * d + Hq * D * d + 3 * d * F)
    kv_per_token = layers * 2 * Hkv * D * 2

    def decode_bytes(batch, ctx):
        return 2 * (linear + V * d) + batch * ctx * kv_per_token

    def prefill_flops(T):
        return 2 * T * linear + layers * 2 * Hq * D * T * T + 2 * d * V

    return decode_bytes, prefill_flops


def build_engine(args, cfg_dict, rows, num_blocks, max_new, token_budget=2048):
    import torch

    from socrates_b200 import Engine
    from socrates_b200.config import config_from_dict
    from socrates_b200.engine.engine import build_random_model

    torch.cuda.set_device(0)
    config = config_from_dict(cfg_dict)
    model = build_random_model(config, 0, torch.bfloat16, torch.device("cuda:0"))
    return Engine(model, device="cuda:0", dtype="bfloat16", compile=True, max_batch=rows, max_len=8192,
                  max_new_tokens=max_new, block_size=16, num_blocks=num_blocks,
                  token_budget=max(token_budget, rows))


def shape_config(name, cfg, layers):
    return {"model": f"{name} shape", "layers": layers, "layers_full": cfg["num_hidden_layers"],
            "hidden": cfg["hidden_size"], "heads": cfg["num_attention_heads"],
            "kv_heads": cfg["num_key_value_heads"], "head_dim": cfg["head_dim"],
            "intermediate": cfg["intermediate_size"], "vocab": cfg["vocab_size"],
            "tied_head": cfg["tie_word_embeddings"]}


def run_decode(args, name, cfg_full):
    """Decode at batch 1/8/64 and one 2,048-token prefill, device-timed; the batch-8 loop again
    through Engine.step() for the end-to-end figure."""
    import torch

    from socrates_b200.engine.runner import SamplingArgs, StepEntry

    dev = torch.device("cuda:0")
    layers = args.layers or cfg_full["num_hidden_layers"]
    cfg_dict = dict(cfg_full, num_hidden_layers=layers)
    pk = peaks()
    decode_bytes, prefill_flops = arithmetic(cfg_dict, layers)
    V = cfg_dict["vocab_size"]
    gen = torch.Generator().manual_seed(0)
    K, W, B, ctx = args.steps, args.warmup, args.batch, args.context
    max_len, page = 8192, 16

    rows_needed = max(B, 1 if args.skip_points else 64)
    pages_per_row = -(-(ctx + 2 * (K + W) + rows_needed + 96) // page)
    engine = build_engine(args, cfg_dict, rows_needed, rows_needed * pages_per_row + 8,
                          K + W + rows_needed + 32)
    cache, runner = engine.cache, engine.runner
    for g in cache.groups:                      # live KV: any finite values, the bytes are what is timed
        g.k.normal_(0, 1, generator=None)
        g.v.normal_(0, 1, generator=None)

    def decode_run(batch, steps, warmup):
        """`steps` decode steps of `batch` rows at `ctx` tokens; returns (ms per step, launches, span)."""
        for r in range(batch):
            cache.assign(r)
            assert cache.reserve(r, ctx + steps + warmup + 1)
            cache.commit(r, ctx)
        ids = torch.randint(0, V, (steps + warmup, batch), generator=gen).tolist()
        sampling = [SamplingArgs() for _ in range(batch)]

        def one(i):
            entries = [StepEntry(r, [ids[i][r]], cache.lengths[r], [0]) for r in range(batch)]
            runner.step(entries, sampling)
            for r in range(batch):
                cache.commit(r, cache.lengths[r] + 1)

        for i in range(warmup):
            one(i)
        torch.cuda.synchronize()
        before = runner.kernel_launches
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0 = time.perf_counter()
        start.record()
        for i in range(warmup, warmup + steps):
            one(i)
        end.record()
        torch.cuda.synchronize()
        t1 = time.perf_counter()
        ms = start.elapsed_time(end) / steps
        launches = runner.kernel_launches - before
        for r in range(batch):
            cache.release(r)
        return ms, launches, (t0, t1)

    sampler = ClockSampler()
    sampler.start()
    time.sleep(0.3)
    ms, launches, span = decode_run(B, K, W)
    clocks = sampler.summary(*span)
    value = B * 1000.0 / ms
    achieved = decode_bytes(B, ctx) / (ms * 1e-3) / 1e9

    points = {}
    if not args.skip_points:
        for b in (1, 64):
            pms, _, _ = decode_run(b, max(8, K // 2), W)
            points[f"decode_b{b}"] = round(b * 1000.0 / pms, 1)
            points[f"decode_b{b}_hbm_frac"] = round(decode_bytes(b, ctx) / (pms * 1e-3) / 1e9 / pk["hbm_gbs"], 4)

    prefill = None
    if not args.skip_prefill:
        T = 2048
        prompt = torch.randint(0, V, (T,), generator=gen).tolist()
        times = []
        for i in range(W + 3):
            cache.assign(0)
            assert cache.reserve(0, T)
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.synchronize()
            s.record()
            runner.step([StepEntry(0, prompt, 0, [T - 1])], [SamplingArgs()])
            e.record()
            torch.cuda.synchronize()
            cache.release(0)
            if i >= W:
                times.append(s.elapsed_time(e))
        pms = sorted(times)[len(times) // 2]
        prefill = {"value": round(T * 1000.0 / pms, 1), "tokens": T, "ms": round(pms, 3),
                   "frac": round(prefill_flops(T) / (pms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}
        if "bf16_tflops_sustained" in pk:      # the rate cuBLAS holds for seconds under the power cap
            prefill["frac_of_sustained"] = round(prefill_flops(T) / (pms * 1e-3) / (pk["bf16_tflops_sustained"] * 1e12), 4)

    e2e = None
    if not args.skip_e2e:
        # Through the entry point: B requests with ctx-token prompts are prefilled by the
        # scheduler, then K decode steps are timed; each step copies its inputs from pinned
        # host memory and reads its sampled tokens back to the host.
        # (prompts are prefilled one a step, so the first request is B tokens ahead of the last:
        # room for that, so that nobody finishes inside the timed region)
        prompts = torch.randint(1, V, (B, ctx), generator=gen).tolist()
        reqs = [engine.submit(p, max_new_tokens=K + W + B + 16) for p in prompts]
        while any(r.cached < ctx for r in reqs):
            engine.step()
        for _ in range(W):
            engine.step()
        torch.cuda.synchronize()
        done_before = sum(len(r.output) for r in reqs)
        t0 = time.perf_counter()
        for _ in range(K):
            engine.step()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        made = sum(len(r.output) for r in reqs) - done_before
        assert made == B * K, "a request finished inside the timed region"
        for r in reqs:
            r.cancelled = True
        engine.scheduler.sweep()
        e2e = {"value": round(made / dt, 1), "unit": "tokens/s",
               "h2d_bytes_per_step": runner.layout.total * 4, "d2h_bytes_per_step": (B + 1) * 4}
    sampler.stop()

    line = {
        "metric": f"decode tokens/s ({name} shape, batch {B}, {ctx}-token contexts)",
        "value": round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": K, "warmup": W,
        "ms_per_step": round(ms, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic: random weights N(0,0.02), token ids uniform over the vocabulary",
        "config": dict(shape_config(name, cfg_full, layers), global_batch=B, seq_len=ctx, max_len=max_len,
                       page_size=page, parallelism="single GPU", cuda_graph=True,
                       l2="inputs larger than L2 (the weights of a step)", peaks=pk["source"]),
        "clocks": clocks, "gpu_launches": launches, "impl": "ours",
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
    }
    if prefill is not None:
        line["prefill"] = prefill
    if e2e is not None:
        line["e2e"] = e2e
    if points:
        line["points"] = points
    print(json.dumps(line))
    return 0


def run_serve(args, name, cfg_full):
    """Continuous batching through Engine: `--requests` requests with prompt lengths uniform in
    [128, 4096] arrive as a Poisson process of `--rate` a second (seeded), each generates
    `--max-new` tokens; the page pool is sized from free memory.  The load has the shape of the
    reference's own load generator (backend/server.py:443-447: seeded exponential gaps), with
    token ids in place of its prompt texts.  A "step" here is one Engine.step()."""
    import random

    import torch

    layers = args.layers or cfg_full["num_hidden_layers"]
    cfg_dict = dict(cfg_full, num_hidden_layers=layers)
    V = cfg_dict["vocab_size"]
    n, max_new = args.requests, args.max_new
    engine = build_engine(args, cfg_dict, 64, None, max_new)
    engine.warmup()
    rng = random.Random(0)
    gen = torch.Generator().manual_seed(0)
    lengths = [rng.randint(128, 4096) for _ in range(n)]
    arrivals, t = [], 0.0
    for _ in range(n):
        t += rng.expovariate(args.rate)
        arrivals.append(t)
    prompts = [torch.randint(1, V, (L,), generator=gen).tolist() for L in lengths]

    sampler = ClockSampler()
    sampler.start()
    time.sleep(0.3)
    sch, runner = engine.scheduler, engine.runner
    reqs, step_tokens = [], []
    before = runner.kernel_launches
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    i = 0
    while i < n or sch.has_work():
        now = time.perf_counter() - t0
        while i < n and arrivals[i] <= now:
            r = engine.submit(prompts[i], max_new_tokens=max_new)
            r.submitted = t0 + arrivals[i]          # the moment it was due, not the moment the loop saw it
            reqs.append(r)
            i += 1
        done = sch.prompt_tokens + sch.output_tokens
        if engine.step():
            step_tokens.append(sch.prompt_tokens + sch.output_tokens - done)
        elif i < n:
            time.sleep(max(0.0, min(0.002, arrivals[i] - (time.perf_counter() - t0))))
    torch.cuda.synchronize()
    t1 = time.perf_counter()
    sampler.stop()
    wall = t1 - t0
    out_tokens = sum(len(r.output) for r in reqs)
    assert all(r.done for r in reqs) and out_tokens == n * max_new

    def pct(xs, q):
        xs = sorted(xs)
        return xs[min(len(xs) - 1, int(q * len(xs)))]

    ttft = [r.first_token - r.submitted for r in reqs]
    itl = [(r.finished - r.first_token) / max(1, len(r.output) - 1) for r in reqs]
    steps = len(step_tokens)
    pk = peaks()
    line = {
        "metric": f"continuous batching output tokens/s ({name} shape, {n} requests, Poisson {args.rate}/s)",
        "value": round(out_tokens / wall, 1), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": 0,
        "ms_per_step": round(wall * 1e3 / steps, 4), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: random weights N(0,0.02), token ids uniform over the vocabulary, seeded arrivals",
        "config": dict(shape_config(name, cfg_full, layers), global_batch=64, seq_len="128..4096 prompt",
                       max_len=8192, page_size=16, parallelism="single GPU",
                       requests=n, rate_per_s=args.rate, max_new=max_new,
                       pool_pages=engine.cache.groups[0].allocator.num_pages, peaks=pk["source"]),
        "clocks": sampler.summary(t0, t1), "gpu_launches": runner.kernel_launches - before, "impl": "ours",
        "e2e": {"value": round(out_tokens / wall, 1), "unit": "tokens/s",
                "h2d_bytes_per_step": runner.layout.total * 4, "d2h_bytes_per_step": 65 * 4},
        "serve": {"wall_s": round(wall, 2), "prompt_tokens": sum(lengths), "output_tokens": out_tokens,
                  "total_tokens_per_s": round((sum(lengths) + out_tokens) / wall, 1),
                  "mean_tokens_per_step": round(sum(step_tokens) / steps, 1),
                  "preemptions": sch.preemptions, "ahead_launched": engine.ahead_launched,
                  "ahead_discarded": engine.ahead_discarded,
                  "ttft_s": {"p50": round(pct(ttft, 0.5), 4), "p99": round(pct(ttft, 0.99), 4)},
                  "itl_ms": {"p50": round(pct(itl, 0.5) * 1e3, 3), "p99": round(pct(itl, 0.99) * 1e3, 3)}},
    }
    print(json.dumps(line))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=("ours", "reference"))
    ap.add_argument("--shape", default="4b", choices=sorted(SHAPES),
                    help="4b (the headline), 32b: decode and prefill points; 8b: continuous batching")
    ap.add_argument("--workload", default=None, choices=("decode", "serve"),
                    help="default: serve for 8b, decode for the others")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=None)
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers than the configuration has (both numbers are reported)")
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--rate", type=float, default=4.0)
    ap.add_argument("--max-new", type=int, default=512)
    ap.add_argument("--skip-points", action="store_true")
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-prefill", action="store_true")
    args = ap.parse_args()

    if args.gpus != 1:
        print("bench.py: this engine runs on one GPU; --gpus must be 1")
        return 2
    args.warmup = max(args.warmup, 3)
    name, cfg_full, ctx = SHAPES[args.shape]
    args.context = args.context or ctx
    workload = args.workload or ("serve" if args.shape == "8b" else "decode")

    if args.impl == "reference":
        sys.path.insert(0, str(ROOT / "baseline"))
        import reference_arm
        if os.environ.get("SOCRATES_REFERENCE_CHILD") != "1":
            return reference_arm.run(args, [str(Path(__file__).resolve()), *sys.argv[1:]])
        layers = args.layers or cfg_full["num_hidden_layers"]
        return reference_arm.measure(args, dict(cfg_full, num_hidden_layers=layers), name,
                                     cfg_full["num_hidden_layers"], ClockSampler, peaks, arithmetic)
    if workload == "serve":
        return run_serve(args, name, cfg_full)
    return run_decode(args, name, cfg_full)


if __name__ == "__main__":
    sys.exit(main())
