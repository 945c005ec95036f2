"""The Python entry point: a model folder in, generated tokens out.

    engine = Engine("model_folder")            # config.json + model.safetensors
    req = engine.submit([5, 17, 3])            # token ids, or text with a tokenizer
    engine.run()
    req.output                                 # generated token ids

Shape and argument names follow the reference's Engine (model/inference_paged.py:54-108:
model, tok, device, dtype, compile, max_batch, max_len, max_new_tokens, block_size,
num_blocks; submit / run / req.output, :132-148, 231-251).  `model` is a folder here,
`compile` switches the CUDA graphs of the decode step, and `token_budget` (new) bounds
the tokens of one step.
"""

from __future__ import annotations

import time
from pathlib import Path
from typing import List, Optional, Sequence, Union

import torch

from ..cache import CacheManager
from ..config import EngineConfig, load_config
from ..kernels import require_kernels
from ..sampling import SamplingParams
from ..weights import load_weights, random_tensors_on_device
from .model import Model
from .runner import ModelRunner, SamplingArgs, StepEntry
from .tokenizer import encode_prompt
from .scheduler import PlannedEntry, QueueFull, Request, Scheduler, StepPlan, TooLong

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32,
           "fp32": torch.float32, torch.bfloat16: torch.bfloat16, torch.float32: torch.float32}


def resolve_dtype(dtype) -> torch.dtype:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype must be bfloat16 or float32, not {dtype!r}") from None


def build_model(model_dir, dtype: torch.dtype, device):
    """(configuration, Model with its weights bound) of a model folder."""
    config = load_config(model_dir)
    model = Model(config.plan())
    tensors = load_weights(model_dir, model.parameters(), dtype, device, model.duplicates())
    model.bind(tensors, dtype)
    return config, model


def build_random_model(config, seed: int, dtype: torch.dtype, device):
    """(configuration, Model) with random weights drawn on the device (no folder)."""
    model = Model(config.plan())
    model.bind(random_tensors_on_device(model.parameters(), seed, dtype, device), dtype)
    return config, model


class Engine:
    def __init__(self, model, tok=None, device: str = "cuda:0", dtype="bfloat16",
                 compile: bool = True, max_batch: int = 64, max_len: int = 8192,
                 max_new_tokens: int = 1024, block_size: int = 16, num_blocks: Optional[int] = None,
                 token_budget: int = 2048, max_queue: Optional[int] = None, warmup: bool = False,
                 run_ahead: bool = True, kv_memory_fraction: float = 0.9):
        if not torch.cuda.is_available():
            raise RuntimeError("socrates_b200.Engine needs a CUDA device; there is no CPU path")
        require_kernels()                      # fail at start-up, not on the first step
        self.config = EngineConfig(max_batch=max_batch, max_len=max_len, max_new_tokens=max_new_tokens,
                                   block_size=block_size, num_blocks=num_blocks,
                                   token_budget=max(token_budget, max_batch), max_queue=max_queue,
                                   dtype="float32" if resolve_dtype(dtype) == torch.float32 else "bfloat16",
                                   compile=compile, kv_memory_fraction=kv_memory_fraction)
        self.config.validate()
        self.device = torch.device(device)
        self.dtype = resolve_dtype(dtype)
        torch.cuda.set_device(self.device)
        if isinstance(model, (str, Path)):
            self.model_config, self.model = build_model(model, self.dtype, self.device)
        else:
            self.model_config, self.model = model          # (configuration, Model with weights bound)
        self.tok = tok
        self.max_batch, self.max_len, self.max_new_tokens = max_batch, max_len, max_new_tokens

        # Pages: as many as num_blocks says, else what the memory left after the weights pays
        # for (the step's scratch is small beside it and comes out of the fraction kept back).
        needs = self.model.cache_needs()
        free_bytes, _ = torch.cuda.mem_get_info(self.device)
        self.num_blocks = self.config.pages_from_memory(
            free_bytes, CacheManager.bytes_per_page(needs, block_size, self.dtype))
        if num_blocks is None and self.num_blocks < self.config.pool_blocks:
            print(f"page pool: {self.num_blocks} pages of {block_size} slots per cache group "
                  f"({self.config.pool_blocks} would hold every row at full length); "
                  f"requests are preempted when pages run out", flush=True)
        self.cache = CacheManager(needs, max_rows=max_batch, max_len=max_len,
                                  page_size=block_size, num_pages=self.num_blocks,
                                  dtype=self.dtype, device=self.device)
        self.runner = ModelRunner(self.model, self.cache, self.dtype, self.device,
                                  max_tokens=self.config.token_budget, max_seqs=max_batch,
                                  use_graphs=compile, max_wanted=max_batch)
        stop = set(getattr(self.model_config, "eos_token_ids", ()) or ())
        if tok is not None:
            stop |= set(getattr(tok, "all_special_ids", ()) or ())
        self.scheduler = Scheduler(self.cache, max_batch, max_len, self.config.token_budget,
                                   self.config.queue_limit, stop)
        self.steps = 0
        # run_ahead: while the host waits for a decode step's tokens, the step after it is already
        # on the GPU (see step()); results are the same with and without
        self.run_ahead = run_ahead
        self._ahead = None          # (plan, read handle, sampling args) of a step launched early
        self._planned = None        # a plan the scheduler made that is not launched yet
        self.ahead_launched = self.ahead_discarded = 0
        if warmup:
            self.warmup()

    def warmup(self) -> None:
        """Record one decode graph per batch width now instead of at the first step of each
        width (the reference warms all its widths in its constructor,
        model/inference_paged.py:110-130)."""
        t0 = time.perf_counter()
        n = self.runner.warmup(self.max_batch)
        if n:
            print(f"paged decode graphs warm for 1..{self.max_batch} rows in {time.perf_counter() - t0:.1f}s",
                  flush=True)

    # ------------------------------------------------------------------ requests
    def submit(self, prompt: Union[str, Sequence[int]], max_new_tokens: Optional[int] = None,
               temperature: float = 0.0, seed: int = 0, stream: bool = False) -> Request:
        """Queue a prompt (token ids, or text if the engine has a tokenizer).
        Raises QueueFull or TooLong as the reference does (model/inference_paged.py:132-148).
        `stream`: the request gets a thread-safe queue `req.stream` that receives each token as
        it is produced and None at the end (the reference's `stream` flag, :132-138)."""
        text = None
        if isinstance(prompt, str):
            if self.tok is None:
                raise ValueError("a text prompt needs a tokenizer (Engine(..., tok=...)); pass token ids instead")
            text = prompt
            ids = encode_prompt(self.tok, prompt)
        else:
            ids = [int(i) for i in prompt]
        vocab = self.model.plan.vocab_size
        for t in ids:
            if not 0 <= t < vocab:
                raise ValueError(f"token id {t} is outside the vocabulary of {vocab}")
        req = Request(ids=ids, max_new_tokens=max_new_tokens or self.max_new_tokens,
                      sampling=SamplingParams(float(temperature), int(seed)), prompt=text)
        if stream:
            import queue
            req.stream = queue.Queue()
        return self.scheduler.submit(req)

    # ------------------------------------------------------------------ stepping
    def _launch(self, plan):
        """Launch the step of `plan`; returns the handle of its read-back (None: nothing sampled)."""
        entries = [StepEntry(e.row, [e.request.token_at(i) for i in range(e.start, e.start + e.count)],
                             e.start, [e.count - 1] if e.samples else [])
                   for e in plan.entries]
        args = [SamplingArgs(t, s, c) for (t, s, c) in self.scheduler.sampling_args(plan)]
        result = self.runner.step(entries, args)
        return self.runner.begin_read(len(args)) if result.tokens is not None else None

    def _foresee(self, plan):
        """The plan of the step after `plan`, if it can be known before `plan`'s tokens are:
        every live request decodes in `plan`, none can end by length, nobody waits to be
        admitted, and each row has (or gets) the page for one more token.  None otherwise."""
        sch = self.scheduler
        if self.cache.states:
            # A step launched early may be dropped and run again.  That is harmless for paged
            # keys (the dropped step wrote past the rows' lengths) but not for a mixer's
            # per-request state, which the dropped step has already advanced by one token.
            return None
        if sch.pending or plan.preempted or len(plan.entries) != sch.n_active:
            return None
        entries = []
        for e in plan.entries:
            req = e.request
            if e.count != 1 or not e.samples or len(req.output) + 1 >= req.max_new_tokens:
                return None
            if e.start + 2 > self.max_len or not self.cache.reserve(e.row, e.start + 2):
                return None
            entries.append((req, e.row, e.start + 1))
        return entries

    def step(self) -> bool:
        """Plan and run one step; False when there was nothing to run.

        While the host waits for the tokens of a pure decode step, the step after it is launched
        already (its tokens stay on the device: the embedding reads what the sampler wrote).
        When the tokens are in, the scheduler records them and plans; if its plan is the one
        that was launched, the next call only has to collect it, else the early step is dropped
        (it wrote nothing that counts: keys past the rows' lengths, tokens nobody reads)."""
        plan = handle = None
        if self._ahead is not None:
            plan, handle, _ = self._ahead
            self._ahead = None
            if any(e.request.row != e.row for e in plan.entries):
                plan = handle = None        # a request left in between (cancelled and swept): drop the early step
                self.ahead_discarded += 1
        if plan is None:
            plan = self._planned if self._planned is not None else self.scheduler.plan()
            self._planned = None
            if plan is None:
                return False
            handle = self._launch(plan)
        guess = self._foresee(plan) if (self.run_ahead and handle is not None) else None
        early = None
        if guess is not None:
            early_plan = StepPlan([PlannedEntry(req, row, start, 1, True) for (req, row, start) in guess], [])
            # sampling counters are those the scheduler will name once this step's tokens are recorded
            args = [SamplingArgs(req.sampling.temperature, req.sampling.seed, len(req.output) + 1)
                    for (req, _, _) in guess]
            entries = [StepEntry(row, [-1 - j], start, [0]) for j, (_, row, start) in enumerate(guess)]
            self.runner.step(entries, args, ahead=1)
            early = (early_plan, self.runner.begin_read(len(args)), args)
            self.ahead_launched += 1
        # the step's one read-back: sampled tokens and the kernels' status word together
        tokens = self.runner.finish_read(handle) if handle is not None else []
        if handle is None:
            self.runner.check_status()
        self.scheduler.complete(plan, tokens)
        self.steps += 1
        if early is not None:
            nxt = self.scheduler.plan()
            if nxt is not None and self._same_step(nxt, early[0], early[2]):
                self._ahead = (nxt, early[1], early[2])
            else:
                self.ahead_discarded += 1
                self._planned = nxt          # planned (pages reserved): launched by the next call
        return True

    def _same_step(self, plan, early_plan, early_args) -> bool:
        if plan.preempted or len(plan.entries) != len(early_plan.entries):
            return False
        for a, b in zip(plan.entries, early_plan.entries):
            if a.request is not b.request or a.row != b.row or a.start != b.start or a.count != 1 or not a.samples:
                return False
        now = self.scheduler.sampling_args(plan)
        return all((x.temperature, x.seed, x.counter) == tuple(y) for x, y in zip(early_args, now))

    def run(self) -> None:
        """Until every submitted request is finished (model/inference_paged.py:231-237)."""
        while self.scheduler.has_work():
            if not self.step():
                if self.scheduler.has_work():
                    raise RuntimeError("the scheduler has requests but could plan no step")

    def generate(self, prompts: Sequence[Union[str, Sequence[int]]], max_new_tokens: Optional[int] = None,
                 temperature: float = 0.0, seed: int = 0) -> List[List[int]]:
        """Submit, run, and return the generated ids of each prompt, in order.
        Request i samples with seed + i."""
        reqs = [self.submit(p, max_new_tokens, temperature, seed + i) for i, p in enumerate(prompts)]
        self.run()
        return [r.output for r in reqs]


__all__ = ["Engine", "Request", "QueueFull", "TooLong", "build_model", "build_random_model",
           "resolve_dtype"]
