"""Generation through the Python entry point against the plain implementation."""

import pytest
import torch

import plain_qwen3 as plain
from tiny_configs import CONFIGS, make_folder

pytestmark = pytest.mark.gpu


def engine_for(folder, dtype, **kw):
    from socrates_b200 import Engine
    args = dict(device="cuda:0", dtype=dtype, max_batch=4, max_len=512, max_new_tokens=8, block_size=16,
                token_budget=64)
    args.update(kw)
    return Engine(str(folder), **args)


def prompts_for(name, lengths, seed=3):
    vocab = CONFIGS[name][0]["vocab_size"]
    g = torch.Generator().manual_seed(seed)
    return [torch.randint(1, vocab, (n,), generator=g).tolist() for n in lengths]


def check_teacher_forced(cfg, w, prompt, output, margin, temperature=0.0, seed=0):
    """Every produced token must be the plain implementation's choice given the tokens
    before it, or lose to that choice by less than `margin` (a tie within rounding)."""
    seq = list(prompt) + list(output)
    logits = plain.logits(w, cfg, seq[:-1] if output else seq)
    scale = float(logits.abs().max())
    for i, tok in enumerate(output):
        row = logits[len(prompt) - 1 + i]
        if temperature > 0:
            scores = plain.temperature_scores(row, temperature, seed, i)
            gap = margin * scale / temperature
        else:
            scores, gap = row, margin * scale
        best = int(torch.argmax(scores))
        assert tok == best or float(scores[best] - scores[tok]) <= gap, (
            f"token {i}: engine chose {tok}, plain chose {best}, "
            f"score gap {float(scores[best] - scores[tok]):.3g} > {gap:.3g}")


@pytest.mark.parametrize("dtype,margin", [("float32", 1e-4), ("bfloat16", 2e-2)])
def test_greedy_config_a(tmp_path, dtype, margin):
    """Tiny A: prompts of 5, 11 and 17 tokens, 8 new tokens each, greedy, 16-slot pages."""
    folder = make_folder(tmp_path, "A")
    cfg, w = plain.load_folder(folder)
    ps = prompts_for("A", [5, 11, 17])
    eng = engine_for(folder, dtype)
    outs = eng.generate(ps, max_new_tokens=8)
    assert all(len(o) == 8 for o in outs)
    for p, o in zip(ps, outs):
        check_teacher_forced(cfg, w, p, o, margin)
    if dtype == "float32":
        for p, o in zip(ps, outs):                     # free-running: exactly the plain greedy tokens
            seq = list(p)
            for t in o:
                assert t == plain.greedy(plain.logits(w, cfg, seq)[-1])
                seq.append(t)
    assert eng.cache.free_pages() == [g.allocator.num_pages for g in eng.cache.groups]


@pytest.mark.parametrize("dtype,margin", [("float32", 1e-4), ("bfloat16", 2e-2)])
def test_temperature_config_b_portions_beside_decode(tmp_path, dtype, margin):
    """Tiny B: prompts of 1, 16, 23 and 40 tokens cut into 8-token portions that share
    steps with decoding rows; 6 new tokens at temperature 0.8, seeded."""
    folder = make_folder(tmp_path, "B")
    cfg, w = plain.load_folder(folder)
    ps = prompts_for("B", [1, 16, 23, 40])
    eng = engine_for(folder, dtype, token_budget=8, max_batch=4)
    outs = eng.generate(ps, max_new_tokens=6, temperature=0.8, seed=100)
    assert all(len(o) == 6 for o in outs)
    for i, (p, o) in enumerate(zip(ps, outs)):
        check_teacher_forced(cfg, w, p, o, margin, temperature=0.8, seed=100 + i)
    # Another way of cutting and batching: whole prompts, two rows.  In float32 a portion of a
    # prompt and a whole prompt round alike to far below any score gap, and the tokens are the
    # same.  In bfloat16 prompt portions of other sizes run through other tiles of the
    # tensor-core products and round differently (by design: the logits agree "beyond rounding"),
    # so a draw that two candidates nearly tie for may fall the other way; what must hold is that
    # the other schedule's tokens pass the same check against the plain implementation and that
    # a schedule repeated gives the same tokens.
    again = engine_for(folder, dtype, token_budget=64, max_batch=2)
    outs2 = again.generate(ps, max_new_tokens=6, temperature=0.8, seed=100)
    if dtype == "float32":
        assert outs2 == outs
    else:
        for i, (p, o) in enumerate(zip(ps, outs2)):
            check_teacher_forced(cfg, w, p, o, margin, temperature=0.8, seed=100 + i)
        same = engine_for(folder, dtype, token_budget=8, max_batch=4)
        assert same.generate(ps, max_new_tokens=6, temperature=0.8, seed=100) == outs


def test_long_decoding_float32(tmp_path):
    """200 decode steps (the recorded CUDA graph path) across many page edges and, in
    config B, far past the window."""
    for name in ("A", "B"):
        folder = make_folder(tmp_path / name, name)
        cfg, w = plain.load_folder(folder)
        p = prompts_for(name, [3])[0]
        eng = engine_for(folder, "float32", max_new_tokens=200)
        out = eng.generate([p], max_new_tokens=200)[0]
        assert len(out) == 200
        assert eng.runner.graph_replays >= 190
        check_teacher_forced(cfg, w, p, out, 1e-4)


def test_graphs_and_eager_agree(tmp_path):
    folder = make_folder(tmp_path, "A")
    ps = prompts_for("A", [9, 30, 2])
    a = engine_for(folder, "bfloat16", compile=True).generate(ps, max_new_tokens=40)
    b = engine_for(folder, "bfloat16", compile=False).generate(ps, max_new_tokens=40)
    assert a == b


@pytest.mark.parametrize("temperature", [0.0, 0.7])
def test_running_ahead_changes_nothing(tmp_path, temperature):
    """While the host waits for a decode step's tokens the engine launches the step after it.
    Requests of different lengths (so that early steps are dropped when one ends), one that
    arrives while the others decode, one that is cancelled: the same tokens as without, and
    the bookkeeping holds after every step."""
    folder = make_folder(tmp_path, "B")
    ps = prompts_for("B", [20, 7, 33, 12])
    new = [37, 9, 60, 25]
    outs = {}
    for ahead in (False, True):
        eng = engine_for(folder, "float32", max_batch=4, max_new_tokens=64, run_ahead=ahead)
        reqs = [eng.submit(p, max_new_tokens=n, temperature=temperature, seed=5 + i)
                for i, (p, n) in enumerate(zip(ps[:3], new[:3]))]
        steps = 0
        while eng.scheduler.has_work():
            assert eng.step()
            eng.scheduler.check()
            steps += 1
            if steps == 12:                               # a late arrival beside running decodes
                reqs.append(eng.submit(ps[3], max_new_tokens=new[3], temperature=temperature, seed=8))
            if steps == 30:
                reqs[2].cancelled = True                  # leaves at the next plan
        outs[ahead] = [r.output for r in reqs]
        assert [len(r.output) for r in reqs[:2]] == new[:2] and len(reqs[3].output) == new[3]
        assert eng.cache.free_pages() == [g.allocator.num_pages for g in eng.cache.groups]
        if ahead:
            assert eng.ahead_launched > 20 and 0 < eng.ahead_discarded < eng.ahead_launched
        else:
            assert eng.ahead_launched == 0
    assert outs[True][:2] == outs[False][:2] and outs[True][3] == outs[False][3]
    n = min(len(outs[True][2]), len(outs[False][2]))      # the cancelled one: the same tokens while it ran
    assert n >= 20 and outs[True][2][:n] == outs[False][2][:n]


def test_running_ahead_and_stop_tokens(tmp_path):
    """A stop token ends a request one step after the engine has already launched that request's
    next step: the early step is dropped and nothing of it shows."""
    import json
    from socrates_b200.config import config_from_dict
    from socrates_b200.weights import write_model_folder
    from tiny_configs import TINY_A
    free = engine_for(make_folder(tmp_path / "free", "A"), "float32", max_batch=3, max_new_tokens=40)
    ps = prompts_for("A", [6, 19, 11])
    outs = free.generate(ps, max_new_tokens=40, temperature=0.9, seed=21)
    # a token that some request first produces well into its decoding
    late = [(o.index(t), t) for o in outs for t in set(o) if o.index(t) >= 5]
    assert late, "every token of every output appears within the first five: choose other prompts"
    stop = min(late)[1]
    folder = write_model_folder(config_from_dict(dict(TINY_A, eos_token_id=stop)), 0, tmp_path / "stop")
    assert json.loads((folder / "config.json").read_text())["eos_token_id"] == stop
    got = {}
    for ahead in (False, True):
        eng = engine_for(folder, "float32", max_batch=3, max_new_tokens=40, run_ahead=ahead)
        got[ahead] = eng.generate(ps, max_new_tokens=40, temperature=0.9, seed=21)
        for want, have in zip(outs, got[ahead]):
            cut = want.index(stop) if stop in want else len(want)
            assert have == want[:cut]                    # the stop token itself is not appended
        assert eng.cache.free_pages() == [g.allocator.num_pages for g in eng.cache.groups]
        if ahead:
            assert eng.ahead_discarded >= 1
    assert got[True] == got[False] and any(len(g) < 40 for g in got[True])


def test_few_pages_preemption_keeps_outputs(tmp_path):
    """A pool too small for all requests at once: some are preempted and recomputed, and
    every request still gets the tokens it gets when it runs alone."""
    folder = make_folder(tmp_path, "B")
    ps = prompts_for("B", [40, 25, 33, 8, 50, 12])
    alone = [engine_for(folder, "float32", max_batch=1).generate([p], max_new_tokens=30)[0] for p in ps]
    eng = engine_for(folder, "float32", max_batch=4, num_blocks=9, max_len=96, token_budget=16)
    reqs = [eng.submit(p, max_new_tokens=30) for p in ps]
    while eng.scheduler.has_work():
        assert eng.step()
        eng.scheduler.check()
    assert [r.output for r in reqs] == alone
    assert eng.scheduler.preemptions > 0
    assert eng.cache.free_pages() == [9, 9]


@pytest.mark.parametrize("block_size", [32, 64])
def test_other_page_sizes(tmp_path, block_size):
    """Pages of 32 and 64 slots through the whole engine (float32 and bfloat16), prompts in
    portions beside decoding rows, few pages so that they are used again."""
    folder = make_folder(tmp_path, "B")
    cfg, w = plain.load_folder(folder)
    ps = prompts_for("B", [70, 3, 130, 41, 66])
    for dtype, margin in (("float32", 1e-4), ("bfloat16", 2e-2)):
        eng = engine_for(folder, dtype, block_size=block_size, max_batch=3, max_len=256, token_budget=24,
                         num_blocks=3 * (256 // block_size) // 2, max_new_tokens=40)
        outs = eng.generate(ps, max_new_tokens=40)
        for p, o in zip(ps, outs):
            assert len(o) == 40
            check_teacher_forced(cfg, w, p, o, margin)
        assert eng.cache.free_pages() == [g.allocator.num_pages for g in eng.cache.groups]


@pytest.mark.parametrize("partition", ["0", "16", "128"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_paged_partition_env(tmp_path, monkeypatch, partition, name):
    """PAGED_PARTITION as the reference reads it: 0 = one pass over all keys, n = n keys per
    partition.  Decode steps then run the streaming kernel (bfloat16) or the SIMT kernel with
    that split (float32); 150 decoded tokens cross many partition edges."""
    monkeypatch.setenv("PAGED_PARTITION", partition)
    folder = make_folder(tmp_path, name)
    cfg, w = plain.load_folder(folder)
    ps = prompts_for(name, [3, 40])
    for dtype, margin in (("float32", 1e-4), ("bfloat16", 2e-2)):
        eng = engine_for(folder, dtype, max_new_tokens=150)
        outs = eng.generate(ps, max_new_tokens=150)
        assert eng.runner.graph_replays >= 140
        for p, o in zip(ps, outs):
            check_teacher_forced(cfg, w, p, o, margin)


def decode_logits(eng, prompt, fed, others=()):
    """Prefill `prompt` alone in one step, then feed the tokens `fed` one by one, together with one
    decode token of each row of `others` ([(prompt, tokens)]) in the same steps; returns the
    float32 logits of the first request's decode steps."""
    from socrates_b200.engine.runner import StepEntry
    cache, runner = eng.cache, eng.runner
    rows = [(0, list(prompt), list(fed))] + [(i + 1, list(p), list(t)) for i, (p, t) in enumerate(others)]
    for r, p, _ in rows:
        cache.assign(r)
        assert cache.reserve(r, len(p))
        runner.step([StepEntry(r, p, 0, [])])
        cache.commit(r, len(p))
    got = []
    for i in range(len(fed)):
        entries = []
        for r, p, t in rows:
            assert cache.reserve(r, len(p) + i + 1)
            entries.append(StepEntry(r, [t[i]], len(p) + i, [0]))
        got.append(runner.step(entries).logits[0].clone())
        for r, p, _ in rows:
            cache.commit(r, len(p) + i + 1)
    for r, _, _ in rows:
        cache.release(r)
    return torch.stack(got)


@pytest.mark.parametrize("dtype,partition", [("float32", "auto"), ("bfloat16", "64"), ("bfloat16", "0")])
def test_decoded_logits_do_not_depend_on_the_batch(tmp_path, monkeypatch, dtype, partition):
    """A request decoded alone and the same request decoded beside three others of other
    lengths: the same BITS of logits at every step.  Holds in float32 always (the SIMT kernel's
    split depends on the cache's limits alone) and in bfloat16 with PAGED_PARTITION set (chunks at
    fixed key positions); with "auto" the bfloat16 partition count follows the batch width and
    the logits agree only beyond rounding."""
    monkeypatch.setenv("PAGED_PARTITION", partition)
    folder = make_folder(tmp_path, "B")
    ps = prompts_for("B", [150, 9, 77, 200], seed=5)
    g = torch.Generator().manual_seed(9)
    fed = [torch.randint(1, 384, (40,), generator=g).tolist() for _ in ps]
    eng = engine_for(folder, dtype, max_batch=4, max_len=512, token_budget=256)
    alone = decode_logits(eng, ps[0], fed[0])
    beside = decode_logits(eng, ps[0], fed[0], others=list(zip(ps[1:], fed[1:])))
    assert torch.equal(alone, beside)


def test_page_pressure_at_real_widths():
    """Two layers at the Qwen3-4B widths, 60 requests of 16 to 1,500 tokens submitted at once into 16
    rows and a pool of 260 pages (4,160 tokens): portions beside decode tokens, many preemptions and
    recomputations, greedy and temperature requests mixed.  Every request gets exactly its tokens,
    the bookkeeping holds throughout, every page comes back, and the same run again gives the same
    tokens (nothing depends on timing or on what a reused page held)."""
    import random
    from socrates_b200 import Engine
    from socrates_b200.config import config_from_dict
    from socrates_b200.engine.engine import build_random_model
    cfg = {"architectures": ["Qwen3ForCausalLM"], "vocab_size": 4096, "hidden_size": 2560, "intermediate_size": 9728,
           "num_hidden_layers": 2, "num_attention_heads": 32, "num_key_value_heads": 8, "head_dim": 128,
           "rms_norm_eps": 1e-6, "rope_theta": 1e6, "tie_word_embeddings": True}
    built = build_random_model(config_from_dict(cfg), 0, torch.bfloat16, torch.device("cuda:0"))
    outs = []
    for _ in range(2):
        eng = Engine(built, device="cuda:0", dtype="bfloat16", max_batch=16, max_len=2048, max_new_tokens=64,
                     block_size=16, num_blocks=260, token_budget=512)
        rng = random.Random(1)
        g = torch.Generator().manual_seed(1)
        reqs = []
        for i in range(60):
            p = torch.randint(1, 4096, (rng.randint(16, 1500),), generator=g).tolist()
            reqs.append(eng.submit(p, max_new_tokens=rng.randint(4, 64), temperature=0.7 if i % 3 else 0.0, seed=i))
        steps = 0
        while eng.scheduler.has_work():
            assert eng.step()
            steps += 1
            if steps % 25 == 0:
                eng.scheduler.check()
        eng.scheduler.check()
        assert all(r.done and len(r.output) == r.max_new_tokens for r in reqs)
        assert eng.scheduler.preemptions > 10
        assert eng.cache.free_pages() == [260]
        outs.append([r.output for r in reqs])
    assert outs[0] == outs[1]


def test_first_tokens_of_a_sequence(tmp_path):
    """Positions 0 and 1 alone: one-token and two-token prompts, and a first portion of one token."""
    from socrates_b200.engine.runner import StepEntry
    folder = make_folder(tmp_path, "A")
    cfg, w = plain.load_folder(folder)
    eng = engine_for(folder, "float32")
    ids = [7, 201, 33]
    ref = plain.logits(w, cfg, ids)
    cache, runner = eng.cache, eng.runner
    cache.assign(0)
    cache.reserve(0, 1)
    l0 = runner.step([StepEntry(0, ids[:1], 0, [0])]).logits.cpu().double()
    cache.commit(0, 1)
    cache.reserve(0, 3)
    l12 = runner.step([StepEntry(0, ids[1:], 1, [0, 1])]).logits.cpu().double()
    cache.commit(0, 3)
    cache.release(0)
    scale = float(ref.abs().max())
    assert float((l0[0] - ref[0]).abs().max()) / scale < 1e-4
    assert float((l12 - ref[1:]).abs().max()) / scale < 1e-4


def test_warmup_records_every_width_and_changes_nothing(tmp_path):
    folder = make_folder(tmp_path, "B")
    ps = prompts_for("B", [9, 30, 2, 17])
    cold = engine_for(folder, "bfloat16").generate(ps, max_new_tokens=12)
    eng = engine_for(folder, "bfloat16", warmup=True)
    assert len(eng.runner._graphs) == 4                     # widths 1..max_batch
    replays = eng.runner.graph_replays
    assert eng.generate(ps, max_new_tokens=12) == cold
    assert eng.runner.graph_replays > replays
    assert len(eng.runner._graphs) == 4                     # nothing was recorded while serving


def test_command_line(tmp_path):
    import json
    import subprocess
    import sys
    from tiny_configs import TINY_A
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(TINY_A))
    root = __import__("pathlib").Path(__file__).resolve().parent.parent
    proc = subprocess.run([sys.executable, "-m", "socrates_b200.inference_paged", "--random-config", str(cfg),
                           "--num-prompts", "3", "--prompt-len", "9", "--max-new-tokens", "5", "--max-len", "64",
                           "--max-batch", "2", "--prompt", "hello"], cwd=str(root), capture_output=True, text=True,
                          timeout=300)
    assert proc.returncode == 0, proc.stderr[-2000:]
    assert "4 requests, 2 rows" in proc.stdout and "tok/s" in proc.stdout.splitlines()[-1]
    assert "> hello" in proc.stdout


def test_command_line_with_the_folders_tokenizer(tmp_path):
    """A model folder that carries tokenizer.json: text goes in through its chat template and
    text comes out (the 8 words of the test's tokenizer, never bare ids)."""
    import subprocess
    import sys
    from test_tokenizer import WORDS, write_tokenizer
    folder = make_folder(tmp_path, "A")
    write_tokenizer(folder)
    root = __import__("pathlib").Path(__file__).resolve().parent.parent
    proc = subprocess.run([sys.executable, "-m", "socrates_b200.inference_paged", "--model", str(folder),
                           "--prompt", "hello world", "--prompt", "how are you", "--max-new-tokens", "6",
                           "--max-len", "64", "--max-batch", "2", "--dtype", "float32"], cwd=str(root),
                          capture_output=True, text=True, timeout=300, env={**__import__("os").environ,
                                                                            "HF_HUB_OFFLINE": "1"})
    assert proc.returncode == 0, proc.stderr[-2000:]
    lines = proc.stdout.splitlines()
    assert "> hello world" in lines and "> how are you" in lines
    out = lines[lines.index("> hello world") + 1]
    # ids above the tokenizer's 8 words decode to nothing, ids within to words: never digits
    assert not any(ch.isdigit() for ch in out), out
    assert all(w in WORDS for w in out.split()), out


def test_entry_point_guards(tmp_path):
    from socrates_b200 import Engine, TooLong
    folder = make_folder(tmp_path, "A")
    eng = engine_for(folder, "bfloat16", max_len=64)
    with pytest.raises(TooLong):
        eng.submit(list(range(1, 60)), max_new_tokens=10)
    with pytest.raises(ValueError):
        eng.submit([1, 2, 999])                        # outside the vocabulary
    with pytest.raises(ValueError):
        eng.submit("text without a tokenizer")
    from socrates_b200.engine.tokenizer import ByteTokenizer
    eng2 = Engine(str(folder), tok=ByteTokenizer(256), max_batch=2, max_len=64, max_new_tokens=4)
    r = eng2.submit("hi there")
    eng2.run()
    assert r.done and len(r.output) <= 4 and 0 not in r.output
    with pytest.raises(ValueError):
        Engine(str(folder), dtype="float16")
