"""The scheduler's decisions, with a stand-in for the model: the next token is a
function of the whole sequence so far, so any slip in what is fed shows."""

import random

import pytest
import torch

from socrates_b200.cache import CacheManager, CacheNeeds, PagedKVSpec
from socrates_b200.engine.scheduler import QueueFull, Request, Scheduler, TooLong
from socrates_b200.sampling import SamplingParams

VOCAB = 50
STOP = 0


def next_token(seq):
    h = 17
    for t in seq:
        h = (h * 31 + t + 1) % 1000003
    return h % VOCAB


class FakeEngine:
    """Runs plans without a GPU: checks what is fed against what the cache holds."""

    def __init__(self, num_pages=64, max_batch=4, max_len=256, budget=32, window=None, max_queue=100,
                 only_windowed=False):
        needs = [CacheNeeds(PagedKVSpec(1, 16, None)), CacheNeeds(PagedKVSpec(1, 16, window))]
        if only_windowed:
            needs = needs[1:]
        self.cache = CacheManager(needs, max_batch, max_len, 16, num_pages, torch.float32, "cpu")
        self.s = Scheduler(self.cache, max_batch, max_len, budget, max_queue, stop_ids=[STOP])
        self.fed = {}                     # request id -> tokens the "cache" holds for its current row
        self.steps, self.max_tokens_seen, self.mixed_steps = 0, 0, 0

    def submit(self, ids, max_new=8):
        return self.s.submit(Request(ids=list(ids), max_new_tokens=max_new, sampling=SamplingParams()))

    def step(self):
        plan = self.s.plan()
        if plan is None:
            return False
        for r in plan.preempted:
            self.fed.pop(id(r), None)
        assert plan.num_tokens <= self.s.token_budget
        rows = [e.row for e in plan.entries]
        assert len(set(rows)) == len(rows)
        kinds = {e.count == 1 and e.samples for e in plan.entries}
        self.mixed_steps += len(kinds) == 2
        tokens = []
        for e in plan.entries:
            req = e.request
            held = self.fed.setdefault(id(req), [])
            assert e.row == req.row and e.start == len(held) == self.cache.lengths[e.row]
            assert not any(self.cache.pages_needed(e.row, e.start + e.count))   # pages were reserved
            new = [req.token_at(i) for i in range(e.start, e.start + e.count)]
            held.extend(new)
            assert e.samples == (len(held) == req.sequence_len)
            if e.samples:
                tokens.append(next_token(held))
        self.max_tokens_seen = max(self.max_tokens_seen, plan.num_tokens)
        self.s.complete(plan, tokens)
        for r in [r for r in list(self.fed)]:
            pass
        self.s.check()
        self.steps += 1
        return True

    def run(self, limit=10000):
        while self.s.has_work():
            assert self.step(), "requests are waiting but no step was planned"
            limit -= 1
            assert limit > 0


def expected_output(ids, max_new):
    seq, out = list(ids), []
    while len(out) < max_new:
        t = next_token(seq)
        if t == STOP:
            break
        out.append(t)
        seq.append(t)
    return out


def prompts(rng, n, lo=1, hi=60):
    return [[rng.randrange(1, VOCAB) for _ in range(rng.randint(lo, hi))] for _ in range(n)]


def test_outputs_do_not_depend_on_batching():
    rng = random.Random(0)
    ps = prompts(rng, 12)
    e = FakeEngine()
    reqs = [e.submit(p, 12) for p in ps]
    e.run()
    for p, r in zip(ps, reqs):
        assert r.done and r.output == expected_output(p, 12)
        alone = FakeEngine(max_batch=1, budget=7)
        one = alone.submit(p, 12)
        alone.run()
        assert one.output == r.output
    assert e.mixed_steps > 0                                  # prompt portions ran beside decode tokens
    assert e.cache.free_pages() == [64]


def test_prompts_are_cut_under_the_budget():
    e = FakeEngine(budget=16, num_pages=64)
    r = e.submit(list(range(1, 41)), 3)
    counts = []
    while e.s.has_work():
        plan = e.s.plan()
        counts.append([(x.start, x.count, x.samples) for x in plan.entries])
        toks = [next_token([x.request.token_at(i) for i in range(x.start + x.count)])
                for x in plan.entries if x.samples]
        e.s.complete(plan, toks)
    assert counts[:3] == [[(0, 16, False)], [(16, 16, False)], [(32, 8, True)]]
    assert counts[3] == [(40, 1, True)]


def test_decode_tokens_come_first_and_keep_their_budget():
    e = FakeEngine(budget=8, max_batch=4)
    a = e.submit([1, 2, 3], 20)
    e.step()                                                   # a is decoding now
    b = e.submit(list(range(1, 30)), 2)
    plan = e.s.plan()
    assert [(x.request is a, x.count) for x in plan.entries] == [(True, 1), (False, 7)]


def test_stop_token_and_max_new():
    e = FakeEngine()
    # find a prompt whose continuation hits the stop token early
    rng = random.Random(1)
    hit = None
    for p in prompts(rng, 300, 1, 6):
        out = expected_output(p, 30)
        if len(out) < 30:
            hit = (p, out)
            break
    assert hit is not None
    r = e.submit(hit[0], 30)
    q = e.submit([5, 6, 7], 4)
    e.run()
    assert r.output == hit[1] and STOP not in r.output and r.done
    assert len(q.output) <= 4 and q.done and q.event.is_set()


def test_door_checks():
    e = FakeEngine(max_len=64, num_pages=2, max_queue=2)
    with pytest.raises(TooLong):
        e.submit([1] * 60, 8)                                  # longer than a row
    with pytest.raises(TooLong):
        e.submit([1] * 30, 8)                                  # more pages than the pool has
    e.submit([1] * 10, 4)
    e.submit([1] * 10, 4)
    with pytest.raises(QueueFull):
        e.submit([1], 1)
    with pytest.raises(ValueError):
        FakeEngine().s.submit(Request(ids=[], max_new_tokens=1))


def test_windowed_pool_too_small_is_refused_at_the_door():
    """A windowed group needs the window and the token being written at once, which can straddle
    one page edge more than their count fills: 32 + 1 tokens in 16-slot pages are up to 4 pages.
    A pool one page short is refused at submit, not found out in the middle of generation."""
    small = FakeEngine(num_pages=3, window=32, only_windowed=True, max_batch=1)
    with pytest.raises(TooLong):
        small.submit([3] * 100, 20)
    small.submit([3] * 20, 8)                                  # 28 tokens never fill the window: 2 pages
    enough = FakeEngine(num_pages=4, window=32, only_windowed=True, max_batch=1)
    r = enough.submit([3 + (i % 40) for i in range(100)], 20)
    enough.run()
    assert r.done and enough.cache.free_pages() == [4]


def test_stream_receives_every_token_and_the_end():
    import queue
    e = FakeEngine()
    a = e.submit([4, 9, 2], 6)
    b = e.submit([7] * 20, 9)
    c = e.submit([11, 12], 5)
    for r in (a, b, c):
        r.stream = queue.Queue()
    e.step()
    c.cancelled = True                                     # a cancelled request's stream ends too
    e.run()
    for r in (a, b, c):
        got = []
        while True:
            item = r.stream.get_nowait()
            if item is None:
                break
            got.append(item)
        assert got == r.output and r.stream.empty()


def test_cancel_frees_the_row():
    e = FakeEngine()
    a, b = e.submit([1, 2, 3], 50), e.submit([4, 5, 6], 50)
    c = e.submit([7, 8], 5)
    c.cancelled = True
    e.step()
    e.step()
    a.cancelled = True
    e.run()
    assert not a.done and a.event.is_set() and b.done
    assert len(a.output) < 50 and c.output == []
    assert e.cache.free_pages() == [64]


def test_pages_run_out_latest_request_is_preempted_and_recomputed():
    """Four pages, two requests of one page each that grow to three: both are admitted (there
    is room for the newer one's prompt and a page to spare for the older), both take a second
    page, and when the older one needs its third the newer one gives up its pages, goes back to
    the front of the queue, is recomputed later, and still produces exactly its own tokens."""
    e = FakeEngine(num_pages=4, max_batch=2, budget=32)
    pa, pb = list(range(1, 15)), list(range(20, 34))           # 14 tokens each: one page, 44 with the new ones
    a, b = e.submit(pa, 30), e.submit(pb, 30)
    e.run()
    assert e.s.preemptions >= 1 and b.preemptions >= 1 and a.preemptions == 0
    assert a.output == expected_output(pa, 30) and b.output == expected_output(pb, 30)
    assert e.cache.free_pages() == [4]


def test_no_admission_into_pages_the_live_requests_need_next():
    """Three pages, the older request holds one: a newcomer whose prompt needs two would leave no
    page to spare for the older one's growth, would be the newest, and so would lose its pages
    again at once.  It waits in the queue instead; nobody is preempted."""
    e = FakeEngine(num_pages=3, max_batch=2, budget=32)
    pa, pb = list(range(1, 15)), list(range(20, 40))           # 14 tokens: one page; 20 tokens: two
    a, b = e.submit(pa, 12), e.submit(pb, 12)
    e.step()
    assert a.row == 0 and b.row == -1 and list(e.s.pending) == [b]
    e.run()
    assert e.s.preemptions == 0
    assert a.output == expected_output(pa, 12) and b.output == expected_output(pb, 12)
    assert e.cache.free_pages() == [3]


def test_pages_run_out_newest_request_waits():
    """The request that lacks a page is itself the newest: it keeps its pages and waits
    until the older one has finished; nobody is preempted."""
    e = FakeEngine(num_pages=3, max_batch=2, budget=32)
    pa, pb = list(range(1, 15)), list(range(20, 34))           # both grow from one page into two
    a, b = e.submit(pa, 12), e.submit(pb, 12)
    waited = 0
    while e.s.has_work():
        before = len(b.output)
        assert e.step()
        waited += (not a.done) and len(b.output) == before and b.cached >= 14
    assert e.s.preemptions == 0 and waited > 0
    assert a.output == expected_output(pa, 12) and b.output == expected_output(pb, 12)


def test_portion_shrinks_to_free_pages():
    """The newest request is in the middle of its prompt when the older one has taken the last
    free page: its next portion is cut to what its own last page still holds; nobody is preempted
    (only a request admitted later may be)."""
    e = FakeEngine(num_pages=4, max_batch=2, budget=12)
    a = e.submit(list(range(1, 16)), 10)                       # 15 tokens, grows into a second page
    b = e.submit(list(range(1, 41)), 4)                        # 40 tokens: three pages
    shrunk = False
    while e.s.has_work():
        free_before = e.cache.free_pages()[0]
        plan = e.s.plan()
        assert plan is not None
        for x in plan.entries:
            left = x.request.sequence_len - x.request.cached
            room = -x.request.cached % 16                  # slots left in the request's last page
            if x.request is b and b.cached < 40 and free_before == 0 and left > room:
                shrunk = True                              # it wanted more than its page holds and no page is free
                assert x.count == room and plan.preempted == []
        tokens = []
        for x in plan.entries:
            held = e.fed.setdefault(id(x.request), [])
            held.extend(x.request.token_at(i) for i in range(x.start, x.start + x.count))
            if x.samples:
                tokens.append(next_token(held))
        for r in plan.preempted:
            e.fed.pop(id(r), None)
        e.s.complete(plan, tokens)
    assert shrunk
    assert a.output == expected_output(list(range(1, 16)), 10) and b.output == expected_output(list(range(1, 41)), 4)


@pytest.mark.parametrize("seed", range(5))
def test_random_load_with_few_pages(seed):
    rng = random.Random(seed)
    window = rng.choice([None, 24])
    e = FakeEngine(num_pages=rng.choice([5, 8, 13]), max_batch=rng.choice([2, 3, 4]),
                   budget=rng.choice([4, 9, 32]), max_len=80, window=window)
    ps = prompts(rng, 25, 1, 50)
    reqs = []
    while ps or e.s.has_work():
        for _ in range(rng.randint(0, 3)):
            if ps:
                p = ps.pop()
                reqs.append((p, e.submit(p, rng.randint(1, 20))))
        if e.s.has_work():
            assert e.step()
    for p, r in reqs:
        assert r.done and r.output == expected_output(p, r.max_new_tokens)
    assert all(f == g.allocator.num_pages for f, g in zip(e.cache.free_pages(), e.cache.groups))
