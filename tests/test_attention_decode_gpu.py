"""The streaming decode-attention kernel alone against the float64 reference: chunk sizes from one
subtile to the whole row, chunk and page seams, windows, group sizes 1 to 16, head sizes 16 to
128, page sizes 16 to 64, a far key that must dominate, poisoned slots, the shapes the benchmark
times (batch 1/8/64, 2,048 to 7,800 keys, a table 512 pages wide), and that a token's numbers are
the same bits whatever else is in the batch."""

import pytest
import torch

from test_kernels_gpu import paged_case, rand

pytestmark = pytest.mark.gpu
DEV = "cuda"
BF = torch.bfloat16
TOL = dict(atol=2e-3, rtol=1.6e-2)      # the reference's kernel tolerance (tests/test_kernel_cuda.py:27)


@pytest.fixture(scope="module")
def ops():
    from socrates_b200.kernels import ops, require_kernels
    require_kernels()
    return ops


@pytest.fixture(scope="module")
def ref():
    from socrates_b200.kernels import reference
    return reference


def run(ops, q, k_pool, v_pool, table, trows, pos, Hq, scale, window, chunk, max_len, variant=0, scratch=None):
    N, D = q.shape[0], k_pool.shape[3]
    Hkv = k_pool.shape[1]
    span = min(max_len, window) if window else max_len
    chunks = 1 if chunk >= max_len else -(-span // chunk) + 1
    if scratch is None:
        scratch = (torch.full((N * Hq * chunks * D,), float("nan"), device=DEV),
                   torch.full((N * Hq * chunks * 2,), float("nan"), device=DEV),
                   torch.zeros(N * Hkv, dtype=torch.int32, device=DEV))
    out = torch.full_like(q, float("nan"))
    ops.attention_decode_stream(out, q, k_pool, v_pool, table, trows, pos, Hq, scale, window, chunk, chunks,
                                *scratch, variant=variant)
    return out, scratch


@pytest.mark.parametrize("Hq,Hkv,D", [(4, 2, 16), (8, 2, 32), (8, 8, 64), (32, 8, 128), (16, 1, 64),
                                      (12, 4, 128), (12, 1, 128), (10, 2, 128), (64, 8, 128)])
@pytest.mark.parametrize("window", [0, 37])
@pytest.mark.parametrize("chunk", [16, 48, 128, 4096])
def test_decode_stream(ops, ref, Hq, Hkv, D, window, chunk):
    lens = [1, 15, 16, 17, 63, 64, 65, 130, 257, 700]
    k_pool, v_pool, table = paged_case(lens, 16, Hkv, D, BF, seed=5)
    N = len(lens)
    trows = torch.arange(N, dtype=torch.int32, device=DEV)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    q = rand(N, Hq * D, dtype=BF, seed=6)
    out, scratch = run(ops, q, k_pool, v_pool, table, trows, pos, Hq, D ** -0.5, window, chunk, 720)
    want = ref.paged_attention_ref(q, k_pool, v_pool, table, trows, pos, Hq, D ** -0.5, window)
    assert torch.allclose(out.double(), want, **TOL)
    # the counters are back at zero: a second call with the same scratch gives the same bits
    assert int(scratch[2].abs().sum()) == 0
    again, _ = run(ops, q, k_pool, v_pool, table, trows, pos, Hq, D ** -0.5, window, chunk, 720, scratch=scratch)
    assert torch.equal(again, out)
    for variant in (1, 2, 3, 4):
        other, _ = run(ops, q, k_pool, v_pool, table, trows, pos, Hq, D ** -0.5, window, chunk, 720, variant=variant)
        assert torch.equal(other, out)          # the ring's depth changes no number


@pytest.mark.parametrize("BS", [16, 32, 64])
def test_decode_stream_page_sizes(ops, ref, BS):
    Hq, Hkv, D = 8, 2, 64
    lens = [1, BS - 1, BS, BS + 1, 5 * BS + 3, 300]
    k_pool, v_pool, table = paged_case(lens, BS, Hkv, D, BF, seed=8)
    N = len(lens)
    trows = torch.arange(N, dtype=torch.int32, device=DEV)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    q = rand(N, Hq * D, dtype=BF, seed=9)
    for chunk in (32, 128):
        out, _ = run(ops, q, k_pool, v_pool, table, trows, pos, Hq, D ** -0.5, 0, chunk, 320)
        want = ref.paged_attention_ref(q, k_pool, v_pool, table, trows, pos, Hq, D ** -0.5, 0)
        assert torch.allclose(out.double(), want, **TOL)


@pytest.mark.parametrize("needle", [0, 15, 16, 63, 64, 127, 128, 255, 256, 299])
def test_decode_stream_needle(ops, needle):
    """Zero queries, V zero except one slot: the output is marker/n if that slot is read exactly
    once, whatever chunk it falls into."""
    Hq, Hkv, D, n = 4, 2, 32, 300
    k_pool, v_pool, table = paged_case([n], 16, Hkv, D, BF, seed=9)
    v_pool.zero_()
    v_pool[int(table[0, needle // 16]), :, needle % 16, :] = 8.0
    q = torch.zeros(1, Hq * D, dtype=BF, device=DEV)
    trows = torch.zeros(1, dtype=torch.int32, device=DEV)
    pos = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
    want = torch.full((1, Hq * D), 8.0 / n, device=DEV)
    for chunk in (16, 64, 128, 512):
        out, _ = run(ops, q, k_pool, v_pool, table, trows, pos, Hq, 1.0, 0, chunk, 304)
        assert torch.allclose(out.float(), want, rtol=1e-2)


def test_decode_stream_ignores_poisoned_slots(ops, ref):
    """Slots past a row's length, behind its window, and the whole null page hold inf and NaN."""
    Hq, Hkv, D = 8, 2, 64
    lens = [21, 150]
    k_pool, v_pool, table = paged_case(lens, 16, Hkv, D, BF, seed=5)
    trows = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    pos = torch.tensor([20, 149], dtype=torch.int32, device=DEV)
    q = rand(2, Hq * D, dtype=BF, seed=6)
    want = ref.paged_attention_ref(q, k_pool, v_pool, table, trows, pos, Hq, D ** -0.5, 40)
    for pool in (k_pool, v_pool):
        pool[0] = float("nan")
        pool[int(table[0, 1]), :, 5:, :] = float("inf")            # row 0 holds 21 keys: slots 21.. of its 2nd page
        pool[int(table[1, 9]), :, 6:, :] = float("nan")            # row 1 holds 150 keys
        for b in range(6):                                         # keys 0..95 lie wholly behind the window of 40
            pool[int(table[1, b])] = float("inf")
    for chunk in (16, 64, 128):
        out, _ = run(ops, q, k_pool, v_pool, table, trows, pos, Hq, D ** -0.5, 40, chunk, 160)
        assert torch.isfinite(out.float()).all()
        assert torch.allclose(out.double(), want, **TOL)


def bench_case(N, ctx, Hq, Hkv, D, seed):
    """N rows of `ctx` keys in 16-slot pages, a block table 512 pages wide (8,192-token rows)."""
    g = torch.Generator().manual_seed(seed)
    BS, W = 16, 512
    per_row = -(-ctx // BS)
    pages = torch.randperm(N * per_row + 7, generator=g) + 1
    table = torch.zeros(N, W, dtype=torch.int32)
    for r in range(N):
        table[r, :per_row] = pages[r * per_row:(r + 1) * per_row]
    shape = (N * per_row + 8, Hkv, BS, D)
    k = torch.randn(shape, device=DEV, dtype=torch.float32).to(BF)
    v = torch.randn(shape, device=DEV, dtype=torch.float32).to(BF)
    q = torch.randn(N, Hq * D, device=DEV, dtype=torch.float32).to(BF)
    return q, k, v, table.to(DEV)


@pytest.mark.parametrize("N", [1, 8, 64])
@pytest.mark.parametrize("ctx", [2048, 4095, 4096, 7800])
@pytest.mark.parametrize("Hq", [32, 64])
def test_decode_stream_at_the_benchmark_shapes(ops, ref, N, ctx, Hq):
    """What bench.py times (8 KV heads of 128, groups of 4 and 8, chunks of 128 keys), checked for once.
    One far key of each checked row is made to match its query, so that a chunk that is skipped,
    read twice or merged with a wrong weight changes the result by far more than the tolerance."""
    DECODE_CHUNK_KEYS = 128      # PAGED_PARTITION=128, the reference's own split size
    Hkv, D = 8, 128
    q, k_pool, v_pool, table = bench_case(N, ctx, Hq, Hkv, D, seed=N + ctx)
    trows = torch.arange(N, dtype=torch.int32, device=DEV)
    pos = torch.full((N,), ctx - 1, dtype=torch.int32, device=DEV)
    check = sorted({0, N // 2, N - 1})
    for i, n in enumerate(check):
        far = (37 + 1000 * i) % ctx
        page, slot = int(table[n, far // 16]), far % 16
        k_pool[page, :, slot, :] = (q[n].view(Hq, D)[::Hq // Hkv] * 0.5).to(BF)    # score ~ 0.5 |q|^2 / sqrt(D)
    out, _ = run(ops, q, k_pool, v_pool, table, trows, pos, Hq, D ** -0.5, 0, DECODE_CHUNK_KEYS, 8192)
    sel = torch.tensor(check, device=DEV)
    want = ref.paged_attention_ref(q[sel], k_pool, v_pool, table, trows[sel], pos[sel], Hq, D ** -0.5, 0)
    assert torch.allclose(out[sel].double(), want, **TOL)
    assert torch.isfinite(out.float()).all()


def test_decode_stream_numbers_do_not_depend_on_the_batch(ops):
    """A token alone, and the same token among 63 others of other lengths: the same bits."""
    Hq, Hkv, D = 32, 8, 128
    lens = [1 + (977 * i) % 3000 for i in range(64)]
    lens[17] = 2500
    k_pool, v_pool, table = paged_case(lens, 16, Hkv, D, BF, seed=11)
    N = len(lens)
    trows = torch.arange(N, dtype=torch.int32, device=DEV)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    q = rand(N, Hq * D, dtype=BF, seed=12)
    full, _ = run(ops, q, k_pool, v_pool, table, trows, pos, Hq, D ** -0.5, 0, 128, 3008)
    for n in (0, 17, 63):
        alone, _ = run(ops, q[n:n + 1].contiguous(), k_pool, v_pool, table, trows[n:n + 1].contiguous(),
                       pos[n:n + 1].contiguous(), Hq, D ** -0.5, 0, 128, 3008)
        assert torch.equal(alone[0], full[n])


@pytest.mark.parametrize("N", [1, 8, 64])
@pytest.mark.parametrize("ctx_len", [2048, 4095, 4096, 7800])
@pytest.mark.parametrize("Hq", [32, 64])
@pytest.mark.parametrize("partition", ["auto", "128"])
def test_the_mixers_decode_choice_at_the_benchmark_shapes(ops, ref, monkeypatch, N, ctx_len, Hq, partition):
    """`paged_attention` as a decode step of the benchmark calls it (graph shapes: the longest
    possible row bounds the split): the split-key kernel with the partition count that the batch
    width gives ("auto"), and the streaming kernel ("128"), against the reference, with a far key
    made to match each checked query."""
    from socrates_b200.engine.context import Buffers, StepContext
    from socrates_b200.parts.attention import paged_attention
    monkeypatch.setenv("PAGED_PARTITION", partition)
    Hkv, D = 8, 128
    q, k_pool, v_pool, table = bench_case(N, ctx_len, Hq, Hkv, D, seed=N + ctx_len + 1)
    trows = torch.arange(N, dtype=torch.int32, device=DEV)
    pos = torch.full((N,), ctx_len - 1, dtype=torch.int32, device=DEV)
    check = sorted({0, N // 2, N - 1})
    for i, n in enumerate(check):
        far = (53 + 1000 * i) % ctx_len
        k_pool[int(table[n, far // 16]), :, far % 16, :] = (q[n].view(Hq, D)[::Hq // Hkv] * 0.5).to(BF)
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    ctx = StepContext(BF, torch.device(DEV), Buffers(64, DEV), N, N, None, pos, trows, None, None, None, None,
                      all_decode=True, max_context=8192, num_sms=sms,
                      status=torch.zeros(1, dtype=torch.int32, device=DEV))
    out = torch.full_like(q, float("nan"))
    paged_attention(ctx, out, q, k_pool, v_pool, table, Hq, D ** -0.5, 0, 8192)
    sel = torch.tensor(check, device=DEV)
    want = ref.paged_attention_ref(q[sel], k_pool, v_pool, table, trows[sel], pos[sel], Hq, D ** -0.5, 0)
    assert torch.allclose(out[sel].double(), want, **TOL)
    assert torch.isfinite(out.float()).all()
