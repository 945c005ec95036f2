"""The tcgen05 attention tile kernel alone against the float64 reference: portions that
read earlier context from the pages, windows, group sizes 1 to 16, head sizes 64 and 128,
page sizes 16 to 64, a needle in every kind of slot, and poisoned slots."""

import pytest
import torch

from test_attention_mma_gpu import portions
from test_kernels_gpu import rand

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


def paged(lens, BS, Hkv, D, seed, spare=5):
    g = torch.Generator().manual_seed(seed)
    W = max(-(-n // BS) for n in lens) + 1
    need = sum(-(-n // BS) for n in lens)
    pages = (torch.randperm(need + spare, generator=g) + 1).tolist()
    table = torch.zeros(len(lens), W, dtype=torch.int32)
    for r, n in enumerate(lens):
        for b in range(-(-n // BS)):
            table[r, b] = pages.pop()
    shape = (need + spare + 1, Hkv, BS, D)
    k = torch.randn(shape, generator=g).to(BF).to(DEV)
    v = torch.randn(shape, generator=g).to(BF).to(DEV)
    return k, v, table.to(DEV)


def status():
    return torch.zeros(1, dtype=torch.int32, device=DEV)


@pytest.mark.parametrize("Hq,Hkv,D,BS", [(32, 8, 128, 16), (8, 8, 64, 16), (16, 1, 64, 32), (2, 1, 128, 64),
                                         (8, 2, 128, 16), (4, 2, 64, 64), (40, 8, 128, 16), (9, 3, 64, 32),
                                         (14, 2, 128, 16)])
@pytest.mark.parametrize("window", [0, 37, 200])
def test_prefill_tcgen05_portions_with_earlier_context(ops, ref, Hq, Hkv, D, BS, window):
    lens = [300, 70, 17, 1, 129, 700]
    k_pool, v_pool, table = paged(lens, BS, Hkv, D, seed=3)
    spec = [(0, 250, 50), (1, 0, 70), (2, 15, 2), (3, 0, 1), (4, 100, 28), (5, 0, 700)]
    starts, rows, firsts, trows, pos = portions(spec)
    N = int(starts[-1])
    q = rand(N, Hq * D, dtype=BF, seed=4)
    out = torch.full_like(q, float("nan"))
    st = status()
    ops.attention_prefill_tcgen05(out, q, k_pool, v_pool, table, starts, rows, firsts, Hq, D ** -0.5, st, window)
    assert int(st.item()) == 0
    want = ref.paged_attention_ref(q, k_pool, v_pool, table, trows, pos, Hq, D ** -0.5, window)
    err = (out.double() - want).abs()
    bad = (err > 2e-3 + 1.6e-2 * want.abs())
    assert not bool(bad.any()), (f"{int(bad.sum())} of {bad.numel()} wrong, worst {float(err.max()):.4g} at "
                                f"token {int(bad.nonzero()[0, 0])} (row {int(trows[int(bad.nonzero()[0, 0])])}, "
                                f"position {int(pos[int(bad.nonzero()[0, 0])])})")


def test_prefill_tcgen05_agrees_with_mma_kernel(ops):
    Hq, Hkv, D = 32, 8, 128
    lens = [2048]
    k_pool, v_pool, table = paged(lens, 16, Hkv, D, seed=8)
    starts, rows, firsts, trows, pos = portions([(0, 0, 2048)])
    q = rand(2048, Hq * D, dtype=BF, seed=9)
    a, b = torch.empty_like(q), torch.empty_like(q)
    st = status()
    ops.attention_prefill_tcgen05(a, q, k_pool, v_pool, table, starts, rows, firsts, Hq, D ** -0.5, st)
    ops.attention_prefill_mma(b, q, k_pool, v_pool, table, starts, rows, firsts, Hq, D ** -0.5)
    assert int(st.item()) == 0
    assert torch.allclose(a.float(), b.float(), **TOL)


def test_prefill_tcgen05_is_deterministic_under_repetition(ops):
    """The softmax warps and the issuing warp run unsynchronised except through mbarriers;
    a missing dependency shows as a run that differs (it did: a fast warp once read O before
    the last product).  Short rows (two key tiles) are where warps get furthest apart."""
    Hq, Hkv, D = 32, 8, 128
    k_pool, v_pool, table = paged([1024], 16, Hkv, D, seed=8)
    starts, rows, firsts, _, _ = portions([(0, 0, 1024)])
    q = rand(1024, Hq * D, dtype=BF, seed=9)
    st = status()
    first = torch.empty_like(q)
    ops.attention_prefill_tcgen05(first, q, k_pool, v_pool, table, starts, rows, firsts, Hq, D ** -0.5, st)
    for _ in range(150):
        again = torch.empty_like(q)
        ops.attention_prefill_tcgen05(again, q, k_pool, v_pool, table, starts, rows, firsts, Hq, D ** -0.5, st)
        assert torch.equal(again, first)
    assert int(st.item()) == 0


@pytest.mark.parametrize("needle", [0, 15, 16, 63, 64, 127, 128, 255, 256, 299])
def test_prefill_tcgen05_needle(ops, needle):
    """Zero queries give uniform weights; V is zero except one slot, so a query at position
    p outputs marker/(p+1) if the slot is at or before p and is read exactly once, else 0."""
    Hq, Hkv, D, n = 4, 2, 64, 300
    k_pool, v_pool, table = paged([n], 16, Hkv, D, seed=9)
    v_pool.zero_()
    v_pool[int(table[0, needle // 16]), :, needle % 16, :] = 8.0
    first = max(0, needle - 2)
    count = min(5, n - first)
    starts, rows, firsts, trows, pos = portions([(0, first, count)])
    q = torch.zeros(count, Hq * D, dtype=BF, device=DEV)
    out = torch.full_like(q, float("nan"))
    st = status()
    ops.attention_prefill_tcgen05(out, q, k_pool, v_pool, table, starts, rows, firsts, Hq, 1.0, st)
    for i, p in enumerate(range(first, first + count)):
        expect = 8.0 / (p + 1) if needle <= p else 0.0
        assert torch.allclose(out[i].float(), torch.full((Hq * D,), expect, device=DEV), rtol=1e-2, atol=1e-6), (p, needle)


def test_prefill_tcgen05_ignores_poisoned_slots(ops):
    """Slots past the rows' lengths, pages of nobody and the null page hold inf/NaN: whole
    pages are copied into shared memory, and still the result is bit-identical."""
    Hq, Hkv, D = 8, 2, 128
    lens = [21, 150]
    k_pool, v_pool, table = paged(lens, 16, Hkv, D, seed=5)
    starts, rows, firsts, _, _ = portions([(0, 10, 11), (1, 100, 50)])
    q = rand(61, Hq * D, dtype=BF, seed=7)

    def run():
        o = torch.empty_like(q)
        st = status()
        ops.attention_prefill_tcgen05(o, q, k_pool, v_pool, table, starts, rows, firsts, Hq, D ** -0.5, st)
        assert int(st.item()) == 0
        return o

    clean = run()
    owned = torch.zeros(k_pool.shape[0], 16, dtype=torch.bool, device=DEV)
    for r, n in enumerate(lens):
        for p in range(n):
            owned[int(table[r, p // 16]), p % 16] = True
    for pool, bad in ((k_pool, float("inf")), (v_pool, float("nan"))):
        pool.transpose(1, 2)[~owned] = bad
    dirty = run()
    assert torch.equal(clean, dirty)
    assert bool(torch.isfinite(dirty.float()).all())


def test_prefill_tcgen05_far_key_stands_out(ops, ref):
    Hq, Hkv, D, n = 4, 1, 128, 3000
    k_pool, v_pool, table = paged([n], 16, Hkv, D, seed=11)
    starts, rows, firsts, trows, pos = portions([(0, n - 40, 40)])
    q = rand(40, Hq * D, dtype=BF, seed=12)
    page, off = int(table[0, 0]), 3
    k_pool[page, 0, off, :] = (q.view(40, Hq, D)[39, 0].float() * 4).to(BF)
    out = torch.empty_like(q)
    st = status()
    ops.attention_prefill_tcgen05(out, q, k_pool, v_pool, table, starts, rows, firsts, Hq, 1.0, st)
    want = ref.paged_attention_ref(q, k_pool, v_pool, table, trows, pos, Hq, 1.0)
    assert torch.allclose(out.double(), want, **TOL)
    assert torch.allclose(out.view(40, Hq, D)[39, 0].float(), v_pool[page, 0, off].float(), atol=1e-2)


def test_tcgen05_support_matrix(ops):
    assert ops.attention_tcgen05_supports(32, 8, 128, 16)
    assert not ops.attention_tcgen05_supports(4, 2, 32, 16)            # head size: the mma.sync kernel's
    assert ops.attention_tcgen05_supports(9, 3, 64, 16)                # groups of 3: 42 tokens a tile, 2 rows idle
    assert ops.attention_tcgen05_supports(40, 8, 128, 16)              # groups of 5
    assert not ops.attention_tcgen05_supports(258, 2, 64, 16)          # a group larger than a tile
    assert not ops.attention_tcgen05_supports(32, 8, 128, 128)         # page size
