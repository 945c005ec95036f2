"""The tensor-core attention kernels alone against the float64 reference: prompt
portions that read earlier context from the pages, decode tokens with split keys,
windows, group sizes 1 to 16, head sizes 16 to 128, needles and poisoned slots."""

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


def portions(spec):
    """spec: [(row, first_pos, count)] -> (seq_starts, seq_rows, seq_first_pos, token_rows, positions)."""
    starts, rows, firsts, trows, pos = [0], [], [], [], []
    for row, first, count in spec:
        rows.append(row)
        firsts.append(first)
        trows += [row] * count
        pos += list(range(first, first + count))
        starts.append(len(trows))
    t = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    return t(starts), t(rows), t(firsts), t(trows), t(pos)


@pytest.mark.parametrize("Hq,Hkv,D", [(4, 2, 16), (8, 2, 32), (8, 8, 64), (32, 8, 128), (16, 1, 64), (2, 1, 128)])
@pytest.mark.parametrize("window", [0, 37])
def test_prefill_mma_portions_with_earlier_context(ops, ref, Hq, Hkv, D, window):
    lens = [300, 70, 17, 1, 129]
    k_pool, v_pool, table = paged_case(lens, 16, Hkv, D, BF, seed=3)
    # whole short rows, the tail of a long row (earlier context in pages), a 2-token
    # portion, a single token, and a portion that ends on a page edge
    spec = [(0, 250, 50), (1, 0, 70), (2, 15, 2), (3, 0, 1), (4, 100, 28)]
    starts, rows, firsts, trows, pos = portions(spec)
    N = int(starts[-1])
    q = rand(N, Hq * D, dtype=BF, seed=4)
    out = torch.full_like(q, float("nan"))
    ops.attention_prefill_mma(out, q, k_pool, v_pool, table, starts, rows, firsts, Hq, D ** -0.5, window)
    want = ref.paged_attention_ref(q, k_pool, v_pool, table, trows, pos, Hq, D ** -0.5, window)
    assert torch.allclose(out.double(), want, **TOL)


@pytest.mark.parametrize("Hq,Hkv,D,NP", [(4, 2, 16, 1), (8, 2, 32, 3), (8, 8, 64, 2), (32, 8, 128, 5),
                                         (16, 1, 64, 7), (12, 4, 128, 4), (12, 1, 128, 2), (10, 2, 128, 1)])
@pytest.mark.parametrize("window", [0, 37])
def test_decode_mma(ops, ref, Hq, Hkv, D, NP, window):
    lens = [1, 15, 16, 17, 63, 64, 65, 130, 257, 700]
    k_pool, v_pool, table = paged_case(lens, 16, Hkv, D, BF, seed=5)
    N = len(lens)
    trows = torch.arange(N, dtype=torch.int32, device=DEV)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    q = rand(N, Hq * D, dtype=BF, seed=6)
    out = torch.full_like(q, float("nan"))
    part_o = torch.empty(N * Hq * NP * D, device=DEV)
    part_ml = torch.empty(N * Hq * NP * 2, device=DEV)
    ops.attention_decode_mma(out, q, k_pool, v_pool, table, trows, pos, Hq, D ** -0.5, window, NP, part_o, part_ml)
    want = ref.paged_attention_ref(q, k_pool, v_pool, table, trows, pos, Hq, D ** -0.5, window)
    assert torch.allclose(out.double(), want, **TOL)
    # 2 to 4 partitions merge inside the kernel (a cluster), more through the reduce kernel: both
    # paths must leave what a second call needs (nothing) and give the same result again
    again = torch.full_like(q, float("nan"))
    ops.attention_decode_mma(again, q, k_pool, v_pool, table, trows, pos, Hq, D ** -0.5, window, NP, part_o, part_ml)
    assert torch.equal(again, out)
    other = torch.full_like(q, float("nan"))
    ops.attention_decode_mma(other, q, k_pool, v_pool, table, trows, pos, Hq, D ** -0.5, window, NP, part_o, part_ml,
                             variant=1)
    assert torch.allclose(other.double(), want, **TOL)


@pytest.mark.parametrize("needle", [0, 15, 16, 63, 64, 255, 256, 299])
def test_mma_needle(ops, needle):
    """Zero queries, V zero except one slot: the output is marker/n if the slot is read
    exactly once, for the decode kernel (1 and 4 partitions) and for the tile kernel."""
    Hq, Hkv, D, n = 4, 2, 32, 300
    k_pool, v_pool, table = paged_case([n], 16, Hkv, D, BF, seed=9)
    v_pool.zero_()
    v_pool[int(table[0, needle // 16]), :, needle % 16, :] = 8.0
    q = torch.zeros(1, Hq * D, dtype=BF, device=DEV)
    trows = torch.zeros(1, dtype=torch.int32, device=DEV)
    pos = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
    want = torch.full((1, Hq * D), 8.0 / n, device=DEV)
    for NP in (1, 4):
        out = torch.empty_like(q)
        ops.attention_decode_mma(out, q, k_pool, v_pool, table, trows, pos, Hq, 1.0, 0, NP,
                                 torch.empty(Hq * NP * D, device=DEV), torch.empty(Hq * NP * 2, device=DEV))
        assert torch.allclose(out.float(), want, rtol=1e-2)
    starts, rows, firsts, trows2, pos2 = portions([(0, n - 3, 3)])
    q3 = torch.zeros(3, Hq * D, dtype=BF, device=DEV)
    out = torch.empty_like(q3)
    ops.attention_prefill_mma(out, q3, k_pool, v_pool, table, starts, rows, firsts, Hq, 1.0, 0)
    for i, p in enumerate(range(n - 3, n)):
        expect = 8.0 / (p + 1) if needle <= p else 0.0
        assert torch.allclose(out[i].float(), torch.full((Hq * D,), expect, device=DEV), rtol=1e-2, atol=1e-6)


def test_mma_ignores_poisoned_slots(ops):
    Hq, Hkv, D = 8, 2, 64
    lens = [21, 150]
    k_pool, v_pool, table = paged_case(lens, 16, Hkv, D, BF, seed=5)
    trows = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    pos = torch.tensor([20, 149], dtype=torch.int32, device=DEV)
    q = rand(2, Hq * D, dtype=BF, seed=6)
    starts, rows, firsts, _, _ = portions([(0, 10, 11), (1, 100, 50)])
    q2 = rand(61, Hq * D, dtype=BF, seed=7)

    def run():
        a, b = torch.empty_like(q), torch.empty_like(q2)
        NP = 3
        ops.attention_decode_mma(a, q, k_pool, v_pool, table, trows, pos, Hq, D ** -0.5, 0, NP,
                                 torch.empty(2 * Hq * NP * D, device=DEV), torch.empty(2 * Hq * NP * 2, device=DEV))
        ops.attention_prefill_mma(b, q2, k_pool, v_pool, table, starts, rows, firsts, Hq, D ** -0.5, 0)
        return a, b

    clean = run()
    owned = torch.zeros(k_pool.shape[0], 16, dtype=torch.bool, device=DEV)
    for r, n in enumerate(lens):
        for p in range(n):
            owned[int(table[r, p // 16]), p % 16] = True
    for pool, bad in ((k_pool, float("inf")), (v_pool, float("nan"))):
        pool.transpose(1, 2)[~owned] = bad
    dirty = run()
    assert torch.equal(clean[0], dirty[0]) and torch.equal(clean[1], dirty[1])


def test_mma_far_key_stands_out(ops, ref):
    Hq, Hkv, D, n = 4, 1, 128, 3000
    k_pool, v_pool, table = paged_case([n], 16, Hkv, D, BF, seed=11)
    q = rand(1, Hq * D, dtype=BF, seed=12)
    page, off = int(table[0, 0]), 3
    k_pool[page, 0, off, :] = (q.view(Hq, D)[0].float() * 4).to(BF)
    trows = torch.zeros(1, dtype=torch.int32, device=DEV)
    pos = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
    NP = 6
    out = torch.empty_like(q)
    ops.attention_decode_mma(out, q, k_pool, v_pool, table, trows, pos, Hq, 1.0, 0, NP,
                             torch.empty(Hq * NP * D, device=DEV), torch.empty(Hq * NP * 2, device=DEV))
    want = ref.paged_attention_ref(q, k_pool, v_pool, table, trows, pos, Hq, 1.0)
    assert torch.allclose(out.double(), want, **TOL)
    assert torch.allclose(out.view(Hq, D)[0].float(), v_pool[page, 0, off].float(), atol=1e-2)


def test_mma_support_matrix(ops):
    assert ops.attention_mma_supports(32, 8, 128, 16, True) and ops.attention_mma_supports(32, 8, 128, 16, False)
    assert not ops.attention_mma_supports(32, 8, 48, 16, True)          # head size not built
    assert not ops.attention_mma_supports(9, 3, 64, 16, False)          # 64 rows do not split into groups of 3
    assert ops.attention_mma_supports(9, 3, 64, 16, True)
    assert not ops.attention_mma_supports(32, 1, 64, 16, True)          # more than 16 heads per KV head
