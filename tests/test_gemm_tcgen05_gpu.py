"""The tcgen05 matrix product alone against a float64 product of the same bfloat16
operands: many rows (activations on the accumulator lanes), few rows (weights on the
lanes, K cut into parts), ragged sizes that are no multiple of any tile."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"


@pytest.fixture(scope="module")
def ops():
    from socrates_b200.kernels import ops, require_kernels
    require_kernels()
    return ops


def operands(M, N, K, seed=0):
    g = torch.Generator().manual_seed(seed + M * 7 + N * 3 + K)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(N, K, generator=g).to(torch.bfloat16).to(DEV)
    return a, w, a.double() @ w.double().T


def close(out, want, K, bf16_out):
    # float32 accumulation of K products of unit-variance numbers, then one rounding
    atol = 1e-4 * math.sqrt(K) + (2 ** -8 * float(want.abs().max()) if bf16_out else 0.0)
    err = float((out.double() - want).abs().max())
    assert err <= atol, f"max error {err:.4g} > {atol:.4g}"


SHAPES = [
    # few rows: the weights fill the accumulator lanes
    (1, 384, 64), (8, 2560, 2560), (16, 200, 96), (17, 1000, 160), (33, 128, 256), (64, 6144, 2560),
    (5, 151936 // 16, 72),
    # many rows: the activations fill the lanes
    (65, 384, 96), (128, 64, 64), (300, 2560, 4096), (1000, 96, 160), (257, 6144, 2560), (130, 200, 72),
]


@pytest.mark.parametrize("M,N,K", SHAPES)
def test_gemm_tcgen05(ops, M, N, K):
    a, w, want = operands(M, N, K)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for dtype in (torch.bfloat16, torch.float32):
        out = torch.full((M, N), float("nan"), dtype=dtype, device=DEV)
        ops.gemm_tcgen05(out, a, w, status)
        close(out, want, K, dtype == torch.bfloat16)
    assert int(status.item()) == 0


@pytest.mark.parametrize("M,N,K,splits", [(8, 2560, 4096, 14), (1, 2560, 9728, 14), (64, 384, 160, 3),
                                          (16, 96, 64, 4), (300, 2560, 4096, 3)])
def test_gemm_tcgen05_split_k(ops, M, N, K, splits):
    a, w, want = operands(M, N, K, seed=1)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    S = ops.gemm_tcgen05_splits(K, splits)
    assert 1 <= S <= splits
    out = torch.full((S, M, N), float("nan"), dtype=torch.float32, device=DEV)
    assert ops.gemm_tcgen05(out, a, w, status, splits) == S
    close(out.sum(0), want, K, False)
    assert int(status.item()) == 0


@pytest.mark.parametrize("M", [3, 24, 50])
def test_gemm_tcgen05_few_rows_long_k(ops, M):
    """K so long that the ring of stages is refilled dozens of times, in each of the three tile
    widths for few rows: the threads that share the issuing of the MMAs must each meet their
    stages' refills in order.  Launched back to back many times, one result for all."""
    N, K = 640, 17408
    a, w, want = operands(M, N, K, seed=2)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    outs = [torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV) for _ in range(40)]
    for out in outs:
        ops.gemm_tcgen05(out, a, w, status)
    close(outs[0], want, K, False)
    for out in outs[1:]:
        assert torch.equal(out, outs[0])
    assert int(status.item()) == 0


def test_gemm_tcgen05_one_hot_rows_and_columns(ops):
    """Operands that are rows of the identity: the product must reproduce the other
    operand exactly, which shows a transposed, shifted or swizzle-scrambled tile."""
    for M, N, K in ((8, 256, 128), (200, 384, 192)):
        w = torch.randn(N, K).to(torch.bfloat16).to(DEV)
        a = torch.zeros(M, K, dtype=torch.bfloat16, device=DEV)
        idx = torch.arange(M) * 5 % K
        a[torch.arange(M), idx] = 1.0
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        out = torch.empty(M, N, dtype=torch.float32, device=DEV)
        ops.gemm_tcgen05(out, a, w, status)
        assert torch.equal(out, w.float()[:, idx.to(DEV)].T.contiguous())


@pytest.mark.parametrize("M,N,K", [(2048, 2560, 4096), (300, 19456, 256), (129, 6144, 320), (1000, 130, 64),
                                   (70, 128, 72), (5000, 384, 96)])
def test_gemm_tcgen05_persistent_many_tiles(ops, M, N, K):
    """Shapes that give one block several tiles (two accumulators in turn), ragged edges,
    and every tile width; compared with the one-tile-per-block kernel too: the same bits at the
    full tile width, where one thread adds a tile's K blocks in the same order in both kernels
    (narrower tiles add them as two halves)."""
    a, w, want = operands(M, N, K, seed=2)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
    ops.gemm_tcgen05(out, a, w, status)
    close(out, want, K, False)
    other = torch.empty_like(out)
    ops.gemm_tcgen05(other, a, w, status, variant=4)
    close(other, want, K, False)
    full = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
    ops.gemm_tcgen05(full, a, w, status, variant=256)
    assert torch.equal(full, other)
    outb = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_tcgen05(outb, a, w, status)
    close(outb, want, K, True)
    assert int(status.item()) == 0


@pytest.mark.parametrize("width", [128, 160, 256])
def test_gemm_tcgen05_persistent_every_tile_width(ops, width):
    """Each tile width of the persistent kernel, forced, on a ragged shape with several
    tiles per block and a last column tile that is cut."""
    M, N, K = 700, 5 * width + 40, 328
    a, w, want = operands(M, N, K, seed=width)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for dtype in (torch.bfloat16, torch.float32):
        out = torch.full((M, N), float("nan"), dtype=dtype, device=DEV)
        ops.gemm_tcgen05(out, a, w, status, variant=width)
        close(out, want, K, dtype == torch.bfloat16)
    assert int(status.item()) == 0


@pytest.mark.parametrize("width", [128, 160, 192, 256])
@pytest.mark.parametrize("M,K", [(700, 328), (100, 64), (257, 72), (1024, 2048)])
def test_gemm_tcgen05_pair_kernel(ops, width, M, K):
    """The kernel in which two SMs share a tile of 256 rows (cta_group::2), forced, at every
    tile width: row counts that leave the second block of a pair partly or wholly without rows,
    a last column tile that is cut, several tiles per pair."""
    N = 5 * width + 40
    a, w, want = operands(M, N, K, seed=1000 + width)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    for dtype in (torch.bfloat16, torch.float32):
        out = torch.full((M, N), float("nan"), dtype=dtype, device=DEV)
        ops.gemm_tcgen05(out, a, w, status, variant=1000 + width)
        close(out, want, K, dtype == torch.bfloat16)
    assert int(status.item()) == 0


def test_gemm_tcgen05_pair_kernel_is_the_choice_for_many_rows(ops):
    """8,192 rows of a narrow projection: the default path (the pair kernel there) and the
    fused SiLU*mul epilogue on it."""
    M, N, K = 8192, 2560, 512
    a, w, want = operands(M, N, K, seed=77)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
    ops.gemm_tcgen05(out, a, w, status)
    close(out, want, K, False)
    forced = torch.full((M, N), float("nan"), dtype=torch.float32, device=DEV)
    ops.gemm_tcgen05(forced, a, w, status, variant=1256)
    assert torch.equal(out, forced)
    gate, up = want[:, 0::2], want[:, 1::2]
    act = torch.full((M, N // 2), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_tcgen05(act, a, w, status, epilogue=1)
    ref = up * gate * torch.sigmoid(gate)
    err = float((act.double() - ref).abs().max())
    assert err <= 2 ** -7 * float(ref.abs().max()) + 1e-2, err
    assert int(status.item()) == 0


@pytest.mark.parametrize("M,N,K", [(2048, 2560, 4096), (2048, 2560, 9728), (2048, 5120, 8192), (1024, 2560, 4096),
                                   (1999, 2500, 1000), (8192, 2560, 512), (300, 6144, 2560)])
def test_gemm_tcgen05_equal_shares(ops, M, N, K):
    """The pair kernel dealing equal shares of K blocks: the parts add up to the product; a tile
    that one pair finishes alone has zeros in the other parts; a second call into a buffer full of
    NaN gives the same bits (every element of every part is written).  Shapes: the narrow
    projections of the 4B and 32B widths at 2,048 rows, fewer tiles than pairs (three pieces to a
    tile), ragged rows, columns and K."""
    a, w, want = operands(M, N, K, seed=2)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    S = ops.gemm_tcgen05_shares_parts(M, N, K)
    assert 1 <= S <= 4
    out = torch.full((S, M, N), float("nan"), dtype=torch.float32, device=DEV)
    assert ops.gemm_tcgen05(out, a, w, status, S, variant=ops.SHARES_VARIANT) == S
    assert int(status.item()) == 0
    assert torch.isfinite(out).all()
    close(out.double().sum(0), want, K, False)
    again = torch.full_like(out, float("nan"))
    ops.gemm_tcgen05(again, a, w, status, S, variant=ops.SHARES_VARIANT)
    assert torch.equal(again, out)


def test_equal_shares_are_chosen_for_the_narrow_projections_of_a_long_portion(ops):
    """The step context's choice: 2,048 rows through o and down of the 4B widths run as equal
    shares (two parts); the wide products and short portions do not."""
    from socrates_b200.engine.context import Buffers, StepContext
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    ctx = StepContext(torch.bfloat16, torch.device(DEV), Buffers(64, DEV), 1, 1, None, None, None, None, None, None,
                      None, all_decode=False, max_context=1, num_sms=sms,
                      status=torch.zeros(1, dtype=torch.int32, device=DEV))
    shape = lambda n, k: torch.empty(n, k, dtype=torch.bfloat16, device=DEV)
    if sms == 148:
        assert ctx.gemm_splits(2048, shape(2560, 4096), torch.bfloat16) == 2
        assert ctx.gemm_splits(2048, shape(2560, 9728), torch.bfloat16) == 2
        assert ctx.gemm_splits(2048, shape(6144, 2560), torch.bfloat16, shares=False) == 1
        assert ctx.gemm_shares(128, shape(2560, 4096), torch.bfloat16) == 0
    a, wt, want = operands(2048, 2560, 4096, seed=3)
    S = ctx.gemm_splits(2048, wt, torch.bfloat16)
    out = torch.full((S, 2048, 2560), float("nan"), dtype=torch.float32, device=DEV)
    ctx.gemm(out, a, wt)
    close(out.double().sum(0), want, 4096, False)
    assert int(ctx.status.item()) == 0


@pytest.mark.parametrize("M,F,K", [(200, 320, 96), (2048, 9728, 256), (65, 64, 64), (300, 203, 72),
                                   (8, 9728, 2560), (1, 80, 64), (64, 203, 72), (17, 64, 96)])
def test_gemm_tcgen05_fused_silu_mul(ops, M, F, K):
    """Interleaved gate/up rows: the epilogue writes up * silu(gate)."""
    g = torch.Generator().manual_seed(M + F)
    a = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    gate = torch.randn(F, K, generator=g).to(torch.bfloat16).to(DEV)
    up = torch.randn(F, K, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.stack([gate, up], dim=1).reshape(2 * F, K).contiguous()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    out = torch.full((M, F), float("nan"), dtype=torch.bfloat16, device=DEV)
    ops.gemm_tcgen05(out, a, w, status, epilogue=1)
    gf, uf = a.double() @ gate.double().T, a.double() @ up.double().T
    want = uf * gf * torch.sigmoid(gf)
    err = float((out.double() - want).abs().max())
    assert err <= 1e-4 * math.sqrt(K) * 8 + 2 ** -8 * float(want.abs().max()), err
    assert int(status.item()) == 0


def test_gemm_tcgen05_refuses(ops):
    from socrates_b200.kernels import KernelError
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    a = torch.zeros(4, 20, dtype=torch.bfloat16, device=DEV)
    w = torch.zeros(8, 20, dtype=torch.bfloat16, device=DEV)
    with pytest.raises(KernelError, match="multiple of 8"):
        ops.gemm_tcgen05(torch.empty(4, 8, dtype=torch.float32, device=DEV), a, w, status)
    with pytest.raises(KernelError):
        ops.gemm_tcgen05(torch.empty(4, 8, device=DEV), a.float(), w, status)
