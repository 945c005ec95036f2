"""Each CUDA kernel alone against its plain PyTorch reference, at sizes the tiny
models do not use (widths and vocabularies that are no power of two, head sizes in
steps of 16, group sizes 1 to 8), with needles and poisoned slots where random
numbers would hide a fault."""

import math

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    # float32: a few ulp of sums of a few thousand terms.  bfloat16 outputs are rounded
    # once to 8 bits of mantissa (2^-9 relative); the reference's own kernel test uses
    # atol 2e-3, rtol 1.6e-2 (tests/test_kernel_cuda.py:27).
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-3, rtol=1.6e-2)


def rand(*shape, dtype=torch.float32, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed + sum(shape))
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


@pytest.fixture(scope="module")
def ops():
    from socrates_b200.kernels import ops, require_kernels
    require_kernels()
    return ops


@pytest.fixture(scope="module")
def ref():
    from socrates_b200.kernels import reference
    return reference


# ---------------------------------------------------------------------------- embedding
@pytest.mark.parametrize("dtype", DTYPES)
def test_embed(ops, ref, dtype):
    V, d, N = 301, 72, 19
    table = rand(V, d, dtype=dtype)
    ids = torch.randint(0, V, (N,), dtype=torch.int32, device=DEV)
    ids[0], ids[1] = 0, V - 1
    out = torch.empty(N, d, dtype=torch.float32, device=DEV)
    ops.embed(out, table, ids)
    assert torch.equal(out, ref.embed_ref(table, ids))


# ---------------------------------------------------------------------------- add + rmsnorm
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("d,S", [(72, 0), (200, 1), (2560, 3), (13000, 2)])
def test_add_rmsnorm(ops, ref, dtype, d, S):
    N, eps = 7, 1e-5
    residual = rand(N, d, scale=2.0)
    delta = rand(S, N, d, seed=1) if S else None
    gain = 1 + 0.1 * rand(d, seed=2)
    out = torch.empty(N, d, dtype=dtype, device=DEV)
    want_res, want = ref.add_rmsnorm_ref(residual, delta, gain, eps)
    res = residual.clone()
    ops.add_rmsnorm(res, delta, gain, out, eps)
    assert torch.allclose(res, want_res, atol=1e-6, rtol=1e-6)
    assert torch.allclose(out.float(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_add_rmsnorm_selected_rows_leave_residual(ops, ref, dtype):
    N, d = 9, 96
    residual, delta, gain = rand(N, d), rand(2, N, d, seed=3), 1 + 0.1 * rand(d, seed=4)
    idx = torch.tensor([8, 0, 3, 3], dtype=torch.int32, device=DEV)
    out = torch.empty(4, d, dtype=dtype, device=DEV)
    res = residual.clone()
    ops.add_rmsnorm(res, delta, gain, out, 1e-6, idx)
    assert torch.equal(res, residual)
    _, want = ref.add_rmsnorm_ref(residual, delta, gain, 1e-6, idx)
    assert torch.allclose(out.float(), want, **tol(dtype))


# ---------------------------------------------------------------------------- silu * mul
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("F", [355, 360, 96])
def test_silu_mul(ops, ref, dtype, F):
    N = 13
    gu = rand(N, 2 * F, dtype=dtype, scale=3.0)
    out = torch.empty(N, F, dtype=dtype, device=DEV)
    ops.silu_mul(out, gu)
    assert torch.allclose(out.float(), ref.silu_mul_ref(gu), **tol(dtype))
    inter = torch.stack([gu[:, :F], gu[:, F:]], dim=2).reshape(N, 2 * F).contiguous()
    out2 = torch.empty_like(out)
    ops.silu_mul(out2, inter, interleaved=True)
    assert torch.equal(out2, out)


# ---------------------------------------------------------------------------- matrix product
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M,N,K", [(1, 40, 24), (5, 130, 72), (77, 200, 333), (130, 65, 1000)])
def test_gemm_simt(ops, ref, dtype, M, N, K):
    a, w = rand(M, K, dtype=dtype), rand(N, K, dtype=dtype, seed=1)
    want = ref.gemm_ref(a, w)
    out = torch.empty(M, N, dtype=dtype, device=DEV)
    ops.gemm_simt(out, a, w)
    t = tol(dtype)
    assert torch.allclose(out.double(), want, atol=t["atol"] * math.sqrt(K), rtol=t["rtol"])
    out32 = torch.empty(M, N, dtype=torch.float32, device=DEV)
    ops.gemm_simt(out32, a, w)
    assert torch.allclose(out32.double(), want, atol=2e-5 * math.sqrt(K), rtol=2e-5)
    parts = torch.empty(3, M, N, dtype=torch.float32, device=DEV)
    ops.gemm_simt(parts, a, w, splits=3)
    assert torch.allclose(parts.sum(0).double(), want, atol=2e-5 * math.sqrt(K), rtol=2e-5)


def test_gemm_simt_mixed_weight_dtype(ops, ref):
    a, w = rand(6, 100, dtype=torch.bfloat16), rand(50, 100, dtype=torch.float32, seed=1)
    out = torch.empty(6, 50, dtype=torch.float32, device=DEV)
    ops.gemm_simt(out, a, w)
    assert torch.allclose(out.double(), ref.gemm_ref(a, w), atol=2e-4, rtol=2e-5)


# ---------------------------------------------------------------------------- qk-norm, rotation, KV write
def paged_case(rows_len, BS, Hkv, D, dtype, spare=5, seed=0):
    """Shuffled pages for rows of the given lengths; returns pools, table, owner map."""
    g = torch.Generator().manual_seed(seed)
    W = max(-(-n // BS) for n in rows_len) + 1
    need = sum(-(-n // BS) for n in rows_len)
    pages = (torch.randperm(need + spare, generator=g) + 1).tolist()
    table = torch.zeros(len(rows_len), W, dtype=torch.int32)
    for r, n in enumerate(rows_len):
        for b in range(-(-n // BS)):
            table[r, b] = pages.pop()
    shape = (need + spare + 1, Hkv, BS, D)
    k = (torch.randn(shape, generator=g)).to(dtype).to(DEV)
    v = (torch.randn(shape, generator=g)).to(dtype).to(DEV)
    return k, v, table.to(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hkv,D,R", [(6, 3, 48, 48), (5, 5, 16, 16), (8, 1, 128, 64), (4, 2, 80, 0),
                                        (4, 2, 128, 128), (6, 2, 64, 64), (2, 1, 256, 256), (4, 4, 128, 0)])
def test_qk_norm_rope_kvwrite(ops, ref, dtype, Hq, Hkv, D, R):
    BS, eps = 16, 1e-5
    lens = [33, 16, 5]
    k_pool, v_pool, table = paged_case(lens, BS, Hkv, D, dtype)
    k0, v0 = k_pool.clone(), v_pool.clone()
    # tokens: the last 3 positions of row 0, all of row 2, position 15 of row 1 (a page's last slot)
    rows = [0, 0, 0] + [2] * 5 + [1]
    pos = [30, 31, 32] + list(range(5)) + [15]
    N = len(rows)
    token_rows = torch.tensor(rows, dtype=torch.int32, device=DEV)
    positions = torch.tensor(pos, dtype=torch.int32, device=DEV)
    qkv = rand(N, (Hq + 2 * Hkv) * D, dtype=dtype, seed=5)
    qg, kg = 1 + 0.1 * rand(D, seed=6), 1 + 0.1 * rand(D, seed=7)
    inv_freq = (1.0 / (1e4 ** (torch.arange(0, max(R, 2), 2).float() / max(R, 2)))).to(DEV)
    q_out = torch.empty(N, Hq * D, dtype=dtype, device=DEV)
    ops.qk_norm_rope_kvwrite(qkv, q_out, k_pool, v_pool, qg, kg, inv_freq, R, positions, token_rows,
                             table, eps, Hq, Hkv, D)
    q, k, v = ref.qk_norm_rope_ref(qkv, qg, kg, inv_freq, R, positions, eps, Hq, Hkv, D)
    assert torch.allclose(q_out.float().view(N, Hq, D), q, **tol(dtype))
    page, off = ref.kv_slots(table, token_rows, positions, BS)
    assert torch.allclose(k_pool[page, :, off].float(), k, **tol(dtype))
    assert torch.allclose(v_pool[page, :, off].float(), v.to(dtype).float())
    # nothing else in the pools changed
    mask = torch.ones(k_pool.shape[0], BS, dtype=torch.bool, device=DEV)
    mask[page, off] = False
    assert torch.equal(k_pool.transpose(1, 2)[mask], k0.transpose(1, 2)[mask])
    assert torch.equal(v_pool.transpose(1, 2)[mask], v0.transpose(1, 2)[mask])
    # without pools only q is produced
    q2 = torch.empty_like(q_out)
    ops.qk_norm_rope_kvwrite(qkv, q2, None, None, qg, kg, inv_freq, R, positions, token_rows, table,
                             eps, Hq, Hkv, D)
    assert torch.equal(q2, q_out)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("D", [32, 128])
def test_qk_norm_rope_from_partial_sums(ops, ref, dtype, D):
    """The split-K partial sums of the QKV product are added inside the kernel."""
    Hq, Hkv, BS, S = 4, 2, 16, 5
    k_pool, v_pool, table = paged_case([20], BS, Hkv, D, dtype)
    N = 6
    token_rows = torch.zeros(N, dtype=torch.int32, device=DEV)
    positions = torch.arange(14, 20, dtype=torch.int32, device=DEV)
    parts = rand(S, N, (Hq + 2 * Hkv) * D, seed=8)
    qg, kg = 1 + 0.1 * rand(D, seed=6), 1 + 0.1 * rand(D, seed=7)
    inv_freq = (1.0 / (1e4 ** (torch.arange(0, D, 2).float() / D))).to(DEV)
    q_out = torch.empty(N, Hq * D, dtype=dtype, device=DEV)
    ops.qk_norm_rope_kvwrite(parts, q_out, k_pool, v_pool, qg, kg, inv_freq, D, positions, token_rows, table,
                             1e-6, Hq, Hkv, D)
    total = parts[0]
    for s in range(1, S):
        total = total + parts[s]
    q, k, v = ref.qk_norm_rope_ref(total, qg, kg, inv_freq, D, positions, 1e-6, Hq, Hkv, D)
    page, off = ref.kv_slots(table, token_rows, positions, BS)
    assert torch.allclose(q_out.float().view(N, Hq, D), q, **tol(dtype))
    assert torch.allclose(k_pool[page, :, off].float(), k, **tol(dtype))
    assert torch.allclose(v_pool[page, :, off].float(), v, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hkv,D,R,partial", [(5, 3, 128, 128, False), (7, 1, 64, 64, False), (4, 2, 256, 256, False),
                                                (6, 3, 128, 0, False), (5, 1, 128, 128, True)])
def test_qk_norm_rope_kvwrite_many_tokens(ops, ref, dtype, Hq, Hkv, D, R, partial):
    """So many tokens that the kernel with half a warp per head runs (prompt portions): odd head
    counts, so that the two heads of a warp are a query and a key, a key and a value, or one
    head and nothing; all rotating or none; from split-K partial sums too."""
    BS, eps, n = 16, 1e-5, 1500
    k_pool, v_pool, table = paged_case([n], BS, Hkv, D, dtype)
    k0, v0 = k_pool.clone(), v_pool.clone()
    N = n - 20                                               # positions 20 .. n-1 of row 0
    token_rows = torch.zeros(N, dtype=torch.int32, device=DEV)
    positions = torch.arange(20, n, dtype=torch.int32, device=DEV)
    width = (Hq + 2 * Hkv) * D
    if partial:
        parts = rand(3, N, width, seed=5)
        src, total = parts, parts[0] + parts[1] + parts[2]
    else:
        src = total = rand(N, width, dtype=dtype, seed=5)
    qg, kg = 1 + 0.1 * rand(D, seed=6), 1 + 0.1 * rand(D, seed=7)
    inv_freq = (1.0 / (1e4 ** (torch.arange(0, max(R, 2), 2).float() / max(R, 2)))).to(DEV)
    q_out = torch.full((N, Hq * D), float("nan"), dtype=dtype, device=DEV)
    ops.qk_norm_rope_kvwrite(src, q_out, k_pool, v_pool, qg, kg, inv_freq, R, positions, token_rows,
                             table, eps, Hq, Hkv, D)
    q, k, v = ref.qk_norm_rope_ref(total, qg, kg, inv_freq, R, positions, eps, Hq, Hkv, D)
    assert torch.allclose(q_out.float().view(N, Hq, D), q, **tol(dtype))
    page, off = ref.kv_slots(table, token_rows, positions, BS)
    assert torch.allclose(k_pool[page, :, off].float(), k, **tol(dtype))
    assert torch.allclose(v_pool[page, :, off].float(), v.to(dtype).float(), **tol(dtype))
    mask = torch.ones(k_pool.shape[0], BS, dtype=torch.bool, device=DEV)
    mask[page, off] = False
    assert torch.equal(k_pool.transpose(1, 2)[mask], k0.transpose(1, 2)[mask])
    assert torch.equal(v_pool.transpose(1, 2)[mask], v0.transpose(1, 2)[mask])
    q2 = torch.full_like(q_out, float("nan"))
    ops.qk_norm_rope_kvwrite(src, q2, None, None, qg, kg, inv_freq, R, positions, token_rows, table,
                             eps, Hq, Hkv, D)
    assert torch.equal(q2, q_out)


def test_rotation_far_positions_float32(ops, ref):
    """Angles are float32(position) * inv_freq; at position 8191 a sloppy sine shows."""
    Hq, Hkv, D = 2, 1, 64
    positions = torch.tensor([0, 1, 4095, 8191], dtype=torch.int32, device=DEV)
    rows = torch.zeros(4, dtype=torch.int32, device=DEV)
    table = torch.zeros(1, 512, dtype=torch.int32, device=DEV)
    qkv = rand(4, (Hq + 2 * Hkv) * D)
    inv_freq = (1.0 / (1e6 ** (torch.arange(0, D, 2).float() / D))).to(DEV)
    q_out = torch.empty(4, Hq * D, device=DEV)
    ops.qk_norm_rope_kvwrite(qkv, q_out, None, None, None, None, inv_freq, D, positions, rows, table,
                             0.0, Hq, Hkv, D)
    q, _, _ = ref.qk_norm_rope_ref(qkv, None, None, inv_freq, D, positions, 0.0, Hq, Hkv, D)
    assert torch.allclose(q_out.view(4, Hq, D), q, atol=3e-6, rtol=1e-5)


# ---------------------------------------------------------------------------- attention
def attention_case(lens, Hq, Hkv, D, dtype, BS=16, seed=0):
    k_pool, v_pool, table = paged_case(lens, BS, Hkv, D, dtype, seed=seed)
    return k_pool, v_pool, table


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hkv,D,NP", [(4, 2, 16, 1), (8, 1, 64, 3), (6, 6, 32, 2), (12, 3, 128, 5),
                                         (9, 1, 48, 4)])
def test_attention_simt_decode_and_portions(ops, ref, dtype, Hq, Hkv, D, NP):
    lens = [1, 15, 16, 17, 130, 257]
    k_pool, v_pool, table = attention_case(lens, Hq, Hkv, D, dtype)
    # one decode token per row at its last position, plus a portion of row 5 (positions 100..111)
    rows = list(range(len(lens))) + [5] * 12
    pos = [n - 1 for n in lens] + list(range(100, 112))
    N = len(rows)
    token_rows = torch.tensor(rows, dtype=torch.int32, device=DEV)
    positions = torch.tensor(pos, dtype=torch.int32, device=DEV)
    q = rand(N, Hq * D, dtype=dtype, seed=3)
    out = torch.empty_like(q)
    part_o = torch.empty(N * Hq * NP * D, device=DEV)
    part_ml = torch.empty(N * Hq * NP * 2, device=DEV)
    ops.attention_simt(out, q, k_pool, v_pool, table, token_rows, positions, Hq, D ** -0.5, 0, NP,
                       part_o, part_ml)
    want = ref.paged_attention_ref(q, k_pool, v_pool, table, token_rows, positions, Hq, D ** -0.5)
    assert torch.allclose(out.double(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [1, 16, 37, 200])
def test_attention_simt_window(ops, ref, dtype, window):
    Hq, Hkv, D, NP = 4, 2, 32, 3
    lens = [40, 129]
    k_pool, v_pool, table = attention_case(lens, Hq, Hkv, D, dtype, seed=2)
    rows = [0, 0, 1, 1, 1]
    pos = [36, 39, 37, 64, 128]
    token_rows = torch.tensor(rows, dtype=torch.int32, device=DEV)
    positions = torch.tensor(pos, dtype=torch.int32, device=DEV)
    q = rand(5, Hq * D, dtype=dtype, seed=4)
    out = torch.empty_like(q)
    part_o, part_ml = torch.empty(5 * Hq * NP * D, device=DEV), torch.empty(5 * Hq * NP * 2, device=DEV)
    ops.attention_simt(out, q, k_pool, v_pool, table, token_rows, positions, Hq, D ** -0.5, window, NP,
                       part_o, part_ml)
    want = ref.paged_attention_ref(q, k_pool, v_pool, table, token_rows, positions, Hq, D ** -0.5, window)
    assert torch.allclose(out.double(), want, **tol(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("needle", [0, 15, 16, 255, 256, 299])
def test_attention_simt_needle(ops, dtype, needle):
    """Zero queries give uniform weights; V is zero except one slot, so the output is
    exactly marker/n if that slot is read once and 0 if it is skipped
    (the reference's needle test, tests/test_kernel_cuda.py:70-107)."""
    Hq, Hkv, D, n = 4, 2, 32, 300
    k_pool, v_pool, table = attention_case([n], Hq, Hkv, D, dtype, seed=9)
    v_pool.zero_()
    page, off = int(table[0, needle // 16]), needle % 16
    v_pool[page, :, off, :] = 8.0
    q = torch.zeros(1, Hq * D, dtype=dtype, device=DEV)
    token_rows = torch.zeros(1, dtype=torch.int32, device=DEV)
    positions = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
    for NP in (1, 4):
        out = torch.empty_like(q)
        part_o, part_ml = torch.empty(Hq * NP * D, device=DEV), torch.empty(Hq * NP * 2, device=DEV)
        ops.attention_simt(out, q, k_pool, v_pool, table, token_rows, positions, Hq, 1.0, 0, NP, part_o, part_ml)
        assert torch.allclose(out.float(), torch.full_like(out, 8.0 / n, dtype=torch.float32), rtol=1e-2 if dtype == torch.bfloat16 else 1e-5)
    # a query one position before the needle must not see it
    if needle > 0:
        positions = torch.tensor([needle - 1], dtype=torch.int32, device=DEV)
        out = torch.ones_like(q)
        ops.attention_simt(out, q, k_pool, v_pool, table, token_rows, positions, Hq, 1.0, 0, 1)
        assert float(out.abs().max()) == 0.0


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_simt_far_key_stands_out(ops, ref, dtype):
    """One far key is made to match the query; the output must be its value row."""
    Hq, Hkv, D, n = 2, 1, 64, 700
    k_pool, v_pool, table = attention_case([n], Hq, Hkv, D, dtype, seed=11)
    q = rand(1, Hq * D, dtype=dtype, seed=12)
    far = 3
    page, off = int(table[0, 0]), far
    k_pool[page, 0, off, :] = (q.view(Hq, D)[0].float() * 4).to(dtype)     # score ~ 4*|q|^2*scale >> others
    token_rows = torch.zeros(1, dtype=torch.int32, device=DEV)
    positions = torch.tensor([n - 1], dtype=torch.int32, device=DEV)
    out = torch.empty_like(q)
    NP = 6
    part_o, part_ml = torch.empty(Hq * NP * D, device=DEV), torch.empty(Hq * NP * 2, device=DEV)
    ops.attention_simt(out, q, k_pool, v_pool, table, token_rows, positions, Hq, 1.0, 0, NP, part_o, part_ml)
    want = ref.paged_attention_ref(q, k_pool, v_pool, table, token_rows, positions, Hq, 1.0)
    assert torch.allclose(out.double(), want, **tol(dtype))
    assert torch.allclose(out.view(Hq, D)[0].float(), v_pool[page, 0, off].float(), atol=1e-2)


@pytest.mark.parametrize("dtype", DTYPES)
def test_attention_simt_ignores_poisoned_slots(ops, dtype):
    """Slots past a row's length, pages of other rows and the null page hold inf/NaN:
    the result is bit-identical (tests/test_kernel_cuda.py:120-133)."""
    Hq, Hkv, D = 4, 2, 32
    lens = [21, 50]
    k_pool, v_pool, table = attention_case(lens, Hq, Hkv, D, dtype, seed=5)
    token_rows = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    positions = torch.tensor([20, 49], dtype=torch.int32, device=DEV)
    q = rand(2, Hq * D, dtype=dtype, seed=6)
    NP = 2
    part_o, part_ml = torch.empty(2 * Hq * NP * D, device=DEV), torch.empty(2 * Hq * NP * 2, device=DEV)
    clean = torch.empty_like(q)
    ops.attention_simt(clean, q, k_pool, v_pool, table, token_rows, positions, Hq, D ** -0.5, 0, NP, part_o, part_ml)
    owned = torch.zeros(k_pool.shape[0], 16, dtype=torch.bool, device=DEV)
    for r, n in enumerate(lens):
        for p in range(n):
            owned[int(table[r, p // 16]), p % 16] = True
    for pool, bad in ((k_pool, float("inf")), (v_pool, float("nan"))):
        t = pool.transpose(1, 2)
        t[~owned] = bad
    dirty = torch.empty_like(q)
    ops.attention_simt(dirty, q, k_pool, v_pool, table, token_rows, positions, Hq, D ** -0.5, 0, NP, part_o, part_ml)
    assert torch.equal(clean, dirty)


def test_attention_refuses_bad_sizes(ops):
    from socrates_b200.kernels import KernelError
    k = torch.zeros(4, 2, 16, 24, device=DEV)
    q = torch.zeros(1, 4 * 24, device=DEV)
    z = torch.zeros(1, dtype=torch.int32, device=DEV)
    table = torch.zeros(1, 4, dtype=torch.int32, device=DEV)
    with pytest.raises(KernelError, match="head_dim"):
        ops.attention_simt(torch.empty_like(q), q, k, k, table, z, z, 4, 1.0)
    k = torch.zeros(4, 3, 16, 32, device=DEV)
    q = torch.zeros(1, 4 * 32, device=DEV)
    with pytest.raises(KernelError, match="multiple"):
        ops.attention_simt(torch.empty_like(q), q, k, k, table, z, z, 4, 1.0)
    with pytest.raises(KernelError):
        ops.attention_simt(torch.empty_like(q), q.cpu(), k, k, table, z, z, 4, 1.0)


# ---------------------------------------------------------------------------- sampling
SCRATCH = None


@pytest.fixture(autouse=True)
def _scratch():
    global SCRATCH
    if SCRATCH is None and torch.cuda.is_available():
        SCRATCH = torch.zeros(64 * 1024, dtype=torch.int32, device=DEV)
    yield


def test_sample_large_vocabulary_many_slices(ops):
    """A vocabulary that is cut into several slices per row; the winner sits in each slice in turn."""
    M, V = 7, 151936
    logits = rand(M, V)
    want = []
    for m in range(M):
        i = (m * 25013 + 7) % V
        logits[m, i] = 30.0
        want.append(i)
    logits[3, 5] = 30.0                              # an earlier slice holds an equal value: lowest index wins
    want[3] = min(want[3], 5)
    out = torch.empty(M, dtype=torch.int32, device=DEV)
    for _ in range(3):                               # the scratch counters must be left ready for the next call
        ops.sample(out, logits, scratch=SCRATCH)
        assert out.tolist() == want


def test_sample_greedy_ties_and_sizes(ops):
    M, V = 5, 1337
    logits = rand(M, V)
    logits[1, 700] = logits[1, 200] = 50.0          # tie: the lower index wins
    logits[2, V - 1] = 60.0
    logits[3, 0] = 60.0
    out = torch.empty(M, dtype=torch.int32, device=DEV)
    ops.sample(out, logits)
    want = logits.argmax(-1)
    assert out[1] == 200 and out[2] == V - 1 and out[3] == 0
    assert torch.equal(out.long()[[0, 4]], want[[0, 4]])


def test_sample_temperature_matches_reference_and_is_seeded(ops, ref):
    M, V = 64, 999
    logits = rand(M, V, scale=2.0)
    temperature = torch.full((M,), 0.8, device=DEV)
    temperature[::7] = 0.0
    seeds = torch.arange(M, dtype=torch.int32, device=DEV) * 7919 - 5
    counters = torch.arange(M, dtype=torch.int32, device=DEV) % 5
    out = torch.empty(M, dtype=torch.int32, device=DEV)
    ops.sample(out, logits, temperature, seeds, counters)
    scores = ref.sample_scores_ref(logits.cpu(), temperature.cpu(), seeds.cpu(), counters.cpu())
    want = scores.argmax(-1)
    got = out.cpu().long()
    for m in range(M):
        if got[m] != want[m]:           # float32 log against float64: only a near-tie may differ
            assert abs(float(scores[m, got[m]] - scores[m, want[m]])) < 1e-4
    assert (got == want).float().mean() > 0.95
    again = torch.empty_like(out)
    ops.sample(again, logits, temperature, seeds, counters)
    assert torch.equal(out, again)
    # a row's draw does not depend on its place in the batch
    perm = torch.randperm(M, device=DEV)
    out_p = torch.empty_like(out)
    ops.sample(out_p, logits[perm].contiguous(), temperature[perm].contiguous(),
               seeds[perm].contiguous(), counters[perm].contiguous())
    assert torch.equal(out_p, out[perm])


def test_sample_temperature_follows_the_distribution(ops):
    V, n = 6, 4000
    logits = torch.tensor([[0.0, 1.0, 2.0, -1.0, 0.5, 1.5]], device=DEV).repeat(n, 1).contiguous()
    T = 0.7
    out = torch.empty(n, dtype=torch.int32, device=DEV)
    ops.sample(out, logits, torch.full((n,), T, device=DEV), torch.full((n,), 11, dtype=torch.int32, device=DEV),
               torch.arange(n, dtype=torch.int32, device=DEV))
    freq = torch.bincount(out.long(), minlength=V).float() / n
    p = torch.softmax(logits[0] / T, 0)
    assert torch.allclose(freq, p, atol=0.03)
