"""The decode-attention entry point that allocates nothing (socrates_b200/csrc/no_alloc.h).

It is meant for callers that cannot obtain device memory at call time (a plain C host
program, a loop that must stay out of the allocator, a process whose memory is all
handed out), so this test reaches it the way they do: through the exported C symbol,
with raw pointers.  Its output must equal that of the regular entry point, which takes
its scratch from the caller, on two calls in a row (the second call finds the built-in
scratch array full of the first call's leftovers).  The file sorts last so that a run
that stops at the first failure has already run every other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda"
MAX_FLOATS = 2 * 1024 * 1024


def case(lens, Hq, Hkv, D, seed):
    g = torch.Generator().manual_seed(seed)
    BS = 16
    need = sum(-(-n // BS) for n in lens)
    W = max(-(-n // BS) for n in lens) + 1
    pages = (torch.randperm(need + 3, generator=g) + 1).tolist()
    table = torch.zeros(len(lens), W, dtype=torch.int32)
    for r, n in enumerate(lens):
        for b in range(-(-n // BS)):
            table[r, b] = pages.pop()
    shape = (need + 4, Hkv, BS, D)
    k = torch.randn(shape, generator=g).to(torch.bfloat16).to(DEV)
    v = torch.randn(shape, generator=g).to(torch.bfloat16).to(DEV)
    q = torch.randn(len(lens), Hq * D, generator=g).to(torch.bfloat16).to(DEV)
    rows = torch.arange(len(lens), dtype=torch.int32, device=DEV)
    pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    return q, k, v, table.to(DEV), rows, pos


def call_no_alloc(lib, out, q, k, v, table, rows, pos, Hq, scale, window, NP):
    _, Hkv, BS, D = k.shape
    P = ctypes.c_void_p
    fn = lib.sb_attention_decode_mma_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [P, P, P, P, P, ctypes.c_int, P, P] + [ctypes.c_int] * 6 + [ctypes.c_float, ctypes.c_int, P]
    stream = torch.cuda.current_stream().cuda_stream
    return fn(out.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), table.data_ptr(), table.shape[1],
              rows.data_ptr(), pos.data_ptr(), q.shape[0], Hq, Hkv, D, BS, window, scale, NP, stream)


def test_no_alloc_entry_point_matches_the_regular_one_twice():
    from socrates_b200.kernels import ops, require_kernels
    from socrates_b200.kernels.library import library
    require_kernels()
    lib = library()
    # Two different problems in a row, both with more than four partitions, so that both go
    # through the scratch array (up to four merge inside a thread-block cluster and never
    # touch it): the second finds another problem's (m, l, o) at the same offsets, with other
    # lengths, head counts and head size, and has a one-page row whose later partitions are
    # empty.  A partition slot that a call read without writing it first would show.
    for (lens, Hq, Hkv, D, NP, window, seed) in (([700, 65, 16, 300], 8, 2, 64, 5, 0, 1),
                                                  ([33, 1, 257, 900, 9], 32, 8, 128, 6, 37, 2)):
        q, k, v, table, rows, pos = case(lens, Hq, Hkv, D, seed)
        N = len(lens)
        scale = D ** -0.5
        want = torch.empty_like(q)
        ops.attention_decode_mma(want, q, k, v, table, rows, pos, Hq, scale, window, NP,
                                 torch.empty(N * Hq * NP * D, device=DEV),
                                 torch.empty(N * Hq * NP * 2, device=DEV))
        for _ in range(2):
            got = torch.full_like(q, float("nan"))
            rc = call_no_alloc(lib, got, q, k, v, table, rows, pos, Hq, scale, window, NP)
            assert rc == 0, lib.sb_last_error().decode()
            torch.cuda.synchronize()
            # same kernels, same order of additions: the kernel tests' tolerance is far from needed
            assert torch.allclose(got.float(), want.float(), atol=2e-3, rtol=1.6e-2)
            assert torch.equal(got, want)


def test_no_alloc_entry_point_refuses_more_than_its_scratch():
    from socrates_b200.kernels import require_kernels
    from socrates_b200.kernels.library import library
    require_kernels()
    lib = library()
    lens = [40] * 64
    Hq, Hkv, D = 32, 8, 128
    q, k, v, table, rows, pos = case(lens, Hq, Hkv, D, 3)
    NP = MAX_FLOATS // (64 * Hq * (D + 2)) + 1
    out = torch.zeros_like(q)
    rc = call_no_alloc(lib, out, q, k, v, table, rows, pos, Hq, D ** -0.5, 0, NP)
    assert rc != 0
    assert b"exceed the built-in scratch" in lib.sb_last_error()
    torch.cuda.synchronize()
    assert float(out.float().abs().max()) == 0.0            # nothing was launched
