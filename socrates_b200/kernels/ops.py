"""Typed Python entry points of the CUDA kernels.

Each function checks device, dtype, shape and contiguity of its tensors, then calls
the C entry point with raw pointers on torch's current stream.  Outputs are written
into tensors the caller passes: nothing here allocates, so every call can be
recorded in a CUDA graph.  (The reference performs the same checks in C++,
model/kernels/csrc/ops.cpp:29-72.)
"""

from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch

from .library import KernelError, check, library

DTYPE_CODE = {torch.float32: 0, torch.bfloat16: 1}


def _code(dtype: torch.dtype) -> int:
    try:
        return DTYPE_CODE[dtype]
    except KeyError:
        raise KernelError(f"dtype {dtype} is not supported; float32 and bfloat16 are") from None


def _ptr(t: Optional[torch.Tensor]):
    """The tensor's device address as ctypes takes it for a pointer argument (an int; None = null)."""
    return None if t is None else t.data_ptr()


_scoped_stream = None      # the stream handle inside a stream_scope, else None


class stream_scope:
    """Inside the scope every kernel of this module goes to the stream that was current when the
    scope was entered, looked up once.  `torch.cuda.current_stream()` costs several microseconds a
    call, which with some 330 launches was a quarter of the host's time for a step; a step's
    kernels all go to one stream anyway.  The caller must not switch streams inside the scope."""

    def __enter__(self):
        global _scoped_stream
        self._outer = _scoped_stream
        _scoped_stream = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _scoped_stream
        _scoped_stream = self._outer
        return False


def _stream():
    return _scoped_stream if _scoped_stream is not None else torch.cuda.current_stream().cuda_stream


def _want(t: torch.Tensor, name: str, dtype=None, shape=None) -> None:
    if not t.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if not t.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {t.dtype}")
    if shape is not None and t.shape != shape:              # torch.Size compares with tuples
        raise KernelError(f"{name} must have shape {tuple(shape)}, got {tuple(t.shape)}")


def embed(out: torch.Tensor, table: torch.Tensor, ids: torch.Tensor,
          feedback: Optional[torch.Tensor] = None) -> None:
    """out[n, :] = float32(table[ids[n], :]); out float32 [N, d], ids int32 [N].
    With `feedback` (int32, on the device) an id -1 - j stands for feedback[j]: a token that an
    earlier kernel on the stream wrote."""
    V, d = table.shape
    N = ids.numel()
    _want(table, "table")
    _want(ids, "ids", torch.int32)
    _want(out, "out", torch.float32, (N, d))
    if feedback is not None:
        _want(feedback, "feedback", torch.int32)
    lib = library()
    check(lib, lib.sb_embed(_ptr(out), _ptr(table), _ptr(ids), N, d, V, _code(table.dtype), _ptr(feedback),
                            _stream()), "embed")


def add_rmsnorm(residual: torch.Tensor, delta: Optional[torch.Tensor], gain: torch.Tensor,
                out: torch.Tensor, eps: float, row_index: Optional[torch.Tensor] = None) -> None:
    """residual += sum(delta, 0); out = rmsnorm(residual) * gain.

    residual float32 [N, d]; delta float32 [S, N, d] or None; gain float32 [d];
    out [M, d] in the model dtype, M = len(row_index) or N.  With row_index only the
    named rows are normed and the residual is left as it is.
    """
    N, d = residual.shape
    _want(residual, "residual", torch.float32)
    _want(gain, "gain", torch.float32, (d,))
    S, stride = 0, 0
    if delta is not None:
        _want(delta, "delta", torch.float32)
        if delta.dim() != 3 or delta.shape[1:] != (N, d):
            raise KernelError(f"delta must be [S, {N}, {d}], got {tuple(delta.shape)}")
        S, stride = delta.shape[0], N * d
    M = N
    if row_index is not None:
        _want(row_index, "row_index", torch.int32)
        M = row_index.numel()
    _want(out, "out", None, (M, d))
    lib = library()
    check(lib, lib.sb_add_rmsnorm(_ptr(residual), _ptr(delta), S, stride, _ptr(gain), _ptr(out),
                                  _ptr(row_index), M, d, float(eps), _code(out.dtype), _stream()),
          "add_rmsnorm")


def qk_norm_rope_kvwrite(qkv: torch.Tensor, q_out: torch.Tensor, k_pool: Optional[torch.Tensor],
                         v_pool: Optional[torch.Tensor], q_gain: Optional[torch.Tensor],
                         k_gain: Optional[torch.Tensor], inv_freq: torch.Tensor, rotary_dim: int,
                         positions: torch.Tensor, token_rows: torch.Tensor, block_table: torch.Tensor,
                         eps: float, num_heads: int, num_kv_heads: int, head_dim: int) -> None:
    """Per-head norm, rotation and paged KV write for N tokens.

    qkv [N, (Hq+2Hkv)*D] in the model dtype, or float32 [S, N, (Hq+2Hkv)*D] partial sums
    of a split product (added here); q_out [N, Hq*D]; pools [pages, Hkv, BS, D] (None:
    the keys and values of this step are not stored, the layer reads another layer's cache).
    """
    Hq, Hkv, D = num_heads, num_kv_heads, head_dim
    width = (Hq + 2 * Hkv) * D
    parts = qkv.dim() == 3
    N = qkv.shape[-2]
    if parts:
        _want(qkv, "qkv partial sums", torch.float32, (qkv.shape[0], N, width))
    else:
        _want(qkv, "qkv", q_out.dtype, (N, width))
    _want(q_out, "q_out", None, (N, Hq * D))
    _want(positions, "positions", torch.int32, (N,))
    _want(token_rows, "token_rows", torch.int32, (N,))
    _want(block_table, "block_table", torch.int32)
    _want(inv_freq, "inv_freq", torch.float32)
    if inv_freq.numel() < rotary_dim // 2:
        raise KernelError(f"inv_freq has {inv_freq.numel()} entries for rotary_dim {rotary_dim}")
    write_kv = k_pool is not None
    page_size = 1
    if write_kv:
        _want(k_pool, "k_pool", q_out.dtype)
        _want(v_pool, "v_pool", q_out.dtype, k_pool.shape)
        if k_pool.dim() != 4 or k_pool.shape[1] != Hkv or k_pool.shape[3] != D:
            raise KernelError(f"pools must be [pages, {Hkv}, page_size, {D}], got {tuple(k_pool.shape)}")
        page_size = k_pool.shape[2]
    for g, nm in ((q_gain, "q_gain"), (k_gain, "k_gain")):
        if g is not None:
            _want(g, nm, torch.float32, (D,))
    lib = library()
    check(lib, lib.sb_qk_norm_rope_kvwrite(
        None if parts else _ptr(qkv), _ptr(qkv) if parts else None, qkv.shape[0] if parts else 0,
        N * width, _ptr(q_out), _ptr(k_pool), _ptr(v_pool), _ptr(q_gain), _ptr(k_gain), _ptr(inv_freq),
        rotary_dim, _ptr(positions), _ptr(token_rows), _ptr(block_table), block_table.shape[1],
        page_size, float(eps), Hq, Hkv, D, N, int(write_kv), _code(q_out.dtype), _stream()),
        "qk_norm_rope_kvwrite")


def silu_mul(out: torch.Tensor, gate_up: torch.Tensor, interleaved: bool = False) -> None:
    """out[n, f] = up * silu(gate) with gate = gate_up[n, f], up = gate_up[n, F + f], or, when
    `interleaved`, gate = gate_up[n, 2f], up = gate_up[n, 2f + 1]."""
    N, F2 = gate_up.shape
    _want(gate_up, "gate_up")
    _want(out, "out", gate_up.dtype, (N, F2 // 2))
    lib = library()
    check(lib, lib.sb_silu_mul(_ptr(out), _ptr(gate_up), N, F2 // 2, int(interleaved), _code(out.dtype), _stream()),
          "silu_mul")


def sample_scratch_size(M: int, V: int) -> int:
    """int32 entries of scratch that `sample` needs for M rows of V logits."""
    return M * (2 * library().sb_sample_slices(int(V)) + 1)


def sample(out: torch.Tensor, logits: torch.Tensor, temperature: Optional[torch.Tensor] = None,
           seeds: Optional[torch.Tensor] = None, counters: Optional[torch.Tensor] = None,
           scratch: Optional[torch.Tensor] = None) -> None:
    """out[m] = argmax(logits[m]) where temperature[m] == 0 (or temperature is None),
    else a draw from softmax(logits[m] / temperature[m]) fixed by (seeds[m], counters[m]).

    `scratch`: int32 with at least sample_scratch_size(M, V) entries that were zero before
    its first use (the kernel leaves it ready for the next call); allocated here if None.
    """
    M, V = logits.shape
    _want(logits, "logits", torch.float32)
    _want(out, "out", torch.int32, (M,))
    if temperature is not None:
        _want(temperature, "temperature", torch.float32, (M,))
        _want(seeds, "seeds", torch.int32, (M,))
        _want(counters, "counters", torch.int32, (M,))
    need = sample_scratch_size(M, V)
    if scratch is None:
        scratch = torch.zeros(need, dtype=torch.int32, device=logits.device)
    _want(scratch, "scratch", torch.int32)
    if scratch.numel() < need:
        raise KernelError(f"sample scratch has {scratch.numel()} entries, {need} are needed")
    lib = library()
    check(lib, lib.sb_sample(_ptr(out), _ptr(logits), _ptr(temperature), _ptr(seeds), _ptr(counters),
                             M, V, _ptr(scratch), _stream()), "sample")


def gemm_simt(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, splits: int = 1) -> None:
    """out = a @ w.T on the CUDA cores with float32 accumulation.

    a [M, K], w [N, K]; out [M, N], or float32 [splits, M, N] partial sums.
    """
    M, K = a.shape
    N = w.shape[0]
    _want(a, "a")
    _want(w, "w", None, (N, K))
    if splits == 1 and out.dim() == 2:
        _want(out, "out", None, (M, N))
    else:
        _want(out, "out", torch.float32, (splits, M, N))
    lib = library()
    check(lib, lib.sb_gemm_simt(_ptr(out), _ptr(a), _ptr(w), M, N, K, _code(a.dtype), _code(w.dtype),
                                _code(out.dtype), splits, _stream()), "gemm_simt")


def attention_simt(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                   block_table: torch.Tensor, token_rows: torch.Tensor, positions: torch.Tensor,
                   num_heads: int, scale: float, window: int = 0, num_partitions: int = 1,
                   part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None) -> None:
    """Paged causal attention, one query per token, on the CUDA cores.

    q, out [N, Hq*D]; pools [pages, Hkv, BS, D]; block_table int32 [rows, W];
    window 0 = all keys.  Scratch for num_partitions > 1: part_o float32 with at least
    N*Hq*NP*D elements, part_ml with N*Hq*NP*2.
    """
    N = q.shape[0]
    pages, Hkv, BS, D = k_pool.shape
    Hq = num_heads
    _want(q, "q", k_pool.dtype, (N, Hq * D))
    _want(out, "out", q.dtype, (N, Hq * D))
    _want(k_pool, "k_pool")
    _want(v_pool, "v_pool", k_pool.dtype, k_pool.shape)
    _want(block_table, "block_table", torch.int32)
    _want(token_rows, "token_rows", torch.int32, (N,))
    _want(positions, "positions", torch.int32, (N,))
    if num_partitions > 1:
        _want(part_o, "part_o", torch.float32)
        _want(part_ml, "part_ml", torch.float32)
        if part_o.numel() < N * Hq * num_partitions * D or part_ml.numel() < N * Hq * num_partitions * 2:
            raise KernelError("attention scratch buffers are too small")
    lib = library()
    check(lib, lib.sb_attention_simt(
        _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
        block_table.shape[1], _ptr(token_rows), _ptr(positions), N, Hq, Hkv, D, BS, int(window),
        float(scale), num_partitions, _code(q.dtype), _stream()), "attention",
        kernels=2 if num_partitions > 1 else 1)


def gemm_tcgen05_splits(K: int, splits: int) -> int:
    """How many K parts `gemm_tcgen05` writes when `splits` are asked for (never more)."""
    return library().sb_gemm_tcgen05_splits(int(K), int(splits))


SHARES_VARIANT = 2000      # gemm_tcgen05 variant: the pair kernel dealing equal shares of K blocks


def gemm_tcgen05_shares_parts(M: int, N: int, K: int) -> int:
    """How many float32 parts `gemm_tcgen05(..., variant=SHARES_VARIANT)` writes for this shape: the
    pair kernel (two SMs per 256 x 256 tile) with the tiles' K blocks dealt to the pairs in equal
    shares, a tile that a share's end cuts being finished by the next pair into another part.
    0: the shape is not served (few rows, N below 256, more than four pieces to a tile)."""
    return int(library().sb_gemm_tcgen05_shares_parts(int(M), int(N), int(K)))


def gemm_tcgen05(out: torch.Tensor, a: torch.Tensor, w: torch.Tensor, status: torch.Tensor,
                 splits: int = 1, variant: int = 0, epilogue: int = 0,
                 prefetch: Optional[Tuple[torch.Tensor, int]] = None) -> int:
    """out = a @ w.T on the tcgen05 tensor cores; a [M, K] and w [N, K] bfloat16, K % 8 == 0.

    out is bfloat16 or float32 [M, N], or float32 [S, M, N] partial sums where S =
    gemm_tcgen05_splits(K, splits).  `status` is an int32 device tensor that receives a
    non-zero code if a bounded wait inside the kernel gave up.  Returns S.
    `prefetch`: (tensor, bytes), the leading bytes of the weights that the next product
    streams; the weight-streaming kernel (M <= 64) asks for them in L2 once its own loads
    are issued.
    """
    M, K = a.shape
    N = w.shape[0]
    _want(a, "a", torch.bfloat16)
    _want(w, "w", torch.bfloat16, (N, K))
    _want(status, "status", torch.int32)
    S = gemm_tcgen05_shares_parts(M, N, K) if variant == SHARES_VARIANT else gemm_tcgen05_splits(K, splits)
    if variant == SHARES_VARIANT and (S == 0 or out.dim() != 3):
        raise KernelError(f"the equal-shares kernel does not serve M={M} N={N} K={K} (or out is not [S, M, N])")
    if out.dim() == 2:
        if S != 1:
            raise KernelError("a split product needs a float32 [S, M, N] output")
        _want(out, "out", None, (M, N // 2 if epilogue == 1 else N))
    else:
        _want(out, "out", torch.float32, (S, M, N))
    lib = library()
    s_io = ctypes.c_int(S)
    pf_ptr, pf_bytes = None, 0
    if prefetch is not None and M <= 64:
        tensor, nbytes = prefetch
        if not tensor.is_cuda or not tensor.is_contiguous():
            raise KernelError("a prefetch range must be a contiguous CUDA tensor")
        pf_ptr = tensor.data_ptr()
        pf_bytes = max(0, min(int(nbytes), tensor.numel() * tensor.element_size()))
    check(lib, lib.sb_gemm_tcgen05(_ptr(out), _ptr(a), _ptr(w), M, N, K, _code(out.dtype),
                                   ctypes.byref(s_io), _ptr(status), int(variant), int(epilogue),
                                   pf_ptr, pf_bytes, _stream()),
          "gemm_tcgen05")
    if s_io.value != S:
        raise KernelError(f"gemm_tcgen05 wrote {s_io.value} parts where {S} were expected")
    return S


def attention_mma_supports(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int,
                           decode: bool) -> bool:
    """Whether the tensor-core attention kernels take this shape (bfloat16 only)."""
    return bool(library().sb_attention_mma_supports(num_heads, num_kv_heads, head_dim, page_size,
                                                    int(decode)))


def attention_prefill_mma(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                          block_table: torch.Tensor, seq_starts: torch.Tensor, seq_rows: torch.Tensor,
                          seq_first_pos: torch.Tensor, num_heads: int, scale: float, window: int = 0) -> None:
    """Paged causal attention of prompt portions on the tensor cores (bfloat16).

    Request r brings tokens seq_starts[r] .. seq_starts[r+1]-1 (rows of q and out) at
    positions seq_first_pos[r], +1, ... of cache row seq_rows[r]; its keys, earlier
    portions included, are read from the pages.
    """
    N = q.shape[0]
    _, Hkv, BS, D = k_pool.shape
    R = seq_rows.numel()
    _want(q, "q", torch.bfloat16, (N, num_heads * D))
    _want(out, "out", torch.bfloat16, (N, num_heads * D))
    _want(k_pool, "k_pool", torch.bfloat16)
    _want(v_pool, "v_pool", torch.bfloat16, k_pool.shape)
    _want(block_table, "block_table", torch.int32)
    _want(seq_starts, "seq_starts", torch.int32, (R + 1,))
    _want(seq_rows, "seq_rows", torch.int32, (R,))
    _want(seq_first_pos, "seq_first_pos", torch.int32, (R,))
    lib = library()
    check(lib, lib.sb_attention_prefill_mma(
        _ptr(out), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table), block_table.shape[1],
        _ptr(seq_starts), _ptr(seq_rows), _ptr(seq_first_pos), R, N, num_heads, Hkv, D, BS, int(window),
        float(scale), _stream()), "attention_prefill_mma")


def attention_decode_mma(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                         block_table: torch.Tensor, token_rows: torch.Tensor, positions: torch.Tensor,
                         num_heads: int, scale: float, window: int = 0, num_partitions: int = 1,
                         part_o: Optional[torch.Tensor] = None,
                         part_ml: Optional[torch.Tensor] = None, variant: int = 0) -> None:
    """Paged attention of single decode tokens on the tensor cores (bfloat16), the keys
    of each token cut into `num_partitions` parts; arguments as `attention_simt`.
    `variant` picks the kernel's (warps, stages); 0 is the default.  2 to 4 partitions are
    merged inside the kernel (a thread-block cluster per token and KV head), more by a
    reduce kernel through the scratch buffers.

    The kernel reads the block table, rows, positions and the keys and values below each
    position before it waits for the kernel that precedes it on the stream: those must be
    older than that kernel (a host copy, an earlier step)."""
    N = q.shape[0]
    _, Hkv, BS, D = k_pool.shape
    Hq = num_heads
    _want(q, "q", torch.bfloat16, (N, Hq * D))
    _want(out, "out", torch.bfloat16, (N, Hq * D))
    _want(k_pool, "k_pool", torch.bfloat16)
    _want(v_pool, "v_pool", torch.bfloat16, k_pool.shape)
    _want(block_table, "block_table", torch.int32)
    _want(token_rows, "token_rows", torch.int32, (N,))
    _want(positions, "positions", torch.int32, (N,))
    if num_partitions > 1:
        _want(part_o, "part_o", torch.float32)
        _want(part_ml, "part_ml", torch.float32)
        if part_o.numel() < N * Hq * num_partitions * D or part_ml.numel() < N * Hq * num_partitions * 2:
            raise KernelError("attention scratch buffers are too small")
    lib = library()
    check(lib, lib.sb_attention_decode_mma(
        _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(block_table),
        block_table.shape[1], _ptr(token_rows), _ptr(positions), N, Hq, Hkv, D, BS, int(window),
        float(scale), num_partitions, int(variant), _stream()), "attention_decode_mma",
        kernels=lib.sb_attention_decode_mma_kernels(num_partitions))


def attention_decode_stream_supports(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether the streaming decode kernel takes this shape (bfloat16; head sizes 16 to 128, groups
    of up to 16 query heads, pages of at least 16 slots)."""
    return bool(library().sb_attention_decode_stream_supports(num_heads, num_kv_heads, head_dim, page_size))


def attention_decode_stream(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                            block_table: torch.Tensor, token_rows: torch.Tensor, positions: torch.Tensor,
                            num_heads: int, scale: float, window: int, chunk_keys: int, max_chunks: int,
                            part_o: Optional[torch.Tensor] = None, part_ml: Optional[torch.Tensor] = None,
                            counters: Optional[torch.Tensor] = None, variant: int = 0) -> None:
    """Paged attention of single decode tokens (bfloat16) as one persistent kernel whose warps
    stream fixed chunks of `chunk_keys` keys (a multiple of 16) of each (token, KV head); a row's
    chunks lie at fixed key positions, so its numbers do not depend on the rest of the batch.

    `max_chunks` bounds the chunks the visible keys of any token span.  Scratch for max_chunks > 1:
    part_o float32 with N*Hq*max_chunks*D elements, part_ml with N*Hq*max_chunks*2, and int32
    `counters` with N*Hkv entries that are zero before the first call (the kernel leaves them zero).

    The kernel reads the block table, rows, positions and the keys and values below each
    position before it waits for the kernel that precedes it on the stream: those must be
    older than that kernel (a host copy, an earlier step)."""
    N = q.shape[0]
    _, Hkv, BS, D = k_pool.shape
    Hq = num_heads
    _want(q, "q", torch.bfloat16, (N, Hq * D))
    _want(out, "out", torch.bfloat16, (N, Hq * D))
    _want(k_pool, "k_pool", torch.bfloat16)
    _want(v_pool, "v_pool", torch.bfloat16, k_pool.shape)
    _want(block_table, "block_table", torch.int32)
    _want(token_rows, "token_rows", torch.int32, (N,))
    _want(positions, "positions", torch.int32, (N,))
    if max_chunks > 1:
        _want(part_o, "part_o", torch.float32)
        _want(part_ml, "part_ml", torch.float32)
        _want(counters, "counters", torch.int32)
        if (part_o.numel() < N * Hq * max_chunks * D or part_ml.numel() < N * Hq * max_chunks * 2
                or counters.numel() < N * Hkv):
            raise KernelError("attention scratch buffers are too small")
    lib = library()
    check(lib, lib.sb_attention_decode_stream(
        _ptr(out), _ptr(part_o), _ptr(part_ml), _ptr(counters), _ptr(q), _ptr(k_pool), _ptr(v_pool),
        _ptr(block_table), block_table.shape[1], _ptr(token_rows), _ptr(positions), N, Hq, Hkv, D, BS,
        int(window), float(scale), int(chunk_keys), int(max_chunks), int(variant), _stream()),
        "attention_decode_stream")


def attention_decode_mma_blocks_per_sm(head_dim: int, variant: int = 0) -> int:
    """Blocks of the decode attention kernel that are resident on one SM at a time."""
    return library().sb_attention_decode_mma_blocks_per_sm(int(head_dim), int(variant))


def attention_tcgen05_supports(num_heads: int, num_kv_heads: int, head_dim: int, page_size: int) -> bool:
    """Whether the tcgen05 tile kernel takes this shape (bfloat16, head_dim 64 or 128)."""
    return bool(library().sb_attention_tcgen05_supports(num_heads, num_kv_heads, head_dim, page_size))


def attention_prefill_tcgen05(out: torch.Tensor, q: torch.Tensor, k_pool: torch.Tensor, v_pool: torch.Tensor,
                              block_table: torch.Tensor, seq_starts: torch.Tensor, seq_rows: torch.Tensor,
                              seq_first_pos: torch.Tensor, num_heads: int, scale: float, status: torch.Tensor,
                              window: int = 0) -> None:
    """Paged causal attention of prompt portions on tcgen05 (scores and P.V in tensor
    memory, pages brought in by TMA).  Arguments as `attention_prefill_mma`, plus the int32
    status word that receives a non-zero code if a bounded wait inside the kernel gave up."""
    N = q.shape[0]
    pages, Hkv, BS, D = k_pool.shape
    R = seq_rows.numel()
    _want(q, "q", torch.bfloat16, (N, num_heads * D))
    _want(out, "out", torch.bfloat16, (N, num_heads * D))
    _want(k_pool, "k_pool", torch.bfloat16)
    _want(v_pool, "v_pool", torch.bfloat16, k_pool.shape)
    _want(block_table, "block_table", torch.int32)
    _want(seq_starts, "seq_starts", torch.int32, (R + 1,))
    _want(seq_rows, "seq_rows", torch.int32, (R,))
    _want(seq_first_pos, "seq_first_pos", torch.int32, (R,))
    _want(status, "status", torch.int32)
    lib = library()
    check(lib, lib.sb_attention_prefill_tcgen05(
        _ptr(out), _ptr(q), _ptr(k_pool), _ptr(v_pool), pages, _ptr(block_table), block_table.shape[1],
        _ptr(seq_starts), _ptr(seq_rows), _ptr(seq_first_pos), R, N, num_heads, Hkv, D, BS, int(window),
        float(scale), _ptr(status), _stream()), "attention_prefill_tcgen05")
