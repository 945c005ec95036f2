"""Load the CUDA library and declare its C entry points.

The library is reached through ctypes: every entry point takes raw device pointers,
sizes and a stream, so it needs no Python or torch headers and builds in seconds.
If the library cannot be built or loaded, `library()` raises: there is no fallback
path (the reference fails at start-up in the same way,
model/kernels/__init__.py:82-92 require_cuda_kernel).
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_longlong, c_void_p
from typing import Optional

from .build import BuildError, build_core


class KernelError(RuntimeError):
    """A kernel refused its arguments or failed to launch."""


_lib: Optional[ctypes.CDLL] = None
_lib_path: Optional[str] = None

P, I, F, LL = c_void_p, c_int, c_float, c_longlong

_SIGNATURES = {
    "sb_abi_version": [],
    "sb_embed": [P, P, P, I, I, I, I, P, P],
    "sb_add_rmsnorm": [P, P, I, LL, P, P, P, I, I, F, I, P],
    "sb_qk_norm_rope_kvwrite": [P, P, I, LL, P, P, P, P, P, P, I, P, P, P, I, I, F, I, I, I, I, I, I, P],
    "sb_silu_mul": [P, P, I, I, I, I, P],
    "sb_sample": [P, P, P, P, P, I, I, P, P],
    "sb_sample_slices": [I],
    "sb_gemm_simt": [P, P, P, I, I, I, I, I, I, I, P],
    "sb_attention_simt": [P, P, P, P, P, P, P, I, P, P, I, I, I, I, I, I, F, I, I, P],
    "sb_gemm_tcgen05": [P, P, P, I, I, I, I, P, P, I, I, P, LL, P],
    "sb_gemm_tcgen05_splits": [I, I],
    "sb_gemm_tcgen05_shares_parts": [I, I, I],
    "sb_attention_mma_supports": [I, I, I, I, I],
    "sb_attention_prefill_mma": [P, P, P, P, P, I, P, P, P, I, I, I, I, I, I, I, F, P],
    "sb_attention_decode_mma": [P, P, P, P, P, P, P, I, P, P, I, I, I, I, I, I, F, I, I, P],
    "sb_attention_decode_mma_blocks_per_sm": [I, I],
    "sb_attention_decode_mma_kernels": [I],
    "sb_attention_decode_stream_supports": [I, I, I, I],
    "sb_attention_decode_stream": [P, P, P, P, P, P, P, P, I, P, P, I, I, I, I, I, I, F, I, I, I, P],
    "sb_attention_tcgen05_supports": [I, I, I, I],
    "sb_attention_prefill_tcgen05": [P, P, P, P, I, P, I, P, P, P, I, I, I, I, I, I, I, F, P, P],
}


def declare(lib: ctypes.CDLL, signatures: dict) -> None:
    for name, argtypes in signatures.items():
        fn = getattr(lib, name)
        fn.argtypes = argtypes
        fn.restype = c_int
    lib.sb_last_error.argtypes = []
    lib.sb_last_error.restype = c_char_p


def library() -> ctypes.CDLL:
    """The loaded CUDA library; built at first call.  Raises if that is not possible."""
    global _lib, _lib_path
    if _lib is None:
        try:
            path = build_core()
            lib = ctypes.CDLL(str(path))
        except (BuildError, OSError) as e:
            raise KernelError(
                f"the socrates_b200 CUDA library is unavailable and there is no fallback: {e}") from e
        declare(lib, _SIGNATURES)
        _lib, _lib_path = lib, str(path)
    return _lib


def library_path() -> Optional[str]:
    return _lib_path


class Counters:
    """Kernels launched through the entry points since import.  A launch recorded into a
    CUDA graph counts once here; every replay launches the same kernels again."""
    launches = 0


def check(lib: ctypes.CDLL, code: int, what: str, kernels: int = 1) -> None:
    Counters.launches += kernels
    if code != 0:
        msg = lib.sb_last_error().decode(errors="replace")
        raise KernelError(f"{what}: {msg} (code {code})")
