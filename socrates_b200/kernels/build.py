"""Compile the CUDA sources under `socrates_b200/csrc` for sm_100a into shared libraries.

nvcc is called directly (one process per source file, in parallel, then one link),
so a fresh checkout builds in about a minute and prints a line per file meanwhile.
Libraries are kept under `csrc/_build/` keyed by a hash of the sources and flags; if
that folder cannot be written (a read-only install), a per-user folder under the
system's temporary directory is used instead.

The reference builds one extension ahead of time for sm_86/sm_89
(model/kernels/setup.py:20-40); here the library is built at first use and the only
target is sm_100a.
"""

from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import Iterable, Optional, Sequence

CSRC = Path(__file__).resolve().parent.parent / "csrc"

ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
COMMON_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "--expt-relaxed-constexpr",
                "-Xcompiler", "-fPIC"]

# Sources of the core library, in link order.
CORE_SOURCES = ["errors.cu", "elementwise.cu", "sampling.cu", "gemm_simt.cu", "attention_simt.cu",
                "gemm_tcgen05.cu", "gemm_tcgen05_rows.cu", "attention_mma.cu", "attention_decode.cu",
                "attention_tcgen05.cu"]


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[socrates_b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise BuildError("nvcc was not found (looked at $NVCC, PATH and /usr/local/cuda/bin); "
                     "the CUDA kernels cannot be built")


def _hash(sources: Sequence[Path], flags: Sequence[str]) -> str:
    h = hashlib.sha256()
    for p in sorted([*CSRC.glob("*.cuh"), *CSRC.glob("*.h")]) + list(sources):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def _build_root() -> Path:
    env = os.environ.get("SOCRATES_B200_BUILD_DIR")
    if env:
        root = Path(env)
        root.mkdir(parents=True, exist_ok=True)
        return root
    root = CSRC / "_build"
    try:
        root.mkdir(parents=True, exist_ok=True)
        probe = root / f".probe{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return root
    except OSError:
        root = Path(tempfile.gettempdir()) / f"socrates_b200_build_{os.getuid()}"
        root.mkdir(parents=True, exist_ok=True)
        return root


def _run(cmd: list[str], what: str) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"{what} failed:\n{' '.join(cmd)}\n{proc.stdout}\n{proc.stderr}")


def build_library(name: str, sources: Iterable[str], defines: Optional[dict] = None,
                  libs: Sequence[str] = ()) -> Path:
    """Build `lib<name>.so` from `sources` (file names under csrc/) and return its path.

    Nothing is rebuilt when a library with the same hash of sources, headers, flags
    and defines already exists.
    """
    srcs = [CSRC / s for s in sources]
    for s in srcs:
        if not s.exists():
            raise BuildError(f"{s} does not exist")
    flags = ARCH_FLAGS + COMMON_FLAGS + [f"-D{k}={v}" for k, v in sorted((defines or {}).items())]
    tag = _hash(srcs, flags + list(libs))
    root = _build_root()
    out = root / f"lib{name}-{tag}.so"
    if out.exists():
        return out
    nvcc = find_nvcc()
    work = root / f"obj-{name}-{tag}-{os.getpid()}"
    work.mkdir(parents=True, exist_ok=True)
    t0 = time.time()
    _say(f"compiling {len(srcs)} file(s) for sm_100a into {out.name} (first use only)")

    def compile_one(src: Path) -> Path:
        obj = work / (src.stem + ".o")
        t = time.time()
        _run([nvcc, *flags, "-I", str(CSRC), "-c", str(src), "-o", str(obj)], f"compiling {src.name}")
        _say(f"  {src.name} done in {time.time() - t:.0f}s")
        return obj

    try:
        with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as pool:
            objs = list(pool.map(compile_one, srcs))
        tmp = work / out.name
        _run([nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *[str(o) for o in objs],
              *[f"-l{l}" for l in libs]], f"linking {out.name}")
        os.replace(tmp, out)      # atomic: a concurrent builder sees a whole file or none
        for old in root.glob(f"lib{name}-*.so"):      # earlier builds of other sources
            if old != out:
                try:
                    old.unlink()
                except OSError:
                    pass
    finally:
        shutil.rmtree(work, ignore_errors=True)
    _say(f"built {out.name} in {time.time() - t0:.0f}s")
    return out


def build_core() -> Path:
    return build_library("socrates_b200", CORE_SOURCES)


def build_all() -> list:
    """Every library of the package (what `__graft_entry__.build()` compiles)."""
    return [build_core()]
