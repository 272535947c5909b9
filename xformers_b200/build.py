"""Build recipe of libxfb200.so (the C-ABI library holding every CUDA kernel).

``python -m xformers_b200.build`` compiles ``csrc/*.cu`` for sm_100a with nvcc
and links them into ``csrc/libxfb200.so`` next to the sources, so that the
library is found in-tree.  nvcc cross-compiles without a GPU.
"""

from __future__ import annotations

import concurrent.futures
import hashlib
import os
import shutil
import subprocess
import sys
from pathlib import Path

CSRC = Path(__file__).resolve().parent / "csrc"
LIB = CSRC / "libxfb200.so"
SOURCES = [
    "runtime.cu",
    "merge.cu",
    "decode_splitk.cu",
    "prefill_generic.cu",
    "prefill_sm100_host.cu",
    "prefill_sm100_m256.cu",
    "prefill_sm100_persist.cu",
    "prefill_api.cu",
    "rope_padded.cu",
]
HEADERS = ["internal.h", "ptx.cuh", "prefill_sm100.h", "../../include/xfb200.h"]
NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--use_fast_math",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-fvisibility=hidden",
    # a function that can fall off its end without a return value is an error, not a warning
    "-Xcompiler",
    "-Werror=return-type",
    "-Werror",
    "cross-execution-space-call",
]


def _nvcc() -> str:
    exe = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    if not os.path.exists(exe):
        raise RuntimeError("nvcc not found: libxfb200.so cannot be built")
    return exe


def _stamp() -> str:
    h = hashlib.sha256()
    for name in SOURCES + HEADERS:
        h.update((CSRC / name).read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


def build(force: bool = False, verbose: bool = False, extra_flags=(), out: Path = LIB) -> Path:
    """``extra_flags`` / ``out`` build an experimental variant beside the
    default library (selected at run time with XFB200_LIBRARY)."""
    variant = bool(extra_flags) or Path(out) != LIB
    objdir = CSRC / "build" / (hashlib.sha256(" ".join(extra_flags).encode()).hexdigest()[:8] if variant else "")
    stamp_file = objdir / "stamp"
    stamp = _stamp() + " ".join(extra_flags)
    if not force and Path(out).exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
        return Path(out)
    objdir.mkdir(parents=True, exist_ok=True)
    nvcc = _nvcc()

    def compile_one(src: str) -> Path:
        obj = objdir / (Path(src).stem + ".o")
        cmd = [nvcc, *NVCC_FLAGS, *extra_flags, "-c", str(CSRC / src), "-o", str(obj)]
        if verbose:
            cmd.insert(1, "-Xptxas=-v")
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {src}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            sys.stderr.write(r.stderr)
        return obj

    with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, len(SOURCES))) as ex:
        objs = list(ex.map(compile_one, SOURCES))
    cmd = [nvcc, "-shared", "-o", str(out), *map(str, objs)]
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        raise RuntimeError(f"link failed:\n{r.stdout}\n{r.stderr}")
    stamp_file.write_text(stamp)
    return Path(out)


if __name__ == "__main__":
    defs = [a for a in sys.argv[1:] if a.startswith("-D")]
    outs = [a.split("=", 1)[1] for a in sys.argv[1:] if a.startswith("--out=")]
    print(build(force="--force" in sys.argv, verbose="-v" in sys.argv, extra_flags=tuple(defs), out=Path(outs[0]) if outs else LIB))
