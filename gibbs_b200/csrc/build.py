"""Compiles the CUDA sources of this folder for sm_100a with nvcc and links
them into shared libraries that ``gibbs_b200.ops`` loads through ctypes.

The sources include no framework headers, so a library builds in well under a
minute.  Libraries are built on first use, in ``_build/`` beside the sources
(or in a per-user temporary folder when the tree is read-only), and rebuilt
when a source, a header or the flags change.  While nvcc runs, a line is
printed every few seconds so that a first call does not look hung.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent

# library name -> sources.  A model needs "core" always and "tensorcore" when
# it computes in bfloat16; "runtime" holds no kernels: it walks a step's list of operations
# and calls into the other two.
LIBRARIES = {
    "core": ["errors.cu", "elementwise.cu", "gemm_simt.cu", "conv.cu", "attention.cu", "sampling.cu"],
    "tensorcore": ["errors.cu", "gemm_tc.cu", "gemm_tc_decode.cu", "attention_tc.cu", "attention_tcgen05.cu"],
    "runtime": ["errors.cu", "step_plan.cu"],
}

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC,-fvisibility=hidden", "--expt-relaxed-constexpr",
] + os.environ.get("GIBBS_B200_NVCC_FLAGS", "").split()      # e.g. -DGB_DECODE_TRACE for a build that stamps times


class BuildError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[gibbs_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("GIBBS_B200_NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise BuildError("nvcc was not found (PATH, /usr/local/cuda/bin, or set GIBBS_B200_NVCC); "
                     "the CUDA kernels of gibbs_b200 cannot be built")


def build_dir() -> Path:
    d = HERE / "_build"
    try:
        d.mkdir(exist_ok=True)
        probe = d / f".write_probe_{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return d
    except OSError:
        d = Path(tempfile.gettempdir()) / f"gibbs_b200_build_{os.getuid()}"
        d.mkdir(parents=True, exist_ok=True)
        return d


def _fingerprint(sources: list[str]) -> str:
    h = hashlib.sha256(" ".join(NVCC_FLAGS).encode())
    for name in sorted(sources) + sorted(p.name for p in list(HERE.glob("*.cuh")) + list(HERE.glob("*.h"))):
        h.update(name.encode())
        h.update((HERE / name).read_bytes())
    return h.hexdigest()


def library_path(lib: str) -> Path:
    return build_dir() / f"libgibbs_b200_{lib}.so"


def is_current(lib: str) -> bool:
    so = library_path(lib)
    stamp = so.with_suffix(".stamp")
    return so.exists() and stamp.exists() and stamp.read_text() == _fingerprint(LIBRARIES[lib])


def _run(cmd: list[str], what: str) -> None:
    env = dict(os.environ)
    env.setdefault("TMPDIR", tempfile.gettempdir())
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=env)
    if proc.returncode != 0:
        raise BuildError(f"{what} failed:\n$ {' '.join(cmd)}\n{proc.stdout}")


def build(lib: str, force: bool = False, verbose_ptxas: bool = False) -> Path:
    """Build one library if it is missing or stale; return its path."""
    if lib not in LIBRARIES:
        raise BuildError(f"unknown kernel library '{lib}'; known: {sorted(LIBRARIES)}")
    so = library_path(lib)
    if not force and is_current(lib):
        return so
    nvcc = find_nvcc()
    out = build_dir()
    sources = LIBRARIES[lib]
    _log(f"compiling kernel library '{lib}' ({len(sources)} files) for sm_100a into {out}")
    t0 = time.time()
    done = threading.Event()

    def heartbeat():
        while not done.wait(8.0):
            _log(f"  ... still compiling '{lib}' ({time.time() - t0:.0f} s)")

    hb = threading.Thread(target=heartbeat, daemon=True)
    hb.start()
    try:
        objs = []

        def compile_one(src: str) -> Path:
            obj = out / f"{lib}_{Path(src).stem}.{os.getpid()}.o"
            flags = list(NVCC_FLAGS) + (["-Xptxas", "-v"] if verbose_ptxas else [])
            _run([nvcc, *flags, "-I", str(HERE), "-c", str(HERE / src), "-o", str(obj)], f"nvcc {src}")
            _log(f"  compiled {src} ({time.time() - t0:.0f} s)")
            return obj

        with ThreadPoolExecutor(max_workers=min(8, len(sources))) as pool:
            objs = list(pool.map(compile_one, sources))
        tmp_so = out / f"{so.name}.{os.getpid()}.tmp"
        _run([nvcc, "-shared", "-o", str(tmp_so), *map(str, objs), "-lcudart"], f"link {so.name}")
        os.replace(tmp_so, so)      # atomic: a concurrent process never loads a half-written file
        for o in objs:
            o.unlink(missing_ok=True)
        so.with_suffix(".stamp").write_text(_fingerprint(sources))
    finally:
        done.set()
    _log(f"built {so.name} in {time.time() - t0:.0f} s")
    return so


def build_all(force: bool = False) -> list[Path]:
    return [build(lib, force=force) for lib in LIBRARIES]


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
