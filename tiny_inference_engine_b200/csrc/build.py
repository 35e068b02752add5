"""Compiles the CUDA sources of this folder into one shared library, in the tree, at first use.

nvcc cross-compiles for sm_100a without a GPU, so the same call serves the build check on a
CPU machine and the first run on a B200. Objects and the library live in `csrc/_build/`
(or, if the tree is read-only, in a per-user folder under the system's temporary folder);
a stamp of the sources and flags decides whether anything has to be rebuilt. No network, no
HOME and no torch headers are needed: the kernels take raw pointers.
"""
from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
ARCH_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a"]
NVCC_FLAGS = ["-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden",
              "--expt-relaxed-constexpr", "-Xptxas", "-v"]
LIB_NAME = "libtie_b200_kernels.so"


def _say(msg: str) -> None:
    print(f"[tie-b200 build] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found: the engine's kernels have to be compiled (looked at $NVCC, PATH and "
                       "/usr/local/cuda/bin/nvcc)")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def _stamp(nvcc: str) -> str:
    h = hashlib.sha256()
    for p in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(ARCH_FLAGS + NVCC_FLAGS).encode())
    h.update(nvcc.encode())
    return h.hexdigest()


def build_dir() -> Path:
    d = CSRC / "_build"
    try:
        d.mkdir(exist_ok=True)
        probe = d / f".w{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return d
    except OSError:
        d = Path(tempfile.gettempdir()) / f"tie_b200_build_{os.getuid()}"
        d.mkdir(parents=True, exist_ok=True)
        return d


def _compile_one(nvcc: str, src: Path, obj: Path, log: Path) -> None:
    cmd = [nvcc, *ARCH_FLAGS, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    t0 = time.time()
    r = subprocess.run(cmd, capture_output=True, text=True)
    log.write_text("$ " + " ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
    _say(f"compiled {src.name} in {time.time() - t0:.0f} s")


def build(force: bool = False) -> Path:
    """Returns the path of the up-to-date shared library, compiling what is stale."""
    nvcc = find_nvcc()
    out = build_dir()
    lib, stamp_file = out / LIB_NAME, out / "stamp"
    stamp = _stamp(nvcc)
    with open(out / ".lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        if not force and lib.exists() and stamp_file.exists() and stamp_file.read_text() == stamp:
            return lib
        srcs = sources()
        _say(f"compiling {len(srcs)} CUDA files for sm_100a into {out} (first use; about a minute)")
        t0 = time.time()
        objs = [out / (s.stem + ".o") for s in srcs]
        with ThreadPoolExecutor(max_workers=min(8, len(srcs), os.cpu_count() or 1)) as pool:
            futures = [pool.submit(_compile_one, nvcc, s, o, out / (s.stem + ".log")) for s, o in zip(srcs, objs)]
            for f in futures:
                f.result()
        tmp = out / (LIB_NAME + f".{os.getpid()}.tmp")
        cmd = [nvcc, *ARCH_FLAGS, "-shared", "-o", str(tmp), *map(str, objs), "-lcudart"]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise RuntimeError(f"linking {LIB_NAME} failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, lib)
        stamp_file.write_text(stamp)
        _say(f"built {lib.name} in {time.time() - t0:.0f} s")
        return lib


if __name__ == "__main__":
    print(build(force="--force" in sys.argv))
