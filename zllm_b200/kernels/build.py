"""Builds the CUDA sources of ``zllm_b200/csrc`` for sm_100a with nvcc and loads
them through ctypes.

Each ``<name>.cu`` becomes ``csrc/_build/<name>.so`` (in-tree, so a built tree can be
copied to a machine as it is); a library is rebuilt when its source, a header or
the flags changed.  A kernel group is compiled the first time it is asked for,
so a program compiles what its model and precision need.  While nvcc runs, a
line is printed to stderr every few seconds.  A missing compiler or a failed
build raises BackendError: there is no other path.
"""
from __future__ import annotations

import ctypes
import hashlib
import os
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path
from typing import Dict, Iterable

from ..errors import BackendError

CSRC = Path(__file__).resolve().parent.parent / "csrc"
# precise math is nvcc's default and no fast-math flag is passed: softmax, norms and rotations stay exact float32
NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-lineinfo", "-std=c++17",
              "-shared", "-Xcompiler", "-fPIC", "-Xcompiler", "-fvisibility=hidden"]

_loaded: Dict[str, ctypes.CDLL] = {}
_lock = threading.Lock()


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise BackendError("nvcc not found: the CUDA kernels cannot be built (set NVCC or put it on PATH)")


def _build_dir() -> Path:
    d = CSRC / "_build"
    try:
        d.mkdir(exist_ok=True)
        probe = d / f".w{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return d
    except OSError:
        alt = Path(tempfile.gettempdir()) / f"zllm_b200_build_{os.getuid()}"
        alt.mkdir(parents=True, exist_ok=True)
        return alt


def _digest(src: Path) -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(src.read_bytes())
    for hdr in sorted(CSRC.glob("*.cuh")):
        h.update(hdr.read_bytes())
    return h.hexdigest()[:16]


def _compile(name: str, out: Path, digest: str, verbose: bool) -> None:
    src = CSRC / f"{name}.cu"
    tmp = out.with_suffix(f".tmp{os.getpid()}.so")
    cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), "-o", str(tmp), str(src)]
    t0 = time.time()
    print(f"[zllm_b200] compiling {src.name} for sm_100a ...", file=sys.stderr, flush=True)
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    done = threading.Event()

    def ticker():
        while not done.wait(10.0):
            print(f"[zllm_b200]   still compiling {src.name} ({time.time() - t0:.0f} s)", file=sys.stderr, flush=True)

    th = threading.Thread(target=ticker, daemon=True)
    th.start()
    log, _ = proc.communicate()
    done.set()
    if proc.returncode != 0:
        tmp.unlink(missing_ok=True)
        raise BackendError(f"nvcc failed on {src.name} (exit {proc.returncode}):\n{log}")
    os.replace(tmp, out)
    out.with_suffix(".hash").write_text(digest)
    print(f"[zllm_b200] built {out.name} in {time.time() - t0:.1f} s", file=sys.stderr, flush=True)


def build(names: Iterable[str], verbose: bool = True) -> Dict[str, Path]:
    """Compile the named sources that are out of date (in parallel); returns name -> .so path."""
    bdir = _build_dir()
    todo = []
    paths = {}
    for n in names:
        src = CSRC / f"{n}.cu"
        if not src.exists():
            raise BackendError(f"kernel source {src} is missing")
        out = bdir / f"{n}.so"
        paths[n] = out
        dg = _digest(src)
        hf = out.with_suffix(".hash")
        if not (out.exists() and hf.exists() and hf.read_text() == dg):
            todo.append((n, out, dg))
    errors = []

    def work(item):
        try:
            _compile(item[0], item[1], item[2], verbose)
        except BackendError as e:
            errors.append(e)

    threads = [threading.Thread(target=work, args=(it,)) for it in todo]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    if errors:
        raise errors[0]
    return paths


def load(name: str) -> ctypes.CDLL:
    """The library of ``csrc/<name>.cu``, built first if needed."""
    with _lock:
        lib = _loaded.get(name)
        if lib is None:
            path = build([name])[name]
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as e:
                raise BackendError(f"cannot load {path}: {e}") from e
            _loaded[name] = lib
        return lib


def all_sources():
    return sorted(p.stem for p in CSRC.glob("*.cu"))
