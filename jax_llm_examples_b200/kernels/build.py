"""Builds the CUDA kernel libraries (sm_100a) and the C++ host library, on first use.

Every ``csrc/<name>.cu`` becomes one shared library ``_build/<name>-<hash>.so`` next to the
package; ``csrc/host/*.cpp`` become ``_build/host-<hash>.so`` with g++ alone.  A library is built
when something first asks for it, so a model compiles what it needs and nothing else; a list of
names is built in parallel.  The hash covers the source, the shared headers and the flags, so an
edited source never meets a stale binary.  While compiling, a line goes to stderr for every
library that starts or finishes and every few seconds in between.

The build folder is inside the checkout (so that the libraries in use are the in-tree ones); if
that is not writable, a per-user folder under the system's temporary directory is used.
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

CSRC = Path(__file__).resolve().parent.parent / "csrc"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared",
]
HOST_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-shared"]

_lock = threading.Lock()
_built: dict[str, Path] = {}


class KernelBuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[jax_llm_examples_b200 build] {msg}", file=sys.stderr, flush=True)


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).is_file():
            return cand
    raise KernelBuildError("nvcc was not found (PATH, $NVCC, /usr/local/cuda/bin): the CUDA kernels cannot be built, "
                           "and there is no fallback path")


_build_dir: Path | None = None


def build_dir() -> Path:
    """Chosen once per process (the probe below must not race between compile threads)."""
    global _build_dir
    if _build_dir is None:
        _build_dir = _choose_build_dir()
    return _build_dir


def _choose_build_dir() -> Path:
    d = Path(os.environ.get("JLX_B200_BUILD_DIR", CSRC.parent / "_build"))
    try:
        d.mkdir(parents=True, exist_ok=True)
        probe = d / f".w{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return d
    except OSError:
        d = Path(tempfile.gettempdir()) / f"jax_llm_examples_b200_build_{os.getuid()}"
        d.mkdir(parents=True, exist_ok=True)
        return d


def _hash(files: list[Path], flags: list[str]) -> str:
    h = hashlib.sha256()
    for f in files:
        h.update(f.name.encode())
        h.update(f.read_bytes())
    h.update(" ".join(flags).encode())
    return h.hexdigest()[:16]


def _headers() -> list[Path]:
    return sorted(CSRC.glob("*.cuh")) + sorted(CSRC.glob("*.h"))


def _target(name: str) -> tuple[Path, list[str]]:
    if name == "host":
        srcs = sorted((CSRC / "host").glob("*.cpp"))
        hdrs = sorted((CSRC / "host").glob("*.h"))
        out = build_dir() / f"host-{_hash(srcs + hdrs, HOST_FLAGS)}.so"
        return out, ["g++", *HOST_FLAGS, "-o", str(out) + ".tmp", *map(str, srcs)]
    src = CSRC / f"{name}.cu"
    if not src.is_file():
        raise KernelBuildError(f"no kernel source {src}")
    extra = os.environ.get("JLX_B200_NVCC_EXTRA", "").split()
    out = build_dir() / f"{name}-{_hash([src] + _headers(), NVCC_FLAGS + extra)}.so"
    return out, [_nvcc(), *NVCC_FLAGS, *extra, "-I", str(CSRC), "-o", str(out) + ".tmp", str(src)]


def _compile(name: str) -> Path:
    out, cmd = _target(name)
    if out.is_file():
        return out
    tmp = Path(str(out) + ".tmp")
    # a unique temporary name per process, so that two processes building at once do not collide
    tmp_unique = Path(f"{out}.{os.getpid()}.tmp")
    cmd = [c if c != str(tmp) else str(tmp_unique) for c in cmd]
    t0 = time.time()
    _say(f"compiling {name} ...")
    proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    while True:
        try:
            output, _ = proc.communicate(timeout=10)
            break
        except subprocess.TimeoutExpired:
            _say(f"still compiling {name} ({time.time() - t0:.0f} s)")
    if proc.returncode != 0:
        tmp_unique.unlink(missing_ok=True)
        raise KernelBuildError(f"building {name} failed:\n{' '.join(cmd)}\n{output}")
    os.replace(tmp_unique, out)
    _say(f"built {name} in {time.time() - t0:.1f} s")
    return out


def ensure_built(names: list[str] | tuple[str, ...]) -> dict[str, Path]:
    """Builds the named libraries (in parallel) unless they exist; returns their paths."""
    with _lock:
        todo = [n for n in dict.fromkeys(names) if n not in _built]
        if todo:
            build_dir()
            with ThreadPoolExecutor(max_workers=min(len(todo), os.cpu_count() or 4)) as pool:
                for n, path in zip(todo, pool.map(_compile, todo)):
                    _built[n] = path
        return {n: _built[n] for n in names}


def build_source(src: str | Path) -> Path:
    """Builds one .cu file from anywhere (a test's own kernel) with the package's flags and headers."""
    src = Path(src).resolve()
    with _lock:
        key = f"@{src}"
        if key not in _built:
            out = build_dir() / f"{src.stem}-{_hash([src] + _headers(), NVCC_FLAGS)}.so"
            if not out.is_file():
                tmp = Path(f"{out}.{os.getpid()}.tmp")
                cmd = [_nvcc(), *NVCC_FLAGS, "-I", str(CSRC), "-o", str(tmp), str(src)]
                _say(f"compiling {src.name} ...")
                proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
                if proc.returncode != 0:
                    tmp.unlink(missing_ok=True)
                    raise KernelBuildError(f"building {src} failed:\n{' '.join(cmd)}\n{proc.stdout}")
                os.replace(tmp, out)
            _built[key] = out
        return _built[key]


def all_kernel_names() -> list[str]:
    return sorted(p.stem for p in CSRC.glob("*.cu"))


def build_all() -> dict[str, Path]:
    return ensure_built(all_kernel_names() + ["host"])
