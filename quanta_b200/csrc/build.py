"""Compile the CUDA sources of this folder for sm_100a into shared libraries and load them.

The sources fall into units (``UNITS``): the kernels every model needs, and one unit per family of
mixers and feed-forwards.  A unit is compiled and loaded when the first of its entry points is
called, so a model's first step builds what that model runs and nothing else; ``build()`` compiles
all of them.  The libraries are plain C ABI (raw device pointers and a stream), compile in seconds per
file with nvcc alone and are loaded with ctypes.  They are built in-tree under ``csrc/_build`` when
that is writable (an already-built library travels with the folder), else under
``$QUANTA_B200_BUILD_DIR`` or a per-user folder of the temporary directory.  Nothing is fetched; a
missing compiler or a failed build raises: there is no fallback path.

A unit's build is reused while the hash of its sources, the shared headers and the flags matches the
one stored beside it.
"""

from __future__ import annotations

import concurrent.futures
import ctypes
import hashlib
import os
import re
import shutil
import subprocess
import sys
import tempfile
import threading
import time
from pathlib import Path

SRC_DIR = Path(__file__).resolve().parent
# unit -> its sources.  A file that calls into another one is in the same unit.
UNITS = {
    "core": ["norm_embed.cu", "grouped_norm.cu", "sampling.cu"],
    "attention": ["rope_cache.cu", "attention_simt.cu", "attention_mma.cu", "attention_tc.cu"],
    "experts": ["moe.cu", "router_gemm_mma.cu", "expert_gemm_tc.cu"],
    "recurrent": ["short_conv.cu", "delta_rule.cu", "gated_delta.cu"],
    "latent": ["latent_attention.cu"],
    "linear_attention": ["gla.cu"],
    "window_attention": ["window_attention.cu"],
    "state_space": ["selective_scan.cu"],
}


def lib_name(unit: str) -> str:
    return f"libquanta_b200_{unit}.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a", "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "--expt-relaxed-constexpr",
]


class KernelBuildError(RuntimeError):
    pass


def _log(msg: str) -> None:
    print(f"[quanta_b200] {msg}", file=sys.stderr, flush=True)


def sources(unit: str | None = None) -> list[Path]:
    names = UNITS[unit] if unit is not None else [n for u in UNITS.values() for n in u]
    return [SRC_DIR / n for n in names]


def _unassigned() -> list[str]:
    known = {n for u in UNITS.values() for n in u}
    return sorted(p.name for p in SRC_DIR.glob("*.cu") if p.name not in known)


def _fingerprint(unit: str) -> str:
    h = hashlib.sha256()
    for p in sorted(sources(unit) + list(SRC_DIR.glob("*.cuh")) + list(SRC_DIR.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    h.update(" ".join(NVCC_FLAGS).encode())
    return h.hexdigest()


_ENTRY = re.compile(r'extern\s+"C"\s+[A-Za-z_][A-Za-z0-9_ ]*?\b(qb_[A-Za-z0-9_]+)\s*\(')


def entry_points() -> dict[str, str]:
    """Entry point -> the unit that defines it, read from the sources."""
    out = {}
    for unit in UNITS:
        for src in sources(unit):
            for name in _ENTRY.findall(src.read_text()):
                out.setdefault(name, unit)
    return out


def _find_nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and Path(cand).exists():
            return cand
    raise KernelBuildError("nvcc not found (looked at $NVCC, PATH, /usr/local/cuda/bin): the CUDA kernels "
                           "cannot be built, and there is no other execution path")


def _writable(d: Path) -> bool:
    try:
        d.mkdir(parents=True, exist_ok=True)
        probe = d / f".probe_{os.getpid()}_{threading.get_ident()}"
        probe.write_text("x")
        probe.unlink()
        return True
    except OSError:
        return False


def build_dir() -> Path:
    env = os.environ.get("QUANTA_B200_BUILD_DIR")
    if env:
        d = Path(env)
        if not _writable(d):
            raise KernelBuildError(f"QUANTA_B200_BUILD_DIR={env} is not writable")
        return d
    d = SRC_DIR / "_build"
    if _writable(d):
        return d
    d = Path(tempfile.gettempdir()) / f"quanta_b200_build_{os.getuid()}"
    if _writable(d):
        return d
    raise KernelBuildError("no writable folder for the kernel build (tried csrc/_build and the temp folder)")


def _up_to_date(d: Path, unit: str, fp: str) -> bool:
    stamp = d / f"fingerprint_{unit}.txt"
    return (d / lib_name(unit)).exists() and stamp.exists() and stamp.read_text().strip() == fp


def build_unit(unit: str, verbose: bool = True, force: bool = False) -> Path:
    """Build (if needed) one unit and return the path of its shared library."""
    if unit not in UNITS:
        raise KernelBuildError(f"no build unit {unit!r}; units: {sorted(UNITS)}")
    fp = _fingerprint(unit)
    # a library built in-tree is used even when the tree itself is read-only
    intree = SRC_DIR / "_build"
    if not force and _up_to_date(intree, unit, fp):
        return intree / lib_name(unit)
    d = build_dir()
    if not force and _up_to_date(d, unit, fp):
        return d / lib_name(unit)
    nvcc = _find_nvcc()
    srcs = sources(unit)
    if verbose:
        _log(f"compiling the {unit} kernels ({len(srcs)} CUDA file(s)) for sm_100a into {d} (first call only)")
    t0 = time.time()
    done = threading.Event()

    def heartbeat():
        while not done.wait(15.0):
            _log(f"still compiling ... {time.time() - t0:.0f} s")

    hb = threading.Thread(target=heartbeat, daemon=True)
    if verbose:
        hb.start()

    def compile_one(src: Path) -> Path:
        obj = d / f"{src.stem}.{os.getpid()}.o"
        cmd = [nvcc, *NVCC_FLAGS, "-I", str(SRC_DIR), "-c", str(src), "-o", str(obj)]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise KernelBuildError(f"nvcc failed on {src.name}:\n{r.stdout}\n{r.stderr}")
        if verbose:
            _log(f"compiled {src.name} ({time.time() - t0:.0f} s)")
        return obj

    objs = []
    try:
        with concurrent.futures.ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
            objs = list(pool.map(compile_one, srcs))
        tmp = d / (lib_name(unit) + f".tmp{os.getpid()}")
        cmd = [nvcc, "-shared", "-o", str(tmp), *[str(o) for o in objs]]
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            raise KernelBuildError(f"link failed:\n{r.stdout}\n{r.stderr}")
        os.replace(tmp, d / lib_name(unit))
        (d / f"fingerprint_{unit}.txt").write_text(fp)
    finally:
        done.set()
        for o in objs:
            try:
                o.unlink()
            except OSError:
                pass
    if verbose:
        _log(f"{unit} kernels built in {time.time() - t0:.0f} s")
    return d / lib_name(unit)


def build(verbose: bool = True, force: bool = False) -> Path:
    """Build every unit (those that are not up to date); returns the folder of the last one."""
    stray = _unassigned()
    if stray:
        raise KernelBuildError(f"CUDA sources that belong to no build unit: {stray}")
    with concurrent.futures.ThreadPoolExecutor(max_workers=len(UNITS)) as pool:
        paths = list(pool.map(lambda u: build_unit(u, verbose=verbose, force=force), UNITS))
    return paths[-1].parent


class _Library:
    """All entry points as attributes; the unit of an entry point is built and loaded at its first use."""

    def __init__(self):
        self._units: dict[str, ctypes.CDLL] = {}
        self._where = entry_points()
        self._lock = threading.Lock()

    def unit(self, unit: str) -> ctypes.CDLL:
        with self._lock:
            if unit not in self._units:
                path = build_unit(unit)
                try:
                    self._units[unit] = ctypes.CDLL(str(path))
                except OSError as e:
                    raise KernelBuildError(f"cannot load {path}: {e}") from e
            return self._units[unit]

    def __getattr__(self, name: str):
        if name.startswith("_"):
            raise AttributeError(name)
        unit = self._where.get(name)
        if unit is None:
            raise AttributeError(f"no kernel entry point {name!r} in {sorted(UNITS)}")
        fn = getattr(self.unit(unit), name)
        setattr(self, name, fn)          # found once: later calls skip this lookup
        return fn


_LIB = None


def load(unit: str | None = None) -> _Library:
    """The kernel library; ``unit`` builds and loads that unit now (the others at their first use)."""
    global _LIB
    if _LIB is None:
        _LIB = _Library()
    if unit is not None:
        _LIB.unit(unit)
    return _LIB
