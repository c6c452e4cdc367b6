"""Builds and loads the CUDA library of the engine (sm_100a only).

All `.cu` files of this folder are compiled by nvcc into one shared library whose entry
points are plain `extern "C"` functions taking device pointers and a stream; Python
calls them through ctypes, so no torch header is compiled and a full build takes well
under a minute.  The library lives in `_build/<hash of the sources>/` beside the
sources when that folder can be written, else under the system's temporary folder; it
is rebuilt only when a source changes.  While compiling, a line is printed to stderr
for every finished file and every few seconds in between.

There is no fallback: without the library (no nvcc, or a failed build) every op raises.
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
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
LIB_NAME = "libtokensprint_b200.so"
NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-lineinfo", "-O3", "-std=c++17",
    "-Xcompiler", "-fPIC",
    "-Xcompiler", "-fvisibility=hidden",
]

# extra flags for tuning builds (for instance -DTS_GEMM_PROBE); they are part of the build's hash
NVCC_FLAGS += os.environ.get("TS_NVCC_EXTRA_FLAGS", "").split()

_lock = threading.Lock()
_library: ctypes.CDLL | None = None


class BuildError(RuntimeError):
    pass


def _say(msg: str) -> None:
    print(f"[tokensprint_b200] {msg}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    candidates = []
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            candidates.append(Path(os.environ[var]) / "bin" / "nvcc")
    candidates.append(Path("/usr/local/cuda/bin/nvcc"))
    for c in candidates:
        if c.is_file():
            return str(c)
    found = shutil.which("nvcc")
    if found:
        return found
    raise BuildError("nvcc was not found (CUDA_HOME, /usr/local/cuda, PATH): the CUDA library cannot be built")


def sources() -> list[Path]:
    return sorted(CSRC.glob("*.cu"))


def source_hash() -> str:
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    for p in sorted(list(CSRC.glob("*.cu")) + list(CSRC.glob("*.cuh")) + list(CSRC.glob("*.h"))):
        h.update(p.name.encode())
        h.update(p.read_bytes())
    return h.hexdigest()[:16]


def _build_root() -> Path:
    in_tree = CSRC / "_build"
    try:
        in_tree.mkdir(exist_ok=True)
        # a name of its own for every caller: variants are built from several threads at once
        fd, probe = tempfile.mkstemp(prefix=".w", dir=in_tree)
        os.close(fd)
        os.unlink(probe)
        return in_tree
    except OSError:
        root = Path(tempfile.gettempdir()) / f"tokensprint_b200-build-{os.getuid()}"
        root.mkdir(parents=True, exist_ok=True)
        return root


def library_path() -> Path:
    """Where the library for the current sources is (or will be)."""
    digest = source_hash()
    in_tree = CSRC / "_build" / digest / LIB_NAME
    if in_tree.is_file():
        return in_tree
    return _build_root() / digest / LIB_NAME


def _compile_one(nvcc: str, src: Path, obj: Path) -> None:
    cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), "-c", str(src), "-o", str(obj)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {src.name}:\n{proc.stdout}\n{proc.stderr}")


def build(force: bool = False) -> Path:
    """Compiles what is missing and returns the library's path."""
    target = library_path()
    if target.is_file() and not force:
        return target
    nvcc = find_nvcc()
    out_dir = target.parent
    out_dir.mkdir(parents=True, exist_ok=True)
    srcs = sources()
    if not srcs:
        raise BuildError(f"no .cu sources in {CSRC}")
    _say(f"compiling {len(srcs)} CUDA files for sm_100a into {out_dir} (first call only)")
    start = time.time()
    done = 0
    stop = threading.Event()

    def ticker() -> None:
        while not stop.wait(8.0):
            _say(f"still compiling: {done}/{len(srcs)} files done after {time.time() - start:.0f} s")

    t = threading.Thread(target=ticker, daemon=True)
    t.start()
    try:
        objs = [out_dir / (s.stem + f".{os.getpid()}.o") for s in srcs]
        with ThreadPoolExecutor(max_workers=min(len(srcs), os.cpu_count() or 2, 8)) as pool:
            futures = [pool.submit(_compile_one, nvcc, s, o) for s, o in zip(srcs, objs)]
            for s, f in zip(srcs, futures):
                f.result()
                done += 1
                _say(f"compiled {s.name} ({done}/{len(srcs)})")
        tmp = out_dir / f".{LIB_NAME}.{os.getpid()}"
        cmd = [nvcc, "-shared", "-gencode", "arch=compute_100a,code=sm_100a", "-o", str(tmp), *map(str, objs)]
        proc = subprocess.run(cmd, capture_output=True, text=True)
        if proc.returncode != 0:
            raise BuildError(f"linking {LIB_NAME} failed:\n{proc.stdout}\n{proc.stderr}")
        os.replace(tmp, target)
        for o in objs:
            try:
                o.unlink()
            except OSError:
                pass
    finally:
        stop.set()
    _say(f"built {target.name} in {time.time() - start:.0f} s")
    return target


def load() -> ctypes.CDLL:
    """The loaded library; built on the first call of a fresh checkout."""
    global _library
    with _lock:
        if _library is None:
            path = build()
            try:
                _library = ctypes.CDLL(str(path))
            except OSError as e:
                raise BuildError(f"cannot load {path}: {e}") from e
        return _library


# ---------------------------------------------------------------------------
# variants: kernels compiled for one value of a size (a head size), each a library of its own,
# built the first time a model needs that size

VARIANTS = CSRC / "variants"
ATTENTION_HEAD_DIMS = tuple(range(16, 257, 16))
_variants: dict[tuple[str, tuple], ctypes.CDLL] = {}


def variant_path(name: str, defines: dict[str, int]) -> Path:
    src = VARIANTS / f"{name}.cu"
    h = hashlib.sha256()
    h.update(" ".join(NVCC_FLAGS).encode())
    h.update(repr(sorted(defines.items())).encode())
    h.update(src.read_bytes())
    for p in sorted(list(CSRC.glob("*.cuh")) + list(VARIANTS.glob("*.cuh")) + list(VARIANTS.glob("*.h"))):
        h.update(p.read_bytes())
    tag = "_".join(f"{k.lower()}{v}" for k, v in sorted(defines.items()))
    rel = Path(h.hexdigest()[:16]) / f"libtokensprint_b200_{name}_{tag}.so"
    in_tree = CSRC / "_build" / rel
    if in_tree.is_file():
        return in_tree
    return _build_root() / rel


def build_variant(name: str, defines: dict[str, int]) -> Path:
    target = variant_path(name, defines)
    if target.is_file():
        return target
    src = VARIANTS / f"{name}.cu"
    if not src.is_file():
        raise BuildError(f"no kernel source {src}")
    nvcc = find_nvcc()
    target.parent.mkdir(parents=True, exist_ok=True)
    what = ", ".join(f"{k}={v}" for k, v in sorted(defines.items()))
    _say(f"compiling {src.name} for {what} (first use of this size only)")
    start = time.time()
    tmp = target.parent / f".{target.name}.{os.getpid()}"
    cmd = [nvcc, *NVCC_FLAGS, "-I", str(CSRC), *[f"-D{k}={v}" for k, v in sorted(defines.items())],
           "-shared", str(src), "-o", str(tmp)]
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise BuildError(f"nvcc failed on {src.name} ({what}):\n{proc.stdout}\n{proc.stderr}")
    os.replace(tmp, target)
    _say(f"built {target.name} in {time.time() - start:.0f} s")
    return target


def load_variant(name: str, defines: dict[str, int]) -> ctypes.CDLL:
    key = (name, tuple(sorted(defines.items())))
    with _lock:
        lib = _variants.get(key)
        if lib is None:
            path = build_variant(name, defines)
            try:
                lib = ctypes.CDLL(str(path))
            except OSError as e:
                raise BuildError(f"cannot load {path}: {e}") from e
            _variants[key] = lib
        return lib


def build_all() -> list[Path]:
    """The main library and every head-size variant of the attention kernel."""
    paths = [build()]
    with ThreadPoolExecutor(max_workers=min(os.cpu_count() or 2, 8)) as pool:
        paths += list(pool.map(lambda d: build_variant("attention_mma", {"TS_HEAD_DIM": d}), ATTENTION_HEAD_DIMS))
    paths.append(build_variant("attention_tcgen05", {"TS_HEAD_DIM": 128}))
    return paths


if __name__ == "__main__":
    if "--all" in sys.argv:
        for path in build_all():
            print(path)
    else:
        print(build(force="--force" in sys.argv))
