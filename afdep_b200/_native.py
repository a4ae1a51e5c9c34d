"""Build and load the sm_100a extension, in-tree and content-addressed.

The native sources under ``csrc/`` are compiled ahead of time into
``afdep_b200/_lib/_afdep_native_<digest>.so`` where ``<digest>`` hashes every source file,
the build flags and the toolchain (torch build, Python ABI, nvcc release).  A matching library is simply imported; otherwise the library is
(re)built under a file lock, so the ranks of one job do not compile concurrently, and
published with an atomic rename.  There is no run-time kernel JIT: shapes are run-time
arguments of a fixed set of kernels.

The reference does the same job with a setuptools subprocess, a cache under ``~/.cache``
and an nvcc JIT behind it (afdep/_build.py:142-278, csrc/jit/compiler.hpp).  Importing this
module does not import torch.
"""

from __future__ import annotations

import fcntl
import functools
import hashlib
import importlib.metadata
import importlib.util
import os
import shutil
import subprocess
import sys
import sysconfig
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

PACKAGE_DIR = Path(__file__).resolve().parent
CSRC = PACKAGE_DIR / "csrc"
LIB_DIR = Path(os.environ.get("AFDEP_CACHE_DIR", PACKAGE_DIR / "_lib"))

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler",
    "-fPIC",
]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wno-deprecated-declarations"]

_loaded = None


def native_sources() -> list[Path]:
    """Every file the library is built from, in a stable order."""
    files = [p for p in CSRC.rglob("*") if p.is_file() and p.suffix in {".cu", ".cpp", ".h", ".hpp", ".cuh"}]
    return sorted(files)


def source_digest() -> str:
    """SHA-256 over names and contents of the native sources and the build flags."""
    h = hashlib.sha256()
    for path in native_sources():
        h.update(str(path.relative_to(CSRC)).encode())
        h.update(b"\0")
        h.update(path.read_bytes())
        h.update(b"\0")
    h.update(" ".join(NVCC_FLAGS + CXX_FLAGS).encode())
    return h.hexdigest()


@functools.lru_cache(maxsize=1)
def _nvcc_version() -> str:
    try:
        out = subprocess.run([resolve_nvcc(), "--version"], capture_output=True, text=True, timeout=30).stdout
        return out.strip().splitlines()[-1] if out.strip() else "unknown"
    except (OSError, RuntimeError, subprocess.SubprocessError):
        return "unavailable"


def toolchain_signature() -> dict:
    """What the binary depends on besides the sources: the torch build it links against (its
    version string, with the CUDA tag, also fixes the C++ ABI of libtorch), the Python ABI of the
    extension module and the nvcc release.  Read without importing torch.  The reference's
    build signature covers the same ground (afdep/_build.py:153-184)."""
    try:
        torch_version = importlib.metadata.version("torch")
    except importlib.metadata.PackageNotFoundError:
        torch_version = "absent"
    return {
        "torch": torch_version,
        "python_abi": sysconfig.get_config_var("SOABI") or sys.version.split()[0],
        "nvcc": _nvcc_version(),
        "arch": "sm_100a",
    }


def build_signature() -> str:
    """SHA-256 over the source digest and the toolchain: a torch, Python or CUDA upgrade
    changes the library's name, so a stale binary is never picked up."""
    h = hashlib.sha256(source_digest().encode())
    for key, value in sorted(toolchain_signature().items()):
        h.update(f"{key}={value}\0".encode())
    return h.hexdigest()


def module_name() -> str:
    return f"_afdep_native_{build_signature()[:16]}"


def library_path() -> Path:
    return LIB_DIR / f"{module_name()}.so"


def resolve_nvcc() -> str:
    """Locate nvcc: explicit override, CUDA_HOME, PATH, then the default install prefix."""
    candidates = []
    if os.environ.get("CUDA_NVCC_EXECUTABLE"):
        candidates.append(os.environ["CUDA_NVCC_EXECUTABLE"])
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            candidates.append(os.path.join(os.environ[var], "bin", "nvcc"))
    found = shutil.which("nvcc")
    if found:
        candidates.append(found)
    candidates.append("/usr/local/cuda/bin/nvcc")
    for c in candidates:
        if os.path.isfile(c) and os.access(c, os.X_OK):
            return c
    raise RuntimeError("nvcc not found; set CUDA_HOME or CUDA_NVCC_EXECUTABLE")


def cuda_home() -> str:
    return str(Path(resolve_nvcc()).resolve().parent.parent)


def _run(cmd: list[str]) -> None:
    proc = subprocess.run(cmd, capture_output=True, text=True)
    if proc.returncode != 0:
        raise RuntimeError("native build step failed:\n  " + " ".join(cmd) + "\n" + proc.stdout + proc.stderr)


def build(verbose: bool = False, force: bool = False) -> Path:
    """Compile every ``.cu``/``.cpp`` for sm_100a and link the extension; returns its path.
    ``force=True`` rebuilds even when a library with the current signature exists."""
    import torch
    from torch.utils import cpp_extension

    target = library_path()
    if target.exists() and not force:
        return target
    LIB_DIR.mkdir(parents=True, exist_ok=True)
    name = module_name()
    with open(LIB_DIR / ".build.lock", "w") as lock:
        fcntl.flock(lock, fcntl.LOCK_EX)
        try:
            if target.exists() and not force:
                return target
            work = LIB_DIR / f"build-{name}-{os.getpid()}"
            work.mkdir(parents=True, exist_ok=True)
            nvcc, home = resolve_nvcc(), cuda_home()
            includes = [str(CSRC / "include"), str(CSRC / "runtime"), os.path.join(home, "include")]
            torch_includes = cpp_extension.include_paths() + [sysconfig.get_paths()["include"]]
            abi = int(getattr(torch._C, "_GLIBCXX_USE_CXX11_ABI", True))
            defines = [f"-DTORCH_EXTENSION_NAME={name}", "-DTORCH_API_INCLUDE_EXTENSION_H", f"-D_GLIBCXX_USE_CXX11_ABI={abi}"]
            jobs = []
            objects = []
            for src in native_sources():
                if src.suffix not in {".cu", ".cpp"}:
                    continue
                obj = work / (src.stem + ".o")
                objects.append(str(obj))
                inc = [f"-I{d}" for d in includes]
                if src.suffix == ".cu":
                    cmd = [nvcc, *NVCC_FLAGS, *inc, "-c", str(src), "-o", str(obj)]
                else:
                    cxx = os.environ.get("CXX", "g++")
                    tinc = [f"-isystem{d}" for d in torch_includes]
                    cmd = [cxx, *CXX_FLAGS, *defines, *inc, *tinc, "-c", str(src), "-o", str(obj)]
                jobs.append(cmd)
            if verbose:
                for cmd in jobs:
                    print(" ".join(cmd), file=sys.stderr)
            with ThreadPoolExecutor(max_workers=int(os.environ.get("MAX_JOBS", "8"))) as pool:
                list(pool.map(_run, jobs))
            torch_lib = os.path.join(os.path.dirname(torch.__file__), "lib")
            tmp = work / f"{name}.so"
            link = [
                os.environ.get("CXX", "g++"),
                "-shared",
                *objects,
                "-o",
                str(tmp),
                f"-L{torch_lib}",
                f"-L{os.path.join(home, 'lib64')}",
                "-lc10",
                "-lc10_cuda",
                "-ltorch_cpu",
                "-ltorch_cuda",
                "-ltorch",
                "-ltorch_python",
                "-lcudart",
                f"-Wl,-rpath,{torch_lib}",
                f"-Wl,-rpath,{os.path.join(home, 'lib64')}",
            ]
            _run(link)
            os.replace(tmp, target)
            shutil.rmtree(work, ignore_errors=True)
            for old in stale_libraries():     # keep the tree (and what travels with it) small
                try:
                    old.unlink()
                except OSError:
                    pass
            return target
        finally:
            fcntl.flock(lock, fcntl.LOCK_UN)


def load_native(allow_build: bool = True):
    """Import the extension, building it first if no library matches the sources."""
    global _loaded
    if _loaded is not None:
        return _loaded
    import torch  # noqa: F401  (the extension links against libtorch)

    path = library_path()
    if not path.exists():
        if not allow_build:
            raise RuntimeError(f"native library {path.name} has not been built; run `python -m afdep_b200 doctor --build`")
        path = build()
    name = module_name()
    spec = importlib.util.spec_from_file_location(name, path)
    module = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(module)
    sys.modules[name] = module
    _loaded = module
    return module


def stale_libraries() -> list[Path]:
    """Libraries in the cache that no longer match the sources."""
    if not LIB_DIR.exists():
        return []
    keep = library_path().name
    return [p for p in LIB_DIR.glob("_afdep_native_*.so") if p.name != keep]
