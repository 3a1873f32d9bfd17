"""Compiles the CUDA kernel library and the C++ host module, in-tree, on first use.

Two artefacts are built under ``csrc/_build`` (or under the system temp folder when the
source tree is read-only):

* ``libb200_kernels.so`` from ``csrc/kernels/*.cu`` with ``nvcc`` for sm_100a only; it has a
  plain C interface and is loaded with ``ctypes``.
* ``b200_host`` (a pybind11 extension) from ``csrc/host/*.cpp`` with ``g++``; it needs no
  CUDA and also builds on a machine without a GPU.

A build is keyed by a hash of its sources and flags, protected by a file lock so that
concurrent processes compile once, and reports progress on stderr every few seconds.
"""

from __future__ import annotations

import fcntl
import hashlib
import os
import shutil
import subprocess
import sys
import sysconfig
import tempfile
import threading
import time
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

CSRC = Path(__file__).resolve().parent
KERNEL_DIR = CSRC / "kernels"
HOST_DIR = CSRC / "host"

NVCC_FLAGS = [
    "-gencode",
    "arch=compute_100a,code=sm_100a",
    "-lineinfo",
    "-O3",
    "-std=c++17",
    "--expt-relaxed-constexpr",
    "-Xcompiler",
    "-fPIC",
    "-Xcompiler",
    "-fvisibility=hidden",
]
CXX_FLAGS = ["-O2", "-std=c++20", "-fPIC", "-fvisibility=hidden", "-Wall", "-Wextra"]


class BuildError(RuntimeError):
    pass


def _say(message: str) -> None:
    print(f"[llm_inference_b200 build] {message}", file=sys.stderr, flush=True)


def find_nvcc() -> str:
    candidates = []
    for var in ("CUDA_HOME", "CUDA_PATH"):
        if os.environ.get(var):
            candidates.append(Path(os.environ[var]) / "bin" / "nvcc")
    candidates.append(Path("/usr/local/cuda/bin/nvcc"))
    for candidate in candidates:
        if candidate.is_file():
            return str(candidate)
    found = shutil.which("nvcc")
    if found:
        return found
    raise BuildError("nvcc was not found (looked in CUDA_HOME, /usr/local/cuda/bin and PATH)")


def cuda_include_dir() -> Path:
    return Path(find_nvcc()).resolve().parent.parent / "include"


def build_dir() -> Path:
    """The in-tree build folder, or a per-user temp folder if the tree cannot be written."""
    override = os.environ.get("LLM_INFERENCE_B200_BUILD_DIR")
    if override:
        path = Path(override)
        path.mkdir(parents=True, exist_ok=True)
        return path
    local = CSRC / "_build"
    try:
        local.mkdir(exist_ok=True)
        probe = local / f".write_probe_{os.getpid()}"
        probe.write_text("")
        probe.unlink()
        return local
    except OSError:
        tag = hashlib.sha256(str(CSRC).encode()).hexdigest()[:12]
        path = Path(tempfile.gettempdir()) / f"llm_inference_b200_build_{os.getuid()}_{tag}"
        path.mkdir(parents=True, exist_ok=True)
        return path


def _digest(files: list[Path], flags: list[str]) -> str:
    h = hashlib.sha256()
    for flag in flags:
        h.update(flag.encode())
    for path in sorted(files):
        h.update(path.name.encode())
        h.update(path.read_bytes())
    return h.hexdigest()


class _Progress:
    """Prints a line every few seconds while a long build runs."""

    def __init__(self, what: str, total: int) -> None:
        self.what, self.total, self.done = what, total, 0
        self._stop = threading.Event()
        self._start = time.time()
        self._thread = threading.Thread(target=self._run, daemon=True)

    def _run(self) -> None:
        while not self._stop.wait(5.0):
            _say(
                f"{self.what}: {self.done}/{self.total} files done, "
                f"{time.time() - self._start:.0f} s elapsed"
            )

    def __enter__(self) -> "_Progress":
        _say(f"{self.what}: compiling {self.total} files (first use; cached afterwards)")
        self._thread.start()
        return self

    def __exit__(self, *_: object) -> None:
        self._stop.set()
        self._thread.join()
        _say(f"{self.what}: finished in {time.time() - self._start:.1f} s")


def _run(cmd: list[str]) -> None:
    result = subprocess.run(cmd, capture_output=True, text=True)
    if result.returncode != 0:
        raise BuildError(
            "command failed: " + " ".join(cmd) + "\n" + result.stdout + "\n" + result.stderr
        )


def _locked(path: Path):
    class _Lock:
        def __enter__(self_inner):
            self_inner.handle = open(path, "w")
            fcntl.flock(self_inner.handle, fcntl.LOCK_EX)
            return self_inner

        def __exit__(self_inner, *_: object) -> None:
            fcntl.flock(self_inner.handle, fcntl.LOCK_UN)
            self_inner.handle.close()

    return _Lock()


def _compile_all(
    what: str, sources: list[Path], out: Path, make_cmd, link_cmd, stamp_value: str
) -> None:
    objects = [out.parent / (out.stem + "_" + src.stem + ".o") for src in sources]
    with _Progress(what, len(sources)) as progress:

        def one(pair: tuple[Path, Path]) -> None:
            _run(make_cmd(pair[0], pair[1]))
            progress.done += 1

        with ThreadPoolExecutor(max_workers=min(8, os.cpu_count() or 2)) as pool:
            list(pool.map(one, zip(sources, objects)))
        tmp = out.with_suffix(out.suffix + f".tmp{os.getpid()}")
        _run(link_cmd(objects, tmp))
        os.replace(tmp, out)
    (out.parent / (out.name + ".stamp")).write_text(stamp_value)


def kernel_sources() -> list[Path]:
    return sorted(KERNEL_DIR.glob("*.cu"))


def build_kernels(force: bool = False) -> Path:
    """Build (if stale) and return the path of the CUDA kernel library."""
    sources = kernel_sources()
    headers = sorted(KERNEL_DIR.glob("*.cuh")) + sorted(KERNEL_DIR.glob("*.h"))
    out = build_dir() / "libb200_kernels.so"
    stamp = out.parent / (out.name + ".stamp")
    digest = _digest(sources + headers, NVCC_FLAGS)
    if not force and out.is_file() and stamp.is_file() and stamp.read_text() == digest:
        return out
    with _locked(out.parent / "kernels.lock"):
        if not force and out.is_file() and stamp.is_file() and stamp.read_text() == digest:
            return out
        nvcc = find_nvcc()
        _compile_all(
            "CUDA kernels (sm_100a)",
            sources,
            out,
            lambda src, obj: [nvcc, *NVCC_FLAGS, "-I", str(KERNEL_DIR), "-c", str(src), "-o", str(obj)],
            lambda objs, target: [
                nvcc,
                "-shared",
                "-o",
                str(target),
                *[str(o) for o in objs],
            ],
            digest,
        )
    return out


def host_module_path() -> Path:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    return build_dir() / f"b200_host{suffix}"


def build_host(force: bool = False) -> Path:
    """Build (if stale) and return the path of the C++ host extension module."""
    import pybind11

    sources = sorted(HOST_DIR.glob("*.cpp"))
    headers = sorted(HOST_DIR.glob("*.h"))
    out = host_module_path()
    includes = ["-I", str(HOST_DIR), "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"]]
    digest = _digest(sources + headers, CXX_FLAGS + [sys.version])
    stamp = out.parent / (out.name + ".stamp")
    if not force and out.is_file() and stamp.is_file() and stamp.read_text() == digest:
        return out
    with _locked(out.parent / "host.lock"):
        if not force and out.is_file() and stamp.is_file() and stamp.read_text() == digest:
            return out
        cxx = os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
        if not cxx:
            raise BuildError("no C++ compiler found (g++ / c++)")
        _compile_all(
            "C++ host runtime",
            sources,
            out,
            lambda src, obj: [cxx, *CXX_FLAGS, *includes, "-c", str(src), "-o", str(obj)],
            lambda objs, target: [cxx, "-shared", "-o", str(target), *[str(o) for o in objs]],
            digest,
        )
    return out


def build_all(force: bool = False) -> dict[str, Path]:
    return {"host": build_host(force), "kernels": build_kernels(force)}


if __name__ == "__main__":
    for name, path in build_all(force="--force" in sys.argv).items():
        print(f"{name}: {path}")
