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


# The checked build of the host runtime: AddressSanitizer and UndefinedBehaviorSanitizer, as the
# reference's CI runs its host C++ under them (.github/workflows/ci.yml:62-79). Python must then
# start with the sanitizer's runtime preloaded: see `sanitizer_environment`.
SANITIZE_FLAGS = ["-fsanitize=address,undefined", "-fno-sanitize-recover=undefined", "-fno-omit-frame-pointer", "-O1", "-g"]


def host_module_path(sanitize: bool = False) -> Path:
    suffix = sysconfig.get_config_var("EXT_SUFFIX") or ".so"
    folder = build_dir() / "sanitize" if sanitize else build_dir()
    return folder / f"b200_host{suffix}"


def _sanitizing_compiler() -> tuple[str, str]:
    """(compiler, its AddressSanitizer runtime): the first of $CXX, g++, c++ and /usr/bin/g++
    that ships one."""
    tried = []
    for cxx in (os.environ.get("CXX"), shutil.which("g++"), shutil.which("c++"), "/usr/bin/g++"):
        if not cxx or cxx in tried or not Path(cxx).exists():
            continue
        tried.append(cxx)
        runtime = subprocess.run([cxx, "-print-file-name=libasan.so"], capture_output=True, text=True).stdout.strip()
        if runtime and Path(runtime).is_absolute() and Path(runtime).exists():
            return cxx, str(Path(runtime).resolve())
    raise BuildError(f"no C++ compiler with an AddressSanitizer runtime (tried {', '.join(tried) or 'none'})")


def sanitizer_environment() -> dict[str, str]:
    """Environment for a Python process that is to load the checked host build: the
    sanitizer's runtime preloaded, leak checking off (the interpreter itself never frees
    everything), and the switch that makes `host_module.host()` pick that build."""
    cxx, runtime = _sanitizing_compiler()
    # The C++ runtime goes in with it: the sanitizer hooks exception throwing when it starts, and
    # the interpreter itself does not link libstdc++.
    stdcxx = subprocess.run([cxx, "-print-file-name=libstdc++.so.6"], capture_output=True, text=True).stdout.strip()
    preload = runtime + (" " + str(Path(stdcxx).resolve()) if stdcxx and Path(stdcxx).is_absolute() and Path(stdcxx).exists() else "")
    return {
        "LD_PRELOAD": preload,
        "ASAN_OPTIONS": "detect_leaks=0:abort_on_error=0:halt_on_error=1",
        "UBSAN_OPTIONS": "print_stacktrace=1:halt_on_error=1",
        "LLM_INFERENCE_B200_SANITIZE": "1",
    }


def build_host(force: bool = False, sanitize: bool = False) -> Path:
    """Build (if stale) and return the path of the C++ host extension module; with
    ``sanitize`` the checked build (in a folder of its own)."""
    import pybind11

    sources = sorted(HOST_DIR.glob("*.cpp"))
    headers = sorted(HOST_DIR.glob("*.h"))
    out = host_module_path(sanitize)
    out.parent.mkdir(parents=True, exist_ok=True)
    includes = ["-I", str(HOST_DIR), "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"]]
    flags = [f for f in CXX_FLAGS if f != "-O2"] + SANITIZE_FLAGS if sanitize else CXX_FLAGS
    digest = _digest(sources + headers, flags + [sys.version])
    stamp = out.parent / (out.name + ".stamp")
    if not force and out.is_file() and stamp.is_file() and stamp.read_text() == digest:
        return out
    with _locked(out.parent / "host.lock"):
        if not force and out.is_file() and stamp.is_file() and stamp.read_text() == digest:
            return out
        cxx = _sanitizing_compiler()[0] if sanitize else os.environ.get("CXX") or shutil.which("g++") or shutil.which("c++")
        if not cxx:
            raise BuildError("no C++ compiler found (g++ / c++)")
        _compile_all(
            "C++ host runtime (checked build)" if sanitize else "C++ host runtime",
            sources,
            out,
            lambda src, obj: [cxx, *flags, *includes, "-c", str(src), "-o", str(obj)],
            lambda objs, target: [cxx, "-shared", *(SANITIZE_FLAGS[:1] if sanitize else []), "-o", str(target), *[str(o) for o in objs]],
            digest,
        )
    return out


def build_all(force: bool = False) -> dict[str, Path]:
    return {"host": build_host(force), "kernels": build_kernels(force)}


if __name__ == "__main__":
    for name, path in build_all(force="--force" in sys.argv).items():
        print(f"{name}: {path}")
