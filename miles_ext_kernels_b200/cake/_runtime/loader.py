"""The loader of the native kernel library: plain nvcc, a file-locked cache, and a ctypes load of its C ABI.

One shared library per architecture, ``libmek_b200_<arch>.so``, holds every kernel of the gated-delta-rule path (the
sources are ``miles_ext_kernels_b200/csrc/*.cu``; the C ABI is ``include/mek_gdn.h``).  It takes the place of the
reference's per-kernel tvm-ffi libraries and of its ``JitSpec`` (reference:
miles_ext_kernels/cake/_runtime/loader.py:241-348): same life cycle, one library instead of hundreds.

Where a library is looked for, in order:

1. ``miles_ext_kernels_b200/_lib/<name>_<key16>.so`` -- built ahead of time in the source tree (``prebuild(...,
   in_tree=True)``; what ``__graft_entry__.build()`` does), used as it is;
2. ``cache_dir()/<name>_<key16>.so`` -- built on first use, or by ``prebuild``.

The key hashes the nvcc flags, the full nvcc version, the machine and the bytes of every source and header, so a
changed kernel never loads a stale build.  All ranks may start a build at once: one compiles under ``flock`` into a
temporary file and renames it into place, the others wait and load it (reference: loader.py:304-334).  A waiting rank
logs every 30 s and gives up after 30 minutes.  Inside :func:`no_build` a missing library raises instead of
compiling, which is how the tests check the ``prebuild`` contract (reference: loader.py:439-447).

A loaded library is refused when it was compiled against another CUDART than the toolkit reports (reference:
loader.py:336-348), and when it lacks a symbol ``include/mek_gdn.h`` declares.

Importing this module imports neither torch nor the library.
"""

from __future__ import annotations

import ctypes
import fcntl
import functools
import hashlib
import json
import logging
import os
import platform
import re
import shutil
import subprocess
import threading
import time
import uuid
from collections.abc import Iterable, Iterator
from contextlib import contextmanager
from pathlib import Path
from typing import Any, NamedTuple

__all__ = [
    "ARCH_BY_CAPABILITY",
    "LIBRARIES",
    "MIN_CUDA",
    "CudaVersion",
    "LibrarySpec",
    "NativeLibrary",
    "cache_dir",
    "check_toolkit",
    "declared_symbols",
    "device_arch",
    "find_nvcc",
    "get_cuda_version",
    "install_op",
    "library_spec",
    "load_library",
    "no_build",
    "prebuild_libraries",
    "release",
]

# The architecture of every compute capability the kernels serve: B200 only.
ARCH_BY_CAPABILITY = {(10, 0): "sm_100a"}
# The oldest CUDA toolkit that compiles tcgen05 / TMA for each architecture.
MIN_CUDA = {"sm_100a": (12, 8)}

_NVCC_RELEASE = re.compile(r"release (\d+)\.(\d+)")
_NVCC_BUILD = re.compile(r"\bV(\d+\.\d+\.\d+)")
_STDERR_LINES = 40
_LOCK_POLL_SECONDS = 1.0
_LOCK_LOG_SECONDS = 30.0
_LOCK_TIMEOUT_SECONDS = 30 * 60

logger = logging.getLogger(__name__)

_ROOT = Path(__file__).resolve().parents[2]  # the package directory
_CSRC = _ROOT / "csrc"
_IN_TREE = _ROOT / "_lib"
_HEADER_CANDIDATES = (_ROOT.parent / "include" / "mek_gdn.h", _ROOT / "include" / "mek_gdn.h")

# library -> the sources under csrc/ it is made of (headers are found by suffix)
LIBRARIES: dict[str, tuple[str, ...]] = {"libmek_b200": ("*.cu",)}
# op -> libraries it launches
_OP_LIBRARIES: dict[str, tuple[str, ...]] = {}
_NO_BUILD = 0
_LOADED: dict[Path, NativeLibrary] = {}
_LOAD_LOCK = threading.Lock()

_COMMON_FLAGS = (
    "-std=c++17",
    "-O3",
    "-lineinfo",
    "--expt-relaxed-constexpr",
    "-Xcompiler",
    "-fPIC",
    "-shared",
)


class CudaVersion(NamedTuple):
    """The toolkit of ``nvcc --version``: ``release X.Y`` and the full ``VX.Y.Z``."""

    major: int
    minor: int
    full: str

    @property
    def cudart(self) -> int:
        """``CUDART_VERSION`` of the toolkit: ``1000 * major + 10 * minor``."""
        return 1000 * self.major + 10 * self.minor


def find_nvcc() -> str:
    """``$CUDA_HOME/bin/nvcc``, else ``nvcc`` on ``PATH``, else ``/usr/local/cuda/bin/nvcc``."""
    cuda_home = os.environ.get("CUDA_HOME")
    if cuda_home:
        return str(Path(cuda_home) / "bin" / "nvcc")
    found = shutil.which("nvcc")
    if found is None:
        fallback = Path("/usr/local/cuda/bin/nvcc")
        if fallback.is_file():
            return str(fallback)
        raise RuntimeError("no nvcc to build the kernels: set CUDA_HOME or put nvcc on PATH")
    return found


@functools.lru_cache(maxsize=None)
def _nvcc_version(nvcc: str, stamp: tuple[int, int]) -> CudaVersion:
    # ``stamp`` (mtime, size) re-runs nvcc when the file at that path changes
    try:
        proc = subprocess.run([nvcc, "--version"], capture_output=True, text=True, check=False)
    except OSError as exc:
        raise RuntimeError(f"cannot run {nvcc} --version: {exc}") from exc
    release_ = _NVCC_RELEASE.search(proc.stdout)
    build = _NVCC_BUILD.search(proc.stdout)
    if proc.returncode or release_ is None or build is None:
        raise RuntimeError(
            f"{nvcc} --version (exit {proc.returncode}) reports no 'release X.Y, VX.Y.Z':\n{proc.stdout}{proc.stderr}"
        )
    return CudaVersion(int(release_.group(1)), int(release_.group(2)), build.group(1))


def _toolkit(nvcc: str | None = None) -> tuple[str, CudaVersion]:
    nvcc = nvcc or find_nvcc()
    try:
        stat = os.stat(nvcc)
    except OSError as exc:
        raise RuntimeError(f"cannot run {nvcc}: {exc}") from exc
    return nvcc, _nvcc_version(nvcc, (stat.st_mtime_ns, stat.st_size))


def get_cuda_version() -> CudaVersion:
    """The toolkit of :func:`find_nvcc`."""
    return _toolkit()[1]


def check_toolkit(arch: str, what: str, nvcc: str | None = None) -> CudaVersion:
    """The toolkit of ``nvcc``, checked to compile ``arch`` (:data:`MIN_CUDA`); ``RuntimeError`` when it is older."""
    nvcc, cuda = _toolkit(nvcc)
    need = MIN_CUDA.get(arch)
    if need is not None and (cuda.major, cuda.minor) < need:
        raise RuntimeError(
            f"compiling {what} for {arch} needs CUDA {need[0]}.{need[1]} or newer, but {nvcc} is CUDA {cuda.full}: "
            f"set CUDA_HOME to a CUDA {need[0]}.{need[1]} or newer toolkit"
        )
    return cuda


def cache_dir() -> Path:
    """``$MILES_EXT_KERNELS_CACHE_DIR``, else ``$TVM_FFI_CACHE_DIR/miles_ext_kernels`` (the reference's variable),
    else ``~/.cache/miles_ext_kernels_b200``."""
    own = os.environ.get("MILES_EXT_KERNELS_CACHE_DIR")
    if own:
        return Path(own).expanduser()
    shared = os.environ.get("TVM_FFI_CACHE_DIR")
    if shared:
        return Path(shared).expanduser() / "miles_ext_kernels"
    return Path("~/.cache/miles_ext_kernels_b200").expanduser()


def _header() -> Path:
    for candidate in _HEADER_CANDIDATES:
        if candidate.is_file():
            return candidate
    raise RuntimeError(f"the C-ABI header mek_gdn.h was not found in {[str(c.parent) for c in _HEADER_CANDIDATES]}")


def declared_symbols(header: Path | None = None) -> tuple[str, ...]:
    """Every function ``include/mek_gdn.h`` declares (``mek_*`` followed by an argument list)."""
    text = (header or _header()).read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return tuple(dict.fromkeys(re.findall(r"\b(mek_[a-z0-9_]+)\s*\(", text)))


def _lock_exclusive(lock: Any, lock_path: Path, name: str) -> None:
    """Take the exclusive flock of the open file ``lock``, waiting at most ``_LOCK_TIMEOUT_SECONDS``."""
    start = time.monotonic()
    logged = start
    while True:
        try:
            fcntl.flock(lock, fcntl.LOCK_EX | fcntl.LOCK_NB)
            return
        except BlockingIOError:
            pass
        now = time.monotonic()
        if now - start >= _LOCK_TIMEOUT_SECONDS:
            raise RuntimeError(
                f"gave up building {name} after waiting {now - start:.0f} s for the build lock {lock_path}: another "
                "process holds it. Retry, or point MILES_EXT_KERNELS_CACHE_DIR at a node-local directory."
            )
        if now - logged >= _LOCK_LOG_SECONDS:
            logged = now
            logger.warning("waiting %.0f s for the build lock %s of %s", now - start, lock_path, name)
        time.sleep(_LOCK_POLL_SECONDS)


class LibrarySpec:
    """One library for one architecture: its nvcc command, its cache key and its two possible locations."""

    def __init__(self, name: str, arch: str, *, nvcc: str | None = None) -> None:
        if name not in LIBRARIES:
            raise KeyError(f"no library {name!r}; the libraries are {sorted(LIBRARIES)}")
        if arch not in MIN_CUDA:
            raise NotImplementedError(f"the kernels are written for {sorted(MIN_CUDA)}, not {arch}")
        self.name = name
        self.arch = arch
        self.nvcc, self.cuda = _toolkit(nvcc)
        self.sources = sorted(str(p) for pattern in LIBRARIES[name] for p in _CSRC.glob(pattern))
        if not self.sources:
            raise RuntimeError(f"{name}: no sources under {_CSRC}")
        self.flags = [f"-gencode=arch=compute_{arch[3:]},code={arch}", *_COMMON_FLAGS]
        digest = hashlib.sha256()
        for path in sorted([*self.sources, *(str(p) for p in _CSRC.glob("*.cuh")), str(_header())]):
            digest.update(Path(path).name.encode())
            digest.update(Path(path).read_bytes())
        key = json.dumps(
            {
                "flags": self.flags,
                "nvcc": self.cuda.full,
                "machine": platform.machine(),
                "sources": digest.hexdigest(),
            },
            sort_keys=True,
        )
        self.key = hashlib.sha256(key.encode()).hexdigest()
        self.file_name = f"{name}_{arch}_{self.key[:16]}.so"

    def command(self, output: Path) -> list[str]:
        """The nvcc command writing the library to ``output``."""
        return [self.nvcc, *self.flags, f"-I{_header().parent}", *self.sources, "-o", str(output)]

    def in_tree_path(self) -> Path:
        return _IN_TREE / self.file_name

    def cache_path(self) -> Path:
        return cache_dir() / self.file_name

    def find(self) -> Path | None:
        """The built library, ``None`` when neither location holds it."""
        for path in (self.in_tree_path(), self.cache_path()):
            if path.is_file():
                return path
        return None

    def build(self, *, in_tree: bool = False) -> Path:
        """Compile the library unless it exists; return its path."""
        found = self.find()
        if found is not None and not (in_tree and found != self.in_tree_path()):
            return found
        if _NO_BUILD:
            ops = sorted(op for op, names in _OP_LIBRARIES.items() if self.name in names) or [self.name]
            raise RuntimeError(f"{self.name} would compile inside a call: prebuild({ops[0]!r}, ...) first")
        check_toolkit(self.arch, self.name, self.nvcc)
        path = self.in_tree_path() if in_tree else self.cache_path()
        path.parent.mkdir(parents=True, exist_ok=True)
        lock_path = path.with_suffix(".lock")
        with open(lock_path, "a") as lock:
            _lock_exclusive(lock, lock_path, self.name)  # released when the file closes
            if path.is_file():  # another rank built it while this one waited
                return path
            temporary = path.with_name(f"{path.stem}.{os.getpid()}.{uuid.uuid4().hex[:8]}.tmp.so")
            command = self.command(temporary)
            try:
                try:
                    proc = subprocess.run(command, capture_output=True, text=True, check=False)
                except OSError as exc:
                    raise RuntimeError(f"cannot run {self.nvcc} to build {self.name}: {exc}") from exc
                if proc.returncode or not temporary.is_file():
                    stderr = "\n".join(proc.stderr.splitlines()[:_STDERR_LINES])
                    raise RuntimeError(
                        f"nvcc failed to build {self.name} (exit {proc.returncode}):\n{' '.join(command)}\n{stderr}"
                    )
                os.replace(temporary, path)
            finally:
                temporary.unlink(missing_ok=True)
        if in_tree:  # drop builds of older sources so the tree ships one library
            for stale in _IN_TREE.glob(f"{self.name}_{self.arch}_*.so"):
                if stale != path:
                    stale.unlink(missing_ok=True)
                    stale.with_suffix(".lock").unlink(missing_ok=True)
        return path


class NativeLibrary:
    """A loaded library: its exported functions by attribute, and :meth:`check` turning status codes into the
    exception classes of the reference's typed FFI errors."""

    def __init__(self, path: Path, cudart: int | None) -> None:
        self.path = path
        self._dll = ctypes.CDLL(str(path))
        missing = [name for name in declared_symbols() if not hasattr(self._dll, name)]
        if missing:
            raise RuntimeError(f"{path} lacks the symbols {missing} that mek_gdn.h declares")
        self._dll.mek_last_error.restype = ctypes.c_char_p
        self._dll.mek_build_cuda_version.restype = ctypes.c_int
        built = int(self._dll.mek_build_cuda_version())
        if cudart is not None and built != cudart:
            raise RuntimeError(f"{path} was compiled against CUDART {built}, but the toolkit is CUDART {cudart}")
        self.build_cuda_version = built

    def __getattr__(self, name: str) -> Any:
        function = getattr(self._dll, name)
        function.restype = ctypes.c_int
        setattr(self, name, function)
        return function

    def last_error(self) -> str:
        return (self._dll.mek_last_error() or b"").decode(errors="replace")

    def check(self, code: int) -> None:
        """Raise for a nonzero status: 1 ``ValueError``, 2 ``NotImplementedError``, anything else ``RuntimeError``."""
        if code == 0:
            return
        text = self.last_error() or f"native call failed with status {code}"
        if code == 1:
            raise ValueError(text)
        if code == 2:
            raise NotImplementedError(text)
        raise RuntimeError(text)


def library_spec(name: str = "libmek_b200", arch: str = "sm_100a") -> LibrarySpec:
    return LibrarySpec(name, arch)


def load_library(name: str = "libmek_b200", arch: str = "sm_100a") -> NativeLibrary:
    """The loaded library ``name`` for ``arch``, built first if it is in neither location (unless :func:`no_build`).

    Without a toolkit on the machine a library that was built in the tree is still found by its name and loaded;
    the CUDART stamp is then not compared.
    """
    try:
        spec: LibrarySpec | None = LibrarySpec(name, arch)
    except RuntimeError:
        spec = None
    if spec is None:
        candidates = sorted(_IN_TREE.glob(f"{name}_{arch}_*.so"), key=lambda p: p.stat().st_mtime)
        if not candidates:
            raise RuntimeError(f"{name} is not built for {arch} and no nvcc was found to build it")
        path, cudart = candidates[-1], None
    else:
        path, cudart = spec.build(), spec.cuda.cudart
    with _LOAD_LOCK:
        library = _LOADED.get(path)
        if library is None:
            library = _LOADED[path] = NativeLibrary(path, cudart)
    return library


def install_op(op: str, libraries: Iterable[str] = ("libmek_b200",)) -> None:
    """Register the libraries ``op`` launches; called once by ``_impl/<op>`` at import (idempotent).

    The reference's ``install_op`` installs its loader on every vendored package of the op (reference:
    loader.py:403-413); here an op only names its libraries, which :func:`prebuild_libraries` builds.
    """
    names = tuple(libraries)
    for name in names:
        if name not in LIBRARIES:
            raise KeyError(f"no library {name!r}; the libraries are {sorted(LIBRARIES)}")
    _OP_LIBRARIES[op] = names


def op_libraries(op: str) -> tuple[str, ...]:
    return _OP_LIBRARIES.get(op, ())


def prebuild_libraries(names: Iterable[str], arch: str, max_workers: int | None = None, *, in_tree: bool = False):
    """Compile the libraries ``names`` for ``arch`` ahead of their first call; returns their paths, in order.

    A built library is not compiled again.  ``in_tree`` writes to the package's ``_lib`` directory instead of the
    cache.  ``max_workers`` is accepted for the reference's signature; one nvcc call builds one library.
    """
    del max_workers
    return [LibrarySpec(name, arch).build(in_tree=in_tree) for name in dict.fromkeys(names)]


@contextmanager
def no_build() -> Iterator[None]:
    """Inside this block, a library that is not built raises ``RuntimeError`` instead of compiling (nestable)."""
    global _NO_BUILD
    _NO_BUILD += 1
    try:
        yield
    finally:
        _NO_BUILD -= 1


def device_arch(device: Any = None) -> str:
    """``"sm_100a"``: the architecture of the CUDA ``device`` (default: current).

    ``NotImplementedError`` for any other compute capability.  Imports torch.
    """
    import torch

    capability = tuple(torch.cuda.get_device_capability(device))
    try:
        return ARCH_BY_CAPABILITY[capability]
    except KeyError:
        major, minor = capability
        raise NotImplementedError(
            f"the kernels need SM100a (B200), not compute capability {major}.{minor}"
        ) from None


def release() -> None:
    """Forget the loaded library handles (the shared objects stay mapped; a later call loads them again by path)."""
    with _LOAD_LOCK:
        _LOADED.clear()
