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
import dataclasses
import fcntl
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
from typing import Any

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


@dataclasses.dataclass(frozen=True, order=True)
class CudaVersion:
    """A CUDA toolkit as its compiler names it: the release pair and the full build string (``12.9.86``)."""

    major: int
    minor: int
    full: str

    @property
    def cudart(self) -> int:
        """The integer ``CUDART_VERSION`` takes for this release (12.9 -> 12090)."""
        return self.major * 1000 + self.minor * 10

    @classmethod
    def parse(cls, banner: str) -> CudaVersion | None:
        """From the text of ``nvcc --version``; ``None`` when it names no release and build."""
        release_, build = _NVCC_RELEASE.search(banner), _NVCC_BUILD.search(banner)
        if not (release_ and build):
            return None
        return cls(int(release_[1]), int(release_[2]), build[1])


def _nvcc_candidates() -> Iterator[Path]:
    home = os.environ.get("CUDA_HOME")
    if home:  # an explicit toolkit wins, whether or not it exists: a wrong CUDA_HOME should be reported, not skipped
        yield Path(home, "bin", "nvcc")
        return
    on_path = shutil.which("nvcc")
    if on_path:
        yield Path(on_path)
    yield Path("/usr/local/cuda/bin/nvcc")


def find_nvcc() -> str:
    """The compiler to use: ``$CUDA_HOME/bin/nvcc`` when ``CUDA_HOME`` is set, else the first of ``nvcc`` on ``PATH``
    and ``/usr/local/cuda/bin/nvcc`` that exists.  ``RuntimeError`` when there is none."""
    explicit = bool(os.environ.get("CUDA_HOME"))
    for candidate in _nvcc_candidates():
        if explicit or candidate.is_file():
            return str(candidate)
    raise RuntimeError("no nvcc to build the kernels: set CUDA_HOME or put nvcc on PATH")


class _Toolkits:
    """Remembers what each compiler binary reported, per (path, modification time, size): swapping the file at a
    path asks it again, an unchanged one is never run twice."""

    def __init__(self) -> None:
        self._seen: dict[tuple[str, int, int], CudaVersion] = {}

    def version_of(self, nvcc: str) -> CudaVersion:
        try:
            info = os.stat(nvcc)
        except OSError as exc:
            raise RuntimeError(f"cannot run {nvcc}: {exc}") from exc
        identity = (nvcc, info.st_mtime_ns, info.st_size)
        if identity not in self._seen:
            self._seen[identity] = self._ask(nvcc)
        return self._seen[identity]

    @staticmethod
    def _ask(nvcc: str) -> CudaVersion:
        try:
            done = subprocess.run([nvcc, "--version"], capture_output=True, text=True, check=False)
        except OSError as exc:
            raise RuntimeError(f"cannot run {nvcc} --version: {exc}") from exc
        version = None if done.returncode else CudaVersion.parse(done.stdout)
        if version is None:
            raise RuntimeError(f"{nvcc} --version (exit {done.returncode}) reports no 'release X.Y, VX.Y.Z':\n"
                               f"{done.stdout}{done.stderr}")
        return version


_TOOLKITS = _Toolkits()


def _toolkit(nvcc: str | None = None) -> tuple[str, CudaVersion]:
    """``(compiler path, its version)`` for ``nvcc`` or, without one, for :func:`find_nvcc`."""
    path = find_nvcc() if nvcc is None else nvcc
    return path, _TOOLKITS.version_of(path)


def get_cuda_version() -> CudaVersion:
    """The toolkit of :func:`find_nvcc`."""
    return _toolkit()[1]


def check_toolkit(arch: str, what: str, nvcc: str | None = None) -> CudaVersion:
    """The toolkit of ``nvcc``, checked to compile ``arch`` (:data:`MIN_CUDA`); ``RuntimeError`` when it is older."""
    path, have = _toolkit(nvcc)
    oldest = MIN_CUDA.get(arch)
    if oldest is None or (have.major, have.minor) >= tuple(oldest):
        return have
    wanted = ".".join(str(part) for part in oldest)
    raise RuntimeError(f"compiling {what} for {arch} needs CUDA {wanted} or newer, but {path} is CUDA {have.full}: "
                       f"set CUDA_HOME to a CUDA {wanted} or newer toolkit")


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


@contextmanager
def _build_lock(target: Path, what: str) -> Iterator[None]:
    """Hold the exclusive ``flock`` of ``<target>.lock`` for the block: one process per node builds ``target``, the
    others wait here (a line in the log every ``_LOCK_LOG_SECONDS``) and give up after ``_LOCK_TIMEOUT_SECONDS``."""
    lock_path = target.with_suffix(".lock")
    began = time.monotonic()
    next_report = began + _LOCK_LOG_SECONDS
    with open(lock_path, "a") as handle:
        while True:
            try:
                fcntl.flock(handle, fcntl.LOCK_EX | fcntl.LOCK_NB)
                break
            except BlockingIOError:
                waited = time.monotonic() - began
            if waited >= _LOCK_TIMEOUT_SECONDS:
                raise RuntimeError(
                    f"gave up building {what} after waiting {waited:.0f} s for the build lock {lock_path}: another "
                    "process holds it. Retry, or point MILES_EXT_KERNELS_CACHE_DIR at a node-local directory.")
            if time.monotonic() >= next_report:
                next_report += _LOCK_LOG_SECONDS
                logger.warning("waiting %.0f s for the build lock %s of %s", waited, lock_path, what)
            time.sleep(_LOCK_POLL_SECONDS)
        yield  # closing the file drops the lock


def _run_compiler(command: list[str], output: Path, what: str) -> None:
    """Run ``command`` (which writes ``output``); ``RuntimeError`` with the command and the head of nvcc's stderr when
    it fails or writes nothing."""
    try:
        done = subprocess.run(command, capture_output=True, text=True, check=False)
    except OSError as exc:
        raise RuntimeError(f"cannot run {command[0]} to build {what}: {exc}") from exc
    if done.returncode == 0 and output.is_file():
        return
    head = "\n".join(done.stderr.splitlines()[:_STDERR_LINES])
    raise RuntimeError(f"nvcc failed to build {what} (exit {done.returncode}):\n{' '.join(command)}\n{head}")


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
        target = self.in_tree_path() if in_tree else self.cache_path()
        existing = target if (in_tree and target.is_file()) else (None if in_tree else self.find())
        if existing is not None:
            return existing
        if _NO_BUILD:
            users = sorted(op for op, names in _OP_LIBRARIES.items() if self.name in names)
            raise RuntimeError(f"{self.name} would compile inside a call: prebuild({(users or [self.name])[0]!r}, ...) "
                               "first")
        check_toolkit(self.arch, self.name, self.nvcc)
        target.parent.mkdir(parents=True, exist_ok=True)
        with _build_lock(target, self.name):
            if not target.is_file():  # else another rank built it while this one waited
                # compile beside the target and rename: a reader never sees half a library
                scratch = target.with_name(f"{target.stem}.{os.getpid()}.{uuid.uuid4().hex[:8]}.tmp.so")
                try:
                    _run_compiler(self.command(scratch), scratch, self.name)
                    os.replace(scratch, target)
                finally:
                    scratch.unlink(missing_ok=True)
        if in_tree:  # the tree ships one library: builds of older sources go
            for other in _IN_TREE.glob(f"{self.name}_{self.arch}_*.so"):
                if other != target:
                    other.unlink(missing_ok=True)
                    other.with_suffix(".lock").unlink(missing_ok=True)
        return target


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
