"""Binding of the GDN stages of the native library: the ``MekGdnDims`` structure and one Python launcher per C-ABI
entry point of ``include/mek_gdn.h``.

The reference binds each generated library's ``run`` to a positional launcher from a JSON ``arg_plan`` (reference:
miles_ext_kernels/cake/_impl/gdn/native.py:72-155).  Here the plan is the C prototype itself: a launcher takes torch
tensors (or ``None`` for an optional pointer), passes their device pointers and the current stream, and raises the
exception class the status code stands for.  Launchers enqueue on torch's current stream and never synchronise.
"""

from __future__ import annotations

import ctypes
from typing import Any

import torch

from ..._runtime import loader

__all__ = ["Dims", "LaunchLog", "library", "launch", "release", "set_launch_log"]


class Dims(ctypes.Structure):
    """``MekGdnDims`` of ``include/mek_gdn.h``."""

    _fields_ = [
        ("total_tokens", ctypes.c_int64),
        ("num_qk_heads", ctypes.c_int32),
        ("num_v_heads", ctypes.c_int32),
        ("head_dim", ctypes.c_int32),
        ("num_seqs", ctypes.c_int32),
        ("num_chunks", ctypes.c_int32),
        ("scale", ctypes.c_float),
        ("chunk_start", ctypes.c_void_p),
        ("chunk_len", ctypes.c_void_p),
        ("chunk_seq", ctypes.c_void_p),
        ("seq_chunk_start", ctypes.c_void_p),
        # token strides (elements) of operands that are column slices of a packed row; 0 = dense
        ("qk_pitch", ctypes.c_int64),
        ("v_pitch", ctypes.c_int64),
        ("raw_pitch", ctypes.c_int64),
        ("dqk_pitch", ctypes.c_int64),
        ("dv_pitch", ctypes.c_int64),
        # optional device table: the order in which the scans take the sequences (longest first)
        ("seq_order", ctypes.c_void_p),
    ]


_library: loader.NativeLibrary | None = None


def library() -> loader.NativeLibrary:
    """The loaded native library (built first when it is in neither the tree nor the cache)."""
    global _library
    if _library is None:
        _library = loader.load_library("libmek_b200", "sm_100a")
    return _library


def _argument(value: Any) -> Any:
    if value is None:
        return ctypes.c_void_p(0)
    if isinstance(value, torch.Tensor):
        return ctypes.c_void_p(value.data_ptr())
    if isinstance(value, Dims):
        return ctypes.byref(value)
    if isinstance(value, float):
        return ctypes.c_float(value)
    if isinstance(value, int):
        return ctypes.c_int64(value)
    return value


class LaunchLog:
    """Counts the kernels launched and, when ``timed``, brackets each launch with CUDA events on the launching
    stream (``bench.py`` reads per-kernel device times from it; ordinary calls never time)."""

    def __init__(self, timed: bool = False) -> None:
        self.timed = timed
        self.count = 0
        self.events: list[tuple[str, Any, Any]] = []

    def milliseconds(self) -> dict[str, list[float]]:
        """Per kernel name, the device time of each launch (call after synchronising)."""
        times: dict[str, list[float]] = {}
        for name, start, end in self.events:
            times.setdefault(name, []).append(start.elapsed_time(end))
        return times


_log: LaunchLog | None = None


def set_launch_log(log: LaunchLog | None) -> None:
    global _log
    _log = log


def launch(name: str, *arguments: Any, device: torch.device | None = None) -> None:
    """Call ``mek_<name>(*arguments, stream)`` with torch's current stream of ``device`` appended."""
    lib = library()
    current = torch.cuda.current_stream(device)
    log = _log
    if log is not None:
        log.count += 1
        if log.timed:
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(current)
    code = getattr(lib, f"mek_{name}")(*(_argument(a) for a in arguments), ctypes.c_void_p(current.cuda_stream))
    if log is not None and log.timed:
        end.record(current)
        log.events.append((name, start, end))
    lib.check(code)


def release() -> None:
    global _library
    _library = None
