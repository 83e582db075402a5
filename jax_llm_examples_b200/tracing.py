"""Op-level tracing: named ranges around the parts' operations, and a timer around every kernel launch.

The reference wraps its op groups in ``jax.named_scope`` (llama4/llama4_jax/model.py:906-954, 1076-1138,
1145-1181) so that a profile shows them by name, and traces its kernel benchmarks
(llama4_jax/ragged_attention.py:413, llama4_jax/decode_ragged_dot.py:284).  Here:

* ``scope(name)`` marks the same op groups under the reference's names.  With the environment variable
  ``JLX_B200_NVTX=1`` (or after ``enable_nvtx()``) each scope is an NVTX range, which Nsight Systems and
  Nsight Compute (``--nvtx``) show; otherwise a scope costs one check.
* ``KernelTimer`` brackets every launch of this package's kernels with CUDA events and adds the times up by
  kernel entry point and by scope: ``Generator(profile="kernels")`` runs its steps under one.

While either is on, the engine does not replay captured graphs (a replayed graph launches its kernels without
passing through the host code that marks them).
"""

from __future__ import annotations

import contextlib
import os
from collections import defaultdict

import torch

_nvtx = os.environ.get("JLX_B200_NVTX", "") not in ("", "0")
_timer: "KernelTimer | None" = None
_stack: list[str] = []
_NULL = contextlib.nullcontext()


def enable_nvtx(on: bool = True) -> None:
    global _nvtx
    _nvtx = bool(on)


def active() -> bool:
    """True while scopes are being marked or launches timed."""
    return _nvtx or _timer is not None


class _Scope:
    __slots__ = ("name",)

    def __init__(self, name: str):
        self.name = name

    def __enter__(self):
        _stack.append(self.name)
        if _nvtx:
            torch.cuda.nvtx.range_push(self.name)

    def __exit__(self, *exc):
        if _nvtx:
            torch.cuda.nvtx.range_pop()
        _stack.pop()
        return False


def scope(name: str):
    """A named range around an op group (a no-op unless tracing is on)."""
    return _Scope(name) if (_nvtx or _timer is not None) else _NULL


class KernelTimer:
    """Times every kernel launch that goes through ``kernels.api`` while it is installed (``with timer:``)."""

    def __init__(self):
        self._pending: list[tuple[str, str, torch.cuda.Event, torch.cuda.Event]] = []
        self.by_kernel: dict[str, list[float]] = defaultdict(lambda: [0, 0.0])  # entry point -> [launches, ms]
        self.by_scope: dict[str, list[float]] = defaultdict(lambda: [0, 0.0])  # innermost scope -> [launches, ms]

    def __enter__(self):
        global _timer
        self._outer, _timer = _timer, self
        return self

    def __exit__(self, *exc):
        global _timer
        _timer = self._outer
        self.collect()
        return False

    def around(self, name: str, launch) -> None:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        launch()
        e1.record()
        self._pending.append((name, _stack[-1] if _stack else "(no scope)", e0, e1))

    def collect(self) -> None:
        """Waits for the launches so far and adds their times up."""
        if not self._pending:
            return
        torch.cuda.synchronize()
        for name, where, e0, e1 in self._pending:
            ms = e0.elapsed_time(e1)
            for table, key in ((self.by_kernel, name), (self.by_scope, where)):
                table[key][0] += 1
                table[key][1] += ms
        self._pending.clear()

    def report(self, by: str = "kernel") -> str:
        self.collect()
        table = self.by_kernel if by == "kernel" else self.by_scope
        total = sum(v[1] for v in table.values()) or 1.0
        rows = sorted(table.items(), key=lambda kv: -kv[1][1])
        return "\n".join(f"{name:32s} {int(n):7d} launches {ms:10.3f} ms {100 * ms / total:5.1f} %" for name, (n, ms) in rows)


def current_timer() -> "KernelTimer | None":
    return _timer
