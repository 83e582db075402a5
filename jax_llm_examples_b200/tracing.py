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


# ------------------------------------------------------------------------------------------ device timeline
TIMELINE_FLAG = "-DJLX_TIMELINE"
TIMELINE_KERNELS = ("?", "embed", "add_rmsnorm", "add_rmsnorm_router", "gemm_stream", "gemm_stream_pair", "rope_kv_store",
                    "attention_decode", "attention_combine", "expert_sort", "permute_scale", "argmax", "attention_prefill_tc",
                    "router_rows", "other", "attention_generic", "gemm_simt", "sample", "kv_store", "moe_combine", "splitk_reduce",
                    "silu_mul", "attention_prefill_mma", "attention_decode_plain")  # the order of JlxTimelineId in csrc/common.cuh


class DeviceTimeline:
    """Where the kernels of a step lie on the GPU's own clock, also inside a replayed graph.

    Neither CUDA events nor a profiler's serialised replay show how the kernels of a captured decode step overlap
    (programmatic dependent launch lets each start during its predecessor) or where the GPU waits.  Kernel
    libraries compiled with ``-DJLX_TIMELINE`` (put it into ``JLX_B200_NVCC_EXTRA`` before the first kernel is
    loaded; ``python -m jax_llm_examples_b200.timeline`` does) make thread 0 of every block record the global timer
    at the block's start, at the end of its wait for the predecessor, at up to four marked places inside the
    kernel, and at its exit.  This class owns the record buffer, hands it to every loaded library, and groups the
    records into launches.
    """

    WORDS = 8  # per record: what, start, waited, end, four marks

    def __init__(self, capacity: int = 1 << 16):
        self.capacity = capacity
        self.buf = torch.zeros(1 + self.WORDS * capacity, dtype=torch.int64, device="cuda")
        self._attached: set[str] = set()

    def attach(self) -> None:
        """Gives the buffer to every kernel library loaded so far (call again after more were loaded)."""
        import ctypes

        from .kernels import api

        for name in api.loaded_libraries():
            if name in self._attached or name == "host":
                continue
            lib = api.library(name)
            if not hasattr(lib, "jlx_timeline_set"):
                raise RuntimeError(f"kernel library {name} was built without {TIMELINE_FLAG}")
            if lib.jlx_timeline_set(ctypes.c_void_p(self.buf.data_ptr()), ctypes.c_uint(self.capacity)) != 0:
                raise RuntimeError(f"jlx_timeline_set failed in {name}")
            self._attached.add(name)

    def reset(self) -> None:
        self.buf[:1].zero_()

    def records(self):
        """[n, 8] int64 on the host: (what, start, waited, end, marks), times in ns of the GPU's global timer."""
        torch.cuda.synchronize()
        n = int(self.buf[0].item())
        if n > self.capacity:
            raise RuntimeError(f"the timeline holds {self.capacity} block records, {n} were written: shorten the run")
        return self.buf[1:1 + self.WORDS * n].view(n, self.WORDS).cpu().numpy()

    def launches(self) -> list[dict]:
        """Records grouped into launches, in the order of their first block's start: a launch is complete when as many
        blocks of its kernel and grid shape were seen as the grid has.  Per launch: ``start`` (first block in),
        ``ready`` (the first block that waited for the predecessor got through: the predecessor had ended), ``end``
        (last block out), ``marks`` (block 0's), in microseconds after the first record."""
        rec = self.records()
        if not len(rec):
            return []
        order = rec[:, 1].argsort(kind="stable")
        t_zero = int(rec[:, 1].min())
        open_by_key: dict[int, dict] = {}
        seen: dict[int, int] = {}
        out: list[dict] = []
        for what, t0, t1, t3, *marks in rec[order].tolist():
            key = what & 0xFFFFFFFFFFFF
            g = open_by_key.get(key)
            if g is None:
                gx, gy, gz = (key >> 8) & 0xFFFF, (key >> 24) & 0xFFFF, (key >> 40) & 0xFF
                g = {"kernel": TIMELINE_KERNELS[min(key & 0xFF, len(TIMELINE_KERNELS) - 1)], "grid": (gx, gy, gz), "blocks": 0,
                     "occurrence": seen.get(key, 0), "start": t0, "ready": None, "end": t3, "marks": None, "_key": key}
                seen[key] = g["occurrence"] + 1
                open_by_key[key] = g
                out.append(g)
            g["blocks"] += 1
            g["end"] = max(g["end"], t3)
            if t1:
                g["ready"] = t1 if g["ready"] is None else min(g["ready"], t1)
            if what < 0 or what >> 63:  # the grid's block 0 (the word's top bit)
                g["marks"] = marks if any(marks) else None
            if g["blocks"] == g["grid"][0] * g["grid"][1] * g["grid"][2]:
                del open_by_key[key]
        for g in out:
            for k in ("start", "ready", "end"):
                g[k] = None if g[k] is None else (g[k] - t_zero) / 1e3
            if g["marks"] is not None:
                g["marks"] = [None if m == 0 else (m - t_zero) / 1e3 for m in g["marks"]]
        return out

    @staticmethod
    def summary(steps: list[list[dict]]) -> list[dict]:
        """Medians over several recordings of the same step.  The k-th launch of a kernel with a grid shape is the
        same launch in every recording.  Per launch: ``at`` (when it was ready, or started, after the step's first
        record; the rows are in this order), ``busy`` (from then to its end), ``adds`` (how much later it ended than
        every launch that was ready before it: what it added to the chain; kernels of a second stream that hide
        behind others add nothing), ``early`` (how long before it was ready its first block was in), and the marks
        as microseconds after ``ready``."""
        import statistics

        per_launch: dict[tuple, list[dict]] = {}
        for s in steps:
            ordered = sorted(s, key=lambda g: g["ready"] if g["ready"] is not None else g["start"])
            so_far = None
            for g in ordered:
                ready = g["ready"] if g["ready"] is not None else g["start"]
                m = {"at": ready, "busy": g["end"] - ready, "early": ready - g["start"],
                     "adds": max(0.0, g["end"] - (so_far if so_far is not None else g["start"])),
                     "marks": None if g["marks"] is None else [None if x is None else x - ready for x in g["marks"]]}
                so_far = g["end"] if so_far is None else max(so_far, g["end"])
                per_launch.setdefault((g["_key"], g["occurrence"]), []).append({**g, **m})
        rows = []
        for (key, occ), ms in per_launch.items():
            if len(ms) != len(steps):
                continue  # a launch that not every recording has (another graph was replayed)
            row = {"kernel": ms[0]["kernel"], "grid": ms[0]["grid"], "blocks": ms[0]["blocks"], "marks": None}
            for k in ("at", "busy", "adds", "early"):
                row[k] = statistics.median(m[k] for m in ms)
            with_marks = [m["marks"] for m in ms if m["marks"] is not None]
            if with_marks:
                row["marks"] = [None if any(w[j] is None for w in with_marks) else statistics.median(w[j] for w in with_marks)
                                for j in range(4)]
            rows.append(row)
        rows.sort(key=lambda r: r["at"])
        return rows

    @staticmethod
    def table(rows: list[dict]) -> str:
        """One line per launch of a summary."""
        lines = [f"{'kernel':22s} {'grid':>12s} {'at':>8s} {'early':>7s} {'busy':>7s} {'adds':>7s}  marks after ready"]
        for g in rows:
            marks = "" if g["marks"] is None else " ".join("-" if m is None else f"{m:.2f}" for m in g["marks"])
            lines.append(f"{g['kernel']:22s} {'x'.join(map(str, g['grid'])):>12s} {g['at']:8.2f} {g['early']:7.2f} "
                         f"{g['busy']:7.2f} {g['adds']:7.2f}  {marks}")
        return "\n".join(lines)
