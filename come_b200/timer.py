"""CUDA-event timer with named ranges and a percentile table, mirroring the reference's ``Timer``
(``src/utility/timer.py:15-93``) as its end-to-end benchmark uses it (``src/bench.py:14-15,29,42,46``):
``Timer.activate()``, ``with Timer.range(name): ...`` around each inference, ``Timer.report()`` for the table of
count, median, P90 and P99 in milliseconds.

Ranges are recorded on the current stream of the current device (the reference records on the default stream, which is
where its models run); the table is plain text with the reference's columns.
"""
from __future__ import annotations

import typing as tp
from contextlib import contextmanager
from dataclasses import dataclass

import numpy as np
import torch

__all__ = ["Timer"]


class Timer:
    @dataclass(kw_only=True, frozen=True, eq=False, slots=True)
    class Entry:
        name: str
        count: int
        P50: float
        P90: float
        P99: float

    _is_activate: tp.ClassVar[bool] = False
    _timer_queue: tp.ClassVar[dict] = dict()

    @classmethod
    def is_active(cls) -> bool:
        return cls._is_activate

    @classmethod
    def activate(cls, mode: bool = True) -> None:
        cls._is_activate = mode

    @classmethod
    def reset(cls) -> None:
        cls._timer_queue.clear()

    @classmethod
    @contextmanager
    def range(cls, name: str) -> tp.Iterator[None]:
        if not cls._is_activate:
            yield
            return
        start = torch.cuda.Event(enable_timing=True)
        end = torch.cuda.Event(enable_timing=True)
        start.record()
        try:
            yield
        finally:
            end.record()
            cls._timer_queue.setdefault(name, []).append((start, end))

    @classmethod
    def summarise(cls, name: str, elapsed_ms: tp.Sequence[float]) -> "Timer.Entry":
        elapsed = np.asarray(elapsed_ms, dtype=np.float64)
        return Timer.Entry(name=name, count=int(elapsed.size), P50=float(np.median(elapsed)),
                           P90=float(np.percentile(elapsed, 90)), P99=float(np.percentile(elapsed, 99)))

    @classmethod
    def results(cls) -> tp.List["Timer.Entry"]:
        if cls._timer_queue:
            torch.cuda.synchronize()
        return [cls.summarise(name, [s.elapsed_time(e) for s, e in events]) for name, events in cls._timer_queue.items()]

    @staticmethod
    def format_table(entries: tp.Sequence["Timer.Entry"]) -> str:
        header = ("Name", "Count", "Median (ms)", "P90 (ms)", "P99 (ms)")
        rows = [(e.name, f"{e.count}", f"{e.P50:.2f}", f"{e.P90:.2f}", f"{e.P99:.2f}") for e in entries]
        widths = [max(len(r[i]) for r in [header] + rows) for i in range(5)]
        def line(r):  # the name column is left-aligned, the figures right-aligned
            return "  ".join([r[0].ljust(widths[0])] + [r[i].rjust(widths[i]) for i in range(1, 5)])
        return "\n".join([line(header), "  ".join("-" * w for w in widths)] + [line(r) for r in rows]) + "\n"

    @classmethod
    def report(cls) -> str:
        return cls.format_table(cls.results())
