"""``do_bench`` / ``do_bench_paired``: CUDA-event timing with an L2 flush before every rep.

Protocol of cutile/src/bench.rs:178-254: at least one warm-up call and then until the warm-up
budget is spent; the rep count comes from one timed estimate and the ``rep`` budget, clamped to
``[min_reps, max_reps]``; before every timed rep a buffer of twice the L2 size is memset so the
rep sees a cold cache (:124-151); the median is the headline (:98-101).
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Callable, List, Tuple

import torch


@dataclass
class BenchOptions:
    warmup_ms: float = 25.0
    rep_ms: float = 100.0
    min_reps: int = 5
    max_reps: int = 1000
    clear_l2: bool = True


class Measurement:
    def __init__(self, times_ms: List[float]):
        self._t = list(times_ms)

    def reps(self) -> int:
        return len(self._t)

    def times_ms(self) -> List[float]:
        return list(self._t)

    def min_ms(self) -> float:
        return min(self._t)

    def mean_ms(self) -> float:
        return sum(self._t) / len(self._t)

    def median_ms(self) -> float:
        return self.quantile_ms(0.5)

    def quantile_ms(self, q: float) -> float:
        s = sorted(self._t)
        q = min(max(q, 0.0), 1.0)
        pos = q * (len(s) - 1)
        lo, hi = int(pos // 1), int(-(-pos // 1))
        if lo == hi:
            return s[lo]
        frac = pos - lo
        return s[lo] * (1.0 - frac) + s[hi] * frac


class L2Clear:
    """Device buffer of ~2x the L2 size (clamped to 64..512 MiB), memset to evict residency."""

    def __init__(self, stream: torch.cuda.Stream):
        props = torch.cuda.get_device_properties(torch.cuda.current_device())
        l2 = int(getattr(props, "L2_cache_size", 64 << 20))
        self.num_bytes = min(max(2 * l2, 64 << 20), 512 << 20)
        self.stream = stream
        self.buf = torch.empty(self.num_bytes, dtype=torch.uint8, device="cuda")

    def clear(self) -> None:
        with torch.cuda.stream(self.stream):
            self.buf.zero_()


def _time_one(stream: torch.cuda.Stream, f: Callable[[torch.cuda.Stream], None]) -> float:
    start = torch.cuda.Event(enable_timing=True)
    end = torch.cuda.Event(enable_timing=True)
    start.record(stream)
    f(stream)
    end.record(stream)
    end.synchronize()
    return start.elapsed_time(end)


def do_bench(stream: torch.cuda.Stream, opts: BenchOptions,
             f: Callable[[torch.cuda.Stream], None]) -> Measurement:
    t0 = time.perf_counter()
    f(stream)
    while (time.perf_counter() - t0) * 1e3 < opts.warmup_ms:
        f(stream)
    est = max(_time_one(stream, f), 1e-4)
    reps = min(max(int(round(opts.rep_ms / est)), opts.min_reps), opts.max_reps)
    l2 = L2Clear(stream) if opts.clear_l2 else None
    times = []
    for _ in range(reps):
        if l2:
            l2.clear()
        times.append(_time_one(stream, f))
    return Measurement(times)


def do_bench_paired(stream: torch.cuda.Stream, opts: BenchOptions,
                    a: Callable[[torch.cuda.Stream], None],
                    b: Callable[[torch.cuda.Stream], None]) -> Tuple[Measurement, Measurement]:
    """Strict A/B/A/B alternation (cutile/src/bench.rs:210-254)."""
    t0 = time.perf_counter()
    a(stream)
    b(stream)
    while (time.perf_counter() - t0) * 1e3 < opts.warmup_ms:
        a(stream)
        b(stream)
    est = max(_time_one(stream, a), 1e-4)
    reps = min(max(int(round(opts.rep_ms / est / 2.0)), opts.min_reps), opts.max_reps)
    l2 = L2Clear(stream) if opts.clear_l2 else None
    ta, tb = [], []
    for _ in range(reps):
        if l2:
            l2.clear()
        ta.append(_time_one(stream, a))
        if l2:
            l2.clear()
        tb.append(_time_one(stream, b))
    return Measurement(ta), Measurement(tb)
