"""Autotuner over the fixed table of precompiled configurations.

Mirror of cutile/src/tune.rs: ``Config`` with a derived stable id (:70-104), ``space_hash`` =
FNV-1a over the sorted ids (:127-138), ``Trial``/``TrialState`` (:143-173), exhaustive
``GridSearch`` with resume (:202-252), ``best_config`` (:256-277), ``Autotuner`` with prune /
budget / bench / log and a paired A/B/A/B runoff of the two best candidates (:312-455,503-616),
and the JSONL ``TrialLog`` headed by an identity record that refuses a foreign log (:647-757).
The JSON field names are the reference's, so logs are interchangeable.

Where the reference tunes open-ended tile-size generics through its JIT, candidates here are rows
of ``b200tile_query_configs``; a candidate the library does not contain surfaces as an error from
``setup`` and is recorded as ``Invalid`` -- the search goes on.
"""
from __future__ import annotations

import json
import math
import os
import time
from dataclasses import dataclass, field
from typing import Callable, Dict, List, Optional, Sequence, Tuple, Union

from .benching import BenchOptions, Measurement, do_bench, do_bench_paired

ParamValue = Union[int, str]


def _quote_key(k: str) -> str:
    return json.dumps(k) if any(ch in k for ch in '=,"') else k


class Config:
    """Ordered parameter map with an id of the form ``k1=v1,k2=v2`` (keys sorted)."""

    def __init__(self, params: Dict[str, ParamValue]):
        self.params: Dict[str, ParamValue] = dict(sorted(params.items()))
        parts = []
        for k, v in self.params.items():
            if isinstance(v, bool) or not isinstance(v, (int, str)):
                raise TypeError("config values are integers or strings")
            parts.append(f"{_quote_key(k)}={v}" if isinstance(v, int) else
                         f"{_quote_key(k)}={json.dumps(v)}")
        self.id = ",".join(parts)

    def int(self, key: str) -> Optional[int]:
        v = self.params.get(key)
        return v if isinstance(v, int) and not isinstance(v, bool) else None

    def str(self, key: str) -> Optional[str]:
        v = self.params.get(key)
        return v if isinstance(v, str) else None

    def __eq__(self, other) -> bool:
        return isinstance(other, Config) and self.id == other.id

    def __repr__(self) -> str:
        return f"Config({self.id})"


def space_hash(configs: Sequence[Config]) -> str:
    h = 0xCBF29CE484222325
    for cid in sorted(c.id for c in configs):
        for b in cid.encode("utf-8") + b"\x00":
            h ^= b
            h = (h * 0x100000001B3) & 0xFFFFFFFFFFFFFFFF
    return f"{h:016x}"


@dataclass
class Trial:
    config_id: str
    state: Dict  # {"Measured": {median_ms, min_ms, reps}} | {"Invalid": {reason}}

    @staticmethod
    def measured(config_id: str, m: Measurement) -> "Trial":
        if m.reps() == 0:
            return Trial.invalid(config_id, "no timed reps (check BenchOptions)")
        return Trial(config_id, {"Measured": {"median_ms": m.median_ms(), "min_ms": m.min_ms(),
                                              "reps": m.reps()}})

    @staticmethod
    def invalid(config_id: str, reason: str) -> "Trial":
        return Trial(config_id, {"Invalid": {"reason": reason}})

    def median_ms(self) -> Optional[float]:
        m = self.state.get("Measured")
        return None if m is None else float(m["median_ms"])

    def to_json(self) -> str:
        return json.dumps({"config_id": self.config_id, "state": self.state})

    @staticmethod
    def from_json(line: str) -> Optional["Trial"]:
        try:
            d = json.loads(line)
            st = d["state"]
            if not isinstance(st, dict) or not (("Measured" in st) ^ ("Invalid" in st)):
                return None
            return Trial(str(d["config_id"]), st)
        except (ValueError, KeyError, TypeError):
            return None


def best_config(configs: Sequence[Config], trials: Sequence[Trial]) -> Optional[Config]:
    best: Optional[Tuple[Config, float]] = None
    by_id = {c.id: c for c in configs}
    for t in trials:
        ms = t.median_ms()
        if ms is None or not math.isfinite(ms):
            continue
        c = by_id.get(t.config_id)
        if c is None:
            continue
        if best is None or ms < best[1]:
            best = (c, ms)
    return None if best is None else best[0]


def top_two(configs: Sequence[Config], trials: Sequence[Trial]
            ) -> Optional[Tuple[Config, Optional[Config]]]:
    ranked: List[List] = []
    by_id = {c.id: c for c in configs}
    for t in trials:
        ms = t.median_ms()
        if ms is None or not math.isfinite(ms) or t.config_id not in by_id:
            continue
        for entry in ranked:
            if entry[0].id == t.config_id:
                entry[1] = min(entry[1], ms)
                break
        else:
            ranked.append([by_id[t.config_id], ms])
    ranked.sort(key=lambda e: e[1])
    if not ranked:
        return None
    return ranked[0][0], (ranked[1][0] if len(ranked) > 1 else None)


class TrialLog:
    """Append-only JSONL log headed by ``{"log_schema":1,"tuner":...,"space":...}``."""

    def __init__(self, path: Optional[str], tuner: str, space: str):
        self._file = None
        self.existing: List[Trial] = []
        if path is None:
            return
        expected = {"log_schema": 1, "tuner": tuner, "space": space}
        fresh, needs_newline = True, False
        try:
            with open(path, "r", encoding="utf-8") as fh:
                contents = fh.read()
        except FileNotFoundError:
            contents = ""
        except OSError as e:
            raise ValueError(f"trial log {path} is unreadable: {e}") from None
        if contents.strip():
            lines = contents.splitlines()
            try:
                header = json.loads(lines[0])
                if not isinstance(header, dict) or set(header) != set(expected):
                    raise ValueError
            except ValueError:
                raise ValueError(f"trial log {path} has no valid header; delete it or point "
                                 ".log() elsewhere") from None
            if header != expected:
                raise ValueError(
                    f"trial log {path} belongs to tuner {header['tuner']!r} (space "
                    f"{header['space']}), not {tuner!r} (space {space}); delete it or point "
                    ".log() elsewhere")
            self.existing = [t for t in (Trial.from_json(l) for l in lines[1:]) if t is not None]
            needs_newline = not contents.endswith("\n")
            fresh = False
        try:
            self._file = open(path, "w" if fresh else "a", encoding="utf-8")
        except OSError as e:
            raise ValueError(f"trial log {path} cannot be opened for append: {e}") from None
        if needs_newline:
            self._file.write("\n")
        if fresh:
            self._file.write(json.dumps(expected) + "\n")
        self._file.flush()

    def existing_trials(self) -> List[Trial]:
        return list(self.existing)

    def append(self, trial: Trial) -> None:
        if self._file is not None:
            try:
                self._file.write(trial.to_json() + "\n")
                self._file.flush()
            except OSError:
                pass

    def close(self) -> None:
        if self._file is not None:
            self._file.close()
            self._file = None


class GridSearch:
    """Visits every candidate once in declaration order; resumed *measured* trials of candidates
    still in the space are not re-measured, resumed Invalid ones are retried."""

    def __init__(self):
        self.known: List[Trial] = []

    def resume(self, known: Sequence[Trial]) -> "GridSearch":
        self.known = list(known)
        return self

    def search(self, oracle) -> List[Trial]:
        current = {c.id for c in oracle.configs()}
        trials = [t for t in self.known if t.config_id in current and t.median_ms() is not None]
        self.known = []
        visited = {t.config_id for t in trials}
        for i, c in enumerate(oracle.configs()):
            if c.id in visited:
                continue
            if oracle.budget_remaining() == 0.0:
                break
            trials.append(oracle.measure(i))
        return trials


@dataclass
class Output:
    trials: List[Trial]
    best: Optional[Config]


class _BenchOracle:
    def __init__(self, configs, stream, setup, bench, deadline, log, bench_fn, paired_fn):
        self._configs = configs
        self.stream = stream
        self.setup = setup
        self.bench = bench
        self.deadline = deadline
        self.log = log
        self._bench_fn = bench_fn
        self._paired_fn = paired_fn

    def configs(self) -> List[Config]:
        return self._configs

    def measure(self, index: int) -> Trial:
        config = self._configs[index]
        try:
            f = self.setup(self.stream, config)
            trial = Trial.measured(config.id, self._bench_fn(self.stream, self.bench, f))
        except Exception as e:  # a bad candidate never aborts the search (tune.rs:503-514)
            trial = Trial.invalid(config.id, str(e))
        self.log.append(trial)
        return trial

    def budget_remaining(self) -> Optional[float]:
        if self.deadline is None:
            return None
        return max(self.deadline - time.monotonic(), 0.0)


class Autotuner:
    def __init__(self, name: str):
        self.name = name
        self._configs: List[Config] = []
        self._prune: List[Callable[[Config], bool]] = []
        self._budget_s: Optional[float] = None
        self._bench = BenchOptions()
        self._log_path: Optional[str] = None
        # injectable for CPU-only tests
        self._bench_fn = do_bench
        self._paired_fn = do_bench_paired

    def configs(self, configs: Sequence[Config]) -> "Autotuner":
        self._configs = list(configs)
        return self

    def prune(self, keep: Callable[[Config], bool]) -> "Autotuner":
        self._prune.append(keep)
        return self

    def budget(self, seconds: float) -> "Autotuner":
        self._budget_s = float(seconds)
        return self

    def bench(self, opts: BenchOptions) -> "Autotuner":
        self._bench = opts
        return self

    def log(self, path: str) -> "Autotuner":
        self._log_path = os.fspath(path)
        return self

    def run(self, stream, setup) -> Output:
        return self.run_with(None, stream, setup)

    def run_with(self, searcher, stream, setup) -> Output:
        configs = [c for c in self._configs if all(keep(c) for keep in self._prune)]
        log = TrialLog(self._log_path, self.name, space_hash(configs))
        try:
            if searcher is None:
                searcher = GridSearch().resume(log.existing_trials())
            deadline = None if self._budget_s is None else time.monotonic() + self._budget_s
            oracle = _BenchOracle(configs, stream, setup, self._bench, deadline, log,
                                  self._bench_fn, self._paired_fn)
            trials = searcher.search(oracle)
            tt = top_two(configs, trials)
            if tt is None:
                return Output(trials, None)
            a, b = tt
            if b is None or oracle.budget_remaining() == 0.0:
                return Output(trials, a)
            return Output(trials, self._runoff(oracle, a, b, trials, log))
        finally:
            log.close()

    def _runoff(self, oracle: _BenchOracle, a: Config, b: Config, trials: List[Trial],
                log: TrialLog) -> Config:
        """Contemporaneous A/B/A/B re-measurement decides between the two best (tune.rs:570-616)."""
        fns = []
        for cfg, other in ((a, b), (b, a)):
            try:
                fns.append(oracle.setup(oracle.stream, cfg))
            except Exception as e:
                t = Trial.invalid(cfg.id, f"runoff setup failed: {e}")
                log.append(t)
                trials.append(t)
                return other
        try:
            ma, mb = self._paired_fn(oracle.stream, oracle.bench, fns[0], fns[1])
        except Exception:
            return a  # not attributable to either finalist: sequential medians stand
        ta, tb = Trial.measured(a.id, ma), Trial.measured(b.id, mb)
        for t in (ta, tb):
            log.append(t)
            trials.append(t)
        key = lambda t: (t.median_ms() if t.median_ms() is not None and
                         math.isfinite(t.median_ms()) else math.inf)
        return a if key(ta) <= key(tb) else b


def library_configs(kernel: str, dtype: str) -> List[Config]:
    """Candidates = the precompiled configurations the library reports for ``kernel``/``dtype``."""
    from . import _lib
    lib = _lib.load()
    n = lib.b200tile_query_configs(kernel.encode(), dtype.encode(), None, 0)
    arr = (_lib.ConfigC * max(n, 1))()
    lib.b200tile_query_configs(kernel.encode(), dtype.encode(), arr, n)
    return [Config({"id": arr[i].id, "BM": arr[i].bm, "BN": arr[i].bn, "BK": arr[i].bk,
                    "stages": arr[i].stages, "num_cta_in_cga": arr[i].num_cta_in_cga,
                    "occupancy": arr[i].occupancy}) for i in range(n)]
