"""The same requests through the step function in four ways of cutting, and the comparison of
two runners on them (the bfloat16 kernels against the float32 path of the same weights).

The ways are those of trace replay: each request alone and whole; most of it in one step and
the last tokens one by one; in portions of changing size down to two tokens; and mixed, up to
four live requests with portions of some beside single tokens of others on a pool so small
that pages are used again.  Logits are kept only at the wanted positions, so vocabularies of
real size stay affordable.  ``bench.py`` runs this before it times anything and the tests
run it at real layer sizes; the reference has no counterpart (it has one storage type and
one way of running a prompt, model/src/qwen3_paged_batch.cpp:44-366).
"""
from __future__ import annotations

import random
from typing import Dict, List, Sequence, Tuple

import torch

from .batch import StepEntry
from .runner import ModelRunner

Rows = Dict[Tuple[str, str, int], torch.Tensor]      # (way, request, position) -> logits [vocab]

PORTIONS = (7, 2, 13, 2, 700, 5, 31, 2, 300, 16, 3, 64, 2, 9, 512, 129)
MIXED_PORTIONS = (2, 5, 17, 64, 130, 257, 400)


def wanted_positions(length: int, tail: int = 32, page: int = 16) -> List[int]:
    """Positions worth looking at in a request of ``length`` tokens: the first ones, the edges
    of pages and of the attention kernels' blocks of 64, 128 and 256 rows, and the last ``tail``."""
    marks = {0, 1, 2, page - 1, page, page + 1}
    for edge in (64, 128, 256, 512, 1024, 2048, 4096):
        marks |= {edge - 1, edge, edge + 1}
    marks |= set(range(max(0, length - tail), length))
    return sorted(p for p in marks if 0 <= p < length)


class CutRunner:
    """Feeds requests through ``runner.step`` in one way of cutting and collects the logits at
    the wanted positions."""

    def __init__(self, runner: ModelRunner, requests: Dict[str, Sequence[int]],
                 wanted: Dict[str, Sequence[int]]):
        self.runner, self.requests = runner, {k: list(v) for k, v in requests.items()}
        self.wanted = {k: set(v) for k, v in wanted.items()}
        self.rows: Rows = {}
        self.steps = 0

    def _step(self, way: str, portions: List[Tuple[str, int, int]], end: Sequence[str] = ()) -> None:
        """portions: (request, first position, count)."""
        entries, places = [], []
        for name, start, count in portions:
            want = [p - start for p in range(start, start + count) if p in self.wanted[name]]
            entries.append(StepEntry(f"{way}:{name}", self.requests[name][start:start + count], want))
            places += [(way, name, start + w) for w in want]
        logits = self.runner.step(entries)
        assert logits.shape[0] == len(places)
        for key, row in zip(places, logits):
            self.rows[key] = row.clone()
        for name in end:
            self.runner.release(f"{way}:{name}")
        self.steps += 1

    def whole(self, way: str = "whole") -> None:
        for name, toks in self.requests.items():
            self._step(way, [(name, 0, len(toks))], end=[name])

    def tail_one_by_one(self, tail: int = 32, way: str = "tail") -> None:
        for name, toks in self.requests.items():
            head = max(1, len(toks) - tail)
            self._step(way, [(name, 0, head)], end=[name] if head == len(toks) else [])
            for i in range(head, len(toks)):
                self._step(way, [(name, i, 1)], end=[name] if i == len(toks) - 1 else [])

    def portions(self, sizes: Sequence[int] = PORTIONS, way: str = "portions") -> None:
        for name, toks in self.requests.items():
            i = k = 0
            while i < len(toks):
                n = min(sizes[k % len(sizes)], len(toks) - i)
                k += 1
                self._step(way, [(name, i, n)], end=[name] if i + n == len(toks) else [])
                i += n

    def mixed(self, seed: int = 0, live_max: int = 4, tail: int = 32, sizes: Sequence[int] = MIXED_PORTIONS,
              way: str = "mixed") -> None:
        rng = random.Random(seed)
        waiting = list(self.requests)
        live: List[str] = []
        fed: Dict[str, int] = {}
        while waiting or live:
            while waiting and len(live) < live_max:
                live.append(waiting.pop(0))
                fed[live[-1]] = 0
            chosen = [n for n in live if rng.random() > 0.2] or [live[0]]
            step, ended = [], []
            for name in chosen:
                i, total = fed[name], len(self.requests[name])
                left = total - i
                n = 1 if left <= tail else min(rng.choice(sizes), left - tail)
                step.append((name, i, n))
                fed[name] = i + n
                if fed[name] == total:
                    ended.append(name)
            self._step(way, step, end=ended)
            live = [n for n in live if n not in ended]

    def all_ways(self, seed: int = 0) -> Rows:
        self.whole()
        self.tail_one_by_one()
        self.portions()
        self.mixed(seed)
        return self.rows


def pages_for(requests: Dict[str, Sequence[int]], page_size: int, live_max: int = 4) -> int:
    """Pages that just hold the ``live_max`` longest requests at once: every way of cutting
    then runs on pages that an earlier request has used."""
    longest = sorted((len(t) for t in requests.values()), reverse=True)[:live_max]
    return sum(-(-n // page_size) for n in longest) + 1


def compare(got: Rows, want: Rows, near_tie: float) -> Dict[str, float]:
    """Per way of cutting: the largest absolute difference between ``got`` and ``want`` at the same
    (way, request, position); that difference relative to the spread (standard deviation) of the
    row it lies in (``:relative``); the largest root-mean-square difference of a row relative to
    its spread (``:rms``, which one outlier among 150,000 entries does not move); and the number of
    rows whose argmax in ``got`` is neither the argmax of ``want`` nor within ``near_tie`` of it
    there."""
    out: Dict[str, float] = {}
    assert set(got) == set(want), "the two runs kept different rows"
    for key, row in got.items():
        way = key[0]
        ref = want[key]
        if not bool(torch.isfinite(row).all()):
            raise AssertionError(f"logits at {key} are not finite")
        diff = float((row - ref).abs().max())
        out[way] = max(out.get(way, 0.0), diff)
        spread = max(float(ref.std()), 1e-30)
        out[way + ":relative"] = max(out.get(way + ":relative", 0.0), diff / spread)
        out[way + ":rms"] = max(out.get(way + ":rms", 0.0), float((row - ref).square().mean().sqrt()) / spread)
        pick = int(row.argmax())
        miss = float(ref.max() - ref[pick]) > near_tie
        out[way + ":argmax_misses"] = out.get(way + ":argmax_misses", 0) + int(miss)
    return out


def spread_between_ways(rows: Rows, base: str = "whole") -> Dict[str, float]:
    """Largest difference, relative to the row's largest logit, between each way of cutting and
    the ``base`` way at the same (request, position)."""
    out: Dict[str, float] = {}
    for (way, name, pos), row in rows.items():
        if way == base:
            continue
        ref = rows[(base, name, pos)]
        d = float((row - ref).abs().max()) / max(float(ref.abs().max()), 1e-30)
        out[way] = max(out.get(way, 0.0), d)
    return out
