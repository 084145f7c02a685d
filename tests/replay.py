"""Traces for ``bin/trace_run`` and the comparison of what it writes with the plain
implementation.  A trace is a list of step records plus, per step, the (request, position)
of every wanted row."""
from __future__ import annotations

import json
import random
from pathlib import Path
from typing import Dict, List, Tuple

import numpy as np


def _round64(n: int) -> int:
    return -(-n // 64) * 64


class TraceBuilder:
    def __init__(self):
        self.steps: List[dict] = []
        self.expect: Dict[int, List[Tuple[str, int]]] = {}
        self._fed: Dict[str, int] = {}
        self.max_tokens = 0

    def step(self, portions: List[Tuple[str, List[int]]], end=(), want_all=True):
        """portions: (request id, its next tokens).  Every fed position is wanted."""
        n = len(self.steps)
        entries, rows = [], []
        for rid, toks in portions:
            start = self._fed.get(rid, 0)
            want = list(range(len(toks))) if want_all else [len(toks) - 1]
            entries.append({"id": rid, "tokens": list(toks), "want": want})
            rows += [(rid, start + w) for w in want]
            self._fed[rid] = start + len(toks)
        self.max_tokens = max(self.max_tokens, sum(_round64(v) for v in self._fed.values()))
        self.steps.append({"step": n, "entries": entries, "end": list(end)})
        if rows:
            self.expect[n] = rows
        for rid in end:
            self._fed.pop(rid)

    def text(self) -> str:
        return "".join(json.dumps(s) + "\n" for s in self.steps)


def whole(tb: TraceBuilder, reqs: Dict[str, List[int]], tag="w"):
    """Each request alone and whole."""
    for rid, toks in reqs.items():
        tb.step([(f"{tag}{rid}", toks)], end=[f"{tag}{rid}"])


def tail_one_by_one(tb: TraceBuilder, reqs, tail=32, tag="t"):
    """Most of it in one step and the last ``tail`` tokens one by one."""
    for rid, toks in reqs.items():
        name = f"{tag}{rid}"
        head = max(1, len(toks) - tail)
        tb.step([(name, toks[:head])])
        for i in range(head, len(toks)):
            tb.step([(name, toks[i:i + 1])], end=[name] if i == len(toks) - 1 else [])
        if head == len(toks):
            tb.step([], end=[name])


def portions(tb: TraceBuilder, reqs, sizes=(7, 2, 13, 2, 5, 31, 2, 16, 3, 64, 2, 9), tag="p"):
    """In portions of changing size, down to two tokens."""
    for rid, toks in reqs.items():
        name, i, k = f"{tag}{rid}", 0, 0
        while i < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - i)
            k += 1
            tb.step([(name, toks[i:i + n])], end=[name] if i + n == len(toks) else [])
            i += n


def mixed(tb: TraceBuilder, reqs, seed=0, live_max=4, tail=32, tag="m"):
    """Up to ``live_max`` requests live: portions of some beside single tokens of others;
    some requests sit a step out; finished ones make room for the waiting ones, whose pages
    are therefore pages that were used before."""
    rng = random.Random(seed)
    waiting = [(f"{tag}{rid}", toks) for rid, toks in reqs.items()]
    live: List[Tuple[str, List[int]]] = []
    fed: Dict[str, int] = {}
    while waiting or live:
        while waiting and len(live) < live_max:
            live.append(waiting.pop(0))
            fed[live[-1][0]] = 0
        chosen = [x for x in live if rng.random() > 0.2] or [live[0]]
        step_portions, ended = [], []
        for name, toks in chosen:
            i = fed[name]
            left = len(toks) - i
            if left <= tail:
                n = 1                                   # decode-like single token
            else:
                n = min(rng.choice([2, 3, 5, 8, 13, 17, 29]), left - tail)
            step_portions.append((name, toks[i:i + n]))
            fed[name] = i + n
            if fed[name] == len(toks):
                ended.append(name)
        tb.step(step_portions, end=ended)
        live = [x for x in live if x[0] not in ended]


def read_logits(out_dir, step: int, vocab: int) -> np.ndarray:
    data = np.fromfile(Path(out_dir) / f"{step}.f32", dtype="<f4")
    assert data.size % vocab == 0, f"step {step}: file size is no multiple of the vocabulary"
    return data.reshape(-1, vocab)


def compare(out_dir, tb: TraceBuilder, plain_logits: Dict[str, np.ndarray], vocab: int):
    """Worst absolute difference per mode tag, and the place of the overall worst.
    ``plain_logits[base id]`` is [T, vocab] of the plain implementation; request names are
    one tag letter followed by the base id."""
    worst: Dict[str, float] = {}
    where = None
    top = 0.0
    for step, rows in tb.expect.items():
        got = read_logits(out_dir, step, vocab)
        assert got.shape[0] == len(rows), f"step {step}: {got.shape[0]} rows written, {len(rows)} wanted"
        assert np.isfinite(got).all(), f"step {step}: logits are not finite"
        for r, (name, pos) in enumerate(rows):
            tag, base = name[0], name[1:]
            d = float(np.abs(got[r].astype(np.float64) - plain_logits[base][pos]).max())
            worst[tag] = max(worst.get(tag, 0.0), d)
            if d > top:
                top, where = d, (step, name, pos)
    return worst, where


def row_checks(out_dir, tb: TraceBuilder, plain_logits: Dict[str, np.ndarray], vocab: int):
    """Two figures that a tolerance on single logits does not give: the largest root-mean-square
    difference of a row relative to the row's own spread (its standard deviation), and the largest
    amount by which the engine's argmax falls short of the plain implementation's maximum in the
    plain implementation's own row (0 where the two pick the same token)."""
    worst_rms, worst_gap, where = 0.0, 0.0, None
    for step, rows in tb.expect.items():
        got = read_logits(out_dir, step, vocab).astype(np.float64)
        for r, (name, pos) in enumerate(rows):
            want = plain_logits[name[1:]][pos]
            rms = float(np.sqrt(np.mean((got[r] - want) ** 2)) / max(float(want.std()), 1e-30))
            gap = float(want.max() - want[int(got[r].argmax())])
            if rms > worst_rms:
                worst_rms, where = rms, (step, name, pos)
            worst_gap = max(worst_gap, gap)
    return worst_rms, worst_gap, where
