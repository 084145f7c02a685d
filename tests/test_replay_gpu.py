"""``bin/trace_run`` on the GPU against the plain implementation: the same requests whole;
most of each in one step and the last 32 tokens one by one; in portions of changing size
down to two tokens; and mixed, up to four live requests with portions of some beside
single tokens of others and a pool so small that pages are used again.  In float32 and in
bfloat16, for six tiny configurations (all but A with sharpened attention, so that single
keys matter).

Tolerances.  float32: 1e-4 absolute on logits of size 1 to 3 (the same comparison with
the kernels restated in float32 torch gives 1e-5).  bfloat16: per configuration, three
times what a restatement with the engine's rounding points (weights, activations and
cache in bfloat16, sums in float32) differs from the plain implementation; the ways of
cutting must agree with one another three times closer than that.  Beside the bound on single
logits, per row: the root-mean-square difference relative to the row's own spread (``BF16_RMS``;
1e-4 in float32), and the engine's argmax must be the plain implementation's or fall short of
its maximum by less than half the tolerance (1e-4 in float32)."""
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import plain_qwen3 as plain
import replay
from tiny import TINIES, make_folder, requests_for, sharpen

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
SHARPEN = {"A": 1.0, "B": 1.5, "C": 1.5, "D": 1.5, "E": 1.5, "F": 1.5}
BF16_TOL = {"A": 0.012, "B": 0.15, "C": 0.3, "D": 0.17, "E": 0.24, "F": 0.32}
# a row's root-mean-square difference relative to the row's standard deviation: two and a half times
# what a B200 shows (0.006, 0.036, 0.045, 0.031, 0.033, 0.031); a logit error of a tenth of the row's spread fails
BF16_RMS = {"A": 0.015, "B": 0.09, "C": 0.11, "D": 0.08, "E": 0.08, "F": 0.08}
F32_TOL = 1e-4


@pytest.fixture(scope="module", params=["A", "B", "C", "D", "E", "F"])
def case(request, tmp_path_factory):
    name = request.param
    tiny = TINIES[name]
    folder = make_folder(tiny, tmp_path_factory.mktemp(f"tiny{name}"))
    if SHARPEN[name] != 1.0:
        sharpen(folder, SHARPEN[name])
    cfg, w = plain.read_model(folder)
    reqs = requests_for(tiny)
    want = {rid: plain.logits_of(cfg, w, toks).numpy() for rid, toks in reqs.items()}
    tb = replay.TraceBuilder()
    replay.whole(tb, reqs)
    replay.tail_one_by_one(tb, reqs)
    replay.portions(tb, reqs)
    replay.mixed(tb, reqs, seed=5)
    return name, tiny, folder, cfg, want, tb


def run_tool(folder, dtype, out, tb, page_size):
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
           "--out", str(out), "--max-tokens", str(tb.max_tokens), "--page-size", str(page_size)]
    res = subprocess.run(cmd, input=tb.text(), capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-3000:]
    done = [l for l in res.stdout.splitlines() if l.startswith("done ")]
    assert done == [f"done {i}" for i in range(len(tb.steps))]


def mode_spread(out, tb, vocab):
    """Largest difference between any way of cutting and the whole-request run, per tag."""
    base, spread = {}, {}
    for step, rows in tb.expect.items():
        got = replay.read_logits(out, step, vocab)
        for r, (name, pos) in enumerate(rows):
            key = (name[1:], pos)
            if name[0] == "w":
                base[key] = got[r]
    for step, rows in tb.expect.items():
        got = replay.read_logits(out, step, vocab)
        for r, (name, pos) in enumerate(rows):
            if name[0] != "w":
                d = float(np.abs(got[r] - base[(name[1:], pos)]).max())
                spread[name[0]] = max(spread.get(name[0], 0.0), d)
    return spread


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_replay_all_ways_of_cutting(case, dtype, tmp_path):
    name, tiny, folder, cfg, want, tb = case
    out = tmp_path / "out"
    run_tool(folder, dtype, out, tb, tiny["page_size"])
    worst, where = replay.compare(out, tb, want, cfg["vocab_size"])
    assert set(worst) == {"w", "t", "p", "m"}
    limit = F32_TOL if dtype == "float32" else BF16_TOL[name]
    assert max(worst.values()) < limit, (worst, where)
    spread = mode_spread(out, tb, cfg["vocab_size"])
    assert max(spread.values()) < limit / 3, spread
    rms, gap, at = replay.row_checks(out, tb, want, cfg["vocab_size"])
    print(f"\n[{name} {dtype}] worst {max(worst.values()):.5f}, row rms / row spread {rms:.5f}, argmax short by {gap:.5f}")
    rms_limit, gap_limit = (1e-4, 1e-4) if dtype == "float32" else (BF16_RMS[name], BF16_TOL[name] / 2)
    assert rms < rms_limit, (rms, at)
    assert gap < gap_limit, gap


def test_first_tokens_and_page_edges(case, tmp_path):
    """The first tokens of a sequence one by one from an empty cache, across a page edge."""
    name, tiny, folder, cfg, want, _ = case
    toks = requests_for(tiny)["0"][:2 * tiny["page_size"] + 3]
    tb = replay.TraceBuilder()
    for i, t in enumerate(toks):
        tb.step([("f0", [t])], end=["f0"] if i == len(toks) - 1 else [])
    out = tmp_path / "out"
    run_tool(folder, "float32", out, tb, tiny["page_size"])
    worst, where = replay.compare(out, tb, want, cfg["vocab_size"])
    assert worst["f"] < F32_TOL, (worst, where)
