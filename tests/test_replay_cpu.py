"""Trace replay through the package's step function, cache manager and tool with the
CUDA kernels swapped for torch stand-ins: checks the host logic (cutting, batching, page
reuse, windows) on a machine without a GPU."""
import importlib.machinery
import importlib.util
import io
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_qwen3 as plain
import replay
from tiny import TINIES, make_folder, requests_for, sharpen

ROOT = Path(__file__).resolve().parent.parent


def load_tool():
    loader = importlib.machinery.SourceFileLoader("trace_run_tool", str(ROOT / "bin" / "trace_run"))
    spec = importlib.util.spec_from_loader("trace_run_tool", loader)
    mod = importlib.util.module_from_spec(spec)
    loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("name", ["A", "C"])
def test_replay_modes_cpu(name, tmp_path, cpu_ops, monkeypatch, capsys):
    tiny = TINIES[name]
    folder = make_folder(tiny, tmp_path / "model")
    sharpen(folder, 2.0)
    cfg, w = plain.read_model(folder)
    reqs = requests_for(tiny, (70, 41, 66, 35, 50))
    want = {rid: plain.logits_of(cfg, w, toks).numpy() for rid, toks in reqs.items()}
    tb = replay.TraceBuilder()
    replay.whole(tb, {k: reqs[k] for k in ("0", "1")})
    replay.tail_one_by_one(tb, {"2": reqs["2"]})
    replay.portions(tb, {"0": reqs["0"]})
    replay.mixed(tb, reqs, seed=3)
    monkeypatch.setattr(sys, "stdin", io.StringIO(tb.text()))
    tool = load_tool()
    rc = tool.main(["--model", str(folder), "--dtype", "float32", "--out", str(tmp_path / "out"),
                    "--max-tokens", str(tb.max_tokens), "--page-size", str(tiny["page_size"]),
                    "--device", "cpu"])
    assert rc == 0
    done = [l for l in capsys.readouterr().out.splitlines() if l.startswith("done ")]
    assert done == [f"done {i}" for i in range(len(tb.steps))]
    worst, where = replay.compare(tmp_path / "out", tb, want, cfg["vocab_size"])
    assert set(worst) == {"w", "t", "p", "m"}
    assert max(worst.values()) < 2e-4, (worst, where)
