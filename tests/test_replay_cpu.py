"""Trace replay through the package's step function, cache manager and tool with the
CUDA kernels swapped for torch stand-ins: checks the host logic (cutting, batching, page
reuse, windows) on a machine without a GPU."""
import importlib.machinery
import importlib.util
import io
import sys
from pathlib import Path

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


def test_a_step_prepared_ahead_with_a_late_token(tmp_path, cpu_ops):
    """prepare() lays a step out before one of its tokens is known, run() fills it in: the
    logits are those of the same step made in one go; a second prepare() before run(), a
    missing late token and one outside the vocabulary are refused, and the runner can go on."""
    from tiny_llm_infer_b200.cache import CacheManager
    from tiny_llm_infer_b200.engine import ModelRunner, StepEntry, load_model
    from tiny_llm_infer_b200.engine.runner import StepError
    tiny = TINIES["A"]
    folder = make_folder(tiny, tmp_path / "model")
    model, _ = load_model(str(folder), torch.float32, "cpu")
    toks = requests_for(tiny, (20, 9))

    def fresh():
        cache = CacheManager(model.cache_needs(), tiny["page_size"], 16, max_slots=4, max_seq_len=128,
                             dtype=torch.float32, device="cpu")
        return ModelRunner(model, cache, max_batch_tokens=64)

    a, b = toks["0"], toks["1"]
    plain_runner, runner = fresh(), fresh()
    for r in (plain_runner, runner):
        r.step([StepEntry("a", a[:12], []), StepEntry("b", b[:8], [])])
    want = plain_runner.step([StepEntry("a", a[12:], [7]), StepEntry("b", b[8:9], [0])]).clone()
    late = [StepEntry("a", a[12:19] + [-1], [7], late=7), StepEntry("b", [-1], [0], late=0)]
    prepared = runner.prepare(late)
    assert [i for i, _ in prepared.late] == [0, 1]
    with pytest.raises(StepError, match="has not been run"):
        runner.prepare([StepEntry("c", [1, 2], [])])
    with pytest.raises(StepError, match="late tokens"):
        runner.run(prepared, [a[19]])
    prepared = runner.prepare(late)                     # the refusal freed the runner; pages are already reserved
    with pytest.raises(StepError, match="outside"):
        runner.run(prepared, [a[19], 10 ** 6])
    got = runner.run(runner.prepare(late), [a[19], b[8]])
    assert torch.equal(got, want)
    assert late[0].tokens[7] == a[19] and runner.cache.computed("a") == 20 and runner.cache.computed("b") == 9
    runner.cache.audit()
    # the same with the tokens still on the device, as rows of what a step before has sampled
    third = fresh()
    third.step([StepEntry("a", a[:12], []), StepEntry("b", b[:8], [])])
    late = [StepEntry("a", a[12:19] + [-1], [7], late=7), StepEntry("b", [-1], [0], late=0)]
    sampled = torch.tensor([77, b[8], 5, a[19]], dtype=torch.int32)
    with pytest.raises(StepError, match="rows were named"):
        third.run(third.prepare(late), late_source=(sampled, [3]))
    got = third.run(third.prepare(late), late_source=(sampled, [3, 1]))
    assert torch.equal(got, want)
    assert late[0].tokens[7] == -1 and third.cache.computed("a") == 20       # the host has not seen them


def test_selfcheck_ways_of_cutting_cpu(tmp_path, cpu_ops):
    """The four ways of cutting of ``engine.selfcheck`` on tiny A with the stand-in kernels:
    every way leaves a row at every wanted position, all agree with the plain implementation,
    and the pool that just holds four requests ends without a page lost."""
    from tiny_llm_infer_b200.cache import CacheManager
    from tiny_llm_infer_b200.engine import ModelRunner, load_model, selfcheck
    tiny = TINIES["A"]
    folder = make_folder(tiny, tmp_path / "model")
    cfg, w = plain.read_model(folder)
    reqs = requests_for(tiny, (150, 41, 66, 35, 50))
    wanted = {k: selfcheck.wanted_positions(len(v), tail=8) for k, v in reqs.items()}
    model, _ = load_model(folder, torch.float32, "cpu")
    pages = selfcheck.pages_for(reqs, 16)
    cache = CacheManager(model.cache_needs(), 16, pages, max_slots=4, max_seq_len=192, dtype=torch.float32,
                         device="cpu")
    runner = ModelRunner(model, cache, max_batch_tokens=192)
    cut = selfcheck.CutRunner(runner, reqs, wanted)
    rows = cut.all_ways(seed=1)
    cache.audit()
    assert len(rows) == 4 * sum(len(v) for v in wanted.values())
    want = {}
    for name, toks in reqs.items():
        full = plain.logits_of(cfg, w, toks).to(torch.float32)
        for way in ("whole", "tail", "portions", "mixed"):
            for pos in wanted[name]:
                want[(way, name, pos)] = full[pos]
    result = selfcheck.compare(rows, want, near_tie=1e-5)
    assert max(result[k] for k in ("whole", "tail", "portions", "mixed")) < 2e-4, result
    assert all(result[k + ":argmax_misses"] == 0 for k in ("whole", "tail", "portions", "mixed"))
    assert max(selfcheck.spread_between_ways(rows).values()) < 1e-3
    # a wrong row is seen
    key = ("mixed", "0", wanted["0"][-1])
    rows[key] = rows[key] + 1.0 * (torch.arange(rows[key].numel()) == 3)
    assert selfcheck.compare(rows, want, near_tie=1e-5)["mixed"] > 0.9
