"""The engine's host side (LLM entry point, scheduler, sampler keys, toy parts) with the
CUDA kernels swapped for torch stand-ins."""
import pytest

import plain_qwen3 as plain
from tiny import TINIES, make_folder, prompt


@pytest.mark.parametrize("budget,blocks", [(256, 32), (8, 32), (8, 5), (8, 4)])
def test_greedy_matches_plain_under_budgets_and_few_pages(tmp_path, cpu_ops, budget, blocks):
    from tiny_llm_infer_b200 import LLM, SamplingParams
    folder = make_folder(TINIES["A"], tmp_path / "m")
    cfg, w = plain.read_model(folder)
    prompts = [prompt(i, n, 256) for i, n in enumerate((5, 17, 33))]
    want = [plain.greedy(cfg, w, p, 8) for p in prompts]
    llm = LLM(str(folder), dtype="float32", max_model_len=128, num_kv_blocks=blocks, block_size=16,
              max_num_batched_tokens=budget, max_num_seqs=4, device="cpu")
    outs = llm.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))
    assert [o.token_ids for o in outs] == want
    # the reference's engine takes 8, 16, 20 and 22 steps for these four settings
    assert llm.engine.counters.steps == {(256, 32): 8, (8, 32): 16, (8, 5): 20, (8, 4): 22}[(budget, blocks)]
    llm.cache.audit()
    assert llm.cache.free_pages() == {None: blocks}


def test_tiny_b_tied_takes_the_reference_engines_steps(tmp_path, cpu_ops):
    """The reference's engine on tiny B with a tied head (tests/golden/tiny_b_tied_engine.json):
    prompts of 1/9/40/70 tokens, 12 greedy tokens each, pages of 8, token budgets 32 and 256, a
    pool that holds everything and one of 14 pages (the longest request alone needs 11).  This
    engine gives the same tokens in the same number of steps."""
    import json
    from pathlib import Path

    from test_plain import b_tied
    from tiny_llm_infer_b200 import LLM, SamplingParams
    meta = json.loads((Path(__file__).parent / "golden" / "tiny_b_tied_engine.json").read_text())
    folder = make_folder(b_tied(), tmp_path / "m")
    for run in meta["runs"]:
        llm = LLM(str(folder), dtype="float32", max_model_len=meta["max_model_len"], num_kv_blocks=run["pages"],
                  block_size=meta["page_size"], max_num_batched_tokens=run["budget"], max_num_seqs=4, device="cpu",
                  overlap_scheduling=False)
        outs = llm.generate(meta["prompts"], SamplingParams(max_tokens=meta["max_tokens"], ignore_eos=True))
        assert [o.token_ids for o in outs] == run["tokens"], run
        assert llm.engine.counters.steps == run["steps"], (run["budget"], run["pages"])
        llm.cache.audit()


def test_preemption_and_sampling_keys(tmp_path, cpu_ops):
    from tiny_llm_infer_b200 import LLM, SamplingParams
    folder = make_folder(TINIES["A"], tmp_path / "m")
    prompts = [prompt(i, 15, 256) for i in range(3)]
    params = [SamplingParams(max_tokens=12, temperature=0.8, ignore_eos=True, seed=7 + i) for i in range(3)]
    runs = []
    for blocks in (12, 5):
        llm = LLM(str(folder), dtype="float32", max_model_len=64, num_kv_blocks=blocks, block_size=16,
                  max_num_batched_tokens=64, max_num_seqs=3, device="cpu")
        runs.append(([o.token_ids for o in llm.generate(prompts, params)], llm.engine.counters.preemptions))
    assert runs[0][1] == 0 and runs[1][1] > 0
    assert runs[0][0] == runs[1][0]            # draws survive preemption and recomputation


def test_toy_parts_on_the_host_side(tmp_path, cpu_ops):
    from test_engine_gpu import run_toy
    run_toy(tmp_path, "cpu")


def test_sandwich_parts_on_the_host_side(tmp_path, cpu_ops):
    from test_engine_gpu import run_sandwich
    run_sandwich(tmp_path, "cpu")


def test_prefix_cache_changes_no_token(tmp_path, cpu_ops):
    """Prompts that begin alike share full pages (the second call finds the pages of the first,
    freed but not yet handed out again); what is generated is what the plain implementation
    generates, with the cache on and off."""
    from tiny_llm_infer_b200 import LLM, SamplingParams
    folder = make_folder(TINIES["A"], tmp_path / "m")
    cfg, w = plain.read_model(folder)
    stem = prompt(1, 40, 256)
    prompts = [stem, stem[:37] + prompt(2, 6, 256), stem[:32], stem + prompt(3, 3, 256)]
    want = [plain.greedy(cfg, w, p, 6) for p in prompts]
    for on in (True, False):
        llm = LLM(str(folder), dtype="float32", max_model_len=128, num_kv_blocks=24, block_size=16,
                  max_num_batched_tokens=64, max_num_seqs=4, device="cpu", enable_prefix_caching=on)
        sp = SamplingParams(max_tokens=6, ignore_eos=True)
        first = llm.generate(prompts[:1], sp)
        rest = llm.generate(prompts[1:], sp)
        assert [o.token_ids for o in first + rest] == want
        llm.cache.audit()
        assert llm.cache.free_pages() == {None: 24}
        # stem[:37] shares 2 pages, stem[:32] one (its last page is computed), stem + 3 two
        assert llm.engine.counters.prefix_cached_tokens == (16 * (2 + 1 + 2) if on else 0)


@pytest.mark.parametrize("blocks,budget", [(32, 64), (6, 8)])
def test_overlapped_scheduling_changes_no_token(tmp_path, cpu_ops, blocks, budget):
    """With the next step scheduled and laid out while the present one runs, requests that
    end on an end-of-sequence token have a row in a step made before that was known: the
    tokens, the finished requests and the pages given back are the same as without."""
    from tiny_llm_infer_b200 import LLM, SamplingParams
    folder = make_folder(TINIES["A"], tmp_path / "m")
    stem = prompt(9, 35, 256)                      # two prompts begin alike: pages are shared while both live
    prompts = [prompt(i, n, 256) for i, n in enumerate((5, 17, 33, 9))] + [stem, stem[:33] + prompt(8, 4, 256)]
    params = [SamplingParams(max_tokens=14, temperature=0.9, seed=11 + i) for i in range(6)]

    def run(overlap, eos):
        llm = LLM(str(folder), dtype="float32", max_model_len=64, num_kv_blocks=blocks, block_size=16,
                  max_num_batched_tokens=budget, max_num_seqs=3, device="cpu", overlap_scheduling=overlap)
        llm.engine.eos = frozenset(eos)
        outs = [o.token_ids for o in llm.generate(prompts, params)]
        llm.cache.audit()
        assert llm.cache.free_pages() == {None: blocks} and llm.cache.free_slots == 3
        assert not llm.engine._flying and llm.engine.is_finished()
        return outs, llm.engine.counters

    free_run, _ = run(False, ())
    # tokens that end some requests early: the third token of one, the last-but-one of another
    eos = {free_run[0][2], free_run[3][12]}
    plain_outs, plain_counters = run(False, eos)
    ahead_outs, ahead_counters = run(True, eos)
    assert any(len(o) < 14 for o in plain_outs)
    for o, full in zip(plain_outs, free_run):
        assert o == full[:len(o)] and (len(o) == 14 or o[-1] in eos)
    assert ahead_outs == plain_outs
    assert ahead_counters.generated_tokens == plain_counters.generated_tokens == sum(map(len, plain_outs))


@pytest.mark.parametrize("seed", [0, 1, 2, 3, 8])
def test_overlapped_scheduling_under_random_workloads(tmp_path, cpu_ops, seed):
    """Random prompts, lengths, limits, pool sizes, budgets and end-of-sequence tokens: the
    engine that schedules ahead gives the tokens of the one that does not and gives every page
    back.  (A request that ends on an end-of-sequence token holds its pages one step longer, so
    the order in which the others are admitted and finish may differ.)"""
    import random
    from tiny_llm_infer_b200 import LLM, SamplingParams
    rng = random.Random(seed)
    folder = make_folder(TINIES["A"], tmp_path / "m")
    n = rng.randint(3, 7)
    prompts = [prompt(100 * seed + i, rng.randint(1, 40), 256) for i in range(n)]
    if rng.random() < 0.5:
        prompts[-1] = prompts[0][:rng.randint(1, len(prompts[0]))] + prompts[-1][:5]     # a shared beginning
    params = [SamplingParams(max_tokens=rng.randint(1, 16), temperature=rng.choice([0.0, 0.8]),
                             top_p=rng.choice([1.0, 0.7]), seed=rng.randint(1, 10 ** 6)) for _ in range(n)]
    blocks, budget, seqs = rng.randint(5, 12), rng.choice([4, 16, 64]), rng.randint(1, 4)
    eos = frozenset(rng.sample(range(256), rng.randint(0, 60)))

    def run(overlap):
        llm = LLM(str(folder), dtype="float32", max_model_len=64, num_kv_blocks=blocks, block_size=16,
                  max_num_batched_tokens=budget, max_num_seqs=seqs, device="cpu", overlap_scheduling=overlap)
        llm.engine.eos = eos
        ids = [llm.engine.add_request(p, s) for p, s in zip(prompts, params)]
        order, results = [], {}
        while not llm.engine.is_finished():
            for r in llm.engine.step():
                order.append(r.request_id)
                results[r.request_id] = r.token_ids
        llm.cache.audit()
        assert llm.cache.free_pages() == {None: blocks} and llm.cache.free_slots == seqs
        assert not llm.engine._flying
        for i, s in zip(ids, params):
            out = results[i]
            assert 1 <= len(out) <= s.max_tokens and all(0 <= t < 256 for t in out)
            assert len(out) == s.max_tokens or out[-1] in eos
            assert not any(t in eos for t in out[:-1])
        return [results[i] for i in ids], order, llm.engine.counters.steps

    ahead, plain_run = run(True), run(False)
    assert ahead[0] == plain_run[0] and sorted(ahead[1]) == sorted(plain_run[1])


@pytest.mark.parametrize("overlap", [True, False])
def test_a_step_that_cannot_be_laid_out_is_taken_back(tmp_path, cpu_ops, overlap):
    """The runner refuses to lay a step out once (as it would a step over its token limit): the
    error reaches the caller, the plan is taken back, and stepping on gives the tokens of a run
    without the fault; nothing is decoded from a cache that lacks its prompt."""
    from tiny_llm_infer_b200 import LLM, SamplingParams
    from tiny_llm_infer_b200.engine import StepError
    folder = make_folder(TINIES["A"], tmp_path / "m")
    prompts = [prompt(i, n, 256) for i, n in enumerate((5, 17, 33, 9))]
    sp = SamplingParams(max_tokens=8, ignore_eos=True)

    def make():
        return LLM(str(folder), dtype="float32", max_model_len=128, num_kv_blocks=16, block_size=16,
                   max_num_batched_tokens=24, max_num_seqs=4, device="cpu", overlap_scheduling=overlap)
    want = [o.token_ids for o in make().generate(prompts, sp)]

    llm = make()
    engine, runner = llm.engine, llm.runner
    ids = [engine.add_request(p, sp) for p in prompts]
    real_prepare, calls = runner.prepare, {"n": 0}

    def prepare(entries):
        calls["n"] += 1
        if calls["n"] == 3:                          # a step that completes one prompt and decodes others
            raise StepError("refused for the test")
        return real_prepare(entries)
    runner.prepare = prepare
    results, errors = {}, 0
    for _ in range(200):
        if engine.is_finished():
            break
        try:
            for r in engine.step():
                results[r.request_id] = r.token_ids
        except StepError:
            errors += 1
    assert errors == 1 and engine.is_finished()
    assert [results[i] for i in ids] == want
    llm.cache.audit()
    assert llm.cache.free_pages() == {None: 16}


def test_an_error_in_a_launched_step_stops_the_engine(tmp_path, cpu_ops):
    """A step fails after it was laid out (a kernel refusing its arguments, a device error): what
    ran and what the cache booked is unknown, so the error is raised, and every later step and
    request is refused instead of running on."""
    from tiny_llm_infer_b200 import LLM, SamplingParams
    from tiny_llm_infer_b200.engine.llm_engine import EngineStopped
    folder = make_folder(TINIES["A"], tmp_path / "m")
    llm = LLM(str(folder), dtype="float32", max_model_len=128, num_kv_blocks=16, block_size=16,
              max_num_batched_tokens=24, max_num_seqs=4, device="cpu")
    engine, runner = llm.engine, llm.runner
    for i, n in enumerate((5, 17, 33)):
        engine.add_request(prompt(i, n, 256), SamplingParams(max_tokens=8, ignore_eos=True))
    engine.step()
    real_run = runner.run

    def run(*a, **kw):
        raise RuntimeError("device error for the test")
    runner.run = run
    with pytest.raises(RuntimeError, match="device error"):
        for _ in range(3):                           # the step launched ahead fails: raised by the step it belongs to
            engine.step()
    runner.run = real_run
    with pytest.raises(EngineStopped):
        for _ in range(3):
            engine.step()
    with pytest.raises(EngineStopped):
        engine.add_request([1, 2, 3])
