"""Generation through the Python entry point on the GPU: greedy tokens against the plain
implementation under several budgets and pool sizes (with preemption), long decoding,
temperature sampling that does not depend on batching, and the generality of the parts:
a toy mixer with state of its own and a run order that names a layer twice and lets a
layer read another layer's cache, all registered from this file."""
import json

import pytest
import torch

import plain_qwen3 as plain
from tiny import TINIES, make_folder, prompt

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    out = {}
    for name in ("A", "B", "C", "E"):
        out[name] = make_folder(TINIES[name], tmp_path_factory.mktemp(f"m{name}"))
    return out


def teacher_forced_ok(cfg, w, prompt_ids, generated, margin):
    """Every generated token is the plain implementation's argmax given the same prefix,
    or within ``margin`` of it (bfloat16 may swap near-ties)."""
    ids = list(prompt_ids) + list(generated)
    logits = plain.logits_of(cfg, w, ids[:-1]).numpy()
    for i, tok in enumerate(generated):
        row = logits[len(prompt_ids) - 1 + i]
        if row[tok] < row.max() - margin:
            return False, (i, tok, int(row.argmax()), float(row.max() - row[tok]))
    return True, None


@pytest.mark.parametrize("name", ["A", "B"])
@pytest.mark.parametrize("budget,blocks", [(256, 64), (8, 64), (8, 12), (32, 9)])
def test_greedy_float32_equals_plain(folders, name, budget, blocks):
    from tiny_llm_infer_b200 import LLM, SamplingParams
    tiny = TINIES[name]
    cfg, w = plain.read_model(folders[name])
    prompts = [prompt(i, n, cfg["vocab_size"]) for i, n in enumerate((5, 17, 33, 1))]
    want = [plain.greedy(cfg, w, p, 8) for p in prompts]
    llm = LLM(str(folders[name]), dtype="float32", max_model_len=128, num_kv_blocks=blocks,
              block_size=tiny["page_size"], max_num_batched_tokens=budget, max_num_seqs=4)
    outs = llm.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))
    assert [o.token_ids for o in outs] == want
    llm.cache.audit()
    assert all(v == blocks for v in llm.cache.free_pages().values())


def test_preemption_recomputes_and_still_matches(folders):
    from tiny_llm_infer_b200 import LLM, SamplingParams
    cfg, w = plain.read_model(folders["A"])
    prompts = [prompt(i, 15, 256) for i in range(3)]
    want = [plain.greedy(cfg, w, p, 20) for p in prompts]
    llm = LLM(str(folders["A"]), dtype="float32", max_model_len=64, num_kv_blocks=5, block_size=16,
              max_num_batched_tokens=64, max_num_seqs=3)
    outs = llm.generate(prompts, SamplingParams(max_tokens=20, ignore_eos=True))
    assert llm.engine.counters.preemptions > 0
    assert [o.token_ids for o in outs] == want


@pytest.mark.parametrize("name", ["B", "C"])
def test_long_decoding(folders, name):
    """300 tokens decoded one by one after a short prompt, across many pages (and, for C,
    far past the window), each checked against the plain implementation on the same prefix."""
    from tiny_llm_infer_b200 import LLM, SamplingParams
    tiny = TINIES[name]
    cfg, w = plain.read_model(folders[name])
    p = prompt(7, 9, cfg["vocab_size"])
    for dtype, margin in (("float32", 1e-4), ("bfloat16", 0.08)):
        llm = LLM(str(folders[name]), dtype=dtype, max_model_len=320, num_kv_blocks=48,
                  block_size=tiny["page_size"], max_num_seqs=2)
        out = llm.generate([p], SamplingParams(max_tokens=300, ignore_eos=True))[0]
        assert len(out.token_ids) == 300
        ok, info = teacher_forced_ok(cfg, w, p, out.token_ids, margin)
        assert ok, (dtype, info)


@pytest.mark.parametrize("budget", [1024, 160])
def test_long_prompts_head_width_128(folders, budget):
    """Prompts longer than the 128-row blocks of the tcgen05 prompt kernel (whole, and cut by
    a budget that is no multiple of the block), then decoding, in bfloat16 against the plain
    implementation on the same prefix."""
    from tiny_llm_infer_b200 import LLM, SamplingParams
    tiny = TINIES["E"]
    cfg, w = plain.read_model(folders["E"])
    prompts = [prompt(20 + i, n, cfg["vocab_size"]) for i, n in enumerate((300, 129, 257))]
    llm = LLM(str(folders["E"]), dtype="bfloat16", max_model_len=400, num_kv_blocks=40,
              block_size=tiny["page_size"], max_num_batched_tokens=budget, max_num_seqs=3)
    outs = llm.generate(prompts, SamplingParams(max_tokens=24, ignore_eos=True))
    for p, o in zip(prompts, outs):
        assert len(o.token_ids) == 24
        ok, info = teacher_forced_ok(cfg, w, p, o.token_ids, 0.08)
        assert ok, info


@pytest.mark.parametrize("prompt_graphs", [False, True])
def test_short_portions_of_a_long_prompt_share_out_their_keys(tmp_path, monkeypatch, prompt_graphs):
    """A prompt of 1500 tokens under a budget of 128: a step then has three blocks of query rows
    and up to 24 tiles of keys, so the full-attention layer cuts every block's keys into runs
    for several blocks and combines them (the windowed layer never sees enough keys).  With
    ``prompt_graphs`` the steps, which repeat their layout, are replayed as graphs, the context
    bucket deciding the number of runs.  Generated tokens against the plain implementation on
    the same prefix."""
    import dataclasses
    from tiny_llm_infer_b200 import LLM, SamplingParams, ops
    tiny = dict(TINIES["E"])
    tiny["cfg"] = dataclasses.replace(tiny["cfg"], max_position_embeddings=2048)
    folder = make_folder(tiny, tmp_path / "long")
    cfg, w = plain.read_model(folder)
    seen = []
    inner = ops.paged_attention_prefill_tcgen05

    def spy(*args, **kwargs):
        seen.append(args[13] if len(args) > 13 else kwargs.get("splits", 1))
        return inner(*args, **kwargs)
    monkeypatch.setattr(ops, "paged_attention_prefill_tcgen05", spy)
    p = prompt(77, 1500, cfg["vocab_size"])
    llm = LLM(str(folder), dtype="bfloat16", max_model_len=1600, num_kv_blocks=60, block_size=tiny["page_size"],
              max_num_batched_tokens=128, max_num_seqs=2, prompt_graphs=prompt_graphs)
    out = llm.generate([p], SamplingParams(max_tokens=12, ignore_eos=True))[0]
    assert 2 in seen and 1 in seen, sorted(set(seen))
    ok, info = teacher_forced_ok(cfg, w, p, out.token_ids, 0.08)
    assert ok, info


def test_prefix_cache_on_the_gpu(folders):
    """Shared beginnings: the pages of an earlier prompt are read instead of computed again, by
    live requests and after the earlier one has ended; float32 tokens equal the plain
    implementation's, bfloat16 ones are within its margin.  A model with a windowed layer (E)
    shares nothing and is none the worse for the option."""
    from tiny_llm_infer_b200 import LLM, SamplingParams
    for name, dtype, margin in (("B", "float32", None), ("B", "bfloat16", 0.08), ("E", "bfloat16", 0.08)):
        tiny = TINIES[name]
        cfg, w = plain.read_model(folders[name])
        ps = tiny["page_size"]
        stem = prompt(31, 5 * ps + 3, cfg["vocab_size"])
        prompts = [stem, stem[:4 * ps + 1] + prompt(32, 9, cfg["vocab_size"]), stem[:2 * ps],
                   stem + prompt(33, 2 * ps, cfg["vocab_size"])]
        llm = LLM(str(folders[name]), dtype=dtype, max_model_len=400, num_kv_blocks=40, block_size=ps,
                  max_num_batched_tokens=512, max_num_seqs=4)
        sp = SamplingParams(max_tokens=10, ignore_eos=True)
        outs = llm.generate(prompts[:1], sp) + llm.generate(prompts[1:], sp)
        assert llm.engine.counters.prefix_cached_tokens == (ps * (4 + 1 + 5) if name == "B" else 0)
        for p, o in zip(prompts, outs):
            if margin is None:
                assert o.token_ids == plain.greedy(cfg, w, p, 10)
            else:
                ok, info = teacher_forced_ok(cfg, w, p, o.token_ids, margin)
                assert ok, info
        llm.cache.audit()


def test_eos_stops_and_is_ignored_on_request(folders, tmp_path):
    from tiny_llm_infer_b200 import LLM, SamplingParams
    cfg, w = plain.read_model(folders["A"])
    p = prompt(3, 12, 256)
    ref = plain.greedy(cfg, w, p, 6)
    raw = json.loads((folders["A"] / "config.json").read_text())
    raw["eos_token_id"] = ref[2]
    folder = tmp_path / "eos"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(raw))
    (folder / "model.safetensors").write_bytes((folders["A"] / "model.safetensors").read_bytes())
    llm = LLM(str(folder), dtype="float32", max_model_len=64, num_kv_blocks=8)
    stop_at = ref.index(ref[2]) + 1
    assert llm.generate([p], SamplingParams(max_tokens=6))[0].token_ids == ref[:stop_at]
    assert llm.generate([p], SamplingParams(max_tokens=6, ignore_eos=True))[0].token_ids == ref


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_overlapped_scheduling_with_requests_that_end_early(folders, tmp_path, dtype):
    """Requests that end on an end-of-sequence token have a row in the step launched before that was
    known, and the step at which a waiting request is admitted moves with it, so the rows that share
    a step (and with them, in bfloat16, the product kernel and the last bits) can differ between a
    run with the overlap and one without.  In float32 the tokens are equal; in bfloat16 every token
    of either run is the plain implementation's choice for its own prefix or within its margin, each
    request ends on an end-of-sequence token or at its length, and no page is lost."""
    from tiny_llm_infer_b200 import LLM, SamplingParams
    cfg, w = plain.read_model(folders["B"])
    prompts = [prompt(20 + i, n, cfg["vocab_size"]) for i, n in enumerate((5, 17, 33, 9, 40, 12))]
    greedy = [plain.greedy(cfg, w, p, 10) for p in prompts]
    eos = sorted({g[3] for g in greedy[:3]} | {greedy[4][6]})      # some requests stop after a few tokens
    raw = json.loads((folders["B"] / "config.json").read_text())
    raw["eos_token_id"] = eos
    folder = tmp_path / "eos"
    folder.mkdir()
    (folder / "config.json").write_text(json.dumps(raw))
    (folder / "model.safetensors").write_bytes((folders["B"] / "model.safetensors").read_bytes())
    runs = []
    for overlap in (True, False):
        llm = LLM(str(folder), dtype=dtype, max_model_len=128, num_kv_blocks=24, block_size=8,
                  max_num_batched_tokens=32, max_num_seqs=3, overlap_scheduling=overlap)
        outs = llm.generate(prompts, SamplingParams(max_tokens=10))
        runs.append([o.token_ids for o in outs])
        llm.cache.audit()
        assert llm.cache.free_pages() == {None: 24}
        for p, toks in zip(prompts, runs[-1]):
            assert 0 < len(toks) <= 10 and (len(toks) == 10 or toks[-1] in eos) and not set(toks[:-1]) & set(eos)
            ok, info = teacher_forced_ok(cfg, w, p, toks, 1e-4 if dtype == "float32" else 0.08)
            assert ok, info
    assert any(len(t) < 10 for t in runs[0])
    if dtype == "float32":
        assert runs[0] == runs[1]


def test_temperature_draws_do_not_depend_on_batching(folders):
    from tiny_llm_infer_b200 import LLM, SamplingParams
    cfg, w = plain.read_model(folders["B"])
    prompts = [prompt(i, n, cfg["vocab_size"]) for i, n in enumerate((1, 9, 40, 70))]
    params = [SamplingParams(max_tokens=12, temperature=0.7, ignore_eos=True, seed=100 + i) for i in range(4)]
    runs = []
    for budget, blocks, seqs in ((256, 64, 4), (32, 64, 4), (32, 20, 4), (256, 64, 1)):
        llm = LLM(str(folders["B"]), dtype="float32", max_model_len=128, num_kv_blocks=blocks, block_size=8,
                  max_num_batched_tokens=budget, max_num_seqs=seqs)
        runs.append([o.token_ids for o in llm.generate(prompts, params)])
    assert runs[0] == runs[1] == runs[2] == runs[3]
    assert len({tuple(r) for r in runs[0]}) == 4                       # different seeds, different draws
    # the first draw of request 2 restated on the host from the plain logits
    from tiny_llm_infer_b200.sampling import draw_key
    scores = plain.gumbel_scores(plain.logits_of(cfg, w, prompts[2])[-1].numpy(), 0.7, draw_key(102, 0))
    assert scores[runs[0][2][0]] >= scores.max() - 1e-3
    top = SamplingParams(max_tokens=5, temperature=1.0, top_p=0.3, ignore_eos=True, seed=5)
    llm = LLM(str(folders["B"]), dtype="float32", max_model_len=128, num_kv_blocks=32, block_size=8)
    toks = llm.generate([prompts[1]], top)[0].token_ids
    keep = plain.nucleus(plain.logits_of(cfg, w, prompts[1])[-1].numpy(), 1.0, 0.3)
    assert toks[0] in set(keep.tolist())


def test_request_checks(folders):
    from tiny_llm_infer_b200 import LLM, SamplingParams
    llm = LLM(str(folders["A"]), dtype="bfloat16", max_model_len=32, num_kv_blocks=4)
    eng = llm.engine
    for bad, match in (((list(range(33)), SamplingParams()), "max_model_len"),
                       (([], SamplingParams()), "prompt is empty"),
                       (([1], SamplingParams(max_tokens=0)), "max_tokens is 0"),
                       (([1, 2], SamplingParams(max_tokens=32)), "leaves room for 31"),
                       (([1], SamplingParams(top_p=0.0)), "top_p"),
                       (([1], SamplingParams(temperature=-1.0)), "temperature"),
                       (([300], SamplingParams(max_tokens=1)), "outside")):
        with pytest.raises(ValueError, match=match):
            eng.add_request(*bad)
    assert eng.is_finished()


def run_toy(tmp_path, device):
    from toys import register_toys, toy_plain
    ToyConfig = register_toys()
    from tiny_llm_infer_b200.cache import CacheManager
    from tiny_llm_infer_b200.engine import ModelRunner, StepEntry, load_model
    from tiny_llm_infer_b200.weights import write_random_model
    folder = write_random_model(tmp_path / "toy", ToyConfig(), seed=4, std=0.15, norm_range=(0.7, 1.3))
    _, w = plain.read_model(folder)
    model, cfg = load_model(folder, torch.float32, device)
    needs = model.cache_needs()
    assert sum(1 for c, s in needs.values() if s is not None) == 2        # two visits of the stateful layer
    assert sum(1 for c, s in needs.values() if c is not None) == 3        # cache 10 is shared, two more
    cache = CacheManager(needs, 8, 24, 3, 128, torch.float32, device)
    runner = ModelRunner(model, cache, 256)
    a, b = prompt(1, 50, 160), prompt(2, 37, 160)
    want_a, want_b = toy_plain(w, a, 1e-5), toy_plain(w, b, 1e-5)
    got_a, got_b, ia, ib = [], [], 0, 0
    for na, nb in ((7, 0), (2, 20), (13, 1), (1, 1), (1, 15), (26, 0)):
        entries = []
        if na:
            entries.append(StepEntry("a", a[ia:ia + na], list(range(na))))
        if nb:
            entries.append(StepEntry("b", b[ib:ib + nb], list(range(nb))))
        out = runner.step(entries).cpu().double()
        got_a.append(out[:na]), got_b.append(out[na:])
        ia, ib = ia + na, ib + nb
    assert (torch.cat(got_a) - want_a).abs().max() < 2e-4
    assert (torch.cat(got_b) - want_b).abs().max() < 2e-4
    runner.release("a")
    whole = runner.step([StepEntry("c", a, list(range(50)))]).cpu().double()     # slot and state used again
    assert (whole - want_a).abs().max() < 2e-4


def test_toy_parts_and_run_order_need_no_change_to_the_framework(tmp_path):
    """A stateful mixer, a feed-forward with a router over experts, a position encoding the
    kernels do not know (and a partial rotary one), a layer run twice and a layer reading
    another's cache: registered from the tests, built from a folder, stepped in portions
    and mixed with a second request, compared with a plain restatement."""
    run_toy(tmp_path, "cuda:0")


def run_sandwich(tmp_path, device):
    """A block of four norms, a block with two mixers (two caches per visit, named in the run order) and
    a mixer whose cache is one vector per token: built from a folder, pool sized through the parts' own
    ``workspace_floats``, stepped in portions beside a second request, against a plain restatement."""
    from toys import register_sandwich, sandwich_plain
    Config = register_sandwich()
    from tiny_llm_infer_b200.cache import CacheManager
    from tiny_llm_infer_b200.engine import ModelRunner, StepEntry, load_model
    from tiny_llm_infer_b200.weights import write_random_model
    folder = write_random_model(tmp_path / "sandwich", Config(), seed=6, std=0.15, norm_range=(0.7, 1.3))
    _, w = plain.read_model(folder)
    model, cfg = load_model(folder, torch.float32, device)
    needs = model.cache_needs()
    # layer 0 visited twice (a cache each), layer 1 once with the two caches the run order names
    assert sorted(needs) == [7, 8, 9, 10]
    assert needs[8][0].planes == ((1, 24),) and needs[7][0].planes == ((1, 16), (1, 16))
    per_page = CacheManager.bytes_per_page(needs, 8, torch.float32)
    assert per_page == {None: 4 * 8 * (3 * 2 * 16 + 24)}
    assert model.workspace_floats(10, 2) == 6 * 10 * 40 + 10 * 3 * 56 + 2 * 120    # the SwiGLU is the widest part
    cache = CacheManager(needs, 8, 24, 3, 128, torch.float32, device)
    assert cache.kv[8].shape == (24, 1, 1, 8, 24) and cache.kv[7].shape == (24, 2, 1, 8, 16)
    runner = ModelRunner(model, cache, 256)
    a, b = prompt(3, 50, 120), prompt(4, 37, 120)
    want_a, want_b = sandwich_plain(w, a, 1e-5), sandwich_plain(w, b, 1e-5)
    got_a, got_b, ia, ib = [], [], 0, 0
    for na, nb in ((7, 0), (2, 20), (13, 1), (1, 1), (1, 15), (26, 0)):
        entries = []
        if na:
            entries.append(StepEntry("a", a[ia:ia + na], list(range(na))))
        if nb:
            entries.append(StepEntry("b", b[ib:ib + nb], list(range(nb))))
        out = runner.step(entries).cpu().double()
        got_a.append(out[:na]), got_b.append(out[na:])
        ia, ib = ia + na, ib + nb
    assert (torch.cat(got_a) - want_a).abs().max() < 2e-4
    assert (torch.cat(got_b) - want_b).abs().max() < 2e-4
    runner.release("a")
    runner.release("b")
    cache.audit()
    whole = runner.step([StepEntry("c", b, list(range(37)))]).cpu().double()     # pages used again
    assert (whole - want_b).abs().max() < 2e-4


def test_blocks_with_four_norms_and_two_mixers_and_a_one_vector_cache(tmp_path):
    run_sandwich(tmp_path, "cuda:0")


@pytest.mark.parametrize("name,dtype", [("B", "float32"), ("E", "bfloat16")])
def test_repeated_prompt_layouts_replay_as_graphs(folders, name, dtype):
    """A step layout that comes a second time is captured as a CUDA graph and replayed from the
    third time on; the logits are those of a runner that launches every kernel itself: equal to
    the bit for prompt-only steps (the same kernels on the same data), and within rounding where
    one-token rows run beside a portion (their key splits follow the context bucket)."""
    from tiny_llm_infer_b200.cache import CacheManager
    from tiny_llm_infer_b200.engine import DTYPES, ModelRunner, StepEntry, load_model
    tiny = TINIES[name]
    model, cfg = load_model(str(folders[name]), DTYPES[dtype], "cuda:0")
    runners = []
    for graphs in (True, False):
        cache = CacheManager(model.cache_needs(), tiny["page_size"], 160, 8, 512, DTYPES[dtype], "cuda:0")
        runners.append(ModelRunner(model, cache, max_batch_tokens=512, use_graphs=graphs, prompt_graphs=graphs))
    with_graphs, plain_runner = runners
    vocab = cfg.vocab_size
    for i in range(5):                                   # five prompts of 200 tokens, each in one step
        toks = prompt(50 + i, 200, vocab)
        got = [r.step([StepEntry(f"p{i}", toks, [0, 199])]).clone() for r in runners]
        assert torch.equal(got[0], got[1]), i
        if i >= 2:
            for r in runners:
                r.release(f"p{i - 2}")
    assert len(with_graphs._prompt_graphs) == 1 and not plain_runner._prompt_graphs
    for i in range(4):                                   # two live requests decode beside a portion of a new one
        toks = prompt(70 + i, 150, vocab)
        entries = [StepEntry("p3", [i + 1], [0]), StepEntry("p4", [i + 2], [0]), StepEntry(f"q{i}", toks, [149])]
        got = [r.step(entries).clone() for r in runners]
        assert (got[0] - got[1]).abs().max() < (1e-4 if dtype == "float32" else 0.05), i
        for r in runners:
            r.release(f"q{i}")
    assert len(with_graphs._prompt_graphs) == 2
    with_graphs.check_kernels()
