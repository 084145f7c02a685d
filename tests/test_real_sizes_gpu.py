"""Logits at real layer sizes: the bfloat16 kernels that the benchmark times (the tcgen05
product at K = 12288 and N = 24576 interleaved, the weight-streaming product at 151,936 rows,
the tcgen05 prompt attention over more than 2048 keys with 32 / 8 or 64 / 8 heads, the
split-key decode attention inside CUDA graphs) against the engine's float32 path with the same
weights, under the four ways of cutting of trace replay, for

* Qwen3-0.6B sizes, all 28 layers, tied head;
* Qwen3-8B widths, 4 layers, the whole untied head of 151,936 rows;
* Qwen3-32B widths, 2 layers.

The weights are random (``random_model``, one seed for both storage types: values are drawn
as bfloat16 and widened exactly for the float32 model), with the query head-norm gains
doubled (exact in both types), so that attention scores spread and single far keys among the
2,200 matter.  One request of 2,200 tokens and three short ones; the pool holds just the four
at once, so every way of cutting runs on pages that were used before.

And, the one place where the float64 plain implementation can follow at real widths: a
two-layer cut of the 0.6B sizes written as a model folder, loaded through the loader, whole
requests in float32 against ``plain_qwen3``.

Tolerances.  float32, ways of cutting against one another: 1e-4 of the row's largest logit
(library products of different row counts add in different orders).  bfloat16 against float32:
the logits of a row have a standard deviation of 0.6 to 1.6 at these sizes.  Measured on a B200,
as fractions of that standard deviation: the largest difference among a row's 151,936 entries is
0.12 to 0.13 (0.6B, 8B widths) and 0.09 to 0.10 (32B widths) in every way of cutting alike, a row's
root-mean-square difference 0.018 to 0.026; the ways of cutting differ from the whole request by
0.05 to 0.08.  Allowed: ``BF16_TOL`` for the largest difference (2.5 times what was measured: it is
the extreme of 150,000 entries), ``BF16_RMS`` for a row's root-mean-square difference (a little over twice what
was measured), the same ``BF16_TOL`` between the ways of cutting, and the bfloat16 argmax must be
the float32 argmax or within ``NEAR_TIE`` (absolute) of it.  A kernel that drops a key tile, a K
slice or a page moves a row by its whole spread.
"""
import json

import pytest
import torch

import plain_qwen3 as plain
from tiny_llm_infer_b200 import ops
from tiny_llm_infer_b200.cache import CacheManager
from tiny_llm_infer_b200.config import Qwen3Config
from tiny_llm_infer_b200.engine import ModelRunner, load_model, random_model
from tiny_llm_infer_b200.engine import selfcheck
from tiny_llm_infer_b200.weights import write_random_model

pytestmark = pytest.mark.gpu

COMMON = dict(head_dim=128, vocab_size=151936, max_position_embeddings=40960, rms_norm_eps=1e-6, rope_theta=1e6)
SIZES = {
    "0.6b": dict(hidden_size=1024, intermediate_size=3072, num_hidden_layers=28, num_attention_heads=16,
                 num_key_value_heads=8, tie_word_embeddings=True, **COMMON),
    "8b": dict(hidden_size=4096, intermediate_size=12288, num_hidden_layers=4, num_attention_heads=32,
               num_key_value_heads=8, tie_word_embeddings=False, **COMMON),
    "32b": dict(hidden_size=5120, intermediate_size=25600, num_hidden_layers=2, num_attention_heads=64,
                num_key_value_heads=8, tie_word_embeddings=False, **COMMON),
}
LENGTHS = (2200, 300, 150, 90)
PAGE = 16
F32_SPREAD = 1e-4
BF16_TOL = 0.3          # largest difference in a row, of the row's standard deviation
BF16_RMS = 0.06         # root-mean-square difference of a row, of the row's standard deviation
NEAR_TIE = 0.3          # absolute


def config_of(name):
    sizes = SIZES[name]
    return Qwen3Config(layer_types=("full_attention",) * sizes["num_hidden_layers"], **sizes)


def requests_of(vocab, lengths=LENGTHS):
    gen = torch.Generator().manual_seed(7)
    return {str(i): torch.randint(0, vocab, (n,), generator=gen).tolist() for i, n in enumerate(lengths)}


def sharpen(model, factor=2.0):
    for block in model.blocks:
        for mixer in block.mixers():
            mixer.q_gain.mul_(factor)


def runner_for(model, dtype, requests):
    longest = max(len(t) for t in requests.values())
    pages = selfcheck.pages_for(requests, PAGE)
    cache = CacheManager(model.cache_needs(), PAGE, pages, max_slots=4, max_seq_len=-(-longest // 64) * 64,
                         dtype=dtype, device="cuda:0")
    return ModelRunner(model, cache, max_batch_tokens=-(-longest // 64) * 64)


def all_ways(name, dtype, requests, wanted):
    model = random_model(config_of(name), seed=11, dtype=dtype, device="cuda:0", std=0.02)
    sharpen(model)
    runner = runner_for(model, dtype, requests)
    cut = selfcheck.CutRunner(runner, requests, wanted)
    rows = cut.all_ways(seed=3)
    runner.check_kernels()
    runner.cache.audit()
    return rows


@pytest.mark.parametrize("name", ["0.6b", "8b", "32b"])
def test_bfloat16_kernels_against_the_float32_path_at_real_sizes(name):
    cfg = config_of(name)
    requests = requests_of(cfg.vocab_size)
    wanted = {k: selfcheck.wanted_positions(len(v)) for k, v in requests.items()}
    exact = all_ways(name, torch.float32, requests, wanted)
    torch.cuda.empty_cache()
    calls = ops.tcgen05_calls
    fast = all_ways(name, torch.bfloat16, requests, wanted)
    assert ops.tcgen05_calls > calls, "no tcgen05 kernel ran"
    assert {k[0] for k in fast} == {"whole", "tail", "portions", "mixed"}

    spread32 = selfcheck.spread_between_ways(exact)
    assert max(spread32.values()) <= F32_SPREAD, spread32

    result = selfcheck.compare(fast, exact, NEAR_TIE)
    print(f"\n[{name}] bfloat16 against float32: " + json.dumps({k: round(v, 4) for k, v in result.items()}))
    for way in ("whole", "tail", "portions", "mixed"):
        assert result[way + ":relative"] <= BF16_TOL, (way, result)
        assert result[way + ":rms"] <= BF16_RMS, (way, result)
        assert result[way + ":argmax_misses"] == 0, (way, result)
    # the ways of cutting against one another in bfloat16, as differences relative to the row's spread
    worst = 0.0
    for (way, req, pos), row in fast.items():
        if way != "whole":
            base = fast[("whole", req, pos)]
            worst = max(worst, float((row - base).abs().max()) / float(exact[(way, req, pos)].std()))
    print(f"[{name}] bfloat16 ways of cutting against the whole request: {worst:.4f} of a row's spread")
    assert worst <= BF16_TOL, worst


def test_a_long_context_at_real_widths():
    """One request of 20,000 tokens (two layers of the 0.6B sizes): the prompt in portions of 4096 and of
    300 tokens (few query rows against many keys: the prompt kernel's key splits and their combine
    step), then 16 tokens one by one (decode attention over 20,000 keys in some twenty splits), the
    bfloat16 kernels against the float32 path at the last positions of every portion."""
    sizes = {**SIZES["0.6b"], "num_hidden_layers": 2}
    cfg = Qwen3Config(layer_types=("full_attention",) * 2, **sizes)
    gen = torch.Generator().manual_seed(9)
    toks = torch.randint(0, cfg.vocab_size, (20000,), generator=gen).tolist()
    cuts = [4096, 4096, 300, 4096, 2, 4096, 3298] + [1] * 16
    assert sum(cuts) == len(toks)
    rows = {}
    for dtype in (torch.float32, torch.bfloat16):
        model = random_model(cfg, seed=13, dtype=dtype, device="cuda:0", std=0.02)
        sharpen(model)
        cache = CacheManager(model.cache_needs(), PAGE, 20000 // PAGE + 2, max_slots=1, max_seq_len=20032, dtype=dtype,
                             device="cuda:0")
        runner = ModelRunner(model, cache, max_batch_tokens=4096)
        got, at = [], 0
        for n in cuts:
            want = sorted({max(0, n - 2), n - 1})
            got += list(runner.step([selfcheck.StepEntry("long", toks[at:at + n], want)]).clone())
            at += n
        runner.check_kernels()
        rows[dtype] = torch.stack(got)
        del model, cache, runner
        torch.cuda.empty_cache()
    exact, fast = rows[torch.float32], rows[torch.bfloat16]
    spread = exact.std(dim=1, keepdim=True)
    assert torch.isfinite(fast).all()
    rel = ((fast - exact).abs() / spread).max().item()
    rms = ((fast - exact).square().mean(dim=1).sqrt() / spread[:, 0]).max().item()
    print(f"\n[20,000 tokens] bfloat16 against float32: largest {rel:.4f}, rms {rms:.4f} of a row's spread")
    assert rel <= BF16_TOL and rms <= BF16_RMS
    picks = fast.argmax(dim=1)
    assert ((exact.max(dim=1).values - exact.gather(1, picks[:, None])[:, 0]) <= NEAR_TIE).all()


def test_float32_path_against_the_plain_implementation_at_real_widths(tmp_path):
    """Two layers of the 0.6B sizes from a model folder (the loader at real widths too)."""
    cfg = Qwen3Config(**{**SIZES["0.6b"], "num_hidden_layers": 2}, layer_types=("full_attention",) * 2)
    folder = write_random_model(tmp_path / "model", cfg, seed=5, std=0.02)
    requests = requests_of(cfg.vocab_size, (300, 70))
    wanted = {k: selfcheck.wanted_positions(len(v), tail=8) for k, v in requests.items()}
    model, _ = load_model(folder, torch.float32, "cuda:0")
    runner = runner_for(model, torch.float32, requests)
    cut = selfcheck.CutRunner(runner, requests, wanted)
    cut.whole()
    cut.portions(sizes=(7, 2, 13, 2, 129, 5))
    pcfg, w = plain.read_model(folder)
    for name, toks in requests.items():
        want = plain.logits_of(pcfg, w, toks)
        for pos in wanted[name]:
            ref = want[pos].to(torch.float32)
            for way in ("whole", "portions"):
                got = cut.rows[(way, name, pos)].cpu()
                assert float((got - ref).abs().max()) <= 1e-4 * max(1.0, float(ref.abs().max())), (way, name, pos)
                assert int(got.argmax()) == int(ref.argmax()) or float(ref.max() - ref[int(got.argmax())]) < 1e-5
