"""The plain implementation against the reference's own CPU code (golden outputs made by
tests/golden/make_golden.py), and its own consistency."""
import json
from pathlib import Path

import numpy as np
import torch

import plain_qwen3 as plain
from tiny import TINIES, TINY_A, make_folder, prompt

GOLDEN = Path(__file__).resolve().parent / "golden"


def test_logits_match_the_reference_cpu_path(tmp_path):
    """The reference rounds every tensor between operations to FP16, so agreement is to
    FP16 rounding (a few 1e-4 at logits of size 1), with the same argmax in every row."""
    meta = json.loads((GOLDEN / "tiny_a_engine.json").read_text())
    ref = np.load(GOLDEN / "tiny_a_logits.npy")
    cfg, w = plain.read_model(make_folder(TINY_A, tmp_path / "m"))
    ours = plain.logits_of(cfg, w, meta["logits_prompt"]).numpy()
    assert ref.shape == ours.shape == (33, 256)
    assert np.abs(ref - ours).max() < 2e-3 and np.abs(ref).max() > 0.5
    assert (ref.argmax(-1) == ours.argmax(-1)).all()


def test_greedy_tokens_match_the_reference_engine(tmp_path):
    meta = json.loads((GOLDEN / "tiny_a_engine.json").read_text())
    cfg, w = plain.read_model(make_folder(TINY_A, tmp_path / "m"))
    ours = [plain.greedy(cfg, w, p, meta["max_tokens"]) for p in meta["prompts"]]
    for run in meta["runs"]:
        assert run["tokens"] == ours, run           # whatever the budget and the pool
    assert [r["steps"] for r in meta["runs"]] == [8, 16, 20, 22]


def b_tied():
    import dataclasses
    return dict(TINIES["B"], cfg=dataclasses.replace(TINIES["B"]["cfg"], tie_word_embeddings=True))


def test_tiny_b_with_a_tied_head_matches_the_reference(tmp_path):
    """Everything tiny B has that tiny A has not, on the reference's own output: three query heads
    per key/value head, head width 32 with a q width that is not the model's, feed-forward width
    200, eps 1e-5, theta 1e6, pages of 8, 70 tokens.  (The reference always multiplies by the
    embedding for the head, so B's head is tied here.)  Weights N(0, 0.05): logits up to 4, FP16
    rounding of every intermediate tensor accordingly larger than for A."""
    meta = json.loads((GOLDEN / "tiny_b_tied_engine.json").read_text())
    ref = np.load(GOLDEN / "tiny_b_tied_logits.npy")
    cfg, w = plain.read_model(make_folder(b_tied(), tmp_path / "m"))
    ours = plain.logits_of(cfg, w, meta["logits_prompt"]).numpy()
    assert ref.shape == ours.shape == (70, 384)
    assert np.abs(ref).max() > 1.0
    assert np.abs(ref - ours).max() < 4e-3 * np.abs(ref).max()
    top = ours.argmax(-1)
    assert (np.take_along_axis(ref, top[:, None], 1)[:, 0] >= ref.max(-1) - 2e-3).all()
    greedy = [plain.greedy(cfg, w, p, meta["max_tokens"]) for p in meta["prompts"]]
    for run in meta["runs"]:
        assert run["tokens"] == greedy, run
    assert [r["steps"] for r in meta["runs"]] == [15, 27, 12]


def test_causality_and_window(tmp_path):
    """Logits at a position do not depend on later tokens; in a windowed layer not on keys
    the window has passed either."""
    cfg, w = plain.read_model(make_folder(TINIES["C"], tmp_path / "m"))
    ids = prompt(0, 60, cfg["vocab_size"])
    full = plain.logits_of(cfg, w, ids)
    assert torch.allclose(plain.logits_of(cfg, w, ids[:40]), full[:40], atol=1e-12)
    T, nh, hd = 50, 2, 8
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn(T, nh, hd, generator=g, dtype=torch.float64) for _ in range(3))
    out = plain.causal_attention(q, k, v, window=5)
    k2, v2 = k.clone(), v.clone()
    k2[:40] += 3.0
    v2[:40] -= 2.0
    out2 = plain.causal_attention(q, k2, v2, window=5)
    assert torch.equal(out[44:], out2[44:]) and not torch.allclose(out[43], out2[43])
    one = plain.causal_attention(q[:1], k[:1], v[:1])
    assert torch.allclose(one[0], v[0].repeat_interleave(1, 0))


def test_rotary_pairs_and_norm():
    x = torch.arange(16, dtype=torch.float64).view(1, 1, 16) + 1
    r = plain.rotary_half(x, torch.tensor([3]), 100.0)
    f = torch.tensor([100.0 ** (-2 * i / 16) for i in range(8)], dtype=torch.float32)
    a = (torch.tensor(3.0, dtype=torch.float32) * f).double()
    assert torch.allclose(r[0, 0, :8], x[0, 0, :8] * torch.cos(a) - x[0, 0, 8:] * torch.sin(a))
    assert torch.allclose(r[0, 0, 8:], x[0, 0, :8] * torch.sin(a) + x[0, 0, 8:] * torch.cos(a))
    assert torch.equal(plain.rotary_half(x, torch.tensor([0]), 100.0), x)
    y = plain.rms_norm(torch.tensor([[3.0, 4.0]], dtype=torch.float64), torch.tensor([2.0, 0.5], dtype=torch.float64), 0.5)
    assert torch.allclose(y, torch.tensor([[3.0 * 2, 4.0 * 0.5]], dtype=torch.float64) / (12.5 + 0.5) ** 0.5)


def test_sampler_restatement():
    u = [plain.uniform_of(9, t) for t in range(2000)]
    assert 0 < min(u) and max(u) < 1 and abs(np.mean(u) - 0.5) < 0.03
    keep = plain.nucleus([0.0, 2.0, 1.0, -5.0], 1.0, 0.8)
    assert keep.tolist() == [1, 2]
