"""Each CUDA kernel alone against a plain torch restatement of the same operation, at
sizes other than the tiny models': widths and vocabularies that are no power of two, head
widths in steps of 16, odd head counts and groups.  Inputs are shaped so that faults show:
one far key that dominates, a window's edge, a page's edge, pages in scrambled order."""
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu

DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype, scale=1.0):
    return (2e-5 if dtype == torch.float32 else 1.6e-2) * scale


@pytest.fixture(scope="module")
def ops():
    from tiny_llm_infer_b200 import ops as o
    o.lib()
    from tiny_llm_infer_b200.engine.runner import strict_float32
    strict_float32()
    return o


def dev(t):
    return t.cuda().contiguous()


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float64) * scale


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("vocab,hidden", [(1000, 136), (517, 4104)])
def test_embedding(ops, dtype, vocab, hidden):
    table = rnd(vocab, hidden, seed=1).to(dtype)
    ids = torch.tensor([0, vocab - 1, 5, -1, 17, 5, -1, 3], dtype=torch.int32)
    out = torch.full((len(ids), hidden), 7.0, dtype=torch.float32, device="cuda")
    ops.embedding(dev(ids), dev(table), out)
    want = table.float()[ids.clamp(min=0).long()]
    want[ids < 0] = 0
    assert torch.equal(out.cpu(), want)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [72, 1000, 4104])
@pytest.mark.parametrize("eps", [1e-6, 1e-2])
def test_add_rmsnorm(ops, dtype, width, eps):
    T = 7
    h = rnd(T, width, seed=2, scale=3.0).float()
    delta = rnd(T, width, seed=3).to(dtype)
    gain = (rnd(width, seed=4) * 0.2 + 1).to(dtype)
    v = h.double() + delta.double()
    want = gain.double() * v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps)
    hd = dev(h)
    out = torch.empty((T, width), dtype=dtype, device="cuda")
    ops.add_rmsnorm(hd, dev(delta), dev(gain), eps, out)
    assert (hd.cpu().double() - v).abs().max() < 1e-6 * 10          # residual sum written back in float32
    assert (out.cpu().double() - want).abs().max() < tol(dtype, want.abs().max().item())
    # without a delta nothing is written back; with rows only those rows are normed, h untouched
    h2 = dev(h)
    rows = torch.tensor([5, 0, 5], dtype=torch.int32)
    out2 = torch.empty((3, width), dtype=dtype, device="cuda")
    ops.add_rmsnorm(h2, dev(delta), dev(gain), eps, out2, dev(rows))
    assert torch.equal(h2.cpu(), h)
    assert (out2.cpu().double() - want[rows.long()]).abs().max() < tol(dtype, want.abs().max().item())
    out3 = torch.empty((T, width), dtype=dtype, device="cuda")
    ops.add_rmsnorm(h2, None, dev(gain.float()), eps, out3)          # float32 gain with any storage
    w3 = gain.double() * h.double() * torch.rsqrt((h.double() ** 2).mean(-1, keepdim=True) + eps)
    assert (out3.cpu().double() - w3).abs().max() < tol(dtype, w3.abs().max().item())
    assert torch.equal(h2.cpu(), h)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", [1024, 4096, 5120, 1000])
def test_add_rmsnorm_of_many_rows_is_that_of_few(ops, dtype, width):
    """Thousands of rows in one launch give to the bit what the same rows give a few at a time (a
    token's logits must not depend on how many tokens share its step), with and without a delta."""
    T, eps = 2500, 1e-6
    h = rnd(T, width, seed=12, scale=3.0).float()
    delta = rnd(T, width, seed=13).to(dtype)
    gain = (rnd(width, seed=14) * 0.2 + 1).to(dtype)
    for with_delta in (True, False):
        h_all, out_all = dev(h), torch.empty((T, width), dtype=dtype, device="cuda")
        ops.add_rmsnorm(h_all, dev(delta) if with_delta else None, dev(gain), eps, out_all)
        h_few, out_few = dev(h), torch.empty((T, width), dtype=dtype, device="cuda")
        for a in range(0, T, 500):
            ops.add_rmsnorm(h_few[a:a + 500], dev(delta[a:a + 500]) if with_delta else None, dev(gain), eps, out_few[a:a + 500])
        assert torch.equal(out_all, out_few) and torch.equal(h_all, h_few)
        v = h.double() + (delta.double() if with_delta else 0)
        want = gain.double() * v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps)
        assert (out_all.cpu().double() - want).abs().max() < tol(dtype, want.abs().max().item())
        assert torch.equal(h_all.cpu(), v.float()) or (h_all.cpu().double() - v).abs().max() < 1e-5


def interleaved_columns(t):
    """[rows, 2 I] with gate columns first, up columns after -> gate and up interleaved by eight."""
    rows, two_i = t.shape
    inter = two_i // 2
    return torch.stack([t[:, :inter].reshape(rows, inter // 8, 8), t[:, inter:].reshape(rows, inter // 8, 8)],
                       dim=2).reshape(rows, two_i).contiguous()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("inter,interleaved", [(200, False), (1000, False), (77, False), (200, True), (1000, True)])
def test_swiglu(ops, dtype, inter, interleaved):
    gu = rnd(9, 2 * inter, seed=5, scale=3.0).to(dtype)
    out = torch.empty((9, inter), dtype=dtype, device="cuda")
    ops.swiglu(dev(interleaved_columns(gu) if interleaved else gu), out, interleaved)
    g, u = gu[:, :inter].double(), gu[:, inter:].double()
    want = plain.silu(g) * u
    assert (out.cpu().double() - want).abs().max() < tol(dtype, want.abs().max().item())


def scrambled_tables(slots, max_pages, num_pages, seed):
    """Every slot gets distinct pages in a scrambled order."""
    g = torch.Generator().manual_seed(seed)
    perm = torch.randperm(num_pages, generator=g)[:slots * max_pages]
    return perm.view(slots, max_pages).to(torch.int32)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,rot", [(6, 2, 48, 48), (5, 5, 80, 32), (8, 1, 128, 128), (3, 3, 16, 16),
                                           (2, 1, 256, 256)])
def test_qk_norm_rope_store(ops, dtype, nh, nkv, hd, rot):
    T, ps, slots, max_pages = 11, 8, 3, 6
    eps, theta = 1e-5, 5e4
    qkv = rnd(T, (nh + 2 * nkv) * hd, seed=6, scale=2.0).to(dtype)
    qg = (rnd(hd, seed=7) * 0.3 + 1).to(dtype)
    kg = (rnd(hd, seed=8) * 0.3 + 1).to(dtype)
    positions = torch.tensor([0, 1, 7, 8, 9, 15, 16, 40, 3, 47, 5], dtype=torch.int32)
    slot = torch.tensor([0, 0, 0, 0, 1, 1, 1, 2, -1, 2, 1], dtype=torch.int32)
    table = scrambled_tables(slots, max_pages, 20, seed=9)
    inv_freq = (theta ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).float()
    cache = torch.zeros((20, 2, nkv, ps, hd), dtype=dtype, device="cuda")
    q_out = torch.full((T, nh * hd), 9.0, dtype=dtype, device="cuda")
    flags = ops.QK_NORM | ops.QK_ROPE | ops.QK_STORE | ops.QK_QOUT
    ops.qk_norm_rope_store(dev(qkv), dev(qg), dev(kg), eps, dev(inv_freq), rot, dev(positions), dev(slot),
                           dev(table), cache, ps, q_out, nh, nkv, hd, flags)
    x = qkv.double().view(T, nh + 2 * nkv, hd)
    q, k, v = x[:, :nh], x[:, nh:nh + nkv], x[:, nh + nkv:]

    def rope(t):      # rotate the first `rot` elements with the plain implementation's rule
        r = plain.rotary_half(t[..., :rot], positions, theta)
        return torch.cat([r, t[..., rot:]], -1)
    qn = rope(plain.rms_norm(q, qg.double(), eps))
    kn = rope(plain.rms_norm(k, kg.double(), eps))
    scale = max(qn.abs().max().item(), 1.0)
    cache_h, q_h = cache.cpu().double(), q_out.cpu().double().view(T, nh, hd)
    touched = torch.zeros(20, ps, dtype=torch.bool)
    for t in range(T):
        if slot[t] < 0:
            assert (q_out[t].cpu() == 9.0).all()          # padding rows are skipped
            continue
        assert (q_h[t] - qn[t]).abs().max() < tol(dtype, scale)
        page, off = int(table[slot[t], positions[t] // ps]), int(positions[t] % ps)
        touched[page, off] = True
        assert (cache_h[page, 0, :, off] - kn[t]).abs().max() < tol(dtype, scale)
        assert (cache_h[page, 1, :, off] - v[t]).abs().max() < tol(dtype, scale)
    untouched = cache_h.permute(0, 3, 1, 2, 4)[~touched]
    assert (untouched == 0).all()                        # nothing else was written
    if rot == hd:
        # with the step's table of cosines and sines instead of sincosf in the kernel: the same bits
        rope_table = ops.rope_table(dev(positions), dev(inv_freq))
        angle = positions.float()[:, None] * inv_freq[None, :]
        assert torch.equal(rope_table[:, 0].cpu()[slot >= 0], torch.cos(angle)[slot >= 0]) or \
            (rope_table[:, 0].cpu() - torch.cos(angle)).abs().max() < 1e-6
        cache2 = torch.zeros_like(cache)
        q_out2 = torch.full_like(q_out, 9.0)
        ops.qk_norm_rope_store(dev(qkv), dev(qg), dev(kg), eps, dev(inv_freq), rot, dev(positions), dev(slot),
                               dev(table), cache2, ps, q_out2, nh, nkv, hd, flags, table=rope_table)
        assert torch.equal(q_out2, q_out) and torch.equal(cache2, cache)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd", [(7, 3, 128), (5, 2, 64), (3, 1, 256), (32, 8, 128)])
def test_qk_norm_rope_store_with_many_tokens(ops, dtype, nh, nkv, hd):
    """More than 64 tokens take the form in which a warp has six heads on their way: head counts that
    fill neither a warp nor a round, every token at its own place, with and without the step's table."""
    T, ps, eps, theta = 150, 16, 1e-6, 1e6
    g = torch.Generator().manual_seed(21)
    qkv = rnd(T, (nh + 2 * nkv) * hd, seed=16, scale=2.0).to(dtype)
    qg = (rnd(hd, seed=17) * 0.3 + 1).to(dtype)
    kg = (rnd(hd, seed=18) * 0.3 + 1).to(dtype)
    slots, max_pages, pages = 3, 8, 30
    slot = torch.randint(0, slots, (T,), generator=g).to(torch.int32)
    slot[5] = slot[77] = -1
    positions = torch.zeros(T, dtype=torch.int32)
    for s in range(slots):                      # distinct positions inside a slot, in a scrambled order
        mine = (slot == s).nonzero()[:, 0]
        positions[mine] = torch.randperm(max_pages * ps, generator=g)[:len(mine)].to(torch.int32)
    table = scrambled_tables(slots, max_pages, pages, seed=19)
    inv_freq = (theta ** (-2.0 * torch.arange(hd // 2, dtype=torch.float64) / hd)).float()
    flags = ops.QK_NORM | ops.QK_ROPE | ops.QK_STORE | ops.QK_QOUT
    x = qkv.double().view(T, nh + 2 * nkv, hd)
    qn = plain.rotary_half(plain.rms_norm(x[:, :nh], qg.double(), eps), positions, theta)
    kn = plain.rotary_half(plain.rms_norm(x[:, nh:nh + nkv], kg.double(), eps), positions, theta)
    want = torch.zeros(pages, 2, nkv, ps, hd, dtype=torch.float64)
    live = slot >= 0
    for t in live.nonzero()[:, 0].tolist():
        page, off = int(table[slot[t], positions[t] // ps]), int(positions[t] % ps)
        want[page, 0, :, off], want[page, 1, :, off] = kn[t], x[t, nh + nkv:]
    scale = max(qn.abs().max().item(), 1.0)
    results = []
    for with_table in (False, True):
        cache = torch.zeros((pages, 2, nkv, ps, hd), dtype=dtype, device="cuda")
        q_out = torch.full((T, nh * hd), 9.0, dtype=dtype, device="cuda")
        rope_table = ops.rope_table(dev(positions), dev(inv_freq)) if with_table else None
        ops.qk_norm_rope_store(dev(qkv), dev(qg), dev(kg), eps, dev(inv_freq), hd, dev(positions), dev(slot),
                               dev(table), cache, ps, q_out, nh, nkv, hd, flags, table=rope_table)
        q_h = q_out.cpu().double().view(T, nh, hd)
        assert (q_h[live] - qn[live]).abs().max() < tol(dtype, scale)
        assert (q_h[~live] == 9.0).all()
        assert (cache.cpu().double() - want).abs().max() < tol(dtype, scale)
        assert (cache.cpu()[want == 0] == 0).all()
        results.append((q_out, cache))
    assert torch.equal(results[0][0], results[1][0]) and torch.equal(results[0][1], results[1][1])


def fill_cache(cache, table, slot, keys, vals, ps):
    """Write keys/vals [n, nkv, hd] of one request into its pages."""
    for j in range(keys.shape[0]):
        page = int(table[slot, j // ps])
        cache[page, 0, :, j % ps] = keys[j].to(cache.dtype)
        cache[page, 1, :, j % ps] = vals[j].to(cache.dtype)


def plain_rows(q, keys, vals, positions, window):
    """Rows of the plain implementation's attention for queries at ``positions``."""
    n = keys.shape[0]
    full_q = torch.zeros((n,) + q.shape[1:], dtype=torch.float64)
    full_q[positions] = q
    return plain.causal_attention(full_q, keys, vals, window)[positions]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("nh,nkv,hd,ps,window", [
    (6, 2, 48, 8, None), (4, 4, 16, 16, None), (8, 1, 128, 16, None), (5, 5, 80, 4, 37),
    (32, 8, 128, 16, None), (2, 2, 256, 32, 64), (16, 8, 64, 16, None), (3, 1, 112, 64, 130)])
def test_paged_attention_far_key_and_edges(ops, dtype, nh, nkv, hd, ps, window):
    """One request of 300 keys.  For every query one far key dominates the softmax (its
    score is lifted), placed at a page's edge or on the first key the window still admits;
    the key just outside the window is made just as strong and must not count."""
    n = 300
    max_pages = -(-n // ps) + 1
    table = scrambled_tables(2, max_pages, 2 * max_pages + 3, seed=11)
    keys = rnd(n, nkv, hd, seed=12).to(dtype).double()
    vals = rnd(n, nkv, hd, seed=13).to(dtype).double()
    positions = torch.tensor([0, 1, ps - 1, ps, ps + 1, 37, 130, 131, 255, 256, 299])
    q = rnd(len(positions), nh, hd, seed=14).to(dtype).double()
    group = nh // nkv
    for r, pos in enumerate(positions.tolist()):
        lo = max(0, pos - window + 1) if window else 0
        target = lo if r % 2 == 0 else (pos // ps) * ps - 1 if pos >= ps else lo   # window edge or page edge
        target = min(max(target, lo), pos)
        for h in range(nh):
            q[r, h] = (keys[target, h // group] * 4.0 + q[r, h] * 0.1).to(dtype).double()
        if window and lo > 0:
            keys[lo - 1] = keys[target]               # as strong, but outside the window
    scale = 1.0 / math.sqrt(hd)
    want = plain_rows(q, keys, vals, positions, window)
    cache = torch.zeros((2 * max_pages + 3, 2, nkv, ps, hd), dtype=dtype, device="cuda")
    cache.normal_()                                   # stale data in every page
    fill_cache(cache, table, 1, keys, vals, ps)
    T = len(positions) + 2
    qd = torch.zeros((T, nh * hd), dtype=dtype)
    qd[1:-1] = q.reshape(len(positions), -1).to(dtype)
    pos_d = torch.zeros(T, dtype=torch.int32)
    pos_d[1:-1] = positions.int()
    slot_d = torch.full((T,), -1, dtype=torch.int32)
    slot_d[1:-1] = 1
    out = torch.full((T, nh * hd), 5.0, dtype=dtype, device="cuda")
    ops.paged_attention(dev(qd), cache, dev(pos_d), dev(slot_d), dev(table), ps, nh, nkv, hd, window,
                        scale, out)
    got = out.cpu().double()
    assert (got[0] == 0).all() and (got[-1] == 0).all()          # padding rows give zeros
    err = (got[1:-1].view(len(positions), nh, hd) - want).abs().max().item()
    assert err < tol(dtype, want.abs().max().item()), err


@pytest.mark.parametrize("dtype", DTYPES)
def test_paged_attention_many_requests(ops, dtype):
    """Rows of several requests interleaved, prompt portions beside single tokens."""
    nh, nkv, hd, ps = 6, 3, 32, 8
    lens = [45, 9, 130, 1]
    max_pages = 20
    table = scrambled_tables(4, max_pages, 90, seed=21)
    cache = torch.zeros((90, 2, nkv, ps, hd), dtype=dtype, device="cuda").normal_()
    K = [rnd(n, nkv, hd, seed=30 + i).to(dtype).double() for i, n in enumerate(lens)]
    V = [rnd(n, nkv, hd, seed=40 + i).to(dtype).double() for i, n in enumerate(lens)]
    for s in range(4):
        fill_cache(cache, table, s, K[s], V[s], ps)
    rows = [(0, p) for p in range(30, 45)] + [(1, 8)] + [(2, p) for p in range(0, 130, 7)] + [(3, 0)]
    q = rnd(len(rows), nh, hd, seed=50, scale=2.0).to(dtype).double()
    out = torch.empty((len(rows), nh * hd), dtype=dtype, device="cuda")
    ops.paged_attention(dev(q.reshape(len(rows), -1).to(dtype)), cache,
                        dev(torch.tensor([p for _, p in rows], dtype=torch.int32)),
                        dev(torch.tensor([s for s, _ in rows], dtype=torch.int32)), dev(table), ps,
                        nh, nkv, hd, None, 1 / math.sqrt(hd), out)
    got = out.cpu().double().view(len(rows), nh, hd)
    for s in range(4):
        idx = [i for i, (ss, _) in enumerate(rows) if ss == s]
        pos = torch.tensor([rows[i][1] for i in idx])
        want = plain_rows(q[idx], K[s], V[s], pos, None)
        assert (got[idx] - want).abs().max() < tol(dtype, want.abs().max().item())


def test_sample_greedy_ties_and_temperature(ops):
    V = 5003
    logits = rnd(6, V, seed=60, scale=2.0).float()
    logits[0, 4000] = logits[0, 17] = 9.0                # tie: the lower id wins
    logits[1, V - 1] = 12.0
    params = torch.tensor([[0.0, 1.0], [0.0, 1.0], [0.7, 1.0], [1.3, 1.0], [0.7, 0.6], [1.0, 0.05]])
    seeds = torch.tensor([1, 2, 3, 2 ** 62 + 12345, -5, 77], dtype=torch.int64)
    out = torch.empty(6, dtype=torch.int32, device="cuda")
    ops.sample(dev(logits), dev(params), dev(seeds), out)
    got = out.cpu().tolist()
    assert got[0] == 17 and got[1] == V - 1
    for r in range(2, 6):
        temp, top_p = params[r].tolist()
        seed = int(seeds[r]) & ((1 << 64) - 1)
        scores = plain.gumbel_scores(logits[r].numpy(), temp, seed)
        if top_p < 1:
            keep = plain.nucleus(logits[r].numpy(), temp, top_p)
            assert got[r] in set(keep.tolist())
            best = max(scores[keep])
        else:
            best = scores.max()
        assert scores[got[r]] >= best - 1e-4, (r, got[r], int(np.argmax(scores)))
    assert abs(ops.uniform_of(12345, 678) - plain.uniform_of(12345, 678)) < 1e-9


@pytest.mark.parametrize("V", [151937, 3001])
def test_sample_nucleus(ops, V):
    """Top-p over a vocabulary no power of two (the larger is shared by several blocks a row,
    the smaller takes the one-block kernel), many rows with their own temperature, top_p and
    seed: the token drawn is the best-scoring one of the plain nucleus.  One row is peaked
    (a single token holds the mass), one is flat (every key ties, so all are kept)."""
    rows = 24
    logits = rnd(rows, V, seed=61, scale=3.0).float()
    logits[0] = 0.0
    logits[0, V // 2] = 30.0                             # alone in every nucleus
    logits[1] = 1.25                                     # all tie
    gen = np.random.default_rng(5)
    temps = gen.uniform(0.3, 1.6, rows)
    tops = gen.uniform(0.02, 0.999, rows)
    tops[0], tops[1] = 0.9, 0.5
    params = torch.tensor(np.stack([temps, tops], 1), dtype=torch.float32)
    seeds = torch.tensor(gen.integers(0, 2 ** 62, rows), dtype=torch.int64)
    for nucleus in (True, None):
        out = torch.full((rows,), -1, dtype=torch.int32, device="cuda")
        ops.sample(dev(logits), dev(params), dev(seeds), out, any_nucleus=nucleus)
        got = out.cpu().tolist()
        assert got[0] == V // 2
        for r in range(1, rows):
            temp, top_p = params[r].tolist()
            scores = plain.gumbel_scores(logits[r].numpy(), temp, int(seeds[r]))
            if r == 1:
                assert scores[got[r]] >= scores.max() - 1e-4
                continue
            keep = plain.nucleus(logits[r].numpy(), temp, top_p)
            assert got[r] in set(keep.tolist()), (r, temp, top_p, len(keep))
            assert scores[got[r]] >= max(scores[keep]) - 1e-4, (r, temp, top_p, len(keep))


def test_sample_distribution(ops):
    """Frequencies of many seeds follow softmax(logits / T)."""
    V, n, temp = 11, 4000, 0.8
    lg = torch.tensor([0.0, 1.0, 2.0, -1.0, 0.5, 3.0, -2.0, 1.5, 0.2, 2.5, -0.5])
    logits = lg.repeat(n, 1)
    params = torch.tensor([[temp, 1.0]]).repeat(n, 1)
    seeds = torch.arange(n, dtype=torch.int64) * 7919 + 13
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    ops.sample(dev(logits), dev(params), dev(seeds), out)
    freq = torch.bincount(out.cpu().long(), minlength=V).double() / n
    p = torch.softmax(lg.double() / temp, 0)
    assert (freq - p).abs().max() < 4 * math.sqrt(0.25 / n)


@pytest.mark.parametrize("dtype", DTYPES)
def test_linear_precision(ops, dtype):
    """float32 products must be true float32 (a reduced-precision matrix mode would miss
    this bound by two orders of magnitude); bfloat16 inputs accumulate in float32."""
    x = rnd(33, 1000, seed=70).to(dtype)
    w = rnd(200, 1000, seed=71).to(dtype)
    want = x.double() @ w.double().T
    got32 = ops.linear(dev(x), dev(w), out_dtype=torch.float32).cpu().double()
    assert (got32 - want).abs().max() < (3e-4 if dtype == torch.float32 else 1e-3)
    got = ops.linear(dev(x), dev(w)).cpu().double()
    assert (got - want).abs().max() < tol(dtype, want.abs().max().item()) * 2


def test_mixed_storage_linear(ops):
    """A weight kept in float32 is multiplied in float32 under bfloat16 activations."""
    x = rnd(5, 64, seed=72).to(torch.bfloat16)
    w = rnd(24, 64, seed=73).float()
    got = ops.linear(dev(x), dev(w), out_dtype=torch.float32).cpu().double()
    assert (got - x.double() @ w.double().T).abs().max() < 1e-4


def test_refusals(ops):
    """Sizes a kernel does not take are refused with an error, never computed wrongly."""
    q = torch.zeros((1, 2 * 1024), dtype=torch.bfloat16, device="cuda")
    cache = torch.zeros((2, 2, 2, 16, 1024), dtype=torch.bfloat16, device="cuda")
    z = torch.zeros(1, dtype=torch.int32, device="cuda")
    table = torch.zeros((1, 2), dtype=torch.int32, device="cuda")
    with pytest.raises(ops.KernelError, match="head_dim"):
        ops.paged_attention(q, cache, z, z, table, 16, 2, 2, 1024, None, 1.0, torch.empty_like(q))
    q3 = torch.zeros((1, 3 * 32), dtype=torch.bfloat16, device="cuda")
    cache3 = torch.zeros((2, 2, 2, 16, 32), dtype=torch.bfloat16, device="cuda")
    with pytest.raises(ops.KernelError, match="heads"):
        ops.paged_attention(q3, cache3, z, z, table, 16, 3, 2, 32, None, 1.0, torch.empty_like(q3))


# ----------------------------------------------------------------- tensor-core attention kernels
def request_data(lens, nkv, hd, ps, seed, num_pages, max_pages):
    table = scrambled_tables(len(lens), max_pages, num_pages, seed=seed)
    cache = torch.zeros((num_pages, 2, nkv, ps, hd), dtype=torch.bfloat16, device="cuda").normal_()
    K = [rnd(n, nkv, hd, seed=seed + 1 + i).to(torch.bfloat16).double() for i, n in enumerate(lens)]
    V = [rnd(n, nkv, hd, seed=seed + 50 + i).to(torch.bfloat16).double() for i, n in enumerate(lens)]
    for s in range(len(lens)):
        fill_cache(cache, table, s, K[s], V[s], ps)
    return table, cache, K, V


@pytest.mark.parametrize("nh,nkv,hd,ps,window", [(32, 8, 128, 16, None), (4, 2, 64, 16, None), (16, 1, 128, 32, None),
                                                 (6, 2, 64, 64, 100), (3, 3, 128, 16, 33), (14, 2, 64, 16, None)])
@pytest.mark.parametrize("splits", [1, 3, 8, 13, 20])
def test_decode_kernel_split_keys(ops, nh, nkv, hd, ps, window, splits):
    """One-token rows of four requests (contexts 1 to 700), a padding row, a row list; for
    each query one far key dominates: the first key the window admits or a page's last."""
    lens = [700, 1, 130, 65]
    max_pages = -(-700 // ps) + 1
    table, cache, K, V = request_data(lens, nkv, hd, ps, 100, 4 * max_pages + 2, max_pages)
    group = nh // nkv
    T = 7
    slot = torch.tensor([0, 1, -1, 2, 3, 0, 2], dtype=torch.int32)
    pos = torch.tensor([699, 0, 0, 129, 64, 351, 17], dtype=torch.int32)
    q = rnd(T, nh, hd, seed=101, scale=0.2).to(torch.bfloat16).double()
    for t in range(T):
        if slot[t] < 0:
            continue
        p = int(pos[t])
        lo = max(0, p - window + 1) if window else 0
        target = lo if t % 2 == 0 else max(lo, (p // ps) * ps - 1)
        for h in range(nh):
            q[t, h] += K[slot[t]][target, h // group] * 3.0
    q = q.to(torch.bfloat16).double()
    rows = torch.tensor([0, 1, 3, 4, 6, 5, 2], dtype=torch.int32)          # every row, in another order
    out = torch.full((T, nh * hd), 3.0, dtype=torch.bfloat16, device="cuda")
    ops.paged_attention_decode(dev(q.reshape(T, -1).to(torch.bfloat16)), cache, dev(pos), dev(slot), dev(rows), T,
                               dev(table), ps, nh, nkv, hd, window, 1 / math.sqrt(hd), out, 700, splits=splits)
    got = out.cpu().double().view(T, nh, hd)
    assert (got[2] == 0).all()
    for t in range(T):
        if slot[t] < 0:
            continue
        s = int(slot[t])
        want = plain_rows(q[t:t + 1], K[s][:pos[t] + 1], V[s][:pos[t] + 1], torch.tensor([int(pos[t])]), window)[0]
        err = (got[t] - want).abs().max().item()
        assert err < tol(torch.bfloat16, want.abs().max().item()), (t, err)


@pytest.mark.parametrize("nh,nkv,hd,ps,window", [(8, 2, 128, 16, None), (4, 4, 64, 32, None), (6, 1, 64, 16, 70),
                                                 (2, 1, 128, 64, 9)])
def test_prefill_kernel_segments(ops, nh, nkv, hd, ps, window):
    """Segments that start inside a request (their earlier keys only in the cache), are
    shorter and longer than a block of 64 rows, start and end off tile edges."""
    lens = [300, 64, 131, 5]
    max_pages = -(-300 // ps) + 1
    table, cache, K, V = request_data(lens, nkv, hd, ps, 200, 4 * max_pages + 2, max_pages)
    group = nh // nkv
    segs = [(0, 93, 207), (1, 0, 64), (2, 128, 3), (3, 0, 5), (2, 1, 100)]      # slot, pos0, len (slot 2 twice is fine here)
    seg_info, tiles, pos_rows, slot_rows, row = [], [], [], [], 0
    for i, (s, p0, n) in enumerate(segs):
        seg_info.append([s, row, n, p0])
        tiles += [[i, off] for off in range(0, n, 64)]
        pos_rows += list(range(p0, p0 + n))
        slot_rows += [s] * n
        row += n
    T = row
    q = rnd(T, nh, hd, seed=201, scale=0.2).to(torch.bfloat16).double()
    for t in range(T):
        p, s = pos_rows[t], slot_rows[t]
        lo = max(0, p - window + 1) if window else 0
        target = [lo, p, max(lo, (p // 64) * 64 - 1), max(lo, p - 1)][t % 4]
        for h in range(nh):
            q[t, h] += K[s][target, h // group] * 3.0
    q = q.to(torch.bfloat16).double()
    out = torch.zeros((T, nh * hd), dtype=torch.bfloat16, device="cuda")
    tiles = tiles[::-1]
    ops.paged_attention_prefill(dev(q.reshape(T, -1).to(torch.bfloat16)), cache,
                                dev(torch.tensor(seg_info, dtype=torch.int32)),
                                dev(torch.tensor(tiles, dtype=torch.int32)), len(tiles), dev(table), ps, nh, nkv,
                                hd, window, 1 / math.sqrt(hd), out)
    got = out.cpu().double().view(T, nh, hd)
    for (s, r0, n, p0) in seg_info:
        pos = torch.arange(p0, p0 + n)
        want = plain_rows(q[r0:r0 + n], K[s][:p0 + n], V[s][:p0 + n], pos, window)
        err = (got[r0:r0 + n] - want).abs().max().item()
        assert err < tol(torch.bfloat16, want.abs().max().item()), (s, p0, n, err)


@pytest.mark.parametrize("splits", [1, 2, 3, 16])
@pytest.mark.parametrize("nh,nkv,ps,window", [(8, 2, 16, None), (3, 3, 32, None), (6, 1, 16, 70), (2, 1, 64, 9),
                                              (4, 2, 48, 200), (5, 1, 16, None), (3, 1, 32, 130)])
def test_prefill_tcgen05_kernel_segments(ops, nh, nkv, ps, window, splits):
    """The tcgen05 kernel (head width 128; a thread block takes two heads at 128 positions where
    the group is even, else 256 positions of one head) on segments that start inside a
    request, are shorter and longer than a block, start and end off the edges of key tiles
    and pages; each row's query points at one key (the window's first, the row's own, the
    last of the tile before, the one before its own), so that a key that is missed, masked
    wrongly or read from the wrong page changes the result; every other four rows have no such
    key, so that a tile whose share is lost or counted twice shows as well.  With ``splits``
    every block's key tiles go to that many blocks in equal runs (16: more runs than most blocks
    have tiles, so some are empty, and with 256-row blocks the earlier 128 rows have no key in
    the later runs) and a second kernel combines them."""
    hd = 128
    lens = [600, 128, 259, 5]
    max_pages = -(-600 // ps) + 1
    table, cache, K, V = request_data(lens, nkv, hd, ps, 210, 4 * max_pages + 2, max_pages)
    group = nh // nkv
    segs = [(0, 93, 507), (1, 0, 128), (2, 256, 3), (3, 0, 5), (2, 1, 200)]
    seg_info, tiles, pos_rows, slot_rows, row = [], [], [], [], 0
    for i, (s, p0, n) in enumerate(segs):
        seg_info.append([s, row, n, p0])
        tiles += [[i, off] for off in range(0, n, ops.prefill_tcgen05_block_rows(nh, nkv))]
        pos_rows += list(range(p0, p0 + n))
        slot_rows += [s] * n
        row += n
    T = row
    q = rnd(T, nh, hd, seed=211, scale=0.2).to(torch.bfloat16).double()
    for t in range(T):
        if t % 8 >= 4:
            continue        # these rows spread their weight over all keys: each key's share counts
        p, s = pos_rows[t], slot_rows[t]
        lo = max(0, p - window + 1) if window else 0
        target = [lo, p, max(lo, (p // 64) * 64 - 1), max(lo, p - 1)][t % 4]
        for h in range(nh):
            q[t, h] += K[s][target, h // group] * 3.0
    q = q.to(torch.bfloat16).double()
    out = torch.zeros((T, nh * hd), dtype=torch.bfloat16, device="cuda")
    tiles = tiles[::-1]
    ops.paged_attention_prefill_tcgen05(dev(q.reshape(T, -1).to(torch.bfloat16)), cache,
                                        dev(torch.tensor(seg_info, dtype=torch.int32)),
                                        dev(torch.tensor(tiles, dtype=torch.int32)), len(tiles), dev(table), ps,
                                        nh, nkv, hd, window, 1 / math.sqrt(hd), out, splits)
    ops.check_error_word(torch.device("cuda"))
    got = out.cpu().double().view(T, nh, hd)
    for (s, r0, n, p0) in seg_info:
        pos = torch.arange(p0, p0 + n)
        want = plain_rows(q[r0:r0 + n], K[s][:p0 + n], V[s][:p0 + n], pos, window)
        err = (got[r0:r0 + n] - want).abs().max().item()
        assert err < tol(torch.bfloat16, want.abs().max().item()), (s, p0, n, err)


def test_prefill_splits_rule(ops):
    assert ops.prefill_splits(32, 256) == 1 and ops.prefill_splits(32, 1024) == 2
    assert ops.prefill_splits(32, 4096) == 4 and ops.prefill_splits(16, 8192) == 8
    assert ops.prefill_splits(64, 4096) == 2 and ops.prefill_splits(128, 65536) == 1


@pytest.mark.parametrize("splits", [1, 4])
@pytest.mark.parametrize("nh,nkv,window", [(4, 2, None), (3, 1, None), (2, 1, 1000)])
def test_prefill_tcgen05_long_request(ops, nh, nkv, window, splits):
    """One portion of 3000 tokens behind 1100 that are already in the cache: some 65 key tiles per
    block, so the rings of key and value tiles, the S buffers and every barrier's parity wrap
    many times.  Checked against float64 attention on sampled rows of every block."""
    hd, ps, have, new = 128, 16, 1100, 3000
    n = have + new
    pages = -(-n // ps)
    g = torch.Generator(device="cuda").manual_seed(7)
    cache = (torch.randn((pages + 3, 2, nkv, ps, hd), generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    table = (torch.randperm(pages + 3, generator=torch.Generator().manual_seed(8))[:pages]).to(torch.int32).view(1, -1)
    q = (torch.randn((new, nh * hd), generator=g, device="cuda") * 0.5).to(torch.bfloat16)
    rows = ops.prefill_tcgen05_block_rows(nh, nkv)
    tiles = torch.tensor([[0, off] for off in range(0, new, rows)][::-1], dtype=torch.int32)
    out = torch.zeros_like(q)
    ops.paged_attention_prefill_tcgen05(q, cache, dev(torch.tensor([[0, 0, new, have]], dtype=torch.int32)),
                                        dev(tiles), len(tiles), dev(table), ps, nh, nkv, hd, window,
                                        1 / math.sqrt(hd), out, splits)
    ops.check_error_word(torch.device("cuda"))
    # keys and values of the request in position order, float64
    kv = cache[table[0].long().cuda()].double()                       # [pages, 2, nkv, ps, hd]
    K = kv[:, 0].permute(1, 0, 2, 3).reshape(nkv, pages * ps, hd)[:, :n]
    V = kv[:, 1].permute(1, 0, 2, 3).reshape(nkv, pages * ps, hd)[:, :n]
    sample = torch.cat([torch.arange(0, new, 37), torch.tensor([127, 128, 255, 256, new - 1])]).cuda()
    pos = have + sample
    qq = q.double().view(new, nh, hd)[sample]
    got = out.double().view(new, nh, hd)[sample]
    keys = torch.arange(n, device="cuda")
    mask = keys[None, :] <= pos[:, None]
    if window:
        mask &= keys[None, :] > pos[:, None] - window
    for h in range(nh):
        s = qq[:, h] @ K[h // (nh // nkv)].T / math.sqrt(hd)
        want = torch.softmax(s.masked_fill(~mask, float("-inf")), -1) @ V[h // (nh // nkv)]
        err = (got[:, h] - want).abs().max().item()
        assert err < tol(torch.bfloat16, want.abs().max().item()), (h, err)       # a lost key tile would show at four times this


def test_prefill_tcgen05_refuses_other_shapes(ops):
    z = torch.zeros((1, 4), dtype=torch.int32, device="cuda")
    for nh, nkv, hd, ps, match in ((2, 2, 64, 16, "head_dim"), (2, 2, 128, 8, "page size"), (3, 2, 128, 16, "heads")):
        q = torch.zeros((4, nh * hd), dtype=torch.bfloat16, device="cuda")
        cache = torch.zeros((4, 2, nkv, ps, hd), dtype=torch.bfloat16, device="cuda")
        with pytest.raises(ops.KernelError, match=match):
            ops.paged_attention_prefill_tcgen05(q, cache, z, z[:, :2], 1, z, ps, nh, nkv, hd, None, 1.0,
                                                torch.empty_like(q))


def test_fast_attention_refuses_other_shapes(ops):
    z = torch.zeros(1, dtype=torch.int32, device="cuda")
    table = torch.zeros((1, 4), dtype=torch.int32, device="cuda")
    for nh, nkv, hd, ps, match in ((2, 2, 48, 16, "head_dim"), (2, 2, 64, 8, "page size"), (34, 2, 64, 16, "group")):
        q = torch.zeros((1, nh * hd), dtype=torch.bfloat16, device="cuda")
        cache = torch.zeros((4, 2, nkv, ps, hd), dtype=torch.bfloat16, device="cuda")
        assert not ops.fast_attention_ok(torch.bfloat16, ps, nh, nkv, hd)
        with pytest.raises(ops.KernelError, match=match):
            ops.paged_attention_decode(q, cache, z, z, None, 1, table, ps, nh, nkv, hd, None, 1.0,
                                       torch.empty_like(q), 1, splits=1)
    assert not ops.fast_attention_ok(torch.float32, 16, 4, 2, 64)


@pytest.mark.parametrize("xd,wd,yd", [(torch.float32, torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16, torch.float32),
                                      (torch.bfloat16, torch.bfloat16, torch.bfloat16), (torch.float32, torch.bfloat16, torch.float32)])
@pytest.mark.parametrize("M,N,K", [(1, 1, 1), (3, 77, 131), (33, 200, 1000)])
def test_gemm_plain_against_float64(ops, xd, wd, yd, M, N, K):
    """The plain product (one thread per output, float32 sum in order) against a float64 product."""
    x, w = rnd(M, K, seed=700).to(xd), rnd(N, K, seed=701, scale=0.2).to(wd)
    y = ops.gemm_plain(dev(x), dev(w), yd)
    ref = x.double() @ w.double().T
    assert y.dtype == yd and y.shape == (M, N)
    assert (y.cpu().double() - ref).abs().max() < (1e-5 if yd == torch.float32 else 1.6e-2) * max(ref.abs().max().item(), 1.0)


@pytest.mark.parametrize("what,M,N,K", [("skinny", 8, 6144, 4096), ("skinny", 5, 4096, 12288), ("skinny_head", 3, 151936, 1024),
                                        ("tcgen05", 2048, 4096, 12288), ("tcgen05_swiglu", 2048, 24576, 4096),
                                        ("library", 64, 6144, 4096), ("library_f32", 40, 5120, 5120)])
def test_fast_products_against_their_plain_twin_at_real_shapes(ops, what, M, N, K):
    """Every product the engine can take, at shapes of Qwen3-8B / 0.6B / 32B layers, against the plain
    kernel of this package on the same operands (a float64 product of these sizes on the host takes
    too long): through ``ops.linear`` / ``ops.linear_swiglu``, which must choose the kernel named."""
    f32 = what == "library_f32"
    dt = torch.float32 if f32 else torch.bfloat16
    g = torch.Generator(device="cuda").manual_seed(11)
    x = (torch.randn(M, K, device="cuda", generator=g) * 0.5).to(dt)
    w = (torch.randn(N, K, device="cuda", generator=g) * 0.02).to(dt)
    w[N // 2 + 3] *= 7.0                                   # one row that stands out
    w[N - 1] *= 5.0
    before = ops.tcgen05_calls
    if what == "tcgen05_swiglu":
        inter = N // 2
        got = ops.linear_swiglu(x, ops.interleave_gate_up(w[:inter], w[inter:]).contiguous(), torch.bfloat16, interleaved=True)
        full = ops.gemm_plain(x, w, torch.float32)
        ref = torch.nn.functional.silu(full[:, :inter]) * full[:, inter:]
    else:
        got = ops.linear(x, w, out_dtype=torch.float32 if what in ("skinny_head", "library_f32") else None)
        ref = ops.gemm_plain(x, w, torch.float32)
    assert (ops.tcgen05_calls > before) == what.startswith("tcgen05")
    ops.check_error_word("cuda:0")
    scale = ref.abs().max().item()
    assert scale > 1.0
    err = (got.float() - ref).abs().max().item()
    assert err < (1e-5 if f32 else 1.6e-2 if got.dtype == torch.bfloat16 else 2e-3) * scale, (err, scale)


@pytest.mark.parametrize("M", [1, 2, 7, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("N,K", [(200, 96), (1000, 1000), (77, 4104), (4096, 264)])
def test_gemm_skinny(ops, M, N, K):
    """The weight-streaming product for few rows: widths that are no multiple of the 16-row
    tile or of the 32-wide k-block, one weight row much larger than the rest (a wrong row or
    a dropped k-block would show)."""
    x = rnd(M, K, seed=300 + M).to(torch.bfloat16)
    w = rnd(N, K, seed=301, scale=0.1).to(torch.bfloat16)
    w[N - 1] *= 30
    w[5, K - 3:] = 4.0
    want = x.double() @ w.double().T
    for out_dtype, bound in ((torch.float32, 2e-3), (torch.bfloat16, 1.6e-2)):
        y = ops.gemm_skinny(dev(x), dev(w), out_dtype)
        assert y.dtype == out_dtype and y.shape == (M, N)
        assert (y.cpu().double() - want).abs().max() < bound * want.abs().max()
    # linear() takes this path for bfloat16 and agrees with the library path on more rows
    y16 = ops.linear(dev(x), dev(w), out_dtype=torch.float32)
    assert (y16.cpu().double() - want).abs().max() < 2e-3 * want.abs().max()
    with pytest.raises(ops.KernelError, match="multiple of 8"):
        ops.gemm_skinny(dev(x[:, :K - 4].contiguous()), dev(w[:, :K - 4].contiguous()), torch.float32)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (200, 304, 328), (300, 1000, 136), (1000, 512, 4104),
                                   (2048, 1536, 1024)])
@pytest.mark.parametrize("swiglu", [False, "stacked", "interleaved"])
@pytest.mark.parametrize("short_tiles", [False, True])
def test_gemm_tcgen05(ops, M, N, K, swiglu, short_tiles):
    """The TMA + tcgen05 product: row and column counts that end inside a tile, K that ends
    inside a 64-wide block, several tiles per block (both accumulators in turn), fused SwiGLU
    with gate and up rows stacked or interleaved by eight.  One weight row and one k-column are
    made much larger than the rest."""
    if swiglu == "interleaved" and N % 16:
        pytest.skip("interleaved rows come in sixteens")
    x = rnd(M, K, seed=400, scale=0.5).to(torch.bfloat16)
    w = rnd(N, K, seed=401, scale=0.5).to(torch.bfloat16)
    w[N - 1] *= 8
    w[:, K - 1] *= 6
    ref = x.double() @ w.double().T
    if swiglu:
        ref = plain.silu(ref[:, :N // 2]) * ref[:, N // 2:]
    if swiglu == "interleaved":
        w = ops.interleave_gate_up(w[:N // 2], w[N // 2:])
    y = ops.gemm_tcgen05(dev(x), dev(w), bool(swiglu), short_tiles, interleaved=swiglu == "interleaved")
    ops.check_error_word("cuda:0")
    assert y.shape == ref.shape and y.dtype == torch.bfloat16
    assert (y.cpu().double() - ref).abs().max() < 1.6e-2 * ref.abs().max()


def test_linear_takes_the_tcgen05_path_for_many_rows(ops):
    assert ops.tcgen05_pays(2048, 4096, 4096, torch.bfloat16) and not ops.tcgen05_pays(2048, 6144, 4096, torch.bfloat16)
    assert not ops.tcgen05_pays(64, 4096, 4096, torch.bfloat16) and not ops.tcgen05_pays(2048, 4096, 4096, torch.float32)
    x = rnd(600, 136, seed=410).to(torch.bfloat16)
    w = rnd(2 * 5376, 136, seed=411, scale=0.3).to(torch.bfloat16)
    before = ops.tcgen05_calls
    act = ops.linear_swiglu(dev(x), dev(w), torch.bfloat16)
    assert ops.tcgen05_calls == before + 1
    ref = x.double() @ w.double().T
    ref = plain.silu(ref[:, :5376]) * ref[:, 5376:]
    ops.check_error_word("cuda:0")
    assert (act.cpu().double() - ref).abs().max() < 1.6e-2 * ref.abs().max()
    small = ops.linear_swiglu(dev(x[:9]), dev(w), torch.bfloat16)           # few rows: two kernels, same values
    assert ops.tcgen05_calls == before + 1
    assert (small.cpu().double() - ref[:9]).abs().max() < 1.6e-2 * ref.abs().max()
    wi = dev(ops.interleave_gate_up(w[:5376], w[5376:]))                     # the layout the feed-forward part stores
    for rows in (600, 9, 40):
        act = ops.linear_swiglu(dev(x[:rows]), wi, torch.bfloat16, interleaved=True)
        ops.check_error_word("cuda:0")
        assert (act.cpu().double() - ref[:rows]).abs().max() < 1.6e-2 * ref.abs().max()
    assert ops.tcgen05_calls == before + 2
    # the plain product through ``linear``: 3 x 42 tiles of 256 x 256
    w2 = rnd(10752, 136, seed=412, scale=0.3).to(torch.bfloat16)
    y = ops.linear(dev(x), dev(w2))
    assert ops.tcgen05_calls == before + 3
    ops.check_error_word("cuda:0")
    full = x.double() @ w2.double().T
    assert (y.cpu().double() - full).abs().max() < 1.6e-2 * full.abs().max()
    y9 = ops.linear(dev(x[:9]), dev(w2))                                     # the library's, same values
    assert ops.tcgen05_calls == before + 3
    assert (y9.cpu().double() - full[:9]).abs().max() < 1.6e-2 * full.abs().max()


@pytest.mark.parametrize("M", [1, 5, 8])
@pytest.mark.parametrize("inter,K", [(200, 96), (1000, 1000), (77, 4104)])
def test_linear_swiglu_few_rows(ops, M, inter, K):
    """Gate/up product and SwiGLU for few rows, as the engine runs them and as one
    weight-streaming kernel, against the plain formulas."""
    x = rnd(M, K, seed=500 + M, scale=0.5).to(torch.bfloat16)
    w = rnd(2 * inter, K, seed=501, scale=0.2).to(torch.bfloat16)
    w[inter - 1] *= 10
    w[2 * inter - 1] *= 10
    ref = x.double() @ w.double().T
    ref = plain.silu(ref[:, :inter]) * ref[:, inter:]
    acts = [ops.linear_swiglu(dev(x), dev(w), torch.bfloat16)]
    if inter % 8 == 0:
        wi = dev(ops.interleave_gate_up(w[:inter], w[inter:]))
        acts += [ops.gemm_skinny_swiglu(dev(x), wi),
                 ops.linear_swiglu(dev(x), wi, torch.bfloat16, interleaved=True)]
    else:
        with pytest.raises(ops.KernelError, match="multiple of 8"):
            ops.gemm_skinny_swiglu(dev(x), dev(w))
    for act in acts:
        assert act.shape == (M, inter)
        assert (act.cpu().double() - ref).abs().max() < 1.6e-2 * ref.abs().max()
