"""Stand-ins for the CUDA kernels, for tests that run without a GPU.

The package has no CPU path.  To exercise its host-side logic (step function, cache
manager, scheduler, trace replay) on a machine without a GPU, tests swap the functions
of ``tiny_llm_infer_b200.ops`` for these slow torch restatements with the same
signatures.  They are test doubles, not a fallback: nothing in the package imports them.
"""
from __future__ import annotations


import torch

from tiny_llm_infer_b200 import ops

NAMES = ["embedding", "add_rmsnorm", "swiglu", "cast", "qk_norm_rope_store", "paged_attention",
         "sample", "linear", "linear_swiglu", "interleave_gate_up", "feed_tokens"]


def install(monkeypatch):
    for name in NAMES:
        monkeypatch.setattr(ops, name, globals()[name])


def embedding(ids, table, out):
    idx = ids.long()
    out.copy_(torch.where((idx >= 0)[:, None], table[idx.clamp(min=0)].float(), torch.zeros(())))
    return out


def add_rmsnorm(h, delta, gain, eps, out, rows=None):
    v = h if delta is None else h + delta.float()
    if rows is None:
        if delta is not None:
            h.copy_(v)
    else:
        v = v[rows.long()]
    y = gain.float() * v * torch.rsqrt((v * v).mean(-1, keepdim=True) + eps)
    out[:y.shape[0]].copy_(y.to(out.dtype))
    return out


def swiglu(gate_up, out, interleaved=False):
    inter = out.shape[1]
    if interleaved:                  # groups of sixteen columns: eight gates, their eight ups
        pairs = gate_up.float().reshape(gate_up.shape[0], inter // 8, 2, 8)
        g, u = pairs[:, :, 0].reshape(-1, inter), pairs[:, :, 1].reshape(-1, inter)
    else:
        g, u = gate_up[:, :inter].float(), gate_up[:, inter:].float()
    out.copy_((g / (1 + torch.exp(-g)) * u).to(out.dtype))
    return out


def cast(src, dtype):
    return src.to(dtype)


def feed_tokens(ids, places, rows, sampled):
    ids[places.long()] = sampled[rows.long()]


def linear(x, weight, out_dtype=None):
    want = out_dtype or x.dtype
    return (x.float() @ weight.float().t()).to(want)


def interleave_gate_up(gate, up):
    inter, k = gate.shape
    return torch.stack([gate.reshape(inter // 8, 8, k), up.reshape(inter // 8, 8, k)], dim=1).reshape(2 * inter, k)


def linear_swiglu(x, w_gate_up, out_dtype, interleaved=False):
    gate_up = linear(x, w_gate_up, out_dtype)
    out = torch.empty((x.shape[0], w_gate_up.shape[0] // 2), dtype=out_dtype)
    return swiglu(gate_up, out, interleaved)


def qk_norm_rope_store(qkv, q_gain, k_gain, eps, inv_freq, rotary_dim, positions, token_slot,
                       block_table, cache, page_size, q_out, q_heads, kv_heads, head_dim, flags, table=None):
    T = qkv.shape[0]
    x = qkv.float().view(T, q_heads + 2 * kv_heads, head_dim)
    q, k, v = x[:, :q_heads], x[:, q_heads:q_heads + kv_heads], x[:, q_heads + kv_heads:]
    if flags & ops.QK_NORM:
        q = q_gain.float() * q * torch.rsqrt((q * q).mean(-1, keepdim=True) + eps)
        k = k_gain.float() * k * torch.rsqrt((k * k).mean(-1, keepdim=True) + eps)
    if flags & ops.QK_ROPE and rotary_dim:
        half = rotary_dim // 2
        ang = positions.float()[:, None] * inv_freq[None, :]
        c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]

        def rot(t):
            a, b, rest = t[..., :half], t[..., half:rotary_dim], t[..., rotary_dim:]
            return torch.cat([a * c - b * s, a * s + b * c, rest], -1)
        q, k = rot(q), rot(k)
    live = token_slot >= 0
    if flags & ops.QK_QOUT:
        q_out[live] = q.reshape(T, -1).to(q_out.dtype)[live]
    if flags & ops.QK_KVOUT:
        qd = q_heads * head_dim
        qkv[:, qd:qd + kv_heads * head_dim][live] = k.reshape(T, -1).to(qkv.dtype)[live]
    if flags & ops.QK_STORE:
        for t in range(T):
            slot = int(token_slot[t])
            if slot < 0:
                continue
            pos = int(positions[t])
            page = int(block_table[slot, pos // page_size])
            assert page >= 0, "store into a page that is not held"
            cache[page, 0, :, pos % page_size] = k[t].to(cache.dtype)
            cache[page, 1, :, pos % page_size] = v[t].to(cache.dtype)


def paged_attention(q, cache, positions, token_slot, block_table, page_size, q_heads, kv_heads,
                    head_dim, window, scale, out, ctx=None):
    T = q.shape[0]
    group = q_heads // kv_heads
    for t in range(T):
        slot = int(token_slot[t])
        if slot < 0:
            out[t] = 0
            continue
        pos = int(positions[t])
        lo = max(0, pos - window + 1) if window else 0
        js = torch.arange(lo, pos + 1)
        pages = block_table[slot, js // page_size].long()
        assert (pages >= 0).all(), "attention reads a page that is not held"
        keys = cache[pages, 0, :, js % page_size].float()      # [n, kvh, hd]
        vals = cache[pages, 1, :, js % page_size].float()
        qt = q[t].float().view(q_heads, head_dim)
        for h in range(q_heads):
            g = h // group
            s = (keys[:, g] @ qt[h]) * scale
            p = torch.softmax(s, 0)
            out[t, h * head_dim:(h + 1) * head_dim] = (p @ vals[:, g]).to(out.dtype)
    return out


def sample(logits, params, seeds, out, any_nucleus=None):
    from plain_qwen3 import gumbel_scores, nucleus
    import numpy as np
    for r in range(logits.shape[0]):
        temp, top_p = float(params[r, 0]), float(params[r, 1])
        lg = logits[r].double().numpy()
        if not temp > 1e-6:
            out[r] = int(np.argmax(lg))
            continue
        scores = gumbel_scores(lg, temp, int(seeds[r]) & ((1 << 64) - 1))
        if top_p < 1.0:
            keep = nucleus(lg, temp, top_p)
            mask = np.full_like(scores, -np.inf)
            mask[keep] = scores[keep]
            scores = mask
        out[r] = int(np.argmax(scores))
    return out
