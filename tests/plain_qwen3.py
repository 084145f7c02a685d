"""Plain, slow implementation of Qwen3 dense: whole sequences, no cache, no batching,
one function per part, float64 arithmetic on the CPU.  It shares no code with the
package: it reads config.json as a dict and the weights through the ``safetensors``
library, and every formula is restated from the reference's source (cited per function,
paths inside xu797/tiny-llm-infer).

It rests on the reference's formulas and is cross-checked once against the reference's
own CPU code path on a tiny random model (tests/golden/).  The sliding window and the
untied head are not in the reference; their definitions are stated where they appear.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import numpy as np
import torch
from safetensors import safe_open

F = torch.float64


def read_model(folder):
    """(config dict, {name: float64 tensor}) of a model folder."""
    folder = Path(folder)
    cfg = json.loads((folder / "config.json").read_text())
    files = sorted(folder.glob("*.safetensors"))
    weights = {}
    for f in files:
        with safe_open(str(f), framework="pt") as fh:
            for name in fh.keys():
                weights[name] = fh.get_tensor(name).to(F)
    return cfg, weights


def head_dim_of(cfg):
    # model/src/qwen3_checkpoint.cpp:35,46: head_dim, or hidden / heads when absent or 0
    return cfg.get("head_dim") or cfg["hidden_size"] // cfg["num_attention_heads"]


def layer_window(cfg, layer):
    """Window of a layer or None.  Not in the reference (full attention only); the keys
    follow the checkpoint's own config.json: ``layer_types[layer] == 'sliding_attention'``,
    or ``use_sliding_window`` with layers >= ``max_window_layers`` sliding."""
    types = cfg.get("layer_types")
    if types is not None:
        sliding = types[layer] == "sliding_attention"
    elif cfg.get("use_sliding_window"):
        sliding = layer >= cfg.get("max_window_layers", cfg["num_hidden_layers"])
    else:
        sliding = False
    return cfg["sliding_window"] if sliding else None


def rms_norm(x, gain, eps):
    # kernels/src/rmsnorm_kernel_cpu.cpp:27-43: scale = 1/sqrt(sum(x^2)/n + eps); out = gain * x * scale
    return gain * x * torch.rsqrt((x * x).mean(-1, keepdim=True) + eps)


def rotary_half(x, positions, theta):
    """x [T, heads, hd].  kernels/src/rope_kernel_cpu.cpp:127-141 (table: frequency
    theta^(-2i/hd), angle = pos * frequency, both float32) and :143-180 (pairs (i, i+hd/2):
    x_i cos - x_{i+hd/2} sin,  x_i sin + x_{i+hd/2} cos)."""
    hd = x.shape[-1]
    half = hd // 2
    i = torch.arange(half, dtype=F)
    freq = (theta ** (-2.0 * i / hd)).to(torch.float32)
    angle = (positions.to(torch.float32)[:, None] * freq[None, :]).to(F)   # float32 product
    cos, sin = torch.cos(angle)[:, None, :], torch.sin(angle)[:, None, :]
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1)


def causal_attention(q, k, v, window=None):
    """q [T, nh, hd], k and v [T, nkv, hd] of one whole sequence.
    kernels/src/paged_attention_cpu.cpp:16-69: query head h uses kv head h / (nh / nkv);
    score_j = (q . k_j) / sqrt(hd) for j <= pos only; softmax with the maximum subtracted;
    output = sum_j p_j v_j.  With a window (not in the reference) the keys are
    pos - window + 1 .. pos."""
    T, nh, hd = q.shape
    nkv = k.shape[1]
    group = nh // nkv
    scale = 1.0 / math.sqrt(hd)
    out = torch.zeros_like(q)
    pos = torch.arange(T)
    allowed = pos[None, :] <= pos[:, None]
    if window is not None:
        allowed &= pos[None, :] > pos[:, None] - window
    for h in range(nh):
        g = h // group
        s = (q[:, h] @ k[:, g].T) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        s = s - s.max(-1, keepdim=True).values
        p = torch.exp(s)
        p = p / p.sum(-1, keepdim=True)
        out[:, h] = p @ v[:, g]
    return out


def silu(x):
    # kernels/src/swiglu_kernel_cpu.cpp:20-24: x / (1 + exp(-x))
    return x / (1.0 + torch.exp(-x))


def feed_forward(x, w_gate, w_up, w_down):
    # model/src/qwen3_paged_batch.cpp:281-295: down(silu(gate(x)) * up(x)), no biases
    return (silu(x @ w_gate.T) * (x @ w_up.T)) @ w_down.T


def attention_block(x, w, prefix, cfg, layer, positions):
    """model/src/qwen3_paged_batch.cpp:150-271: q, k, v projections without bias; RMSNorm
    of every q and k head over head_dim with the model's eps and a gain shared by the heads
    (model/src/qwen3_layers.cpp:224-228), before the rotation; v untouched; attention;
    output projection."""
    T = x.shape[0]
    nh, nkv, hd = cfg["num_attention_heads"], cfg.get("num_key_value_heads") or cfg["num_attention_heads"], head_dim_of(cfg)
    eps, theta = cfg.get("rms_norm_eps", 1e-6), cfg.get("rope_theta", 1e6)
    q = (x @ w[prefix + "q_proj.weight"].T).view(T, nh, hd)
    k = (x @ w[prefix + "k_proj.weight"].T).view(T, nkv, hd)
    v = (x @ w[prefix + "v_proj.weight"].T).view(T, nkv, hd)
    q = rotary_half(rms_norm(q, w[prefix + "q_norm.weight"], eps), positions, theta)
    k = rotary_half(rms_norm(k, w[prefix + "k_norm.weight"], eps), positions, theta)
    o = causal_attention(q, k, v, layer_window(cfg, layer))
    return o.reshape(T, nh * hd) @ w[prefix + "o_proj.weight"].T


def decoder_layer(h, w, cfg, layer, positions):
    # model/src/qwen3_paged_batch.cpp:146-301: pre-norm attention, residual, pre-norm MLP, residual
    p = f"model.layers.{layer}."
    eps = cfg.get("rms_norm_eps", 1e-6)
    h = h + attention_block(rms_norm(h, w[p + "input_layernorm.weight"], eps), w, p + "self_attn.",
                            cfg, layer, positions)
    x = rms_norm(h, w[p + "post_attention_layernorm.weight"], eps)
    return h + feed_forward(x, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"],
                            w[p + "mlp.down_proj.weight"])


def hidden_states(cfg, w, token_ids):
    """Residual stream after the last layer, [T, H]."""
    ids = torch.as_tensor(token_ids, dtype=torch.long)
    positions = torch.arange(len(ids))
    h = w["model.embed_tokens.weight"][ids]          # kernels/src/embed_kernel_cpu.cpp:8-45, no scaling
    for layer in range(cfg["num_hidden_layers"]):
        h = decoder_layer(h, w, cfg, layer, positions)
    return h


def logits_of(cfg, w, token_ids):
    """Logits at every position of one whole sequence, [T, V] float64.
    model/src/qwen3_paged_batch.cpp:304-346: final RMSNorm, then the head.  The reference
    always multiplies by the embedding matrix (model/src/qwen3_layers.cpp:246-265); an
    untied head (``tie_word_embeddings`` false) uses ``lm_head.weight`` instead."""
    h = hidden_states(cfg, w, token_ids)
    x = rms_norm(h, w["model.norm.weight"], cfg.get("rms_norm_eps", 1e-6))
    head = w["model.embed_tokens.weight"] if cfg.get("tie_word_embeddings", False) else w["lm_head.weight"]
    return x @ head.T


def greedy(cfg, w, prompt, n):
    """n greedy tokens after ``prompt``; lowest id on ties
    (engine/src/llm_engine.cpp:81-86, kernels/src/sampling_kernel_cuda.cu:25-27)."""
    ids = list(prompt)
    for _ in range(n):
        ids.append(int(torch.argmax(logits_of(cfg, w, ids)[-1])))
    return ids[len(prompt):]


# ---------------------------------------------------------------- sampling, restated
_M = (1 << 64) - 1


def _mix64(z):
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _M
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _M
    return z ^ (z >> 31)


def uniform_of(seed, token):
    """The engine's own counter-based generator (the reference uses Philox from cuRAND,
    kernels/src/sampling_kernel_cuda.cu:43-52, which cannot be restated on the host)."""
    r = _mix64((seed + 0x9E3779B97F4A7C15 * (token + 1)) & _M)
    return (float(r >> 41) + 0.5) / 8388608.0


def gumbel_scores(logits, temperature, seed):
    """logit_v + temperature * -log(-log u_v) (kernels/src/sampling_kernel_cuda.cu:50-54)."""
    u = np.array([uniform_of(seed, v) for v in range(len(logits))], dtype=np.float64)
    return np.asarray(logits, dtype=np.float64) + temperature * -np.log(-np.log(u))


def nucleus(logits, temperature, top_p):
    """Indices kept by top-p: weights exp((l - max)/T) sorted descending, kept until the
    running sum reaches top_p * total (engine/src/llm_engine.cpp:110-140)."""
    lg = np.asarray(logits, dtype=np.float64)
    w = np.exp((lg - lg.max()) / temperature)
    order = np.argsort(-w, kind="stable")
    csum = np.cumsum(w[order])
    k = int(np.searchsorted(csum, top_p * w.sum(), side="left")) + 1
    return order[:k]
