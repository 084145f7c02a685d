"""Grouped-query attention over the paged cache, with optional per-head norm of queries
and keys, a position encoding of its own choice and an optional sliding window.

Per layer the reference computes q, k, v with three products, norms q and k per head
with the layer's eps before the rotation, rotates, writes k and v of every row of the
step into the cache and only then attends, each row against the keys j <= pos of its own
request, scale 1/sqrt(head_dim) (model/src/qwen3_paged_batch.cpp:150-264,
kernels/src/paged_attention_cuda.cu:70-120).  Here the three projections are one product
with the row-wise concatenation [Wq; Wk; Wv] (fused at load time; the checkpoint keeps
them apart, model/src/qwen3_layers.cpp:220-222), and norm, rotation and cache write are
one kernel.  The window (keys pos - window + 1 .. pos) has no counterpart in the
reference, which has full attention only.
"""
from __future__ import annotations

import math
from typing import Dict, Optional

import torch

from .. import ops
from .registry import lookup, register
from .spec import CacheSpec, ParamSpec, PartSpec, StateSpec


@register("mixer", "gq_attention")
class GroupedQueryAttention:
    graph_safe = True      # every launch reads the step's data from device buffers: capturable

    def __init__(self, hidden_size: int, q_heads: int, kv_heads: int, head_dim: int,
                 dtype: torch.dtype, device, qk_norm_eps: Optional[float] = None,
                 position: Optional[PartSpec] = None, window: Optional[int] = None,
                 scale: Optional[float] = None):
        if q_heads % kv_heads:
            raise ValueError(f"{q_heads} query heads cannot share {kv_heads} key/value heads")
        if qk_norm_eps is not None and not qk_norm_eps > 0.0:
            raise ValueError(f"qk_norm_eps must be positive (or None for no head norm), got {qk_norm_eps}")
        self.hidden, self.q_heads, self.kv_heads, self.head_dim = hidden_size, q_heads, kv_heads, head_dim
        self.dtype, self.device = dtype, device
        self.qk_norm_eps = qk_norm_eps
        self.window = window
        self.scale = float(scale) if scale is not None else 1.0 / math.sqrt(head_dim)
        self.position = None
        if position is not None:
            self.position = lookup("position", position.kind)(dtype=dtype, device=device, **position.params)
        self.w_qkv = self.w_o = self.q_gain = self.k_gain = None

    # ---- weights
    @classmethod
    def param_specs(cls, hidden_size, q_heads, kv_heads, head_dim, qk_norm_eps=None, **_) -> Dict[str, ParamSpec]:
        specs = {
            "q_proj.weight": ParamSpec((q_heads * head_dim, hidden_size)),
            "k_proj.weight": ParamSpec((kv_heads * head_dim, hidden_size)),
            "v_proj.weight": ParamSpec((kv_heads * head_dim, hidden_size)),
            "o_proj.weight": ParamSpec((hidden_size, q_heads * head_dim)),
        }
        if qk_norm_eps is not None:
            specs["q_norm.weight"] = ParamSpec((head_dim,), "norm")
            specs["k_norm.weight"] = ParamSpec((head_dim,), "norm")
        return specs

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        parts = [t["q_proj.weight"], t["k_proj.weight"], t["v_proj.weight"]]
        common = torch.float32 if any(p.dtype == torch.float32 for p in parts) else parts[0].dtype
        self.w_qkv = torch.cat([p.to(common) for p in parts], dim=0).contiguous()
        self.w_o = t["o_proj.weight"].contiguous()
        if self.qk_norm_eps is not None:
            gains = [t["q_norm.weight"], t["k_norm.weight"]]
            gd = torch.float32 if any(g.dtype == torch.float32 for g in gains) else gains[0].dtype
            self.q_gain, self.k_gain = (g.to(gd).contiguous() for g in gains)

    # ---- what the cache manager has to provide
    def cache_spec(self) -> Optional[CacheSpec]:
        return CacheSpec.keys_and_values(self.kv_heads, self.head_dim, self.window)

    def state_spec(self) -> Optional[StateSpec]:
        return None

    def workspace_floats(self, tokens: int) -> int:
        return tokens * (3 * self.q_heads + 2 * self.kv_heads) * self.head_dim     # q|k|v, q, the heads' outputs

    # ---- one step
    def forward(self, x: torch.Tensor, ctx, cache) -> torch.Tensor:
        tokens = x.shape[0]
        qkv = ops.linear(x, self.w_qkv, out_dtype=self.dtype)
        q = torch.empty((tokens, self.q_heads * self.head_dim), dtype=self.dtype, device=x.device)
        norm = ops.QK_NORM if self.qk_norm_eps is not None else 0
        store = ops.QK_STORE if cache.writes else 0
        eps = self.qk_norm_eps if self.qk_norm_eps is not None else 1.0
        args = dict(positions=ctx.positions, token_slot=ctx.token_slot, block_table=cache.block_table,
                    cache=cache.kv, page_size=cache.page_size, q_out=q, q_heads=self.q_heads,
                    kv_heads=self.kv_heads, head_dim=self.head_dim)
        fused = self.position.fused_rotary() if self.position is not None and hasattr(self.position, "fused_rotary") else None
        if self.position is None or fused is not None:
            inv_freq, rotary_dim = fused if fused is not None else (None, 0)
            rope = ops.QK_ROPE if fused is not None else 0
            table = None
            if fused is not None and rotary_dim == self.head_dim and hasattr(self.position, "step_table"):
                table = self.position.step_table(ctx)          # cosines and sines once per step, not per layer
            ops.qk_norm_rope_store(qkv, self.q_gain, self.k_gain, eps, inv_freq, rotary_dim,
                                   flags=norm | rope | store | ops.QK_QOUT, table=table, **args)
        else:
            # a position encoding the kernel does not know: norm, let the part rotate, then store
            ops.qk_norm_rope_store(qkv, self.q_gain, self.k_gain, eps, None, 0,
                                   flags=norm | ops.QK_QOUT | ops.QK_KVOUT, **args)
            qd = self.q_heads * self.head_dim
            kd = self.kv_heads * self.head_dim
            self.position.apply(q.view(tokens, self.q_heads, self.head_dim),
                                qkv[:, qd:qd + kd].view(tokens, self.kv_heads, self.head_dim),
                                ctx.positions)
            if store:
                ops.qk_norm_rope_store(qkv, None, None, 1.0, None, 0, flags=ops.QK_STORE, **args)
        out = torch.empty_like(q)
        ops.paged_attention(q, cache.kv, ctx.positions, ctx.token_slot, cache.block_table,
                            cache.page_size, self.q_heads, self.kv_heads, self.head_dim,
                            self.window, self.scale, out, ctx=ctx)
        return ops.linear(out, self.w_o, out_dtype=self.dtype)
