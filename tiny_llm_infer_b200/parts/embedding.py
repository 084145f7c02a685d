"""Token embedding and the output head.

h0[t] = E[token[t]], no scaling (reference: kernels/src/embed_kernel_cuda.cu:6-28); the
logits of the wanted rows are hN[row] . W^T in float32.  The reference always uses the
embedding matrix as W (model/src/qwen3_layers.cpp:246-265); here ``tied`` decides, and an
untied head reads ``lm_head.weight``.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import ops
from .registry import register
from .spec import ParamSpec


@register("embedding", "token_embedding")
class TokenEmbedding:
    def __init__(self, vocab_size: int, hidden_size: int, dtype: torch.dtype, device):
        self.vocab, self.hidden, self.dtype, self.device = vocab_size, hidden_size, dtype, device
        self.weight: Optional[torch.Tensor] = None

    @classmethod
    def param_specs(cls, vocab_size, hidden_size) -> Dict[str, ParamSpec]:
        return {"weight": ParamSpec((vocab_size, hidden_size))}

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        self.weight = t["weight"].contiguous()

    def forward(self, token_ids: torch.Tensor) -> torch.Tensor:
        h = torch.empty((token_ids.numel(), self.hidden), dtype=torch.float32, device=token_ids.device)
        return ops.embedding(token_ids, self.weight, h)


@register("head", "lm_head")
class LMHead:
    def __init__(self, vocab_size: int, hidden_size: int, tied: bool, dtype: torch.dtype, device):
        self.vocab, self.hidden, self.tied, self.dtype, self.device = vocab_size, hidden_size, tied, dtype, device
        self.weight: Optional[torch.Tensor] = None

    @classmethod
    def param_specs(cls, vocab_size, hidden_size, tied) -> Dict[str, ParamSpec]:
        return {} if tied else {"weight": ParamSpec((vocab_size, hidden_size))}

    def load(self, t: Dict[str, torch.Tensor]) -> None:
        if not self.tied:
            self.weight = t["weight"].contiguous()

    def tie(self, embedding: TokenEmbedding) -> None:
        if self.tied:
            self.weight = embedding.weight

    def workspace_floats(self, rows: int) -> int:
        return rows * self.vocab                 # the logits

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return ops.linear(x, self.weight, out_dtype=torch.float32)
