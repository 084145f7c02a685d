"""Tiny configurations for the tests.  A and B differ in every size and option: layers,
width, heads and groups, head width, feed-forward width (200 is no multiple of 128),
vocabulary, rope base, eps, tied or untied head, spread of the weights.  C adds sliding
layers (window 24) between full ones, with sizes of its own.  D has a head width (64) and
a page size (16) that the tensor-core attention kernels take, one full and one sliding layer.  E has
head width 128 (the tcgen05 prompt kernel); F has sizes that fit no fast path."""
from __future__ import annotations

import tempfile
from pathlib import Path

import torch

from tiny_llm_infer_b200.config import Qwen3Config
from tiny_llm_infer_b200.weights import write_random_model

FULL, SLIDING = "full_attention", "sliding_attention"

TINY_A = dict(cfg=Qwen3Config(hidden_size=64, intermediate_size=128, num_hidden_layers=2,
                              num_attention_heads=4, num_key_value_heads=2, head_dim=16, vocab_size=256,
                              max_position_embeddings=512, rms_norm_eps=1e-6, rope_theta=1e4,
                              tie_word_embeddings=True, layer_types=(FULL,) * 2),
              seed=0, std=0.02, norm_range=(0.8, 1.2), page_size=16)
TINY_B = dict(cfg=Qwen3Config(hidden_size=96, intermediate_size=200, num_hidden_layers=3,
                              num_attention_heads=6, num_key_value_heads=2, head_dim=32, vocab_size=384,
                              max_position_embeddings=512, rms_norm_eps=1e-5, rope_theta=1e6,
                              tie_word_embeddings=False, layer_types=(FULL,) * 3),
              seed=1, std=0.05, norm_range=(0.5, 1.5), page_size=8)
TINY_C = dict(cfg=Qwen3Config(hidden_size=80, intermediate_size=176, num_hidden_layers=4,
                              num_attention_heads=5, num_key_value_heads=5, head_dim=48, vocab_size=300,
                              max_position_embeddings=512, rms_norm_eps=1e-5, rope_theta=5e4,
                              tie_word_embeddings=False, sliding_window=24,
                              layer_types=(SLIDING, FULL, SLIDING, SLIDING)),
              seed=2, std=0.08, norm_range=(0.6, 1.4), page_size=16)
TINY_D = dict(cfg=Qwen3Config(hidden_size=128, intermediate_size=344, num_hidden_layers=2,
                              num_attention_heads=6, num_key_value_heads=2, head_dim=64, vocab_size=500,
                              max_position_embeddings=512, rms_norm_eps=1e-6, rope_theta=1e5,
                              tie_word_embeddings=True, sliding_window=80,
                              layer_types=(FULL, SLIDING)),
              seed=3, std=0.06, norm_range=(0.7, 1.3), page_size=16)
# head width 128: the width of the tcgen05 prompt kernel, with requests longer than its blocks
TINY_E = dict(cfg=Qwen3Config(hidden_size=192, intermediate_size=328, num_hidden_layers=2,
                              num_attention_heads=3, num_key_value_heads=1, head_dim=128, vocab_size=640,
                              max_position_embeddings=512, rms_norm_eps=3e-6, rope_theta=2e5,
                              tie_word_embeddings=False, sliding_window=150,
                              layer_types=(SLIDING, FULL)),
              seed=4, std=0.05, norm_range=(0.7, 1.3), page_size=32, lengths=(70, 300, 130, 41, 200, 35))
# sizes that fit no fast path: a head width of 80, three query heads on one key/value head, a model width
# and a feed-forward width that are no multiples of 16 (136, 100: gate and up stay stacked), an odd vocabulary
TINY_F = dict(cfg=Qwen3Config(hidden_size=136, intermediate_size=100, num_hidden_layers=2,
                              num_attention_heads=3, num_key_value_heads=1, head_dim=80, vocab_size=1001,
                              max_position_embeddings=512, rms_norm_eps=2e-6, rope_theta=3e4,
                              tie_word_embeddings=True, layer_types=(FULL,) * 2),
              seed=5, std=0.07, norm_range=(0.6, 1.4), page_size=16, lengths=(70, 97, 41, 35))
TINIES = {"A": TINY_A, "B": TINY_B, "C": TINY_C, "D": TINY_D, "E": TINY_E, "F": TINY_F}


def make_folder(tiny, folder=None, dtype=torch.bfloat16, shards=1) -> Path:
    folder = Path(folder or tempfile.mkdtemp(prefix="tllm_tiny_"))
    return write_random_model(folder, tiny["cfg"], tiny["seed"], tiny["std"], tiny["norm_range"],
                              dtype=dtype, shards=shards)


def prompt(seed: int, length: int, vocab: int):
    g = torch.Generator().manual_seed(1000 + seed)
    return torch.randint(0, vocab, (length,), generator=g).tolist()


def sharpen(folder, factor: float) -> None:
    """Scale the q/k head-norm gains so that attention scores spread out and single keys
    dominate: a wrong or missing key then changes the logits visibly."""
    from safetensors import safe_open
    from tiny_llm_infer_b200.weights import save_file
    path = Path(folder) / "model.safetensors"
    tensors = {}
    with safe_open(str(path), framework="pt") as fh:
        for name in fh.keys():
            t = fh.get_tensor(name).clone()      # the file is rewritten below
            if name.endswith("q_norm.weight") or name.endswith("k_norm.weight"):
                t = (t.float() * factor).to(t.dtype)
            tensors[name] = t
    save_file(tensors, path)


def requests_for(tiny, lengths=None):
    lengths = lengths or tiny.get("lengths", (70, 97, 130, 41, 66, 35))
    vocab = tiny["cfg"].vocab_size
    return {str(i): prompt(i, n, vocab) for i, n in enumerate(lengths)}
