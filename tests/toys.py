"""Parts and an architecture that exist only in the tests: a mixer with state of its own
(a running mean), a partial rotary encoding, a run order that names a layer twice and lets
a layer read another layer's cache.  They are registered through the package's public
registries, without a change to its files, and restated with the plain implementation's
functions."""
from dataclasses import dataclass

import torch

import plain_qwen3 as plain

def register_toys():
    from tiny_llm_infer_b200 import ops
    from tiny_llm_infer_b200.config.base import ModelConfig, register_architecture
    from tiny_llm_infer_b200.parts import ExecEntry, LayerSpec, ModelDescription, ParamSpec, PartSpec, StateSpec
    from tiny_llm_infer_b200.parts.registry import register

    @register("mixer", "toy_running_mean")
    class RunningMean:
        """delta[t] = W . mean(x[0..t]) of the token's own request; the sum so far and the
        count are its per-request state."""

        def __init__(self, hidden_size, dtype, device):
            self.h, self.dtype = hidden_size, dtype
            self.w = None

        @classmethod
        def param_specs(cls, hidden_size):
            return {"mix.weight": ParamSpec((hidden_size, hidden_size))}

        def load(self, t):
            self.w = t["mix.weight"].contiguous()

        def cache_spec(self):
            return None

        def state_spec(self):
            return StateSpec((self.h + 1,), "float32")

        def forward(self, x, ctx, cache):
            out = torch.zeros_like(x)
            for seg in ctx.segments:
                st = cache.state[seg.slot]
                xs = x[seg.start:seg.start + seg.length].float()
                sums = torch.cumsum(xs, 0) + st[:self.h]
                count = st[self.h] + torch.arange(1, seg.length + 1, device=x.device)
                out[seg.start:seg.start + seg.length] = (sums / count[:, None]).to(x.dtype)
                st[:self.h] = sums[-1]
                st[self.h] += seg.length
            return ops.linear(out, self.w, out_dtype=self.dtype)

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        hidden_size: int = 48
        vocab_size: int = 160
        intermediate_size: int = 72
        max_position_embeddings: int = 256
        norm_eps: float = 1e-5
        architecture: str = "ToyStatefulLM"

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["hidden_size"], raw["vocab_size"], raw["intermediate_size"],
                       raw["max_position_embeddings"], raw["norm_eps"])

        def to_dict(self):
            return dict(architectures=[self.architecture], hidden_size=self.hidden_size,
                        vocab_size=self.vocab_size, intermediate_size=self.intermediate_size,
                        max_position_embeddings=self.max_position_embeddings, norm_eps=self.norm_eps)

        def validate(self):
            assert self.hidden_size > 0

    def describe(cfg):
        H = cfg.hidden_size
        norm = dict(width=H, eps=cfg.norm_eps)
        attn = dict(hidden_size=H, q_heads=3, kv_heads=1, head_dim=16, qk_norm_eps=cfg.norm_eps,
                    position=PartSpec("rotary_half", dict(head_dim=16, theta=1e4, rotary_dim=8)))
        ffn = PartSpec("swiglu", dict(hidden_size=H, intermediate_size=cfg.intermediate_size))

        def layer(i, mixer):
            p = f"layers.{i}."
            return LayerSpec("prenorm", {
                "norm1": PartSpec("rmsnorm", norm, p + "n1."), "mixer": PartSpec(mixer[0], mixer[1], p + "mixer."),
                "norm2": PartSpec("rmsnorm", norm, p + "n2."),
                "ffn": PartSpec(ffn.kind, ffn.params, p + "ffn.")})
        layers = (layer(0, ("toy_running_mean", dict(hidden_size=H))), layer(1, ("gq_attention", attn)),
                  layer(2, ("gq_attention", attn)))
        # layer 1 runs twice (second visit with a cache of its own); layer 2 reads the cache
        # that the first visit of layer 1 wrote
        order = (ExecEntry(0), ExecEntry(1, cache=10), ExecEntry(2, cache=10, writes_cache=False),
                 ExecEntry(1), ExecEntry(0))
        return ModelDescription(H, cfg.vocab_size, cfg.max_position_embeddings,
                                PartSpec("token_embedding", dict(vocab_size=cfg.vocab_size, hidden_size=H), "embed."),
                                layers, order, PartSpec("rmsnorm", norm, "final."),
                                PartSpec("lm_head", dict(vocab_size=cfg.vocab_size, hidden_size=H, tied=False), "head."))

    register_architecture("ToyStatefulLM", ToyConfig, describe)
    return ToyConfig


def toy_plain(w, ids, eps):
    """The toy model restated with the plain implementation's functions."""
    F = torch.float64
    T = len(ids)
    pos = torch.arange(T)
    h = w["embed.weight"][torch.tensor(ids)]

    def rope8(x):
        return torch.cat([plain.rotary_half(x[..., :8], pos, 1e4), x[..., 8:]], -1)

    def qkv(x, p):
        q = (x @ w[p + "q_proj.weight"].T).view(T, 3, 16)
        k = (x @ w[p + "k_proj.weight"].T).view(T, 1, 16)
        v = (x @ w[p + "v_proj.weight"].T).view(T, 1, 16)
        return (rope8(plain.rms_norm(q, w[p + "q_norm.weight"], eps)),
                rope8(plain.rms_norm(k, w[p + "k_norm.weight"], eps)), v)

    def ffn(h, p):
        x = plain.rms_norm(h, w[p + "n2.weight"], eps)
        return h + plain.feed_forward(x, w[p + "ffn.gate_proj.weight"], w[p + "ffn.up_proj.weight"],
                                      w[p + "ffn.down_proj.weight"])

    def mean_layer(h):
        x = plain.rms_norm(h, w["layers.0.n1.weight"], eps)
        m = torch.cumsum(x, 0) / torch.arange(1, T + 1, dtype=F)[:, None]
        return ffn(h + m @ w["layers.0.mixer.mix.weight"].T, "layers.0.")

    def attn_layer(h, i, kv=None):
        p = f"layers.{i}."
        q, k, v = qkv(plain.rms_norm(h, w[p + "n1.weight"], eps), p + "mixer.")
        if kv is not None:
            k, v = kv
        o = plain.causal_attention(q, k, v).reshape(T, 48) @ w[p + "mixer.o_proj.weight"].T
        return ffn(h + o, p), (k, v)

    h = mean_layer(h)
    h, kv1 = attn_layer(h, 1)
    h, _ = attn_layer(h, 2, kv1)
    h, _ = attn_layer(h, 1)
    h = mean_layer(h)
    return plain.rms_norm(h, w["final.weight"], eps) @ w["head.weight"].T
