"""Parts and an architecture that exist only in the tests: a mixer with state of its own
(a running mean), a feed-forward with a router over two experts, a position encoding that is
no rotation (and a partial rotary one), a run order that names a layer twice and lets a
layer read another layer's cache.  They are registered through the package's public
registries, without a change to its files, and restated with the plain implementation's
functions.  A second toy architecture (``register_sandwich``) has a block of four norms (one before
and one after each sub-layer), a block with two mixers side by side, and a mixer whose cache is
one vector per token (a single plane) instead of keys and values."""
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

    @register("feed_forward", "toy_routed")
    class RoutedExperts:
        """Two SwiGLU experts weighted by a router: delta = sum_e softmax(x Wr^T)_e * expert_e(x),
        router logits and weights in float32."""

        def __init__(self, hidden_size, intermediate_size, dtype, device):
            self.h, self.i, self.dtype = hidden_size, intermediate_size, dtype
            self.router = None
            self.experts = []

        @classmethod
        def param_specs(cls, hidden_size, intermediate_size):
            specs = {"router.weight": ParamSpec((2, hidden_size))}
            for e in range(2):
                specs[f"experts.{e}.gate_proj.weight"] = ParamSpec((intermediate_size, hidden_size))
                specs[f"experts.{e}.up_proj.weight"] = ParamSpec((intermediate_size, hidden_size))
                specs[f"experts.{e}.down_proj.weight"] = ParamSpec((hidden_size, intermediate_size))
            return specs

        def load(self, t):
            self.router = t["router.weight"].float().contiguous()
            self.experts = [(torch.cat([t[f"experts.{e}.gate_proj.weight"], t[f"experts.{e}.up_proj.weight"]]).contiguous(),
                             t[f"experts.{e}.down_proj.weight"].contiguous()) for e in range(2)]

        def forward(self, x, ctx):
            weights = torch.softmax(x.float() @ self.router.T, dim=-1)
            out = torch.zeros(x.shape, dtype=torch.float32, device=x.device)
            for e, (w_gate_up, w_down) in enumerate(self.experts):
                act = ops.linear_swiglu(x, w_gate_up, out_dtype=self.dtype)
                out += weights[:, e:e + 1] * ops.linear(act, w_down, out_dtype=self.dtype).float()
            return out.to(self.dtype)

    @register("position", "toy_cosine_gate")
    class CosineGate:
        """Not a rotation: element i of every query and key head is scaled by cos(pos * (i + 1) / 40).
        The attention part does not know it and calls ``apply`` between its norm and the cache."""

        def __init__(self, head_dim, dtype, device):
            self.freq = ((torch.arange(head_dim, dtype=torch.float32) + 1) / 40).to(device)

        @classmethod
        def param_specs(cls, **params):
            return {}

        def load(self, tensors):
            pass

        def apply(self, q, k, positions):
            gate = torch.cos(positions.float()[:, None] * self.freq[None, :])[:, None, :]
            q.copy_((q.float() * gate).to(q.dtype))
            k.copy_((k.float() * gate).to(k.dtype))

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
        gated = dict(attn, position=PartSpec("toy_cosine_gate", dict(head_dim=16)))
        routed = PartSpec("toy_routed", dict(hidden_size=H, intermediate_size=40))

        def layer3():
            p = "layers.3."
            return LayerSpec("prenorm", {
                "norm1": PartSpec("rmsnorm", norm, p + "n1."), "mixer": PartSpec("gq_attention", gated, p + "mixer."),
                "norm2": PartSpec("rmsnorm", norm, p + "n2."), "ffn": PartSpec(routed.kind, routed.params, p + "ffn.")})
        layers = (layer(0, ("toy_running_mean", dict(hidden_size=H))), layer(1, ("gq_attention", attn)),
                  layer(2, ("gq_attention", attn)), layer3())
        # layer 1 runs twice (second visit with a cache of its own); layer 2 reads the cache
        # that the first visit of layer 1 wrote
        order = (ExecEntry(0), ExecEntry(1, cache=10), ExecEntry(2, cache=10, writes_cache=False),
                 ExecEntry(3), ExecEntry(1), ExecEntry(0))
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

    def gated_routed_layer(h):
        p = "layers.3."
        x = plain.rms_norm(h, w[p + "n1.weight"], eps)
        gate = torch.cos(pos.to(F)[:, None] * ((torch.arange(16, dtype=F) + 1) / 40)[None, :])[:, None, :]
        q = plain.rms_norm((x @ w[p + "mixer.q_proj.weight"].T).view(T, 3, 16), w[p + "mixer.q_norm.weight"], eps) * gate
        k = plain.rms_norm((x @ w[p + "mixer.k_proj.weight"].T).view(T, 1, 16), w[p + "mixer.k_norm.weight"], eps) * gate
        v = (x @ w[p + "mixer.v_proj.weight"].T).view(T, 1, 16)
        h = h + plain.causal_attention(q, k, v).reshape(T, 48) @ w[p + "mixer.o_proj.weight"].T
        x = plain.rms_norm(h, w[p + "n2.weight"], eps)
        weights = torch.softmax(x @ w[p + "ffn.router.weight"].T, dim=-1)
        return h + sum(weights[:, e:e + 1] * plain.feed_forward(x, *(w[p + f"ffn.experts.{e}.{n}_proj.weight"]
                                                                     for n in ("gate", "up", "down"))) for e in range(2))

    h = mean_layer(h)
    h, kv1 = attn_layer(h, 1)
    h, _ = attn_layer(h, 2, kv1)
    h = gated_routed_layer(h)
    h, _ = attn_layer(h, 1)
    h = mean_layer(h)
    return plain.rms_norm(h, w["final.weight"], eps) @ w["head.weight"].T


def register_sandwich():
    """ToySandwichLM: layer 0 is a block of four norms around attention and SwiGLU; layer 1 has two
    mixers that read the same normed input, attention and a mixer that caches one latent vector of
    24 numbers per token and returns a projection of the mean of its request's latents so far."""
    from tiny_llm_infer_b200 import ops
    from tiny_llm_infer_b200.config.base import ModelConfig, register_architecture
    from tiny_llm_infer_b200.parts import (CacheSpec, ExecEntry, LayerSpec, ModelDescription, ParamSpec,
                                           PartSpec)
    from tiny_llm_infer_b200.parts.block import Block
    from tiny_llm_infer_b200.parts.registry import register

    @register("mixer", "toy_latent_mean")
    class LatentMean:
        LATENT = 24

        def __init__(self, hidden_size, dtype, device):
            self.h, self.dtype = hidden_size, dtype
            self.w_in = self.w_out = None

        @classmethod
        def param_specs(cls, hidden_size):
            return {"in.weight": ParamSpec((cls.LATENT, hidden_size)), "out.weight": ParamSpec((hidden_size, cls.LATENT))}

        def load(self, t):
            self.w_in, self.w_out = t["in.weight"].contiguous(), t["out.weight"].contiguous()

        def cache_spec(self):
            return CacheSpec(((1, self.LATENT),))        # one plane, one head: no keys, no values

        def state_spec(self):
            return None

        def workspace_floats(self, tokens):
            return tokens * (self.LATENT + self.h)

        def forward(self, x, ctx, cache):
            assert cache.kv is not None and len(cache.planes) == 1 and tuple(cache.planes[0].shape[1:]) == (1, cache.page_size, self.LATENT)
            latents = ops.linear(x, self.w_in, out_dtype=self.dtype)
            pages, ps = cache.planes[0], cache.page_size
            means = torch.zeros((x.shape[0], self.LATENT), dtype=torch.float32, device=x.device)
            for seg in ctx.segments:
                end = seg.pos0 + seg.length
                pos = torch.arange(end, device=x.device)
                page = cache.block_table[seg.slot, pos // ps].long()
                if cache.writes:
                    pages[page[seg.pos0:], 0, pos[seg.pos0:] % ps] = latents[seg.start:seg.start + seg.length]
                so_far = torch.cumsum(pages[page, 0, pos % ps].float(), 0) / (pos + 1)[:, None]
                means[seg.start:seg.start + seg.length] = so_far[seg.pos0:]
            return ops.linear(means.to(self.dtype), self.w_out, out_dtype=self.dtype)

    @register("block", "toy_sandwich")
    class Sandwich(Block):
        """h += post1(mixer(pre1(h)));  h += post2(ffn(pre2(h)))."""
        roles = {"pre1": "norm", "mixer": "mixer", "post1": "norm", "pre2": "norm", "ffn": "feed_forward",
                 "post2": "norm"}

        def forward(self, h, pending, ctx, cache):
            x = self.pre1.forward(h, pending)
            a = self.post1.forward(self.mixer.forward(x, ctx, cache).float(), None)
            x = self.pre2.forward(h, a)
            return self.post2.forward(self.ffn.forward(x, ctx).float(), None)

    @register("block", "toy_two_mixers")
    class TwoMixers(Block):
        """h += attention(norm1(h)) + latent(norm1(h));  h += ffn(norm2(h)): two mixers, two caches."""
        roles = {"norm1": "norm", "attention": "mixer", "latent": "mixer", "norm2": "norm", "ffn": "feed_forward"}

        def forward(self, h, pending, ctx, cache):
            x = self.norm1.forward(h, pending)
            a = self.attention.forward(x, ctx, cache[0])
            b = self.latent.forward(x, ctx, cache[1])
            x = self.norm2.forward(h, (a.float() + b.float()).to(a.dtype))
            return self.ffn.forward(x, ctx)

    @dataclass(frozen=True)
    class SandwichConfig(ModelConfig):
        hidden_size: int = 40
        vocab_size: int = 120
        max_position_embeddings: int = 256
        norm_eps: float = 1e-5
        architecture: str = "ToySandwichLM"

        @classmethod
        def from_dict(cls, raw):
            return cls(raw["hidden_size"], raw["vocab_size"], raw["max_position_embeddings"], raw["norm_eps"])

        def to_dict(self):
            return dict(architectures=[self.architecture], hidden_size=self.hidden_size, vocab_size=self.vocab_size,
                        max_position_embeddings=self.max_position_embeddings, norm_eps=self.norm_eps)

        def validate(self):
            assert self.hidden_size > 0

    def describe(cfg):
        H = cfg.hidden_size
        norm = dict(width=H, eps=cfg.norm_eps)
        attn = dict(hidden_size=H, q_heads=2, kv_heads=1, head_dim=16, qk_norm_eps=cfg.norm_eps,
                    position=PartSpec("rotary_half", dict(head_dim=16, theta=1e4)))
        ffn = dict(hidden_size=H, intermediate_size=56)
        layers = (
            LayerSpec("toy_sandwich", {
                "pre1": PartSpec("rmsnorm", norm, "l0.pre1."), "mixer": PartSpec("gq_attention", attn, "l0.attn."),
                "post1": PartSpec("rmsnorm", norm, "l0.post1."), "pre2": PartSpec("rmsnorm", norm, "l0.pre2."),
                "ffn": PartSpec("swiglu", ffn, "l0.ffn."), "post2": PartSpec("rmsnorm", norm, "l0.post2.")}),
            LayerSpec("toy_two_mixers", {
                "norm1": PartSpec("rmsnorm", norm, "l1.n1."), "attention": PartSpec("gq_attention", attn, "l1.attn."),
                "latent": PartSpec("toy_latent_mean", dict(hidden_size=H), "l1.latent."),
                "norm2": PartSpec("rmsnorm", norm, "l1.n2."), "ffn": PartSpec("swiglu", ffn, "l1.ffn.")}))
        order = (ExecEntry(0), ExecEntry(1, cache=(7, 8)), ExecEntry(0))
        return ModelDescription(H, cfg.vocab_size, cfg.max_position_embeddings,
                                PartSpec("token_embedding", dict(vocab_size=cfg.vocab_size, hidden_size=H), "embed."),
                                layers, order, PartSpec("rmsnorm", norm, "final."),
                                PartSpec("lm_head", dict(vocab_size=cfg.vocab_size, hidden_size=H, tied=True), "head."))

    register_architecture("ToySandwichLM", SandwichConfig, describe)
    return SandwichConfig


def sandwich_plain(w, ids, eps):
    """ToySandwichLM restated with the plain implementation's functions."""
    F = torch.float64
    T = len(ids)
    pos = torch.arange(T)
    h = w["embed.weight"][torch.tensor(ids)]

    def attention(x, p):
        q = (x @ w[p + "q_proj.weight"].T).view(T, 2, 16)
        k = (x @ w[p + "k_proj.weight"].T).view(T, 1, 16)
        v = (x @ w[p + "v_proj.weight"].T).view(T, 1, 16)
        q = plain.rotary_half(plain.rms_norm(q, w[p + "q_norm.weight"], eps), pos, 1e4)
        k = plain.rotary_half(plain.rms_norm(k, w[p + "k_norm.weight"], eps), pos, 1e4)
        return plain.causal_attention(q, k, v).reshape(T, 32) @ w[p + "o_proj.weight"].T

    def ffn(x, p):
        return plain.feed_forward(x, w[p + "gate_proj.weight"], w[p + "up_proj.weight"], w[p + "down_proj.weight"])

    def sandwich(h):
        a = attention(plain.rms_norm(h, w["l0.pre1.weight"], eps), "l0.attn.")
        h = h + plain.rms_norm(a, w["l0.post1.weight"], eps)
        m = ffn(plain.rms_norm(h, w["l0.pre2.weight"], eps), "l0.ffn.")
        return h + plain.rms_norm(m, w["l0.post2.weight"], eps)

    def two_mixers(h):
        x = plain.rms_norm(h, w["l1.n1.weight"], eps)
        latents = x @ w["l1.latent.in.weight"].T
        mean = torch.cumsum(latents, 0) / torch.arange(1, T + 1, dtype=F)[:, None]
        h = h + attention(x, "l1.attn.") + mean @ w["l1.latent.out.weight"].T
        return h + ffn(plain.rms_norm(h, w["l1.n2.weight"], eps), "l1.ffn.")

    h = sandwich(two_mixers(sandwich(h)))
    return plain.rms_norm(h, w["final.weight"], eps) @ w["embed.weight"].T
