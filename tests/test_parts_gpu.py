"""Each part of a layer alone on the GPU against the plain implementation's function for
it: norm, position encoding, attention mixer (through a cache of its own, in two portions),
feed-forward, the block arrangement, embedding and head.  Sizes differ from the tiny
models'."""

import pytest
import torch

import plain_qwen3 as plain

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rnd(*shape, seed=0, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return torch.randn(*shape, generator=g, dtype=torch.float64) * scale


def tol(dtype, scale):
    return (5e-5 if dtype == torch.float32 else 3e-2) * max(scale, 1.0)


def context(segments, device=DEV):
    """StepContext for rows given as (slot, pos0, length) segments."""
    from tiny_llm_infer_b200.engine import Segment, StepContext
    pos, slot, segs, row = [], [], [], 0
    for s, p0, n in segments:
        pos += list(range(p0, p0 + n))
        slot += [s] * n
        segs.append(Segment(f"r{s}", s, row, n, p0))
        row += n
    t = lambda x: torch.tensor(x, dtype=torch.int32, device=device)
    return StepContext(tokens=row, token_ids=t([0] * row), positions=t(pos), token_slot=t(slot),
                       want_rows=t(list(range(row))), segments=segs, decode_only=False,
                       max_context=max(p + n for _, p, n in segments), max_segment=max(n for *_, n in segments))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from tiny_llm_infer_b200.parts.norm import RMSNorm
    part = RMSNorm(width=136, eps=3e-4, dtype=dtype, device=DEV)
    assert list(RMSNorm.param_specs(width=136, eps=3e-4)) == ["weight"]
    gain = (rnd(136, seed=1) * 0.2 + 1).to(dtype)
    part.load({"weight": gain.to(DEV)})
    h, delta = rnd(9, 136, seed=2).float(), rnd(9, 136, seed=3).to(dtype)
    hd = h.to(DEV)
    x = part.forward(hd, delta.to(DEV))
    v = h.double() + delta.double()
    want = plain.rms_norm(v, gain.double(), 3e-4)
    assert x.dtype == dtype and (x.cpu().double() - want).abs().max() < tol(dtype, want.abs().max().item())
    assert (hd.cpu().double() - v).abs().max() < 1e-5


def test_rotary_part_frequencies():
    from tiny_llm_infer_b200.parts.position import RotaryHalf
    part = RotaryHalf(head_dim=48, theta=5e4, dtype=torch.float32, device=DEV, rotary_dim=32)
    inv_freq, rot = part.fused_rotary()
    want = torch.tensor([5e4 ** (-2.0 * i / 32) for i in range(16)], dtype=torch.float64).float()
    assert rot == 32 and torch.equal(inv_freq.cpu(), want)
    with pytest.raises(ValueError):
        RotaryHalf(head_dim=48, theta=1e4, dtype=torch.float32, device=DEV, rotary_dim=50)


def attention_weights(H, nh, nkv, hd, dtype, seed):
    names = {"q_proj.weight": (nh * hd, H), "k_proj.weight": (nkv * hd, H), "v_proj.weight": (nkv * hd, H),
             "o_proj.weight": (H, nh * hd)}
    w = {k: rnd(*s, seed=seed + i, scale=0.08).to(dtype) for i, (k, s) in enumerate(names.items())}
    w["q_norm.weight"] = (rnd(hd, seed=seed + 7) * 0.2 + 1.5).to(dtype)
    w["k_norm.weight"] = (rnd(hd, seed=seed + 8) * 0.2 + 1.5).to(dtype)
    return w


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nh,nkv,hd,window", [(5, 1, 48, None), (4, 2, 80, 19)])
def test_attention_part_through_its_own_cache(dtype, nh, nkv, hd, window):
    from tiny_llm_infer_b200.cache import CacheManager
    from tiny_llm_infer_b200.parts import PartSpec
    from tiny_llm_infer_b200.parts.attention import GroupedQueryAttention
    H, T, eps, theta = 136, 45, 1e-5, 3e4
    part = GroupedQueryAttention(hidden_size=H, q_heads=nh, kv_heads=nkv, head_dim=hd, dtype=dtype, device=DEV,
                                 qk_norm_eps=eps, window=window,
                                 position=PartSpec("rotary_half", dict(head_dim=hd, theta=theta)))
    w = attention_weights(H, nh, nkv, hd, dtype, seed=10)
    part.load({k: v.to(DEV) for k, v in w.items()})
    cache = CacheManager({0: (part.cache_spec(), part.state_spec())}, 8, 12, 2, 64, dtype, DEV)
    cache.admit("x"), cache.admit("r")
    x = rnd(T, H, seed=20).to(dtype)
    outs = []
    for p0, n in ((0, 29), (29, 16)):                # two portions: the second reads the first from the cache
        cache.reserve("r", p0 + n)
        cache.sync()
        outs.append(part.forward(x[p0:p0 + n].to(DEV), context([(1, p0, n)]), cache.view(0)))
        cache.commit("r", p0 + n)
    got = torch.cat(outs).cpu().double()
    cfg = {"num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": hd, "hidden_size": H,
           "rms_norm_eps": eps, "rope_theta": theta, "num_hidden_layers": 1,
           "layer_types": ["sliding_attention" if window else "full_attention"], "sliding_window": window}
    want = plain.attention_block(x.double(), {"p." + k: v.double() for k, v in w.items()}, "p.", cfg, 0,
                                 torch.arange(T))
    assert (got - want).abs().max() < tol(dtype, want.abs().max().item())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("I", [328, 330])       # gate and up rows interleaved by eight, or stacked
def test_swiglu_part(dtype, I):
    from tiny_llm_infer_b200.parts.feed_forward import SwiGLUFeedForward
    H = 136
    part = SwiGLUFeedForward(hidden_size=H, intermediate_size=I, dtype=dtype, device=DEV)
    w = {"gate_proj.weight": rnd(I, H, seed=1, scale=0.1).to(dtype), "up_proj.weight": rnd(I, H, seed=2, scale=0.1).to(dtype),
         "down_proj.weight": rnd(H, I, seed=3, scale=0.1).to(dtype)}
    part.load({k: v.to(DEV) for k, v in w.items()})
    assert part.interleaved == (I % 8 == 0)
    for rows in (5, 11, 300):                    # the few-row kernels, the library (300 rows are too few tiles for tcgen05)
        x = rnd(rows, H, seed=4).to(dtype)
        got = part.forward(x.to(DEV), None).cpu().double()
        want = plain.feed_forward(x.double(), *(w[k].double() for k in ("gate_proj.weight", "up_proj.weight", "down_proj.weight")))
        assert (got - want).abs().max() < tol(dtype, want.abs().max().item())


def test_swiglu_part_on_the_tcgen05_product():
    """A feed-forward wide enough, with rows enough, that both of its products run on the tcgen05
    kernel (3 x 42 tiles of 256 x 128 for gate/up with SwiGLU, 3 x 42 of 256 x 256 for down)."""
    from tiny_llm_infer_b200 import ops
    from tiny_llm_infer_b200.parts.feed_forward import SwiGLUFeedForward
    H, I, rows, dtype = 10752, 5376, 600, torch.bfloat16
    part = SwiGLUFeedForward(hidden_size=H, intermediate_size=I, dtype=dtype, device=DEV)
    w = {"gate_proj.weight": rnd(I, H, seed=1, scale=0.02).to(dtype), "up_proj.weight": rnd(I, H, seed=2, scale=0.02).to(dtype),
         "down_proj.weight": rnd(H, I, seed=3, scale=0.02).to(dtype)}
    part.load({k: v.to(DEV) for k, v in w.items()})
    x = rnd(rows, H, seed=4).to(dtype)
    before = ops.tcgen05_calls
    got = part.forward(x.to(DEV), None)
    assert ops.tcgen05_calls == before + 2
    ops.check_error_word(DEV)
    xd = x.to(DEV).double()
    wd = {k: v.to(DEV).double() for k, v in w.items()}
    act = plain.silu(xd @ wd["gate_proj.weight"].T) * (xd @ wd["up_proj.weight"].T)
    want = act.to(dtype).double() @ wd["down_proj.weight"].T          # the part rounds the activation to bfloat16
    assert (got.double() - want).abs().max() < tol(dtype, want.abs().max().item())


def test_prenorm_block_equals_a_plain_decoder_layer():
    from tiny_llm_infer_b200.cache import CacheManager
    from tiny_llm_infer_b200.parts import PartSpec
    from tiny_llm_infer_b200.parts.attention import GroupedQueryAttention
    from tiny_llm_infer_b200.parts.block import PreNormBlock
    from tiny_llm_infer_b200.parts.feed_forward import SwiGLUFeedForward
    from tiny_llm_infer_b200.parts.norm import RMSNorm
    H, I, nh, nkv, hd, T, eps, theta, dtype = 72, 200, 3, 3, 16, 21, 1e-6, 1e4, torch.float32
    mixer = GroupedQueryAttention(hidden_size=H, q_heads=nh, kv_heads=nkv, head_dim=hd, dtype=dtype, device=DEV,
                                  qk_norm_eps=eps, position=PartSpec("rotary_half", dict(head_dim=hd, theta=theta)))
    ffn = SwiGLUFeedForward(hidden_size=H, intermediate_size=I, dtype=dtype, device=DEV)
    n1, n2 = (RMSNorm(width=H, eps=eps, dtype=dtype, device=DEV) for _ in range(2))
    aw = attention_weights(H, nh, nkv, hd, dtype, seed=30)
    fw = {"gate_proj.weight": rnd(I, H, seed=41, scale=0.1).float(), "up_proj.weight": rnd(I, H, seed=42, scale=0.1).float(),
          "down_proj.weight": rnd(H, I, seed=43, scale=0.1).float()}
    g1, g2 = ((rnd(H, seed=s) * 0.2 + 1).float() for s in (51, 52))
    mixer.load({k: v.to(DEV) for k, v in aw.items()}), ffn.load({k: v.to(DEV) for k, v in fw.items()})
    n1.load({"weight": g1.to(DEV)}), n2.load({"weight": g2.to(DEV)})
    block = PreNormBlock({"norm1": n1, "mixer": mixer, "norm2": n2, "ffn": ffn})
    cache = CacheManager({0: (mixer.cache_spec(), None)}, 16, 4, 1, 64, dtype, DEV)
    cache.admit("r"), cache.reserve("r", T), cache.sync()
    h0, pend0 = rnd(T, H, seed=60).float(), rnd(T, H, seed=61).float()
    h = h0.to(DEV)
    pending = block.forward(h, pend0.to(DEV), context([(0, 0, T)]), cache.view(0))
    got = h.cpu().double() + pending.cpu().double()
    w = {"model.layers.0.self_attn." + k: v.double() for k, v in aw.items()}
    w.update({"model.layers.0.mlp." + k: v.double() for k, v in fw.items()})
    w["model.layers.0.input_layernorm.weight"], w["model.layers.0.post_attention_layernorm.weight"] = g1.double(), g2.double()
    cfg = {"num_attention_heads": nh, "num_key_value_heads": nkv, "head_dim": hd, "hidden_size": H,
           "rms_norm_eps": eps, "rope_theta": theta, "num_hidden_layers": 1}
    want = plain.decoder_layer(h0.double() + pend0.double(), w, cfg, 0, torch.arange(T))
    assert (got - want).abs().max() < 1e-4


@pytest.mark.parametrize("tied", [True, False])
def test_embedding_and_head(tied):
    from tiny_llm_infer_b200.parts.embedding import LMHead, TokenEmbedding
    V, H, dtype = 517, 72, torch.bfloat16
    emb = TokenEmbedding(vocab_size=V, hidden_size=H, dtype=dtype, device=DEV)
    head = LMHead(vocab_size=V, hidden_size=H, tied=tied, dtype=dtype, device=DEV)
    assert (LMHead.param_specs(vocab_size=V, hidden_size=H, tied=tied) == {}) == tied
    E, W = rnd(V, H, seed=1).to(dtype), rnd(V, H, seed=2).to(dtype)
    emb.load({"weight": E.to(DEV)})
    head.load({} if tied else {"weight": W.to(DEV)})
    head.tie(emb)
    ids = torch.tensor([3, 516, 0, 3], dtype=torch.int32, device=DEV)
    h = emb.forward(ids)
    assert h.dtype == torch.float32 and torch.equal(h.cpu(), E.float()[ids.cpu().long()])
    x = rnd(4, H, seed=3).to(dtype)
    logits = head.forward(x.to(DEV))
    want = x.double() @ (E if tied else W).double().T
    assert logits.dtype == torch.float32 and (logits.cpu().double() - want).abs().max() < 1e-3 * want.abs().max()
