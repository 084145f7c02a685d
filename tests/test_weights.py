"""Weights by tensor name: container, storage rule, the one error that lists everything,
random-weights mode."""

import pytest
import torch

from tiny_llm_infer_b200 import models  # noqa: F401
from tiny_llm_infer_b200.config import describe_model, load_config
from tiny_llm_infer_b200.models import expected_tensors
from tiny_llm_infer_b200.weights import (SafetensorsFile, WeightsError, load_weights, save_file,
                                         write_random_model)
from tiny import TINIES, make_folder


def expected_of(folder):
    return expected_tensors(describe_model(load_config(folder)))


def test_container_round_trip_against_the_library(tmp_path):
    from safetensors import safe_open
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).to(torch.bfloat16), "c": torch.arange(6, dtype=torch.int64).view(2, 3)}
    save_file(t, tmp_path / "x.safetensors", metadata={"k": "v"})
    with safe_open(str(tmp_path / "x.safetensors"), framework="pt") as fh:     # the library reads ours
        for k in t:
            assert torch.equal(fh.get_tensor(k), t[k])
    f = SafetensorsFile(tmp_path / "x.safetensors")                             # and we read it back
    for k in t:
        assert torch.equal(f.read(k).clone(), t[k])
    f.close()


def test_load_single_and_sharded_agree(tmp_path):
    a = make_folder(TINIES["B"], tmp_path / "one")
    b = make_folder(TINIES["B"], tmp_path / "four", shards=4)
    assert (b / "model.safetensors.index.json").is_file() and not (b / "model.safetensors").exists()
    exp, ign = expected_of(a)
    wa = load_weights(a, exp, torch.bfloat16, "cpu", ign)
    wb = load_weights(b, exp, torch.bfloat16, "cpu", ign)
    assert set(wa) == set(exp) == set(wb)
    assert all(torch.equal(wa[k], wb[k]) for k in wa)          # values do not depend on sharding
    assert all(v.dtype == torch.bfloat16 for v in wa.values())
    wf = load_weights(a / "model.safetensors", exp, torch.float32, "cpu", ign)   # a file path works too
    assert all(v.dtype == torch.float32 for v in wf.values())
    assert all(torch.equal(wf[k], wa[k].float()) for k in wa)  # widened exactly


def test_random_mode_is_seeded(tmp_path):
    a = make_folder(TINIES["A"], tmp_path / "a")
    b = make_folder(TINIES["A"], tmp_path / "b")
    c = write_random_model(tmp_path / "c", TINIES["A"]["cfg"], seed=99)
    assert (a / "model.safetensors").read_bytes() == (b / "model.safetensors").read_bytes()
    assert (a / "model.safetensors").read_bytes() != (c / "model.safetensors").read_bytes()
    exp, ign = expected_of(a)
    w = load_weights(a, exp, torch.float32, "cpu", ign)
    g = w["model.layers.1.input_layernorm.weight"]
    assert 0.8 <= g.min() and g.max() <= 1.2
    assert abs(w["model.embed_tokens.weight"].std().item() - 0.02) < 0.002
    assert "lm_head.weight" not in exp and ign == ["lm_head.weight"]     # tied head


def test_a_tensor_stored_in_32_bit_stays_so(tmp_path):
    folder = make_folder(TINIES["A"], tmp_path / "m", dtype=torch.float32)
    exp, ign = expected_of(folder)
    w = load_weights(folder, exp, torch.bfloat16, "cpu", ign)
    assert all(v.dtype == torch.float32 for v in w.values())


def rewrite(folder, edit):
    f = SafetensorsFile(folder / "model.safetensors")
    t = {k: f.read(k).clone() for k in f.tensors}
    f.close()
    edit(t)
    save_file(t, folder / "model.safetensors")


def test_one_error_lists_missing_unexpected_and_wrong_shapes(tmp_path):
    folder = make_folder(TINIES["B"], tmp_path / "m")

    def edit(t):
        del t["model.layers.1.mlp.up_proj.weight"]
        del t["model.norm.weight"]
        t["model.layers.7.extra.weight"] = torch.zeros(3)
        t["model.layers.0.self_attn.q_norm.weight"] = torch.zeros(31, dtype=torch.bfloat16)
        t["model.layers.2.self_attn.k_proj.weight"] = torch.zeros((64, 95), dtype=torch.bfloat16)
        t["model.embed_tokens.weight"] = torch.zeros((384, 96), dtype=torch.int32)
    rewrite(folder, edit)
    exp, ign = expected_of(folder)
    with pytest.raises(WeightsError) as info:
        load_weights(folder, exp, torch.bfloat16, "cpu", ign)
    err = info.value
    assert err.missing == ["model.layers.1.mlp.up_proj.weight", "model.norm.weight"]
    assert err.unexpected == ["model.layers.7.extra.weight"]
    assert sorted(n for n, _, _ in err.wrong_shape) == ["model.layers.0.self_attn.q_norm.weight",
                                                       "model.layers.2.self_attn.k_proj.weight"]
    assert err.wrong_dtype == [("model.embed_tokens.weight", "I32")]
    text = str(err)
    for needle in ("missing (2)", "unexpected (1)", "wrong shape (2)", "expected [32] found [31]", "extra.weight"):
        assert needle in text


def test_untied_head_needs_its_own_tensor(tmp_path):
    folder = make_folder(TINIES["B"], tmp_path / "m")
    rewrite(folder, lambda t: t.pop("lm_head.weight"))
    exp, ign = expected_of(folder)
    with pytest.raises(WeightsError, match="lm_head.weight"):
        load_weights(folder, exp, torch.bfloat16, "cpu", ign)


def test_broken_containers(tmp_path):
    folder = make_folder(TINIES["A"], tmp_path / "m")
    exp, ign = expected_of(folder)
    data = (folder / "model.safetensors").read_bytes()
    (folder / "model.safetensors").write_bytes(data[:len(data) // 2])
    with pytest.raises(WeightsError, match="offsets|header"):
        load_weights(folder, exp, torch.bfloat16, "cpu", ign)
    (folder / "model.safetensors").unlink()
    with pytest.raises(WeightsError, match="neither"):
        load_weights(folder, exp, torch.bfloat16, "cpu", ign)


def test_random_tensors_do_not_depend_on_slabs_or_device_order():
    """An element is a function of (seed, tensor name, its index): a tensor made whole, made as a flat
    vector or cut out of a longer run of the same counters holds the same values; other seeds and names
    hold others; the draws have the spread that was asked for."""
    from tiny_llm_infer_b200.parts.spec import ParamSpec
    from tiny_llm_infer_b200.weights import random_init as ri
    a = ri.random_tensor("w.weight", ParamSpec((37, 91)), 5, 0.05, (0.5, 1.5), torch.float32, "cpu")
    flat = ri.random_tensor("w.weight", ParamSpec((37 * 91,)), 5, 0.05, (0.5, 1.5), torch.float32, "cpu")
    assert torch.equal(a.view(-1), flat)
    key = ri._tensor_key(5, "w.weight")
    for start, n in ((0, 10), (1, 9), (3, 100), (1000, 37 * 91 - 1000)):          # odd starts cut a pair in two
        piece = (ri._normal(key, start, n, "cpu") * 0.05).to(torch.float32)
        assert torch.equal(piece, flat[start:start + n])
    assert not torch.equal(a, ri.random_tensor("w.weight", ParamSpec((37, 91)), 6, 0.05, (0.5, 1.5), torch.float32, "cpu"))
    assert not torch.equal(a, ri.random_tensor("v.weight", ParamSpec((37, 91)), 5, 0.05, (0.5, 1.5), torch.float32, "cpu"))
    big = ri.random_tensor("big", ParamSpec((400, 500)), 1, 0.05, (0.5, 1.5), torch.float32, "cpu")
    assert abs(big.mean().item()) < 1e-3 and abs(big.std().item() - 0.05) < 1e-3 and big.abs().max() < 0.3
    gains = ri.random_tensor("n.weight", ParamSpec((4096,), "norm"), 1, 0.05, (0.5, 1.5), torch.float32, "cpu")
    assert 0.5 <= gains.min() and gains.max() <= 1.5 and abs(gains.mean().item() - 1.0) < 0.02
    assert ri.random_tensor("t", ParamSpec((3,), "index"), 1, 0.05, (0.5, 1.5), torch.float32, "cpu").dtype == torch.int32


@pytest.mark.gpu
def test_a_model_filled_on_the_device_holds_the_folders_weights(tmp_path):
    """``random_model`` (tensors made on the GPU, part by part) and a folder written on the host from
    the same configuration and seed, read back through the loader, hold the same weights to the bit
    (the generator is integer and float64 arithmetic that both run alike), in both storage types."""
    from tiny_llm_infer_b200.engine import load_model, random_model
    tiny = TINIES["B"]
    folder = write_random_model(tmp_path / "m", tiny["cfg"], tiny["seed"], tiny["std"], tiny["norm_range"])
    for dtype in (torch.bfloat16, torch.float32):
        loaded, _ = load_model(folder, dtype, "cuda:0")
        made = random_model(tiny["cfg"], tiny["seed"], dtype, "cuda:0", std=tiny["std"], norm_range=tiny["norm_range"])
        for a, b in zip(loaded.parts(), made.parts()):
            for name, value in vars(a).items():
                if isinstance(value, torch.Tensor):
                    assert torch.equal(value, getattr(b, name)), (type(a).__name__, name)
        mixer_a, mixer_b = loaded.blocks[0].mixers()[0], made.blocks[0].mixers()[0]
        assert torch.equal(mixer_a.w_qkv, mixer_b.w_qkv) and mixer_a.w_qkv.dtype == dtype
