"""The command line (``bin/model_main`` = ``tiny_llm_infer_b200.cli``): its modes, the flags it
shares with the reference's ``model_main`` (model/model_main.cpp:41-60, 465-559) and what it
prints.  Without a GPU the engine behind it runs on the torch stand-ins (``--device cpu``, in
this process); with one, the script itself is run as a user would run it."""
import json
import subprocess
import sys
from pathlib import Path

import pytest
import torch

import plain_qwen3 as plain
from tiny import TINIES, make_folder, prompt

ROOT = Path(__file__).resolve().parent.parent
TOOL = ROOT / "bin" / "model_main"


def ids(text):
    return [int(t) for t in text.split(",")] if text else []


def csv(tokens):
    return ",".join(str(t) for t in tokens)


# ------------------------------------------------------------------ no GPU: in this process
def run_main(argv, capsys):
    from tiny_llm_infer_b200 import cli
    rc = cli.main(argv)
    out = capsys.readouterr()
    return rc, out.out, out.err


def test_write_random_model_and_what_needs_no_engine(tmp_path, capsys):
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(TINIES["B"]["cfg"].to_dict()))
    rc, out, _ = run_main(["--write-random-model", str(tmp_path / "m"), "--config", str(cfg_file),
                           "--random-weights", "1", "--weight-std", "0.05"], capsys)
    assert rc == 0 and out.strip() == str(tmp_path / "m")
    cfg, w = plain.read_model(tmp_path / "m")
    assert cfg["hidden_size"] == 96 and w["lm_head.weight"].shape == (384, 96)
    # the same seed gives the tensors that the tests' own folders have (norm gains differ by their range)
    again = plain.read_model(make_folder(dict(TINIES["B"], norm_range=(0.8, 1.2)), tmp_path / "m2"))[1]
    assert all(torch.equal(w[k], again[k]) for k in w)
    # --max-new-tokens 0 prints one empty line per prompt and loads nothing (model/model_main.cpp:396-400)
    rc, out, _ = run_main(["--infer", "--model", str(tmp_path / "nowhere"), "--prompt-ids", "1,2", "--prompt-ids", "3",
                           "--max-new-tokens", "0"], capsys)
    assert rc == 0 and out == "\n\n"
    for bad in (["--write-random-model", str(tmp_path / "x")],                 # no --config
                ["--infer", "--prompt-ids", "1"],                               # no --model
                ["--infer", "--model", "m"],                                    # no prompt
                ["--infer", "--model", "m", "--prompt", "text"],                # text without a tokenizer
                ["--bench", "--model", "m", "--min-input-len", "9", "--max-input-len", "5"],
                ["--bench", "--model", "m", "--repeats", "0"],
                ["--bench", "--model", "m", "--max-input-len", "200", "--max-output-len", "64"]):   # beyond --max-seq-len 256
        rc, _, err = run_main(bad, capsys)
        assert rc == 2 and err.strip(), bad
    with pytest.raises(SystemExit) as exit_info:                                # no mode at all
        run_main(["--model", "m"], capsys)
    assert exit_info.value.code == 2
    capsys.readouterr()


def test_infer_and_bench_on_the_host_side(tmp_path, capsys, cpu_ops):
    folder = make_folder(TINIES["A"], tmp_path / "m")
    cfg, w = plain.read_model(folder)
    prompts = [prompt(i, n, 256) for i, n in enumerate((5, 17))]
    argv = ["--infer", "--model", str(folder), "--device", "cpu", "--dtype", "float32", "--max-seq-len", "64",
            "--num-kv-blocks", "8", "--max-new-tokens", "6"]
    for p in prompts:
        argv += ["--prompt-ids", csv(p)]
    rc, out, _ = run_main(argv, capsys)
    assert rc == 0
    assert [ids(line) for line in out.splitlines()] == [plain.greedy(cfg, w, p, 6) for p in prompts]
    rc, out, err = run_main(["--bench", "--model", str(folder), "--device", "cpu", "--dtype", "float32",
                             "--num-seqs", "3", "--min-input-len", "4", "--max-input-len", "9", "--min-output-len", "2",
                             "--max-output-len", "5", "--warmup", "1", "--repeats", "2", "--max-seq-len", "32",
                             "--num-kv-blocks", "8", "--max-token-id", "255", "--manifest-prefix", str(tmp_path / "man")],
                            capsys)
    assert rc == 0 and "Warmup 1 complete." in err
    check_bench_output(out, tmp_path / "man", seqs=3, repeats=2)


def check_bench_output(out, manifest_prefix, seqs, repeats):
    """run= lines as the reference prints them (model/model_main.cpp:366-374) whose token counts are
    those of the requests in the manifests, and an aggregate line that adds them up."""
    runs = [dict(part.split("=") for part in line.split()) for line in out.splitlines() if line.startswith("run=")]
    total = [dict(part.split("=") for part in line.split()) for line in out.splitlines() if line.startswith("aggregate_runs=")]
    assert [int(r["run"]) for r in runs] == list(range(1, repeats + 1)) and len(total) == 1
    for r in runs:
        manifest = json.loads(Path(f"{manifest_prefix}_run{r['run']}.json").read_text())["requests"]
        assert len(manifest) == seqs == int(r["requests"])
        assert int(r["output_tokens"]) == sum(m["max_tokens"] for m in manifest)
        assert all(m["temperature"] == 0.6 and m["ignore_eos"] and m["top_p"] == 1.0 for m in manifest)
        assert float(r["output_tokens_per_second"]) == pytest.approx(int(r["output_tokens"]) / float(r["elapsed_seconds"]), rel=1e-3)
    assert int(total[0]["aggregate_runs"]) == repeats
    assert int(total[0]["output_tokens"]) == sum(int(r["output_tokens"]) for r in runs)
    assert float(total[0]["elapsed_seconds"]) == pytest.approx(sum(float(r["elapsed_seconds"]) for r in runs), abs=1e-4)


# ------------------------------------------------------------------ on the GPU: the script itself
def run_tool(*argv, timeout=600):
    res = subprocess.run([sys.executable, str(TOOL), *map(str, argv)], capture_output=True, text=True, timeout=timeout)
    return res.returncode, res.stdout, res.stderr


@pytest.mark.gpu
def test_model_main_on_the_gpu(tmp_path):
    cfg_file = tmp_path / "config.json"
    cfg_file.write_text(json.dumps(TINIES["B"]["cfg"].to_dict()))
    folder = tmp_path / "model"
    rc, out, err = run_tool("--write-random-model", folder, "--config", cfg_file, "--random-weights", 1, "--weight-std", 0.05)
    assert rc == 0, err
    cfg, w = plain.read_model(folder)
    prompts = [prompt(i, n, cfg["vocab_size"]) for i, n in enumerate((1, 9, 40))]
    common = ["--model", folder, "--max-seq-len", 128, "--num-kv-blocks", 40]
    flags = [x for p in prompts for x in ("--prompt-ids", csv(p))]

    # greedy in float32 is the plain implementation's choice, token for token
    rc, out, err = run_tool("--infer", *common, *flags, "--dtype", "float32", "--max-new-tokens", 7)
    assert rc == 0, err[-2000:]
    assert [ids(line) for line in out.splitlines()] == [plain.greedy(cfg, w, p, 7) for p in prompts]

    # the model may be named by its .safetensors file, with config.json beside it (model/src/qwen3_checkpoint.cpp:19-22)
    rc, out2, err = run_tool("--infer", "--model", folder / "model.safetensors", "--max-seq-len", 128, "--num-kv-blocks", 40,
                             *flags, "--dtype", "float32", "--max-new-tokens", 7)
    assert rc == 0 and out2 == out, err[-2000:]

    # sampling flags give what LLM.generate gives for the same settings
    rc, out, err = run_tool("--infer", *common, *flags, "--dtype", "float32", "--max-new-tokens", 6,
                            "--temperature", 0.8, "--top-p", 0.7, "--seed", 21)
    assert rc == 0, err[-2000:]
    from tiny_llm_infer_b200 import LLM, SamplingParams
    llm = LLM(str(folder), dtype="float32", max_model_len=128, num_kv_blocks=40, block_size=16,
              max_num_batched_tokens=128, max_num_seqs=3)
    want = llm.generate(prompts, SamplingParams(max_tokens=6, temperature=0.8, top_p=0.7, seed=21))
    assert [ids(line) for line in out.splitlines()] == [o.token_ids for o in want]

    rc, out, err = run_tool("--infer", *common, *flags, "--max-new-tokens", 0)
    assert rc == 0 and out == "\n\n\n"

    rc, out, err = run_tool("--bench", "--model", folder, "--num-seqs", 5, "--min-input-len", 8, "--max-input-len", 40,
                            "--min-output-len", 3, "--max-output-len", 9, "--warmup", 1, "--repeats", 2,
                            "--max-seq-len", 64, "--max-token-id", cfg["vocab_size"] - 1, "--manifest-prefix", tmp_path / "man")
    assert rc == 0, err[-2000:]
    check_bench_output(out, tmp_path / "man", seqs=5, repeats=2)

    for bad in (["--infer", *common], ["--bench", "--model", folder, "--min-output-len", 0],
                ["--infer", "--model", folder, "--prompt", "text"]):
        rc, _, err = run_tool(*bad)
        assert rc == 2 and err.strip(), bad


@pytest.mark.gpu
def test_pool_sized_from_free_memory(tmp_path):
    """``num_kv_blocks=0``: the pool is what the reference's rule leaves beside the weights
    (model/src/qwen3.cpp:96-151: total * utilisation - used - max(256 MiB, total / 20, workspace)),
    capped at what ``max_num_seqs`` requests of ``max_model_len`` tokens can hold
    (model/model_main.cpp:284-303); and the engine then generates."""
    from tiny_llm_infer_b200 import LLM, SamplingParams
    from tiny_llm_infer_b200.cache import CacheManager
    from tiny_llm_infer_b200.engine import load_model
    from tiny_llm_infer_b200.engine.llm_engine import estimate_num_kv_blocks
    tiny = TINIES["B"]
    folder = make_folder(tiny, tmp_path / "m")
    cfg, w = plain.read_model(folder)
    model, config = load_model(folder, torch.bfloat16, "cuda:0")
    # the arithmetic, with a made-up device of 10 GiB of which 3 GiB are in use
    total, free = 10 << 30, 7 << 30
    per_page = 3 * 2 * 2 * 8 * 32 * 2                   # layers * (K, V) * kv heads * page * head width * bytes
    assert CacheManager.bytes_per_page(model.cache_needs(), 8, torch.bfloat16) == {None: per_page}
    # residual stream and rows of the model's width; the widest part (attention: q|k|v, q and the heads'
    # outputs, wider here than the SwiGLU's 3 * 200 per token); the logits of 16 rows
    workspace = 4 * (6 * 32 * 96 + max(3 * 32 * 200, 32 * (3 * 6 + 2 * 2) * 32) + 16 * 384)
    assert 4 * model.workspace_floats(32, 16) == workspace
    want = (int(total * 0.5) - (total - free) - max(256 << 20, total // 20, workspace)) // per_page
    assert estimate_num_kv_blocks(model, 8, torch.bfloat16, 32, 0.5, "cuda:0", 16, memory=(free, total)) == want
    assert estimate_num_kv_blocks(model, 8, torch.bfloat16, 32, 0.2, "cuda:0", 16, memory=(free, total)) == 0
    with pytest.raises(ValueError):
        estimate_num_kv_blocks(model, 8, torch.bfloat16, 32, 0.99, "cuda:0")
    # on the real device more pages fit than four requests of 96 tokens can use: the cap decides
    assert estimate_num_kv_blocks(model, 8, torch.bfloat16, 32, 0.9, "cuda:0", 4) > 4 * 12
    llm = LLM(None, dtype="bfloat16", max_model_len=96, num_kv_blocks=0, block_size=8, max_num_batched_tokens=32,
              max_num_seqs=4, gpu_memory_utilization=0.9, loaded=(model, config))
    assert llm.cache.capacity_pages() == {None: 4 * 12}
    prompts = [prompt(i, n, cfg["vocab_size"]) for i, n in enumerate((5, 19, 40))]
    outs = llm.generate(prompts, SamplingParams(max_tokens=6, ignore_eos=True))
    for p, o in zip(prompts, outs):
        logits = plain.logits_of(cfg, w, (p + o.token_ids)[:-1]).numpy()
        for i, tok in enumerate(o.token_ids):
            row = logits[len(p) - 1 + i]
            assert row[tok] >= row.max() - 0.1, (i, tok, int(row.argmax()))
    llm.cache.audit()
