#!/usr/bin/env python3
"""Benchmark of the engine on one B200: decode and prefill throughput of a Qwen3-8B-shaped
model with random weights, in bfloat16.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl reference] [--model 8b|0.6b|32b] [--mixed]

A "step" is one decode step of a batch of 8 requests.  The headline ``value`` is decoded
tokens per second timed on the device (CUDA events around each step); ``e2e`` is the same
through the Python entry point (``LLMEngine.step``), host token ids in and out, timed by
the wall clock.  One JSON line is printed.  The sizes are those of Qwen3-8B
(the benchmark configuration); every request stands at a context of about 4096 tokens while it decodes
(the prompts are really prefilled, in portions of 2048 tokens, outside the timed region).

Beside the headline, in ``points`` (flat, numbers only): decode at batch 1 and 64 at the same context;
the reference's own benchmark workload (``p128_*``: 128-token prompts, 128 outputs, batch 1 / 8 / 64:
the decode steps alone timed on the device with their share of the HBM peak, and output tokens per
second end to end with the prompts inside the timed region, median of five runs after three
warm-ups); the mixed continuous-batching run that goes with the Qwen3-0.6B sizes.  ``prefill`` is one
prompt of 2048 tokens.  ``check``: the logits of the model that was timed, bfloat16 kernels against
the float32 path under four ways of cutting; a mismatch ends the run with an error line and code 1.

``--impl reference`` runs the unmodified reference (built by baseline/reference_arm/build.py into
baseline/_ref/) on the same sizes and the same decode workload through its own LLMEngine, and its own
``model_main --bench`` on the 128-token workload; it prints the same line with ``"impl": "reference"``,
or ``{"impl": "reference", "unavailable": why}``.

For more than one GPU this engine has nothing to run: it prints one line and exits 2.
"""
import argparse
import json
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# the benchmark configuration: Qwen3-8B shape, random weights N(0, 0.02), untied head, page 16
QWEN3_8B = dict(hidden_size=4096, intermediate_size=12288, num_hidden_layers=36, num_attention_heads=32,
                num_key_value_heads=8, head_dim=128, vocab_size=151936, max_position_embeddings=40960,
                rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)
# the two other sizes the reference is quoted on: the 0.6B shape (tied head) and the 32B shape (--model)
QWEN3_06B = dict(hidden_size=1024, intermediate_size=3072, num_hidden_layers=28, num_attention_heads=16,
                 num_key_value_heads=8, head_dim=128, vocab_size=151936, max_position_embeddings=40960,
                 rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=True)
QWEN3_32B = dict(hidden_size=5120, intermediate_size=25600, num_hidden_layers=64, num_attention_heads=64,
                 num_key_value_heads=8, head_dim=128, vocab_size=151936, max_position_embeddings=40960,
                 rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False)
MODELS = {"8b": ("Qwen3-8B shape", QWEN3_8B), "0.6b": ("Qwen3-0.6B shape", QWEN3_06B),
          "32b": ("Qwen3-32B shape", QWEN3_32B)}
CONTEXT = 4096
PAGE = 16
PREFILL_TOKENS = 2048
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


def peaks():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            raw = json.loads(path.read_text())
            out = {"hbm_gbs": float(raw["hbm_gbs"]), "bf16_tflops": float(raw["bf16_tflops"]),
                   "source": "measured"}
            if raw.get("bf16_tflops_sustained"):          # a seconds-long loop under the power cap
                out["bf16_tflops_sustained"] = float(raw["bf16_tflops_sustained"])
            return out
        except (KeyError, ValueError, TypeError):
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed regions run."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap,clocks.mem,power.draw")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.samples.append((time.perf_counter(), line.strip()))

    def stop(self, windows):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
        mhz, max_mhz, reasons = [], 0, set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for a, b, what in windows:                 # per timed region, for the log
            lines = [[p.strip() for p in line.split(",")] for t, line in self.samples if a <= t <= b]
            inside = [int(p[0]) for p in lines if p[0].isdigit()]
            if inside:
                mem = sorted({p[6] for p in lines if len(p) > 7})
                watts = [float(p[7]) for p in lines if len(p) > 7 and p[7].replace(".", "", 1).isdigit()]
                print(f"[bench] clocks during {what}: SM median {int(statistics.median(inside))} MHz, min {min(inside)}; "
                      f"memory {'/'.join(mem)} MHz; {int(statistics.median(watts)) if watts else '?'} W; {len(inside)} samples",
                      file=sys.stderr, flush=True)
        for t, line in self.samples:
            if windows and not any(a <= t <= b for a, b, _ in windows):
                continue
            parts = [p.strip() for p in line.split(",")]
            try:
                mhz.append(int(parts[0]))
                max_mhz = max(max_mhz, int(parts[1]))
            except (ValueError, IndexError):
                continue
            for name, val in zip(names, parts[2:]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": int(statistics.median(mhz)) if mhz else None, "sm_max_mhz": max_mhz or None,
                "reasons": sorted(reasons), "samples": len(mhz)}


# ---------------------------------------------------------------------- the reference arm
REF_BIN = ROOT / "baseline" / "_ref" / "bin"


def _unavailable(why: str) -> int:
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


def _reference_binaries():
    """The reference built by baseline/reference_arm/build.py (its sources unchanged, three stand-in
    headers); built now if its sources are at hand and the binaries are not."""
    need = [REF_BIN / "decode_main", REF_BIN / "model_main"]
    if all(p.is_file() for p in need):
        return need, None
    import os
    src = Path(os.environ.get("TLLM_REFERENCE", str(ROOT.parent / "reference")))    # or a folder beside this one
    if not (src / "model" / "model_main.cpp").is_file():
        return None, (f"the reference is not built (no {REF_BIN}) and its sources are not at {src}: "
                      "run baseline/reference_arm/build.py where they are")
    res = subprocess.run([sys.executable, str(ROOT / "baseline" / "reference_arm" / "build.py"), "--reference", str(src)],
                         capture_output=True, text=True)
    if res.returncode != 0 or not all(p.is_file() for p in need):
        return None, "building the reference failed: " + (res.stderr or res.stdout).strip().splitlines()[-1][:200]
    return need, None


def _write_reference_model(folder: Path, sizes: dict, seed: int = 0):
    """config.json, tokenizer.json and model.safetensors (FP16, the reference's storage type) of the
    given sizes with random weights N(0, 0.02) and norm gains U[0.8, 1.2], written with torch and the
    safetensors library alone.  The reference's tokenizer must know every id it may have to print
    (layers/src/encode.cpp:311-315): the vocabulary is t0, t1, ..."""
    import torch
    from safetensors.torch import save_file
    folder.mkdir(parents=True, exist_ok=True)
    cfg = dict(sizes, model_type="qwen3", architectures=["Qwen3ForCausalLM"], torch_dtype="float16")
    (folder / "config.json").write_text(json.dumps(cfg))
    vocab, hidden, inter = sizes["vocab_size"], sizes["hidden_size"], sizes["intermediate_size"]
    q = sizes["num_attention_heads"] * sizes["head_dim"]
    kv = sizes["num_key_value_heads"] * sizes["head_dim"]
    (folder / "tokenizer.json").write_text(json.dumps(
        {"model": {"vocab": {f"t{i}": i for i in range(vocab)}, "merges": []}, "added_tokens": []}))
    gen = torch.Generator(device="cuda").manual_seed(seed)

    def normal(*shape):
        return (torch.randn(shape, generator=gen, device="cuda", dtype=torch.float32) * 0.02).to(torch.float16).cpu()

    def gain(n):
        return (torch.rand(n, generator=gen, device="cuda") * 0.4 + 0.8).to(torch.float16).cpu()

    tensors = {"model.embed_tokens.weight": normal(vocab, hidden), "model.norm.weight": gain(hidden)}
    if not sizes.get("tie_word_embeddings"):
        tensors["lm_head.weight"] = normal(vocab, hidden)     # present as in a real checkpoint; the reference never reads it
    for i in range(sizes["num_hidden_layers"]):
        p = f"model.layers.{i}."
        tensors.update({
            p + "input_layernorm.weight": gain(hidden), p + "post_attention_layernorm.weight": gain(hidden),
            p + "self_attn.q_proj.weight": normal(q, hidden), p + "self_attn.k_proj.weight": normal(kv, hidden),
            p + "self_attn.v_proj.weight": normal(kv, hidden), p + "self_attn.o_proj.weight": normal(hidden, q),
            p + "self_attn.q_norm.weight": gain(sizes["head_dim"]), p + "self_attn.k_norm.weight": gain(sizes["head_dim"]),
            p + "mlp.gate_proj.weight": normal(inter, hidden), p + "mlp.up_proj.weight": normal(inter, hidden),
            p + "mlp.down_proj.weight": normal(hidden, inter)})
    save_file(tensors, str(folder / "model.safetensors"))
    del tensors
    torch.cuda.empty_cache()


def _standing_prompt_len(batch: int, steps: int, warmup: int, budget: int = 256) -> int:
    """Longest prompt with which decode_main's requests (which keep decoding while the other prompts
    are computed) stay inside CONTEXT until the timed steps are over."""
    n = CONTEXT
    while n > 1:
        budget_steps = -(-batch * n // budget)
        if n + warmup + steps + budget_steps + budget_steps // 8 + 16 <= CONTEXT:
            return n
        n -= 1
    return 1


def reference_arm(args, model_name: str, model_sizes: dict) -> int:
    """The unmodified reference on the same sizes and workload: decode steps of ``--batch`` requests
    standing at a context of about 4096 through its LLMEngine (``value`` and ``e2e``: its step() takes
    host token ids in and gives host token ids out, so the two are one number), and its own
    ``model_main --bench`` on 128-token prompts with 128 outputs (``points``)."""
    import os
    import shutil
    import tempfile
    if args.gpus != 1:
        print(f"bench.py: the reference runs on one GPU; --gpus {args.gpus} has nothing to measure")
        return 2
    bins, why = _reference_binaries()
    if bins is None:
        return _unavailable(why)
    try:
        import torch
        if not torch.cuda.is_available():
            return _unavailable("no CUDA device")
    except ImportError:
        return _unavailable("torch is needed to write the random model file")
    args.warmup = max(args.warmup, 3)
    layers = args.layers or model_sizes["num_hidden_layers"]
    sizes = dict(model_sizes, num_hidden_layers=layers)
    need_bytes = 2.2 * (layers * _layer_params(sizes) + 2 * sizes["vocab_size"] * sizes["hidden_size"]) + (1 << 30)
    base = None
    for cand in ("/dev/shm", tempfile.gettempdir()):
        try:
            if shutil.disk_usage(cand).free > need_bytes:
                base = cand
                break
        except OSError:
            continue
    if base is None:
        return _unavailable("no room for the reference's model file")
    work = Path(tempfile.mkdtemp(prefix="tllm_ref_", dir=base))
    pk = peaks()
    try:
        t0 = time.perf_counter()
        _write_reference_model(work, sizes)
        print(f"[bench] reference model written to {work} in {time.perf_counter() - t0:.1f} s", file=sys.stderr, flush=True)
        clocks = ClockSampler()
        clocks.start()
        windows = []
        vocab = sizes["vocab_size"]
        prompt_len = _standing_prompt_len(args.batch, args.steps, args.warmup)
        blocks = args.batch * (CONTEXT // PAGE) + 64
        cmd = [str(bins[0]), str(work / "model.safetensors"), str(work / "tokenizer.json"), str(args.batch),
               str(prompt_len), str(args.warmup), str(args.steps), str(CONTEXT), str(blocks), str(vocab - 1), "0"]
        w0 = time.perf_counter()
        res = subprocess.run(cmd, capture_output=True, text=True, timeout=1500)
        windows.append((w0, time.perf_counter(), "reference decode"))
        sys.stderr.write(res.stderr[-2000:])
        if res.returncode != 0:
            return _unavailable(f"the reference's decode run ended with {res.returncode}: "
                                + (res.stderr.strip().splitlines() or ["no message"])[-1][:200])
        dec = json.loads(res.stdout.strip().splitlines()[-1])
        print(f"[bench] reference decode: {dec}", file=sys.stderr, flush=True)

        points = {}
        for b in ([1, 8, 64] if args.ref_all else [args.batch]):
            cmd = [str(bins[1]), "--bench", "--tokenizer", str(work / "tokenizer.json"), "--model",
                   str(work / "model.safetensors"), "--device", "cuda", "--num-seqs", str(b), "--min-input-len", "128",
                   "--max-input-len", "128", "--min-output-len", "128", "--max-output-len", "128", "--warmup", "3",
                   "--repeats", "5", "--max-seq-len", str(CONTEXT), "--num-kv-blocks", str(b * (256 // PAGE) + 16),
                   "--max-token-id", str(vocab - 1), "--seed", "0"]
            w0 = time.perf_counter()
            res = subprocess.run(cmd, capture_output=True, text=True, timeout=1500)
            windows.append((w0, time.perf_counter(), f"reference 128/128 b{b}"))
            rates = [float(part.split("=")[1]) for line in res.stdout.splitlines() if line.startswith("run=")
                     for part in line.split() if part.startswith("output_tokens_per_second=")]
            if res.returncode != 0 or len(rates) != 5:
                print(f"[bench] reference model_main --bench b{b} ended with {res.returncode}: {res.stderr[-400:]}",
                      file=sys.stderr, flush=True)
                continue
            points[f"p128_e2e_b{b}"] = round(statistics.median(rates), 1)
            print(f"[bench] reference 128/128 b{b}: {points[f'p128_e2e_b{b}']} output tok/s (median of 5)",
                  file=sys.stderr, flush=True)
    finally:
        shutil.rmtree(work, ignore_errors=True)

    weight_bytes = 2 * (layers * _layer_params(sizes) + vocab * sizes["hidden_size"])
    kv_per_token = 2 * sizes["num_key_value_heads"] * sizes["head_dim"] * 2 * layers
    # request i has decoded about (batch - 1 - i) / batch of the prompt steps' tokens before the timed steps
    prefill_steps = dec.get("prefill_steps", 0)
    mean_ctx = prompt_len + prefill_steps / 2.0 + args.warmup + (args.steps + 1) / 2.0
    achieved = (weight_bytes + args.batch * mean_ctx * kv_per_token) / dec["seconds"] * args.steps / 1e9
    table_entries = CONTEXT // PAGE
    record = {
        "impl": "reference",
        "metric": f"decode tok/s @ batch {args.batch} ({model_name}, context 4096, 1 B200)",
        "value": round(dec["tokens_per_second"], 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": round(dec["ms_per_step"], 4), "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "fp16",
        "data": "synthetic (random weights N(0,0.02), uniform random token ids); the reference multiplies by the "
                "embedding matrix for the head whatever tie_word_embeddings says",
        "config": _config(model_name, args.batch, layers, model_sizes, sizes, mean_ctx, weight_bytes, pk),
        "e2e": {"value": round(dec["tokens_per_second"], 1), "unit": "tokens/s",
                "h2d_bytes_per_step": args.batch * (8 + 4 * table_entries + 20), "d2h_bytes_per_step": args.batch * 4},
        "gpu_launches": (17 * layers + 6) * args.steps,
        "prefill": None,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": points,
        "clocks": clocks.stop(windows),
    }
    print(json.dumps(record))
    return 0


def _layer_params(sizes: dict) -> int:
    q = sizes["num_attention_heads"] * sizes["head_dim"]
    kv = sizes["num_key_value_heads"] * sizes["head_dim"]
    h = sizes["hidden_size"]
    return (q + 2 * kv) * h + h * q + 3 * h * sizes["intermediate_size"]


def _config(model_name, batch, layers, model_sizes, sizes, mean_ctx, weight_bytes, pk) -> dict:
    """The ``config`` of the record, the same for both arms (flat, at most 20 keys)."""
    return {"model": model_name, "global_batch": batch, "seq_len": CONTEXT, "parallelism": "single GPU",
            "layers": layers, "layers_of_model": model_sizes["num_hidden_layers"],
            "hidden_size": sizes["hidden_size"], "intermediate_size": sizes["intermediate_size"],
            "q_heads": sizes["num_attention_heads"], "kv_heads": sizes["num_key_value_heads"],
            "head_dim": sizes["head_dim"], "vocab_size": sizes["vocab_size"], "page_size": PAGE,
            "decode_context": None if mean_ctx is None else round(mean_ctx, 1), "prefill_tokens": PREFILL_TOKENS,
            "p128": "128-token prompts, 128 outputs, temperature 0.6",
            "l2": f"inputs larger than L2 ({weight_bytes / 1e9:.1f} GB of weights per step)", "peaks": pk["source"]}


def precheck(model, cfg, sizes, device) -> dict:
    """The logits of the very model that is timed, by the bfloat16 kernels, against the float32 path
    of the same weights, on one request of 2,200 tokens and three short ones cut in four ways (whole;
    the last 32 tokens one by one, which are replayed CUDA graphs; portions of 2 to 700 tokens; mixed
    on a pool that just holds the four).  If the float32 twin of all layers does not fit beside the
    model, both are cut to the layers that do.

    Limits, as fractions of the standard deviation of a row of logits (0.9 to 1.6 at these sizes):
    a row's root-mean-square difference 0.12 and its largest difference among 151,936 entries 0.6,
    a little over twice what 36 layers of Qwen3-8B sizes show on a B200 (0.052 and 0.26; the
    difference grows with the square root of the depth: 4 layers show 0.026 and 0.13); the bfloat16
    argmax must be the float32 argmax or within 0.5 of it; the float32 ways of cutting must agree to
    1e-4 of a row's largest logit.  A kernel that loses a tile of keys, a slice of K or a page moves
    a row by its whole spread."""
    import torch

    from tiny_llm_infer_b200.cache import CacheManager
    from tiny_llm_infer_b200.config import Qwen3Config
    from tiny_llm_infer_b200.engine import ModelRunner, random_model, selfcheck

    layers = sizes["num_hidden_layers"]
    free, _ = torch.cuda.mem_get_info()
    per_layer, ends = 4 * _layer_params(sizes), 4 * 2 * sizes["vocab_size"] * sizes["hidden_size"]
    fit = int((free * 0.8 - ends - (8 << 30)) // (per_layer * 1.5))        # the twin, and the cut bfloat16 model if one is needed
    check_layers = layers if layers * per_layer + ends + (8 << 30) < free * 0.8 else max(1, min(layers, fit))
    gen = torch.Generator().manual_seed(7)
    requests = {str(i): torch.randint(0, cfg.vocab_size, (n,), generator=gen).tolist()
                for i, n in enumerate((2200, 300, 150, 90))}
    wanted = {k: selfcheck.wanted_positions(len(v)) for k, v in requests.items()}

    def ways(m, dtype):
        cache = CacheManager(m.cache_needs(), PAGE, selfcheck.pages_for(requests, PAGE), max_slots=4,
                             max_seq_len=2240, dtype=dtype, device=device)
        runner = ModelRunner(m, cache, max_batch_tokens=2240)
        rows = selfcheck.CutRunner(runner, requests, wanted).all_ways(seed=3)
        runner.check_kernels()
        cache.audit()
        return rows

    cut_cfg = Qwen3Config(layer_types=("full_attention",) * check_layers, **dict(sizes, num_hidden_layers=check_layers))
    exact_model = random_model(cut_cfg, seed=0, dtype=torch.float32, device=device, std=0.02)
    exact = ways(exact_model, torch.float32)
    del exact_model
    torch.cuda.empty_cache()
    fast_model = model if check_layers == layers else random_model(cut_cfg, seed=0, dtype=torch.bfloat16, device=device, std=0.02)
    fast = ways(fast_model, torch.bfloat16)
    del fast_model
    result = selfcheck.compare(fast, exact, near_tie=0.5)
    spread32 = max(selfcheck.spread_between_ways(exact).values())
    del exact, fast
    torch.cuda.empty_cache()
    names = ("whole", "tail", "portions", "mixed")
    out = {"layers": check_layers, "rows": len(wanted["0"]) + sum(len(wanted[k]) for k in "123"),
           "max_of_row_std": round(max(result[w + ":relative"] for w in names), 4),
           "rms_of_row_std": round(max(result[w + ":rms"] for w in names), 4),
           "argmax_misses": int(sum(result[w + ":argmax_misses"] for w in names)),
           "float32_ways_relative": float(f"{spread32:.2e}")}
    out["ok"] = bool(out["max_of_row_std"] <= 0.6 and out["rms_of_row_std"] <= 0.12 and out["argmax_misses"] == 0
                     and spread32 <= 1e-4)
    return out


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--model", default="8b", choices=sorted(MODELS),
                    help="the sizes: 8b is the benchmark configuration, 0.6b and 32b the other two the reference is quoted on")
    ap.add_argument("--layers", type=int, default=None,
                    help="fewer layers than the model has (named in the record) if memory or time needs it")
    ap.add_argument("--mixed", action="store_true",
                    help="the mixed run (64 requests, prompts of 16 to 1024 tokens, 256 outputs each at temperature "
                         "0.6, budget 2048, through LLM.generate) with the sizes of --model; at the default sizes it "
                         "runs anyway, with the Qwen3-0.6B sizes it belongs to")
    ap.add_argument("--skip-points", action="store_true",
                    help="leave out the batch 1 and 64 points, the 128-token workload and the 0.6B mixed run")
    ap.add_argument("--skip-check", action="store_true", help="leave out the logits check before the timed phases")
    ap.add_argument("--ref-all", action="store_true",
                    help="reference arm: its model_main --bench at batch 1, 8 and 64 instead of --batch alone")
    ap.add_argument("--only", default="all", choices=["all", "prefill", "decode", "e2e", "mixed", "p128"],
                    help="run one phase only (for profiling a small case); the record then lacks the others")
    args = ap.parse_args()
    model_name, model_sizes = MODELS[args.model]
    if args.layers is None:
        args.layers = model_sizes["num_hidden_layers"]
    if args.only == "mixed":
        args.mixed = True

    if args.impl == "reference":
        return reference_arm(args, model_name, model_sizes)
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} has nothing to measure")
        return 2
    args.warmup = max(args.warmup, 3)

    import torch

    from tiny_llm_infer_b200 import ops
    from tiny_llm_infer_b200.config import Qwen3Config
    from tiny_llm_infer_b200.engine import LLM, StepEntry, random_model
    from tiny_llm_infer_b200.sampling import SamplingParams

    assert torch.cuda.is_available(), "bench.py needs a CUDA device"
    device = "cuda:0"
    pk = peaks()
    sizes = dict(model_sizes, num_hidden_layers=args.layers)
    cfg = Qwen3Config(layer_types=("full_attention",) * args.layers, **sizes)
    ops.lib()
    t0 = time.perf_counter()
    model = random_model(cfg, seed=0, dtype=torch.bfloat16, device=device, std=0.02)
    torch.cuda.synchronize()
    print(f"[bench] model built in {time.perf_counter() - t0:.1f} s", file=sys.stderr, flush=True)

    max_batch = 64 if (not args.skip_points or args.mixed) else max(args.batch, 1)
    pages = max_batch * (CONTEXT // PAGE) + 2 * (PREFILL_TOKENS // PAGE) + 64
    llm = LLM(None, dtype="bfloat16", max_model_len=CONTEXT, num_kv_blocks=pages, block_size=PAGE,
              max_num_batched_tokens=PREFILL_TOKENS, max_num_seqs=max_batch, device=device, loaded=(model, cfg))
    runner, engine = llm.runner, llm.engine
    gen = torch.Generator().manual_seed(0)
    vocab = cfg.vocab_size

    def tokens(n):
        return torch.randint(0, vocab, (n,), generator=gen).tolist()

    # byte and flop counts
    layer_params = _layer_params(sizes)
    weight_bytes = 2 * (args.layers * layer_params + vocab * cfg.hidden_size)
    kv_bytes_per_token = 2 * cfg.kv_dim * 2 * args.layers
    windows = []
    clocks = ClockSampler()
    clocks.start()

    # ---------------------------------------------------------------- prefill of 2048 tokens
    def prefill_once():
        toks = tokens(PREFILL_TOKENS)
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        runner.step([StepEntry("prefill", toks, [PREFILL_TOKENS - 1])])
        end.record()
        torch.cuda.synchronize()
        runner.release("prefill")
        return start.elapsed_time(end)

    prefill = None
    if args.only in ("all", "prefill"):
        for _ in range(3):
            prefill_once()
        w0 = time.perf_counter()
        prefill_ms = statistics.median(prefill_once() for _ in range(5))
        windows.append((w0, time.perf_counter(), "prefill"))
        prefill_flops = 2.0 * PREFILL_TOKENS * args.layers * layer_params \
            + args.layers * 2.0 * PREFILL_TOKENS ** 2 * cfg.q_dim + 2.0 * vocab * cfg.hidden_size
        prefill = {"value": round(PREFILL_TOKENS / (prefill_ms / 1e3), 1), "tokens": PREFILL_TOKENS,
                   "ms": round(prefill_ms, 3),
                   "frac": round(prefill_flops / (prefill_ms / 1e3) / (pk["bf16_tflops"] * 1e12), 4)}
        if pk.get("bf16_tflops_sustained"):
            prefill["frac_sustained"] = round(prefill_flops / (prefill_ms / 1e3) / (pk["bf16_tflops_sustained"] * 1e12), 4)
        print(f"[bench] prefill {prefill}", file=sys.stderr, flush=True)

    # ---------------------------------------------------------------- decode, timed on the device
    def decode_device(batch, steps, warmup, end_context=CONTEXT, what="decode"):
        """Tokens per second of `steps` decode steps of `batch` requests that end at `end_context`."""
        start_len = end_context - (steps + warmup)
        names = [f"d{batch}_{i}" for i in range(batch)]
        for name in names:                                   # real prefill, in portions of 2048
            toks = tokens(start_len)
            for i in range(0, start_len, PREFILL_TOKENS):
                runner.step([StepEntry(name, toks[i:i + PREFILL_TOKENS], [])])
        params = torch.tensor([[0.6, 1.0]] * batch, device=device)
        seeds = torch.arange(batch, dtype=torch.int64, device=device)
        out = torch.empty(batch, dtype=torch.int32, device=device)
        nxt = [[int(t)] for t in torch.randint(0, vocab, (batch,), generator=gen)]
        times = []
        torch.cuda.synchronize()
        before = ops.launches
        w_start = None
        for it in range(warmup + steps):
            if it == warmup:
                torch.cuda.synchronize()
                before = ops.launches
                w_start = time.perf_counter()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record()
            logits = runner.step([StepEntry(n, t, [0]) for n, t in zip(names, nxt)])
            ops.sample(logits, params, seeds, out, any_nucleus=False)
            end.record()
            nxt = [[t] for t in out.cpu().tolist()]          # the next step feeds what was sampled
            if it >= warmup:
                times.append((start, end))
        torch.cuda.synchronize()
        windows.append((w_start, time.perf_counter(), f"{what} b{batch}"))
        launches = ops.launches - before
        ms = sum(a.elapsed_time(b) for a, b in times) / steps
        for name in names:
            runner.release(name)
        mean_ctx = start_len + warmup + (steps - 1) / 2.0 + 1
        return batch / (ms / 1e3), ms, launches, mean_ctx

    def hbm_fraction(batch, ms, ctx):
        return (weight_bytes + batch * ctx * kv_bytes_per_token) / (ms / 1e3) / 1e9

    value = ms_per_step = launches = mean_ctx = roofline = None
    if args.only in ("all", "decode"):
        value, ms_per_step, launches, mean_ctx = decode_device(args.batch, args.steps, args.warmup)
        achieved = hbm_fraction(args.batch, ms_per_step, mean_ctx)
        roofline = {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s",
                    "frac": round(achieved / pk["hbm_gbs"], 4)}
        print(f"[bench] decode b{args.batch}: {value:.1f} tok/s, {ms_per_step:.3f} ms/step, {roofline}",
              file=sys.stderr, flush=True)

    # ---------------------------------------------------------------- the same through the entry point
    def decode_e2e(batch, steps, warmup):
        # requests whose prompts are done decode while the others' prompts are still computed:
        # leave them room for those steps too, so that all are still running when timing ends
        extra = batch * -(-CONTEXT // PREFILL_TOKENS) + 2
        sp = SamplingParams(max_tokens=steps + warmup + extra, temperature=0.6, ignore_eos=True)
        start_len = CONTEXT - sp.max_tokens - 1
        for i in range(batch):
            engine.add_request(tokens(start_len), SamplingParams(**{**sp.__dict__, "seed": i + 1}))
        while engine.scheduler.waiting:                      # prompts, outside the timed region
            engine.step()
        for _ in range(warmup):
            engine.step()
        torch.cuda.synchronize()
        t_start = time.perf_counter()
        for _ in range(steps):
            engine.step()
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - t_start
        windows.append((t_start, t_start + elapsed, f"e2e b{batch}"))
        while not engine.is_finished():
            engine.step()
        bucket = 1
        while bucket < batch:
            bucket *= 2
        # rows' ids/positions/slots/wanted, where the tokens sampled by the step before go, sampling params, keys
        h2d = (4 * bucket + 2 * batch) * 4 + batch * 8 + batch * 8
        return batch * steps / elapsed, h2d, batch * 4

    e2e = None
    if args.only in ("all", "e2e"):
        e2e_value, h2d, d2h = decode_e2e(args.batch, args.steps, args.warmup)
        e2e = {"value": round(e2e_value, 1), "unit": "tokens/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h}
        print(f"[bench] e2e b{args.batch}: {e2e_value:.1f} tok/s", file=sys.stderr, flush=True)

    points = {}
    if not args.skip_points and args.only == "all":
        for b in (1, 64):
            v, ms_b, _, ctx_b = decode_device(b, min(args.steps, 32), args.warmup)
            points[f"decode_b{b}"] = round(v, 1)
            bw = hbm_fraction(b, ms_b, ctx_b)
            points[f"decode_b{b}_hbm_frac"] = round(bw / pk["hbm_gbs"], 4)
            print(f"[bench] decode b{b}: {v:.1f} tok/s, {ms_b:.3f} ms/step, {bw:.0f} GB/s", file=sys.stderr, flush=True)

    # ---------------------------------------------------------------- 128-token prompts, 128 outputs
    # The reference's own benchmark (benchmark/run_benchmark.sh:32-42, model/model_main.cpp:150-175,
    # 354-368): `batch` prompts of 128 uniform token ids, 128 outputs each at temperature 0.6 with
    # end-of-sequence ignored, output tokens / wall time from the first add_request to the last result,
    # prompts included; three warm-up runs, then the median of five.  Beside it the decode steps of the
    # same workload alone (contexts 128 to 256), timed on the device, with their share of the HBM peak.
    def p128_e2e(batch):
        rates = []
        for run in range(8):
            prompts = [tokens(128) for _ in range(batch)]
            params = [SamplingParams(max_tokens=128, temperature=0.6, ignore_eos=True, seed=1000 * run + i + 1)
                      for i in range(batch)]
            torch.cuda.synchronize()
            t_start = time.perf_counter()
            outs = llm.generate(prompts, params)
            elapsed = time.perf_counter() - t_start
            assert sum(len(o.token_ids) for o in outs) == 128 * batch
            if run >= 3:
                rates.append(128 * batch / elapsed)
                windows.append((t_start, t_start + elapsed, f"128/128 e2e b{batch}"))
        return statistics.median(rates)

    if (not args.skip_points and args.only == "all") or args.only == "p128":
        for b in (1, 8, 64):
            v, ms_b, _, ctx_b = decode_device(b, 120, 8, end_context=256, what="128/128 decode")
            points[f"p128_decode_b{b}"] = round(v, 1)
            points[f"p128_hbm_frac_b{b}"] = round(hbm_fraction(b, ms_b, ctx_b) / pk["hbm_gbs"], 4)
            points[f"p128_e2e_b{b}"] = round(p128_e2e(b), 1)
            print(f"[bench] 128/128 b{b}: decode steps {v:.1f} tok/s ({ms_b:.3f} ms/step, {points[f'p128_hbm_frac_b{b}']} of HBM), "
                  f"end to end {points[f'p128_e2e_b{b}']} output tok/s", file=sys.stderr, flush=True)

    # ---------------------------------------------------------------- the logits of the model that was timed
    # (after the timed phases: seconds of float32 products before them leave the GPU at lower clocks
    # under its power cap; a mismatch fails the run all the same, and no record is printed)
    check = None
    if not args.skip_check and args.only == "all":
        t0 = time.perf_counter()
        check = precheck(model, cfg, sizes, device)
        print(f"[bench] logits check in {time.perf_counter() - t0:.1f} s: {check}", file=sys.stderr, flush=True)
        if not check["ok"]:
            clocks.stop(windows)
            print(json.dumps({"error": "the bfloat16 kernels' logits do not match the float32 path", "check": check}))
            return 1

    # ---------------------------------------------------------------- the mixed run
    def mixed_run(the_llm, the_vocab):
        g2 = torch.Generator().manual_seed(1)

        def workload():
            lens = torch.randint(16, 1025, (64,), generator=g2).tolist()
            return ([torch.randint(0, the_vocab, (n,), generator=g2).tolist() for n in lens],
                    [SamplingParams(max_tokens=256, temperature=0.6, ignore_eos=True, seed=i + 1) for i in range(64)])
        the_llm.generate(*workload())                               # first run: graphs are captured
        prompts, params = workload()
        torch.cuda.synchronize()
        t_start = time.perf_counter()
        outs = the_llm.generate(prompts, params)
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - t_start
        windows.append((t_start, t_start + elapsed, "mixed run"))
        made = sum(len(o.token_ids) for o in outs)
        return {"value": round(made / elapsed, 1), "unit": "generated tokens/s", "requests": 64,
                "prompt_tokens": sum(map(len, prompts)), "generated_tokens": made, "seconds": round(elapsed, 3)}

    mixed = None
    if args.mixed:
        mixed = dict(mixed_run(llm, vocab), model=model_name)
    elif args.model == "8b" and not args.skip_points and args.only == "all":
        # the mixed continuous-batching run belongs to the Qwen3-0.6B sizes: a second, small model
        del llm, runner, engine, model
        torch.cuda.empty_cache()
        name06, sizes06 = MODELS["0.6b"]
        cfg06 = Qwen3Config(layer_types=("full_attention",) * sizes06["num_hidden_layers"], **sizes06)
        model06 = random_model(cfg06, seed=0, dtype=torch.bfloat16, device=device, std=0.02)
        llm06 = LLM(None, dtype="bfloat16", max_model_len=CONTEXT, num_kv_blocks=64 * (1280 // PAGE) + 64, block_size=PAGE,
                    max_num_batched_tokens=PREFILL_TOKENS, max_num_seqs=64, device=device, loaded=(model06, cfg06))
        mixed = dict(mixed_run(llm06, cfg06.vocab_size), model=name06)
    if mixed is not None:
        points["mixed_run_tokens_per_s"] = mixed["value"]
        print(f"[bench] mixed run: {mixed}", file=sys.stderr, flush=True)

    record = {
        "metric": f"decode tok/s @ batch {args.batch} ({model_name}, context 4096, 1 B200)",
        "value": None if value is None else round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": None if ms_per_step is None else round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights N(0,0.02), uniform random token ids)",
        "config": _config(model_name, args.batch, args.layers, model_sizes, sizes, mean_ctx, weight_bytes, pk),
        "e2e": e2e,
        "gpu_launches": launches,
        "prefill": prefill, "roofline": roofline, "points": points, "mixed": mixed, "check": check,
        "clocks": clocks.stop(windows),
    }
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    sys.exit(main())
