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
                    help="also the mixed run that goes with the 0.6B sizes: 64 requests, prompts of 16 to "
                         "1024 tokens, 256 outputs each at temperature 0.6, budget 2048, through LLM.generate")
    ap.add_argument("--skip-points", action="store_true", help="leave out the batch 1 and 64 points")
    ap.add_argument("--only", default="all", choices=["all", "prefill", "decode", "e2e", "mixed"],
                    help="run one phase only (for profiling a small case); the record then lacks the others")
    args = ap.parse_args()
    model_name, model_sizes = MODELS[args.model]
    if args.layers is None:
        args.layers = model_sizes["num_hidden_layers"]
    if args.only == "mixed":
        args.mixed = True

    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable":
                          "xu797/tiny-llm-infer is a CMake C++/CUDA project without setup.py or pyproject.toml: "
                          "pip reports 'not installable'; it needs glog and armadillo, which are not in the image"}))
        return 0
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
    layer_params = (cfg.q_dim + 2 * cfg.kv_dim) * cfg.hidden_size + cfg.hidden_size * cfg.q_dim \
        + 3 * cfg.hidden_size * cfg.intermediate_size
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
    def decode_device(batch, steps, warmup):
        """Tokens per second of `steps` decode steps of `batch` requests that end at CONTEXT."""
        start_len = CONTEXT - (steps + warmup)
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
        windows.append((w_start, time.perf_counter(), f"decode b{batch}"))
        launches = ops.launches - before
        ms = sum(a.elapsed_time(b) for a, b in times) / steps
        for name in names:
            runner.release(name)
        mean_ctx = start_len + warmup + (steps - 1) / 2.0 + 1
        return batch / (ms / 1e3), ms, launches, mean_ctx

    value = ms_per_step = launches = mean_ctx = roofline = None
    if args.only in ("all", "decode"):
        value, ms_per_step, launches, mean_ctx = decode_device(args.batch, args.steps, args.warmup)
        step_bytes = weight_bytes + args.batch * mean_ctx * kv_bytes_per_token
        achieved = step_bytes / (ms_per_step / 1e3) / 1e9
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
            bw = (weight_bytes + b * ctx_b * kv_bytes_per_token) / (ms_b / 1e3) / 1e9
            print(f"[bench] decode b{b}: {v:.1f} tok/s, {ms_b:.3f} ms/step, {bw:.0f} GB/s", file=sys.stderr, flush=True)

    mixed = None
    if args.mixed:
        g2 = torch.Generator().manual_seed(1)

        def workload():
            lens = torch.randint(16, 1025, (64,), generator=g2).tolist()
            return ([torch.randint(0, vocab, (n,), generator=g2).tolist() for n in lens],
                    [SamplingParams(max_tokens=256, temperature=0.6, ignore_eos=True, seed=i + 1) for i in range(64)])
        llm.generate(*workload())                               # first run: graphs are captured
        prompts, params = workload()
        torch.cuda.synchronize()
        t_start = time.perf_counter()
        outs = llm.generate(prompts, params)
        torch.cuda.synchronize()
        elapsed = time.perf_counter() - t_start
        windows.append((t_start, t_start + elapsed, "mixed run"))
        made = sum(len(o.token_ids) for o in outs)
        mixed = {"value": round(made / elapsed, 1), "unit": "generated tokens/s", "requests": 64,
                 "prompt_tokens": sum(map(len, prompts)), "generated_tokens": made, "seconds": round(elapsed, 3)}
        print(f"[bench] mixed run: {mixed}", file=sys.stderr, flush=True)

    record = {
        "metric": f"decode tok/s @ batch {args.batch} ({model_name}, context 4096, 1 B200)",
        "value": None if value is None else round(value, 1), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": None if ms_per_step is None else round(ms_per_step, 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic (random weights N(0,0.02), uniform random token ids)",
        "config": {"model": model_name, "global_batch": args.batch, "seq_len": CONTEXT,
                   "parallelism": "single GPU", "layers": args.layers, "layers_of_model": model_sizes["num_hidden_layers"],
                   "hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size,
                   "q_heads": cfg.num_attention_heads, "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim,
                   "vocab_size": vocab, "page_size": PAGE, "decode_context": None if mean_ctx is None else round(mean_ctx, 1),
                   "prefill_tokens": PREFILL_TOKENS, "l2": f"inputs larger than L2 ({weight_bytes / 1e9:.1f} GB of weights per step)",
                   "peaks": pk["source"]},
        "e2e": e2e,
        "gpu_launches": launches,
        "prefill": prefill, "roofline": roofline, "points": points, "mixed": mixed,
        "clocks": clocks.stop(windows),
    }
    print(json.dumps(record))
    return 0


if __name__ == "__main__":
    sys.exit(main())
