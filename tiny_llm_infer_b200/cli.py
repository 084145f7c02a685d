"""Command line in the manner of the reference's ``model_main`` (model/model_main.cpp):

    model_main --infer --model P (--prompt-ids 1,2,3 | --prompt TEXT --tokenizer F) ...
    model_main --bench --model P [--num-seqs 8 --min-input-len 64 ...]

Options keep the reference's names, meanings and defaults (model/model_main.cpp:41-60,
465-559): ``--max-new-tokens`` 64, ``--max-seq-len`` 2048 (256 for ``--bench``),
``--num-kv-blocks`` 0 (sized from free memory), ``--gpu-memory-utilization`` 0.9 (0.7 for
``--bench``); the engine runs with up to min(16, prompts) requests (``--bench``: ``--num-seqs``,
model/model_main.cpp:276-279), a token budget of min(max-seq-len, 256) and pages of 16 tokens
(model/model_main.cpp:403-408).  ``--infer``
is greedy unless ``--temperature`` is given.  ``--bench`` makes seeded synthetic requests
as the reference does (:150-175): lengths uniform in the ranges, ids uniform in
[0, min(max-token-id, vocab-1)], temperature 0.6, EOS ignored, request seed
``seed + index + 1``; warm-up runs use seeds ``seed+1..``, measured runs ``seed+1000+i``;
it prints the same ``run=... output_tokens_per_second=...`` lines.

Added here: ``--prompt-ids`` (requests are token ids; text needs ``--tokenizer``),
``--dtype bfloat16|float32``, ``--temperature``, ``--top-p``, ``--seed`` for ``--infer``,
``--random-weights SEED --config FILE`` (write a random model folder first).  There is no
``--device cpu`` and no ``--quantization``.
"""
from __future__ import annotations

import argparse
import json
import random
import sys
import time
from pathlib import Path
from typing import List


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="model_main", description="Qwen3 inference on one B200")
    mode = ap.add_mutually_exclusive_group(required=True)
    mode.add_argument("--infer", action="store_true", help="generate for each prompt")
    mode.add_argument("--bench", action="store_true", help="throughput of synthetic requests")
    mode.add_argument("--write-random-model", metavar="DIR", help="write a random model folder and exit")
    ap.add_argument("--model", help="model folder, or a .safetensors file with config.json beside it")
    ap.add_argument("--tokenizer", help="tokenizer.json (only for text prompts)")
    ap.add_argument("--prompt", action="append", default=[], help="text prompt (repeatable)")
    ap.add_argument("--prompt-ids", action="append", default=[], help="prompt as comma-separated token ids (repeatable)")
    ap.add_argument("--device", default="cuda", help="cuda or cuda:N")
    ap.add_argument("--dtype", default="bfloat16", choices=["bfloat16", "float32"])
    ap.add_argument("--max-new-tokens", type=int, default=64)
    ap.add_argument("--max-seq-len", type=int, default=None)
    ap.add_argument("--num-kv-blocks", type=int, default=0)
    ap.add_argument("--gpu-memory-utilization", type=float, default=None)
    ap.add_argument("--temperature", type=float, default=0.0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-prefix-caching", action="store_true",
                    help="compute every prompt in full (the reference always shares hashed pages)")
    ap.add_argument("--prompt-graphs", action="store_true",
                    help="replay prompt steps whose layout repeats as CUDA graphs too")
    ap.add_argument("--no-overlap-scheduling", action="store_true",
                    help="schedule a step only after the one before it has finished on the GPU")
    ap.add_argument("--num-seqs", type=int, default=8)
    ap.add_argument("--min-input-len", type=int, default=64)
    ap.add_argument("--max-input-len", type=int, default=128)
    ap.add_argument("--min-output-len", type=int, default=32)
    ap.add_argument("--max-output-len", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=1)
    ap.add_argument("--repeats", type=int, default=3)
    ap.add_argument("--max-token-id", type=int, default=10000)
    ap.add_argument("--manifest-prefix", default="")
    ap.add_argument("--config", help="config.json for --write-random-model")
    ap.add_argument("--random-weights", type=int, metavar="SEED", default=0)
    ap.add_argument("--weight-std", type=float, default=0.02)
    return ap


def make_benchmark_requests(args, seed_value: int, vocab: int):
    """Seeded synthetic requests (reference: model/model_main.cpp:150-175; the generator
    differs, the distributions are the same)."""
    from .sampling import SamplingParams
    rng = random.Random(seed_value)
    hi = min(args.max_token_id, vocab - 1)
    out = []
    for index in range(args.num_seqs):
        n = rng.randint(args.min_input_len, args.max_input_len)
        prompt = [rng.randint(0, hi) for _ in range(n)]
        params = SamplingParams(max_tokens=rng.randint(args.min_output_len, args.max_output_len),
                                temperature=0.6, ignore_eos=True, seed=seed_value + index + 1)
        out.append((prompt, params))
    return out


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.write_random_model:
        from . import models  # noqa: F401
        from .config import config_from_dict
        from .weights import write_random_model
        if not args.config:
            print("--write-random-model needs --config FILE", file=sys.stderr)
            return 2
        cfg = config_from_dict(json.loads(Path(args.config).read_text()))
        write_random_model(args.write_random_model, cfg, args.random_weights, args.weight_std)
        print(args.write_random_model)
        return 0
    if not args.model:
        print("--model is required", file=sys.stderr)
        return 2
    device = "cuda:0" if args.device == "cuda" else args.device
    from .engine import LLM
    from .sampling import SamplingParams

    if args.infer:
        prompts: List = [[int(x) for x in p.split(",") if x.strip()] for p in args.prompt_ids] + list(args.prompt)
        if not prompts:
            print("--infer needs --prompt-ids or --prompt", file=sys.stderr)
            return 2
        if args.prompt and not args.tokenizer:
            print("text prompts need --tokenizer", file=sys.stderr)
            return 2
        if args.max_new_tokens == 0:                   # model/model_main.cpp:396-400
            for _ in prompts:
                print()
            return 0
        max_seq_len = args.max_seq_len or 2048
        llm = LLM(args.model, dtype=args.dtype, max_model_len=max_seq_len, num_kv_blocks=args.num_kv_blocks,
                  block_size=16, max_num_batched_tokens=min(max_seq_len, 256),
                  max_num_seqs=min(16, len(prompts)),
                  gpu_memory_utilization=args.gpu_memory_utilization or 0.9, device=device,
                  tokenizer=args.tokenizer, enable_prefix_caching=not args.no_prefix_caching,
                  overlap_scheduling=not args.no_overlap_scheduling, prompt_graphs=args.prompt_graphs)
        params = SamplingParams(max_tokens=args.max_new_tokens, temperature=args.temperature,
                                top_p=args.top_p, seed=args.seed)
        for result in llm.generate(prompts, params):
            print(result.text if llm.tokenizer else ",".join(str(t) for t in result.token_ids))
        return 0

    # --bench
    max_seq_len = args.max_seq_len or 256
    if min(args.num_seqs, args.min_input_len, args.min_output_len, args.repeats) <= 0 or args.warmup < 0 \
            or args.min_input_len > args.max_input_len or args.min_output_len > args.max_output_len \
            or args.max_token_id < 0:
        print("--bench needs positive counts and ranges with min <= max", file=sys.stderr)      # model/model_main.cpp:130-146
        return 2
    if args.max_input_len + args.max_output_len > max_seq_len + 1:
        print("--max-input-len + --max-output-len exceed --max-seq-len", file=sys.stderr)
        return 2
    llm = LLM(args.model, dtype=args.dtype, max_model_len=max_seq_len, num_kv_blocks=args.num_kv_blocks,
              block_size=16, max_num_batched_tokens=min(max_seq_len, 256), max_num_seqs=args.num_seqs,
              gpu_memory_utilization=args.gpu_memory_utilization or 0.7, device=device,
              enable_prefix_caching=not args.no_prefix_caching,
              overlap_scheduling=not args.no_overlap_scheduling, prompt_graphs=args.prompt_graphs)
    vocab = llm.runner.vocab
    import torch

    def wait():
        if device.startswith("cuda"):
            torch.cuda.synchronize()

    def run(requests) -> int:
        outs = llm.engine.generate([p for p, _ in requests], [s for _, s in requests])
        want = sum(s.max_tokens for _, s in requests)
        got = sum(len(o.token_ids) for o in outs)
        if got != want:
            raise RuntimeError(f"benchmark produced {got} tokens, expected {want}")
        return got

    for index in range(args.warmup):
        run(make_benchmark_requests(args, args.seed + index + 1, vocab))
        print(f"Warmup {index + 1} complete.", file=sys.stderr)
    total_tokens, total_elapsed = 0, 0.0
    for index in range(args.repeats):
        requests = make_benchmark_requests(args, args.seed + 1000 + index, vocab)
        if args.manifest_prefix:
            manifest = {"requests": [dict(prompt_token_ids=p, max_tokens=s.max_tokens, temperature=s.temperature,
                                          top_p=s.top_p, ignore_eos=s.ignore_eos, seed=s.seed) for p, s in requests]}
            Path(f"{args.manifest_prefix}_run{index + 1}.json").write_text(json.dumps(manifest, indent=2) + "\n")
        wait()
        started = time.perf_counter()
        tokens = run(requests)
        wait()
        elapsed = time.perf_counter() - started
        total_tokens += tokens
        total_elapsed += elapsed
        print(f"run={index + 1} requests={args.num_seqs} output_tokens={tokens} elapsed_seconds={elapsed:.6f} "
              f"output_tokens_per_second={tokens / elapsed:.2f}")
    print(f"aggregate_runs={args.repeats} output_tokens={total_tokens} elapsed_seconds={total_elapsed:.6f} "
          f"output_tokens_per_second={total_tokens / max(total_elapsed, 1e-9):.2f}")
    return 0


if __name__ == "__main__":
    sys.exit(main())
