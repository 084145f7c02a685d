"""Makes the golden outputs of this folder from the reference's own code.

The reference (xu797/tiny-llm-infer, C++/CUDA, no Python) cannot be imported, but its CPU
code path compiles here with two small stand-in headers (glog and armadillo are not
installed; ``baseline/reference_arm/shim``), its CUDA files compiled only so that the link
succeeds, and the three armadillo-based legacy kernels stubbed (they are not on the Qwen3
path).  This script builds it under ``--work``, writes tiny models of the tests with the
package's random-weights mode, and records

* ``tiny_a_logits.npy``: logits of ``forward_paged_batch`` on the CPU for one whole prompt
  of 33 tokens through a scrambled page table (the reference stores every tensor in FP16);
* ``tiny_a_engine.json``: greedy token ids and step counts of the reference's ``LLMEngine``
  for prompts of 5/17/33 tokens under token budgets 256 and 8 and pools of 8, 5 and 4 pages;
* ``tiny_b_tied_logits.npy``, ``tiny_b_tied_engine.json``: the same for tiny B with its head tied
  to the embedding (the reference has no other head): a prompt of 70 tokens through scrambled
  pages of 8, and prompts of 1/9/40/70 tokens with 12 greedy tokens each under a budget of 32 with
  pools of 32 and 14 pages, and under a budget of 256.

    python tests/golden/make_golden.py --reference /path/to/tiny-llm-infer --work /tmp/golden_build

``tests/test_plain.py`` compares the plain implementation with these files.
"""
import argparse
import json
import subprocess
import sys
from pathlib import Path

import numpy as np

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

sys.path.insert(0, str(ROOT / "baseline" / "reference_arm"))


def sh(cmd, **kw):
    print("+", " ".join(str(c) for c in cmd), flush=True)
    subprocess.run([str(c) for c in cmd], check=True, **kw)


def build(ref: Path, work: Path):
    """The reference's objects as the benchmark's reference arm builds them
    (baseline/reference_arm/build.py), linked with the two small mains of ``harness/``."""
    import build as reference_build
    cxx, objects, link = reference_build.compile_reference(ref, work)
    for name in ("logits_main", "engine_main"):
        sh([*cxx, HERE / "harness" / f"{name}.cpp", *objects, "-o", work / name, *link])


def golden_case(work: Path, tag: str, tiny: dict, page: int, max_len: int, logits_len: int, logits_pages: int,
                prompt_lens, max_tokens: int, settings):
    """Logits of one prompt through a scrambled page table, and the reference engine's greedy tokens
    and step counts for ``prompt_lens`` under each (token budget, pages) of ``settings``."""
    from tiny import make_folder, prompt
    folder = make_folder(tiny, work / f"tiny{tag}")
    raw = json.loads((folder / "config.json").read_text())
    vocab = raw["vocab_size"]
    # the reference detokenises finished requests: its tokenizer must know every id
    (folder / "tokenizer.json").write_text(json.dumps(
        {"model": {"vocab": {f"t{i}": i for i in range(vocab)}, "merges": []}, "added_tokens": []}))
    ids = prompt(2, logits_len, vocab)
    out = work / f"logits_{tag}.bin"
    sh([work / "logits_main", folder, out, page, logits_pages, max_len, *ids])
    logits = np.fromfile(out, dtype=np.float32).reshape(len(ids), vocab)
    np.save(HERE / f"tiny_{tag}_logits.npy", logits.astype(np.float32))
    prompts = [prompt(i, n, vocab) for i, n in enumerate(prompt_lens)]
    runs = []
    for budget, pages in settings:
        res = subprocess.run([str(work / "engine_main"), str(folder), str(budget), str(pages), str(max_tokens),
                              str(page), str(max_len), *[",".join(map(str, p)) for p in prompts]],
                             check=True, capture_output=True, text=True)
        tokens, steps = {}, None
        for line in res.stdout.splitlines():
            parts = line.split()
            if parts[:1] == ["req"]:
                tokens[int(parts[1])] = [int(x) for x in parts[2:]]
            elif parts[:1] == ["steps"]:
                steps = int(parts[1])
        runs.append({"budget": budget, "pages": pages, "steps": steps,
                     "tokens": [tokens[i + 1] for i in range(len(prompts))]})
    return {"logits_prompt": ids, "page_size": page, "max_model_len": max_len, "prompts": prompts,
            "max_tokens": max_tokens, "runs": runs}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--work", required=True)
    args = ap.parse_args()
    ref, work = Path(args.reference), Path(args.work)
    work.mkdir(parents=True, exist_ok=True)
    build(ref, work)

    import dataclasses

    from tiny import TINY_A, TINY_B
    a = golden_case(work, "a", TINY_A, page=16, max_len=128, logits_len=33, logits_pages=8,
                    prompt_lens=(5, 17, 33), max_tokens=8, settings=((256, 8), (8, 8), (8, 5), (8, 4)))
    (HERE / "tiny_a_engine.json").write_text(json.dumps(
        dict(a, model="tests/tiny.py TINY_A, seed 0, weights stored in bfloat16"), indent=1))
    # tiny B with the head tied to the embedding, the only kind of head the reference has
    # (model/src/qwen3_layers.cpp:246-265): group ratio 3, head width 32, q width != hidden,
    # feed-forward width 200, eps 1e-5, theta 1e6, pages of 8; prompts of 1/9/40/70 tokens under a token
    # budget of 32 with a pool that holds everything and one that does not
    b_tied = dict(TINY_B, cfg=dataclasses.replace(TINY_B["cfg"], tie_word_embeddings=True))
    b = golden_case(work, "b_tied", b_tied, page=8, max_len=256, logits_len=70, logits_pages=12,
                    prompt_lens=(1, 9, 40, 70), max_tokens=12, settings=((32, 32), (32, 14), (256, 32)))
    (HERE / "tiny_b_tied_engine.json").write_text(json.dumps(
        dict(b, model="tests/tiny.py TINY_B with tie_word_embeddings, seed 1, weights stored in bfloat16"), indent=1))
    print("wrote the golden files of tiny A and tiny B (tied) into", HERE)


if __name__ == "__main__":
    main()
