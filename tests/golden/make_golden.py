"""Makes the golden outputs of this folder from the reference's own code.

The reference (xu797/tiny-llm-infer, C++/CUDA, no Python) cannot be imported, but its CPU
code path compiles here with two small stand-in headers (glog and armadillo are not
installed; ``harness/shim``), its CUDA files compiled only so that the link succeeds, and
the three armadillo-based legacy kernels stubbed (they are not on the Qwen3 path).  This
script builds it under ``--work``, writes the tiny model A of the tests (seed 0) with the
package's random-weights mode, and records

* ``tiny_a_logits.npy``: logits of ``forward_paged_batch`` on the CPU for one whole prompt
  of 33 tokens through a scrambled page table (the reference stores every tensor in FP16);
* ``tiny_a_engine.json``: greedy token ids and step counts of the reference's ``LLMEngine``
  for prompts of 5/17/33 tokens under token budgets 256 and 8 and pools of 8, 5 and 4 pages.

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

CPU_SOURCES = """utils/src/status.cpp utils/src/unicode.cpp utils/src/unicode-data.cpp
memory/src/*.cpp tensor/src/tensor.cpp
kernels/src/add_kernel_cpu.cpp kernels/src/embed_kernel_cpu.cpp kernels/src/matmul_kernel_cpu.cpp
kernels/src/paged_attention_cpu.cpp kernels/src/rmsnorm_kernel_cpu.cpp kernels/src/rope_kernel_cpu.cpp
kernels/src/swiglu_kernel_cpu.cpp kernels/src/kernels_interface.cpp
layers/src/*.cpp model/src/*.cpp engine/src/*.cpp""".split()


def sh(cmd, **kw):
    print("+", " ".join(str(c) for c in cmd), flush=True)
    subprocess.run([str(c) for c in cmd], check=True, **kw)


def build(ref: Path, work: Path):
    import site
    json_inc = None
    for sp in site.getsitepackages():
        cand = Path(sp) / "include" / "cudnn_frontend" / "thirdparty"
        if (cand / "nlohmann" / "json.hpp").is_file():
            json_inc = cand
    assert json_inc, "nlohmann/json.hpp not found"
    obj = work / "obj"
    obj.mkdir(parents=True, exist_ok=True)
    incs = []
    for d in ("utils", "memory", "tensor", "kernels", "layers", "model", "engine"):
        incs += ["-I", ref / d / "include"]
    incs += ["-I", ref, "-I", HERE / "harness" / "shim", "-I", json_inc, "-I", "/usr/local/cuda/include"]
    common = ["-std=c++17", "-O2", "-fopenmp", "-include", HERE / "harness" / "shim" / "armadillo", "-w"]
    objects = []
    sources = []
    for pat in CPU_SOURCES:
        sources += sorted(ref.glob(pat))
    sources += [HERE / "harness" / "stubs.cpp"]
    procs = []
    for src in sources:
        o = obj / (src.parent.parent.name + "_" + src.stem + ".o")
        objects.append(o)
        if not o.is_file():
            procs.append(subprocess.Popen([str(c) for c in ["g++", *common, *incs, "-c", src, "-o", o]]))
    for cu in sorted((ref / "kernels" / "src").glob("*.cu")) + sorted((ref / "utils" / "src").glob("*.cu")):
        o = obj / (cu.stem + "_cu.o")
        objects.append(o)
        if not o.is_file():
            procs.append(subprocess.Popen([str(c) for c in [
                "nvcc", "-arch=sm_100", "-std=c++17", "-O1", "-w", "-Xcompiler", "-fopenmp",
                "-include", HERE / "harness" / "shim" / "armadillo", *incs, "-c", cu, "-o", o]]))
    for p in procs:
        assert p.wait() == 0, "compilation of the reference failed"
    for name in ("logits_main", "engine_main"):
        sh(["g++", *common, *incs, HERE / "harness" / f"{name}.cpp", *objects, "-o", work / name,
            "-L/usr/local/cuda/lib64", "-lcudart", "-lcublas", "-lcurand", "-lgomp"])


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True)
    ap.add_argument("--work", required=True)
    args = ap.parse_args()
    ref, work = Path(args.reference), Path(args.work)
    build(ref, work)

    from tiny import TINY_A, make_folder, prompt
    folder = make_folder(TINY_A, work / "tinyA")
    raw = json.loads((folder / "config.json").read_text())
    vocab = raw["vocab_size"]
    # the reference detokenises finished requests: its tokenizer must know every id
    (folder / "tokenizer.json").write_text(json.dumps(
        {"model": {"vocab": {f"t{i}": i for i in range(vocab)}, "merges": []}, "added_tokens": []}))
    ids = prompt(2, 33, vocab)
    out = work / "logits.bin"
    sh([work / "logits_main", folder, out, 16, 8, *ids])
    logits = np.fromfile(out, dtype=np.float32).reshape(len(ids), vocab)
    np.save(HERE / "tiny_a_logits.npy", logits.astype(np.float32))
    prompts = [prompt(i, n, vocab) for i, n in enumerate((5, 17, 33))]
    runs = []
    for budget, pages in ((256, 8), (8, 8), (8, 5), (8, 4)):
        res = subprocess.run([str(work / "engine_main"), str(folder), str(budget), str(pages), "8",
                              *[",".join(map(str, p)) for p in prompts]], check=True, capture_output=True, text=True)
        tokens, steps = {}, None
        for line in res.stdout.splitlines():
            parts = line.split()
            if parts[:1] == ["req"]:
                tokens[int(parts[1])] = [int(x) for x in parts[2:]]
            elif parts[:1] == ["steps"]:
                steps = int(parts[1])
        runs.append({"budget": budget, "pages": pages, "steps": steps,
                     "tokens": [tokens[i + 1] for i in range(len(prompts))]})
    (HERE / "tiny_a_engine.json").write_text(json.dumps(
        {"model": "tests/tiny.py TINY_A, seed 0, weights stored in bfloat16", "logits_prompt": ids,
         "page_size": 16, "prompts": prompts, "max_tokens": 8, "runs": runs}, indent=1))
    print("wrote", HERE / "tiny_a_logits.npy", "and", HERE / "tiny_a_engine.json")


if __name__ == "__main__":
    main()
