#!/usr/bin/env python3
"""Builds the reference (xu797/tiny-llm-infer, a CMake C++/CUDA project) for the benchmark's
reference arm, without CMake, glog, armadillo or googletest, none of which the image has:

* every source file of the reference is compiled as it is, its ``.cu`` files for sm_100;
* three stand-in headers (``shim/``: glog's CHECK/LOG macros, the std headers armadillo would
  pull in, two googletest symbols) and stubs for three armadillo-based legacy CPU kernels that
  the Qwen3 path never calls stand in for the missing libraries;
* ``model_main`` is the reference's own command line (model/model_main.cpp, unchanged: its
  ``--bench`` mode is the reference's throughput benchmark); ``decode_main`` is a small driver of
  its LLMEngine for decode steps at a standing context (``decode_main.cpp`` here).

    python baseline/reference_arm/build.py [--reference /path/to/tiny-llm-infer] [--out baseline/_ref]

The result (``<out>/bin/model_main``, ``<out>/bin/decode_main``) needs only the CUDA runtime,
cuBLAS and cuRAND at run time.  Nothing of this repository's engine is compiled or linked in.
"""
import argparse
import os
import site
import subprocess
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent

CPP_SOURCES = """utils/src/status.cpp utils/src/unicode.cpp utils/src/unicode-data.cpp
memory/src/*.cpp tensor/src/tensor.cpp
kernels/src/add_kernel_cpu.cpp kernels/src/embed_kernel_cpu.cpp kernels/src/matmul_kernel_cpu.cpp
kernels/src/paged_attention_cpu.cpp kernels/src/rmsnorm_kernel_cpu.cpp kernels/src/rope_kernel_cpu.cpp
kernels/src/swiglu_kernel_cpu.cpp kernels/src/kernels_interface.cpp
layers/src/*.cpp model/src/*.cpp engine/src/*.cpp""".split()

STUBS = """// the three armadillo-based legacy CPU kernels are unused on the Qwen3 path
#include "tensor.h"
namespace my_vllm {
void scale_inplace_cpu(float, const Tensor&, void*) { std::abort(); }
void softmax_inplace_cpu(const Tensor&, void*) { std::abort(); }
void softmax_inplace_cpu(const float*, size_t) { std::abort(); }
void scale_sum_kernel_cpu(const Tensor&, const Tensor&, const Tensor&, int, int, int, void*) { std::abort(); }
}
"""


def json_include() -> Path:
    for sp in site.getsitepackages():
        cand = Path(sp) / "include" / "cudnn_frontend" / "thirdparty"
        if (cand / "nlohmann" / "json.hpp").is_file():
            return cand
    raise SystemExit("nlohmann/json.hpp not found (the reference needs it)")


def compile_reference(ref: Path, out: Path, jobs: int = 8):
    """Compile every source of the reference into ``out/obj``; returns (the g++ command that
    compiles and links a main against them, the object files, the link flags)."""
    obj = out / "obj"
    obj.mkdir(parents=True, exist_ok=True)
    incs = []
    for d in ("utils", "memory", "tensor", "kernels", "layers", "model", "engine"):
        incs += ["-I", ref / d / "include"]
    incs += ["-I", ref, "-I", HERE / "shim", "-I", json_include(), "-I", "/usr/local/cuda/include"]
    force = ["-include", HERE / "shim" / "armadillo"]
    cxx = ["g++", "-std=c++17", "-O3", "-fopenmp", "-w", *force, *incs]
    nvcc = ["nvcc", "-arch=sm_100", "-std=c++17", "-O3", "-w", "-Xcompiler", "-fopenmp", *force, *incs]
    stubs = obj / "stubs.cpp"
    stubs.write_text(STUBS)
    jobs_list, objects = [], []
    sources = [s for pat in CPP_SOURCES for s in sorted(ref.glob(pat))] + [stubs]
    for src in sources:
        o = obj / (src.parent.parent.name + "_" + src.stem + ".o")
        objects.append(o)
        jobs_list.append([*cxx, "-c", src, "-o", o])
    for cu in sorted((ref / "kernels" / "src").glob("*.cu")) + sorted((ref / "utils" / "src").glob("*.cu")):
        o = obj / (cu.stem + "_cu.o")
        objects.append(o)
        jobs_list.append([*nvcc, "-c", cu, "-o", o])
    running = []
    for cmd in jobs_list:
        if Path(cmd[-1]).is_file():
            continue
        while len(running) >= jobs:
            assert running.pop(0).wait() == 0, "compilation of the reference failed"
        print("+", Path(cmd[-3]).name, flush=True)
        running.append(subprocess.Popen([str(c) for c in cmd]))
    for p in running:
        assert p.wait() == 0, "compilation of the reference failed"
    link = ["-L/usr/local/cuda/lib64", "-Wl,-rpath,/usr/local/cuda/lib64", "-lcudart", "-lcublas", "-lcurand", "-lgomp"]
    return cxx, objects, link


def build(ref: Path, out: Path, jobs: int = 8) -> None:
    cxx, objects, link = compile_reference(ref, out, jobs)
    bins = out / "bin"
    bins.mkdir(parents=True, exist_ok=True)
    for name, main in (("model_main", ref / "model" / "model_main.cpp"), ("decode_main", HERE / "decode_main.cpp")):
        cmd = [*cxx, main, *objects, "-o", bins / name, *link]
        print("+ link", name, flush=True)
        subprocess.run([str(c) for c in cmd], check=True)
    (out / "BUILT_FROM").write_text(f"{ref}\n")


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--reference", default=os.environ.get("TLLM_REFERENCE", str(ROOT.parent / "reference")),
                    help="the reference's source tree (default: $TLLM_REFERENCE, or a folder `reference` beside this repository)")
    ap.add_argument("--out", default=str(ROOT / "baseline" / "_ref"))
    ap.add_argument("--jobs", type=int, default=os.cpu_count() or 4)
    args = ap.parse_args()
    ref = Path(args.reference)
    if not (ref / "model" / "model_main.cpp").is_file():
        print(f"no reference sources at {ref}", file=sys.stderr)
        return 1
    build(ref, Path(args.out), args.jobs)
    print("built", Path(args.out) / "bin")
    return 0


if __name__ == "__main__":
    sys.exit(main())
