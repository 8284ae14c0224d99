"""Compiles the REFERENCE's own CUDA extension (dag_loss.cpp, dag_loss.cu,
dag_best_alignment.cu, logsoftmax_gather.cu of fs_plugins/custom_ops) from the sources where
they lie in a DA-Transformer checkout into oracle/_ref/, unmodified, for sm_100.

    python oracle/build_ref.py [--reference /path/to/DA-Transformer]

TEST INFRASTRUCTURE ONLY: the result is a second checker (and the GPU baseline the benchmark
prints next to our numbers).  Nothing of the reference is copied into this repository; the
build directory oracle/_ref/ is git-ignored.  The same compile line the reference uses at
run time (dag_loss.py:50-61: torch.utils.cpp_extension.load with -O3
-DOF_SOFTMAX_USE_FAST_MATH), with an explicit architecture because there is no GPU here.
"""
import argparse
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "_ref")
NAME = "dag_loss_fn"


def build(reference):
    src_dir = os.path.join(reference, "fs_plugins", "custom_ops")
    sources = [os.path.join(src_dir, f) for f in
               ("dag_loss.cpp", "dag_loss.cu", "dag_best_alignment.cu", "logsoftmax_gather.cu")]
    missing = [s for s in sources if not os.path.exists(s)]
    if missing:
        print(f"reference sources not found: {missing}", file=sys.stderr)
        return 1
    os.makedirs(OUT, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0")
    os.environ.setdefault("MAX_JOBS", "4")
    from torch.utils.cpp_extension import load

    load(NAME, sources=sources, build_directory=OUT,
         extra_cflags=["-DOF_SOFTMAX_USE_FAST_MATH", "-O3"],
         extra_cuda_cflags=["-DOF_SOFTMAX_USE_FAST_MATH", "-O3"],
         extra_include_paths=[src_dir], verbose=False)
    print(os.path.join(OUT, NAME + ".so"))
    return 0


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", default=os.environ.get(
        "DAT_REFERENCE_DIR", os.path.join(os.path.dirname(os.path.dirname(HERE)), "reference")),
        help="DA-Transformer checkout (default: $DAT_REFERENCE_DIR, else ../reference)")
    sys.exit(build(ap.parse_args().reference))
