"""Copies the reference's own kernels, unmodified, from a checkout of the reference into the
git-ignored baseline/_ref/ and compiles them (nvcc cross-compiles without a GPU):

    python baseline/build_reference_kernels.py --ref /path/to/sparse-attention-b200

* q_centric/  -> xomtention_progression.so (p02 / p03), flags of attention/q_centric/progression.py:29-36;
  registers torch.ops.xomtention_progression.{attention, attention_out}; timed by
  `bench.py --workload refcmp`. The only added file is a stub for the archived p01 launcher, which
  the published tree does not contain.
* kv_centric/ -> the round-11 KV-centric extension, built by the reference's own
  optimization_round11/api11.py:load_extension (torch.ops.xomtention_kvopt11); timed by
  `bench.py --workload kvtoken`.
* r1_r4/ holds the reference's Triton selectors (compiled by Triton at run time); timed by
  `bench.py --workload refsel`.
* fp4/ holds the reference's NVFP4 indexer: the vendored MiniMax MSA scorer (CuTe DSL, compiled at
  run time by nvidia-cutlass-dsl) and tile_topk.cu + wrapper.cpp -> xomtention_tile_topk.so
  (flags of indexers/fp4/__init__.py:14-22); timed by `bench.py --workload refsel`.

Nothing under baseline/_ref/ is committed."""
import argparse
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
SRC = os.path.join(REF, "q_centric")
LIB = os.path.join(REF, "xomtention_progression.so")

P01_STUB = """// The archived p01 kernel is not part of the published reference tree: variant 0 is not callable here.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <c10/util/Exception.h>
void dense13_sparse_two_q_launch(const nv_bfloat16*, const nv_bfloat16*, const nv_bfloat16*, const int32_t*, nv_bfloat16*,
                                 int, int, int, int, int, int, cudaStream_t) {
  TORCH_CHECK(false, "p01 is not included in the reference tree");
}
"""


def copy_sources(ref):
    """Plain copies of the reference files the comparisons need."""
    os.makedirs(SRC, exist_ok=True)
    qc = os.path.join(ref, "attention", "q_centric")
    for f in ("progression_attention.cpp", "01_block_sparse.cu", "02_gqa_block_sparse.cu", "approximations.cuh",
              "common.cuh", "smem_layout_swizzle128.cuh",
              # the reference's own gate (run by tests/test_gpu_reference_gates.py against this library)
              "progression.py", "progression_validation.py", "checkpoints.py"):
        shutil.copy(os.path.join(qc, f), os.path.join(SRC, f))
    stub = os.path.join(SRC, "p01_stub.cu")
    if not os.path.exists(stub):
        open(stub, "w").write(P01_STUB)
    for src, dst in (("attention/kv_centric", "kv_centric"), ("indexers/r1_r4", "r1_r4"), ("indexers/fp4", "fp4")):
        target = os.path.join(REF, dst)
        if os.path.isdir(target):
            shutil.rmtree(target)
        shutil.copytree(os.path.join(ref, src), target, ignore=shutil.ignore_patterns("__pycache__", "build"))


def _load(name, sources, include, build_dir):
    from torch.utils.cpp_extension import load
    os.makedirs(build_dir, exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    try:
        load(name=name, sources=sources, extra_include_paths=include, extra_cflags=["-O3"],
             extra_cuda_cflags=["-O3", "-lineinfo", "-gencode=arch=compute_100a,code=sm_100a"],
             extra_ldflags=["-lcuda"], build_directory=build_dir, is_python_module=False, verbose=False)
    except OSError as e:   # the load step needs libcuda; the compile has finished by then
        print("built; not loaded here:", e)


def build():
    _load("xomtention_progression",
          [os.path.join(SRC, f) for f in ("progression_attention.cpp", "01_block_sparse.cu", "02_gqa_block_sparse.cu",
                                          "p01_stub.cu")], [SRC], os.path.join(REF, "build"))
    shutil.copy(os.path.join(REF, "build", "xomtention_progression.so"), LIB)
    print(LIB)


def build_tile_topk():
    root = os.path.join(REF, "fp4")
    if not os.path.isdir(root):
        print("baseline/_ref/fp4 absent: skipped")
        return
    _load("xomtention_tile_topk", [os.path.join(root, "wrapper.cpp"), os.path.join(root, "tile_topk.cu")], [root],
          os.path.join(root, "build"))
    print(os.path.join(root, "build", "xomtention_tile_topk.so"))


def build_kv_centric():
    root = os.path.join(REF, "kv_centric", "optimization_round11")
    if not os.path.isdir(root):
        print("baseline/_ref/kv_centric absent: skipped")
        return
    os.environ["MAX_JOBS"] = os.environ.get("MAX_JOBS", "8")
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    sys.path.insert(0, root)
    import api11
    try:
        api11.load_extension()
    except OSError as e:   # the load step needs libcuda; the compile has finished by then
        print("built; not loaded here:", e)
    print(os.path.join(root, "build"))


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("SPARSE_ATTENTION_REFERENCE", ""),
                    help="checkout of the reference project (dinara-dl/sparse-attention-b200)")
    args = ap.parse_args()
    if args.ref:
        copy_sources(args.ref)
    if not os.path.isdir(SRC):
        sys.exit("pass --ref /path/to/the/reference (nothing has been copied into baseline/_ref/ yet)")
    build()
    build_tile_topk()
    build_kv_centric()
