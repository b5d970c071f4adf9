"""Compile the reference's own kernels from sources copied, unmodified, into the git-ignored
baseline/_ref/ (nvcc cross-compiles without a GPU):

* q_centric/  -> xomtention_progression.so (p02 / p03), flags of attention/q_centric/progression.py:29-36;
  registers torch.ops.xomtention_progression.{attention, attention_out}; timed by
  `bench.py --workload refcmp`. The only added file is a stub for the archived p01 launcher, which
  the published tree does not contain.
* kv_centric/ -> the round-11 KV-centric extension, built by the reference's own
  optimization_round11/api11.py:load_extension (torch.ops.xomtention_kvopt11); timed by
  `bench.py --workload kvtoken`.
* r1_r4/ holds the reference's Triton selectors (compiled by Triton at run time); timed by
  `bench.py --workload refsel`.

Copy the reference's attention/q_centric sources, attention/kv_centric and indexers/r1_r4 into
baseline/_ref/ first; nothing under baseline/_ref/ is committed."""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "_ref", "q_centric")
LIB = os.path.join(HERE, "_ref", "xomtention_progression.so")


def build():
    from torch.utils.cpp_extension import load
    os.makedirs(os.path.join(HERE, "_ref", "build"), exist_ok=True)
    os.environ.setdefault("TORCH_CUDA_ARCH_LIST", "10.0a")
    try:
        load(name="xomtention_progression",
             sources=[os.path.join(SRC, f) for f in ("progression_attention.cpp", "01_block_sparse.cu",
                                                      "02_gqa_block_sparse.cu", "p01_stub.cu")],
             extra_include_paths=[SRC], extra_cflags=["-O3"],
             extra_cuda_cflags=["-O3", "-lineinfo", "-gencode=arch=compute_100a,code=sm_100a"],
             extra_ldflags=["-lcuda"], build_directory=os.path.join(HERE, "_ref", "build"),
             is_python_module=False, verbose=True)
    except OSError as e:   # the load step needs libcuda; the compile has finished by then
        print("built; not loaded here:", e)
    import shutil
    shutil.copy(os.path.join(HERE, "_ref", "build", "xomtention_progression.so"), LIB)
    print(LIB)


def build_kv_centric():
    root = os.path.join(HERE, "_ref", "kv_centric", "optimization_round11")
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
    if not os.path.isdir(SRC):
        sys.exit("copy the reference's attention/q_centric sources into baseline/_ref/q_centric first")
    build()
    build_kv_centric()
