"""Compile the reference's own Q-centric kernels (p02 / p03) from sources copied, unmodified,
into the git-ignored baseline/_ref/q_centric/ (nvcc cross-compiles without a GPU), with the
flags of attention/q_centric/progression.py:29-36. The resulting shared library registers
torch.ops.xomtention_progression.{attention, attention_out}; `bench.py --workload refcmp`
times it next to this repository's kernel on the same box. The only added file is a stub for
the archived p01 launcher, which the published tree does not contain."""
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


if __name__ == "__main__":
    if not os.path.isdir(SRC):
        sys.exit("copy the reference's attention/q_centric sources into baseline/_ref/q_centric first")
    build()
