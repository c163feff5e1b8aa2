"""Build recipe for the reference's own Blackwell kernel (test infrastructure, like the rest of oracle/).

The reference operator ships its selected implementation as one CUDA source,
``operators/moe/nvfp4_fused_moe/candidate/nvfp4_moe.cu`` of bcacdwk/KernelSchema, which exports a flat C ABI
(``moe_init``, ``moe_run``). This script compiles that file, from where it lies in the reference checkout, for
sm_100a into ``oracle/_ref/libnvfp4_moe_ref.so`` (git-ignored). Nothing of the reference is copied into this
repository. It only runs where the reference checkout exists; on a GPU box the prebuilt library is used.

    python oracle/build_ref.py [--force]
"""
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("KERNELSCHEMA_REFERENCE", "/root/reference")
SRC = os.path.join(REF, "kernel_wiki/aka-cuda-operators-20261030/operators/moe/nvfp4_fused_moe/candidate/nvfp4_moe.cu")
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "libnvfp4_moe_ref.so")


def build(force: bool = False):
    """Returns the library path, or None when the reference checkout is absent."""
    if not os.path.exists(SRC):
        return OUT if os.path.exists(OUT) else None
    if os.path.exists(OUT) and not force and os.path.getmtime(OUT) >= os.path.getmtime(SRC):
        return OUT
    os.makedirs(OUT_DIR, exist_ok=True)
    nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
    # the same flags the reference's host passes (candidate/solution.py:66-95), with the arch fixed to sm_100a
    cmd = [nvcc, "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC", "-w",
           "-o", OUT, SRC]
    res = subprocess.run(cmd, capture_output=True, text=True)
    if res.returncode != 0:
        raise RuntimeError("reference kernel does not build with this toolchain:\n" + res.stderr[-2000:])
    return OUT


if __name__ == "__main__":
    print(build("--force" in sys.argv))
