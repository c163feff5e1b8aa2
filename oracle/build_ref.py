"""Build recipe for the reference's own code of this path (test infrastructure, like the rest of oracle/).

Everything this script produces goes to ``oracle/_ref/`` (git-ignored): nothing of the reference enters this
repository's history. It only does work where the reference checkout exists; on a GPU box the prebuilt and staged
files are used as they are.

1. The reference operator ships its selected implementation as one CUDA source,
   ``operators/moe/nvfp4_fused_moe/candidate/nvfp4_moe.cu`` of bcacdwk/KernelSchema, which exports a flat C ABI
   (``moe_init``, ``moe_run``). It is compiled, from where it lies in the checkout, for sm_100a into
   ``oracle/_ref/libnvfp4_moe_ref.so``, with the flags the reference's own host passes (candidate/solution.py:66-95).
   A second copy is placed under the name and directory that host looks for
   (``cache/nvfp4_fused_moe/nvfp4_moe_<sha256[:16]>_sm100a.so`` with ``TORCH_EXTENSIONS_DIR=oracle/_ref/cache``), so
   that the unmodified host loads it without a compiler run.
2. The files a test needs to run the reference's own acceptance check against a drop-in are staged unchanged:
   ``problem/{reference.py,input.py,metadata.json,shape_cases.json,shape_range.json}`` (plus ``shapes.json``, the name
   the harness reads - eval/_runtime.py:575-577 - with the content of shape_cases.json), the check harness as the
   package ``harness/atrex_bench/eval`` (correctness.py, _runtime.py, _timeout.py, reward_hack.py) and the
   reference's own host ``candidate/{solution.py,nvfp4_moe.cu,nvfp4_fast.c}``.

    python oracle/build_ref.py [--force]
"""
import hashlib
import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.environ.get("KERNELSCHEMA_REFERENCE", "/root/reference")
OP = os.path.join(REF, "kernel_wiki/aka-cuda-operators-20261030/operators/moe/nvfp4_fused_moe")
CHK = os.path.join(REF, "kernel_wiki/aka-four-problems-20261019/evidence/qsa_prefill/reproduce/checker/atrex_bench")
SRC = os.path.join(OP, "candidate/nvfp4_moe.cu")
OUT_DIR = os.path.join(HERE, "_ref")
OUT = os.path.join(OUT_DIR, "libnvfp4_moe_ref.so")
CACHE = os.path.join(OUT_DIR, "cache")                 # TORCH_EXTENSIONS_DIR for the staged reference host
PROBLEM = os.path.join(OUT_DIR, "problem")
HARNESS = os.path.join(OUT_DIR, "harness")
CANDIDATE = os.path.join(OUT_DIR, "candidate")

STAGED = (
    [(os.path.join(OP, "problem", n), os.path.join(PROBLEM, n))
     for n in ("reference.py", "input.py", "metadata.json", "shape_cases.json", "shape_range.json")]
    + [(os.path.join(OP, "problem", "shape_cases.json"), os.path.join(PROBLEM, "shapes.json"))]
    + [(os.path.join(CHK, "__init__.py"), os.path.join(HARNESS, "atrex_bench", "__init__.py"))]
    + [(os.path.join(CHK, "eval", n), os.path.join(HARNESS, "atrex_bench", "eval", n))
       for n in ("__init__.py", "correctness.py", "_runtime.py", "_timeout.py", "reward_hack.py")]
    + [(os.path.join(OP, "candidate", n), os.path.join(CANDIDATE, n)) for n in ("solution.py", "nvfp4_moe.cu", "nvfp4_fast.c")]
)


def _newer(src, dst):
    return not os.path.exists(dst) or os.path.getmtime(dst) < os.path.getmtime(src)


def stage(force: bool = False) -> bool:
    """Copies the problem files, the check harness and the reference host into oracle/_ref/. Returns True when the
    staged tree is complete (also when it was staged earlier and the checkout is absent now)."""
    if os.path.exists(SRC):
        for src, dst in STAGED:
            if force or _newer(src, dst):
                os.makedirs(os.path.dirname(dst), exist_ok=True)
                shutil.copyfile(src, dst)
    return all(os.path.exists(dst) for _, dst in STAGED)


def host_cache_name(source_path: str) -> str:
    """File name under which the reference host caches its build of `source_path` on sm_100a (candidate/solution.py:70-75)."""
    with open(source_path, "rb") as f:
        digest = hashlib.sha256(f.read()).hexdigest()[:16]
    return f"nvfp4_moe_{digest}_sm100a.so"


def build(force: bool = False):
    """Returns the library path, or None when neither the reference checkout nor an earlier build exists."""
    if not os.path.exists(SRC):
        return OUT if os.path.exists(OUT) else None
    os.makedirs(OUT_DIR, exist_ok=True)
    if force or _newer(SRC, OUT):
        nvcc = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
        cmd = [nvcc, "-O3", "-std=c++17", "-gencode", "arch=compute_100a,code=sm_100a", "-shared", "-Xcompiler", "-fPIC", "-w",
               "-o", OUT, SRC]
        res = subprocess.run(cmd, capture_output=True, text=True)
        if res.returncode != 0:
            raise RuntimeError("reference kernel does not build with this toolchain:\n" + res.stderr[-2000:])
    stage(force)
    cached = os.path.join(CACHE, "nvfp4_fused_moe", host_cache_name(SRC))
    if force or _newer(OUT, cached):
        os.makedirs(os.path.dirname(cached), exist_ok=True)
        shutil.copyfile(OUT, cached)
    return OUT


if __name__ == "__main__":
    print(build("--force" in sys.argv))
    print("staged:", stage())
