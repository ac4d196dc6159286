"""Build recipe of the checker (TEST INFRASTRUCTURE; nothing here is product code).

  oracle/_build/libpaged_decode_oracle.so   the CPU restatement (paged_decode_oracle.c)
  oracle/_ref/libnova_ref_host.so           the reference's own host headers behind a C shim
  oracle/_ref/libnova_ref_gpu_<model>.so    the reference's own CUDA kernels for this path,
                                            compiled unmodified for sm_100a

The two `_ref` libraries are compiled from the reference tree where it lies (directory named
by $NOVA_REFERENCE_DIR, default: `reference` beside the repository); where that tree is
absent (a GPU box) the prebuilt files are used as they are.  No reference source is copied.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(HERE)
BUILD = os.path.join(HERE, "_build")
REF_OUT = os.path.join(HERE, "_ref")

ORACLE_SO = os.path.join(BUILD, "libpaged_decode_oracle.so")
REF_HOST_SO = os.path.join(REF_OUT, "libnova_ref_host.so")
REF_HOST_BLOCKS = (16, 8, 32, 64)          # NOVA_KV_BLOCK variants of the reference's host headers
# name -> the reference's compile-time switches: the model (include/nova/model/select.h) and, for the
# page-size variants, NOVA_KV_BLOCK (code/graph/kv_pool_cfg.h:12-26)
REF_GPU_MODELS = {
    "qwen25_7b": ["NOVA_MODEL_QWEN25_7B"],
    "qwen25_1p5b": ["NOVA_MODEL_QWEN25_1P5B"],
    "r1_llama8b": ["NOVA_MODEL_R1_LLAMA8B"],              # RopeLayout::Norm, theta 500000, 32 q / 8 kv heads
    "r1_qwen1p5b_abl": ["NOVA_MODEL_R1_QWEN1P5B_ABL"],    # theta 10000
    "qwen25_7b_kb8": ["NOVA_MODEL_QWEN25_7B", "NOVA_KV_BLOCK=8"],
    "qwen25_7b_kb32": ["NOVA_MODEL_QWEN25_7B", "NOVA_KV_BLOCK=32"],
    "qwen25_7b_kb64": ["NOVA_MODEL_QWEN25_7B", "NOVA_KV_BLOCK=64"],
    "qwen25_1p5b_kb32": ["NOVA_MODEL_QWEN25_1P5B", "NOVA_KV_BLOCK=32"],
}


def ref_gpu_so(model: str) -> str:
    return os.path.join(REF_OUT, f"libnova_ref_gpu_{model}.so")


def reference_dir() -> str | None:
    d = os.environ.get("NOVA_REFERENCE_DIR") or os.path.join(os.path.dirname(REPO), "reference")
    return d if os.path.isdir(os.path.join(d, "src", "kernel")) else None


def _newer(out: str, srcs: list[str]) -> bool:
    if not os.path.exists(out):
        return False
    t = os.path.getmtime(out)
    return all(os.path.getmtime(s) <= t for s in srcs if os.path.exists(s))


def _run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise RuntimeError(f"build failed: {cmd[0]}")


def build_oracle(force: bool = False) -> str:
    src = os.path.join(HERE, "paged_decode_oracle.c")
    if not force and _newer(ORACLE_SO, [src]):
        return ORACLE_SO
    os.makedirs(BUILD, exist_ok=True)
    _run(["gcc", "-O2", "-std=c11", "-fopenmp", "-ffp-contract=off", "-fno-fast-math", "-shared", "-fPIC",
          src, "-o", ORACLE_SO, "-lm"])
    return ORACLE_SO


def ref_host_so(kv_block: int = 16) -> str:
    return REF_HOST_SO if kv_block == 16 else os.path.join(REF_OUT, f"libnova_ref_host_kb{kv_block}.so")


def build_ref_host(force: bool = False, kv_block: int = 16) -> str | None:
    ref = reference_dir()
    src = os.path.join(HERE, "ref_host_shim.cpp")
    so = ref_host_so(kv_block)
    if ref is None:
        return so if os.path.exists(so) else None
    if not force and _newer(so, [src]):
        return so
    os.makedirs(REF_OUT, exist_ok=True)
    _run(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", f"-DNOVA_KV_BLOCK={kv_block}", f"-I{ref}/code", f"-I{ref}/include",
          src, "-o", so])
    return so


def build_ref_gpu(force: bool = False) -> dict[str, str]:
    ref = reference_dir()
    out: dict[str, str] = {}
    shim = os.path.join(HERE, "ref_gpu_shim.cu")
    procs = []
    for model, macros in REF_GPU_MODELS.items():
        so = ref_gpu_so(model)
        if ref is None or shutil.which("nvcc") is None:
            if os.path.exists(so):
                out[model] = so
            continue
        if force or not _newer(so, [shim]):
            os.makedirs(REF_OUT, exist_ok=True)
            cmd = ["nvcc", "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
                   *[f"-D{m}" for m in macros], f"-I{ref}/include", f"-I{ref}/code", "-Xcompiler", "-fPIC", "-shared", "-w",
                   shim, f"{ref}/src/kernel/rope.cu", f"{ref}/src/kernel/elem.cu", f"{ref}/src/kernel/attn.cu",
                   "-o", so]
            procs.append((cmd, subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)))
        out[model] = so
    for cmd, p in procs:                  # the variants compile side by side
        text, _ = p.communicate()
        if p.returncode != 0:
            sys.stderr.write(" ".join(cmd) + "\n" + (text or ""))
            raise RuntimeError("build failed: nvcc (reference kernels)")
    return out


SHIM_MODELS = {"qwen25_7b": "NOVA_MODEL_QWEN25_7B", "r1_llama8b": "NOVA_MODEL_R1_LLAMA8B"}


def shim_so(model: str) -> str:
    return os.path.join(REF_OUT, f"libnova_shim_{model}.so")


def build_shim_exec(force: bool = False) -> dict[str, str]:
    """oracle/_ref/libnova_shim_<model>.so: the reference's call sites (include/nova/kernel.h) bound to the product
    through include/nova_b200_shim.h, to be executed by the GPU tests.  Needs the reference tree, g++, the CUDA
    headers and the built product library; elsewhere the prebuilt files are used."""
    ref = reference_dir()
    out: dict[str, str] = {}
    src = os.path.join(HERE, "shim_exec.cpp")
    lib_dir = os.path.join(REPO, "conflux-nova_b200")
    cuda_inc = "/usr/local/cuda/include"
    can_build = (ref is not None and shutil.which("g++") and os.path.isdir(cuda_inc)
                 and os.path.exists(os.path.join(lib_dir, "libnova_b200.so")))
    for model, macro in SHIM_MODELS.items():
        so = shim_so(model)
        if not can_build:
            if os.path.exists(so):
                out[model] = so
            continue
        if force or not _newer(so, [src, os.path.join(REPO, "include", "nova_b200_shim.h"), os.path.join(REPO, "include", "nova_b200.h")]):
            os.makedirs(REF_OUT, exist_ok=True)
            _run(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", f"-D{macro}", f"-I{ref}/include", f"-I{ref}/code",
                  f"-I{REPO}/include", f"-I{cuda_inc}", src, "-o", so, f"-L{lib_dir}", "-lnova_b200",
                  "-Wl,-rpath,$ORIGIN/../../conflux-nova_b200"])
        out[model] = so
    return out


def build_all(force: bool = False) -> None:
    build_oracle(force)
    for kb in REF_HOST_BLOCKS:
        build_ref_host(force, kb)
    build_ref_gpu(force)
    build_shim_exec(force)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv)
    print("oracle:", ORACLE_SO, os.path.exists(ORACLE_SO))
    print("ref host:", REF_HOST_SO, os.path.exists(REF_HOST_SO))
    for m in REF_GPU_MODELS:
        print("ref gpu:", ref_gpu_so(m), os.path.exists(ref_gpu_so(m)))
