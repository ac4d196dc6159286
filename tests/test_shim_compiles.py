"""The reference-side binding (include/nova_b200_shim.h): a translation unit that includes the reference's
own include/nova/kernel.h and calls its four hot-path launchers through the shim compiles and links against
libnova_b200.so, for both model shapes the reference ships for this path.  Needs the reference tree (skipped
where it is absent, e.g. on a GPU box) — nothing is executed."""
import os
import shutil
import subprocess
import sys

import pytest

from conftest import ROOT

sys.path.insert(0, ROOT)
from oracle import build as obuild  # noqa: E402

SRC = r'''
#include "nova/kernel.h"
#include "graph/kv_pool_cfg.h"
#include "nova_b200_shim.h"
// the call sites of code/graph/dense.h:75-95, spelled out
int step(float* q, float* k, float* v, float* pool_k, float* pool_v, const int32_t* table, int layer, int nb,
         int64_t pos, const float* cs, const float* sn, float* out, float* scratch, cudaStream_t s) {
    nova::Kernel::rope_batch(q, k, 1, pos, cs, sn, s);
    nova::Kernel::kv_store_paged(pool_k, pool_v, table, layer, nb, 1, pos, k, v, s);
    nova::Kernel::attn_decode_paged(q, pool_k, pool_v, table, layer, nb, (int)pos + 1, out, scratch, s);
    return 0;
}
int main() { return 0; }
'''


@pytest.mark.parametrize("macro", ["NOVA_MODEL_QWEN25_7B", "NOVA_MODEL_QWEN25_1P5B", "NOVA_MODEL_R1_LLAMA8B"])
def test_shim_compiles_and_links(tmp_path, nv, macro):
    ref = obuild.reference_dir()
    if ref is None or shutil.which("g++") is None:
        pytest.skip("reference tree or compiler not present")
    cuda_inc = "/usr/local/cuda/include"
    if not os.path.isdir(cuda_inc):
        pytest.skip("CUDA headers not present")
    src = tmp_path / "shim_tu.cpp"
    src.write_text(SRC)
    exe = tmp_path / "shim_tu"
    lib_dir = os.path.dirname(nv.LIB_PATH)
    cmd = ["g++", "-std=c++17", f"-D{macro}", f"-I{ref}/include", f"-I{ref}/code", f"-I{ROOT}/include", f"-I{cuda_inc}",
           str(src), "-o", str(exe), f"-L{lib_dir}", "-lnova_b200", f"-Wl,-rpath,{lib_dir}",
           "-L/usr/local/cuda/lib64", "-lcudart"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-3000:]
