"""The reference-side binding (include/nova_b200_shim.h): a translation unit that includes the reference's
own include/nova/kernel.h and calls its four hot-path launchers through the shim compiles and links against
libnova_b200.so, for both model shapes the reference ships for this path.  Needs the reference tree (skipped
where it is absent, e.g. on a GPU box).  test_shim_executes then RUNS the same call sites on a GPU: they are built
into oracle/_ref/libnova_shim_<model>.so by oracle/build.py here and loaded there."""
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


@pytest.mark.gpu
@pytest.mark.parametrize("model", ["qwen25_7b", "r1_llama8b"])
def test_shim_executes(nv, ob, model):
    """The reference's own call sequence for one decode step of one session in one layer - Kernel::rope_batch,
    Kernel::kv_store_paged, Kernel::attn_decode_paged (code/graph/dense.h:75-95) - compiled against the shim header
    and executed on fp32 pools (the reference's format): rotated q/k and pages bit-identical to the oracle's, attention
    within the tolerance, over a context that grows across page boundaries; both RoPE layouts the reference has."""
    import ctypes as C

    import numpy as np
    g = ob.shim_exec(model)
    if g is None:
        pytest.skip("shim library not built")
    shape6 = (C.c_int32 * 6)()
    g.shim_shape(shape6)
    L_model, NH, NKV, HD, KB, theta = list(shape6)
    neox = 0 if model == "r1_llama8b" else 1
    L, ctx = 2, 256
    eng = nv.Engine(L, NH, NKV, ctx=ctx, n_slices=1, kv_dtype=nv.KV_F32, rope_theta=theta, rope_neox=neox, kv_block=KB,
                    rope_positions=4096)
    s = eng.session_create()
    rng = np.random.default_rng(12)
    eng.permute_pages(s, rng.permutation(eng.nblocks))
    table_host = eng.pool.table(eng.session_slice(s))
    table = nv.lib.nova_kv_table_slot(eng.h, eng.session_slice(s))
    cs_d, sn_d = nv.DevBuf(4096 * 64 * 4), nv.DevBuf(4096 * 64 * 4)
    g.shim_rope_table(cs_d.ptr, sn_d.ptr, None)                 # the reference's kCtx rows, through the shim
    nv.check(nv.lib.dev_sync())
    cs, sn = cs_d.download(np.float32).reshape(4096, 64), sn_d.download(np.float32).reshape(4096, 64)
    ecs, esn = eng.rope_tables()
    assert np.array_equal(cs.view(np.uint32), ecs.view(np.uint32)) and np.array_equal(sn.view(np.uint32), esn.view(np.uint32))
    sh = ob.shape(L, NH, NKV, ob.KV_F32, rope_neox=neox, kv_block=KB)
    pk, pv = ob.new_pools(sh, eng.nb)
    scratch = nv.DevBuf(NH * 32 * (HD + 2) * 4)                   # src/model.cpp:148
    out = nv.DevBuf(NH * HD * 4)
    for pos in range(0, 70):
        for layer in range(L):
            q = rng.standard_normal((1, NH, HD)).astype(np.float32)
            k = rng.standard_normal((1, NKV, HD)).astype(np.float32)
            v = rng.standard_normal((1, NKV, HD)).astype(np.float32)
            dq, dk, dv = nv.to_device(q), nv.to_device(k), nv.to_device(v)
            g.shim_decode_layer(dq.ptr, dk.ptr, dv.ptr, eng.k_base, eng.v_base, table, layer, eng.nb, pos, cs_d.ptr, sn_d.ptr,
                                out.ptr, scratch.ptr, None)
            nv.check(nv.lib.dev_sync())
            ob.rope_append_paged(sh, pk, pv, table_host, layer, eng.nb, 1, pos, q, k, v, cs, sn)      # rotates q, k
            assert np.array_equal(dq.download(np.float32).view(np.uint32), q.ravel().view(np.uint32))
            assert np.array_equal(dk.download(np.float32).view(np.uint32), k.ravel().view(np.uint32))
            if pos in (0, 15, 16, 17, 33, 69):
                want = ob.attn_decode_paged(sh, q[0], pk, pv, table_host, layer, eng.nb, pos + 1, exact=True)
                got = out.download(np.float32).reshape(NH, HD)
                rel = float(np.linalg.norm(got.astype(np.float64) - want) / np.linalg.norm(want))
                assert rel <= 2e-3 and float(np.abs(got - want).max()) <= 1e-2, (pos, layer, rel)
    gk, gv = eng.read_pools()
    assert np.array_equal(gk.view(np.uint32), pk.view(np.uint32)) and np.array_equal(gv.view(np.uint32), pv.view(np.uint32))
    eng.close()
