"""The allocation-free attention entry point (nova_launch_attn_decode_paged_static).

It exists for hosts that are not allowed to allocate device memory when they call the library — an
engine that lives inside one start-up arena, code between cudaStreamBeginCapture and EndCapture, a
plug-in sandbox — and therefore cannot pass a scratch buffer.  Its scratch is a fixed array inside the
library, shared by all calls on a GPU, so this file checks, through the C ABI, that two calls in a row
(the second with other inputs and a different split, so that anything left over from the first would
show) give what the caller-scratch entry point gives and what the CPU oracle's exact softmax gives on the
downloaded pages, and that a shape beyond the fixed size is refused.

Collected last on purpose: a failure here must not hide the results of any other test.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

REL_TOL, ABS_TOL = 2e-3, 1e-2     # the tolerance of the other attention tests


def test_static_scratch_matches_caller_scratch(nv, ob):
    NH, NKV, L, layer = 28, 4, 2, 1
    eng = nv.Engine(L, NH, NKV, ctx=2048, n_slices=1, kv_dtype=nv.KV_F16)
    s = eng.session_create()
    rng = np.random.default_rng(99)
    eng.permute_pages(s, rng.permutation(eng.nblocks))
    shp = eng.shape()
    tab = nv.lib.nova_kv_table_slot(eng.h, eng.session_slice(s))
    n_ctx = 1500
    for lyr in range(L):
        k = nv.to_device(rng.standard_normal((n_ctx, NKV, 128)).astype(np.float32))
        v = nv.to_device(rng.standard_normal((n_ctx, NKV, 128)).astype(np.float32))
        nv.check(nv.lib.nova_launch_rope_append_paged(C.byref(shp), eng.k_base, eng.v_base, tab, lyr, eng.nb, n_ctx, 0,
                                                      None, k.ptr, v.ptr, nv.lib.nova_rope_cos(eng.h),
                                                      nv.lib.nova_rope_sin(eng.h), None))
    nv.check(nv.lib.dev_sync())
    scratch = nv.DevBuf(int(nv.lib.nova_attn_scratch_floats(C.byref(shp))) * 4)
    want_d, got_d = nv.DevBuf(NH * 128 * 4), nv.DevBuf(NH * 128 * 4)
    q_host = [rng.standard_normal((NH, 128)).astype(np.float32) for _ in range(2)]
    qs = [nv.to_device(q) for q in q_host]
    nv.check(nv.lib.dev_sync())
    host_k, host_v = eng.read_pools()                                   # for the oracle
    host_table = eng.pool.table(eng.session_slice(s))
    osh = ob.shape(L, NH, NKV, ob.KV_F16)
    free_before = nv.lib.dev_max_alloc()
    for q, qh, n_keys in zip(qs, q_host, (1500, 37)):          # two calls in a row on the shared array
        nv.check(nv.lib.nova_launch_attn_decode_paged(C.byref(shp), q.ptr, eng.k_base, eng.v_base, tab, layer, eng.nb,
                                                      n_keys, want_d.ptr, scratch.ptr, None))
        got_d.zero()
        nv.check(nv.lib.nova_launch_attn_decode_paged_static(C.byref(shp), q.ptr, eng.k_base, eng.v_base, tab, layer,
                                                             eng.nb, n_keys, got_d.ptr, None))
        nv.check(nv.lib.dev_sync())
        want, got = want_d.download(np.float32), got_d.download(np.float32)
        assert np.isfinite(got).all() and np.abs(want).max() > 0
        rel = np.linalg.norm(got - want) / np.linalg.norm(want)
        assert rel <= REL_TOL and np.abs(got - want).max() <= ABS_TOL, (n_keys, rel)
        exact = ob.attn_decode_paged(osh, qh, host_k, host_v, host_table, layer, eng.nb, n_keys, exact=True).ravel()
        rel = np.linalg.norm(got - exact) / np.linalg.norm(exact)
        assert rel <= REL_TOL and np.abs(got - exact).max() <= ABS_TOL, ("oracle", n_keys, rel)
    assert nv.lib.dev_max_alloc() == free_before                   # nothing was allocated on the device
    # a shape the fixed array cannot hold is refused with a clear code, not truncated
    big = nv.KvShape(int(nv.lib.nova_attn_static_scratch_max_heads()) + 8, 8, 128, 16, nv.KV_F16, 1)
    assert nv.lib.nova_launch_attn_decode_paged_static(C.byref(big), want_d.ptr, eng.k_base, eng.v_base, tab, 0,
                                                       eng.nb, 4, got_d.ptr, None) == nv.ERR_TOO_LARGE
    eng.close()
