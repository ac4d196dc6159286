"""Pages of 8, 32 and 64 tokens (NOVA_KV_BLOCK, code/graph/kv_pool_cfg.h:12-26 of the reference) through every
kernel of the path, and the sliding-window prefill (flash_paged_kernel<true>, src/kernel/attn.cu:317).

The kernels stream tiles of min(16, page) keys: a 32- or 64-token page is 2 or 4 tiles behind one block-table
entry, an 8-token page is a half-filled tile.  Checked against the CPU oracle (which takes the page size as a
parameter) and against the reference's own kernels compiled with the same -DNOVA_KV_BLOCK.  Bars as everywhere:
pages bit-exact, attention within rel-L2 <= 2e-3 and max-abs <= 1e-2."""
import ctypes as C

import numpy as np
import pytest

from test_gpu_parity import ABS_TOL, REL_TOL, assert_attn_close, bits, build_case, rel_l2, try_set_kernel

pytestmark = pytest.mark.gpu

REF_LIBS = {("qwen25_7b", 8): "qwen25_7b_kb8", ("qwen25_7b", 32): "qwen25_7b_kb32", ("qwen25_7b", 64): "qwen25_7b_kb64",
            ("qwen25_1p5b", 32): "qwen25_1p5b_kb32"}


@pytest.mark.parametrize("model,kb", list(REF_LIBS))
def test_page_sizes_vs_reference_kernels(nv, ob, model, kb):
    """The reference's rope_batch + kv_store_paged + attn_decode_paged + attn_prefill_paged built with
    -DNOVA_KV_BLOCK=kb: appended fp32 pages and rotated q/k identical, fp16 pages == round-to-nearest-even of them,
    decode and prefill attention of every kernel within tolerance of the reference's."""
    g = ob.ref_gpu(REF_LIBS[(model, kb)])
    if g is None:
        pytest.skip("reference CUDA library not built")
    shape6 = (C.c_int32 * 6)()
    g.ref_gpu_shape(shape6)
    assert shape6[4] == kb
    from test_gpu_parity import SHAPES
    NH, NKV = SHAPES[model]
    L, ctx, n, pos0, layer = 2, 4096, 300, 1000, 1
    rng = np.random.default_rng(5 + kb)
    q = rng.standard_normal((n, NH, 128)).astype(np.float32)
    k = rng.standard_normal((n, NKV, 128)).astype(np.float32)
    v = rng.standard_normal((n, NKV, 128)).astype(np.float32)
    res = {}
    for kvd in (nv.KV_F32, nv.KV_F16):
        eng = nv.Engine(L, NH, NKV, ctx=ctx, n_slices=1, kv_dtype=kvd, rope_positions=4096, kv_block=kb)
        assert eng.nblocks == ctx // kb
        s = eng.session_create()
        eng.permute_pages(s, np.random.default_rng(6).permutation(eng.nblocks))
        tab = nv.lib.nova_kv_table_slot(eng.h, eng.session_slice(s))
        dq, dk, dv = nv.to_device(q), nv.to_device(k), nv.to_device(v)
        shp = eng.shape()
        nv.check(nv.lib.nova_launch_rope_append_paged(C.byref(shp), eng.k_base, eng.v_base, tab, layer, eng.nb, n, pos0,
                                                      dq.ptr, dk.ptr, dv.ptr, nv.lib.nova_rope_cos(eng.h),
                                                      nv.lib.nova_rope_sin(eng.h), None))
        nv.check(nv.lib.dev_sync())
        res[kvd] = (eng.read_pools(), dq.download(np.float32), dk.download(np.float32))
        if kvd == nv.KV_F32:
            rcs, rsn = nv.DevBuf(4096 * 64 * 4), nv.DevBuf(4096 * 64 * 4)
            g.ref_gpu_rope_table(rcs.ptr, rsn.ptr, None)
            rpk = nv.DevBuf(L * eng.nb * eng.page_bytes).zero()
            rpv = nv.DevBuf(L * eng.nb * eng.page_bytes).zero()
            rq, rk, rv = nv.to_device(q), nv.to_device(k), nv.to_device(v)
            g.ref_gpu_rope_batch(rq.ptr, rk.ptr, n, pos0, rcs.ptr, rsn.ptr, None)
            g.ref_gpu_kv_store_paged(rpk.ptr, rpv.ptr, tab, layer, eng.nb, n, pos0, rk.ptr, rv.ptr, None)
            nv.check(nv.lib.dev_sync())
            assert g.ref_gpu_last_error() == 0
            ref = (rpk.download(np.float32), rpv.download(np.float32), rq.download(np.float32), rk.download(np.float32))
        eng.close()
    (k32, v32), q32, kk32 = res[nv.KV_F32]
    assert np.array_equal(bits(q32), bits(ref[2])) and np.array_equal(bits(kk32), bits(ref[3]))
    assert np.array_equal(bits(k32.ravel()), bits(ref[0])) and np.array_equal(bits(v32.ravel()), bits(ref[1]))
    (k16, v16), _, _ = res[nv.KV_F16]
    assert np.array_equal(bits(k16.ravel()), bits(ref[0].astype(np.float16)))
    assert np.array_equal(bits(v16.ravel()), bits(ref[1].astype(np.float16)))
    # attention: decode at lengths around the page and tile boundaries, then a prefill chunk
    for n_ctx in (1, kb - 1, kb, kb + 1, 2 * kb + 3, 700, 2047):
        eng, ss, sh, pk, pv, cs, sn, rng2 = build_case(nv, ob, model, nv.KV_F16, [n_ctx], L=2, seed=n_ctx, kv_block=kb)
        rk, rv = nv.to_device(pk.astype(np.float32)), nv.to_device(pv.astype(np.float32))
        qq = rng2.standard_normal((1, NH, 128)).astype(np.float32)
        dq = nv.to_device(qq)
        tab = nv.lib.nova_kv_table_slot(eng.h, eng.session_slice(ss[0]))
        ro, scr = nv.DevBuf(NH * 128 * 4), nv.DevBuf(NH * 32 * 130 * 4)
        g.ref_gpu_attn_decode_paged(dq.ptr, rk.ptr, rv.ptr, tab, 1, eng.nb, n_ctx, ro.ptr, scr.ptr, None)
        nv.check(nv.lib.dev_sync())
        assert g.ref_gpu_last_error() == 0
        ref_o = ro.download(np.float32).reshape(NH, 128)
        orc = ob.attn_decode_paged(sh, qq[0], pk, pv, eng.pool.table(eng.session_slice(ss[0])), 1, eng.nb, n_ctx)
        assert rel_l2(orc, ref_o) < 2e-6                      # the oracle follows the reference at this page size too
        shp = eng.shape()
        o = nv.DevBuf(NH * 128 * 4)
        nv.check(nv.lib.nova_launch_attn_decode_paged(C.byref(shp), dq.ptr, eng.k_base, eng.v_base, tab, 1, eng.nb, n_ctx,
                                                      o.ptr, scr.ptr, None))
        nv.check(nv.lib.dev_sync())
        assert_attn_close(o.download(np.float32).reshape(NH, 128), ref_o, f"raw launcher n={n_ctx}")
        eng.set_n_past(ss[0], n_ctx - 1)
        batch = eng.batch(ss)
        for kernel in (0, 1):
            if nv.lib.nova_batch_set_kernel(batch.h, kernel) != 0:
                continue
            o.zero()
            batch.attn(1, dq.ptr, o.ptr)
            nv.check(nv.lib.dev_sync())
            assert batch.device_status() == 0
            assert_attn_close(o.download(np.float32).reshape(NH, 128), ref_o, f"kernel {kernel} n={n_ctx}")
        batch.close()
        eng.close()


@pytest.mark.parametrize("kernel", [0, 1, 2])
@pytest.mark.parametrize("model,dtype,kb", [("qwen25_7b", "f16", 8), ("qwen25_7b", "f16", 32), ("qwen25_7b", "f16", 64),
                                            ("qwen25_14b", "f16", 32), ("qwen25_1p5b", "f16", 8), ("qwen25_1p5b", "f16", 64),
                                            ("qwen25_7b", "f32", 8), ("qwen25_7b", "f32", 64)])
def test_page_sizes_decode_steps_vs_oracle(nv, ob, model, dtype, kb, kernel):
    """Ragged sessions around page and tile boundaries, three decode steps per-layer and all-layers: pages bit-exact,
    attention within tolerance of the exact softmax, rotated q/k as everywhere."""
    kvd = nv.KV_F16 if dtype == "f16" else nv.KV_F32
    if kernel >= 1 and kvd != nv.KV_F16:
        pytest.skip("tensor-core kernel is fp16-KV only")
    ctx_lens = [0, 1, 7, 8, 9, 15, 16, 17, 31, 32, 33, 63, 64, 65, 127, 129, 255, 1024, 1500]
    eng, ss, sh, pk, pv, cs, sn, rng = build_case(nv, ob, model, kvd, ctx_lens, kv_block=kb)
    NH, NKV, L, S = eng.NH, eng.NKV, eng.L, len(ss)
    tables = np.stack([eng.pool.table(eng.session_slice(s)) for s in ss])
    batch = eng.batch(ss)
    try_set_kernel(nv, batch, kernel)
    pos = list(ctx_lens)
    out_d = nv.DevBuf(L * S * NH * 128 * 4)
    for step in range(3):
        q = rng.standard_normal((L, S, NH, 128)).astype(np.float32)
        k = rng.standard_normal((L, S, NKV, 128)).astype(np.float32)
        v = rng.standard_normal((L, S, NKV, 128)).astype(np.float32)
        dq, dk, dv = nv.to_device(q), nv.to_device(k), nv.to_device(v)
        assert batch.cow() == 0
        if step % 2 == 0:
            batch.step_all_layers(dq.ptr, dk.ptr, dv.ptr, out_d.ptr)
        else:
            qs, ks = S * NH * 128 * 4, S * NKV * 128 * 4
            for layer in range(L):
                batch.append_attn(layer, dq.ptr + layer * qs, dk.ptr + layer * ks, dv.ptr + layer * ks, out_d.ptr + layer * qs)
        batch.advance()
        nv.check(nv.lib.dev_sync())
        assert batch.device_status() == 0
        want = ob.decode_step(sh, pk, pv, tables, eng.nb, pos, q, k, v, cs, sn, exact=True)
        got = out_d.download(np.float32).reshape(L, S, NH, 128)
        assert np.array_equal(bits(dk.download(np.float32)), bits(k.ravel())), "k rotated in place"
        for i in range(S):
            assert_attn_close(got[:, i], want[:, i], f"kb {kb} step {step} session {i} n_keys {pos[i] + 1}")
        pos = [p + 1 for p in pos]
    gk, gv = eng.read_pools()
    assert np.array_equal(bits(gk), bits(pk)) and np.array_equal(bits(gv), bits(pv))
    batch.close()
    eng.close()


@pytest.mark.parametrize("kb", [8, 32, 64])
def test_page_sizes_cow_cascade_partials_prefill(nv, ob, kb):
    """The rest of the path at another page size: shared prefix with a partly filled tail page (one copy-on-write per
    fork, then the cascade over the shared full pages), partial attention over page windows + log-sum-exp merge,
    chained per-layer launches and graph replay, and a prefill chunk against the oracle."""
    model, kvd, L, P, n_fork = "qwen25_7b", nv.KV_F16, 2, 600 + kb // 2, 6
    eng, ss, sh, pk, pv, cs, sn, rng = build_case(nv, ob, model, kvd, [P], L=L, seed=19 + kb, spare=n_fork + 1, kv_block=kb)
    donor = ss[0]
    forks = []
    for _ in range(n_fork):
        f = eng.session_create()
        forks.append(f)
        eng.attach_prefix(f, donor, P)
    batch = eng.batch(forks)
    try_set_kernel(nv, batch, 4 if kb >= 16 else 2)       # shared-prefix tiles on tcgen05 where the page size allows
    batch.set_cascade(1)
    batch.set_pdl(1)
    NH, NKV, S = eng.NH, eng.NKV, n_fork
    out_d = nv.DevBuf(L * S * NH * 128 * 4)
    st = nv.Stream()
    pos = [P] * S
    for step in range(6):
        q = rng.standard_normal((L, S, NH, 128)).astype(np.float32)
        k = rng.standard_normal((L, S, NKV, 128)).astype(np.float32)
        v = rng.standard_normal((L, S, NKV, 128)).astype(np.float32)
        before = {f: eng.pool.table(eng.session_slice(f)).copy() for f in forks}
        dq, dk, dv = nv.to_device(q), nv.to_device(k), nv.to_device(v)
        if step == 3:
            batch.set_cascade(0)
        batch.run_steps(1, dq.ptr, dk.ptr, dv.ptr, out_d.ptr, q.size, k.size, 1 + step % 2, st.h)
        st.sync()
        assert batch.device_status() == 0
        assert batch.shared_prefix_pages() == (0 if step >= 3 else P // kb), step
        for f in forks:
            after = eng.pool.table(eng.session_slice(f))
            for lb in np.nonzero(after != before[f])[0]:
                ob.cow_copy(sh, pk, pv, eng.nb, int(before[f][lb]), int(after[lb]))
        tables = np.stack([eng.pool.table(eng.session_slice(f)) for f in forks])
        want = ob.decode_step(sh, pk, pv, tables, eng.nb, pos, q, k, v, cs, sn, exact=True)
        assert_attn_close(out_d.download(np.float32).reshape(want.shape), want, f"kb {kb} step {step}")
        pos = [p + 1 for p in pos]
    assert eng.pool.cow_count() == n_fork
    gk, gv = eng.read_pools()
    assert np.array_equal(bits(gk), bits(pk)) and np.array_equal(bits(gv), bits(pv))
    # partial attention over page windows (the multi-GPU cut) + merge == whole attention
    batch.set_fused_append(0)
    for f, p in zip(forks, pos):
        eng.set_n_past(f, p - 1)
    batch.sync_positions()
    qq = rng.standard_normal((S, NH, 128)).astype(np.float32)
    dq = nv.to_device(qq)
    n_pages = (pos[0] + kb - 1) // kb
    ranges = [(0, 3), (3, 4), (4, n_pages // 2), (n_pages // 2, 1 << 40)]
    for kernel in (0, 1):
        batch.set_kernel(kernel)
        parts = nv.DevBuf(len(ranges) * S * NH * 130 * 4)
        for i, (a, b) in enumerate(ranges):
            batch.attn_partial(0, dq.ptr, a, b, parts.ptr + i * S * NH * 130 * 4)
        merged = nv.DevBuf(S * NH * 128 * 4)
        nv.check(nv.lib.nova_lse_combine(parts.ptr, len(ranges), S * NH, 128, merged.ptr, None))
        nv.check(nv.lib.dev_sync())
        got = merged.download(np.float32).reshape(S, NH, 128)
        for i, f in enumerate(forks):
            want = ob.attn_decode_paged(sh, qq[i], pk, pv, eng.pool.table(eng.session_slice(f)), 0, eng.nb, pos[i], exact=True)
            assert_attn_close(got[i], want, f"kb {kb} kernel {kernel} windows, session {i}")
    for f, p in zip(forks, pos):
        eng.set_n_past(f, p)
    batch.sync_positions()
    # a prefill chunk on the same sessions (both kernels write the same rows; the second one re-writes them)
    n_tok = 37
    for kernel in ((1, 3, 0) if kb >= 16 else (1, 0)):
        batch.set_kernel(min(kernel, 1))
        batch.set_prefill_kernel(1 if kernel == 3 else 0) if kernel else None
        q = rng.standard_normal((L, S, n_tok, NH, 128)).astype(np.float32)
        k = rng.standard_normal((L, S, n_tok, NKV, 128)).astype(np.float32)
        v = rng.standard_normal((L, S, n_tok, NKV, 128)).astype(np.float32)
        for layer in range(L):
            dq, dk, dv = nv.to_device(q[layer]), nv.to_device(k[layer]), nv.to_device(v[layer])
            do = nv.DevBuf(q[layer].nbytes)
            batch.prefill(layer, n_tok, dq.ptr, dk.ptr, dv.ptr, do.ptr)
            nv.check(nv.lib.dev_sync())
            got = do.download(np.float32).reshape(S, n_tok, NH, 128)
            for i, f in enumerate(forks):
                table = eng.pool.table(eng.session_slice(f))
                qi, ki = q[layer, i].copy(), k[layer, i].copy()
                ob.rope_append_paged(sh, pk, pv, table, layer, eng.nb, n_tok, pos[i], qi, ki, v[layer, i], cs, sn)
                want = ob.attn_prefill_paged(sh, qi, pk, pv, table, layer, eng.nb, n_tok, pos[i])
                assert_attn_close(got[i], want, f"kb {kb} prefill kernel {kernel} layer {layer} session {i}")
        assert batch.device_status() == 0
        gk, gv = eng.read_pools()
        assert np.array_equal(bits(gk), bits(pk)) and np.array_equal(bits(gv), bits(pv))
    st.close()
    batch.close()
    eng.close()


@pytest.mark.parametrize("tc5", [0, 1])
@pytest.mark.parametrize("kb,window", [(16, 64), (16, 1000), (32, 100), (8, 50)])
def test_sliding_window_prefill(nv, ob, kb, window, tc5):
    """Sliding-window prefill (MaskKind::CausalSWA, flash_paged_kernel<true>, src/kernel/attn.cu:317: a query at
    position p sees keys max(0, p - W + 1) .. p) against the oracle's restatement of that instantiation; sessions
    shorter and longer than the window, chunks that start inside and beyond it.  No model of the reference selects
    this mask, so the reference's own launcher cannot be built with it; the oracle is the checker."""
    eng, ss, sh, pk, pv, cs, sn, rng = build_case(nv, ob, "qwen25_7b", nv.KV_F16, [700, 20, 0], L=2, seed=3 + kb,
                                                  kv_block=kb, extra_ctx=200)
    L, S, NH, NKV = eng.L, 3, eng.NH, eng.NKV
    batch = eng.batch(ss)
    try_set_kernel(nv, batch, 1)
    if tc5:
        if kb < 16:
            assert nv.lib.nova_batch_set_prefill_kernel(batch.h, 1) == nv.ERR_UNSUPPORTED     # 8-token pages stay on mma.sync
            pytest.skip("the tcgen05 prefill takes pages of 16 tokens or more")
        batch.set_prefill_kernel(1)
    else:
        batch.set_prefill_kernel(0)
    batch.set_window(window)
    pos = [700, 20, 0]
    for n_tok in (45, 70):
        q = rng.standard_normal((L, S, n_tok, NH, 128)).astype(np.float32)
        k = rng.standard_normal((L, S, n_tok, NKV, 128)).astype(np.float32)
        v = rng.standard_normal((L, S, n_tok, NKV, 128)).astype(np.float32)
        for layer in range(L):
            dq, dk, dv = nv.to_device(q[layer]), nv.to_device(k[layer]), nv.to_device(v[layer])
            do = nv.DevBuf(q[layer].nbytes)
            batch.prefill(layer, n_tok, dq.ptr, dk.ptr, dv.ptr, do.ptr)
            nv.check(nv.lib.dev_sync())
            got = do.download(np.float32).reshape(S, n_tok, NH, 128)
            for i, s in enumerate(ss):
                table = eng.pool.table(eng.session_slice(s))
                qi, ki = q[layer, i].copy(), k[layer, i].copy()
                ob.rope_append_paged(sh, pk, pv, table, layer, eng.nb, n_tok, pos[i], qi, ki, v[layer, i], cs, sn)
                want = ob.attn_prefill_paged(sh, qi, pk, pv, table, layer, eng.nb, n_tok, pos[i], window=window)
                assert_attn_close(got[i], want, f"window {window} n={n_tok} layer {layer} session {i}")
                if pos[i] + n_tok > window + 5:       # the window really cuts keys off: the causal result differs
                    full = ob.attn_prefill_paged(sh, qi, pk, pv, table, layer, eng.nb, n_tok, pos[i])
                    assert rel_l2(got[i], full) > 1e-2
        batch.advance_by(n_tok)
        pos = [p + n_tok for p in pos]
    assert batch.device_status() == 0
    batch.set_kernel(0)
    d = nv.DevBuf(S * 4 * NH * 128 * 4)
    assert nv.lib.nova_batch_prefill(batch.h, 0, 4, d.ptr, d.ptr, d.ptr, d.ptr, None) == nv.ERR_UNSUPPORTED
    gk, gv = eng.read_pools()
    assert np.array_equal(bits(gk), bits(pk)) and np.array_equal(bits(gv), bits(pv))
    batch.close()
    eng.close()
