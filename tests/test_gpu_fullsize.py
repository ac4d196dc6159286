"""Config 2 at its full size (7B-shaped, 8 sessions, contexts uniform in [2048, 8192], 28 layers, permuted
pages; ~4 GB of pools), checked through properties that need no full-size oracle run:
  * pages written by the context fill and by a fused decode step are bit-identical to the oracle's RoPE of the
    same seeded rows (sampled positions, every layer);
  * the tensor-core and SIMT kernels agree; per-layer and all-layer launches agree;
  * attention over a session == log-sum-exp merge of attention over any split of its pages;
  * one (layer, session) slice is checked against the exact CPU softmax on the downloaded pages."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
REL_TOL, ABS_TOL = 2e-3, 1e-2


def rel_l2(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / max(np.linalg.norm(b), 1e-30))


@pytest.fixture(scope="module")
def work(nv):
    import conflux_nova_b200.workloads as wl
    seed = 0x5EED0001
    lens = wl.context_lengths(seed, 8, 2048, 8192)
    w = wl.Workload("qwen25_7b", lens, seed=seed, steps=16)
    yield w
    w.close()


def test_fullsize_pages_and_kernels(nv, ob, work):
    import conflux_nova_b200.workloads as wl
    eng, batch = work.eng, work.batch
    L, S, NH, NKV = eng.L, len(work.sessions), eng.NH, eng.NKV
    cs, sn = eng.rope_tables()
    sh = ob.shape(1, NH, NKV, ob.KV_F16)
    row = NKV * 128
    rng = np.random.default_rng(0)
    # --- cached context: sampled rows against the oracle's append of the same seeded values
    for si, s in enumerate(work.sessions):
        table = eng.pool.table(eng.session_slice(s))
        for layer in (0, 13, 27):
            for pos in [0, 15, 16, work.ctx_lens[si] - 1] + rng.integers(0, work.ctx_lens[si], 3).tolist():
                k = ob.synth_normal(row, ob.synth_key(work.seed, wl.T_K, work.key_ids[si], layer), pos * row).reshape(1, NKV, 128)
                v = ob.synth_normal(row, ob.synth_key(work.seed, wl.T_V, work.key_ids[si], layer), pos * row).reshape(1, NKV, 128)
                # a one-page oracle pool: every logical block of the table points at page 0
                blk = pos >> 4
                tb = np.zeros(blk + 1, np.int32)
                pk2, pv2 = ob.new_pools(sh, 1)
                ob.rope_append_paged(sh, pk2, pv2, tb, 0, 1, 1, pos, np.zeros((1, NH, 128), np.float32), k, v, cs, sn)
                got_k = eng.read_page("k", layer, table[blk])[pos & 15]
                got_v = eng.read_page("v", layer, table[blk])[pos & 15]
                assert np.array_equal(got_k.view(np.uint16), pk2[0, 0, pos & 15].view(np.uint16)), (si, layer, pos)
                assert np.array_equal(got_v.view(np.uint16), pv2[0, 0, pos & 15].view(np.uint16)), (si, layer, pos)
    # --- one decode step, three ways
    dq, dk, dv = work.device_step_inputs(0)
    hq, hk, hv = (b.download(np.float32) for b in (dq, dk, dv))
    nq = hq.size
    outs = {}
    for name, kernel, fused, per_layer in (("simt", 0, 0, 0), ("mma", 1, 0, 1), ("mma_fused", 1, 1, 0)):
        batch.set_kernel(kernel)
        batch.set_fused_append(fused) if kernel == 1 else None
        q, k, v = nv.to_device(hq), nv.to_device(hk), nv.to_device(hv)
        o = nv.DevBuf(nq * 4)
        if per_layer:
            qs, ks = S * NH * 128 * 4, S * NKV * 128 * 4
            for l in range(L):
                batch.append_attn(l, q.ptr + l * qs, k.ptr + l * ks, v.ptr + l * ks, o.ptr + l * qs)
        else:
            batch.step_all_layers(q.ptr, k.ptr, v.ptr, o.ptr)
        nv.check(nv.lib.dev_sync())
        assert batch.device_status() == 0
        outs[name] = o.download(np.float32).reshape(L, S, NH, 128)
        rot_k = k.download(np.float32).reshape(L, S, NKV, 128)
        for b in (q, k, v, o):
            b.free()
    for name in ("mma", "mma_fused"):
        r, m = rel_l2(outs[name], outs["simt"]), float(np.abs(outs[name] - outs["simt"]).max())
        assert r <= REL_TOL and m <= ABS_TOL, (name, r, m)
    # appended rows (written three times with the same values): bit-exact against the oracle's rotation
    hk4, hv4 = hk.reshape(L, S, NKV, 128), hv.reshape(L, S, NKV, 128)
    for si, s in enumerate(work.sessions):
        pos = work.ctx_lens[si]
        table = eng.pool.table(eng.session_slice(s))
        for layer in (0, 27):
            kk = hk4[layer, si].copy().reshape(1, NKV, 128)
            tb = np.zeros((pos >> 4) + 1, np.int32)
            pk, pv = ob.new_pools(sh, 1)
            ob.rope_append_paged(sh, pk, pv, tb, 0, 1, 1, pos, np.zeros((1, NH, 128), np.float32), kk,
                                 hv4[layer, si].reshape(1, NKV, 128), cs, sn)
            assert np.array_equal(eng.read_page("k", layer, table[pos >> 4])[pos & 15].view(np.uint16),
                                  pk[0, 0, pos & 15].view(np.uint16))
            assert np.array_equal(rot_k[layer, si].view(np.uint32), kk[0].view(np.uint32))     # k rotated in place
    # --- exact CPU softmax for one (layer, session) on the downloaded pages
    layer, si = 9, 4
    n_keys = work.ctx_lens[si] + 1
    n = eng.nb * eng.page_bytes // 2
    off = layer * eng.nb * eng.page_bytes
    shp = (1, eng.nb, 16, NKV, 128)
    pk = nv.download_ptr(eng.k_base + off, np.float16, n).reshape(shp)
    pv = nv.download_ptr(eng.v_base + off, np.float16, n).reshape(shp)
    q_rot = hq.reshape(L, S, NH, 128)[layer, si].copy().reshape(1, NH, 128)
    kdummy = np.zeros((1, NKV, 128), np.float32)
    ob.oracle().oracle_rope_batch(C.byref(sh), q_rot.ctypes.data, kdummy.ctypes.data, 1, work.ctx_lens[si],
                                  cs.ctypes.data, sn.ctypes.data, 1)
    want = ob.attn_decode_paged(sh, q_rot[0], pk, pv, eng.pool.table(eng.session_slice(work.sessions[si])), 0, eng.nb,
                                n_keys, exact=True)
    for name in outs:
        r, m = rel_l2(outs[name][layer, si], want), float(np.abs(outs[name][layer, si] - want).max())
        assert r <= REL_TOL and m <= ABS_TOL, (name, r, m)
    # --- split invariance at full size (tensor-core kernel): any page split merges to the whole
    batch.set_kernel(1)
    batch.set_fused_append(0)
    q = nv.to_device(np.ascontiguousarray(hq.reshape(L, S, NH, 128)))
    qs = S * NH * 128 * 4
    # q on the device is un-rotated here; rotate layer 9's q through the append path of a scratch k (positions = n_past)
    kk, vv = nv.to_device(hk), nv.to_device(hv)
    ranges = [(0, 100), (100, 101), (101, 333), (333, 1 << 30)]
    parts = nv.DevBuf(len(ranges) * S * NH * 130 * 4)
    whole = nv.DevBuf(S * NH * 128 * 4)
    ks = S * NKV * 128 * 4
    batch.append(layer, q.ptr + layer * qs, kk.ptr + layer * ks, vv.ptr + layer * ks)      # rotates q in place, rewrites the same row
    batch.attn(layer, q.ptr + layer * qs, whole.ptr)
    for i, (a, b) in enumerate(ranges):
        batch.attn_partial(layer, q.ptr + layer * qs, a, b, parts.ptr + i * S * NH * 130 * 4)
    merged = nv.DevBuf(S * NH * 128 * 4)
    nv.check(nv.lib.nova_lse_combine(parts.ptr, len(ranges), S * NH, 128, merged.ptr, None))
    nv.check(nv.lib.dev_sync())
    a, b = merged.download(np.float32), whole.download(np.float32)
    # P is rounded to fp16 relative to each range's own running maximum, so the two differ at the 1e-4 level
    assert rel_l2(a, b) < 1e-3 and np.abs(a - b).max() < 1e-3
    assert rel_l2(b.reshape(S, NH, 128)[si], want) <= REL_TOL


# ------------------------------------------------------------------------------------------------------------
def _oracle_row(ob, wl, work, sh, cs, sn, key_session, layer, pos):
    """K and V row of one position as the context fill wrote it: seeded values, K rotated by the oracle."""
    NH, NKV = work.eng.NH, work.eng.NKV
    row = NKV * 128
    k = ob.synth_normal(row, ob.synth_key(work.seed, wl.T_K, key_session, layer), pos * row).reshape(1, NKV, 128)
    v = ob.synth_normal(row, ob.synth_key(work.seed, wl.T_V, key_session, layer), pos * row).reshape(1, NKV, 128)
    tb = np.zeros((pos >> 4) + 1, np.int32)              # a one-page oracle pool
    pk, pv = ob.new_pools(sh, 1)
    ob.rope_append_paged(sh, pk, pv, tb, 0, 1, 1, pos, np.zeros((1, NH, 128), np.float32), k, v, cs, sn)
    return pk[0, 0, pos & 15], pv[0, 0, pos & 15]


def _layer_pools(nv, eng, layer):
    n = eng.nb * eng.page_bytes // 2
    off = layer * eng.nb * eng.page_bytes
    shp = (1, eng.nb, 16, eng.NKV, 128)
    return (nv.download_ptr(eng.k_base + off, np.float16, n).reshape(shp),
            nv.download_ptr(eng.v_base + off, np.float16, n).reshape(shp))


def _exact_slice(nv, ob, eng, sh1, hq_layer_session, cs, sn, layer, session, pos):
    """Exact (float64 softmax) attention of one session in one layer on the pages as they are on the device;
    the query arrives un-rotated and is rotated at `pos` by the oracle."""
    pk, pv = _layer_pools(nv, eng, layer)
    q_rot = hq_layer_session.copy().reshape(1, eng.NH, 128)
    kdummy = np.zeros((1, eng.NKV, 128), np.float32)
    ob.oracle().oracle_rope_batch(C.byref(sh1), q_rot.ctypes.data, kdummy.ctypes.data, 1, pos, cs.ctypes.data,
                                  sn.ctypes.data, 1)
    return ob.attn_decode_paged(sh1, q_rot[0], pk, pv, eng.pool.table(eng.session_slice(session)), 0, eng.nb, pos + 1,
                                exact=True)


def test_fullsize_config3_shared_prefix(nv, ob):
    """Config 3 at its full size: a donor with a 4088-token prefix (255 full pages + a half-filled tail page), 32
    sessions that attach it and take 512 private tokens each, 28 layers.  Exactly one copy-on-write per session
    (on its first private write, into the shared tail page) and none afterwards; the donor owns its tail page alone
    again and its contents did not change; the copied page carries the donor's rows and then the session's own;
    decode steps with the shared pages attended once for all sessions (per-layer launches and graph replay) agree
    with the plain per-session path, and one (layer, session) slice agrees with the exact CPU softmax."""
    import conflux_nova_b200.workloads as wl
    P, n_priv, S = 4088, 512, 32
    seed = 0x5EED0002
    work = wl.Workload("qwen25_7b", [P + n_priv] * S, seed=seed, steps=16, shared_prefix=P)
    eng, batch = work.eng, work.batch
    L, NH, NKV = eng.L, eng.NH, eng.NKV
    cs, sn = eng.rope_tables()
    sh1 = ob.shape(1, NH, NKV, ob.KV_F16)
    try:
        assert work.cow_at_build == S and eng.pool.cow_count() == S          # once per session, at the first private write
        donor_table = eng.pool.table(eng.session_slice(work.donor))
        tail = int(donor_table[(P - 1) >> 4])
        assert eng.pool.refcnt(tail) == 1                                      # the donor owns its tail page again
        for p in range(P >> 4):
            assert eng.pool.refcnt(int(donor_table[p])) == S + 1               # full prefix pages: donor + every session
        rng = np.random.default_rng(1)
        for layer in (0, 11, 27):
            # donor pages (tail page included) still hold the seeded prefix rows
            for pos in [0, 4079, 4080, 4087] + rng.integers(0, P, 3).tolist():
                wk, wv = _oracle_row(ob, wl, work, sh1, cs, sn, 10 ** 6, layer, pos)
                assert np.array_equal(eng.read_page("k", layer, donor_table[pos >> 4])[pos & 15].view(np.uint16), wk.view(np.uint16))
                assert np.array_equal(eng.read_page("v", layer, donor_table[pos >> 4])[pos & 15].view(np.uint16), wv.view(np.uint16))
            for si in (0, 17, 31):
                table = eng.pool.table(eng.session_slice(work.sessions[si]))
                assert np.array_equal(table[: P >> 4], donor_table[: P >> 4])               # shared, not copied
                assert table[P >> 4] != tail and eng.pool.refcnt(int(table[P >> 4])) == 1   # the private copy of the tail page
                got_k = eng.read_page("k", layer, table[P >> 4])
                donor_k = eng.read_page("k", layer, tail)
                assert np.array_equal(got_k[: P & 15].view(np.uint16), donor_k[: P & 15].view(np.uint16))   # rows copied by the COW
                for pos in (P, P + 7, P + 8, P + n_priv - 1):                   # the session's own rows
                    wk, wv = _oracle_row(ob, wl, work, sh1, cs, sn, work.key_ids[si], layer, pos)
                    assert np.array_equal(eng.read_page("k", layer, table[pos >> 4])[pos & 15].view(np.uint16), wk.view(np.uint16))
                    assert np.array_equal(eng.read_page("v", layer, table[pos >> 4])[pos & 15].view(np.uint16), wv.view(np.uint16))
        # --- decode steps: cascade (per layer, graph) against the plain path on the same step
        batch.set_kernel(1)
        batch.set_fused_append(1)
        batch.set_pdl(1)
        st = nv.Stream()
        nq, nk = work.step_input_sizes()
        out_a, out_b = nv.DevBuf(nq * 4), nv.DevBuf(nq * 4)
        for step, mode in ((0, 1), (1, 2)):
            dq, dk, dv = work.device_step_inputs(step)
            hq, hk, hv = (b.download(np.float32) for b in (dq, dk, dv))
            n0 = [eng.n_past(s) for s in work.sessions]
            batch.set_cascade(1)
            batch.run_steps(1, dq.ptr, dk.ptr, dv.ptr, out_a.ptr, nq, nk, mode, st.h)
            st.sync()
            assert batch.device_status() == 0
            assert batch.shared_prefix_pages() == P >> 4
            assert eng.pool.cow_count() == S                                    # no further copy-on-write
            a = out_a.download(np.float32).reshape(L, S, NH, 128)
            # the same step again, plain: positions back, inputs fresh (k was rotated in place)
            for s, n in zip(work.sessions, n0):
                eng.set_n_past(s, n)
            batch.sync_positions()
            batch.set_cascade(0)
            for b_, h in ((dq, hq), (dk, hk), (dv, hv)):
                b_.upload(h)
            batch.run_steps(1, dq.ptr, dk.ptr, dv.ptr, out_b.ptr, nq, nk, 1, st.h)
            st.sync()
            assert batch.device_status() == 0 and batch.shared_prefix_pages() == 0
            b = out_b.download(np.float32).reshape(L, S, NH, 128)
            r, m = rel_l2(a, b), float(np.abs(a - b).max())
            assert r <= REL_TOL and m <= ABS_TOL, ("cascade vs plain", step, r, m)
            layer, si = (5, 3) if step == 0 else (27, 30)
            want = _exact_slice(nv, ob, eng, sh1, hq.reshape(L, S, NH, 128)[layer, si], cs, sn, layer, work.sessions[si], n0[si])
            for name, o in (("cascade", a), ("plain", b)):
                r, m = rel_l2(o[layer, si], want), float(np.abs(o[layer, si] - want).max())
                assert r <= REL_TOL and m <= ABS_TOL, (name, step, r, m)
            for b_ in (dq, dk, dv):
                b_.free()
        st.close()
    finally:
        work.close()


def test_fullsize_config5_long_context_one_gpu(nv, ob):
    """Config 5's session (131072 cached tokens, 7B shape) on one GPU, two layers: a decode step against the exact
    CPU softmax over all 131073 keys, and split invariance - attention over the session == log-sum-exp merge of the
    partials over 2, 4 and 8 page ranges (the cut the multi-GPU split makes)."""
    import conflux_nova_b200.workloads as wl
    n_ctx, L = 131072, 2
    work = wl.Workload("qwen25_7b", [n_ctx], seed=0x5EED0004, steps=8, n_layers=L)
    eng, batch = work.eng, work.batch
    NH, NKV = eng.NH, eng.NKV
    cs, sn = eng.rope_tables()
    sh1 = ob.shape(1, NH, NKV, ob.KV_F16)
    try:
        dq, dk, dv = work.device_step_inputs(0)
        hq = dq.download(np.float32).reshape(L, 1, NH, 128)
        nq, nk = work.step_input_sizes()
        out = nv.DevBuf(nq * 4)
        outs = {}
        hk, hv = dk.download(np.float32), dv.download(np.float32)
        for name, kernel, fused in (("mma_fused", 1, 1), ("simt", 0, 0)):
            batch.set_kernel(kernel)
            if kernel == 1:
                batch.set_fused_append(fused)
            dq.upload(hq)
            dk.upload(hk)
            qs, ks = NH * 128 * 4, NKV * 128 * 4
            for l in range(L):
                batch.append_attn(l, dq.ptr + l * qs, dk.ptr + l * ks, dv.ptr + l * ks, out.ptr + l * qs)
            nv.check(nv.lib.dev_sync())
            assert batch.device_status() == 0
            outs[name] = out.download(np.float32).reshape(L, NH, 128)
        want = _exact_slice(nv, ob, eng, sh1, hq[1, 0], cs, sn, 1, work.sessions[0], n_ctx)
        for name, o in outs.items():
            r, m = rel_l2(o[1], want), float(np.abs(o[1] - want).max())
            assert r <= REL_TOL and m <= ABS_TOL, (name, r, m)
        # split invariance: q rotated in place by the plain append (rewrites the same row), then partials
        batch.set_kernel(1)
        batch.set_fused_append(0)
        dq.upload(hq)
        dk.upload(hk)
        layer = 1
        batch.append(layer, dq.ptr + layer * qs, dk.ptr + layer * ks, dv.ptr + layer * ks)
        whole = nv.DevBuf(NH * 128 * 4)
        batch.attn(layer, dq.ptr + layer * qs, whole.ptr)
        nv.check(nv.lib.dev_sync())
        w = whole.download(np.float32).reshape(NH, 128)
        n_pages = (n_ctx + 1 + 15) // 16
        for parts_n in (2, 4, 8):
            per = -(-n_pages // parts_n)
            parts = nv.DevBuf(parts_n * NH * 130 * 4)
            for r_ in range(parts_n):
                hi = (r_ + 1) * per if r_ + 1 < parts_n else 1 << 40
                batch.attn_partial(layer, dq.ptr + layer * qs, r_ * per, hi, parts.ptr + r_ * NH * 130 * 4)
            merged = nv.DevBuf(NH * 128 * 4)
            nv.check(nv.lib.nova_lse_combine(parts.ptr, parts_n, NH, 128, merged.ptr, None))
            nv.check(nv.lib.dev_sync())
            mg = merged.download(np.float32).reshape(NH, 128)
            assert rel_l2(mg, w) < 1e-3 and np.abs(mg - w).max() < 1e-3, parts_n
            r, m = rel_l2(mg, want), float(np.abs(mg - want).max())
            assert r <= REL_TOL and m <= ABS_TOL, (parts_n, r, m)
            parts.free()
            merged.free()
        assert batch.device_status() == 0
    finally:
        work.close()


def test_fullsize_14b_shape_sessions(nv, ob):
    """The 14B shape of config 4 (40 q / 8 kv heads, two kv-head groups per session) at its context length: three
    sessions x 8192 cached tokens, three layers; one decode step through each kernel against the exact CPU softmax
    of every session in the last layer, and the appended rows bit-exact."""
    import conflux_nova_b200.workloads as wl
    L, S, n_ctx = 3, 3, 8192
    work = wl.Workload("qwen25_14b", [n_ctx] * S, seed=0x5EED0003, steps=8, n_layers=L)
    eng, batch = work.eng, work.batch
    NH, NKV = eng.NH, eng.NKV
    cs, sn = eng.rope_tables()
    sh1 = ob.shape(1, NH, NKV, ob.KV_F16)
    try:
        dq, dk, dv = work.device_step_inputs(0)
        hq, hk, hv = (b.download(np.float32) for b in (dq, dk, dv))
        nq, nk = work.step_input_sizes()
        out = nv.DevBuf(nq * 4)
        st = nv.Stream()
        outs = {}
        for name, kernel, fused, mode in (("simt", 0, 0, 0), ("mma", 1, 0, 1), ("mma_fused_chain", 1, 1, 1), ("mma_fused_graph", 1, 1, 2)):
            batch.set_kernel(kernel)
            if kernel == 1:
                batch.set_fused_append(fused)
                batch.set_pdl(fused)
            for s in work.sessions:
                eng.set_n_past(s, n_ctx)
            batch.sync_positions()
            dq.upload(hq)
            dk.upload(hk)
            batch.run_steps(1, dq.ptr, dk.ptr, dv.ptr, out.ptr, nq, nk, mode, st.h)
            st.sync()
            assert batch.device_status() == 0
            outs[name] = out.download(np.float32).reshape(L, S, NH, 128)
        layer = L - 1
        for si, s in enumerate(work.sessions):
            want = _exact_slice(nv, ob, eng, sh1, hq.reshape(L, S, NH, 128)[layer, si], cs, sn, layer, s, n_ctx)
            for name, o in outs.items():
                r, m = rel_l2(o[layer, si], want), float(np.abs(o[layer, si] - want).max())
                assert r <= REL_TOL and m <= ABS_TOL, (name, si, r, m)
            # the appended row, written four times with the same values
            table = eng.pool.table(eng.session_slice(s))
            kk = hk.reshape(L, S, NKV, 128)[layer, si].copy().reshape(1, NKV, 128)
            tb = np.zeros((n_ctx >> 4) + 1, np.int32)
            pk, pv = ob.new_pools(sh1, 1)
            ob.rope_append_paged(sh1, pk, pv, tb, 0, 1, 1, n_ctx, np.zeros((1, NH, 128), np.float32), kk,
                                 hv.reshape(L, S, NKV, 128)[layer, si].reshape(1, NKV, 128), cs, sn)
            assert np.array_equal(eng.read_page("k", layer, table[n_ctx >> 4])[n_ctx & 15].view(np.uint16),
                                  pk[0, 0, n_ctx & 15].view(np.uint16))
            assert np.array_equal(eng.read_page("v", layer, table[n_ctx >> 4])[n_ctx & 15].view(np.uint16),
                                  pv[0, 0, n_ctx & 15].view(np.uint16))
        st.close()
    finally:
        work.close()


@pytest.mark.parametrize("kernel", [1, 3, 0])
def test_fullsize_prefill_chunk(nv, ob, kernel):
    """Prefill at the size the benchmark runs it: 512 new tokens per session over 2-3k cached keys (7B shape, two
    sessions, two layers; many query tiles, many pages per ring).  One (layer, session) slice against the oracle's
    restatement of flash_paged_kernel and against the reference's own launch_attn_prefill_paged
    (src/kernel/attn.cu:514-527) on an fp32 copy of the pages; first and last appended rows bit-exact."""
    import conflux_nova_b200.workloads as wl
    L, n_tok = 2, 512
    lens = [2304, 3001]
    work = wl.Workload("qwen25_7b", lens, seed=0x5EED0011, steps=n_tok + 16, n_layers=L)
    eng, batch = work.eng, work.batch
    S, NH, NKV = len(lens), eng.NH, eng.NKV
    cs, sn = eng.rope_tables()
    sh1 = ob.shape(1, NH, NKV, ob.KV_F16)
    try:
        batch.set_kernel(min(kernel, 1))
        if kernel:
            batch.set_prefill_kernel(1 if kernel == 3 else 0)      # tcgen05 + tensor memory | mma.sync tiles
        assert batch.prefill_max_tokens() >= n_tok
        rng = np.random.default_rng(5)
        q = rng.standard_normal((L, S, n_tok, NH, 128)).astype(np.float32)
        k = rng.standard_normal((L, S, n_tok, NKV, 128)).astype(np.float32)
        v = rng.standard_normal((L, S, n_tok, NKV, 128)).astype(np.float32)
        outs = []
        for layer in range(L):
            dq, dk, dv = nv.to_device(q[layer]), nv.to_device(k[layer]), nv.to_device(v[layer])
            do = nv.DevBuf(q[layer].nbytes)
            batch.prefill(layer, n_tok, dq.ptr, dk.ptr, dv.ptr, do.ptr)
            nv.check(nv.lib.dev_sync())
            outs.append(do.download(np.float32).reshape(S, n_tok, NH, 128))
            for b in (dq, dk, dv, do):
                b.free()
        assert batch.device_status() == 0
        layer, si = 1, 1
        pk, pv = _layer_pools(nv, eng, layer)
        table = eng.pool.table(eng.session_slice(work.sessions[si]))
        # the oracle's own append of the chunk gives the rotated q and the rows the pages must now hold
        opk, opv = pk.copy(), pv.copy()
        qi, ki = q[layer, si].copy(), k[layer, si].copy()
        ob.rope_append_paged(sh1, opk, opv, table, 0, eng.nb, n_tok, lens[si], qi, ki, v[layer, si], cs, sn)
        assert np.array_equal(opk.view(np.uint16), pk.view(np.uint16)) and np.array_equal(opv.view(np.uint16), pv.view(np.uint16))
        want = ob.attn_prefill_paged(sh1, qi, pk, pv, table, 0, eng.nb, n_tok, lens[si])
        got = outs[layer][si]
        r, m = rel_l2(got, want), float(np.abs(got - want).max())
        assert r <= REL_TOL and m <= ABS_TOL, ("oracle", r, m)
        for t in (0, 1, 255, 511):                                  # single query rows, not only the aggregate
            r = rel_l2(got[t], want[t])
            assert r <= REL_TOL, ("row", t, r)
        g = ob.ref_gpu("qwen25_7b")
        if g is not None and hasattr(g, "ref_gpu_attn_prefill_paged"):
            rk, rv = nv.to_device(pk.astype(np.float32)), nv.to_device(pv.astype(np.float32))
            rq, ro = nv.to_device(qi), nv.DevBuf(qi.nbytes)
            g.ref_gpu_attn_prefill_paged(rq.ptr, rk.ptr, rv.ptr, nv.lib.nova_kv_table_slot(eng.h, eng.session_slice(work.sessions[si])),
                                         0, eng.nb, n_tok, lens[si], ro.ptr, None)
            nv.check(nv.lib.dev_sync())
            assert g.ref_gpu_last_error() == 0
            ref = ro.download(np.float32).reshape(qi.shape)
            assert rel_l2(want, ref) < 2e-6                          # oracle == the reference's kernel
            r, m = rel_l2(got, ref), float(np.abs(got - ref).max())
            assert r <= REL_TOL and m <= ABS_TOL, ("reference kernel", r, m)
    finally:
        work.close()
