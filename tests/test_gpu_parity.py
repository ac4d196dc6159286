"""GPU parity (tiers T1/T2): every CUDA entry point of the path, called through the C ABI, against
the CPU oracle on the same seeded inputs, and against the reference's own CUDA kernels recompiled
for sm_100a where that library is present.  Bars: pages / tables / rotated q,k bit-exact; attention
within rel-L2 <= 2e-3 and max-abs <= 1e-2 (the tolerance the north-star states)."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

REL_TOL, ABS_TOL = 2e-3, 1e-2
SHAPES = {"qwen25_1p5b": (12, 2), "qwen25_7b": (28, 4), "qwen25_14b": (40, 8),
          "r1_llama8b": (32, 8), "r1_qwen1p5b_abl": (12, 2)}
# RoPE of the reference's other models (include/nova/model/matrix.h:52-53, include/nova/arch/traits.h:25):
# (theta, NeoX pairing)
ROPE = {"r1_llama8b": (500000, 0), "r1_qwen1p5b_abl": (10000, 1)}


def rel_l2(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / max(np.linalg.norm(b), 1e-30))


def assert_attn_close(got, want, what=""):
    r, m = rel_l2(got, want), float(np.abs(got - want).max())
    assert r <= REL_TOL and m <= ABS_TOL, (what, r, m)
    return r, m


def bits(a):
    return a.view(np.uint16 if a.dtype == np.float16 else np.uint32)


def kernels_for(nv, kv_dtype):
    return [0, 1] if kv_dtype == nv.KV_F16 else [0]


def try_set_kernel(nv, batch, which):
    """0 = SIMT, 1 = tensor-core (prefill and shared-prefix tiles on mma.sync), 2 = the same with RoPE+append fused into
    the attention launch, 3 and 4 = 1 and 2 with the prefill and the shared-prefix tiles on tcgen05 + tensor memory (the
    library's default where it applies)."""
    rc = nv.lib.nova_batch_set_kernel(batch.h, min(which, 1))
    if rc == nv.ERR_UNSUPPORTED:
        pytest.skip("kernel not built for this dtype")
    assert rc == 0
    if which in (2, 4):
        batch.set_fused_append(1)
    if which >= 3:
        batch.set_prefill_kernel(1)
    elif which >= 1:
        batch.set_prefill_kernel(0)


# --------------------------------------------------------------------------------------------
def test_synth_matches_oracle(nv, ob):
    key = nv.synth_key(0x5EED0002, 2, 5, 9)
    assert key == ob.synth_key(0x5EED0002, 2, 5, 9)
    n = 100_003
    d = nv.DevBuf(n * 4)
    nv.check(nv.lib.nova_synth_normal(d.ptr, n, key, 12345, None))
    nv.check(nv.lib.dev_sync())
    assert np.array_equal(bits(d.download(np.float32)), bits(ob.synth_normal(n, key, 12345)))


def test_hal_roundtrip(nv):
    x = np.arange(1000, dtype=np.float32)
    d = nv.to_device(x)
    assert np.array_equal(d.download(np.float32), x)
    d.zero()
    assert not d.download(np.float32).any()
    assert nv.lib.dev_alloc(0) is None
    assert nv.lib.dev_max_alloc() > (1 << 30)
    assert nv.lib.dev_count() >= 1
    s = C.c_void_p()
    assert nv.lib.dev_stream_create(C.byref(s)) == 0 and nv.lib.dev_stream_sync(s) == 0
    assert nv.lib.dev_stream_destroy(s) == 0


def test_rope_table(nv, ob):
    eng = nv.Engine(1, 12, 2, ctx=8448, n_slices=1, kv_dtype=nv.KV_F32)
    cs, sn = eng.rope_tables()
    assert cs.shape == (8448, 64) and cs[0, 0] == 1.0 and sn[0, 0] == 0.0        # tests/gpu_misc.cu:22
    i = np.arange(64, dtype=np.float64)
    ang = np.arange(8448, dtype=np.float64)[:, None] * (1e6 ** (-i / 64.0))[None, :]
    # fp32 angle rounding dominates: |d angle| <= ~2^-24 * pos
    assert np.abs(cs - np.cos(ang)).max() < 2e-3 and np.abs(sn - np.sin(ang)).max() < 2e-3
    assert np.abs(cs[:64] - np.cos(ang[:64])).max() < 1e-5
    g = ob.ref_gpu("qwen25_7b")
    if g is not None:   # the reference's rope_table_kernel, rows 0..kCtx-1, bit for bit
        n = g.ref_gpu_kctx() * 64
        rc, rs = nv.DevBuf(n * 4), nv.DevBuf(n * 4)
        g.ref_gpu_rope_table(rc.ptr, rs.ptr, None)
        nv.check(nv.lib.dev_sync())
        assert np.array_equal(bits(rc.download(np.float32)), bits(cs[: g.ref_gpu_kctx()].ravel()))
        assert np.array_equal(bits(rs.download(np.float32)), bits(sn[: g.ref_gpu_kctx()].ravel()))
    eng.close()


@pytest.mark.parametrize("model", list(SHAPES))
@pytest.mark.parametrize("dtype", ["f32", "f16"])
def test_append_bit_exact_vs_oracle(nv, ob, model, dtype):
    NH, NKV = SHAPES[model]
    kvd = nv.KV_F16 if dtype == "f16" else nv.KV_F32
    L, ctx = 3, 160
    eng = nv.Engine(L, NH, NKV, ctx=ctx, n_slices=3, kv_dtype=kvd)
    rng = np.random.default_rng(11)
    ss = [eng.session_create() for _ in range(3)]
    for s in ss:
        eng.permute_pages(s, rng.permutation(eng.nblocks))
    cs, sn = eng.rope_tables()
    sh = ob.shape(L, NH, NKV, kvd)
    pk, pv = ob.new_pools(sh, eng.nb)
    shp = eng.shape()
    # multi-token appends that start mid-page and cross page boundaries, in every layer
    for s, (pos0, n) in zip(ss, [(0, 37), (5, 16), (15, 70)]):
        table = eng.pool.table(eng.session_slice(s))
        for layer in range(L):
            q = rng.standard_normal((n, NH, 128)).astype(np.float32)
            k = rng.standard_normal((n, NKV, 128)).astype(np.float32)
            v = rng.standard_normal((n, NKV, 128)).astype(np.float32)
            dq, dk, dv = nv.to_device(q), nv.to_device(k), nv.to_device(v)
            nv.check(nv.lib.nova_launch_rope_append_paged(
                C.byref(shp), eng.k_base, eng.v_base, nv.lib.nova_kv_table_slot(eng.h, eng.session_slice(s)),
                layer, eng.nb, n, pos0, dq.ptr, dk.ptr, dv.ptr, nv.lib.nova_rope_cos(eng.h),
                nv.lib.nova_rope_sin(eng.h), None))
            nv.check(nv.lib.dev_sync())
            ob.rope_append_paged(sh, pk, pv, table, layer, eng.nb, n, pos0, q, k, v, cs, sn)
            assert np.array_equal(bits(dq.download(np.float32)), bits(q.ravel())), "rotated q"
            assert np.array_equal(bits(dk.download(np.float32)), bits(k.ravel())), "rotated k"
    gk, gv = eng.read_pools()
    assert np.array_equal(bits(gk), bits(pk)) and np.array_equal(bits(gv), bits(pv))
    eng.close()


@pytest.mark.parametrize("model", ["qwen25_1p5b", "qwen25_7b"])
def test_append_vs_reference_kernels(nv, ob, model):
    """rope_batch_kernel + kv_store_paged_kernel of the reference (fp32 pools) against the fused
    kernel: fp32 pages identical, fp16 pages == round-to-nearest-even of the reference's."""
    g = ob.ref_gpu(model)
    if g is None:
        pytest.skip("reference CUDA library not built")
    NH, NKV = SHAPES[model]
    L, ctx, n, pos0, layer = 2, 4096, 300, 1000, 1
    rng = np.random.default_rng(5)
    q = rng.standard_normal((n, NH, 128)).astype(np.float32)
    k = rng.standard_normal((n, NKV, 128)).astype(np.float32)
    v = rng.standard_normal((n, NKV, 128)).astype(np.float32)
    res = {}
    for kvd in (nv.KV_F32, nv.KV_F16):
        eng = nv.Engine(L, NH, NKV, ctx=ctx, n_slices=1, kv_dtype=kvd, rope_positions=4096)
        s = eng.session_create()
        perm = np.random.default_rng(6).permutation(eng.nblocks)
        eng.permute_pages(s, perm)
        tab = nv.lib.nova_kv_table_slot(eng.h, eng.session_slice(s))
        dq, dk, dv = nv.to_device(q), nv.to_device(k), nv.to_device(v)
        shp = eng.shape()
        nv.check(nv.lib.nova_launch_rope_append_paged(C.byref(shp), eng.k_base, eng.v_base, tab, layer, eng.nb, n, pos0,
                                                      dq.ptr, dk.ptr, dv.ptr, nv.lib.nova_rope_cos(eng.h),
                                                      nv.lib.nova_rope_sin(eng.h), None))
        nv.check(nv.lib.dev_sync())
        res[kvd] = (eng.read_pools(), dq.download(np.float32), dk.download(np.float32))
        if kvd == nv.KV_F32:
            # the reference on its own tables and an fp32 pool of the same geometry
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


@pytest.mark.parametrize("model", ["r1_llama8b", "r1_qwen1p5b_abl"])
def test_other_rope_layouts_vs_reference_kernels(nv, ob, model):
    """The reference's other RoPE variants - adjacent pairs (2i, 2i+1) with theta 500000 (R1-Llama-8B,
    include/nova/arch/traits.h:25, model/matrix.h:53) and NeoX pairs with theta 10000 (the abliterated 1.5B,
    matrix.h:52) - against the reference's own kernels compiled for those models: cos/sin tables, rotated q/k and
    appended fp32 pages bit-identical; fp16 pages == round-to-nearest-even of the reference's; decode attention
    (batched calls, every kernel that the layout allows) within tolerance of the reference's kernel."""
    g = ob.ref_gpu(model)
    if g is None:
        pytest.skip("reference CUDA library not built")
    NH, NKV = SHAPES[model]
    theta, neox = ROPE[model]
    shape6 = (C.c_int32 * 6)()
    g.ref_gpu_shape(shape6)
    assert (shape6[1], shape6[2], shape6[5]) == (NH, NKV, theta)
    L, ctx, n, pos0, layer = 2, 4096, 200, 3000, 1
    rng = np.random.default_rng(11)
    q = rng.standard_normal((n, NH, 128)).astype(np.float32)
    k = rng.standard_normal((n, NKV, 128)).astype(np.float32)
    v = rng.standard_normal((n, NKV, 128)).astype(np.float32)
    rcs, rsn = nv.DevBuf(4096 * 64 * 4), nv.DevBuf(4096 * 64 * 4)
    g.ref_gpu_rope_table(rcs.ptr, rsn.ptr, None)
    nv.check(nv.lib.dev_sync())
    ref_cs, ref_sn = rcs.download(np.float32).reshape(4096, 64), rsn.download(np.float32).reshape(4096, 64)
    ocs, osn = ob.rope_table(4096, 128, theta)          # the host libm is not the GPU's: close, not identical
    assert np.abs(ocs - ref_cs).max() < 2e-3 and np.abs(osn - ref_sn).max() < 2e-3
    assert ref_cs[0, 0] == 1.0 and ref_sn[0, 0] == 0.0
    res = {}
    for kvd in (nv.KV_F32, nv.KV_F16):
        eng = nv.Engine(L, NH, NKV, ctx=ctx, n_slices=1, kv_dtype=kvd, rope_positions=4096, rope_theta=theta,
                        rope_neox=neox)
        cs, sn = eng.rope_tables()
        assert np.array_equal(bits(cs), bits(ref_cs)) and np.array_equal(bits(sn), bits(ref_sn))
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
            rpk = nv.DevBuf(L * eng.nb * eng.page_bytes).zero()
            rpv = nv.DevBuf(L * eng.nb * eng.page_bytes).zero()
            rq, rk, rv = nv.to_device(q), nv.to_device(k), nv.to_device(v)
            g.ref_gpu_rope_batch(rq.ptr, rk.ptr, n, pos0, rcs.ptr, rsn.ptr, None)
            g.ref_gpu_kv_store_paged(rpk.ptr, rpv.ptr, tab, layer, eng.nb, n, pos0, rk.ptr, rv.ptr, None)
            nv.check(nv.lib.dev_sync())
            assert g.ref_gpu_last_error() == 0
            ref = (rpk.download(np.float32), rpv.download(np.float32), rq.download(np.float32), rk.download(np.float32))
            # the oracle's rotation of the same rows (its non-NeoX branch) is the reference's too
            sh = ob.shape(L, NH, NKV, ob.KV_F32, rope_neox=neox)
            opk, opv = ob.new_pools(sh, eng.nb)
            oq, ok_ = q.copy(), k.copy()
            ob.rope_append_paged(sh, opk, opv, eng.pool.table(eng.session_slice(s)), layer, eng.nb, n, pos0, oq, ok_, v,
                                 cs, sn)
            assert np.array_equal(bits(oq.ravel()), bits(ref[2])) and np.array_equal(bits(ok_.ravel()), bits(ref[3]))
            assert np.array_equal(bits(opk.ravel()), bits(ref[0]))
        eng.close()
    (k32, v32), q32, kk32 = res[nv.KV_F32]
    assert np.array_equal(bits(q32), bits(ref[2])) and np.array_equal(bits(kk32), bits(ref[3]))
    assert np.array_equal(bits(k32.ravel()), bits(ref[0])) and np.array_equal(bits(v32.ravel()), bits(ref[1]))
    (k16, v16), _, _ = res[nv.KV_F16]
    assert np.array_equal(bits(k16.ravel()), bits(ref[0].astype(np.float16)))
    assert np.array_equal(bits(v16.ravel()), bits(ref[1].astype(np.float16)))
    # decode steps through the batched calls with this layout: append kernel + attention, and where the layout
    # allows it the fused launch; attention against the reference's own kernel on an fp32 copy of the pages
    for kernel in (0, 1, 2):
        if kernel == 2 and not neox:
            continue                                      # the fused append is a NeoX-pairs path
        eng, ss, sh, pk, pv, cs, sn, rng2 = build_case(nv, ob, model, nv.KV_F16, [333, 16], L=2, seed=77)
        S = len(ss)
        batch = eng.batch(ss)
        try_set_kernel(nv, batch, kernel)
        tables = np.stack([eng.pool.table(eng.session_slice(x)) for x in ss])
        pos = [333, 16]
        out_d = nv.DevBuf(2 * S * NH * 128 * 4)
        for step in range(2):
            qq = rng2.standard_normal((2, S, NH, 128)).astype(np.float32)
            kk = rng2.standard_normal((2, S, NKV, 128)).astype(np.float32)
            vv = rng2.standard_normal((2, S, NKV, 128)).astype(np.float32)
            dq, dk, dv = nv.to_device(qq), nv.to_device(kk), nv.to_device(vv)
            batch.step_all_layers(dq.ptr, dk.ptr, dv.ptr, out_d.ptr)
            batch.advance()
            nv.check(nv.lib.dev_sync())
            assert batch.device_status() == 0
            want = ob.decode_step(sh, pk, pv, tables, eng.nb, pos, qq, kk, vv, cs, sn, exact=True)   # rotates qq, kk
            got = out_d.download(np.float32).reshape(2, S, NH, 128)
            assert_attn_close(got, want, f"{model} kernel {kernel} step {step}")
            assert np.array_equal(bits(dk.download(np.float32)), bits(kk.ravel())), "k rotated in place"
            # the reference's attention on the same pages (fp32 copies of the fp16 values), layer 1, session 0
            rk, rv = nv.to_device(pk.astype(np.float32)), nv.to_device(pv.astype(np.float32))
            rq = nv.to_device(qq[1, 0])
            ro, scr = nv.DevBuf(NH * 128 * 4), nv.DevBuf(NH * 32 * 130 * 4)
            g.ref_gpu_attn_decode_paged(rq.ptr, rk.ptr, rv.ptr, nv.lib.nova_kv_table_slot(eng.h, eng.session_slice(ss[0])),
                                        1, eng.nb, pos[0] + 1, ro.ptr, scr.ptr, None)
            nv.check(nv.lib.dev_sync())
            assert g.ref_gpu_last_error() == 0
            assert_attn_close(got[1, 0], ro.download(np.float32).reshape(NH, 128), "vs reference attention kernel")
            pos = [p + 1 for p in pos]
        gk, gv = eng.read_pools()
        assert np.array_equal(bits(gk), bits(pk)) and np.array_equal(bits(gv), bits(pv))
        batch.close()
        eng.close()


def build_case(nv, ob, model, kvd, ctx_lens, L=2, seed=21, spare=0, kv_block=16, extra_ctx=40):
    """Engine + sessions with permuted tables and random cached context, mirrored in numpy pools."""
    NH, NKV = SHAPES[model]
    theta, neox = ROPE.get(model, (1000000, 1))
    ctx = ((max(ctx_lens) + extra_ctx + 63) // 64) * 64
    eng = nv.Engine(L, NH, NKV, ctx=ctx, n_slices=len(ctx_lens) + spare, kv_dtype=kvd, rope_theta=theta, rope_neox=neox,
                    kv_block=kv_block)
    rng = np.random.default_rng(seed)
    sh = ob.shape(L, NH, NKV, kvd, rope_neox=neox, kv_block=kv_block)
    pk, pv = ob.new_pools(sh, eng.nb)
    cs, sn = eng.rope_tables()
    shp = eng.shape()
    ss = []
    for n in ctx_lens:
        s = eng.session_create()
        ss.append(s)
        eng.permute_pages(s, rng.permutation(eng.nblocks))
        if n == 0:
            continue
        table = eng.pool.table(eng.session_slice(s))
        for layer in range(L):
            k = rng.standard_normal((n, NKV, 128)).astype(np.float32)
            v = rng.standard_normal((n, NKV, 128)).astype(np.float32)
            dk, dv = nv.to_device(k), nv.to_device(v)
            nv.check(nv.lib.nova_launch_rope_append_paged(
                C.byref(shp), eng.k_base, eng.v_base, nv.lib.nova_kv_table_slot(eng.h, eng.session_slice(s)), layer,
                eng.nb, n, 0, None, dk.ptr, dv.ptr, nv.lib.nova_rope_cos(eng.h), nv.lib.nova_rope_sin(eng.h), None))
            qd = np.zeros((n, NH, 128), np.float32)
            ob.rope_append_paged(sh, pk, pv, table, layer, eng.nb, n, 0, qd, k, v, cs, sn)
        eng.set_n_past(s, n)
    nv.check(nv.lib.dev_sync())
    return eng, ss, sh, pk, pv, cs, sn, rng


@pytest.mark.parametrize("kernel", [0, 1, 2])
@pytest.mark.parametrize("model,dtype", [("qwen25_1p5b", "f16"), ("qwen25_7b", "f16"), ("qwen25_14b", "f16"),
                                         ("qwen25_7b", "f32"), ("qwen25_1p5b", "f32")])
def test_decode_steps_vs_oracle(nv, ob, model, dtype, kernel):
    """Sessions of ragged lengths (a fresh one, page-boundary cases, a long one), three decode steps
    per-layer and all-layers: pages bit-exact, attention within tolerance of the exact softmax."""
    kvd = nv.KV_F16 if dtype == "f16" else nv.KV_F32
    # (kernels 1 and 2 on fp32 pools: the tensor-core kernel converts the rows to fp16 on the way in)
    ctx_lens = [0, 1, 15, 16, 17, 31, 33, 100, 255, 1024, 1500]
    eng, ss, sh, pk, pv, cs, sn, rng = build_case(nv, ob, model, kvd, ctx_lens)
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
                if kernel == 2:
                    batch.append_attn(layer, dq.ptr + layer * qs, dk.ptr + layer * ks, dv.ptr + layer * ks,
                                      out_d.ptr + layer * qs)
                else:
                    batch.append(layer, dq.ptr + layer * qs, dk.ptr + layer * ks, dv.ptr + layer * ks)
                    batch.attn(layer, dq.ptr + layer * qs, out_d.ptr + layer * qs)
        batch.advance()
        nv.check(nv.lib.dev_sync())
        assert batch.device_status() == 0
        q_in = q.copy()
        want = ob.decode_step(sh, pk, pv, tables, eng.nb, pos, q, k, v, cs, sn, exact=True)
        got = out_d.download(np.float32).reshape(L, S, NH, 128)
        if kernel == 2:     # fused: q is rotated in registers only, the buffer keeps the input
            assert np.array_equal(bits(dq.download(np.float32)), bits(q_in.ravel())), "q left as it was"
        else:
            assert np.array_equal(bits(dq.download(np.float32)), bits(q.ravel())), "q rotated in place"
        assert np.array_equal(bits(dk.download(np.float32)), bits(k.ravel())), "k rotated in place"
        for i in range(S):
            assert_attn_close(got[:, i], want[:, i], f"step {step} session {i} n_keys {pos[i] + 1}")
        pos = [p + 1 for p in pos]
    gk, gv = eng.read_pools()
    assert np.array_equal(bits(gk), bits(pk)) and np.array_equal(bits(gv), bits(pv))
    assert [eng.n_past(s) for s in ss] == pos
    batch.close()
    eng.close()


@pytest.mark.parametrize("model", ["qwen25_1p5b", "qwen25_7b"])
def test_attention_vs_reference_kernels(nv, ob, model):
    """fa_split_paged_kernel + fa_combine_kernel of the reference on an fp32 pool holding
    float(half(x)), against this library on the fp16 pool with the same values (both kernels)."""
    g = ob.ref_gpu(model)
    if g is None:
        pytest.skip("reference CUDA library not built")
    for n_ctx in (1, 33, 700, 2047):
        eng, ss, sh, pk, pv, cs, sn, rng = build_case(nv, ob, model, nv.KV_F16, [n_ctx], L=2, seed=n_ctx)
        NH = eng.NH
        rk, rv = nv.to_device(pk.astype(np.float32)), nv.to_device(pv.astype(np.float32))
        q = rng.standard_normal((1, NH, 128)).astype(np.float32)
        dq = nv.to_device(q)
        tab = nv.lib.nova_kv_table_slot(eng.h, eng.session_slice(ss[0]))
        ro, scr = nv.DevBuf(NH * 128 * 4), nv.DevBuf(NH * 32 * 130 * 4)
        layer = 1
        g.ref_gpu_attn_decode_paged(dq.ptr, rk.ptr, rv.ptr, tab, layer, eng.nb, n_ctx, ro.ptr, scr.ptr, None)
        nv.check(nv.lib.dev_sync())
        assert g.ref_gpu_last_error() == 0
        ref = ro.download(np.float32).reshape(NH, 128)
        # the oracle's order-faithful restatement should sit within float noise of the real kernels
        orc = ob.attn_decode_paged(sh, q[0], pk, pv, eng.pool.table(eng.session_slice(ss[0])), layer, eng.nb, n_ctx)
        assert rel_l2(orc, ref) < 2e-6
        # raw launcher (caller scratch, separate merge)
        shp = eng.shape()
        o = nv.DevBuf(NH * 128 * 4)
        for launcher_kernel in (0, 1):           # SIMT (default), then the tensor-core kernel behind the same launcher
            assert nv.lib.nova_launcher_set_kernel(launcher_kernel) == 0
            o.zero()
            nv.check(nv.lib.nova_launch_attn_decode_paged(C.byref(shp), dq.ptr, eng.k_base, eng.v_base, tab, layer, eng.nb,
                                                          n_ctx, o.ptr, scr.ptr, None))
            nv.check(nv.lib.dev_sync())
            assert_attn_close(o.download(np.float32).reshape(NH, 128), ref, f"raw n={n_ctx} launcher kernel {launcher_kernel}")
        assert nv.lib.nova_launcher_set_kernel(0) == 0
        # batched path, both kernels; n_keys = n_past + 1 so step back by one
        eng.set_n_past(ss[0], n_ctx - 1)
        batch = eng.batch(ss)
        for kernel in (0, 1):
            if nv.lib.nova_batch_set_kernel(batch.h, kernel) != 0:
                continue
            o.zero()
            batch.attn(layer, dq.ptr, o.ptr)
            nv.check(nv.lib.dev_sync())
            assert_attn_close(o.download(np.float32).reshape(NH, 128), ref, f"kernel {kernel} n={n_ctx}")
        batch.close()
        eng.close()


def test_decode_layer_sessions_from_c(nv, ob):
    """The two C loops the bench times for the literal drop-in (one call = RopeKvOp + AttnOp of every session of a
    layer, code/graph/dense.h:75-95): this library's launchers and the reference's, on fp32 pools with the same
    contents - appended rows bit-identical, outputs within float reordering."""
    g = ob.ref_gpu("qwen25_7b")
    if g is None or not hasattr(g, "ref_gpu_decode_layer_sessions"):
        pytest.skip("reference CUDA library not built")
    ctx_lens = [5, 100, 1030]
    eng, ss, sh, pk, pv, cs, sn, rng = build_case(nv, ob, "qwen25_7b", nv.KV_F32, ctx_lens, L=2, seed=77)
    NH, NKV, S, layer = eng.NH, eng.NKV, len(ss), 1
    rk, rv = nv.to_device(pk), nv.to_device(pv)                    # the reference works on its own copy of the pools
    q = rng.standard_normal((S, NH, 128)).astype(np.float32)
    k = rng.standard_normal((S, NKV, 128)).astype(np.float32)
    v = rng.standard_normal((S, NKV, 128)).astype(np.float32)
    tabs = (C.c_void_p * S)(*[nv.lib.nova_kv_table_slot(eng.h, eng.session_slice(s)) for s in ss])
    pos = (C.c_int64 * S)(*ctx_lens)
    dcs, dsn = nv.lib.nova_rope_cos(eng.h), nv.lib.nova_rope_sin(eng.h)
    scr = nv.DevBuf(NH * 32 * 130 * 4)
    outs = []
    for which in (0, 1, 2):
        dq, dk, dv, do = nv.to_device(q), nv.to_device(k), nv.to_device(v), nv.DevBuf(q.nbytes)
        if which in (0, 2):       # 2: the same launchers with the tensor-core kernel switched on (the append finds its rows in place)
            shp = eng.shape()
            assert nv.lib.nova_launcher_set_kernel(1 if which == 2 else 0) == 0
            nv.check(nv.lib.nova_launch_decode_layer_sessions(C.byref(shp), S, eng.k_base, eng.v_base, tabs, layer, eng.nb, pos, dq.ptr,
                                                              dk.ptr, dv.ptr, NH * 128, NKV * 128, dcs, dsn, do.ptr, scr.ptr, None))
            assert nv.lib.nova_launcher_set_kernel(0) == 0
        else:
            g.ref_gpu_decode_layer_sessions(S, rk.ptr, rv.ptr, tabs, layer, eng.nb, pos, dq.ptr, dk.ptr, dv.ptr, NH * 128, NKV * 128,
                                            dcs, dsn, do.ptr, scr.ptr, None)
        nv.check(nv.lib.dev_sync())
        outs.append((do.download(np.float32).reshape(S, NH, 128), dq.download(np.float32), dk.download(np.float32)))
    assert g.ref_gpu_last_error() == 0
    gk, gv = eng.read_pools()
    assert np.array_equal(bits(gk), bits(rk.download(np.float32).reshape(gk.shape)))
    assert np.array_equal(bits(gv), bits(rv.download(np.float32).reshape(gv.shape)))
    assert np.array_equal(bits(outs[0][1]), bits(outs[1][1])) and np.array_equal(bits(outs[0][2]), bits(outs[1][2]))   # rotated q, k
    for i in range(S):
        assert_attn_close(outs[0][0][i], outs[1][0][i], f"session {i}")
        assert_attn_close(outs[2][0][i], outs[1][0][i], f"session {i}, tensor-core launcher")
    assert np.array_equal(bits(outs[2][2]), bits(outs[1][2]))
    eng.close()


def test_gpu_misc_known_answers(nv):
    """tests/gpu_misc.cu of the reference: RoPE at position 0 is the identity; one key -> V[0]."""
    eng = nv.Engine(1, 12, 2, ctx=64, n_slices=1, kv_dtype=nv.KV_F32)
    s = eng.session_create()
    q = np.sin(np.arange(12 * 128, dtype=np.float32)).reshape(1, 1, 12, 128)
    k = np.cos(np.arange(2 * 128, dtype=np.float32)).reshape(1, 1, 2, 128)
    v = np.sin(np.arange(2 * 128, dtype=np.float32) * 0.001).reshape(1, 1, 2, 128)
    dq, dk, dv = nv.to_device(q), nv.to_device(k), nv.to_device(v)
    out = nv.DevBuf(12 * 128 * 4)
    b = eng.batch([s])
    b.step_all_layers(dq.ptr, dk.ptr, dv.ptr, out.ptr)
    nv.check(nv.lib.dev_sync())
    assert np.abs(dq.download(np.float32) - q.ravel()).max() <= 1e-6
    assert np.abs(dk.download(np.float32) - k.ravel()).max() <= 1e-6
    o = out.download(np.float32).reshape(12, 128)
    for h in range(12):
        assert np.abs(o[h] - v[0, 0, h // 6]).max() <= 1e-6
    b.close()
    eng.close()


@pytest.mark.parametrize("kernel", [0, 1])
def test_partial_and_lse_combine(nv, ob, kernel):
    """Split-K over page ranges (the multi-GPU cut) + nova_lse_combine == whole attention."""
    eng, ss, sh, pk, pv, cs, sn, rng = build_case(nv, ob, "qwen25_7b", nv.KV_F16, [999, 40], L=1, seed=3)
    NH, S = eng.NH, 2
    batch = eng.batch(ss)
    try_set_kernel(nv, batch, kernel)
    for s in ss:
        eng.set_n_past(s, eng.n_past(s) - 1)
    batch.sync_positions()
    q = rng.standard_normal((S, NH, 128)).astype(np.float32)
    dq = nv.to_device(q)
    ranges = [(0, 20), (20, 21), (21, 50), (50, 70)]
    parts = nv.DevBuf(len(ranges) * S * NH * 130 * 4)
    for i, (a, b) in enumerate(ranges):
        batch.attn_partial(0, dq.ptr, a, b, parts.ptr + i * S * NH * 130 * 4)
    out = nv.DevBuf(S * NH * 128 * 4)
    nv.check(nv.lib.nova_lse_combine(parts.ptr, len(ranges), S * NH, 128, out.ptr, None))
    nv.check(nv.lib.dev_sync())
    got = out.download(np.float32).reshape(S, NH, 128)
    gp = parts.download(np.float32).reshape(len(ranges), S, NH, 130)
    for i, s in enumerate(ss):
        tab = eng.pool.table(eng.session_slice(s))
        want = ob.attn_decode_paged(sh, q[i], pk, pv, tab, 0, eng.nb, [999, 40][i], exact=True)
        assert_attn_close(got[i], want, f"session {i}")
        for j, (a, b) in enumerate(ranges):
            wp = ob.attn_partial(sh, q[i], pk, pv, tab, 0, eng.nb, [999, 40][i], a, b)
            if wp[0, 1] == 0:      # this range holds no key of the session
                assert np.isneginf(gp[j, i, :, 0]).all() and not gp[j, i, :, 1:].any()
            else:                  # compare normalised partial outputs
                assert_attn_close(gp[j, i, :, 2:] / gp[j, i, :, 1:2], wp[:, 2:] / wp[:, 1:2], f"part {j}")
    # the oracle's merge of the GPU partials agrees with the GPU merge
    assert rel_l2(ob.lse_combine(gp.reshape(len(ranges), S * NH, 130)), got.reshape(S * NH, 128)) < 1e-5
    batch.close()
    eng.close()


def ll_encode(rows, epoch):
    """Partial rows [n][130] as they travel between ranks: 65 words of 16 bytes {value, epoch, value, epoch} per row;
    word 0 = (m, l), word j = accumulator values 2(j-1), 2(j-1)+1.  Rows with l <= 0 travel as clean empty rows."""
    rows = np.ascontiguousarray(rows, np.float32).copy()
    empty = ~(rows[:, 1] > 0)
    rows[empty] = 0.0
    rows[empty, 0] = -np.inf
    u = rows.view(np.uint32)
    w = np.zeros((rows.shape[0], 65, 4), np.uint32)
    w[:, :, 1] = epoch
    w[:, :, 3] = epoch
    w[:, 0, 0], w[:, 0, 2] = u[:, 0], u[:, 1]
    acc = u[:, 2:].reshape(rows.shape[0], 64, 2)
    w[:, 1:, 0], w[:, 1:, 2] = acc[:, :, 0], acc[:, :, 1]
    return w


@pytest.mark.parametrize("n_ranks", [4, 8])      # the kernel polls up to four ranks and more than four in different ways
def test_peer_exchange_on_one_gpu(nv, ob, n_ranks):
    """nova_lse_merge_peers: every rank stores its partial rows into the peers' exchange buffers, waits until the
    peers' rows have arrived in its own, and merges in rank order.  Here the 'ranks' are buffers of this one GPU
    and run one after the other (kernels that wait on one another never share a GPU): rank r finds the rows of the
    ranks before it where THEIR kernels stored them, and the rows of the ranks after it where the test put them
    beforehand.  Same result as nova_lse_combine on the stacked rows and as the oracle's merge for every rank, over
    two epochs (both slots); what each rank stored is checked word for word.  Then the bounded wait: rows that never
    arrive -> NOVA_ERR_TIMEOUT in the status word, output left alone."""
    rng = np.random.default_rng(31)
    n_rows = 56
    slot_bytes = int(nv.lib.nova_peer_slot_bytes(n_rows))
    region = slot_bytes // 8
    assert slot_bytes % 128 == 0 and region >= n_rows * 65 * 16
    bufs = [nv.DevBuf(2 * slot_bytes).zero() for _ in range(n_ranks)]
    base = (C.c_void_p * n_ranks)(*[b.ptr for b in bufs])
    status = nv.DevBuf(4).zero()
    out = nv.DevBuf(n_rows * 128 * 4)
    for epoch in (1, 2):
        slot = epoch % 2
        parts = rng.standard_normal((n_ranks, n_rows, 130)).astype(np.float32)
        parts[:, :, 1] = np.abs(parts[:, :, 1]) + 0.1
        parts[2, 5, 1] = 0.0                     # a rank whose page range held no key of that row
        parts[2, 5, 0] = -np.inf
        parts[:, 9, 1] = 0.0                     # a row nobody attended
        stacked = nv.to_device(parts)
        ref = nv.DevBuf(n_rows * 128 * 4)
        nv.check(nv.lib.nova_lse_combine(stacked.ptr, n_ranks, n_rows, 128, ref.ptr, None))
        nv.check(nv.lib.dev_sync())
        want = ref.download(np.float32)
        assert rel_l2(ob.lse_combine(parts).ravel(), want) < 1e-5
        for me in range(n_ranks):
            for later in range(me + 1, n_ranks):          # ranks that have not run yet: their rows, as they would arrive
                bufs[me].upload(ll_encode(parts[later], epoch), offset=slot * slot_bytes + later * region)
            mine = nv.to_device(parts[me])
            out.zero()
            nv.check(nv.lib.nova_lse_merge_peers(mine.ptr, base, n_ranks, me, slot_bytes, slot, n_rows, epoch, 200, out.ptr,
                                                 status.ptr, None))
            nv.check(nv.lib.dev_sync())
            assert int(status.download(np.int32)[0]) == 0
            got = out.download(np.float32)
            assert rel_l2(got, want) < 1e-6 and np.abs(got - want).max() < 1e-6, (epoch, me)
            assert not got.reshape(n_rows, 128)[9].any()
            sent = ll_encode(parts[me], epoch)
            for peer in range(n_ranks):
                if peer != me:
                    landed = bufs[peer].download(np.uint32, sent.size, slot * slot_bytes + me * region).reshape(sent.shape)
                    assert np.array_equal(landed, sent), (epoch, me, peer)
    # rows that never arrive: epoch 3 goes to slot 1, which still holds epoch 1
    out.upload(np.full(n_rows * 128, 7.0, np.float32))
    mine = nv.to_device(parts[0])
    nv.check(nv.lib.nova_lse_merge_peers(mine.ptr, base, n_ranks, 0, slot_bytes, 1, n_rows, 3, 50, out.ptr, status.ptr, None))
    nv.check(nv.lib.dev_sync())
    assert int(status.download(np.int32)[0]) == nv.ERR_TIMEOUT
    assert (out.download(np.float32) == 7.0).all()
    assert nv.lib.nova_lse_merge_peers(mine.ptr, base, 9, 0, slot_bytes, 0, n_rows, 1, 50, out.ptr, None, None) == nv.ERR_INVALID
    assert nv.lib.nova_lse_merge_peers(mine.ptr, base, n_ranks, 0, slot_bytes - 128, 0, n_rows, 1, 50, out.ptr, None, None) == nv.ERR_INVALID
    for b in bufs + [status, out]:
        b.free()


@pytest.mark.parametrize("me", [1, 0])
@pytest.mark.parametrize("kernel,pdl", [(1, 0), (2, 1), (0, 0)])
def test_step_partial_peers_two_ranks_on_one_gpu(nv, ob, kernel, pdl, me):
    """nova_batch_step_partial_peers as one of two ranks, the other one played by the oracle: its partial rows of
    every layer (over its own page range) are placed in this rank's exchange buffer as they would arrive over
    NVLink.  me = 1: this rank owns the pages from `cut` on (the page that receives the new token included);
    me = 0: it owns pages [0, cut), one session lies wholly inside (no page on the other rank), the new tokens of
    the longer sessions belong to the other rank and are not written here.  The merged outputs must be the oracle's
    whole decode step; what this rank stored into the peer's buffer must be its own partial rows."""
    ctx_lens = [1200, 90, 40]
    cut = 2 if me == 1 else 3                     # 41 keys = pages 0..2
    lo, hi = (cut, 1 << 40) if me == 1 else (0, cut)
    olo, ohi = (0, cut) if me == 1 else (cut, 1 << 40)
    eng, ss, sh, pk, pv, cs, sn, rng = build_case(nv, ob, "qwen25_7b", nv.KV_F16, ctx_lens, L=3, seed=43)
    L, S, NH, NKV = eng.L, len(ss), eng.NH, eng.NKV
    tables = np.stack([eng.pool.table(eng.session_slice(s)) for s in ss])
    batch = eng.batch(ss)
    try_set_kernel(nv, batch, kernel)
    batch.set_pdl(pdl)
    rows = S * NH
    slot_bytes = int(nv.lib.nova_peer_slot_bytes(rows))
    region = slot_bytes // 8
    n_slots = 4                                   # one slot per layer of a step, so that all can be filled beforehand
    mine, peer = nv.DevBuf(n_slots * slot_bytes).zero(), nv.DevBuf(n_slots * slot_bytes).zero()
    base = (C.c_void_p * 2)(*([peer.ptr, mine.ptr] if me == 1 else [mine.ptr, peer.ptr]))
    status = nv.DevBuf(4).zero()
    st = nv.Stream()
    pos = list(ctx_lens)
    dout = nv.DevBuf(L * rows * 128 * 4)
    epoch0 = 1
    for step in range(2):
        q = rng.standard_normal((L, S, NH, 128)).astype(np.float32)
        k = rng.standard_normal((L, S, NKV, 128)).astype(np.float32)
        v = rng.standard_normal((L, S, NKV, 128)).astype(np.float32)
        dq, dk, dv = nv.to_device(q), nv.to_device(k), nv.to_device(v)
        want = ob.decode_step(sh, pk, pv, tables, eng.nb, pos, q, k, v, cs, sn, exact=True)       # rotates q, k; appends
        for layer in range(L):                    # the other rank's rows of this step, layer by layer
            other = np.stack([ob.attn_partial(sh, q[layer, i], pk, pv, tables[i], layer, eng.nb, pos[i] + 1, olo, ohi)
                              for i in range(S)]).reshape(rows, 130)
            epoch = epoch0 + layer
            mine.upload(ll_encode(other, epoch), offset=(epoch % n_slots) * slot_bytes + (1 - me) * region)
        nv.check(nv.lib.nova_batch_step_partial_peers(batch.h, dq.ptr, dk.ptr, dv.ptr, lo, hi, base, 2, me, slot_bytes,
                                                      n_slots, epoch0, 500, dout.ptr, status.ptr, st.h))
        st.sync()
        assert batch.device_status() == 0 and int(status.download(np.int32)[0]) == 0
        got = dout.download(np.float32).reshape(want.shape)
        assert_attn_close(got, want, f"step {step}")
        for layer in range(L):                    # what crossed to the peer: this rank's partial rows over its own pages
            epoch = epoch0 + layer
            landed = peer.download(np.uint32, rows * 65 * 4, (epoch % n_slots) * slot_bytes + me * region).reshape(rows, 65, 4)
            assert (landed[:, :, 1] == epoch).all() and (landed[:, :, 3] == epoch).all()
            sent = np.empty((rows, 130), np.float32)
            sent[:, 0], sent[:, 1] = landed[:, 0, 0].view(np.float32), landed[:, 0, 2].view(np.float32)
            sent[:, 2:] = np.stack([landed[:, 1:, 0], landed[:, 1:, 2]], axis=-1).reshape(rows, 128).view(np.float32)
            for i in range(S):
                wp = ob.attn_partial(sh, q[layer, i], pk, pv, tables[i], layer, eng.nb, pos[i] + 1, lo, hi)
                sp = sent.reshape(S, NH, 130)[i]
                if wp[0, 1] == 0:
                    assert not (sp[:, 1] > 0).any()
                else:
                    assert_attn_close(sp[:, 2:] / sp[:, 1:2], wp[:, 2:] / wp[:, 1:2], f"sent rows layer {layer} session {i}")
        pos = [p + 1 for p in pos]
        epoch0 += L
    if me == 1:                                   # the last rank wrote every new token
        gk, gv = eng.read_pools()
        assert np.array_equal(bits(gk), bits(pk)) and np.array_equal(bits(gv), bits(pv))
    st.close()
    batch.close()
    eng.close()


@pytest.mark.parametrize("kernel,pdl", [(0, 0), (1, 0), (2, 0), (2, 1)])
def test_step_partial_peers_single_rank(nv, ob, kernel, pdl):
    """nova_batch_step_partial_peers with one rank (its own exchange buffer, nobody to wait for) is a plain
    decode step in layer order: outputs, pages and positions against the oracle over three steps; the page
    window and the epoch/slot walk are the ones a multi-GPU run uses."""
    ctx_lens = [700, 33, 0, 1500]
    eng, ss, sh, pk, pv, cs, sn, rng = build_case(nv, ob, "qwen25_7b", nv.KV_F16, ctx_lens, L=3, seed=41)
    L, S, NH, NKV = eng.L, len(ss), eng.NH, eng.NKV
    tables = np.stack([eng.pool.table(eng.session_slice(s)) for s in ss])
    batch = eng.batch(ss)
    try_set_kernel(nv, batch, kernel)
    batch.set_pdl(pdl)
    rows = S * NH
    slot_bytes = int(nv.lib.nova_peer_slot_bytes(rows))
    xbuf = nv.DevBuf(2 * slot_bytes).zero()
    base = (C.c_void_p * 1)(xbuf.ptr)
    status = nv.DevBuf(4).zero()
    st = nv.Stream()
    pos = list(ctx_lens)
    dout = nv.DevBuf(L * rows * 128 * 4)
    for step in range(3):
        q = rng.standard_normal((L, S, NH, 128)).astype(np.float32)
        k = rng.standard_normal((L, S, NKV, 128)).astype(np.float32)
        v = rng.standard_normal((L, S, NKV, 128)).astype(np.float32)
        dq, dk, dv = nv.to_device(q), nv.to_device(k), nv.to_device(v)
        nv.check(nv.lib.nova_batch_step_partial_peers(batch.h, dq.ptr, dk.ptr, dv.ptr, 0, 1 << 40, base, 1, 0, slot_bytes, 2,
                                                      1 + step * L, 200, dout.ptr, status.ptr, st.h))
        st.sync()
        assert batch.device_status() == 0 and int(status.download(np.int32)[0]) == 0
        got = dout.download(np.float32).reshape(q.shape)
        want = ob.decode_step(sh, pk, pv, tables, eng.nb, pos, q, k, v, cs, sn, exact=True)
        assert_attn_close(got, want, f"step {step}")
        pos = [p + 1 for p in pos]
    gk, gv = eng.read_pools()
    assert np.array_equal(bits(gk), bits(pk)) and np.array_equal(bits(gv), bits(pv))
    assert [eng.n_past(s) for s in ss] == pos
    st.close()
    batch.close()
    eng.close()


@pytest.mark.parametrize("kernel", [0, 2])
def test_cow_shared_prefix(nv, ob, kernel):
    """Config-3 in miniature: sessions share a donor's prefix whose tail page is partly filled; the
    first append of each un-shares that page exactly once (tests/cow_e2e_demo.cpp:87-105,
    tests/reuse_demo.cpp:72-81).  Pages and attention against the oracle; the host bookkeeping itself is
    diffed against the reference's KvPool in test_host_state.py."""
    model, kvd, L, P, n_fork = "qwen25_7b", nv.KV_F16, 2, 37, 5
    eng, ss, sh, pk, pv, cs, sn, rng = build_case(nv, ob, model, kvd, [P], L=L, seed=8, spare=n_fork + 1)
    donor = ss[0]
    forks = []
    for _ in range(n_fork):
        f = eng.session_create()
        forks.append(f)
        eng.attach_prefix(f, donor, P)
    tail = eng.pool.table(eng.session_slice(donor))[(P - 1) >> 4]
    assert eng.pool.refcnt(tail) == n_fork + 1
    donor_tail_before = eng.read_page("k", 1, tail).copy()
    batch = eng.batch(forks)
    try_set_kernel(nv, batch, kernel)
    NH, NKV, S = eng.NH, eng.NKV, n_fork
    out_d = nv.DevBuf(L * S * NH * 128 * 4)
    pos = [P] * S
    cows = []
    for step in range(4):
        q = rng.standard_normal((L, S, NH, 128)).astype(np.float32)
        k = rng.standard_normal((L, S, NKV, 128)).astype(np.float32)
        v = rng.standard_normal((L, S, NKV, 128)).astype(np.float32)
        before = {f: eng.pool.table(eng.session_slice(f)).copy() for f in forks}
        n_cow = batch.cow()
        cows.append(n_cow)
        for f in forks:      # oracle: same page copies, in the same order
            after = eng.pool.table(eng.session_slice(f))
            for lb in np.nonzero(after != before[f])[0]:
                ob.cow_copy(sh, pk, pv, eng.nb, int(before[f][lb]), int(after[lb]))
        dq, dk, dv = nv.to_device(q), nv.to_device(k), nv.to_device(v)
        batch.step_all_layers(dq.ptr, dk.ptr, dv.ptr, out_d.ptr)
        batch.advance()
        nv.check(nv.lib.dev_sync())
        tables = np.stack([eng.pool.table(eng.session_slice(f)) for f in forks])
        for f, row in zip(forks, tables):      # device mirror follows the host table
            assert np.array_equal(eng.device_table(eng.session_slice(f)), row)
        want = ob.decode_step(sh, pk, pv, tables, eng.nb, pos, q, k, v, cs, sn, exact=True)
        assert_attn_close(out_d.download(np.float32).reshape(want.shape), want, f"step {step}")
        pos = [p + 1 for p in pos]
    assert cows == [n_fork, 0, 0, 0]                                   # exactly once each, never again
    assert eng.pool.cow_count() == n_fork
    assert eng.pool.refcnt(tail) == 1                                  # donor owns its tail page again
    assert np.array_equal(bits(eng.read_page("k", 1, tail)), bits(donor_tail_before))   # donor untouched
    gk, gv = eng.read_pools()
    assert np.array_equal(bits(gk), bits(pk)) and np.array_equal(bits(gv), bits(pv))
    # pool exhaustion is an error code, not an abort (src/model.cpp:173 aborts)
    eng2 = nv.Engine(1, 12, 2, ctx=32, n_slices=2, kv_dtype=kvd)
    a, b = eng2.session_create(), eng2.session_create()
    eng2.set_n_past(a, 20)
    eng2.attach_prefix(b, a, 20)
    assert nv.lib.nova_session_cow(eng2.h, b, 20, 1) == nv.ERR_POOL_FULL
    eng2.close()
    batch.close()
    eng.close()


@pytest.mark.parametrize("kernel,mode", [(1, 1), (2, 1), (2, 2), (3, 1), (4, 1), (4, 2)])
@pytest.mark.parametrize("model,n_fork,P", [("qwen25_7b", 12, 700), ("qwen25_14b", 5, 300), ("qwen25_1p5b", 10, 517),
                                            ("qwen25_7b", 40, 700)])       # 40 sessions x 7 heads: two 256-row tiles per kv head
def test_cascade_over_shared_prefix(nv, ob, model, n_fork, P, kernel, mode):
    """Sessions forked from one prefix (partly filled tail page), private suffixes of different lengths, then
    decode steps with the cascade switched on: the shared full pages are attended once for all sessions, each
    session's own pages (the un-shared tail page onwards) as usual, merged by log-sum-exp.  Per-layer launches,
    plain, chained and replayed from a graph; outputs against the oracle's exact attention, pages bit-exact, the number of shared pages
    found on the host, and the same steps again without the cascade."""
    kvd, L = nv.KV_F16, 2
    eng, ss, sh, pk, pv, cs, sn, rng = build_case(nv, ob, model, kvd, [P], L=L, seed=19, spare=n_fork + 1)
    donor = ss[0]
    forks = []
    for _ in range(n_fork):
        f = eng.session_create()
        forks.append(f)
        eng.attach_prefix(f, donor, P)
    batch = eng.batch(forks)
    try_set_kernel(nv, batch, kernel)
    batch.set_cascade(1)
    batch.set_pdl(1 if kernel in (2, 4) else 0)
    NH, NKV, S = eng.NH, eng.NKV, n_fork
    out_d = nv.DevBuf(L * S * NH * 128 * 4)
    st = nv.Stream()
    pos = [P] * S
    for step in range(20):
        q = rng.standard_normal((L, S, NH, 128)).astype(np.float32)
        k = rng.standard_normal((L, S, NKV, 128)).astype(np.float32)
        v = rng.standard_normal((L, S, NKV, 128)).astype(np.float32)
        before = {f: eng.pool.table(eng.session_slice(f)).copy() for f in forks}
        dq, dk, dv = nv.to_device(q), nv.to_device(k), nv.to_device(v)
        if step == 4:
            batch.set_cascade(0)                          # a few plain steps in between: same results
        if step == 7:
            batch.set_cascade(1)
        # COW guard + per-layer launches, issued directly (mode 1) or replayed from a CUDA graph (mode 2: re-captured
        # whenever the number of shared pages changes)
        batch.run_steps(1, dq.ptr, dk.ptr, dv.ptr, out_d.ptr, q.size, k.size, mode, st.h)
        st.sync()
        assert batch.device_status() == 0
        assert batch.shared_prefix_pages() == (0 if 4 <= step <= 6 else P // 16), step
        for f in forks:      # oracle: same page copies, in the same order
            after = eng.pool.table(eng.session_slice(f))
            for lb in np.nonzero(after != before[f])[0]:
                ob.cow_copy(sh, pk, pv, eng.nb, int(before[f][lb]), int(after[lb]))
        tables = np.stack([eng.pool.table(eng.session_slice(f)) for f in forks])
        want = ob.decode_step(sh, pk, pv, tables, eng.nb, pos, q, k, v, cs, sn, exact=True)
        assert_attn_close(out_d.download(np.float32).reshape(want.shape), want, f"step {step}")
        pos = [p + 1 for p in pos]
    gk, gv = eng.read_pools()
    assert np.array_equal(bits(gk), bits(pk)) and np.array_equal(bits(gv), bits(pv))
    st.close()
    batch.close()
    eng.close()


def test_fork_registry_attach_and_telemetry(nv, ob):
    """EngineHost::fork (client/src/engine_host.cpp:179-192), the telemetry counters (:194-211) and prefix reuse
    found through the block registry: a fork shares every page of its source (refcounts, no copy), a block id
    looked up in the registry attaches its producer's first pos1 tokens, and both keep attention on the shared
    pages identical to the source's."""
    eng, ss, sh, pk, pv, cs, sn, rng = build_case(nv, ob, "qwen25_1p5b", nv.KV_F16, [40], L=2, seed=51, spare=3)
    a = ss[0]
    tel = nv.Telemetry()
    nv.check(nv.lib.nova_engine_telemetry(eng.h, C.byref(tel)))
    total, free0 = tel.blocks_total, tel.blocks_free
    assert (tel.blocks_shared, tel.cow_count, tel.sessions_live) == (0, 0, 1) and tel.kv_bytes_cap > tel.kv_bytes_used > 0
    f = nv.lib.nova_session_fork(eng.h, a)
    assert f >= 0 and f != a and eng.n_past(f) == 40
    ta, tf = eng.pool.table(eng.session_slice(a)), eng.pool.table(eng.session_slice(f))
    assert np.array_equal(ta[:3], tf[:3]) and all(eng.pool.refcnt(int(p)) == 2 for p in ta[:3])
    nv.check(nv.lib.nova_engine_telemetry(eng.h, C.byref(tel)))
    assert (tel.blocks_shared, tel.sessions_live, tel.blocks_total) == (3, 2, total)
    empty = eng.session_create()
    assert nv.lib.nova_session_fork(eng.h, empty) == nv.ERR_INVALID          # nothing to share (the reference returns -1)
    # registry-driven reuse: the block {7, 9} was produced by session a and covers its first 32 tokens
    reg = nv.Registry()
    reg.put(7, 9, session=a, turn=0, pos0=0, pos1=32)
    assert nv.lib.nova_session_attach_block(eng.h, reg.h, 7, 10, empty) == 0  # unknown block
    assert nv.lib.nova_session_attach_block(eng.h, reg.h, 7, 9, empty) == 32
    assert eng.n_past(empty) == 32
    te = eng.pool.table(eng.session_slice(empty))
    assert np.array_equal(te[:2], ta[:2]) and eng.pool.refcnt(int(ta[0])) == 3 and eng.pool.refcnt(int(ta[2])) == 2
    # one decode step of source, fork and the attached session: the first two see the same 40 keys
    batch = eng.batch([a, f, empty])
    try_set_kernel(nv, batch, 2)
    L, NH, NKV = eng.L, eng.NH, eng.NKV
    q = np.repeat(rng.standard_normal((L, 1, NH, 128)).astype(np.float32), 3, axis=1)
    k = np.repeat(rng.standard_normal((L, 1, NKV, 128)).astype(np.float32), 3, axis=1)
    v = np.repeat(rng.standard_normal((L, 1, NKV, 128)).astype(np.float32), 3, axis=1)
    out = np.empty_like(q)
    before = {s: eng.pool.table(eng.session_slice(s)).copy() for s in (a, f, empty)}
    batch.decode_step_host(q.ctypes.data, k.ctypes.data, v.ctypes.data, out.ctypes.data, 1)
    for s in (a, f, empty):
        after = eng.pool.table(eng.session_slice(s))
        for lb in np.nonzero(after != before[s])[0]:
            ob.cow_copy(sh, pk, pv, eng.nb, int(before[s][lb]), int(after[lb]))
    tables = np.stack([eng.pool.table(eng.session_slice(s)) for s in (a, f, empty)])
    want = ob.decode_step(sh, pk, pv, tables, eng.nb, [40, 40, 32], q, k, v, cs, sn, exact=True)
    assert_attn_close(out, want, "shared sessions")
    assert np.array_equal(bits(out[:, 0]), bits(out[:, 1])), "source and fork attend the same keys"
    nv.check(nv.lib.nova_engine_telemetry(eng.h, C.byref(tel)))
    # the partly filled page shared by source and fork is copied once (by whoever appends first); the other then owns it
    assert tel.cow_count == 1 and tel.blocks_free < free0
    batch.close()
    eng.session_destroy(a)
    # the fork and the attached session still read pages of a's slice, which would be handed out next: refused
    assert nv.lib.nova_session_create(eng.h) == nv.ERR_BUSY
    eng.session_destroy(f)
    eng.session_destroy(empty)
    other = eng.session_create()
    assert nv.lib.nova_session_attach_block(eng.h, reg.h, 7, 9, other) in (0, 32)   # producer gone (or its slot re-used)
    eng.close()


def test_sessions_follow_reference_manager(nv):
    """SessionManager semantics (code/session.h:84-142): lowest free slot, slice ids LIFO, errors
    as codes; zeroing of a new session's pages."""
    eng = nv.Engine(2, 12, 2, ctx=64, n_slices=3, kv_dtype=nv.KV_F16, max_sessions=3)
    a, b, c = eng.session_create(), eng.session_create(), eng.session_create()
    assert (a, b, c) == (0, 1, 2)
    assert nv.lib.nova_session_create(eng.h) == nv.ERR_NO_SESSION
    assert [eng.session_slice(x) for x in (a, b, c)] == [0, 1, 2]
    eng.session_destroy(a)
    eng.session_destroy(c)
    d = eng.session_create()
    assert d == 0 and eng.session_slice(d) == 2          # slot: lowest free; slice: last released first
    assert np.array_equal(eng.device_table(2), eng.pool.table(2))
    assert nv.lib.nova_session_live_count(eng.h) == 2
    assert eng.session_stream(d) is not None and eng.session_stream(1) != eng.session_stream(d)
    k, v = eng.read_pools()
    assert not k.any() and not v.any()
    assert nv.lib.nova_session_destroy(eng.h, 7) == nv.ERR_INVALID
    eng.close()


def test_session_errors_are_codes(nv):
    """Host error paths of the session layer: a slice whose pages a fork still maps is not handed out again
    (NOVA_ERR_BUSY until the fork is gone), and a batch that names a destroyed session reports NOVA_ERR_INVALID
    instead of following a dangling slice."""
    eng = nv.Engine(1, 12, 2, ctx=64, n_slices=3, kv_dtype=nv.KV_F16)
    parent = eng.session_create()
    eng.set_n_past(parent, 40)
    fork = nv.lib.nova_session_fork(eng.h, parent)
    assert fork >= 0
    eng.session_destroy(parent)
    assert nv.lib.nova_session_create(eng.h) == nv.ERR_BUSY          # the parent's slice is next, its pages still read
    assert nv.lib.nova_session_live_count(eng.h) == 1 and eng.pool.used() == 1     # and nothing was left half made
    eng.session_destroy(fork)
    again = eng.session_create()
    assert again >= 0
    other = eng.session_create()
    batch = eng.batch([again, other])
    eng.session_destroy(other)
    assert nv.lib.nova_batch_cow(batch.h, None) == nv.ERR_INVALID
    d = nv.DevBuf(2 * 4 * 12 * 128 * 4)
    assert nv.lib.nova_batch_prefill(batch.h, 0, 4, d.ptr, d.ptr, d.ptr, d.ptr, None) == nv.ERR_INVALID
    batch.close()
    eng.close()


def test_bad_table_entry_is_reported_not_followed(nv):
    """A block-table entry outside [0, NB) is checked before it is used: the launch skips the page
    and leaves NOVA_ERR_BAD_TABLE in the status word."""
    eng = nv.Engine(1, 12, 2, ctx=64, n_slices=1, kv_dtype=nv.KV_F16)
    s = eng.session_create()
    eng.set_n_past(s, 20)
    bad = eng.pool.table(eng.session_slice(s)).copy()
    bad[1] = eng.nb + 5
    nv.check(nv.lib.dev_upload(nv.lib.nova_kv_table_slot(eng.h, eng.session_slice(s)), bad.ctypes.data, bad.nbytes))
    b = eng.batch([s])
    q = nv.to_device(np.zeros((12, 128), np.float32))
    o = nv.DevBuf(12 * 128 * 4)
    b.attn(0, q.ptr, o.ptr)
    nv.check(nv.lib.dev_sync())
    assert b.device_status() == nv.ERR_BAD_TABLE
    assert b.device_status() == 0          # reading clears it
    b.close()
    eng.close()


@pytest.mark.parametrize("kernel", [0, 1, 2])
def test_decode_step_from_host_buffers(nv, ob, kernel):
    eng, ss, sh, pk, pv, cs, sn, rng = build_case(nv, ob, "qwen25_1p5b", nv.KV_F16, [50, 7], L=3, seed=13)
    L, S, NH, NKV = eng.L, 2, eng.NH, eng.NKV
    tables = np.stack([eng.pool.table(eng.session_slice(s)) for s in ss])
    batch = eng.batch(ss)
    try_set_kernel(nv, batch, kernel)
    pos = [50, 7]
    for step, per_layer in enumerate((1, 0, 1)):
        q = rng.standard_normal((L, S, NH, 128)).astype(np.float32)
        k = rng.standard_normal((L, S, NKV, 128)).astype(np.float32)
        v = rng.standard_normal((L, S, NKV, 128)).astype(np.float32)
        out = np.empty_like(q)
        batch.decode_step_host(q.ctypes.data, k.ctypes.data, v.ctypes.data, out.ctypes.data, per_layer)
        want = ob.decode_step(sh, pk, pv, tables, eng.nb, pos, q.copy(), k.copy(), v, cs, sn, exact=True)
        assert_attn_close(out, want, f"step {step}")
        pos = [p + 1 for p in pos]
    # queued steps (no synchronisation per step): uploads, kernels and downloads of consecutive steps overlap on two
    # sets of staging buffers; every step in flight has its own pinned host buffers, checked after one wait
    if kernel == 2:
        batch.set_pdl(1)
    st = nv.Stream()
    n_q, n_k = L * S * NH * 128, L * S * NKV * 128
    steps = []
    for step in range(7):
        bufs = [nv.lib.dev_host_alloc(n * 4) for n in (n_q, n_k, n_k, n_q)]
        views = [np.ctypeslib.as_array(C.cast(p, C.POINTER(C.c_float)), shape=(n,)) for p, n in zip(bufs, (n_q, n_k, n_k, n_q))]
        for v_, n in zip(views[:3], (n_q, n_k, n_k)):
            v_[:] = rng.standard_normal(n).astype(np.float32)
        views[3][:] = np.nan
        batch.decode_step_host(bufs[0], bufs[1], bufs[2], bufs[3], step % 3 != 1, st.h, no_sync=True)
        steps.append((bufs, views))
    batch.host_wait(st.h)
    assert batch.device_status() == 0
    for step, (bufs, views) in enumerate(steps):
        q = views[0].reshape(L, S, NH, 128).copy()
        k = views[1].reshape(L, S, NKV, 128).copy()
        v = views[2].reshape(L, S, NKV, 128).copy()
        want = ob.decode_step(sh, pk, pv, tables, eng.nb, pos, q, k, v, cs, sn, exact=True)
        assert_attn_close(views[3].reshape(want.shape), want, f"queued step {step}")
        pos = [p + 1 for p in pos]
        for p_ in bufs:
            nv.lib.dev_host_free(p_)
    gk, gv = eng.read_pools()
    assert np.array_equal(bits(gk), bits(pk)) and np.array_equal(bits(gv), bits(pv))
    st.close()
    batch.close()
    eng.close()


@pytest.mark.parametrize("mode", [0, 1, 2])
@pytest.mark.parametrize("kernel,pdl", [(0, 0), (1, 0), (2, 0), (2, 1)])
def test_run_steps_native_loop(nv, ob, mode, kernel, pdl):
    """nova_batch_run_steps (the native multi-step loop the bench times): all-layer launches, per-layer
    launches and CUDA-graph replay, with and without the fused append and programmatic dependent
    launch, against the oracle over four steps."""
    eng, ss, sh, pk, pv, cs, sn, rng = build_case(nv, ob, "qwen25_7b", nv.KV_F16, [300, 14, 47, 1000], L=3, seed=17)
    L, S, NH, NKV = eng.L, len(ss), eng.NH, eng.NKV
    tables = np.stack([eng.pool.table(eng.session_slice(s)) for s in ss])
    batch = eng.batch(ss)
    try_set_kernel(nv, batch, kernel)
    batch.set_pdl(pdl)
    n_steps = 4
    q = rng.standard_normal((n_steps, L, S, NH, 128)).astype(np.float32)
    k = rng.standard_normal((n_steps, L, S, NKV, 128)).astype(np.float32)
    v = rng.standard_normal((n_steps, L, S, NKV, 128)).astype(np.float32)
    dq, dk, dv = nv.to_device(q), nv.to_device(k), nv.to_device(v)
    dout = nv.DevBuf(q.nbytes)
    st = nv.Stream()
    batch.run_steps(n_steps, dq.ptr, dk.ptr, dv.ptr, dout.ptr, q[0].size, k[0].size, mode, st.h)
    st.sync()
    assert batch.device_status() == 0
    got = dout.download(np.float32).reshape(q.shape)
    pos = [300, 14, 47, 1000]
    for i in range(n_steps):
        want = ob.decode_step(sh, pk, pv, tables, eng.nb, pos, q[i], k[i], v[i], cs, sn, exact=True)
        assert_attn_close(got[i], want, f"step {i}")
        pos = [p + 1 for p in pos]
    gk, gv = eng.read_pools()
    assert np.array_equal(bits(gk), bits(pk)) and np.array_equal(bits(gv), bits(pv))
    assert np.array_equal(bits(dk.download(np.float32)), bits(k.ravel())), "k rotated in place"
    assert [eng.n_past(s) for s in ss] == pos
    st.close()
    batch.close()
    eng.close()


@pytest.mark.parametrize("mode", [1, 2])
@pytest.mark.parametrize("model,n_sessions", [("qwen25_7b", 300), ("qwen25_14b", 120), ("qwen25_1p5b", 200)])
def test_many_short_sessions_chained_launches(nv, ob, model, n_sessions, mode):
    """Far more rows than CTAs: every CTA's page range crosses several row boundaries, so finished
    segments are parked in shared memory (and, past two of them, written after an early dependency
    wait), the merge CTAs loop over many rows, and some sessions are empty.  Per-layer launches chained
    by programmatic dependent launch, plain and replayed from a graph, three steps against the oracle."""
    rng0 = np.random.default_rng(5)
    ctx_lens = [int(x) for x in rng0.integers(0, 90, n_sessions)]
    ctx_lens[3] = 0
    ctx_lens[7] = 16
    eng, ss, sh, pk, pv, cs, sn, rng = build_case(nv, ob, model, nv.KV_F16, ctx_lens, L=3, seed=23)
    L, S, NH, NKV = eng.L, len(ss), eng.NH, eng.NKV
    tables = np.stack([eng.pool.table(eng.session_slice(s)) for s in ss])
    batch = eng.batch(ss)
    try_set_kernel(nv, batch, 2)
    batch.set_pdl(1)
    n_steps = 3
    q = rng.standard_normal((n_steps, L, S, NH, 128)).astype(np.float32)
    k = rng.standard_normal((n_steps, L, S, NKV, 128)).astype(np.float32)
    v = rng.standard_normal((n_steps, L, S, NKV, 128)).astype(np.float32)
    dq, dk, dv = nv.to_device(q), nv.to_device(k), nv.to_device(v)
    dout = nv.DevBuf(q.nbytes)
    st = nv.Stream()
    batch.run_steps(n_steps, dq.ptr, dk.ptr, dv.ptr, dout.ptr, q[0].size, k[0].size, mode, st.h)
    st.sync()
    assert batch.device_status() == 0
    got = dout.download(np.float32).reshape(q.shape)
    pos = list(ctx_lens)
    for i in range(n_steps):
        want = ob.decode_step(sh, pk, pv, tables, eng.nb, pos, q[i], k[i], v[i], cs, sn, exact=True)
        assert_attn_close(got[i], want, f"step {i}")
        pos = [p + 1 for p in pos]
    gk, gv = eng.read_pools()
    assert np.array_equal(bits(gk), bits(pk)) and np.array_equal(bits(gv), bits(pv))
    st.close()
    batch.close()
    eng.close()


@pytest.mark.parametrize("kernel", [0, 1, 3])
@pytest.mark.parametrize("model", ["qwen25_1p5b", "qwen25_7b", "qwen25_14b"])
def test_prefill_vs_oracle_and_reference(nv, ob, model, kernel):
    """Paged prefill (multi-token RoPE+append, then causal attention of the new queries): pages bit-exact,
    attention against the oracle's restatement of flash_paged_kernel and, where the library is present, the
    reference's own launch_attn_prefill_paged on an fp32 pool with the same values; a chunked prefill followed by
    decode steps continues the same cache."""
    eng, ss, sh, pk, pv, cs, sn, rng = build_case(nv, ob, model, nv.KV_F16, [37, 0], L=2, seed=31, extra_ctx=300)
    L, S, NH, NKV = eng.L, 2, eng.NH, eng.NKV
    batch = eng.batch(ss)
    try_set_kernel(nv, batch, kernel)
    assert batch.prefill_max_tokens() >= 64
    pos = [37, 0]
    g = ob.ref_gpu(model)
    for n_tok in (21, 5, 150):
        q = rng.standard_normal((L, S, n_tok, NH, 128)).astype(np.float32)
        k = rng.standard_normal((L, S, n_tok, NKV, 128)).astype(np.float32)
        v = rng.standard_normal((L, S, n_tok, NKV, 128)).astype(np.float32)
        out = np.empty_like(q)
        for layer in range(L):
            dq, dk, dv = nv.to_device(q[layer]), nv.to_device(k[layer]), nv.to_device(v[layer])
            do = nv.DevBuf(q[layer].nbytes)
            batch.prefill(layer, n_tok, dq.ptr, dk.ptr, dv.ptr, do.ptr)
            nv.check(nv.lib.dev_sync())
            out[layer] = do.download(np.float32).reshape(out[layer].shape)
            for i, s in enumerate(ss):
                table = eng.pool.table(eng.session_slice(s))
                qi, ki = q[layer, i].copy(), k[layer, i].copy()
                ob.rope_append_paged(sh, pk, pv, table, layer, eng.nb, n_tok, pos[i], qi, ki, v[layer, i], cs, sn)
                want = ob.attn_prefill_paged(sh, qi, pk, pv, table, layer, eng.nb, n_tok, pos[i])
                assert_attn_close(out[layer, i], want, f"prefill n={n_tok} layer {layer} session {i}")
                assert np.array_equal(bits(dq.download(np.float32).reshape(S, n_tok, NH, 128)[i]), bits(qi))
                if g is not None and hasattr(g, "ref_gpu_attn_prefill_paged") and layer == 1:
                    rk, rv = nv.to_device(pk.astype(np.float32)), nv.to_device(pv.astype(np.float32))
                    rq, ro = nv.to_device(qi), nv.DevBuf(qi.nbytes)
                    g.ref_gpu_attn_prefill_paged(rq.ptr, rk.ptr, rv.ptr, nv.lib.nova_kv_table_slot(eng.h, eng.session_slice(s)),
                                                 layer, eng.nb, n_tok, pos[i], ro.ptr, None)
                    nv.check(nv.lib.dev_sync())
                    ref = ro.download(np.float32).reshape(qi.shape)
                    assert rel_l2(want, ref) < 2e-6                      # oracle == the reference's kernel
                    assert_attn_close(out[layer, i], ref, "vs reference prefill kernel")
        batch.advance_by(n_tok)
        pos = [p + n_tok for p in pos]
    assert batch.device_status() == 0
    gk, gv = eng.read_pools()
    assert np.array_equal(bits(gk), bits(pk)) and np.array_equal(bits(gv), bits(pv))
    # decode continues on the prefilled cache
    tables = np.stack([eng.pool.table(eng.session_slice(s)) for s in ss])
    q = rng.standard_normal((L, S, NH, 128)).astype(np.float32)
    k = rng.standard_normal((L, S, NKV, 128)).astype(np.float32)
    v = rng.standard_normal((L, S, NKV, 128)).astype(np.float32)
    dq, dk, dv, do = nv.to_device(q), nv.to_device(k), nv.to_device(v), nv.DevBuf(q.nbytes)
    batch.step_all_layers(dq.ptr, dk.ptr, dv.ptr, do.ptr)
    nv.check(nv.lib.dev_sync())
    want = ob.decode_step(sh, pk, pv, tables, eng.nb, pos, q, k, v, cs, sn, exact=True)
    assert_attn_close(do.download(np.float32).reshape(want.shape), want, "decode after prefill")
    batch.close()
    eng.close()
