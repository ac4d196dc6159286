"""Pins the CPU oracle (oracle/paged_decode_oracle.c): against outputs of the reference's own decode
attention recorded in tests/golden/attn_sycl_ref.npz, against the known answers of the reference's GPU
unit test (tests/gpu_misc.cu:13-66) and against a plain numpy restatement of the page addressing."""
import os

import numpy as np
import pytest

from conftest import GOLDEN
from golden.make_golden import ATTN_CASES, SYCL_MODELS, attn_inputs


def rel_l2(a, b):
    return float(np.linalg.norm(a.astype(np.float64) - b) / max(np.linalg.norm(b), 1e-30))


def contiguous_as_pages(ob, sh, k, v, n_keys):
    """A contiguous [pos][NKV][HD] cache is a paged one with the identity table."""
    nblocks = (n_keys + 15) // 16
    pk, pv = ob.new_pools(sh, nblocks)
    pk.reshape(-1)[: k.size] = k
    pv.reshape(-1)[: v.size] = v
    return pk, pv, np.arange(nblocks, dtype=np.int32)


@pytest.mark.parametrize("model", list(SYCL_MODELS))
def test_attention_vs_reference_outputs(ob, model):
    gold = np.load(os.path.join(GOLDEN, "attn_sycl_ref.npz"))
    _, NH, NKV = SYCL_MODELS[model]
    sh = ob.shape(1, NH, NKV, ob.KV_F32)
    for n_keys in ATTN_CASES[model]:
        q, k, v = attn_inputs(model, n_keys)
        pk, pv, table = contiguous_as_pages(ob, sh, k, v, n_keys)
        want = gold[f"{model}/{n_keys}"]
        got = ob.attn_decode_paged(sh, q, pk, pv, table, 0, len(table), n_keys)
        exact = ob.attn_decode_paged(sh, q, pk, pv, table, 0, len(table), n_keys, exact=True)
        # the reference's own gate is rel_l2 < 1e-5 (tests/sycl_bench.cpp:939-942)
        assert rel_l2(got, want) < 2e-6, (n_keys, rel_l2(got, want))
        assert rel_l2(exact, want) < 2e-6, (n_keys, rel_l2(exact, want))
        assert np.abs(got - want).max() < 2e-6


def test_attention_permuted_table_is_the_same(ob):
    sh = ob.shape(2, 12, 2, ob.KV_F16)
    rng = np.random.default_rng(0)
    n_keys, nb = 75, 9
    perm = rng.permutation(nb)[:5].astype(np.int32)
    pk, pv = ob.new_pools(sh, nb)
    k = rng.standard_normal((n_keys, 2, 128)).astype(np.float16)
    v = rng.standard_normal((n_keys, 2, 128)).astype(np.float16)
    for p in range(n_keys):
        pk[1, perm[p >> 4], p & 15] = k[p]
        pv[1, perm[p >> 4], p & 15] = v[p]
    q = rng.standard_normal((12, 128)).astype(np.float32)
    got = ob.attn_decode_paged(sh, q, pk, pv, perm, 1, nb, n_keys)
    # dense numpy softmax
    want = np.empty_like(got)
    for h in range(12):
        s = (k[:, h // 6].astype(np.float64) @ q[h].astype(np.float64)) * 0.08838834764831845
        w = np.exp(s - s.max())
        want[h] = (w[:, None] * v[:, h // 6].astype(np.float64)).sum(0) / w.sum()
    assert rel_l2(got, want) < 1e-6


def test_gpu_misc_known_answers(ob):
    cs, sn = ob.rope_table(4096)
    assert cs[0, 0] == 1.0 and sn[0, 0] == 0.0                       # gpu_misc.cu:22
    sh = ob.shape(1, 12, 2, ob.KV_F32)
    q = np.sin(np.arange(12 * 128, dtype=np.float32)).reshape(1, 12, 128)
    k = np.cos(np.arange(2 * 128, dtype=np.float32)).reshape(1, 2, 128)
    q0, k0 = q.copy(), k.copy()
    ob.oracle().oracle_rope_batch(__import__("ctypes").byref(sh), q.ctypes.data, k.ctypes.data, 1, 0,
                                  cs.ctypes.data, sn.ctypes.data, 1)
    assert np.abs(q - q0).max() <= 1e-6 and np.abs(k - k0).max() <= 1e-6   # pos 0 is the identity, :39
    # single key: output == V[0] of the head's kv head, :41-65
    pk, pv = ob.new_pools(sh, 1)
    pv[0, 0, 0] = np.sin(np.arange(2 * 128, dtype=np.float32) * 0.001).reshape(2, 128)
    o = ob.attn_decode_paged(sh, np.full((12, 128), 0.5, np.float32), pk, pv, [0], 0, 1, 1)
    for h in range(12):
        assert np.abs(o[h] - pv[0, 0, 0, h // 6]).max() <= 1e-6


@pytest.mark.parametrize("dtype", ["f32", "f16"])
def test_append_addressing_and_rounding(ob, dtype):
    kvd = ob.KV_F16 if dtype == "f16" else ob.KV_F32
    L, NH, NKV, nb = 3, 28, 4, 12
    sh = ob.shape(L, NH, NKV, kvd)
    rng = np.random.default_rng(1)
    cs, sn = ob.rope_table(256)
    table = rng.permutation(nb)[:6].astype(np.int32)
    pk, pv = ob.new_pools(sh, nb)
    n, pos0, layer = 21, 13, 2
    q = rng.standard_normal((n, NH, 128)).astype(np.float32)
    k = rng.standard_normal((n, NKV, 128)).astype(np.float32)
    v = rng.standard_normal((n, NKV, 128)).astype(np.float32)
    q0, k0 = q.copy(), k.copy()
    ob.rope_append_paged(sh, pk, pv, table, layer, nb, n, pos0, q, k, v, cs, sn, fma_mode=0)
    # numpy restatement (rope.cu:38-58 NeoX pairs (i, i+64); elem.cu:59-76 addressing), unfused arithmetic
    for t in range(n):
        c, s = cs[pos0 + t], sn[pos0 + t]
        for src, rot in ((q0[t], q[t]), (k0[t], k[t])):
            x0, x1 = src[:, :64], src[:, 64:]
            assert np.array_equal(rot[:, :64], x0 * c - x1 * s)
            assert np.array_equal(rot[:, 64:], x0 * s + x1 * c)
        phys, slot = table[(pos0 + t) >> 4], (pos0 + t) & 15
        assert np.array_equal(pk[layer, phys, slot], k[t].astype(pk.dtype))
        assert np.array_equal(pv[layer, phys, slot], v[t].astype(pv.dtype))
    assert not pk[:layer].any() and not pv[:layer].any()
    assert np.count_nonzero(pk.reshape(L, -1).any(axis=1)) == 1


def test_fp16_rounding_is_nearest_even(ob):
    rng = np.random.default_rng(2)
    x = np.concatenate([rng.standard_normal(20000).astype(np.float32) * 3,
                        np.float32([0, -0.0, 65504, 65520, 1e-8, 6e-8, 2.0 ** -24, 1 + 2.0 ** -11, 1 + 3 * 2.0 ** -11])])
    with np.errstate(over="ignore"):
        want = x.astype(np.float16).view(np.uint16)
    got = np.array([ob.oracle().oracle_f2h(float(t)) for t in x], dtype=np.uint16)
    assert np.array_equal(got, want)


def test_cow_copy_and_lse_combine(ob):
    sh = ob.shape(4, 12, 2, ob.KV_F16)
    rng = np.random.default_rng(4)
    nb = 6
    pk, pv = ob.new_pools(sh, nb)
    pk[:] = rng.standard_normal(pk.shape).astype(np.float16)
    pv[:] = rng.standard_normal(pv.shape).astype(np.float16)
    k0, v0 = pk.copy(), pv.copy()
    ob.cow_copy(sh, pk, pv, nb, 2, 5)
    assert np.array_equal(pk[:, 5], k0[:, 2]) and np.array_equal(pv[:, 5], v0[:, 2])
    k0[:, 5], v0[:, 5] = k0[:, 2], v0[:, 2]
    assert np.array_equal(pk, k0) and np.array_equal(pv, v0)
    # split the keys of one session over three page ranges, merge, compare with the whole
    n_keys, layer = 83, 1
    table = np.arange(nb, dtype=np.int32)
    q = rng.standard_normal((12, 128)).astype(np.float32)
    whole = ob.attn_decode_paged(sh, q, pk, pv, table, layer, nb, n_keys, exact=True)
    parts = np.stack([ob.attn_partial(sh, q, pk, pv, table, layer, nb, n_keys, a, b) for a, b in ((0, 2), (2, 3), (3, 6))])
    assert rel_l2(ob.lse_combine(parts), whole) < 1e-6
    empty = ob.attn_partial(sh, q, pk, pv, table, layer, nb, n_keys, 6, 6)
    assert np.isneginf(empty[:, 0]).all() and not empty[:, 1:].any()
    assert rel_l2(ob.lse_combine(np.concatenate([parts, empty[None]])), whole) < 1e-6


def test_synth_generator(ob):
    key = ob.synth_key(0x5EED0001, 1, 3, 7)
    a = ob.synth_normal(1 << 16, key)
    assert np.array_equal(a, ob.synth_normal(1 << 16, key))
    assert np.array_equal(a[100:200], ob.synth_normal(100, key, first=100))      # counter-based
    assert abs(a.mean()) < 0.02 and abs(a.std() - 1.0) < 0.02 and np.abs(a).max() < 6
    assert key != ob.synth_key(0x5EED0001, 2, 3, 7)
    # pure-Python restatement of the generator for a few values
    M = (1 << 64) - 1

    def mix(x):
        x = (x + 0x9E3779B97F4A7C15) & M
        x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & M
        x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & M
        return x ^ (x >> 31)

    for i in (0, 1, 77):
        s = 0
        for r in range(3):
            h = mix((key + 3 * i + r) & M)
            s += (h & 0xFFFF) + ((h >> 16) & 0xFFFF) + ((h >> 32) & 0xFFFF) + (h >> 48)
        assert a[i] == np.float32((s - 393210) / 65536.0)


def test_prefill_oracle_is_causal_decode(ob):
    """flash_paged_kernel's restatement == one exact decode attention per query with n_keys = n_past + qi + 1."""
    sh = ob.shape(2, 12, 2, ob.KV_F16)
    rng = np.random.default_rng(6)
    nb, n_past, n_q, layer = 7, 19, 9, 1
    table = rng.permutation(nb).astype(np.int32)
    pk, pv = ob.new_pools(sh, nb)
    pk[:] = rng.standard_normal(pk.shape).astype(np.float16)
    pv[:] = rng.standard_normal(pv.shape).astype(np.float16)
    q = rng.standard_normal((n_q, 12, 128)).astype(np.float32)
    got = ob.attn_prefill_paged(sh, q, pk, pv, table, layer, nb, n_q, n_past)
    for qi in range(n_q):
        want = ob.attn_decode_paged(sh, q[qi], pk, pv, table, layer, nb, n_past + qi + 1, exact=True)
        assert rel_l2(got[qi], want) < 1e-6
