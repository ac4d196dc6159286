"""KvPool parity (tier T0): tables, refcounts, the ORDER of the free lists, cow_count and the
copy request after every operation — against traces recorded from the reference's kv_pool.h
(tests/golden/pool_traces.json) and, where the reference host library is built, against it live on
random operation sequences."""
import json
import os
import random
import zlib

import pytest

from conftest import GOLDEN

ALIAS = {"cow": "cow_slice", "alloc": "alloc_block", "free": "free_block", "ref": "ref_block",
         "clear": "clear_need_copy"}


def state_crc(st):
    return zlib.crc32(json.dumps(st, sort_keys=True).encode())


def apply_op(pool, op, product):
    name, *a = op
    if name == "init":
        pool.init(*a)
        return 0
    r = getattr(pool, ALIAS.get(name, name))(*a)
    return r


def norm_ret(op, r):
    # the product reports argument errors as codes where the reference returns void/0
    if op[0] in ("free", "ref", "clear", "release", "attach", "attach_prefix"):
        return 0 if r is None else min(r, 0) * 0
    return r


def test_pool_traces_golden(nv):
    traces = json.load(open(os.path.join(GOLDEN, "pool_traces.json")))
    assert len(traces) >= 10
    for tr in traces:
        pool = nv.PoolView()
        for op, want_ret, want_crc in zip(tr["ops"], tr["returns"], tr["state_crc"]):
            got = apply_op(pool, op, True)
            if op[0] in ("acquire", "cow", "alloc", "refcnt"):
                assert got == want_ret, (op, got, want_ret)
            assert state_crc(pool.state()) == want_crc, op
        fin = pool.state()
        fin = {k: ({str(kk): vv for kk, vv in v.items()} if isinstance(v, dict) else v) for k, v in fin.items()}
        assert fin == tr["final_state"]


def test_cow_demo_invariants(nv):
    """The reference's COW demo (tests/cow_e2e_demo.cpp:87-105) on the pool alone: exactly one COW on
    the first write into a shared, partly filled tail page, none in the next ten steps, the donor's
    tail page back at refcount 1."""
    p = nv.PoolView()
    p.init(3, 256)
    a, b = p.acquire(), p.acquire()
    Ps = 37
    p.attach_prefix(b, a, Ps)
    tail = p.table(a)[(Ps - 1) >> 4]
    assert p.refcnt(tail) == 2
    c0 = p.cow_count()
    fresh = p.cow_slice(b, Ps)
    assert fresh >= 0 and p.cow_count() - c0 == 1
    assert p.need_copy(b) == (tail, fresh)
    for i in range(1, 11):
        assert p.cow_slice(b, Ps + i) == -1
    assert p.cow_count() - c0 == 1
    assert p.refcnt(tail) == 1 and p.table(a)[(Ps - 1) >> 4] == tail
    assert p.table(b)[(Ps - 1) >> 4] == fresh


def test_pool_errors_are_codes(nv):
    p = nv.PoolView()
    assert nv.lib.nova_pool_init(p.h, 0, 16) == nv.ERR_INVALID
    p.init(1, 32)
    assert p.acquire() == 0
    assert p.acquire() == nv.ERR_NO_SLICE
    assert p.release(5) == nv.ERR_INVALID
    assert p.attach(0, 3, 1) == nv.ERR_INVALID
    assert p.attach(0, 0, 99) == nv.ERR_INVALID      # the reference would run off the table
    assert nv.lib.nova_pool_create(12) is None       # kKvBlock must be 8/16/32/64
    assert nv.PoolView(kv_block=32).init(2, 100) == 0


@pytest.mark.parametrize("kv_block", [16, 8, 32, 64])
@pytest.mark.parametrize("seed", range(8))
def test_pool_vs_reference_live(nv, ob, seed, kv_block):
    """Random operation sequences against the reference's KvPool compiled with the same NOVA_KV_BLOCK
    (code/graph/kv_pool_cfg.h:12-26): every page size the reference allows."""
    if ob.ref_host(kv_block) is None:
        pytest.skip("reference host library not built here")
    if kv_block != 16 and seed >= 4:
        pytest.skip("four sequences per non-default page size")
    rnd = random.Random(seed * 100 + kv_block)
    n_slices, ctx = rnd.randint(2, 7), rnd.choice([16, 48, 100, 160, 2048])
    nblocks = (ctx + kv_block - 1) // kv_block
    mine, ref = nv.PoolView(kv_block=kv_block), ob.RefPool(kv_block)
    mine.init(n_slices, ctx)
    ref.init(n_slices, ctx)
    live = []
    for _ in range(250):
        k = rnd.random()
        if k < 0.2 or not live:
            op = ["acquire"]
        elif k < 0.3:
            op = ["release", rnd.choice(live)]
        elif k < 0.5 and len(live) >= 2:
            d, s = rnd.sample(live, 2)
            op = ["attach_prefix", d, s, rnd.randint(0, ctx)]
        elif k < 0.58 and len(live) >= 2:
            d, s = rnd.sample(live, 2)
            op = ["attach", d, s, rnd.randint(0, nblocks)]
        elif k < 0.93:
            op = ["cow", rnd.choice(live), rnd.randint(0, ctx + 30)]
        elif k < 0.97:
            op = ["clear", rnd.choice(live)]
        else:
            op = ["alloc"]
        a, b = apply_op(mine, op, True), apply_op(ref, op, False)
        if op[0] in ("acquire", "cow", "alloc"):
            assert a == b, (op, a, b)
        if op[0] == "acquire" and b >= 0:
            live.append(b)
        if op[0] == "release":
            live.remove(op[1])
        assert mine.state() == ref.state(), op


def test_slice_reuse_guard(nv):
    """KvPool::acquire resets the count of every identity page of the slice it hands out (kv_pool.h:100-112).  A
    fork that still maps pages of a released parent, or a copy-on-write page taken from a free slice, would then be
    shared with the next owner of that slice unnoticed.  The pool itself stays state-identical to the reference;
    nova_pool_next_slice / nova_pool_foreign_mappings let the session layer see the hazard and refuse."""
    p = nv.PoolView()
    p.init(3, 64)                       # 3 slices x 4 pages
    parent, fork = p.acquire(), p.acquire()
    assert (parent, fork) == (0, 1) and p.next_slice() == 2
    assert p.attach_prefix(fork, parent, 40) == 0          # 3 pages of the parent, the last one half full
    assert p.foreign_mappings(parent) == 3 and p.foreign_mappings(fork) == 0
    p.release(parent)
    assert p.next_slice() == parent                        # LIFO: the parent's slice would be handed out next ...
    assert p.foreign_mappings(parent) == 3                 # ... while the fork still reads three of its pages
    assert [p.refcnt(b) for b in range(4)] == [1, 1, 1, 0]
    # what the guard prevents: acquire would set those counts to 1 with two tables mapping the pages
    fresh = p.cow_slice(fork, 40)                          # the fork un-shares nothing (count is 1): no copy ...
    assert fresh == -1
    p.release(fork)
    assert p.foreign_mappings(parent) == 0                 # ... and once it is gone the slice is safe again
    # a copy-on-write page taken from a free slice is a foreign mapping of that slice too
    a, b = p.acquire(), p.acquire()
    p.set_n_past(a, 20)
    assert p.attach_prefix(b, a, 20) == 0
    spare = p.next_slice()
    page = p.cow_slice(b, 16)
    assert page >= 0 and page // p.nblocks() == spare
    assert p.foreign_mappings(spare) == 1
    assert p.foreign_mappings(99) == nv.ERR_INVALID
