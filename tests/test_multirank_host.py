"""Multi-rank host logic on CPU ranks (gloo, world_size 2 and 3): the page ranges of the long-context
split, the all-gather of per-rank partials and the rank-order LSE merge reproduce the single-rank
attention; a rank whose range holds no key contributes the neutral partial."""
import os
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _worker(rank, world, port, n_keys, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    import __graft_entry__ as g
    g.load_package()
    import conflux_nova_b200.longctx as lc
    from oracle import binding as ob
    NH, NKV, L, layer = 12, 2, 2, 1
    sh = ob.shape(L, NH, NKV, ob.KV_F16)
    rng = np.random.default_rng(5)                     # every rank builds the same session
    nblocks = (n_keys + 15) // 16 + 2
    table = rng.permutation(nblocks).astype(np.int32)
    pk, pv = ob.new_pools(sh, nblocks)
    pk[:] = rng.standard_normal(pk.shape).astype(np.float16)
    pv[:] = rng.standard_normal(pv.shape).astype(np.float16)
    q = rng.standard_normal((NH, 128)).astype(np.float32)
    n_pages = (n_keys + 15) // 16
    lo, hi = lc.page_range(rank, world, n_pages)
    mine = ob.attn_partial(sh, q, pk, pv, table, layer, nblocks, n_keys, lo, min(hi, n_pages))
    allp = lc.gather_partials(torch.from_numpy(mine), world, dist).numpy()
    merged = ob.lse_combine(allp)
    whole = ob.attn_decode_paged(sh, q, pk, pv, table, layer, nblocks, n_keys, exact=True)
    err = float(np.linalg.norm(merged - whole) / np.linalg.norm(whole))
    ranges = [None] * world
    dist.all_gather_object(ranges, (lo, min(hi, n_pages)))
    if rank == 0:
        ret["err"] = err
        ret["ranges"] = ranges
        ret["empty"] = [bool(np.isneginf(allp[r, :, 0]).all() and not allp[r, :, 1:].any()) for r in range(world)]
    dist.destroy_process_group()


@pytest.mark.parametrize("world,n_keys", [(2, 1000), (3, 77), (2, 5)])
def test_long_context_split_matches_single_rank(world, n_keys):
    port = 29600 + world * 10 + n_keys % 7
    with mp.Manager() as m:
        ret = m.dict()
        mp.spawn(_worker, args=(world, port, n_keys, ret), nprocs=world, join=True)
        assert ret["err"] < 1e-6
        ranges = ret["ranges"]
        n_pages = (n_keys + 15) // 16
        assert ranges[0][0] == 0 and ranges[-1][1] == n_pages
        assert all(ranges[i][1] == ranges[i + 1][0] for i in range(world - 1))     # contiguous tiling
        for r, (lo, hi) in enumerate(ranges):
            assert ret["empty"][r] == (lo >= hi)


def test_page_ranges():
    sys.path.insert(0, ROOT)
    import __graft_entry__ as g
    g.load_package()
    import conflux_nova_b200.longctx as lc
    for world in (1, 2, 4, 8):
        for n_pages in (0, 1, 7, 8, 9, 8194):
            r = [lc.page_range(k, world, n_pages) for k in range(world)]
            assert r[0][0] == 0 and r[-1][1] == lc.OPEN_END
            covered = sum(min(hi, n_pages) - lo for lo, hi in r)
            assert covered == n_pages
            for p in range(n_pages):
                o = lc.owner_of_page(p, world, n_pages)
                assert r[o][0] <= p < r[o][1]
