"""Block-ID hashing and BlockRegistry: bit-exact against values computed by the reference's own
code (tests/golden/hash_kats.json, registry_trace.json), its test's properties
(tests/kv_block_test.cpp:7-21) and — where the reference host library is built — against it live."""
import json
import os
import random

import numpy as np

from conftest import GOLDEN


def test_hash_golden(nv):
    kats = json.load(open(os.path.join(GOLDEN, "hash_kats.json")))
    for c in kats["ids"]:
        assert nv.kv_hash_hex(nv.kv_hash_ids(c["ids"])) == c["hex"], c["ids"][:8]
    for c in kats["text"]:
        assert nv.kv_hash_hex(nv.kv_hash_text(bytes.fromhex(c["bytes_hex"]))) == c["hex"]
    for c in kats["block_id"]:
        assert nv.kv_block_id(c["prefix"], c["suffix"]) == c["text"]


def test_hash_survey_kats(nv):
    # values obtained by running the reference's kv_block.h on the inputs of its own unit test
    assert nv.kv_hash_hex(nv.kv_hash_ids([151644, 8948, 198, 2610])) == "956D626F6C666E6A"
    assert nv.kv_hash_hex(nv.kv_hash_ids([151644, 8948, 198, 2611])) == "966D626F6C666E6A"
    assert nv.kv_hash_ids([]) == 0
    assert nv.kv_hash_hex(nv.kv_hash_text("abc")) == "3937393839390000"
    assert nv.kv_block_id(nv.kv_hash_ids([1]), nv.kv_hash_text("abc") ^ 1) == "{ 3100000000000000 . 3937393839390001 }"


def test_hash_properties(nv):
    a, b = [151644, 8948, 198, 2610], [151644, 8948, 198, 2611]
    assert nv.kv_hash_ids(a) == nv.kv_hash_ids(a)          # deterministic
    assert nv.kv_hash_ids(a) != nv.kv_hash_ids(b)          # last digit matters
    assert len(nv.kv_hash_hex(nv.kv_hash_ids(a))) == 16


def test_hash_vs_reference_live(nv, ob):
    r = ob.ref_host()
    if r is None:
        import pytest
        pytest.skip("reference host library not built here")
    rnd = random.Random(3)
    for _ in range(300):
        n = rnd.choice([0, 1, 2, 3, 5, 8, 9, 31, 100, 700])
        ids = np.asarray([rnd.randint(-5, 200000) for _ in range(n)], dtype=np.int32)
        assert nv.kv_hash_ids(ids) == int(r.ref_kv_hash_ids(ids.ctypes.data_as(ob.c_i32p), ids.size))
        raw = bytes(rnd.randint(0, 255) for _ in range(n))
        assert nv.kv_hash_text(raw) == int(r.ref_kv_hash_text(raw, len(raw)))


def test_registry_golden(nv):
    steps = json.load(open(os.path.join(GOLDEN, "registry_trace.json")))
    reg = nv.Registry()
    for st in steps:
        if st["op"] == "cap":
            reg.set_capacity(st["n"])
            assert (reg.live(), reg.total()) == (st["live"], st["total"])
            if "capacity" in st:
                assert reg.capacity() == st["capacity"]
        elif st["op"] == "put":
            reg.put(st["prefix"], st["suffix"], st["session"], st["turn"], st["pos0"], st["pos1"])
            assert (reg.live(), reg.total()) == (st["live"], st["total"])
        else:
            got = reg.find(st["prefix"], st["suffix"])
            assert (got is not None) == bool(st["found"])
            if got:
                assert (got["turn"], got["pos0"]) == (st["turn"], st["pos0"])
