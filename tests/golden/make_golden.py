"""Regenerate the golden fixtures of tests/golden/ from the reference itself.

Run in a container that has the reference tree (see oracle/build.py for how it is found):

    python tests/golden/make_golden.py

Writes
  hash_kats.json        kv_hash_ids / kv_hash_text / kv_block_id values computed by the reference's
                        code/graph/kv_block.h (inputs include those of its tests/kv_block_test.cpp)
  pool_traces.json      scripted and random KvPool operation sequences with the state the
                        reference's code/graph/kv_pool.h reaches after every operation
  registry_trace.json   BlockRegistry (code/graph/kv_registry.h) put/find/evict sequence
  attn_sycl_ref.npz     outputs of the reference's own decode attention
                        (src/kernel/sycl/attn.cpp through tests/host_sycl/sycl/sycl.hpp, on the CPU)
                        for seeded inputs; the inputs are regenerated from the seeds at test time
Nothing of the reference's source is copied; only values it computes are recorded.
"""
from __future__ import annotations

import ctypes as C
import json
import os
import random
import subprocess
import sys
import tempfile
import zlib

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import binding as ob  # noqa: E402
from oracle import build as obuild  # noqa: E402


def state_crc(st: dict) -> int:
    return zlib.crc32(json.dumps(st, sort_keys=True).encode())


def apply_op(pool, op):
    name, *a = op
    if name == "init":
        pool.init(*a)
        return 0
    return getattr(pool, {"cow": "cow_slice", "alloc": "alloc_block", "free": "free_block",
                          "ref": "ref_block", "clear": "clear_need_copy"}.get(name, name))(*a)


def scripted_sequences():
    seqs = []
    # the survey's observed sequence: init(4,2048), two acquires, attach_prefix(b,a,40), cow(b,40)
    seqs.append([["init", 4, 2048], ["acquire"], ["acquire"], ["attach_prefix", 1, 0, 40], ["cow", 1, 40],
                 ["clear", 1], ["cow", 1, 41], ["cow", 0, 40], ["release", 1], ["release", 0], ["acquire"]])
    # the COW demo shape: prefix not on a page boundary, first write un-shares the tail page once
    seqs.append([["init", 3, 256], ["acquire"], ["acquire"], ["attach_prefix", 1, 0, 37], ["cow", 1, 37], ["clear", 1]]
                + [["cow", 1, 38 + i] for i in range(12)] + [["cow", 0, 37], ["release", 0], ["release", 1]])
    # pool exhaustion: every slice acquired, COW has no page to take
    seqs.append([["init", 2, 64], ["acquire"], ["acquire"], ["attach_prefix", 1, 0, 20], ["cow", 1, 20], ["cow", 0, 3]])
    # attach by block count, k = 0 leaves n_past alone
    seqs.append([["init", 3, 128], ["acquire"], ["acquire"], ["attach", 1, 0, 0], ["attach", 1, 0, 3], ["cow", 1, 0],
                 ["cow", 1, 16], ["cow", 1, 47], ["cow", 1, 48], ["release", 0], ["cow", 1, 32], ["release", 1]])
    # slice ids are reused LIFO, acquire beyond capacity fails
    seqs.append([["init", 3, 32], ["acquire"], ["acquire"], ["acquire"], ["acquire"], ["release", 1], ["release", 0],
                 ["acquire"], ["acquire"], ["acquire"]])
    # block-level calls
    seqs.append([["init", 2, 48], ["alloc"], ["alloc"], ["ref", 0], ["free", 0], ["free", 0], ["free", 1], ["alloc"],
                 ["acquire"], ["alloc"], ["alloc"], ["alloc"], ["alloc"], ["free", 99], ["ref", -1], ["refcnt", 2]])
    return seqs


def random_sequence(seed: int, n_ops: int):
    rnd = random.Random(seed)
    n_slices = rnd.randint(2, 6)
    ctx = rnd.choice([16, 40, 64, 100, 128])
    nblocks = (ctx + 15) // 16
    ops = [["init", n_slices, ctx]]
    live: list[int] = []
    ref = ob.RefPool()
    apply_op(ref, ops[0])
    for _ in range(n_ops):
        kind = rnd.random()
        if kind < 0.22 or not live:
            op = ["acquire"]
        elif kind < 0.32:
            op = ["release", rnd.choice(live)]
        elif kind < 0.52 and len(live) >= 2:
            d, s = rnd.sample(live, 2)
            op = ["attach_prefix", d, s, rnd.randint(0, ctx)]
        elif kind < 0.60 and len(live) >= 2:
            d, s = rnd.sample(live, 2)
            op = ["attach", d, s, rnd.randint(0, nblocks)]
        elif kind < 0.95:
            op = ["cow", rnd.choice(live), rnd.randint(0, ctx + 20)]
        else:
            op = ["clear", rnd.choice(live)]
        ops.append(op)
        r = apply_op(ref, op)
        if op[0] == "acquire" and r >= 0:
            live.append(r)
        if op[0] == "release":
            live.remove(op[1])
    return ops


def make_pool_traces():
    traces = []
    seqs = scripted_sequences() + [random_sequence(1000 + i, 60) for i in range(12)]
    for ops in seqs:
        ref = ob.RefPool()
        rets, crcs = [], []
        for op in ops:
            rets.append(int(apply_op(ref, op)))
            crcs.append(state_crc(ref.state()))
        st = ref.state()
        st["tables"] = {str(k): v for k, v in st["tables"].items()}
        st["n_past"] = {str(k): v for k, v in st["n_past"].items()}
        st["need_copy"] = {str(k): v for k, v in st["need_copy"].items()}
        traces.append(dict(ops=ops, returns=rets, state_crc=crcs, final_state=st))
    return traces


def make_hash_kats():
    r = ob.ref_host()
    rnd = random.Random(5)
    id_cases = [[], [1], [151644], [151644, 8948, 198, 2610], [151644, 8948, 198, 2611], list(range(1, 11)),
                [0], [-7, 12], [2147483647, -2147483648], [9] * 8, [12345678], [123456789],
                list(range(151640, 151700))]
    for n in (3, 17, 64, 257, 1000):
        id_cases.append([rnd.randint(0, 151935) for _ in range(n)])
    text_cases = ["", "abc", "hello world", "用一句话说明什么是导数", "a" * 8, "a" * 9, "\x00\x01\xff"]
    out = {"ids": [], "text": [], "block_id": []}
    buf = C.create_string_buffer(17)
    for ids in id_cases:
        a = np.asarray(ids, dtype=np.int32)
        h = int(r.ref_kv_hash_ids(a.ctypes.data_as(ob.c_i32p), a.size))
        r.ref_kv_hash_hex(h, buf)
        out["ids"].append(dict(ids=ids, hex=buf.value.decode()))
    for t in text_cases:
        b = t.encode("utf-8") if t != "\x00\x01\xff" else b"\x00\x01\xff"
        h = int(r.ref_kv_hash_text(b, len(b)))
        r.ref_kv_hash_hex(h, buf)
        out["text"].append(dict(bytes_hex=b.hex(), hex=buf.value.decode()))
    b40 = C.create_string_buffer(64)
    for p, s in [(0, 0), (0x3100000000000000, 0x3937393839390001), (0xFFFFFFFFFFFFFFFF, 0x0123456789ABCDEF)]:
        r.ref_kv_block_id(p, s, b40)
        out["block_id"].append(dict(prefix=p, suffix=s, text=b40.value.decode()))
    return out


def make_registry_trace():
    r = ob.ref_host()

    class Blk(C.Structure):
        _fields_ = [("prefix", C.c_uint64), ("suffix", C.c_uint64), ("session", C.c_int32), ("turn", C.c_int32),
                    ("pos0", C.c_int64), ("pos1", C.c_int64)]

    h = r.ref_registry_create()
    rnd = random.Random(11)
    steps = []
    r.ref_registry_set_capacity(h, 5)
    steps.append(dict(op="cap", n=5, live=r.ref_registry_live(h), total=r.ref_registry_total(h)))
    for i in range(40):
        p, s = rnd.randint(0, 5), rnd.randint(0, 3)
        if rnd.random() < 0.6:
            b = Blk(p, s, i % 4, i, i * 10, i * 10 + 7)
            r.ref_registry_put(h, C.byref(b))
            steps.append(dict(op="put", prefix=p, suffix=s, session=i % 4, turn=i, pos0=i * 10, pos1=i * 10 + 7,
                              live=r.ref_registry_live(h), total=r.ref_registry_total(h)))
        else:
            o = Blk()
            f = r.ref_registry_find(h, p, s, C.byref(o))
            steps.append(dict(op="find", prefix=p, suffix=s, found=int(f), turn=int(o.turn) if f else None,
                              pos0=int(o.pos0) if f else None))
        if i == 25:
            r.ref_registry_set_capacity(h, 2)
            steps.append(dict(op="cap", n=2, live=r.ref_registry_live(h), total=r.ref_registry_total(h)))
    r.ref_registry_set_capacity(h, 0)
    steps.append(dict(op="cap", n=0, live=r.ref_registry_live(h), total=r.ref_registry_total(h),
                      capacity=int(r.ref_registry_capacity(h))))
    r.ref_registry_destroy(h)
    return steps


SYCL_MODELS = {"qwen25_1p5b": ("NOVA_SYCL_MODEL_QWEN25_1P5B", 12, 2), "qwen25_7b": ("NOVA_SYCL_MODEL_R1_QWEN7B", 28, 4)}
ATTN_CASES = {"qwen25_1p5b": [1, 2, 10, 31, 32, 33, 100, 257], "qwen25_7b": [1, 17, 64, 130]}
ATTN_SEED = 0x5EED0000


def attn_inputs(model: str, n_keys: int):
    """Seeded inputs of one attention fixture: q ~ N(0,1); K, V ~ 0.7 N(0,1) as in the reference's
    own check (tests/sycl_bench.cpp:897-899 scales K and V by 0.7)."""
    _, NH, NKV = SYCL_MODELS[model]
    q = ob.synth_normal(NH * 128, ob.synth_key(ATTN_SEED, 3, n_keys, NH))
    k = ob.synth_normal(n_keys * NKV * 128, ob.synth_key(ATTN_SEED, 1, n_keys, NH)) * np.float32(0.7)
    v = ob.synth_normal(n_keys * NKV * 128, ob.synth_key(ATTN_SEED, 2, n_keys, NH)) * np.float32(0.7)
    return q, k.astype(np.float32), v.astype(np.float32)


def make_attn_fixtures():
    ref = obuild.reference_dir()
    out = {}
    with tempfile.TemporaryDirectory() as tmp:
        for model, (macro, NH, NKV) in SYCL_MODELS.items():
            exe = os.path.join(tmp, f"drv_{model}")
            subprocess.run(["g++", "-std=c++17", "-O2", "-pthread", "-w", "-include", "cstring", f"-D{macro}",
                            "-DNOVA_SYCL_SG=32", f"-I{ref}/tests/host_sycl", f"-I{ref}/include", f"-I{ref}/code",
                            f"-I{ref}/code/device/sycl", f"-I{ref}/src/kernel/sycl",
                            os.path.join(HERE, "ref_sycl_attn_driver.cpp"), "-o", exe], check=True)
            for n_keys in ATTN_CASES[model]:
                q, k, v = attn_inputs(model, n_keys)
                fin, fout = os.path.join(tmp, "in.bin"), os.path.join(tmp, "out.bin")
                with open(fin, "wb") as f:
                    f.write(np.int32(n_keys).tobytes() + q.tobytes() + k.tobytes() + v.tobytes())
                r = subprocess.run([exe, fin, fout], check=True, capture_output=True, text=True)
                assert f"NH={NH} NKV={NKV}" in r.stdout, r.stdout
                out[f"{model}/{n_keys}"] = np.fromfile(fout, dtype=np.float32).reshape(NH, 128)
                print(model, n_keys, "ok")
    return out


def main():
    if obuild.reference_dir() is None:
        sys.exit("reference tree not found; fixtures can only be regenerated where it is present")
    json.dump(make_hash_kats(), open(os.path.join(HERE, "hash_kats.json"), "w"), indent=0)
    json.dump(make_pool_traces(), open(os.path.join(HERE, "pool_traces.json"), "w"))
    json.dump(make_registry_trace(), open(os.path.join(HERE, "registry_trace.json"), "w"), indent=0)
    np.savez_compressed(os.path.join(HERE, "attn_sycl_ref.npz"), **make_attn_fixtures())
    print("fixtures written to", HERE)


if __name__ == "__main__":
    main()
