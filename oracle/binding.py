"""ctypes face of the checker libraries (TEST INFRASTRUCTURE).

Only tests/, the smoke check and the bench's CPU-baseline legs import this module; the
product package never does.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import build as _build

KV_F32, KV_F16 = 0, 1
c_i32p = C.POINTER(C.c_int32)
vp, i32, i64, u64, sz = C.c_void_p, C.c_int, C.c_int64, C.c_uint64, C.c_size_t


class Shape(C.Structure):
    _fields_ = [("n_layers", C.c_int32), ("n_heads", C.c_int32), ("n_kv_heads", C.c_int32),
                ("head_dim", C.c_int32), ("kv_block", C.c_int32), ("kv_dtype", C.c_int32),
                ("rope_neox", C.c_int32)]


_oracle = None
_ref_host: dict[int, C.CDLL] = {}
_ref_gpu: dict[str, C.CDLL] = {}


def oracle() -> C.CDLL:
    global _oracle
    if _oracle is None:
        try:
            so = _build.build_oracle()          # no-op when up to date
        except Exception:
            so = _build.ORACLE_SO               # no compiler here: use the prebuilt file
            if not os.path.exists(so):
                raise
        o = C.CDLL(so)
        P = C.POINTER(Shape)
        o.oracle_f2h.restype, o.oracle_f2h.argtypes = C.c_uint16, [C.c_float]
        o.oracle_h2f.restype, o.oracle_h2f.argtypes = C.c_float, [C.c_uint16]
        o.oracle_synth_key.restype, o.oracle_synth_key.argtypes = u64, [u64, u64, u64, u64]
        o.oracle_synth_normal.restype, o.oracle_synth_normal.argtypes = None, [vp, sz, u64, u64]
        o.oracle_rope_table.restype, o.oracle_rope_table.argtypes = None, [vp, vp, i64, i32, i32]
        o.oracle_rope_batch.restype, o.oracle_rope_batch.argtypes = None, [P, vp, vp, i32, i64, vp, vp, i32]
        o.oracle_kv_store_paged.restype = None
        o.oracle_kv_store_paged.argtypes = [P, vp, vp, vp, i32, i32, i32, i64, vp, vp]
        o.oracle_rope_append_paged.restype = None
        o.oracle_rope_append_paged.argtypes = [P, vp, vp, vp, i32, i32, i32, i64, vp, vp, vp, vp, vp, i32]
        o.oracle_cow_copy.restype, o.oracle_cow_copy.argtypes = None, [P, vp, vp, i32, i32, i32]
        o.oracle_attn_decode_paged.restype = None
        o.oracle_attn_decode_paged.argtypes = [P, vp, vp, vp, vp, i32, i32, i32, vp]
        o.oracle_attn_decode_paged_f64.restype = None
        o.oracle_attn_decode_paged_f64.argtypes = [P, vp, vp, vp, vp, i32, i32, i32, vp]
        o.oracle_attn_prefill_paged.restype = None
        o.oracle_attn_prefill_paged.argtypes = [P, vp, vp, vp, vp, i32, i32, i32, i32, i32, vp]
        o.oracle_attn_partial_f64.restype = None
        o.oracle_attn_partial_f64.argtypes = [P, vp, vp, vp, vp, i32, i32, i32, i64, i64, vp]
        o.oracle_lse_combine.restype, o.oracle_lse_combine.argtypes = None, [vp, i32, i32, i32, vp]
        o.oracle_decode_step.restype = None
        o.oracle_decode_step.argtypes = [P, vp, vp, vp, i64, i32, i32, vp, vp, vp, vp, vp, vp, vp, i32, i32, i32, i32]
        o.oracle_num_threads.restype, o.oracle_num_threads.argtypes = i32, []
        o.oracle_set_num_threads.restype, o.oracle_set_num_threads.argtypes = None, [i32]
        _oracle = o
    return _oracle


def ref_host(kv_block: int = 16) -> C.CDLL | None:
    """The reference's own KvPool / kv_block / BlockRegistry behind a C shim (compiled with NOVA_KV_BLOCK =
    kv_block), or None if unbuilt."""
    if kv_block not in _ref_host:
        so = _build.build_ref_host(kv_block=kv_block)
        if so is None:
            return None
        r = C.CDLL(so)
        r.ref_pool_create.restype = vp
        for name in ("ref_pool_destroy",):
            getattr(r, name).restype, getattr(r, name).argtypes = None, [vp]
        r.ref_pool_init.restype, r.ref_pool_init.argtypes = None, [vp, i32, i64]
        for name in ("ref_pool_acquire", "ref_pool_alloc_block", "ref_pool_nb_total", "ref_pool_nblocks",
                     "ref_pool_cow_count", "ref_pool_free_blocks", "ref_pool_free_slices", "ref_pool_used"):
            getattr(r, name).restype, getattr(r, name).argtypes = i32, [vp]
        for name in ("ref_pool_release", "ref_pool_refcnt", "ref_pool_clear_need_copy"):
            getattr(r, name).restype, getattr(r, name).argtypes = i32, [vp, i32]
        for name in ("ref_pool_free_block", "ref_pool_ref_block"):
            getattr(r, name).restype, getattr(r, name).argtypes = None, [vp, i32]
        r.ref_pool_attach.restype, r.ref_pool_attach.argtypes = i32, [vp, i32, i32, i32]
        r.ref_pool_attach_prefix.restype, r.ref_pool_attach_prefix.argtypes = i32, [vp, i32, i32, i64]
        r.ref_pool_cow_slice.restype, r.ref_pool_cow_slice.argtypes = i32, [vp, i32, i64]
        r.ref_pool_need_copy.restype = i32
        r.ref_pool_need_copy.argtypes = [vp, i32, C.POINTER(i32), C.POINTER(i32)]
        r.ref_pool_n_past.restype, r.ref_pool_n_past.argtypes = i64, [vp, i32]
        r.ref_pool_get_table.restype, r.ref_pool_get_table.argtypes = i32, [vp, i32, c_i32p, i32]
        for name in ("ref_pool_get_refcnts", "ref_pool_get_free_list", "ref_pool_get_free_slices",
                     "ref_pool_get_live_slices"):
            getattr(r, name).restype, getattr(r, name).argtypes = i32, [vp, c_i32p, i32]
        r.ref_kv_hash_ids.restype, r.ref_kv_hash_ids.argtypes = u64, [c_i32p, sz]
        r.ref_kv_hash_text.restype, r.ref_kv_hash_text.argtypes = u64, [C.c_char_p, sz]
        r.ref_kv_hash_hex.restype, r.ref_kv_hash_hex.argtypes = None, [u64, C.c_char_p]
        r.ref_kv_block_id.restype, r.ref_kv_block_id.argtypes = None, [u64, u64, C.c_char_p]
        r.ref_registry_create.restype = vp
        r.ref_registry_destroy.restype, r.ref_registry_destroy.argtypes = None, [vp]
        r.ref_registry_set_capacity.restype, r.ref_registry_set_capacity.argtypes = None, [vp, sz]
        r.ref_registry_capacity.restype, r.ref_registry_capacity.argtypes = sz, [vp]
        r.ref_registry_put.restype, r.ref_registry_put.argtypes = None, [vp, vp]
        r.ref_registry_find.restype, r.ref_registry_find.argtypes = i32, [vp, u64, u64, vp]
        r.ref_registry_live.restype, r.ref_registry_live.argtypes = i32, [vp]
        r.ref_registry_total.restype, r.ref_registry_total.argtypes = i32, [vp]
        _ref_host[kv_block] = r
    return _ref_host[kv_block]


def ref_gpu(model: str) -> C.CDLL | None:
    """The reference's CUDA launchers compiled for sm_100a (model: qwen25_7b | qwen25_1p5b), or None."""
    if model not in _ref_gpu:
        so = _build.ref_gpu_so(model)
        if not os.path.exists(so):
            so = _build.build_ref_gpu().get(model)
            if so is None:
                return None
        g = C.CDLL(so)
        g.ref_gpu_shape.restype, g.ref_gpu_shape.argtypes = None, [c_i32p]
        g.ref_gpu_kctx.restype = i32
        g.ref_gpu_rope_table.restype, g.ref_gpu_rope_table.argtypes = None, [vp, vp, vp]
        g.ref_gpu_rope_batch.restype, g.ref_gpu_rope_batch.argtypes = None, [vp, vp, i32, i64, vp, vp, vp]
        g.ref_gpu_rope.restype, g.ref_gpu_rope.argtypes = None, [vp, vp, i64, vp, vp, vp]
        g.ref_gpu_kv_store_paged.restype = None
        g.ref_gpu_kv_store_paged.argtypes = [vp, vp, vp, i32, i32, i32, i64, vp, vp, vp]
        g.ref_gpu_attn_decode_paged.restype = None
        g.ref_gpu_attn_decode_paged.argtypes = [vp, vp, vp, vp, i32, i32, i32, vp, vp, vp]
        g.ref_gpu_attn_decode.restype, g.ref_gpu_attn_decode.argtypes = None, [vp, vp, vp, vp, i32, vp, vp]
        if hasattr(g, "ref_gpu_attn_prefill_paged"):
            g.ref_gpu_attn_prefill_paged.restype = None
            g.ref_gpu_attn_prefill_paged.argtypes = [vp, vp, vp, vp, i32, i32, i32, i32, vp, vp]
        if hasattr(g, "ref_gpu_decode_layer_sessions"):
            g.ref_gpu_decode_layer_sessions.restype = None
            g.ref_gpu_decode_layer_sessions.argtypes = [i32, vp, vp, vp, i32, i32, vp, vp, vp, vp, C.c_size_t, C.c_size_t, vp, vp, vp, vp, vp]
        g.ref_gpu_last_error.restype = i32
        _ref_gpu[model] = g
    return _ref_gpu[model]


_shim: dict[str, C.CDLL] = {}


def shim_exec(model: str) -> C.CDLL | None:
    """The reference's call sites bound to the product library through include/nova_b200_shim.h (oracle/shim_exec.cpp),
    or None if unbuilt.  The product library must be loaded already (the package import does that)."""
    if model not in _shim:
        so = _build.shim_so(model)
        if not os.path.exists(so):
            so = _build.build_shim_exec().get(model)
            if so is None:
                return None
        g = C.CDLL(so)
        g.shim_shape.restype, g.shim_shape.argtypes = None, [c_i32p]
        g.shim_rope_table.restype, g.shim_rope_table.argtypes = None, [vp, vp, vp]
        g.shim_decode_layer.restype = None
        g.shim_decode_layer.argtypes = [vp, vp, vp, vp, vp, vp, i32, i32, i64, vp, vp, vp, vp, vp]
        _shim[model] = g
    return _shim[model]


class RefPool:
    """The reference's KvPool, same method names as the product's PoolView."""

    def __init__(self, kv_block: int = 16):
        self.r = ref_host(kv_block)
        if self.r is None:
            raise RuntimeError("reference host library is not built")
        self.h = self.r.ref_pool_create()

    def __del__(self):
        if getattr(self, "h", None):
            self.r.ref_pool_destroy(self.h)
            self.h = None

    def init(self, n, ctx): self.r.ref_pool_init(self.h, n, ctx)
    def acquire(self): return self.r.ref_pool_acquire(self.h)
    def release(self, s): return self.r.ref_pool_release(self.h, s)
    def alloc_block(self): return self.r.ref_pool_alloc_block(self.h)
    def free_block(self, b): self.r.ref_pool_free_block(self.h, b); return 0
    def ref_block(self, b): self.r.ref_pool_ref_block(self.h, b); return 0
    def refcnt(self, b): return self.r.ref_pool_refcnt(self.h, b)
    def attach(self, d, s, k): return self.r.ref_pool_attach(self.h, d, s, k)
    def attach_prefix(self, d, s, n): return self.r.ref_pool_attach_prefix(self.h, d, s, n)
    def cow_slice(self, s, pos): return self.r.ref_pool_cow_slice(self.h, s, pos)
    def clear_need_copy(self, s): return self.r.ref_pool_clear_need_copy(self.h, s)
    def nb_total(self): return self.r.ref_pool_nb_total(self.h)
    def nblocks(self): return self.r.ref_pool_nblocks(self.h)
    def cow_count(self): return self.r.ref_pool_cow_count(self.h)
    def free_blocks(self): return self.r.ref_pool_free_blocks(self.h)
    def free_slices(self): return self.r.ref_pool_free_slices(self.h)
    def used(self): return self.r.ref_pool_used(self.h)
    def n_past(self, s): return int(self.r.ref_pool_n_past(self.h, s))

    def need_copy(self, s):
        a, b = C.c_int(), C.c_int()
        self.r.ref_pool_need_copy(self.h, s, C.byref(a), C.byref(b))
        return a.value, b.value

    def _dump(self, fn, *pre):
        n = fn(self.h, *pre, None, 0)
        out = np.empty(max(n, 0), dtype=np.int32)
        fn(self.h, *pre, out.ctypes.data_as(c_i32p), n)
        return out

    def table(self, s): return self._dump(self.r.ref_pool_get_table, s)
    def refcnts(self): return self._dump(self.r.ref_pool_get_refcnts)
    def free_list(self): return self._dump(self.r.ref_pool_get_free_list)
    def free_slice_list(self): return self._dump(self.r.ref_pool_get_free_slices)
    def live_slices(self): return self._dump(self.r.ref_pool_get_live_slices)

    def state(self):
        live = self.live_slices().tolist()
        return dict(nb_total=self.nb_total(), nblocks=self.nblocks(), cow_count=self.cow_count(),
                    free_list=self.free_list().tolist(), free_slices=self.free_slice_list().tolist(),
                    refcnts=self.refcnts().tolist(), live=live,
                    tables={s: self.table(s).tolist() for s in live},
                    n_past={s: self.n_past(s) for s in live},
                    need_copy={s: list(self.need_copy(s)) for s in live})


# ------------------------------------------------------------------ numpy-level oracle calls
def _p(a: np.ndarray):
    return a.ctypes.data


def shape(n_layers, n_heads, n_kv_heads, kv_dtype, head_dim=128, kv_block=16, rope_neox=1) -> Shape:
    return Shape(n_layers, n_heads, n_kv_heads, head_dim, kv_block, kv_dtype, rope_neox)


def synth_key(seed, tensor, session=0, layer=0) -> int:
    return int(oracle().oracle_synth_key(seed, tensor, session, layer))


def synth_normal(n: int, key: int, first: int = 0) -> np.ndarray:
    out = np.empty(n, dtype=np.float32)
    oracle().oracle_synth_normal(_p(out), n, key, first)
    return out


def rope_table(n_pos: int, head_dim: int = 128, theta: int = 1000000):
    cs = np.empty((n_pos, head_dim // 2), dtype=np.float32)
    sn = np.empty_like(cs)
    oracle().oracle_rope_table(_p(cs), _p(sn), n_pos, head_dim, theta)
    return cs, sn


def kv_np(sh: Shape):
    return np.float16 if sh.kv_dtype == KV_F16 else np.float32


def new_pools(sh: Shape, nb: int):
    shp = (sh.n_layers, nb, sh.kv_block, sh.n_kv_heads, sh.head_dim)
    return np.zeros(shp, dtype=kv_np(sh)), np.zeros(shp, dtype=kv_np(sh))


def rope_append_paged(sh, pool_k, pool_v, table, layer, nb, n, pos0, q, k, v, cs, sn, fma_mode=1):
    """In place on pool_k/pool_v/q/k (numpy, C-contiguous)."""
    t = np.ascontiguousarray(table, dtype=np.int32)
    oracle().oracle_rope_append_paged(C.byref(sh), _p(pool_k), _p(pool_v), _p(t), layer, nb, n, pos0, _p(q), _p(k),
                                      _p(v), _p(cs), _p(sn), fma_mode)


def cow_copy(sh, pool_k, pool_v, nb, src, dst):
    oracle().oracle_cow_copy(C.byref(sh), _p(pool_k), _p(pool_v), nb, src, dst)


def attn_decode_paged(sh, q, pool_k, pool_v, table, layer, nb, n_keys, exact=False) -> np.ndarray:
    t = np.ascontiguousarray(table, dtype=np.int32)
    o = np.empty((sh.n_heads, sh.head_dim), dtype=np.float32)
    fn = oracle().oracle_attn_decode_paged_f64 if exact else oracle().oracle_attn_decode_paged
    fn(C.byref(sh), _p(q), _p(pool_k), _p(pool_v), _p(t), layer, nb, n_keys, _p(o))
    return o


def attn_prefill_paged(sh, q, pool_k, pool_v, table, layer, nb, n_q, n_past, window=0) -> np.ndarray:
    """q [n_q][NH][HD] -> o, in the arithmetic order of the reference's flash_paged_kernel; window > 0: its sliding-
    window instantiation with that many visible keys (the reference fixes the window at kCtx)."""
    t = np.ascontiguousarray(table, dtype=np.int32)
    qq = np.ascontiguousarray(q, dtype=np.float32)
    o = np.empty_like(qq)
    oracle().oracle_attn_prefill_paged(C.byref(sh), _p(qq), _p(pool_k), _p(pool_v), _p(t), layer, nb, n_q, n_past, window, _p(o))
    return o


def attn_partial(sh, q, pool_k, pool_v, table, layer, nb, n_keys, page0, page1) -> np.ndarray:
    t = np.ascontiguousarray(table, dtype=np.int32)
    part = np.empty((sh.n_heads, sh.head_dim + 2), dtype=np.float32)
    oracle().oracle_attn_partial_f64(C.byref(sh), _p(q), _p(pool_k), _p(pool_v), _p(t), layer, nb, n_keys, page0,
                                     page1, _p(part))
    return part


def lse_combine(parts: np.ndarray) -> np.ndarray:
    n_parts, n_rows, w = parts.shape
    out = np.empty((n_rows, w - 2), dtype=np.float32)
    p = np.ascontiguousarray(parts, dtype=np.float32)
    oracle().oracle_lse_combine(_p(p), n_parts, n_rows, w - 2, _p(out))
    return out


def decode_step(sh, pool_k, pool_v, tables, nb, pos, q, k, v, cs, sn, fma_mode=1, exact=False, layer0=0,
                layer1=None) -> np.ndarray:
    """q,k rotated in place; returns out [L][S][NH][HD] (layers outside [layer0, layer1) untouched)."""
    t = np.ascontiguousarray(tables, dtype=np.int32)
    ps = np.ascontiguousarray(pos, dtype=np.int64)
    out = np.zeros_like(q)
    oracle().oracle_decode_step(C.byref(sh), _p(pool_k), _p(pool_v), _p(t), t.shape[1], nb, t.shape[0], _p(ps), _p(q),
                                _p(k), _p(v), _p(out), _p(cs), _p(sn), fma_mode, int(exact), layer0,
                                sh.n_layers if layer1 is None else layer1)
    return out


def num_threads() -> int:
    return int(oracle().oracle_num_threads())


def use_all_cores() -> int:
    """Let the checker's parallel loops use every core this process may run on (sched_getaffinity), whatever
    OMP_NUM_THREADS says: launchers such as torchrun export OMP_NUM_THREADS=1 to their children.  Returns the count."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    oracle().oracle_set_num_threads(n)
    return num_threads()
