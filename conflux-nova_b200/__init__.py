"""conflux_nova_b200 — Python face of libnova_b200.so (ctypes over the C ABI of include/nova_b200.h).

The directory name carries a hyphen, so it is loaded through `__graft_entry__.load_package()`
(importlib with an explicit path) under the module name `conflux_nova_b200`.

Nothing here computes: every call goes to the shared library, which holds the hand-written
sm_100a kernels.  If the library is missing the import fails — there is no fallback path.
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("NOVA_B200_LIB") or os.path.join(HERE, "libnova_b200.so")   # override: try another build

OK = 0
ERR_INVALID, ERR_POOL_FULL, ERR_NO_SLICE, ERR_NO_SESSION, ERR_CUDA = -1, -2, -3, -4, -5
ERR_BAD_TABLE, ERR_TIMEOUT, ERR_UNSUPPORTED, ERR_TOO_LARGE, ERR_BUSY = -6, -7, -8, -9, -10
KV_F32, KV_F16 = 0, 1

c_i32p = C.POINTER(C.c_int32)
c_f32p = C.POINTER(C.c_float)


class EngineDesc(C.Structure):
    _fields_ = [("n_layers", C.c_int32), ("n_heads", C.c_int32), ("n_kv_heads", C.c_int32),
                ("head_dim", C.c_int32), ("kv_block", C.c_int32), ("kv_dtype", C.c_int32),
                ("rope_theta", C.c_int32), ("rope_neox", C.c_int32), ("n_slices", C.c_int32),
                ("max_sessions", C.c_int32), ("ctx", C.c_int64), ("rope_positions", C.c_int64),
                ("device", C.c_int32), ("zero_pages", C.c_int32)]


class Telemetry(C.Structure):
    _fields_ = [("blocks_total", C.c_int32), ("blocks_free", C.c_int32), ("blocks_shared", C.c_int32),
                ("cow_count", C.c_int32), ("sessions_live", C.c_int32), ("slices_free", C.c_int32),
                ("kv_bytes_cap", C.c_uint64), ("kv_bytes_used", C.c_uint64)]


class KvShape(C.Structure):
    _fields_ = [("n_heads", C.c_int32), ("n_kv_heads", C.c_int32), ("head_dim", C.c_int32),
                ("kv_block", C.c_int32), ("kv_dtype", C.c_int32), ("rope_neox", C.c_int32)]


class KvBlock(C.Structure):
    _fields_ = [("prefix", C.c_uint64), ("suffix", C.c_uint64), ("session", C.c_int32),
                ("turn", C.c_int32), ("pos0", C.c_int64), ("pos1", C.c_int64)]


vp, i32, i64, u64, sz = C.c_void_p, C.c_int, C.c_int64, C.c_uint64, C.c_size_t

# name -> (restype, argtypes); the full export list of include/nova_b200.h
SIGNATURES = {
    "nova_status_string": (C.c_char_p, [i32]),
    "nova_last_cuda_error": (C.c_char_p, []),
    "dev_select": (i32, [i32]), "dev_count": (i32, []),
    "dev_alloc": (vp, [sz]), "dev_free": (None, [vp]),
    "dev_upload": (i32, [vp, vp, sz]), "dev_download": (i32, [vp, vp, sz]),
    "dev_zero": (i32, [vp, sz]), "dev_sync": (i32, []), "dev_max_alloc": (sz, []),
    "dev_host_alloc": (vp, [sz]), "dev_host_free": (None, [vp]),
    "dev_ipc_export": (i32, [vp, vp]), "dev_ipc_open": (i32, [vp, C.POINTER(vp)]), "dev_ipc_close": (i32, [vp]),
    "dev_stream_create": (i32, [C.POINTER(vp)]), "dev_stream_destroy": (i32, [vp]),
    "dev_stream_sync": (i32, [vp]),
    "dev_event_create": (i32, [C.POINTER(vp)]), "dev_event_destroy": (i32, [vp]),
    "dev_event_record": (i32, [vp, vp]), "dev_event_sync": (i32, [vp]),
    "dev_event_elapsed_ms": (i32, [vp, vp, C.POINTER(C.c_float)]),
    "nova_kv_hash_ids": (u64, [c_i32p, sz]), "nova_kv_hash_text": (u64, [C.c_char_p, sz]),
    "nova_kv_hash_hex": (None, [u64, C.c_char_p]), "nova_kv_block_id": (None, [u64, u64, C.c_char_p]),
    "nova_registry_create": (vp, []), "nova_registry_destroy": (None, [vp]),
    "nova_registry_set_capacity": (None, [vp, sz]), "nova_registry_capacity": (sz, [vp]),
    "nova_registry_put": (None, [vp, C.POINTER(KvBlock)]),
    "nova_registry_find": (i32, [vp, u64, u64, C.POINTER(KvBlock)]),
    "nova_registry_live": (i32, [vp]), "nova_registry_total": (i32, [vp]),
    "nova_pool_create": (vp, [i32]), "nova_pool_destroy": (None, [vp]),
    "nova_pool_init": (i32, [vp, i32, i64]), "nova_pool_acquire": (i32, [vp]),
    "nova_pool_release": (i32, [vp, i32]), "nova_pool_alloc_block": (i32, [vp]),
    "nova_pool_free_block": (i32, [vp, i32]), "nova_pool_ref_block": (i32, [vp, i32]),
    "nova_pool_refcnt": (i32, [vp, i32]), "nova_pool_attach": (i32, [vp, i32, i32, i32]),
    "nova_pool_attach_prefix": (i32, [vp, i32, i32, i64]), "nova_pool_cow_slice": (i32, [vp, i32, i64]),
    "nova_pool_need_copy": (i32, [vp, i32, C.POINTER(i32), C.POINTER(i32)]),
    "nova_pool_clear_need_copy": (i32, [vp, i32]),
    "nova_pool_next_slice": (i32, [vp]), "nova_pool_foreign_mappings": (i32, [vp, i32]),
    "nova_pool_nb_total": (i32, [vp]), "nova_pool_nblocks": (i32, [vp]), "nova_pool_cow_count": (i32, [vp]),
    "nova_pool_free_blocks": (i32, [vp]), "nova_pool_free_slices": (i32, [vp]), "nova_pool_used": (i32, [vp]),
    "nova_pool_n_past": (i64, [vp, i32]), "nova_pool_set_n_past": (i32, [vp, i32, i64]),
    "nova_pool_get_table": (i32, [vp, i32, c_i32p, i32]), "nova_pool_get_refcnts": (i32, [vp, c_i32p, i32]),
    "nova_pool_get_free_list": (i32, [vp, c_i32p, i32]), "nova_pool_get_free_slices": (i32, [vp, c_i32p, i32]),
    "nova_pool_get_live_slices": (i32, [vp, c_i32p, i32]),
    "nova_engine_create": (i32, [C.POINTER(EngineDesc), C.POINTER(vp)]), "nova_engine_destroy": (None, [vp]),
    "nova_engine_desc_get": (i32, [vp, C.POINTER(EngineDesc)]),
    "nova_kv_k_base": (vp, [vp]), "nova_kv_v_base": (vp, [vp]), "nova_kv_table_slot": (vp, [vp, i32]),
    "nova_kv_nb": (i32, [vp]), "nova_kv_nblocks": (i32, [vp]), "nova_kv_width": (i32, [vp]),
    "nova_kv_page_bytes": (sz, [vp]), "nova_rope_cos": (vp, [vp]), "nova_rope_sin": (vp, [vp]),
    "nova_engine_pool": (vp, [vp]),
    "nova_session_create": (i32, [vp]), "nova_session_destroy": (i32, [vp, i32]),
    "nova_session_live_count": (i32, [vp]), "nova_session_slice": (i32, [vp, i32]),
    "nova_session_stream": (vp, [vp, i32]), "nova_session_n_past": (i64, [vp, i32]),
    "nova_session_set_n_past": (i32, [vp, i32, i64]),
    "nova_session_attach": (i32, [vp, i32, i32, i32]), "nova_session_attach_prefix": (i32, [vp, i32, i32, i64]),
    "nova_session_cow": (i32, [vp, i32, i64, i32]), "nova_session_cow_on": (i32, [vp, i32, i64, i32, vp]),
    "nova_session_permute_pages": (i32, [vp, i32, c_i32p, i32]), "nova_session_sync_table": (i32, [vp, i32]),
    "nova_launch_rope_table": (i32, [vp, vp, i64, i32, i32, vp]),
    "nova_launch_rope_append_paged": (i32, [C.POINTER(KvShape), vp, vp, vp, i32, i32, i32, i64, vp, vp, vp, vp, vp, vp]),
    "nova_attn_scratch_floats": (sz, [C.POINTER(KvShape)]),
    "nova_launch_attn_decode_paged": (i32, [C.POINTER(KvShape), vp, vp, vp, vp, i32, i32, i32, vp, vp, vp]),
    "nova_attn_static_scratch_max_heads": (sz, []),
    "nova_launch_attn_decode_paged_static": (i32, [C.POINTER(KvShape), vp, vp, vp, vp, i32, i32, i32, vp, vp]),
    "nova_synth_key": (u64, [u64, u64, u64, u64]), "nova_synth_normal": (i32, [vp, sz, u64, u64, vp]),
    "nova_batch_create": (i32, [vp, c_i32p, i32, C.POINTER(vp)]), "nova_batch_destroy": (None, [vp]),
    "nova_batch_size": (i32, [vp]), "nova_batch_sync_positions": (i32, [vp, vp]),
    "nova_batch_set_timeline": (i32, [vp, vp]), "nova_launcher_set_kernel": (i32, [i32]),
    "nova_launch_decode_layer_sessions": (i32, [vp, i32, vp, vp, vp, i32, i32, vp, vp, vp, vp, C.c_size_t, C.c_size_t, vp, vp, vp, vp, vp]),
    "nova_batch_set_pdl": (i32, [vp, i32]), "nova_batch_set_row_setup_pages": (i32, [vp, i32]),
    "nova_batch_set_split_ctas": (i32, [vp, i32]), "nova_batch_set_window": (i32, [vp, i32]), "nova_batch_set_prefill_kernel": (i32, [vp, i32]),
    "nova_batch_set_fused_append": (i32, [vp, i32]), "nova_batch_append_attn": (i32, [vp, i32, vp, vp, vp, vp, vp]),
    "nova_batch_set_kernel": (i32, [vp, i32]), "nova_batch_get_kernel": (i32, [vp]),
    "nova_batch_cow": (i32, [vp, vp]), "nova_batch_append": (i32, [vp, i32, vp, vp, vp, vp]),
    "nova_batch_append_layers": (i32, [vp, i32, i32, vp, vp, vp, vp]),
    "nova_batch_attn": (i32, [vp, i32, vp, vp, vp]), "nova_batch_advance": (i32, [vp, vp]),
    "nova_batch_prefill_max_tokens": (i32, [vp]), "nova_batch_advance_by": (i32, [vp, i32, vp]),
    "nova_batch_prefill": (i32, [vp, i32, i32, vp, vp, vp, vp, vp]),
    "nova_batch_step_all_layers": (i32, [vp, vp, vp, vp, vp, vp]),
    "nova_batch_decode_step_host": (i32, [vp, vp, vp, vp, vp, i32, vp]), "nova_batch_host_wait": (i32, [vp, vp]),
    "nova_batch_run_steps": (i32, [vp, i32, vp, vp, vp, vp, sz, sz, i32, C.POINTER(C.c_float), vp]),
    "nova_batch_device_status": (i32, [vp]), "nova_launch_count": (u64, []),
    "nova_batch_attn_partial": (i32, [vp, i32, vp, i64, i64, vp, vp]),
    "nova_batch_attn_partial_layers": (i32, [vp, i32, i32, vp, i64, i64, vp, vp]),
    "nova_lse_combine": (i32, [vp, i32, i32, i32, vp, vp]),
    "nova_peer_slot_bytes": (sz, [i32]),
    "nova_session_fork": (i32, [vp, i32]), "nova_session_attach_block": (i64, [vp, vp, u64, u64, i32]),
    "nova_engine_telemetry": (i32, [vp, C.POINTER(Telemetry)]),
    "nova_batch_set_cascade": (i32, [vp, i32]), "nova_batch_shared_prefix_pages": (i32, [vp]),
    "nova_batch_step_partial_peers": (i32, [vp, vp, vp, vp, i64, i64, C.POINTER(vp), i32, i32, sz, i32, i64, i32, vp, vp, vp]),
    "nova_lse_merge_peers": (i32, [vp, C.POINTER(vp), i32, i32, sz, i32, i32, i64, i32, vp, vp, vp]),
}


class NovaError(RuntimeError):
    def __init__(self, code: int, what: str = ""):
        self.code = code
        msg = lib.nova_status_string(code).decode() if lib is not None else str(code)
        if code == ERR_CUDA and lib is not None:
            msg += ": " + lib.nova_last_cuda_error().decode()
        super().__init__(f"{what}: {msg} ({code})" if what else f"{msg} ({code})")


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(f"{LIB_PATH} is not built; run `python -c 'import __graft_entry__ as g; g.build()'`")
    handle = C.CDLL(LIB_PATH, mode=C.RTLD_GLOBAL)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(handle, name)          # AttributeError if a declared symbol is not exported
        fn.restype = res
        fn.argtypes = args
    return handle


lib = None
lib = _load()


def check(rc: int, what: str = "") -> int:
    if rc < 0:
        raise NovaError(rc, what)
    return rc


# --------------------------------------------------------------------------- host-only helpers
def kv_hash_ids(ids) -> int:
    a = np.ascontiguousarray(ids, dtype=np.int32)
    return int(lib.nova_kv_hash_ids(a.ctypes.data_as(c_i32p), a.size))


def kv_hash_text(text) -> int:
    b = text.encode("utf-8") if isinstance(text, str) else bytes(text)
    return int(lib.nova_kv_hash_text(b, len(b)))


def kv_hash_hex(v: int) -> str:
    buf = C.create_string_buffer(17)
    lib.nova_kv_hash_hex(v, buf)
    return buf.value.decode()


def kv_block_id(prefix: int, suffix: int) -> str:
    buf = C.create_string_buffer(40)
    lib.nova_kv_block_id(prefix, suffix, buf)
    return buf.value.decode()


class Registry:
    """BlockRegistry (code/graph/kv_registry.h:26-66 of the reference)."""

    def __init__(self):
        self.h = lib.nova_registry_create()

    def __del__(self):
        if getattr(self, "h", None) and lib is not None:
            lib.nova_registry_destroy(self.h)
            self.h = None

    def set_capacity(self, n): lib.nova_registry_set_capacity(self.h, n)
    def capacity(self): return int(lib.nova_registry_capacity(self.h))
    def live(self): return lib.nova_registry_live(self.h)
    def total(self): return lib.nova_registry_total(self.h)

    def put(self, prefix, suffix, session=-1, turn=0, pos0=0, pos1=0):
        b = KvBlock(prefix, suffix, session, turn, pos0, pos1)
        lib.nova_registry_put(self.h, C.byref(b))

    def find(self, prefix, suffix):
        b = KvBlock()
        if not lib.nova_registry_find(self.h, prefix, suffix, C.byref(b)):
            return None
        return dict(prefix=b.prefix, suffix=b.suffix, session=b.session, turn=b.turn, pos0=b.pos0, pos1=b.pos1)


class PoolView:
    """KvPool (code/graph/kv_pool.h:68-197) through the C ABI; `h` is a nova_pool*."""

    def __init__(self, h=None, kv_block=16):
        self.own = h is None
        self.h = lib.nova_pool_create(kv_block) if h is None else h
        if not self.h:
            raise NovaError(ERR_INVALID, "nova_pool_create")

    def __del__(self):
        if getattr(self, "own", False) and getattr(self, "h", None) and lib is not None:
            lib.nova_pool_destroy(self.h)
            self.h = None

    def init(self, n_slices, ctx): return check(lib.nova_pool_init(self.h, n_slices, ctx), "pool_init")
    def acquire(self): return lib.nova_pool_acquire(self.h)
    def release(self, s): return lib.nova_pool_release(self.h, s)
    def alloc_block(self): return lib.nova_pool_alloc_block(self.h)
    def free_block(self, b): return lib.nova_pool_free_block(self.h, b)
    def ref_block(self, b): return lib.nova_pool_ref_block(self.h, b)
    def refcnt(self, b): return lib.nova_pool_refcnt(self.h, b)
    def attach(self, d, s, k): return lib.nova_pool_attach(self.h, d, s, k)
    def attach_prefix(self, d, s, n): return lib.nova_pool_attach_prefix(self.h, d, s, n)
    def cow_slice(self, s, pos): return lib.nova_pool_cow_slice(self.h, s, pos)
    def clear_need_copy(self, s): return lib.nova_pool_clear_need_copy(self.h, s)
    def nb_total(self): return lib.nova_pool_nb_total(self.h)
    def nblocks(self): return lib.nova_pool_nblocks(self.h)
    def cow_count(self): return lib.nova_pool_cow_count(self.h)
    def free_blocks(self): return lib.nova_pool_free_blocks(self.h)
    def free_slices(self): return lib.nova_pool_free_slices(self.h)
    def used(self): return lib.nova_pool_used(self.h)
    def next_slice(self): return lib.nova_pool_next_slice(self.h)
    def foreign_mappings(self, s): return lib.nova_pool_foreign_mappings(self.h, s)
    def n_past(self, s): return int(lib.nova_pool_n_past(self.h, s))
    def set_n_past(self, s, n): return lib.nova_pool_set_n_past(self.h, s, n)

    def need_copy(self, s):
        a, b = C.c_int(), C.c_int()
        check(lib.nova_pool_need_copy(self.h, s, C.byref(a), C.byref(b)), "need_copy")
        return a.value, b.value

    def _dump(self, fn, *pre):
        n = fn(self.h, *pre, None, 0)
        if n < 0:
            raise NovaError(n, fn.__name__)
        out = np.empty(n, dtype=np.int32)
        fn(self.h, *pre, out.ctypes.data_as(c_i32p), n)
        return out

    def table(self, s): return self._dump(lib.nova_pool_get_table, s)
    def refcnts(self): return self._dump(lib.nova_pool_get_refcnts)
    def free_list(self): return self._dump(lib.nova_pool_get_free_list)
    def free_slice_list(self): return self._dump(lib.nova_pool_get_free_slices)
    def live_slices(self): return self._dump(lib.nova_pool_get_live_slices)

    def state(self):
        """Everything a parity diff looks at, as plain Python."""
        live = self.live_slices().tolist()
        return dict(nb_total=self.nb_total(), nblocks=self.nblocks(), cow_count=self.cow_count(),
                    free_list=self.free_list().tolist(), free_slices=self.free_slice_list().tolist(),
                    refcnts=self.refcnts().tolist(), live=live,
                    tables={s: self.table(s).tolist() for s in live},
                    n_past={s: self.n_past(s) for s in live},
                    need_copy={s: list(self.need_copy(s)) for s in live})


# ------------------------------------------------------------------------------ device helpers
class DevBuf:
    """A device allocation from the HAL (dev_alloc / dev_free)."""

    def __init__(self, nbytes: int):
        self.nbytes = int(nbytes)
        self.ptr = lib.dev_alloc(self.nbytes) if nbytes else None
        if nbytes and not self.ptr:
            raise NovaError(ERR_CUDA, f"dev_alloc({nbytes})")

    def free(self):
        if self.ptr:
            lib.dev_free(self.ptr)
            self.ptr = None

    def __del__(self):
        if lib is not None:
            self.free()

    def upload(self, arr: np.ndarray, offset: int = 0):
        a = np.ascontiguousarray(arr)
        assert offset + a.nbytes <= self.nbytes
        check(lib.dev_upload(self.ptr + offset, a.ctypes.data, a.nbytes), "dev_upload")
        return self

    def download(self, dtype, count: int | None = None, offset: int = 0) -> np.ndarray:
        dt = np.dtype(dtype)
        n = (self.nbytes - offset) // dt.itemsize if count is None else count
        out = np.empty(n, dtype=dt)
        check(lib.dev_download(out.ctypes.data, self.ptr + offset, out.nbytes), "dev_download")
        return out

    def zero(self):
        check(lib.dev_zero(self.ptr, self.nbytes), "dev_zero")
        return self


def to_device(arr: np.ndarray) -> DevBuf:
    a = np.ascontiguousarray(arr)
    return DevBuf(a.nbytes).upload(a)


def download_ptr(ptr: int, dtype, count: int) -> np.ndarray:
    out = np.empty(count, dtype=np.dtype(dtype))
    check(lib.dev_download(out.ctypes.data, ptr, out.nbytes), "dev_download")
    return out


class Stream:
    def __init__(self):
        h = vp()
        check(lib.dev_stream_create(C.byref(h)), "dev_stream_create")
        self.h = h

    def sync(self): check(lib.dev_stream_sync(self.h), "dev_stream_sync")

    def close(self):
        if getattr(self, "h", None):
            lib.dev_stream_destroy(self.h)
            self.h = None


class Event:
    def __init__(self):
        h = vp()
        check(lib.dev_event_create(C.byref(h)), "dev_event_create")
        self.h = h

    def record(self, stream=None): check(lib.dev_event_record(self.h, stream.h if isinstance(stream, Stream) else stream))
    def sync(self): check(lib.dev_event_sync(self.h))

    def elapsed_ms(self, later: "Event") -> float:
        ms = C.c_float()
        check(lib.dev_event_elapsed_ms(self.h, later.h, C.byref(ms)))
        return float(ms.value)


def synth_key(seed, tensor, session=0, layer=0) -> int:
    return int(lib.nova_synth_key(seed, tensor, session, layer))


class Engine:
    """Pools + tables + RoPE tables + sessions of one GPU (nova_engine)."""

    def __init__(self, n_layers, n_heads, n_kv_heads, *, ctx, n_slices, kv_dtype=KV_F16, head_dim=128,
                 kv_block=16, rope_theta=1000000, rope_neox=1, max_sessions=0, rope_positions=0, device=0,
                 zero_pages=1):
        self.desc = EngineDesc(n_layers, n_heads, n_kv_heads, head_dim, kv_block, kv_dtype, rope_theta, rope_neox,
                               n_slices, max_sessions, ctx, rope_positions, device, zero_pages)
        h = vp()
        check(lib.nova_engine_create(C.byref(self.desc), C.byref(h)), "nova_engine_create")
        self.h = h
        check(lib.nova_engine_desc_get(self.h, C.byref(self.desc)))
        self.pool = PoolView(lib.nova_engine_pool(self.h))
        self.kv_np = np.float16 if kv_dtype == KV_F16 else np.float32

    def close(self):
        if getattr(self, "h", None):
            lib.nova_engine_destroy(self.h)
            self.h = None

    def __del__(self):
        if lib is not None:
            self.close()

    # shape
    @property
    def L(self): return self.desc.n_layers
    @property
    def NH(self): return self.desc.n_heads
    @property
    def NKV(self): return self.desc.n_kv_heads
    @property
    def HD(self): return self.desc.head_dim
    @property
    def nb(self): return lib.nova_kv_nb(self.h)
    @property
    def nblocks(self): return lib.nova_kv_nblocks(self.h)
    @property
    def page_bytes(self): return int(lib.nova_kv_page_bytes(self.h))
    @property
    def k_base(self): return lib.nova_kv_k_base(self.h)
    @property
    def v_base(self): return lib.nova_kv_v_base(self.h)
    def shape(self) -> KvShape:
        d = self.desc
        return KvShape(d.n_heads, d.n_kv_heads, d.head_dim, d.kv_block, d.kv_dtype, d.rope_neox)

    # sessions
    def session_create(self): return check(lib.nova_session_create(self.h), "nova_session_create")
    def session_destroy(self, s): return check(lib.nova_session_destroy(self.h, s), "nova_session_destroy")
    def session_slice(self, s): return check(lib.nova_session_slice(self.h, s))
    def session_stream(self, s): return lib.nova_session_stream(self.h, s)
    def n_past(self, s): return int(lib.nova_session_n_past(self.h, s))
    def set_n_past(self, s, n): return check(lib.nova_session_set_n_past(self.h, s, n))
    def attach(self, d, s, k): return check(lib.nova_session_attach(self.h, d, s, k), "session_attach")
    def attach_prefix(self, d, s, n): return check(lib.nova_session_attach_prefix(self.h, d, s, n), "attach_prefix")
    def cow(self, s, pos0, n): return check(lib.nova_session_cow(self.h, s, pos0, n), "session_cow")

    def permute_pages(self, s, perm):
        p = np.ascontiguousarray(perm, dtype=np.int32)
        return check(lib.nova_session_permute_pages(self.h, s, p.ctypes.data_as(c_i32p), p.size), "permute_pages")

    # raw views (host copies)
    def rope_tables(self):
        n = self.desc.rope_positions * (self.HD // 2)
        return (download_ptr(lib.nova_rope_cos(self.h), np.float32, n).reshape(-1, self.HD // 2),
                download_ptr(lib.nova_rope_sin(self.h), np.float32, n).reshape(-1, self.HD // 2))

    def device_table(self, slice_id):
        return download_ptr(lib.nova_kv_table_slot(self.h, slice_id), np.int32, self.nblocks)

    def read_page(self, which: str, layer: int, phys: int) -> np.ndarray:
        base = self.k_base if which == "k" else self.v_base
        off = (int(layer) * self.nb + int(phys)) * self.page_bytes
        n = self.page_bytes // np.dtype(self.kv_np).itemsize
        return download_ptr(base + off, self.kv_np, n).reshape(self.desc.kv_block, self.NKV, self.HD)

    def read_pools(self):
        n = self.L * self.nb * self.page_bytes // np.dtype(self.kv_np).itemsize
        shp = (self.L, self.nb, self.desc.kv_block, self.NKV, self.HD)
        return (download_ptr(self.k_base, self.kv_np, n).reshape(shp),
                download_ptr(self.v_base, self.kv_np, n).reshape(shp))

    def batch(self, sessions) -> "Batch":
        return Batch(self, sessions)


class Batch:
    """A set of sessions decoded together (nova_batch)."""

    def __init__(self, eng: Engine, sessions):
        self.eng = eng
        self.sessions = [int(s) for s in sessions]
        a = np.asarray(self.sessions, dtype=np.int32)
        h = vp()
        check(lib.nova_batch_create(eng.h, a.ctypes.data_as(c_i32p), a.size, C.byref(h)), "nova_batch_create")
        self.h = h
        self.n = len(self.sessions)

    def close(self):
        if getattr(self, "h", None):
            lib.nova_batch_destroy(self.h)
            self.h = None

    def __del__(self):
        if lib is not None and getattr(self.eng, "h", None):
            self.close()

    def set_kernel(self, which): return check(lib.nova_batch_set_kernel(self.h, which), "set_kernel")
    def set_fused_append(self, on): return check(lib.nova_batch_set_fused_append(self.h, int(on)), "set_fused_append")
    def set_pdl(self, on): return check(lib.nova_batch_set_pdl(self.h, int(on)), "set_pdl")
    def set_prefill_kernel(self, which): return check(lib.nova_batch_set_prefill_kernel(self.h, int(which)), "set_prefill_kernel")
    def set_window(self, n): return check(lib.nova_batch_set_window(self.h, int(n)), "set_window")
    def set_split_ctas(self, n): return check(lib.nova_batch_set_split_ctas(self.h, int(n)), "set_split_ctas")
    def set_row_setup_pages(self, n): return check(lib.nova_batch_set_row_setup_pages(self.h, int(n)), "set_row_setup")
    def append_attn(self, layer, q, k, v, out, stream=None):
        return check(lib.nova_batch_append_attn(self.h, layer, q, k, v, out, stream), "append_attn")
    def sync_positions(self, stream=None): return check(lib.nova_batch_sync_positions(self.h, stream))
    def cow(self, stream=None): return check(lib.nova_batch_cow(self.h, stream), "batch_cow")
    def append(self, layer, q, k, v, stream=None):
        return check(lib.nova_batch_append(self.h, layer, q, k, v, stream), "batch_append")
    def set_cascade(self, on): return check(lib.nova_batch_set_cascade(self.h, on), "set_cascade")
    def shared_prefix_pages(self): return lib.nova_batch_shared_prefix_pages(self.h)

    def append_layers(self, layer0, n_layers, q, k, v, stream=None):
        return check(lib.nova_batch_append_layers(self.h, layer0, n_layers, q, k, v, stream), "append_layers")

    def attn(self, layer, q, out, stream=None):
        return check(lib.nova_batch_attn(self.h, layer, q, out, stream), "batch_attn")
    def advance(self, stream=None): return check(lib.nova_batch_advance(self.h, stream), "batch_advance")
    def advance_by(self, n, stream=None): return check(lib.nova_batch_advance_by(self.h, n, stream), "advance_by")
    def prefill_max_tokens(self): return lib.nova_batch_prefill_max_tokens(self.h)
    def prefill(self, layer, n_tokens, q, k, v, out, stream=None):
        return check(lib.nova_batch_prefill(self.h, layer, n_tokens, q, k, v, out, stream), "batch_prefill")
    def step_all_layers(self, q, k, v, out, stream=None):
        return check(lib.nova_batch_step_all_layers(self.h, q, k, v, out, stream), "step_all_layers")
    def decode_step_host(self, q, k, v, out, per_layer=1, stream=None, no_sync=False):
        return check(lib.nova_batch_decode_step_host(self.h, q, k, v, out, (1 if per_layer else 0) | (2 if no_sync else 0), stream),
                     "decode_step_host")
    def host_wait(self, stream=None): return check(lib.nova_batch_host_wait(self.h, stream), "host_wait")
    def run_steps(self, n_steps, q, k, v, out, q_stride, kv_stride, mode, stream=None, time_attn=False):
        """Returns the summed attention-kernel time in ms when time_attn, else None."""
        ms = C.c_float(0.0)
        check(lib.nova_batch_run_steps(self.h, n_steps, q, k, v, out, q_stride, kv_stride, mode,
                                       C.byref(ms) if time_attn else None, stream), "run_steps")
        return float(ms.value) if time_attn else None

    def device_status(self): return lib.nova_batch_device_status(self.h)
    def attn_partial_layers(self, layer0, n_layers, q, page0, page1, part, stream=None):
        return check(lib.nova_batch_attn_partial_layers(self.h, layer0, n_layers, q, page0, page1, part, stream),
                     "attn_partial_layers")

    def attn_partial(self, layer, q, page0, page1, part, stream=None):
        return check(lib.nova_batch_attn_partial(self.h, layer, q, page0, page1, part, stream), "attn_partial")
