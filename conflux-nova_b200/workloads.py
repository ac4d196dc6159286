"""Synthetic workloads of the paged-KV decode path: model-shaped engines, sessions with fragmented
block tables, and cached context pushed through the append path itself.

Inputs stand in for real activations (no dataset is involved): every K, V and Q element is
value(key(seed, tensor, session, layer), position * row_width + element) of the library's
integer-only generator (nova_synth_normal), so host checkers can regenerate them bit for bit.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import (KV_F16, DevBuf, Engine, KvShape, check, lib, synth_key)

# (layers, q heads, kv heads); head_dim 128, page 16 tokens, RoPE theta 1e6 (NeoX pairs)
SHAPES = {"qwen25_1p5b": (28, 12, 2), "qwen25_7b": (28, 28, 4), "qwen25_14b": (48, 40, 8)}
T_K, T_V, T_Q, T_PERM, T_LEN = 1, 2, 3, 9, 10


def mix64(x: int) -> int:
    m = (1 << 64) - 1
    x = (x + 0x9E3779B97F4A7C15) & m
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & m
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & m
    return x ^ (x >> 31)


def page_permutation(seed: int, session: int, n: int) -> np.ndarray:
    """Fisher-Yates shuffle driven by the same 64-bit mixer: fragmented block tables."""
    perm = np.arange(n, dtype=np.int32)
    state = synth_key(seed, T_PERM, session, 0)
    for i in range(n - 1, 0, -1):
        state = mix64(state)
        j = state % (i + 1)
        perm[i], perm[j] = perm[j], perm[i]
    return perm


def context_lengths(seed: int, n_sessions: int, lo: int, hi: int) -> list[int]:
    """Context lengths uniform in [lo, hi] from the hash (config: 8 sessions in [2048, 8192])."""
    return [lo + mix64(synth_key(seed, T_LEN, s, 0)) % (hi - lo + 1) for s in range(n_sessions)]


class Workload:
    """An engine, its sessions and one batch over them, with `ctx_lens[s]` cached tokens each."""

    def __init__(self, model: str, ctx_lens, *, seed: int, steps: int, kv_dtype=KV_F16, device=0, permute=True,
                 spare_slices=0, fill=True, n_layers=None, zero_pages=0, shared_prefix=0, key_base=0, kv_block=16):
        """ctx_lens[s] cached tokens per session.  shared_prefix > 0: one extra donor session holds that
        many tokens; every session attaches them (KvPool::attach_prefix: shared pages, the partly filled
        tail page included), un-shares the tail page on its first private write and appends
        ctx_lens[s] - shared_prefix private tokens (config 3)."""
        L, NH, NKV = SHAPES[model]
        if n_layers:
            L = n_layers
        self.model, self.seed = model, seed
        self.ctx_lens = [int(c) for c in ctx_lens]
        self.shared_prefix = int(shared_prefix)
        S = len(self.ctx_lens)
        self.kv_block = int(kv_block)
        ctx = ((max(self.ctx_lens) + steps + kv_block - 1) // kv_block) * kv_block
        extra = (2 if shared_prefix else 0) + spare_slices        # donor + one slice of spare pages for COW
        self.eng = Engine(L, NH, NKV, ctx=ctx, n_slices=S + extra, kv_dtype=kv_dtype, kv_block=kv_block,
                          rope_positions=ctx, device=device, zero_pages=zero_pages, max_sessions=S + (1 if shared_prefix else 0))
        self.donor = None
        if shared_prefix:
            self.donor = self.eng.session_create()
            if permute:
                self.eng.permute_pages(self.donor, page_permutation(seed, 10 ** 6, self.eng.nblocks))
            self.fill_context(self.donor, 0, shared_prefix, key_session=10 ** 6)
        self.sessions = [self.eng.session_create() for _ in range(S)]
        self.key_ids = [key_base + i for i in range(S)]
        if permute:
            for s, kid in zip(self.sessions, self.key_ids):
                self.eng.permute_pages(s, page_permutation(seed, kid, self.eng.nblocks))
        self.cow_at_build = 0
        if fill:
            for i, s in enumerate(self.sessions):
                if shared_prefix:
                    self.eng.attach_prefix(s, self.donor, shared_prefix)
                    n_priv = self.ctx_lens[i] - shared_prefix
                    if n_priv > 0:
                        self.cow_at_build += self.eng.cow(s, shared_prefix, n_priv)
                        self.fill_context(s, shared_prefix, n_priv, key_session=self.key_ids[i])
                else:
                    self.fill_context(s, 0, self.ctx_lens[i], key_session=self.key_ids[i])
        self.batch = self.eng.batch(self.sessions)

    # -- cached context -------------------------------------------------------------------
    def fill_context(self, session: int, pos0: int, n: int, chunk: int = 4096, key_session=None):
        """Append synthetic K/V rows for positions [pos0, pos0+n) of one session in all layers
        (k rotated by RoPE on the way, as a prefill would)."""
        e = self.eng
        if n <= 0:
            return
        ks = session if key_session is None else key_session
        row = e.NKV * e.HD
        sh = e.shape()
        kbuf, vbuf = DevBuf(min(n, chunk) * row * 4), DevBuf(min(n, chunk) * row * 4)
        table = lib.nova_kv_table_slot(e.h, e.session_slice(session))
        cs, sn = lib.nova_rope_cos(e.h), lib.nova_rope_sin(e.h)
        for layer in range(e.L):
            kk, kv = synth_key(self.seed, T_K, ks, layer), synth_key(self.seed, T_V, ks, layer)
            for p in range(pos0, pos0 + n, chunk):
                m = min(chunk, pos0 + n - p)
                check(lib.nova_synth_normal(kbuf.ptr, m * row, kk, p * row, None))
                check(lib.nova_synth_normal(vbuf.ptr, m * row, kv, p * row, None))
                check(lib.nova_launch_rope_append_paged(C.byref(sh), e.k_base, e.v_base, table, layer, e.nb, m, p,
                                                        None, kbuf.ptr, vbuf.ptr, cs, sn, None), "context fill")
        check(lib.dev_sync())
        e.set_n_past(session, max(e.n_past(session), pos0 + n))
        kbuf.free()
        vbuf.free()

    # -- per-step inputs ------------------------------------------------------------------
    def step_input_sizes(self):
        e, S = self.eng, len(self.sessions)
        return e.L * S * e.NH * e.HD, e.L * S * e.NKV * e.HD

    def host_step_inputs(self, step: int):
        """q [L][S][NH][HD], k, v [L][S][NKV][HD] of decode step `step` (host, fp32)."""
        e, S = self.eng, len(self.sessions)
        q = np.empty((e.L, S, e.NH, e.HD), np.float32)
        k = np.empty((e.L, S, e.NKV, e.HD), np.float32)
        v = np.empty_like(k)
        dq, dk, dv = self.device_step_inputs(step)
        q[:] = dq.download(np.float32).reshape(q.shape)
        k[:] = dk.download(np.float32).reshape(k.shape)
        v[:] = dv.download(np.float32).reshape(v.shape)
        for b in (dq, dk, dv):
            b.free()
        return q, k, v

    def device_step_inputs(self, step: int):
        """The same tensors generated on the device: element index = step * row + element."""
        e, S = self.eng, len(self.sessions)
        nq, nk = self.step_input_sizes()
        dq, dk, dv = DevBuf(nq * 4), DevBuf(nk * 4), DevBuf(nk * 4)
        qrow, krow = e.NH * e.HD, e.NKV * e.HD
        for layer in range(e.L):
            for i, s in enumerate(self.key_ids):
                off = layer * S + i
                check(lib.nova_synth_normal(dq.ptr + off * qrow * 4, qrow, synth_key(self.seed, T_Q, s, layer),
                                            (10 ** 6 + step) * qrow, None))
                check(lib.nova_synth_normal(dk.ptr + off * krow * 4, krow, synth_key(self.seed, T_K, s, layer),
                                            (10 ** 9 + step) * krow, None))
                check(lib.nova_synth_normal(dv.ptr + off * krow * 4, krow, synth_key(self.seed, T_V, s, layer),
                                            (10 ** 9 + step) * krow, None))
        check(lib.dev_sync())
        return dq, dk, dv

    def kv_bytes_per_step(self, n_past=None) -> int:
        """Algorithmic KV bytes of one decode step: every cached key's K and V row read once per
        kv head in every layer (the reference profiler's definition, code/graph/dense.h:88), plus
        the appended rows."""
        e = self.eng
        es = 2 if e.desc.kv_dtype == KV_F16 else 4
        n_past = [e.n_past(s) for s in self.sessions] if n_past is None else n_past
        keys = sum(n + 1 for n in n_past)
        per_tok = 2 * e.NKV * e.HD * es * e.L
        return keys * per_tok + len(self.sessions) * per_tok

    def unique_kv_bytes_per_step(self, n_past=None) -> int:
        """The same with shared-prefix pages counted once (the least HBM traffic a step can have)."""
        e = self.eng
        es = 2 if e.desc.kv_dtype == KV_F16 else 4
        n_past = [e.n_past(s) for s in self.sessions] if n_past is None else n_past
        per_tok = 2 * e.NKV * e.HD * es * e.L
        if not self.shared_prefix:
            return self.kv_bytes_per_step(n_past)
        full_pages = (self.shared_prefix // self.kv_block) * self.kv_block      # the tail page is private after its COW
        keys = full_pages + sum(n + 1 - full_pages for n in n_past)
        return keys * per_tok + len(self.sessions) * per_tok

    def close(self):
        self.batch.close()
        self.eng.close()
