"""One long session split over GPUs (flash-decoding across ranks).

The reference scales a long context only inside one GPU (32 splits, src/kernel/attn.cu:498-512) and
otherwise drops history (code/INPUT_TOKENIZR.h:57-67).  Here rank r of G attends over a contiguous range
of the session's logical pages and leaves un-normalised partials (m, l, acc) per head in the
reference's partial layout (attn.cu:150-158); the partials are all-gathered and merged in rank order
with fa_combine_kernel's arithmetic (attn.cu:163-191).  The merge is latency-bound (14.5 KB per rank per
layer at the 7B shape), never bandwidth-bound.

The page arithmetic and the gather are plain host code so that they run on CPU ranks (gloo) too.
"""
from __future__ import annotations

PART_W = 130          # m, l, acc[128]
OPEN_END = 1 << 40    # "to the end of the session": the last rank's range grows with the context


def page_range(rank: int, world: int, n_pages: int) -> tuple[int, int]:
    """Logical pages [lo, hi) of `rank`; ranges tile [0, n_pages) in rank order, the last one is open-ended
    so that pages appended later (and the page that receives new tokens) belong to the last rank."""
    per = -(-n_pages // world) if n_pages > 0 else 0
    lo = min(rank * per, n_pages)
    hi = min((rank + 1) * per, n_pages)
    if rank == world - 1:
        hi = OPEN_END
    return lo, hi


def owner_of_page(page: int, world: int, n_pages: int) -> int:
    per = -(-n_pages // world) if n_pages > 0 else 1
    return min(page // max(per, 1), world - 1)


def gather_partials(part, world: int, dist=None, out=None):
    """all-gather of one partial tensor [rows][130] -> [world][rows][130] (rank order).  `out`: an optional
    contiguous tensor of world * part.numel() elements that receives the result (no allocation per call)."""
    import torch
    if world == 1 or dist is None:
        return part.unsqueeze(0)
    flat = part.contiguous().reshape(-1)
    if out is None:
        out = torch.empty(world * flat.numel(), dtype=part.dtype, device=part.device)
    flat_out = out.reshape(-1)
    dist.all_gather_into_tensor(flat_out, flat)      # concatenation in rank order, on every backend
    return flat_out.reshape((world,) + tuple(part.shape))


class PeerExchange:
    """Exchange buffers of all ranks of a node for nova_lse_merge_peers / nova_batch_step_partial_peers: every rank
    owns `n_slots` slots in its own device memory that the peers WRITE their partial rows into, exports the buffer
    with dev_ipc_export and opens the others'.  `nv` is the loaded package (ctypes face); `dist` a
    torch.distributed-like module whose all_gather_object carries the 64-byte handles (None or world 1: only the
    local buffer)."""

    def __init__(self, nv, n_rows: int, rank: int, world: int, dist=None, n_slots: int = 2):
        import ctypes as C
        self.nv, self.rank, self.world, self.n_rows, self.n_slots = nv, rank, world, n_rows, n_slots
        self.slot_bytes = int(nv.lib.nova_peer_slot_bytes(n_rows))
        self.buf = nv.DevBuf(self.slot_bytes * n_slots).zero()
        self.part = nv.DevBuf(n_rows * PART_W * 4).zero()       # this rank's rows before they are sent
        self.opened = []
        ptrs = [None] * world
        ptrs[rank] = self.buf.ptr
        if world > 1:
            handle = (C.c_ubyte * 64)()
            nv.check(nv.lib.dev_ipc_export(self.buf.ptr, handle), "dev_ipc_export")
            nv.check(nv.lib.dev_sync())
            handles = [None] * world
            dist.all_gather_object(handles, bytes(handle))
            for r in range(world):
                if r == rank:
                    continue
                h = (C.c_ubyte * 64).from_buffer_copy(handles[r])
                p = C.c_void_p()
                nv.check(nv.lib.dev_ipc_open(h, C.byref(p)), "dev_ipc_open")
                self.opened.append(p)
                ptrs[r] = p.value
        self.base = (C.c_void_p * world)(*ptrs)

    def rows_ptr(self, slot: int = 0) -> int:
        """Where this rank's partial rows go before the exchange (the `part` argument of nova_batch_attn_partial)."""
        return self.part.ptr

    def merge(self, epoch: int, out_ptr: int, stream=None, status_ptr=None, timeout_ms: int = 1000, n_rows=None):
        slot = epoch % self.n_slots
        self.nv.check(self.nv.lib.nova_lse_merge_peers(self.part.ptr, self.base, self.world, self.rank, self.slot_bytes, slot,
                                                        self.n_rows if n_rows is None else n_rows, epoch, timeout_ms,
                                                        out_ptr, status_ptr, stream), "nova_lse_merge_peers")

    def close(self):
        for p in self.opened:
            self.nv.lib.dev_ipc_close(p)
        self.opened = []
        self.buf.free()
        self.part.free()
