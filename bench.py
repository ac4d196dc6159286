"""Benchmark of the paged-KV decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl reference]

One decode step = for every session of the workload and every layer: copy-on-write guard,
fused RoPE+append of the step's K/V at n_past, paged decode attention over n_past+1 keys;
then n_past += 1.  The metric counts session-steps (one session advanced by one token through
all layers) per second, so that it aggregates over sessions and GPUs.

Timed on the device with CUDA events on the launching stream after >= 3 warm-up steps; at N > 1
(one process per GPU, sessions sharded by GPU, no collective on the data path) the time is the
maximum over ranks.  One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import __graft_entry__ as graft  # noqa: E402

# BASELINE.json configs.  scaling: weak = every GPU gets `sessions` sessions of its own;
# strong = the `sessions` sessions (or the one long session's pages) are divided over the GPUs.
WORKLOADS = {
    "c1": dict(model="qwen25_1p5b", sessions=1, ctx=(1024, 1024), cfg=0, scaling="weak", steps=64,
               text="Qwen2.5-1.5B-shaped KV, 1 session x 1024 cached tokens, permuted pages"),
    "c2": dict(model="qwen25_7b", sessions=8, ctx=(2048, 8192), cfg=1, scaling="weak", steps=256,
               text="Qwen2.5-7B-shaped KV, 8 sessions, contexts uniform in [2048, 8192], permuted pages"),
    "c3": dict(model="qwen25_7b", sessions=32, ctx=(4088 + 512, 4088 + 512), cfg=2, scaling="weak", prefix=4088, steps=64,
               text="Qwen2.5-7B-shaped KV, 32 sessions sharing one 4088-token prefix (255 full pages + a partly "
                    "filled tail page, un-shared by copy-on-write on the first private append) + 512 private tokens"),
    "c4": dict(model="qwen25_14b", sessions=64, ctx=(8192, 8192), cfg=3, scaling="strong", steps=128,
               text="Qwen2.5-14B-shaped KV, 64 sessions x 8192 cached tokens, permuted pages, sessions sharded over GPUs"),
    "c5": dict(model="qwen25_7b", sessions=1, ctx=(131072, 131072), cfg=4, scaling="strong", steps=64,
               text="Qwen2.5-7B-shaped KV, 1 session x 131072 cached tokens, pages split over GPUs, partials merged "
                    "(log-sum-exp) after an NCCL all-gather"),
}
# dram__bytes_read + dram__bytes_write per attention launch from the ncu captures summarised in
# profiles/attn_mma_kernel_c2.md (split + merge kernels; config 2 only)
NCU_TRAFFIC = {("c2", "layer"): 91.36e6 + 3.06e6 + 2.33e6, ("c2", "graph"): 91.36e6 + 3.06e6 + 2.33e6,
               ("c2", "fused"): 2.5634e9 + 7.6e6}
BASE_SEED = 0x5EED0000
METRIC, UNIT = "decode_steps_per_s", "session-steps/s"


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks and throttle reasons every 20 ms while the timed regions run."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={index}", f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


def dist_env():
    return int(os.environ.get("RANK", 0)), int(os.environ.get("LOCAL_RANK", 0)), int(os.environ.get("WORLD_SIZE", 1))


# --------------------------------------------------------------------------------------------
def run_ours(args):
    rank, local_rank, world = dist_env()
    nv = graft.load_package()          # ImportError if libnova_b200.so is missing: no fallback
    import conflux_nova_b200.workloads as wl

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    nv.check(nv.lib.dev_select(local_rank))

    w = WORKLOADS[args.workload]
    if args.workload == "c5" and world > 1:
        return run_long_context(args, nv, wl, dist, rank, local_rank, world)
    seed = BASE_SEED + w["cfg"] + 1000 * rank          # every GPU holds its own sessions
    n_sess = w["sessions"] if w["scaling"] == "weak" else max(1, w["sessions"] // world)
    lens = wl.context_lengths(seed, n_sess, *w["ctx"])
    K, W, KE = args.steps, args.warmup, args.e2e_steps
    PF_REPS = 3
    total_steps = 5 * (W + K) + (W + KE) + 8 + (PF_REPS + 1) * 512
    work = wl.Workload(w["model"], lens, seed=seed, steps=total_steps, device=local_rank,
                       shared_prefix=w.get("prefix", 0), kv_dtype=nv.KV_F32 if args.kv == "f32" else nv.KV_F16)
    eng, batch = work.eng, work.batch
    kernel = args.kernel
    if kernel < 0:
        kernel = 1 if nv.lib.nova_batch_set_kernel(batch.h, 1) == nv.OK else 0
    batch.set_kernel(kernel)
    fused = bool(kernel == 1 and not args.no_fused_append)
    if fused:
        batch.set_fused_append(1)
        batch.set_pdl(0 if args.no_pdl else 1)
    if args.row_setup >= 0:
        batch.set_row_setup_pages(args.row_setup)
    cascade = bool(kernel == 1 and w.get("prefix", 0) and not args.no_cascade)
    if cascade:
        batch.set_cascade(1)          # shared prefix pages attended once for all sessions (per-layer launches)
    stream = nv.Stream()
    nq, nk = work.step_input_sizes()
    S, L = len(work.sessions), eng.L

    # step inputs resident in HBM before any timed region: a ring of 4 input sets
    ring = 4
    dq, dk, dv = nv.DevBuf(ring * nq * 4), nv.DevBuf(ring * nk * 4), nv.DevBuf(ring * nk * 4)
    dout = nv.DevBuf(ring * nq * 4)
    for i in range(ring):
        a, b, c = work.device_step_inputs(i)
        for dst, src, n in ((dq, a, nq), (dk, b, nk), (dv, c, nk)):
            host = src.download(np.float32)
            dst.upload(host, i * n * 4)
            src.free()

    def barrier():
        nv.check(nv.lib.dev_sync())
        if dist is not None:
            dist.barrier()
        nv.check(nv.lib.dev_sync())

    def timed(mode, steps, warm, time_attn=False):
        """Run `warm` + `steps` decode steps in `ring`-sized groups; returns (ms, attn_ms, kv_bytes)."""
        def go(n, measure):
            attn = 0.0
            done = 0
            while done < n:
                m = min(ring, n - done)
                r = batch.run_steps(m, dq.ptr, dk.ptr, dv.ptr, dout.ptr, nq, nk, mode, stream.h,
                                    time_attn=measure and time_attn)
                attn += r or 0.0
                done += m
            return attn
        go(warm, False)
        barrier()
        n0 = [eng.n_past(s) for s in work.sessions]
        kv_bytes = sum(work.unique_kv_bytes_per_step([n + i for n in n0]) for i in range(steps))
        e0, e1 = nv.Event(), nv.Event()
        e0.record(stream)
        attn_ms = go(steps, True)
        e1.record(stream)
        e1.sync()
        ms = e0.elapsed_ms(e1)
        barrier()
        return ms, attn_ms, kv_bytes

    if args.quick_prefill:
        pf = prefill_sample(nv, work, stream, 1)
        if rank == 0:
            print(json.dumps({"quick_prefill": True, "kernel": kernel, **(pf or {})}))
        return

    launches0 = nv.lib.nova_launch_count()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    mode = {"layer": 1, "graph": 2, "fused": 0}[args.launch]
    ms_main, _, kv_main = timed(mode, K, W)
    launches = int(nv.lib.nova_launch_count() - launches0) * K // (K + W)
    if args.quick:
        if rank == 0:
            print(json.dumps({"quick": True, "launch": args.launch, "fused_append": fused, "pdl": bool(fused and not args.no_pdl), "cascade_pages": batch.shared_prefix_pages() if cascade else 0, "kv": args.kv, "kernel": kernel, "ms_per_step": ms_main / K,
                              "kv_gbs": kv_main / ms_main / 1e6, "gpu_launches": launches}))
        return
    # end to end through the host-buffer call: pinned host q/k/v in, out back, every step
    hq, hk, hv = nv.lib.dev_host_alloc(nq * 4), nv.lib.dev_host_alloc(nk * 4), nv.lib.dev_host_alloc(nk * 4)
    ho = nv.lib.dev_host_alloc(nq * 4)
    nv.check(nv.lib.dev_download(hq, dq.ptr, nq * 4))
    nv.check(nv.lib.dev_download(hk, dk.ptr, nk * 4))
    nv.check(nv.lib.dev_download(hv, dv.ptr, nk * 4))
    for _ in range(W):
        batch.decode_step_host(hq, hk, hv, ho, 1 if mode else 0, stream.h)
    barrier()
    e0, e1 = nv.Event(), nv.Event()
    e0.record(stream)
    t0 = time.perf_counter()
    for _ in range(KE):
        batch.decode_step_host(hq, hk, hv, ho, 1 if mode else 0, stream.h)
    e1.record(stream)
    e1.sync()
    ms_e2e = max(e0.elapsed_ms(e1), (time.perf_counter() - t0) * 1e3)
    barrier()
    # the same K steps again with an event pair around every attention launch: the dominant kernel's own time
    ms_evt, attn_ms, kv_evt = timed(1 if mode == 2 else mode, K, W, time_attn=True)
    # all layers in one launch (the isolated path; legal because layer inputs are independent here)
    other = {}
    for name, m in (("fused", 0), ("layer", 1), ("graph", 2)):
        if m != mode:
            ms_o, _, kv_o = timed(m, K, W)
            other[name] = dict(ms_per_step=ms_o / K, kv_gbs=kv_o / ms_o / 1e6)
    ms_f, attn_f, kv_f = timed(0, K, W, time_attn=True)

    barrier()
    clocks = sampler.stop() if sampler else None
    status = batch.device_status()
    if status != 0:
        raise RuntimeError(f"device status {status} after the timed regions")

    # max over ranks
    vals = np.array([ms_main, ms_e2e, ms_evt, attn_ms, ms_f, attn_f], dtype=np.float64)
    sums = np.array([kv_main, kv_evt, kv_f], dtype=np.float64)
    if dist is not None:
        import torch
        t = torch.tensor(vals, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        vals = t.cpu().numpy()
        u = torch.tensor(sums, device="cuda")
        dist.all_reduce(u, op=dist.ReduceOp.SUM)
        sums = u.cpu().numpy()
    ms_main, ms_e2e, ms_evt, attn_ms, ms_f, attn_f = [float(x) for x in vals]
    kv_main_all, kv_evt_all, kv_f_all = [float(x) for x in sums]

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline_sample(nv, work, lens, seed)

    prefill = None
    if world == 1 and not args.quick and args.workload in ("c2", "c4"):
        prefill = prefill_sample(nv, work, stream, PF_REPS)

    ref_gpu = None
    if rank == 0 and world == 1 and not args.no_ref_gpu and args.workload in ("c1", "c2"):
        ref_gpu = reference_gpu_sample(nv, work)

    if rank == 0:
        peak, peak_kind = peaks()
        n_attn = K * (1 if mode == 0 else L)
        per_launch_bytes = kv_main / n_attn
        # the attention launch (split + its merge) as it runs in the timed region: launches are back to
        # back there, so its average duration is the region's time over the number of launches
        launch_us = ms_main / n_attn * 1e3
        achieved = per_launch_bytes / launch_us / 1e3
        isolated_us = attn_ms / n_attn * 1e3 if attn_ms > 0 else None     # event pair around each launch
        line = {
            "metric": METRIC, "value": world * S * K / (ms_main / 1e3), "unit": UNIT,
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_main / K,
            "higher_is_better": True, "scaling": w["scaling"], "vs_baseline": None,
            "dtype": args.kv, "data": "synthetic",
            "config": {"workload": f"{args.workload}: {w['text']}", "sessions_per_gpu": S,
                       "context_tokens": lens, "layers": L, "kv_dtype": "fp16" if args.kv == "f16" else "fp32", "page_tokens": 16,
                       "launch": args.launch, "attention_kernel": "mma" if kernel == 1 else "simt", "fused_append": fused, "pdl": bool(fused and not args.no_pdl),
                       "cascade_shared_pages": batch.shared_prefix_pages() if cascade else 0,
                       "l2": "inputs larger than L2 (KV read per step >> 126 MB)"},
            "batch_steps_per_s": K / (ms_main / 1e3),
            "kv_gbs": kv_main_all / ms_main / 1e6,
            "kv_bytes_per_step": kv_main / K,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": NCU_TRAFFIC.get((args.workload, args.launch)),
                         "peak_kind": peak_kind,
                         "kernel": "attention (%s)" % ("all layers per launch" if mode == 0 else "one layer per launch"),
                         "launch_us": launch_us, "algorithmic_bytes_per_launch": per_launch_bytes,
                         "isolated_launch_us": isolated_us,
                         "all_layers_one_launch": {"achieved": kv_f / K / (attn_f / K) / 1e6 if attn_f > 0 else 0.0,
                                                   "frac": (kv_f / K / (attn_f / K) / 1e6) / peak if attn_f > 0 else 0.0,
                                                   "launch_us": attn_f / K * 1e3}},
            "other_launch_modes": other,
            "e2e": {"value": world * S * KE / (ms_e2e / 1e3), "unit": UNIT, "h2d_bytes_per_step": (nq + 2 * nk) * 4,
                    "d2h_bytes_per_step": nq * 4, "ms_per_step": ms_e2e / KE, "steps": KE},
            "gpu_launches": launches,
            "clocks": clocks,
            "cpu_baseline": cpu,
            "reference_kernels_on_this_gpu": ref_gpu,
            "prefill": prefill,
        }
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def run_long_context(args, nv, wl, dist, rank, local_rank, world):
    """Config 5 on several GPUs: every rank attends over its own range of the session's pages
    (nova_batch_attn_partial), the (m, l, acc) partials are all-gathered over NVLink with NCCL and merged
    in rank order (nova_lse_combine).  The all-gather is the only collective of this repository."""
    import torch
    import conflux_nova_b200.longctx as lc
    w = WORKLOADS["c5"]
    seed = BASE_SEED + w["cfg"]                       # the SAME session on every rank
    n_ctx = w["ctx"][0]
    K, W = args.steps, args.warmup
    # Every rank keeps the whole session's pool (7.5 GB) but fills and reads only its own page range.
    work = wl.Workload(w["model"], [n_ctx], seed=seed, steps=2 * (W + K) + 16, device=local_rank, fill=False)
    eng, batch = work.eng, work.batch
    n_pages = (n_ctx + 15) // 16
    lo, hi = lc.page_range(rank, world, n_pages)
    first_tok, last_tok = lo * 16, min(hi * 16, n_ctx)
    if last_tok > first_tok:
        work.fill_context(work.sessions[0], first_tok, last_tok - first_tok, key_session=0)
    eng.set_n_past(work.sessions[0], n_ctx)
    batch.sync_positions()
    batch.set_kernel(1 if args.kernel != 0 else 0)
    if args.kernel != 0 and args.collective == "p2p":
        batch.set_fused_append(1)
        batch.set_pdl(0 if args.no_pdl else 1)
    L, NH, NKV = eng.L, eng.NH, eng.NKV
    tstream = torch.cuda.current_stream()
    st = tstream.cuda_stream
    dq, dk, dv = work.device_step_inputs(0)
    part = torch.empty((L, NH, lc.PART_W), dtype=torch.float32, device="cuda")
    out = torch.empty((L, NH, 128), dtype=torch.float32, device="cuda")
    qs, ks = NH * 128 * 4, NKV * 128 * 4
    es_tok = 2 * NKV * 128 * 2

    gath = torch.empty((L, world, NH, lc.PART_W), dtype=torch.float32, device="cuda")
    per_layer = args.collective == "layer"

    xch = status_word = None
    epoch = [0]
    if args.collective in ("p2p", "p2p-step"):
        # no all-gather: every rank's partial rows stay in its own exchange buffer and each rank's merge
        # kernel reads all of them over NVLink (nova_lse_merge_peers)
        xch = lc.PeerExchange(nv, NH if args.collective == "p2p" else L * NH, rank, world, dist, n_slots=2)
        status_word = nv.DevBuf(4).zero()
        dist.barrier()

    def step(st=st):
        if xch is not None and args.collective == "p2p":
            # the whole step natively: per layer fused append + attention over this rank's pages, merge by peer reads
            nv.check(nv.lib.nova_batch_step_partial_peers(batch.h, dq.ptr, dk.ptr, dv.ptr, lo, hi, xch.base, world, rank,
                                                          xch.slot_bytes, 2, epoch[0] + 1, 1000, out.data_ptr(),
                                                          status_word.ptr, st), "step_partial_peers")
            epoch[0] += L
            return
        elif xch is not None:
            epoch[0] += 1
            batch.append_layers(0, L, dq.ptr, dk.ptr, dv.ptr, st)
            batch.attn_partial_layers(0, L, dq.ptr, lo, hi, xch.rows_ptr(epoch[0] % 2), st)
            xch.merge(epoch[0], out.data_ptr(), st, status_word.ptr)
        elif per_layer:
            for l in range(L):
                batch.append(l, dq.ptr + l * qs, dk.ptr + l * ks, dv.ptr + l * ks, st)
                batch.attn_partial(l, dq.ptr + l * qs, lo, hi, part[l].data_ptr(), st)
                g = lc.gather_partials(part[l], world, dist, out=gath[l])
                nv.check(nv.lib.nova_lse_combine(g.data_ptr(), world, NH, 128, out[l].data_ptr(), st))
        else:
            batch.append_layers(0, L, dq.ptr, dk.ptr, dv.ptr, st)
            batch.attn_partial_layers(0, L, dq.ptr, lo, hi, part.data_ptr(), st)
            g = lc.gather_partials(part.reshape(L * NH, lc.PART_W), world, dist, out=gath.reshape(world, L * NH, lc.PART_W))
            nv.check(nv.lib.nova_lse_combine(g.data_ptr(), world, L * NH, 128, out.data_ptr(), st))
        batch.advance(st)

    for _ in range(W):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    n0 = eng.n_past(work.sessions[0])
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = nv.lib.nova_launch_count()
    e0.record(tstream)
    for _ in range(K):
        step()
    e1.record(tstream)
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    launches = int(nv.lib.nova_launch_count() - launches0)
    dist.barrier()
    clocks = sampler.stop() if sampler else None
    status = batch.device_status()
    if status_word is not None and int(status_word.download(np.int32)[0]) != 0:
        status = int(status_word.download(np.int32)[0])       # a peer's flag never arrived
    t = torch.tensor([ms, float(status != 0)], device="cuda", dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, bad = float(t[0]), float(t[1])
    if bad:
        raise RuntimeError("device status set during the long-context run")
    # check once against a single-GPU style full attention of the last layer on rank 0's data: the merged
    # output must be finite and identical on every rank
    chk = out[-1].clone()
    dist.broadcast(chk, src=0)
    same = bool(torch.equal(chk, out[-1])) and bool(torch.isfinite(out).all())
    flag = torch.tensor([0.0 if same else 1.0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    if float(flag[0]) != 0.0:
        raise RuntimeError("merged outputs differ between ranks")
    if rank == 0:
        peak, peak_kind = peaks()
        kv_bytes = sum((n0 + i + 1) * es_tok * L for i in range(K))          # whole session, all ranks together
        line = {
            "metric": METRIC, "value": K / (ms / 1e3), "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
            "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"c5: {w['text']}", "sessions_per_gpu": 1, "context_tokens": [n_ctx], "layers": L,
                       "kv_dtype": "fp16", "page_tokens": 16, "collective": {"layer": "all-gather per layer", "step": "all-gather per step",
                                      "p2p": "peer reads in the merge kernel, per layer",
                                      "p2p-step": "peer reads in the merge kernel, per step"}[args.collective],
                       "pages_per_gpu": -(-n_pages // world), "l2": "inputs larger than L2"},
            "kv_gbs": kv_bytes / ms / 1e6, "kv_bytes_per_step": kv_bytes / K,
            "roofline": {"bound": "hbm", "achieved": kv_bytes / ms / 1e6 / world, "peak": peak, "unit": "GB/s",
                         "frac": kv_bytes / ms / 1e6 / world / peak, "traffic": None, "peak_kind": peak_kind,
                         "kernel": "attention over this GPU's page range + all-gather + merge (per GPU)"},
            "e2e": None, "gpu_launches": launches, "clocks": clocks, "cpu_baseline": None,
        }
        print(json.dumps(line))
    if xch is not None:
        torch.cuda.synchronize()
        dist.barrier()                 # nobody closes a buffer a peer may still be reading
        xch.close()
    dist.destroy_process_group()


def prefill_sample(nv, work, stream, reps):
    """Paged prefill (the step before decode): every session takes a chunk of new tokens through
    all layers — multi-token RoPE+append, then causal attention of the chunk's queries over the paged keys."""
    eng, batch = work.eng, work.batch
    L, S, NH, NKV = eng.L, len(work.sessions), eng.NH, eng.NKV
    n_tok = min(batch.prefill_max_tokens(), 512)
    if n_tok < 1:
        return None
    nq, nk = S * n_tok * NH * 128, S * n_tok * NKV * 128
    dq, dk, dv, do = nv.DevBuf(nq * 4), nv.DevBuf(nk * 4), nv.DevBuf(nk * 4), nv.DevBuf(nq * 4)
    for buf, n, t in ((dq, nq, 3), (dk, nk, 1), (dv, nk, 2)):
        nv.check(nv.lib.nova_synth_normal(buf.ptr, n, nv.synth_key(work.seed, t, 777, 0), 0, None))
    nv.check(nv.lib.dev_sync())

    def chunk():
        for l in range(L):
            batch.prefill(l, n_tok, dq.ptr, dk.ptr, dv.ptr, do.ptr, stream.h)
        batch.advance_by(n_tok, stream.h)
    chunk()
    stream.sync()
    n0 = [eng.n_past(s) for s in work.sessions]
    e0, e1 = nv.Event(), nv.Event()
    e0.record(stream)
    for _ in range(reps):
        chunk()
    e1.record(stream)
    e1.sync()
    ms = e0.elapsed_ms(e1)
    keys = sum(sum(n + r * n_tok + t + 1 for t in range(n_tok)) for n in n0 for r in range(reps))     # (query, key) pairs per head
    flops = 4.0 * 128 * NH * keys * L
    for b in (dq, dk, dv, do):
        b.free()
    return {"tokens_per_s": S * n_tok * reps / (ms / 1e3), "chunk_tokens_per_session": n_tok, "ms_per_chunk": ms / reps,
            "attention_tflops": flops / (ms / 1e3) / 1e12,
            "note": "tensor-core kernel: query-tiled (64 rows = 9 query tokens x 7 heads per CTA at the 7B shape), K/V pages "
                    "staged once per tile; SIMT kernel: one work-split row per query token"}


def reference_gpu_sample(nv, work):
    """The reference's own CUDA kernels for this path (src/kernel/rope.cu, elem.cu, attn.cu compiled
    unmodified for sm_100a, oracle/_ref) on this GPU, on a bounded sample of the same workload: one layer,
    every session, in the reference's call order (per session: rope_batch, kv_store_paged, attn_decode_paged
    = split + combine), fp32 pools holding the same values.  Time scaled by the layer count."""
    from oracle import binding as ob
    model = {"qwen25_7b": "qwen25_7b", "qwen25_1p5b": "qwen25_1p5b"}.get(work.model)
    g = ob.ref_gpu(model) if model else None
    if g is None:
        return None
    eng = work.eng
    S, NH, NKV = len(work.sessions), eng.NH, eng.NKV
    n = eng.nb * eng.page_bytes // 2
    pk = nv.to_device(nv.download_ptr(eng.k_base, np.float16, n).astype(np.float32))     # layer 0 only
    pv = nv.to_device(nv.download_ptr(eng.v_base, np.float16, n).astype(np.float32))
    rng = np.random.default_rng(2)
    q = nv.to_device(rng.standard_normal((S, NH, 128)).astype(np.float32))
    k = nv.to_device(rng.standard_normal((S, NKV, 128)).astype(np.float32))
    v = nv.to_device(rng.standard_normal((S, NKV, 128)).astype(np.float32))
    o = nv.DevBuf(S * NH * 128 * 4)
    scr = nv.DevBuf(NH * 32 * 130 * 4)
    cs, sn = nv.lib.nova_rope_cos(eng.h), nv.lib.nova_rope_sin(eng.h)      # long enough for every position
    pos = [eng.n_past(s) for s in work.sessions]
    tabs = [nv.lib.nova_kv_table_slot(eng.h, eng.session_slice(s)) for s in work.sessions]
    st = nv.Stream()

    def layer_pass():
        for i in range(S):
            qi, ki, vi = q.ptr + i * NH * 512, k.ptr + i * NKV * 512, v.ptr + i * NKV * 512
            g.ref_gpu_rope_batch(qi, ki, 1, pos[i], cs, sn, st.h)
            g.ref_gpu_kv_store_paged(pk.ptr, pv.ptr, tabs[i], 0, eng.nb, 1, pos[i], ki, vi, st.h)
            g.ref_gpu_attn_decode_paged(qi, pk.ptr, pv.ptr, tabs[i], 0, eng.nb, pos[i] + 1, o.ptr + i * NH * 512,
                                        scr.ptr, st.h)
    for _ in range(3):
        layer_pass()
    st.sync()
    reps = 10
    e0, e1 = nv.Event(), nv.Event()
    e0.record(st)
    for _ in range(reps):
        layer_pass()
    e1.record(st)
    e1.sync()
    ms_layer = e0.elapsed_ms(e1) / reps
    ok = g.ref_gpu_last_error() == 0
    for b in (pk, pv, q, k, v, o, scr):
        b.free()
    ms_step = ms_layer * eng.L
    return {"value": S / (ms_step / 1e3), "unit": UNIT, "ms_per_step": ms_step, "ok": ok,
            "sample": f"{reps} x one layer of {eng.L}, all {S} sessions, fp32 pools, the reference's launch order "
                      f"(4 launches per session per layer); time scaled by {eng.L}"}


def cpu_baseline_sample(nv, work, lens, seed):
    """The CPU restatement of the reference's path (oracle/, the checker) timed on this box's cores on
    a bounded sample of the same workload: one decode step of `sample_layers` layers, scaled to all."""
    from oracle import binding as ob
    eng = work.eng
    L, S = eng.L, len(work.sessions)
    sample_layers = 1
    sh = ob.shape(sample_layers, eng.NH, eng.NKV, ob.KV_F16)
    n = eng.nb * eng.page_bytes // 2
    shp = (sample_layers, eng.nb, 16, eng.NKV, eng.HD)
    pk = nv.download_ptr(eng.k_base, np.float16, n).reshape(shp)
    pv = nv.download_ptr(eng.v_base, np.float16, n).reshape(shp)
    cs, sn = eng.rope_tables()
    tables = np.stack([eng.pool.table(eng.session_slice(s)) for s in work.sessions])
    pos = [eng.n_past(s) for s in work.sessions]
    rng = np.random.default_rng(0)
    q = rng.standard_normal((sample_layers, S, eng.NH, eng.HD)).astype(np.float32)
    k = rng.standard_normal((sample_layers, S, eng.NKV, eng.HD)).astype(np.float32)
    v = rng.standard_normal((sample_layers, S, eng.NKV, eng.HD)).astype(np.float32)
    t0 = time.perf_counter()
    reps = 0
    while True:
        ob.decode_step(sh, pk, pv, tables, eng.nb, pos, q.copy(), k.copy(), v, cs, sn)
        reps += 1
        if time.perf_counter() - t0 > 8.0 or reps >= 5:
            break
    dt = (time.perf_counter() - t0) / reps
    return {"value": S / (dt * L / sample_layers), "unit": UNIT, "cores": ob.num_threads(), "kind": "port",
            "sample": f"{reps} x (1 decode step of {sample_layers} of {L} layers, all {S} sessions at their full "
                      f"context), time scaled by {L}/{sample_layers}; order-faithful fp32 restatement of "
                      "fa_split_paged/fa_combine + rope/kv_store, OpenMP over layer x session"}


# --------------------------------------------------------------------------------------------
def run_reference(args):
    """The reference arm: the reference has no CPU implementation of the attention itself (its only
    implementations are CUDA and SYCL kernels), so this times the CPU restatement of its algorithm
    (oracle/, kind "port") with every host thread, on the same workload, same metric."""
    rank, _, world = dist_env()
    if rank != 0:
        return
    from oracle import binding as ob
    graft.load_package()       # workload definitions (context lengths, page permutations) use the library's hashing
    import conflux_nova_b200.workloads as from_wl
    w = WORKLOADS[args.workload]
    seed = BASE_SEED + w["cfg"]
    lens = from_wl.context_lengths(seed, w["sessions"], *w["ctx"])
    Lfull, NH, NKV = from_wl.SHAPES[w["model"]]
    S = len(lens)
    sample_layers = 1
    sh = ob.shape(sample_layers, NH, NKV, ob.KV_F16)
    nblocks = (max(lens) + args.steps + args.warmup + 16 + 15) // 16
    nb = nblocks * S
    pk, pv = ob.new_pools(sh, nb)
    cs, sn = ob.rope_table(nblocks * 16)
    tables = np.stack([s * nblocks + from_wl.page_permutation(seed, s, nblocks) for s in range(S)]).astype(np.int32)
    row = NKV * 128
    for s in range(S):          # cached context through the oracle's append, same seeded values
        n = lens[s]
        k = ob.synth_normal(n * row, ob.synth_key(seed, 1, s, 0)).reshape(n, NKV, 128)
        v = ob.synth_normal(n * row, ob.synth_key(seed, 2, s, 0)).reshape(n, NKV, 128)
        qd = np.zeros((n, NH, 128), np.float32)
        ob.rope_append_paged(sh, pk, pv, tables[s], 0, nb, n, 0, qd, k, v, cs, sn)
    pos = list(lens)
    rng = np.random.default_rng(1)

    def one_step():
        q = rng.standard_normal((sample_layers, S, NH, 128)).astype(np.float32)
        k = rng.standard_normal((sample_layers, S, NKV, 128)).astype(np.float32)
        v = rng.standard_normal((sample_layers, S, NKV, 128)).astype(np.float32)
        ob.decode_step(sh, pk, pv, tables, nb, pos, q, k, v, cs, sn)
        for i in range(S):
            pos[i] += 1

    for _ in range(args.warmup):
        one_step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        one_step()
    dt = time.perf_counter() - t0
    ms_step = dt / args.steps * 1e3 * (Lfull / sample_layers)
    value = S / (ms_step / 1e3)
    sample = (f"each step = 1 decode step of {sample_layers} of {Lfull} layers over all {S} sessions at full context; "
              f"time scaled by {Lfull}/{sample_layers}")
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": w["scaling"],
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"{args.workload}: {w['text']}", "sessions_per_gpu": S, "context_tokens": lens,
                   "layers": Lfull, "kv_dtype": "fp16", "page_tokens": 16},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": ob.num_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None,
                    help="timed decode steps (default: the configuration's own count: 64 / 256 / 64 / 128 / 64)")
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--e2e-steps", type=int, default=64)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--collective", default="p2p", choices=["layer", "step", "p2p", "p2p-step"],
                    help="c5 on several GPUs: p2p = merge kernel reads the peers over NVLink, per layer (engine order); layer / step = NCCL all-gather + merge per layer / once per step; p2p-step = peer reads once per step")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--launch", default="layer", choices=["layer", "graph", "fused"],
                    help="layer: 2 launches per layer; graph: the same, replayed from a CUDA graph; fused: all layers per launch")
    ap.add_argument("--kernel", type=int, default=-1, help="-1 best available, 0 SIMT, 1 tensor-core")
    ap.add_argument("--no-fused-append", action="store_true",
                    help="keep RoPE+append as its own launch instead of doing it inside the attention launch")
    ap.add_argument("--row-setup", type=int, default=-1, help="work-split weight of a session start, in pages")
    ap.add_argument("--no-cascade", action="store_true", help="config 3: attend the shared prefix per session, as the plain path does")
    ap.add_argument("--no-pdl", action="store_true", help="no programmatic dependent launch between layers")
    ap.add_argument("--kv", default="f16", choices=["f16", "f32"],
                    help="KV pool element type (f32 = the reference's own format; SIMT kernel)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-ref-gpu", action="store_true", help="skip timing the reference's own kernels (sm_100a build)")
    ap.add_argument("--quick-prefill", action="store_true", help="only the prefill sample (for profiler captures)")
    ap.add_argument("--quick", action="store_true",
                    help="only the main timed region (for profiler captures): no other modes, e2e or CPU baseline")
    args = ap.parse_args()
    if args.steps is None:
        args.steps = WORKLOADS[args.workload]["steps"] if args.impl == "ours" and not (args.quick or args.quick_prefill) else 32
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    _, _, world = dist_env()
    if args.gpus != world and world > 1:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}")
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
