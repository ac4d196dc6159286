"""Benchmark of the paged-KV decode path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2] [--impl reference]

One decode step = for every session of the workload and every layer: copy-on-write guard,
fused RoPE+append of the step's K/V at n_past, paged decode attention over n_past+1 keys;
then n_past += 1.  The metric counts session-steps (one session advanced by one token through
all layers) per second, so that it aggregates over sessions and GPUs.

Timed on the device with CUDA events on the launching stream after >= 3 warm-up steps; at N > 1
(one process per GPU, sessions sharded by GPU, no collective on the data path) the time is the
maximum over ranks.  One JSON line is printed by rank 0.

The headline workload is configuration 2 at every N (8 sessions per GPU, weak scaling).  The same line
carries `scaling_workloads`: configuration 4 (64 sessions of the 14B shape divided over the GPUs, strong
scaling, no collective) and configuration 5 (one 131072-token session, its pages split over the GPUs, partial
results merged over NVLink), measured in the same process group after the headline.
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
                    "(log-sum-exp) over NVLink"),
}
# dram__bytes_read + dram__bytes_write per attention launch.  NOT measured by this run: the figures come from the
# ncu captures summarised under profiles/ (file named in `traffic_source`) and describe the kernels as they were
# when those captures were taken.
NCU_TRAFFIC = {("c2", "layer"): 91.36e6 + 3.06e6 + 2.33e6, ("c2", "graph"): 91.36e6 + 3.06e6 + 2.33e6,
               ("c2", "fused"): 2.5634e9 + 7.6e6}
NCU_TRAFFIC_SOURCE = "ncu capture summarised in profiles/attn_mma_kernel_c2.md, not measured by this run"
BASE_SEED = 0x5EED0000
METRIC, UNIT = "decode_steps_per_s", "session-steps/s"
COLLECTIVES = {"layer": "all-gather per layer", "step": "all-gather per step",
               "p2p": "partial rows exchanged by the per-layer launches themselves over NVLink",
               "p2p-step": "peer reads in the merge kernel, per step"}


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


class Ctx:
    """What every measurement needs: the loaded library, the rank layout and the barrier."""

    def __init__(self, nv, wl, dist, rank, local_rank, world):
        self.nv, self.wl, self.dist = nv, wl, dist
        self.rank, self.local_rank, self.world = rank, local_rank, world

    def barrier(self):
        self.nv.check(self.nv.lib.dev_sync())
        if self.dist is not None:
            self.dist.barrier()
        self.nv.check(self.nv.lib.dev_sync())

    def reduce(self, values, op="max"):
        """Max (times) or sum (byte counts) over ranks of a list of floats."""
        if self.dist is None:
            return [float(v) for v in values]
        import torch
        t = torch.tensor([float(v) for v in values], device="cuda", dtype=torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX if op == "max" else self.dist.ReduceOp.SUM)
        return [float(x) for x in t.cpu().numpy()]


def configure_batch(nv, batch, args, prefix=False):
    """Kernel choice and launch options of a batch as the flags ask for them."""
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
    if args.split_ctas > 0 and kernel == 1:
        batch.set_split_ctas(args.split_ctas)
    if kernel == 1 and args.prefill_kernel >= 0:
        nv.lib.nova_batch_set_prefill_kernel(batch.h, args.prefill_kernel)       # refused for page sizes it does not take
    cascade = bool(kernel == 1 and prefix and not args.no_cascade)
    if cascade:
        batch.set_cascade(1)          # shared prefix pages attended once for all sessions (per-layer launches)
    return dict(kernel=kernel, fused=fused, pdl=bool(fused and not args.no_pdl), cascade=cascade)


class StepInputs:
    """A ring of decode-step inputs resident in HBM before any timed region, and the output buffer."""

    def __init__(self, nv, work, ring):
        self.ring = ring
        self.nq, self.nk = work.step_input_sizes()
        self.dq, self.dk, self.dv = nv.DevBuf(ring * self.nq * 4), nv.DevBuf(ring * self.nk * 4), nv.DevBuf(ring * self.nk * 4)
        self.dout = nv.DevBuf(ring * self.nq * 4)
        for i in range(ring):
            a, b, c = work.device_step_inputs(i)
            for dst, src, n in ((self.dq, a, self.nq), (self.dk, b, self.nk), (self.dv, c, self.nk)):
                host = src.download(np.float32)
                dst.upload(host, i * n * 4)
                src.free()

    def free(self):
        for b in (self.dq, self.dk, self.dv, self.dout):
            b.free()


def timed_steps(cx, work, inp, stream, mode, steps, warm, time_attn=False):
    """`warm` + `steps` decode steps in ring-sized groups through nova_batch_run_steps; returns
    (ms, summed attention-launch ms or 0, algorithmic KV bytes of the timed steps)."""
    nv, batch, eng = cx.nv, work.batch, work.eng

    def go(n, measure):
        attn, done = 0.0, 0
        while done < n:
            m = min(inp.ring, n - done)
            r = batch.run_steps(m, inp.dq.ptr, inp.dk.ptr, inp.dv.ptr, inp.dout.ptr, inp.nq, inp.nk, mode, stream.h,
                                time_attn=measure and time_attn)
            attn += r or 0.0
            done += m
        return attn
    go(warm, False)
    cx.barrier()
    n0 = [eng.n_past(s) for s in work.sessions]
    kv_bytes = sum(work.unique_kv_bytes_per_step([n + i for n in n0]) for i in range(steps))
    e0, e1 = nv.Event(), nv.Event()
    e0.record(stream)
    attn_ms = go(steps, True)
    e1.record(stream)
    e1.sync()
    ms = e0.elapsed_ms(e1)
    cx.barrier()
    return ms, attn_ms, kv_bytes


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
    cx = Ctx(nv, wl, dist, rank, local_rank, world)

    w = WORKLOADS[args.workload]
    if args.workload == "c5" and world > 1:
        line = long_context_measure(cx, args, args.steps, args.warmup, args.collective)
        if rank == 0:
            print(json.dumps(line))
        dist.destroy_process_group()
        return
    seed = BASE_SEED + w["cfg"] + 1000 * rank          # every GPU holds its own sessions
    n_sess = w["sessions"] if w["scaling"] == "weak" else max(1, w["sessions"] // world)
    if args.sessions > 0:
        n_sess = args.sessions            # a cut-down case for profiler captures
    lens = wl.context_lengths(seed, n_sess, *w["ctx"])
    K, W, KE = args.steps, args.warmup, args.e2e_steps
    PF_REPS = 3
    total_steps = 7 * (W + K) + (W + KE) + 8 + (PF_REPS + 1) * 512
    work = wl.Workload(w["model"], lens, seed=seed, steps=total_steps, device=local_rank,
                       shared_prefix=w.get("prefix", 0), kv_dtype=nv.KV_F32 if args.kv == "f32" else nv.KV_F16,
                       kv_block=args.page_tokens)
    eng, batch = work.eng, work.batch
    opt = configure_batch(nv, batch, args, prefix=bool(w.get("prefix", 0)))
    kernel, fused, cascade = opt["kernel"], opt["fused"], opt["cascade"]
    stream = nv.Stream()
    S, L = len(work.sessions), eng.L
    inp = StepInputs(nv, work, ring=4)
    nq, nk = inp.nq, inp.nk

    if args.quick_prefill:
        pf = prefill_sample(nv, work, stream, 1)
        if rank == 0:
            print(json.dumps({"quick_prefill": True, "kernel": kernel, **(pf or {})}))
        return

    launches0 = nv.lib.nova_launch_count()
    sampler = ClockSampler(local_rank) if rank == 0 else None
    mode = {"layer": 1, "graph": 2, "fused": 0}[args.launch]
    late_main = bool(args.late_inputs and opt["pdl"] and nv.lib.nova_batch_set_pdl(batch.h, 2) == nv.OK)
    ms_main, _, kv_main = timed_steps(cx, work, inp, stream, mode, K, W)
    launches = int(nv.lib.nova_launch_count() - launches0) * K // (K + W)
    if args.quick:
        if rank == 0:
            print(json.dumps({"quick": True, "launch": args.launch, "fused_append": fused, "pdl": opt["pdl"],
                              "late_inputs": late_main,
                              "cascade_pages": batch.shared_prefix_pages() if cascade else 0, "kv": args.kv, "kernel": kernel,
                              "ms_per_step": ms_main / K, "kv_gbs": kv_main / ms_main / 1e6, "gpu_launches": launches}))
        return
    # per-layer launches whose q / new k / new v are read only after the previous layer's kernels have finished
    # (what an engine needs: layer l+1's inputs come out of the matrix products that consume layer l's output);
    # tables, positions and the first ring of page copies still start early
    ms_late = kv_late = None
    if opt["pdl"] and not late_main and nv.lib.nova_batch_set_pdl(batch.h, 2) == nv.OK:
        ms_late, _, kv_late = timed_steps(cx, work, inp, stream, 1, K, W)
        batch.set_pdl(1)
    # strict stream order: no programmatic dependent launch at all
    ms_strict = kv_strict = None
    if opt["pdl"]:
        batch.set_pdl(0)
        ms_strict, _, kv_strict = timed_steps(cx, work, inp, stream, 1, K, W)
        batch.set_pdl(2 if late_main else 1)

    # end to end through the host-buffer call: pinned host q/k/v in, out back, every step.  Steps are queued (the call
    # does not synchronise per step; two host output buffers are used in turn) and the clock stops when the last
    # step's output has arrived.
    hq, hk, hv = nv.lib.dev_host_alloc(nq * 4), nv.lib.dev_host_alloc(nk * 4), nv.lib.dev_host_alloc(nk * 4)
    ho, ho2 = nv.lib.dev_host_alloc(nq * 4), nv.lib.dev_host_alloc(nq * 4)
    nv.check(nv.lib.dev_download(hq, inp.dq.ptr, nq * 4))
    nv.check(nv.lib.dev_download(hk, inp.dk.ptr, nk * 4))
    nv.check(nv.lib.dev_download(hv, inp.dv.ptr, nk * 4))

    def e2e_steps(n, no_sync):
        for i in range(n):
            batch.decode_step_host(hq, hk, hv, ho if i % 2 == 0 else ho2, 1 if mode else 0, stream.h, no_sync=no_sync)
        batch.host_wait(stream.h)
    e2e_steps(W, True)
    cx.barrier()
    t0 = time.perf_counter()
    e2e_steps(KE, True)
    ms_e2e = (time.perf_counter() - t0) * 1e3
    cx.barrier()
    # the same with a synchronisation after every step (the caller reads each result before it issues the next step)
    e2e_steps(W, False)
    t0 = time.perf_counter()
    e2e_steps(KE, False)
    ms_e2e_sync = (time.perf_counter() - t0) * 1e3
    cx.barrier()
    # the same K steps again with an event pair around every attention launch: the dominant kernel's own time
    ms_evt, attn_ms, kv_evt = timed_steps(cx, work, inp, stream, 1 if mode == 2 else mode, K, W, time_attn=True)
    # the other launch modes
    other = {}
    for name, m in (("fused", 0), ("layer", 1), ("graph", 2)):
        if m != mode:
            ms_o, _, kv_o = timed_steps(cx, work, inp, stream, m, K, W)
            other[name] = dict(ms_per_step=ms_o / K, kv_gbs=kv_o / ms_o / 1e6)
    # all layers in one launch (the isolated path; legal because layer inputs are independent here)
    ms_f, attn_f, kv_f = timed_steps(cx, work, inp, stream, 0, K, W, time_attn=True)
    cx.barrier()
    clocks = sampler.stop() if sampler else None
    status = batch.device_status()
    if status != 0:
        raise RuntimeError(f"device status {status} after the timed regions")

    ms_main, ms_e2e, ms_evt, attn_ms, ms_f, attn_f, ms_late_r, ms_strict_r, ms_e2e_sync = cx.reduce(
        [ms_main, ms_e2e, ms_evt, attn_ms, ms_f, attn_f, ms_late or 0.0, ms_strict or 0.0, ms_e2e_sync], "max")
    kv_main_all, kv_evt_all, kv_f_all = cx.reduce([kv_main, kv_evt, kv_f], "sum")

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline_sample(nv, work, lens, seed)

    prefill = None
    if world == 1 and not args.quick and args.workload in ("c2", "c4"):
        prefill = prefill_sample(nv, work, stream, PF_REPS)

    ref_gpu = drop_in = None
    if rank == 0 and world == 1 and not args.no_ref_gpu and args.workload in ("c1", "c2") and args.page_tokens == 16:
        ref_gpu, drop_in = reference_gpu_sample(nv, work)

    line = None
    if rank == 0:
        peak, peak_kind = peaks()
        n_attn = K * (1 if mode == 0 else L)
        per_launch_bytes = kv_main / n_attn
        # the attention launch as it runs in the timed region: launches are back to back there, so its
        # average duration is the region's time over the number of launches
        launch_us = ms_main / n_attn * 1e3
        achieved = per_launch_bytes / launch_us / 1e3
        isolated_us = attn_ms / n_attn * 1e3 if attn_ms > 0 else None     # event pair around each launch

        def per_layer(ms, kv):
            if not ms or not kv:
                return None
            a = kv / (K * L) / (ms / (K * L) * 1e3) / 1e3
            return {"ms_per_step": ms / K, "achieved": a, "frac": a / peak, "launch_us": ms / (K * L) * 1e3}
        traffic = NCU_TRAFFIC.get((args.workload, args.launch))
        line = {
            "metric": METRIC, "value": world * S * K / (ms_main / 1e3), "unit": UNIT,
            "n_gpus": world, "steps": K, "warmup": W, "ms_per_step": ms_main / K,
            "higher_is_better": True, "scaling": w["scaling"], "vs_baseline": None,
            "dtype": args.kv, "data": "synthetic",
            "config": {"workload": f"{args.workload}: {w['text']}", "sessions_per_gpu": S,
                       "context_tokens": lens, "layers": L, "kv_dtype": "fp16" if args.kv == "f16" else "fp32", "page_tokens": args.page_tokens,
                       "launch": args.launch, "attention_kernel": "mma" if kernel == 1 else "simt", "fused_append": fused,
                       "pdl": opt["pdl"], "late_inputs": late_main,
                       "cascade_shared_pages": batch.shared_prefix_pages() if cascade else 0,
                       "l2": "inputs larger than L2 (KV read per step >> 126 MB)"},
            "batch_steps_per_s": K / (ms_main / 1e3),
            "kv_gbs": kv_main_all / ms_main / 1e6,
            "kv_bytes_per_step": kv_main / K,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": traffic,
                         "traffic_source": NCU_TRAFFIC_SOURCE if traffic else None,
                         "peak_kind": peak_kind,
                         "kernel": "attention (%s)" % ("all layers per launch" if mode == 0 else "one layer per launch"),
                         "launch_us": launch_us, "algorithmic_bytes_per_launch": per_launch_bytes,
                         "isolated_launch_us": isolated_us,
                         "per_layer_dependent_inputs": per_layer(ms_late_r if ms_late else None, kv_late),
                         "per_layer_strict_stream_order": per_layer(ms_strict_r if ms_strict else None, kv_strict),
                         "all_layers_one_launch": {"achieved": kv_f / K / (attn_f / K) / 1e6 if attn_f > 0 else 0.0,
                                                   "frac": (kv_f / K / (attn_f / K) / 1e6) / peak if attn_f > 0 else 0.0,
                                                   "launch_us": attn_f / K * 1e3}},
            "other_launch_modes": other,
            "e2e": {"value": world * S * KE / (ms_e2e / 1e3), "unit": UNIT, "h2d_bytes_per_step": (nq + 2 * nk) * 4,
                    "d2h_bytes_per_step": nq * 4, "ms_per_step": ms_e2e / KE, "steps": KE,
                    "timing": "host wall clock from the first call to the arrival of the last step's output; steps queued",
                    "synchronised_every_step": {"value": world * S * KE / (ms_e2e_sync / 1e3), "ms_per_step": ms_e2e_sync / KE}},
            "gpu_launches": launches,
            "clocks": clocks,
            "cpu_baseline": cpu,
            "reference_kernels_on_this_gpu": ref_gpu,
            "drop_in_launchers": drop_in,
            "prefill": prefill,
        }

    # configurations 4 and 5 in the same process group, after the headline's pools are gone
    inp.free()
    for p in (hq, hk, hv, ho, ho2):
        nv.lib.dev_host_free(p)
    work.close()
    if args.workload == "c2" and not args.no_scaling_workloads:
        sw = {}
        if world == 1 and args.kv == "f16" and line is not None:
            # the reference's own pool format (fp32) through the same batched per-layer calls: the tensor-core kernel
            # converts the rows to fp16 in shared memory (the SIMT kernel where that form does not apply)
            f32 = sharded_measure(cx, args, "c2", steps=32, warm=3, kv_dtype=nv.KV_F32)
            line["fp32_pools"] = {k: f32[k] for k in ("workload", "steps", "ms_per_step", "value", "unit", "kv_gbs", "frac_per_gpu",
                                                      "launch", "attention_kernel", "pdl")}
        sw["c4"] = sharded_measure(cx, args, "c4", steps=8, warm=3)
        if world > 1:
            c5 = long_context_measure(cx, args, 16, 3, "p2p")
            if c5:
                sw["c5"] = {"workload": c5["config"]["workload"], "scaling": "strong", "steps": 16,
                            "ms_per_step": c5["ms_per_step"], "value": c5["value"], "unit": UNIT, "kv_gbs": c5["kv_gbs"],
                            "frac_per_gpu": c5["roofline"]["frac"], "collective": c5["config"]["collective"],
                            "pages_per_gpu": c5["config"]["pages_per_gpu"]}
        else:
            sw["c5"] = sharded_measure(cx, args, "c5", steps=16, warm=3)
        if line is not None:
            line["scaling_workloads"] = sw
    if rank == 0:
        print(json.dumps(line))
    if dist is not None:
        dist.destroy_process_group()


def sharded_measure(cx, args, name, steps, warm, kv_dtype=None):
    """One configuration whose sessions are divided over the GPUs (no collective), per-layer launches in the
    engine's order: ms per step (max over ranks), whole-job KV GB/s and the per-GPU roofline fraction.
    kv_dtype: the pools' element type when it is not the fp16 of the bench configurations."""
    nv, wl = cx.nv, cx.wl
    w = WORKLOADS[name]
    seed = BASE_SEED + w["cfg"] + 1000 * cx.rank
    n_sess = w["sessions"] if w["scaling"] == "weak" else max(1, w["sessions"] // cx.world)
    lens = wl.context_lengths(seed, n_sess, *w["ctx"])
    work = wl.Workload(w["model"], lens, seed=seed, steps=2 * (warm + steps) + 8, device=cx.local_rank,
                       shared_prefix=w.get("prefix", 0), key_base=cx.rank * n_sess,
                       kv_dtype=nv.KV_F16 if kv_dtype is None else kv_dtype)
    try:
        opt = configure_batch(nv, work.batch, args, prefix=bool(w.get("prefix", 0)))
        stream = nv.Stream()
        inp = StepInputs(nv, work, ring=2)
        ms, _, kv = timed_steps(cx, work, inp, stream, 1, steps, warm)
        status = work.batch.device_status()
        inp.free()
        stream.close()
    finally:
        work.close()
    if status != 0:
        raise RuntimeError(f"device status {status} in workload {name}")
    (ms,) = cx.reduce([ms], "max")
    (kv_all,) = cx.reduce([kv], "sum")
    peak, _ = peaks()
    return {"workload": f"{name}: {w['text']}", "scaling": w["scaling"], "sessions_per_gpu": n_sess, "steps": steps,
            "ms_per_step": ms / steps, "value": cx.world * n_sess * steps / (ms / 1e3), "unit": UNIT,
            "kv_gbs": kv_all / ms / 1e6, "frac_per_gpu": kv_all / ms / 1e6 / cx.world / peak,
            "launch": "layer", "attention_kernel": "mma" if opt["kernel"] == 1 else "simt", "pdl": opt["pdl"]}


def long_context_measure(cx, args, K, W, collective):
    """Config 5 on several GPUs: every rank attends over its own range of the session's pages and the
    (m, l, acc) partial rows are merged in rank order.  collective "p2p": the whole step is issued natively,
    layer by layer, and the partial rows cross NVLink inside the per-layer launches (nova_batch_step_partial_peers);
    "layer" / "step": NCCL all-gather + nova_lse_combine per layer / once per step.  Returns the JSON line (rank 0)."""
    import torch
    import conflux_nova_b200.longctx as lc
    nv, wl, dist, rank, world = cx.nv, cx.wl, cx.dist, cx.rank, cx.world
    w = WORKLOADS["c5"]
    seed = BASE_SEED + w["cfg"]                       # the SAME session on every rank
    n_ctx = w["ctx"][0]
    # Every rank keeps the whole session's pool (7.5 GB) but fills and reads only its own page range.
    work = wl.Workload(w["model"], [n_ctx], seed=seed, steps=2 * (W + K) + 16, device=cx.local_rank, fill=False)
    eng, batch = work.eng, work.batch
    n_pages = (n_ctx + 15) // 16
    lo, hi = lc.page_range(rank, world, n_pages)
    first_tok, last_tok = lo * 16, min(hi * 16, n_ctx)
    if last_tok > first_tok:
        work.fill_context(work.sessions[0], first_tok, last_tok - first_tok, key_session=0)
    eng.set_n_past(work.sessions[0], n_ctx)
    batch.sync_positions()
    batch.set_kernel(1 if args.kernel != 0 else 0)
    if args.kernel != 0 and collective == "p2p":
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
    per_layer = collective == "layer"

    xch = status_word = None
    epoch = [0]
    if collective in ("p2p", "p2p-step"):
        xch = lc.PeerExchange(nv, NH if collective == "p2p" else L * NH, rank, world, dist, n_slots=2)
        status_word = nv.DevBuf(4).zero()
        dist.barrier()

    def step(st=st):
        if xch is not None and collective == "p2p":
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
    sampler = ClockSampler(cx.local_rank) if rank == 0 else None
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
    # the merged output must be finite and identical on every rank
    chk = out[-1].clone()
    dist.broadcast(chk, src=0)
    same = bool(torch.equal(chk, out[-1])) and bool(torch.isfinite(out).all())
    flag = torch.tensor([0.0 if same else 1.0], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MAX)
    differ = float(flag[0]) != 0.0
    if xch is not None:
        torch.cuda.synchronize()
        dist.barrier()                 # nobody closes a buffer a peer may still be reading or writing
        xch.close()
    for b in (dq, dk, dv):
        b.free()
    work.close()
    if bad:
        raise RuntimeError("device status set during the long-context run")
    if differ:
        raise RuntimeError("merged outputs differ between ranks")
    if rank != 0:
        return None
    peak, peak_kind = peaks()
    kv_bytes = sum((n0 + i + 1) * es_tok * L for i in range(K))          # whole session, all ranks together
    return {
        "metric": METRIC, "value": K / (ms / 1e3), "unit": UNIT, "n_gpus": world, "steps": K, "warmup": W,
        "ms_per_step": ms / K, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": f"c5: {w['text']}", "sessions_per_gpu": 1, "context_tokens": [n_ctx], "layers": L,
                   "kv_dtype": "fp16", "page_tokens": 16, "collective": COLLECTIVES[collective],
                   "pages_per_gpu": -(-n_pages // world), "l2": "inputs larger than L2"},
        "kv_gbs": kv_bytes / ms / 1e6, "kv_bytes_per_step": kv_bytes / K,
        "roofline": {"bound": "hbm", "achieved": kv_bytes / ms / 1e6 / world, "peak": peak, "unit": "GB/s",
                     "frac": kv_bytes / ms / 1e6 / world / peak, "traffic": None, "peak_kind": peak_kind,
                     "kernel": "attention over this GPU's page range + exchange + merge (per GPU)"},
        "e2e": None, "gpu_launches": launches, "clocks": clocks, "cpu_baseline": None,
    }


def prefill_sample(nv, work, stream, reps):
    """Paged prefill (the step before decode): every session takes a chunk of new tokens through all layers -
    multi-token RoPE+append, then causal attention of the chunk's queries over the paged keys."""
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
            "note": "time of the whole chunk (RoPE+append and attention launches of every layer); fp16 pools with pages of 16 "
                    "tokens or more: attention on tcgen05 + tensor memory unless --prefill-kernel 0 (mma.sync tiles); SIMT "
                    "kernel: one work-split row per query token"}


def reference_gpu_sample(nv, work):
    """The reference's own CUDA kernels for this path (src/kernel/rope.cu, elem.cu, attn.cu compiled
    unmodified for sm_100a, oracle/_ref) on this GPU, on a bounded sample of the same workload: one layer,
    every session, in the reference's call order (per session: rope_batch, kv_store_paged, attn_decode_paged
    = split + combine), fp32 pools holding the same values.  Time scaled by the layer count.  Second result: this
    library's raw launchers with the reference's argument lists (nova_launch_rope_append_paged +
    nova_launch_attn_decode_paged, what the shim header binds the reference's call sites to) in the same call
    order on the same fp32 pools - the literal drop-in."""
    import ctypes as C
    from oracle import binding as ob
    model = {"qwen25_7b": "qwen25_7b", "qwen25_1p5b": "qwen25_1p5b"}.get(work.model)
    g = ob.ref_gpu(model) if model else None
    if g is None:
        return None, None
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
    sh32 = nv.KvShape(NH, NKV, 128, 16, nv.KV_F32, 1)

    # one C call per pass on either side (per session: RopeKvOp then AttnOp): a Python loop over the launchers would
    # measure the interpreter (about 35 us per call), not the GPU
    tab_arr = (C.c_void_p * S)(*tabs)
    pos_arr = (C.c_int64 * S)(*pos)
    c_loops = hasattr(g, "ref_gpu_decode_layer_sessions")

    def ref_pass():
        if c_loops:
            g.ref_gpu_decode_layer_sessions(S, pk.ptr, pv.ptr, tab_arr, 0, eng.nb, pos_arr, q.ptr, k.ptr, v.ptr, NH * 128, NKV * 128,
                                            cs, sn, o.ptr, scr.ptr, st.h)
            return
        for i in range(S):
            qi, ki, vi = q.ptr + i * NH * 512, k.ptr + i * NKV * 512, v.ptr + i * NKV * 512
            g.ref_gpu_rope_batch(qi, ki, 1, pos[i], cs, sn, st.h)
            g.ref_gpu_kv_store_paged(pk.ptr, pv.ptr, tabs[i], 0, eng.nb, 1, pos[i], ki, vi, st.h)
            g.ref_gpu_attn_decode_paged(qi, pk.ptr, pv.ptr, tabs[i], 0, eng.nb, pos[i] + 1, o.ptr + i * NH * 512,
                                        scr.ptr, st.h)

    def ours_pass():
        if c_loops:
            nv.check(nv.lib.nova_launch_decode_layer_sessions(C.byref(sh32), S, pk.ptr, pv.ptr, tab_arr, 0, eng.nb, pos_arr, q.ptr, k.ptr,
                                                              v.ptr, NH * 128, NKV * 128, cs, sn, o.ptr, scr.ptr, st.h))
            return
        for i in range(S):
            qi, ki, vi = q.ptr + i * NH * 512, k.ptr + i * NKV * 512, v.ptr + i * NKV * 512
            nv.lib.nova_launch_rope_append_paged(C.byref(sh32), pk.ptr, pv.ptr, tabs[i], 0, eng.nb, 1, pos[i], qi, ki, vi,
                                                 cs, sn, st.h)
            nv.lib.nova_launch_attn_decode_paged(C.byref(sh32), qi, pk.ptr, pv.ptr, tabs[i], 0, eng.nb, pos[i] + 1,
                                                 o.ptr + i * NH * 512, scr.ptr, st.h)

    def time_pass(fn, reps=10):
        for _ in range(3):
            fn()
        st.sync()
        e0, e1 = nv.Event(), nv.Event()
        e0.record(st)
        for _ in range(reps):
            fn()
        e1.record(st)
        e1.sync()
        return e0.elapsed_ms(e1) / reps, reps
    ms_ref, reps = time_pass(ref_pass)
    ok = g.ref_gpu_last_error() == 0
    ms_ours, _ = time_pass(ours_pass)
    ms_ours_tc = None
    if nv.lib.nova_launcher_set_kernel(1) == nv.OK:          # the same launchers on the tensor-core kernel
        ms_ours_tc, _ = time_pass(ours_pass)
        nv.lib.nova_launcher_set_kernel(0)
    for b in (pk, pv, q, k, v, o, scr):
        b.free()
    sample = (f"{reps} x one layer of {eng.L}, all {S} sessions, fp32 pools, the reference's call order (per session and "
              f"layer){', each pass one C call' if c_loops else ''}; time scaled by {eng.L}")
    ref = {"value": S / (ms_ref * eng.L / 1e3), "unit": UNIT, "ms_per_step": ms_ref * eng.L, "ok": ok,
           "launches_per_session_layer": 4, "sample": sample}
    ours = {"value": S / (ms_ours * eng.L / 1e3), "unit": UNIT, "ms_per_step": ms_ours * eng.L,
            "launches_per_session_layer": 3, "speedup_vs_reference_kernels": ms_ref / ms_ours, "sample": sample,
            "kernel": "SIMT (fp32 arithmetic, the launchers' default)",
            "tensor_core_kernel": None if ms_ours_tc is None else {
                "ms_per_step": ms_ours_tc * eng.L, "value": S / (ms_ours_tc * eng.L / 1e3),
                "speedup_vs_reference_kernels": ms_ref / ms_ours_tc,
                "note": "nova_launcher_set_kernel(1): K/V rows rounded to fp16 on their way into the tensor cores"}}
    return ref, ours


def cpu_baseline_sample(nv, work, lens, seed):
    """The CPU restatement of the reference's path (oracle/, the checker) timed on this box's cores on
    a bounded sample of the same workload: one decode step of `sample_layers` layers, scaled to all."""
    from oracle import binding as ob
    ob.use_all_cores()
    eng = work.eng
    L, S = eng.L, len(work.sessions)
    sample_layers = 1
    sh = ob.shape(sample_layers, eng.NH, eng.NKV, ob.KV_F16, kv_block=eng.desc.kv_block)
    n = eng.nb * eng.page_bytes // 2
    shp = (sample_layers, eng.nb, eng.desc.kv_block, eng.NKV, eng.HD)
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
                      "fa_split_paged/fa_combine + rope/kv_store, OpenMP over (session, head)"}


# --------------------------------------------------------------------------------------------
REF_SHAPES = {"qwen25_1p5b": (28, 12, 2), "qwen25_7b": (28, 28, 4), "qwen25_14b": (48, 40, 8)}


def _mix64(x: int) -> int:
    m = (1 << 64) - 1
    x = (x + 0x9E3779B97F4A7C15) & m
    x = ((x ^ (x >> 30)) * 0xBF58476D1CE4E5B9) & m
    x = ((x ^ (x >> 27)) * 0x94D049BB133111EB) & m
    return x ^ (x >> 31)


def run_reference(args):
    """The reference arm: the reference has no CPU implementation of the attention itself (its only
    implementations are CUDA and SYCL kernels), so this times the CPU restatement of its algorithm
    (oracle/, kind "port") with every host core this process may use, on the same workload, same metric.
    Nothing of the product library is loaded here: the workload's context lengths and page permutations are
    re-derived with the checker's copy of the same integer hash."""
    rank, _, world = dist_env()
    if rank != 0:
        return
    from oracle import binding as ob
    cores = ob.use_all_cores()          # torchrun exports OMP_NUM_THREADS=1 to its children; do not inherit that
    w = WORKLOADS[args.workload]
    seed = BASE_SEED + w["cfg"]
    lo, hi = w["ctx"]
    lens = [lo + _mix64(ob.synth_key(seed, 10, s, 0)) % (hi - lo + 1) for s in range(w["sessions"])]
    Lfull, NH, NKV = REF_SHAPES[w["model"]]
    S = len(lens)

    def permutation(session, n):
        perm = np.arange(n, dtype=np.int32)
        state = ob.synth_key(seed, 9, session, 0)
        for i in range(n - 1, 0, -1):
            state = _mix64(state)
            j = state % (i + 1)
            perm[i], perm[j] = perm[j], perm[i]
        return perm
    sample_layers = 1
    sh = ob.shape(sample_layers, NH, NKV, ob.KV_F16)
    nblocks = (max(lens) + args.steps + args.warmup + 16 + 15) // 16
    nb = nblocks * S
    pk, pv = ob.new_pools(sh, nb)
    cs, sn = ob.rope_table(nblocks * 16)
    tables = np.stack([s * nblocks + permutation(s, nblocks) for s in range(S)]).astype(np.int32)
    row = NKV * 128
    for s in range(S):          # cached context through the checker's append, same seeded values
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
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
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
                    help="c5 on several GPUs: p2p = partial rows exchanged inside the per-layer launches (engine order); "
                         "layer / step = NCCL all-gather + merge per layer / once per step; p2p-step = peer reads once per step")
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--launch", default="layer", choices=["layer", "graph", "fused"],
                    help="layer: one attention launch per layer; graph: the same, replayed from a CUDA graph; fused: all layers per launch")
    ap.add_argument("--kernel", type=int, default=-1, help="-1 best available, 0 SIMT, 1 tensor-core")
    ap.add_argument("--no-fused-append", action="store_true",
                    help="keep RoPE+append as its own launch instead of doing it inside the attention launch")
    ap.add_argument("--row-setup", type=int, default=-1, help="work-split weight of a session start, in pages")
    ap.add_argument("--split-ctas", type=int, default=0, help="CTAs of a tensor-core attention launch (0 = the library's choice)")
    ap.add_argument("--no-cascade", action="store_true", help="config 3: attend the shared prefix per session, as the plain path does")
    ap.add_argument("--no-pdl", action="store_true", help="no programmatic dependent launch between layers")
    ap.add_argument("--late-inputs", action="store_true",
                    help="headline with q / new k / new v read only after the previous layer's kernels have finished")
    ap.add_argument("--kv", default="f16", choices=["f16", "f32"],
                    help="KV pool element type (f32 = the reference's own format)")
    ap.add_argument("--page-tokens", type=int, default=16, choices=[8, 16, 32, 64],
                    help="tokens per KV page (the reference's NOVA_KV_BLOCK; single-GPU workloads)")
    ap.add_argument("--prefill-kernel", type=int, default=-1,
                    help="prefill attention: 0 mma.sync tiles, 1 tcgen05 + tensor memory, -1 the library's default")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-ref-gpu", action="store_true", help="skip timing the reference's own kernels (sm_100a build)")
    ap.add_argument("--no-scaling-workloads", action="store_true", help="skip configurations 4 and 5 after the headline")
    ap.add_argument("--quick-prefill", action="store_true", help="only the prefill sample (for profiler captures)")
    ap.add_argument("--sessions", type=int, default=0, help="override the workload's session count (cut-down cases for profiler captures)")
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
