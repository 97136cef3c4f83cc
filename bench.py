#!/usr/bin/env python
"""Benchmark of the paged-KV decode hot path (fused RoPE + K/V append + paged decode attention).

Workload (`config.workload`): the Llama-3-8B-shaped decode layer - 32 query / 8 KV heads, head_dim 128,
bf16, page_size 16, a pool of 32768 pages with a fragmented (seeded-permutation) page table, 64 requests
with context lengths uniform in [512, 4096]; every step appends one token per request and attends over
all of that request's pages.  Data are synthetic (seeded N(0,1)*0.5); no dataset is involved.

A "step" is one pass of the path over the batch: RoPE of q and of the new k, append of k / v into the
pages and decode attention, in ONE fused kernel launch.  Steps run back to back on one stream from a
captured CUDA graph.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N > 1 (launched by torch.distributed.run, one rank per GPU): requests are sharded across GPUs with
independent page pools and no data-path collective - every rank runs its own 64-request batch
(weak scaling); time is the max over ranks.

Printed JSON line: metric = decode tokens/s (whole job), `value` with inputs resident in HBM, `e2e`
through pie_b200.ops with pinned HOST buffers (H2D of the step's q/k/v + metadata and D2H of the
attention output inside the timed region), `roofline` for the fused kernel of the timed region (algorithmic
bytes / CUDA-event time against the measured HBM copy bandwidth; the attention-only variant beside it),
`cpu_baseline` = the CPU oracle on a bounded sample.  The same line carries sub-records of the secondary
workloads, measured after the headline's timed region: `head_sharded` (70B-shaped decode, KV heads split
over the N ranks and joined by the decode kernel's peer stores, with the NCCL all-gather and the one-GPU
step beside it) and `oproj` (the o_proj of that layer with the sum over the ranks and the residual in the
kernel's epilogue, matmul + NCCL all-reduce + add beside it) at every N, and `prefill` (chunked-prefill mix,
tensor-core roofline), `beam` (beam search with shared pages) and `qkv` (QKV projection with RoPE + append as
its epilogue) at N = 1.  `--impl reference` times the CPU restatement of the reference path
on the host cores; `--impl flashinfer` times the reference's CUDA dependency as a black box.
"""
from __future__ import annotations

import argparse
import datetime
import json
import math
import os
import sys
import threading
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "decode_tokens_per_s"
UNIT = "tokens/s"
WORKLOAD = "llama3-8b-shaped decode layer: 32q/8kv heads, D128, bf16, page16, 32768-page pool, " \
           "64 requests/GPU, ctx U[512,4096], +1 token/request/step"
HORIZON = 512  # distinct consecutive steps of metadata; longer runs wrap around

# DRAM traffic of the decode kernel = (dram__bytes_read.sum + dram__bytes_write.sum) / algorithmic bytes from
# one ncu capture of a 32-request case (328.2 MB moved for 322.5 MB algorithmic; profiles/decode_tma_config2.md).
# Traffic grows with the pages streamed, so the launch's traffic is its algorithmic bytes times this ratio.
NCU_TRAFFIC_RATIO = 1.018


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return float(p["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


def load_peaks_tensor():
    """(sustained bf16 matmul TFLOP/s, where it came from)."""
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["bf16_tflops_sustained"]), "measured (sustained bf16 matmul)"
    except Exception:
        return 1400.0, "fallback"


class ClockSampler:
    """Polls SM clock and throttle reasons through NVML while the timed region runs."""

    REASONS = {
        0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
        0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nv = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = index
            if visible:
                try:
                    phys = int(visible.split(",")[index])
                except Exception:
                    phys = index
            self._h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for bit, name in self.REASONS.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.004)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": ["nvml unavailable"]}
        return {"sm_mhz": float(np.median(self.samples)), "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


# ---------------------------------------------------------------------------------------------
# workload
# ---------------------------------------------------------------------------------------------
def build_steps(rank: int, horizon: int, batch: int = 64, num_pages: int = 32768):
    from pie_b200 import workloads as W

    # weak scaling: every GPU gets the SAME draw of context lengths (the workload's seed 1), so the work
    # per GPU is fixed as N grows and the max over ranks compares like with like; the page tables
    # (fragmentation) and the tensor contents differ per rank
    reqs = W.config2_requests(batch=batch, seed=1, num_pages=num_pages, perm_seed=1 + rank)
    return W.decode_steps(reqs, horizon)


def pack_meta(meta, tmax: int) -> np.ndarray:
    """One int32 row per step: [kv_indptr (B+1) | last_len (B) | pos_ids (B) | qo_indptr (B+1) | indices (tmax)]."""
    row = np.zeros(meta.batch * 4 + 2 + tmax, dtype=np.int32)
    b = meta.batch
    row[: b + 1] = meta.kv_indptr
    row[b + 1: 2 * b + 1] = meta.kv_last_page_len
    row[2 * b + 1: 3 * b + 1] = meta.pos_ids
    row[3 * b + 1: 4 * b + 2] = meta.qo_indptr
    row[4 * b + 2: 4 * b + 2 + len(meta.kv_indices)] = meta.kv_indices
    return row


def views(row: torch.Tensor, b: int):
    return dict(indptr=row[: b + 1], last=row[b + 1: 2 * b + 1], pos=row[2 * b + 1: 3 * b + 1],
                qo=row[3 * b + 1: 4 * b + 2], indices=row[4 * b + 2:])


# ---------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------
def headline_config(W, requests: int, n_gpus: int, num_pages: int, steps: int, warmup: int) -> dict:
    """The `config` object of the headline line.  Both arms (this library and `--impl reference`) print
    exactly this, computed from the same seeded metadata, so that their lines describe one workload."""
    horizon = min(HORIZON, steps + warmup)
    cfg = W.CONFIG2
    metas = W.decode_steps(W.config2_requests(batch=requests, seed=1, num_pages=num_pages, perm_seed=1), horizon)
    mid = metas[(warmup + steps // 2) % horizon]
    return {"workload": WORKLOAD, "requests_per_gpu": requests, "global_requests": requests * n_gpus,
            "pool_pages": num_pages,
            "parallelism": f"request-sharded x{n_gpus}, independent page pools, no collective",
            "l2": "inputs larger than L2 (0.6 GB of KV per step vs 126 MB); no flush",
            "step_algorithmic_bytes": W.decode_step_bytes(mid, cfg)}


def run_ours(args):
    import torch.distributed as dist

    from pie_b200 import ops
    from pie_b200 import workloads as W
    from pie_b200._lib import lib, check
    import ctypes as C

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        # a collective that a failed rank never joins gives up after five minutes, not the default ten
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=300))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    n_gpus = world

    cfg = W.CONFIG2
    if args.pages != cfg.num_pages:
        import dataclasses
        cfg = dataclasses.replace(cfg, num_pages=args.pages)
    B, HQ, HKV, D = args.requests, cfg.num_qo_heads, cfg.num_kv_heads, cfg.head_dim
    steps, warmup = args.steps, args.warmup
    horizon = min(HORIZON, steps + warmup)
    metas = build_steps(rank, horizon, B, cfg.num_pages)
    tmax = max(len(m.kv_indices) for m in metas)
    packed_host = torch.from_numpy(np.stack([pack_meta(m, tmax) for m in metas])).pin_memory()
    packed = packed_host.to(dev)

    pool = W.randn(cfg.pool_shape(), 100 + rank, cfg.dtype, cfg.value_scale, device=dev)
    n_var = 8  # distinct q/k/v inputs cycled over the steps
    qkv_host = W.randn((n_var, B, (HQ + 2 * HKV) * D), 200 + rank, cfg.dtype, cfg.value_scale).pin_memory()
    qkv = qkv_host.to(dev)
    out = torch.empty((B, HQ, D), dtype=cfg.dtype, device=dev)
    ws = torch.zeros(64 << 20, dtype=torch.uint8, device=dev)
    err = torch.zeros(4, dtype=torch.int32, device=dev)
    rope = ops.RopeConfig(mode=cfg.rope_mode, theta=cfg.rope_theta, scale=cfg.rope_scale).to_c(D)
    sm_scale = 1.0 / math.sqrt(D)
    stream = torch.cuda.Stream(dev)
    launches = [0]
    es = 2

    # Programmatic dependent launch: the page tables are static inputs, and the kernel before a step is the
    # previous decode step of the same requests, which wrote one token per request - into what is now a
    # request's last or last-but-one page (mode 3's promise; it also holds where the replayed graph wraps
    # around to its first step, whose contexts are shorter).
    ops.set_programmatic_dependent_launch(args.pdl)

    def qkv_views(t):
        q = t[:, : HQ * D].view(B, HQ, D)
        k = t[:, HQ * D: (HQ + HKV) * D].view(B, HKV, D)
        v = t[:, (HQ + HKV) * D:].view(B, HKV, D)
        return q, k, v

    def step_device(i: int, st: int):
        """One step on device-resident inputs through the C ABI: a single fused launch."""
        mv = views(packed[i % horizon], B)
        q, k, v = qkv_views(qkv[i % n_var])
        check(lib.piekv_decode_step_fused(q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), q.stride(1),
                                          k.stride(0), k.stride(1), v.stride(0), v.stride(1), mv["pos"].data_ptr(),
                                          pool.data_ptr(), out.data_ptr(), None, mv["indptr"].data_ptr(),
                                          mv["indices"].data_ptr(), mv["last"].data_ptr(), B, HQ, HKV, D, 16,
                                          cfg.num_pages, 2, C.byref(rope), sm_scale, ws.data_ptr(), ws.numel(),
                                          err.data_ptr(), st), "decode_step_fused")
        launches[0] += 1

    def barrier():
        # device idle first: the barrier's own NCCL kernel would otherwise run (and spin) beside the
        # timed kernels and take an SM away from a grid that fills all of them
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    def max_over_ranks(x: float) -> float:
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- value: device-resident, CUDA graph of exactly `steps` steps -------------------------------
    # The graph holds the driver's K steps.  It is replayed R times back to back inside ONE event pair so
    # that the timed region lasts about a quarter of a second whatever K is (clock samples, power state);
    # steps / ms_per_step stay per step, `timed_replays` = R.
    torch.cuda.synchronize(dev)  # the inputs were made on the default stream; `stream` is not ordered behind it
    with torch.cuda.stream(stream):
        for i in range(warmup):
            step_device(i, stream.cuda_stream)
    stream.synchronize()
    graph = torch.cuda.CUDAGraph()
    launches[0] = 0
    with torch.cuda.graph(graph, stream=stream):
        for i in range(steps):
            step_device(warmup + i, torch.cuda.current_stream(dev).cuda_stream)
    graph_launches = launches[0]
    p0, p1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(stream):
        graph.replay()  # one untimed replay: graph upload + caches
        p0.record(stream)
        graph.replay()
        p1.record(stream)
    barrier()
    probe_ms = max_over_ranks(p0.elapsed_time(p1))
    replays = 1 if args.min_timed_ms <= 0 else int(min(4096, max(1, math.ceil(args.min_timed_ms / max(probe_ms, 1e-3)))))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(local)
    with sampler:
        barrier()
        with torch.cuda.stream(stream):
            e0.record(stream)
            for _ in range(replays):
                graph.replay()
            e1.record(stream)
        barrier()
    total_ms = max_over_ranks(e0.elapsed_time(e1))
    ms_per_step = total_ms / (steps * replays)
    value = n_gpus * B / (ms_per_step * 1e-3)
    timed_launches = graph_launches * replays
    errw = err.cpu().tolist()

    # ---- roofline: the fused kernel is the timed region; the attention-only variant is timed beside it ---
    reps = args.kernel_reps
    mid = metas[(warmup + steps // 2) % horizon]
    mv = views(packed[(warmup + steps // 2) % horizon], B)
    q, _, _ = qkv_views(qkv[0])

    def decode_only(st):
        check(lib.piekv_decode_run(q.data_ptr(), q.stride(0), q.stride(1), pool.data_ptr(), out.data_ptr(), None,
                                   mv["indptr"].data_ptr(), mv["indices"].data_ptr(), mv["last"].data_ptr(), B, HQ,
                                   HKV, D, 16, cfg.num_pages, 2, sm_scale, ws.data_ptr(), ws.numel(),
                                   err.data_ptr(), st), "decode_run")

    with torch.cuda.stream(stream):
        for _ in range(5):
            decode_only(stream.cuda_stream)
        k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k0.record(stream)
        for _ in range(reps):
            decode_only(stream.cuda_stream)
        k1.record(stream)
    stream.synchronize()
    kern_ms = k0.elapsed_time(k1) / reps
    tokens = int(mid.seq_lens.astype(np.int64).sum())
    kern_bytes = tokens * 2 * HKV * D * es + B * 2 * HQ * D * es + 4 * (len(mid.kv_indices) + 2 * B + 1)
    peak, peak_kind = load_peaks()
    attn_achieved = kern_bytes / (kern_ms * 1e-3) / 1e9
    step_bytes = W.decode_step_bytes(mid, cfg)
    step_achieved = step_bytes / (ms_per_step * 1e-3) / 1e9

    # ---- e2e: public Python API, host buffers, H2D + D2H inside the timed region ---------------------
    # Throughput form: three streams (upload, compute, download) and three buffer sets: the upload of step
    # i+1 and the download of step i-1 overlap the kernel of step i; every step still uploads its own q/k/v
    # and page tables from pinned host memory and downloads its own attention output.  The steps are
    # INDEPENDENT of one another here (a real decode loop feeds step i's output into step i+1's q and cannot
    # overlap them); the un-pipelined per-step latency is reported beside it.
    e2e_steps = max(steps, min(2048, int(args.min_timed_ms / 0.15) if args.min_timed_ms > 0 else steps))
    NB = 3
    out_host = [torch.empty((B, HQ, D), dtype=cfg.dtype).pin_memory() for _ in range(NB)]
    out_devs = [torch.empty((B, HQ, D), dtype=cfg.dtype, device=dev) for _ in range(NB)]
    meta_devs = [torch.empty(packed.shape[1], dtype=torch.int32, device=dev) for _ in range(NB)]
    qkv_devs = [torch.empty_like(qkv[0]) for _ in range(NB)]
    rope_cfg = ops.RopeConfig(mode=cfg.rope_mode, theta=cfg.rope_theta, scale=cfg.rope_scale)
    wrapper = ops.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")
    h2d = packed_host[0].numel() * 4 + qkv_host[0].numel() * es
    d2h = out_host[0].numel() * es
    s_in, s_comp, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)
    ev_in = [torch.cuda.Event() for _ in range(NB)]
    ev_comp = [torch.cuda.Event() for _ in range(NB)]
    ev_out = [torch.cuda.Event() for _ in range(NB)]
    issued = [0]

    def step_e2e(i: int):
        b = issued[0] % NB
        first_use = issued[0] < NB
        issued[0] += 1
        with torch.cuda.stream(s_in):
            if not first_use:
                s_in.wait_event(ev_comp[b])  # the kernel that read this buffer set has finished
            meta_devs[b].copy_(packed_host[i % horizon], non_blocking=True)
            qkv_devs[b].copy_(qkv_host[i % n_var], non_blocking=True)
            ev_in[b].record(s_in)
        with torch.cuda.stream(s_comp):
            s_comp.wait_event(ev_in[b])
            if not first_use:
                s_comp.wait_event(ev_out[b])  # the previous output in this buffer has been downloaded
            mv_ = views(meta_devs[b], B)
            q_, k_, v_ = qkv_views(qkv_devs[b])
            wrapper.plan(mv_["indptr"], mv_["indices"], mv_["last"], HQ, HKV, D, 16, pos_encoding_mode="NONE",
                         q_data_type=cfg.dtype)
            wrapper.run_fused(q_, k_, v_, mv_["pos"], pool, rope_cfg, out=out_devs[b])
            ev_comp[b].record(s_comp)
        with torch.cuda.stream(s_out):
            s_out.wait_event(ev_comp[b])
            out_host[b].copy_(out_devs[b], non_blocking=True)
            ev_out[b].record(s_out)

    ops.set_programmatic_dependent_launch(0)
    torch.cuda.synchronize(dev)  # buffers and the wrapper above were made on the default stream
    for i in range(3):
        step_e2e(i)
    barrier()
    c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    c0.record(s_in)
    for i in range(e2e_steps):
        step_e2e(warmup + i)
    c1.record(s_out)
    barrier()
    e2e_ms = max_over_ranks(c0.elapsed_time(c1))
    e2e_value = n_gpus * B * e2e_steps / (e2e_ms * 1e-3)
    e2e_eager_value, e2e_mode = e2e_value, "eager launches from Python"
    # The same pipeline captured once as a CUDA graph (copy, kernel and copy nodes of 128 steps on three
    # streams) and replayed: no Python or launch latency between the steps, and consecutive kernels are
    # adjacent nodes again, so the promise behind the launch-overlap mode holds as in the headline (the kernel
    # before a step wrote at most the requests' last pages; page tables and q / k / v arrive by copy nodes the
    # kernel depends on in full).
    try:
        g_steps = min(e2e_steps, 128)
        g_replays = max(1, -(-e2e_steps // g_steps))
        ops.set_programmatic_dependent_launch(args.pdl)
        torch.cuda.synchronize(dev)
        issued[0] = 0
        g_e2e = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g_e2e, stream=s_comp):
            fork = torch.cuda.Event()
            fork.record(s_comp)
            s_in.wait_event(fork)
            s_out.wait_event(fork)
            for i in range(g_steps):
                step_e2e(warmup + i)
            j_in, j_out = torch.cuda.Event(), torch.cuda.Event()
            j_in.record(s_in)
            j_out.record(s_out)
            s_comp.wait_event(j_in)
            s_comp.wait_event(j_out)
        with torch.cuda.stream(s_comp):
            g_e2e.replay()
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(s_comp):
            g0.record(s_comp)
            for _ in range(g_replays):
                g_e2e.replay()
            g1.record(s_comp)
        barrier()
        g_ms = max_over_ranks(g0.elapsed_time(g1))
        g_value = n_gpus * B * g_steps * g_replays / (g_ms * 1e-3)
        if ops.device_error(dev, clear=False) is None and g_value > e2e_value:
            e2e_value, e2e_ms, e2e_steps = g_value, g_ms, g_steps * g_replays
            e2e_mode = f"CUDA graph of {g_steps} pipelined steps replayed {g_replays}x"
        del g_e2e
    except Exception as e:  # the eager figure stands
        e2e_mode = f"eager launches from Python (graph capture failed: {type(e).__name__})"
        torch.cuda.synchronize(dev)
    ops.set_programmatic_dependent_launch(0)

    # latency form: one buffer set, one stream, the host waits for the output before it issues the next step
    lat_steps = min(64, max(8, steps))
    s_lat = torch.cuda.Stream(dev)

    def step_latency(i: int):
        with torch.cuda.stream(s_lat):
            meta_devs[0].copy_(packed_host[i % horizon], non_blocking=True)
            qkv_devs[0].copy_(qkv_host[i % n_var], non_blocking=True)
            mv_ = views(meta_devs[0], B)
            q_, k_, v_ = qkv_views(qkv_devs[0])
            wrapper.plan(mv_["indptr"], mv_["indices"], mv_["last"], HQ, HKV, D, 16, pos_encoding_mode="NONE",
                         q_data_type=cfg.dtype)
            wrapper.run_fused(q_, k_, v_, mv_["pos"], pool, rope_cfg, out=out_devs[0])
            out_host[0].copy_(out_devs[0], non_blocking=True)
        s_lat.synchronize()

    for i in range(3):
        step_latency(i)
    barrier()
    t0 = time.perf_counter()
    for i in range(lat_steps):
        step_latency(warmup + i)
    lat_us = max_over_ranks((time.perf_counter() - t0) / lat_steps * 1e6)

    # free the headline's buffers before the secondary workloads allocate theirs
    del graph, pool, qkv, out_devs, qkv_devs, meta_devs, wrapper
    torch.cuda.empty_cache()

    # ---- secondary workloads, reported inside the same line (they do not change metric / value) -------
    sub = {}
    if not args.no_sub:
        try:
            sub["head_sharded"] = measure_head_sharded(world, rank, dev, steps=48, warmup=4)
        except Exception as e:  # a sub-record must never cost the headline its line
            sub["head_sharded"] = {"error": f"{type(e).__name__}: {str(e)[:300]}"}
        try:
            sub["oproj"] = measure_oproj(world, rank, dev, steps=24, warmup=4)
        except Exception as e:
            sub["oproj"] = {"error": f"{type(e).__name__}: {str(e)[:300]}"}
        if world == 1:
            for name, fn in (("prefill", lambda: prefill_subrecord(dev)), ("beam", lambda: beam_subrecord(dev)),
                             ("qkv", lambda: qkv_subrecord(dev))):
                try:
                    sub[name] = fn()
                except Exception as e:
                    sub[name] = {"error": f"{type(e).__name__}: {str(e)[:300]}"}

    # ---- cpu baseline (rank 0, N=1 only): the CPU oracle on a bounded sample --------------------------
    cpu = None
    if world == 1 and not args.no_cpu:
        cpu = cpu_baseline(sample_steps=args.cpu_steps)

    if rank == 0:
        config = headline_config(W, B, n_gpus, cfg.num_pages, steps, warmup)
        assert config["step_algorithmic_bytes"] == step_bytes  # rank 0 timed exactly the workload it names
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": n_gpus, "steps": steps, "warmup": warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": config,
            "launch": f"CUDA graph of the {steps} timed steps, one fused kernel per step, programmatic dependent "
                      f"launch mode {args.pdl}; the graph is replayed {replays}x inside one CUDA-event pair",
            "timed_replays": replays, "timed_region_ms": total_ms,
            "clocks": sampler.summary(),
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "steps": e2e_steps, "ms_per_step": e2e_ms / e2e_steps,
                    "latency_us_per_step": lat_us, "latency_steps": lat_steps,
                    "launch": e2e_mode, "eager_value": e2e_eager_value,
                    "how": "pie_b200.ops wrappers; per step H2D of q/k/v + page tables from pinned memory and D2H of the "
                           "output. `value`: INDEPENDENT steps pipelined over upload / compute / download streams with "
                           "3 buffer sets (throughput), as eager launches (`eager_value`) and as one captured CUDA graph of the "
                           "same calls (`launch` says which the value is). `latency_us_per_step`: one buffer set, upload -> fused step -> "
                           "download, host synchronised after every step (what a dependent decode loop pays)"},
            "gpu_launches": timed_launches,
            "roofline": {"bound": "hbm",
                         "kernel": "decode_tma_kernel<bf16, 8 kv heads, fused RoPE + append + attention> (the timed region)",
                         "achieved": step_achieved, "peak": peak, "unit": "GB/s", "frac": step_achieved / peak,
                         "peak_source": peak_kind,
                         "traffic": int(step_bytes * NCU_TRAFFIC_RATIO),
                         "traffic_source": "ncu capture of a 32-request case, scaled by bytes streamed",
                         "bytes_per_launch": step_bytes, "us_per_launch": ms_per_step * 1e3,
                         "frac_of_nominal_8tbs": step_achieved / 8000.0,
                         "attention_only": {"kernel": "decode_tma_kernel<bf16, 8 kv heads> via piekv_decode_run, "
                                                      f"{reps} back-to-back launches", "achieved": attn_achieved,
                                            "frac": attn_achieved / peak, "bytes_per_launch": kern_bytes,
                                            "us_per_launch": kern_ms * 1e3,
                                            "frac_of_nominal_8tbs": attn_achieved / 8000.0}},
            "device_error_word": errw,
        }
        line.update(sub)
        if cpu is not None:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------
# secondary workload: chunked prefill mix (tensor-core bound); `--workload prefill`
# ---------------------------------------------------------------------------------------------
def prefill_leg(args):
    """8 new prompts of 2048 tokens + 8 chunks of 512 tokens on 6144 cached tokens, causal, 32q/8kv
    heads, D128, bf16, page 16.  A step = RoPE + append of all 20480 tokens, then paged prefill attention.
    Reports causal-exact TFLOP/s (4*D*Hq*allowed pairs) of the attention kernel against the measured
    bf16 matmul peak."""
    from pie_b200 import ops
    from pie_b200 import workloads as W

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    cfg = W.CONFIG3
    scale = args.prefill_scale
    meta = W.config3_meta(num_prompts=max(1, int(8 * scale)), num_chunks=max(1, int(8 * scale)), num_pages=args.pages
                          if args.pages != 32768 else 8192)
    num_pages = args.pages if args.pages != 32768 else 8192
    HQ, HKV, D = cfg.num_qo_heads, cfg.num_kv_heads, cfg.head_dim
    n = meta.nnz
    pool = W.randn((num_pages, 2, 16, HKV, D), 300, cfg.dtype, 0.5, device=dev)
    qkv = W.randn((n, (HQ + 2 * HKV) * D), 301, cfg.dtype, 0.5, device=dev)
    q = qkv[:, : HQ * D].view(n, HQ, D)
    k = qkv[:, HQ * D: (HQ + HKV) * D].view(n, HKV, D)
    v = qkv[:, (HQ + HKV) * D:].view(n, HKV, D)

    def t(x):
        return torch.from_numpy(np.ascontiguousarray(x)).to(dev)

    qo, indptr, indices, last, pos = t(meta.qo_indptr), t(meta.kv_indptr), t(meta.kv_indices), \
        t(meta.kv_last_page_len), t(meta.pos_ids)
    ws = torch.zeros(64 << 20, dtype=torch.uint8, device=dev)
    out = torch.empty((n, HQ, D), dtype=cfg.dtype, device=dev)
    seq = ops.get_seq_lens(indptr, last, 16)
    bi, kp = ops.get_batch_indices_positions(qo, seq, n)
    rope = ops.RopeConfig()
    w = ops.BatchPrefillWithPagedKVCacheWrapper(ws, "NHD")
    w.plan(qo, indptr, indices, last, HQ, HKV, D, 16, causal=True, q_data_type=cfg.dtype)
    mask = None
    mask_plan = None
    if args.prefill_mask or args.prefill_brle:
        # the causal mask in the wire form (one attend run of position + 1 entries per query token), then
        # either expanded on the host to the reference's flat boolean mask and uploaded, or uploaded as
        # runs and expanded to bits on the device
        from pie_b200.batching import decode_brle_batch
        counts = np.diff(meta.qo_indptr).astype(np.int64)
        seq_l = np.asarray(meta.seq_lens, dtype=np.int64)
        tok_pos = np.arange(n, dtype=np.int64) - np.repeat(meta.qo_indptr[:-1].astype(np.int64), counts) \
            + np.repeat(seq_l - counts, counts)
        runs_np = (tok_pos + 1).astype(np.uint32)
        rptr_np = np.arange(n + 1, dtype=np.int32)
        acc = np.zeros(n + 1, dtype=np.int64)
        np.cumsum(np.repeat(seq_l, counts), out=acc[1:])
        mask_bits = int(acc[-1])
        reps = 5
        m0, m1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        if args.prefill_brle:
            h_runs = torch.from_numpy(runs_np.view(np.int32).copy()).pin_memory()
            h_ptr = torch.from_numpy(rptr_np).pin_memory()
            d_runs, d_ptr = torch.empty_like(h_runs, device=dev), torch.empty_like(h_ptr, device=dev)
            t_host0 = time.perf_counter()
            t_host = time.perf_counter() - t_host0  # nothing to expand on the host
            for i in range(reps + 1):
                if i == 1:
                    m0.record()
                d_runs.copy_(h_runs, non_blocking=True)
                d_ptr.copy_(h_ptr, non_blocking=True)
                w.plan(qo, indptr, indices, last, HQ, HKV, D, 16, brle_mask=(d_runs, d_ptr, mask_bits),
                       q_data_type=cfg.dtype)
                w._device_plan(n, num_pages)
            m1.record()
            h2d = h_runs.numel() * 4 + h_ptr.numel() * 4
            form = "BRLE runs expanded to bits on the device"
            mask = d_runs
        else:
            t_host0 = time.perf_counter()
            flat = decode_brle_batch(runs_np, rptr_np, tok_pos, acc)
            t_host = time.perf_counter() - t_host0
            h_mask = torch.from_numpy(flat).pin_memory()
            mask = torch.empty_like(h_mask, device=dev)
            for i in range(reps + 1):
                if i == 1:
                    m0.record()
                mask.copy_(h_mask, non_blocking=True)
                w.plan(qo, indptr, indices, last, HQ, HKV, D, 16, custom_mask=mask, q_data_type=cfg.dtype)
                w._device_plan(n, num_pages)
            m1.record()
            h2d = h_mask.numel()
            form = "flat boolean mask (reference form), bit-packed on the device"
        torch.cuda.synchronize(dev)
        mask_plan = {"form": form, "h2d_bytes": int(h2d), "upload_plus_plan_ms": m0.elapsed_time(m1) / reps,
                     "host_expand_ms": t_host * 1e3, "pairs": mask_bits}

    def step():
        ops.rope_append_paged_kv_cache(q, k, v, pos, bi, kp, pool, indices, indptr, last, rope)
        w.run(q, pool, out=out)

    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize(dev)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(dev.index or 0)
    with sampler:
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize(dev)
    ms = e0.elapsed_time(e1) / args.steps
    # attention kernel alone
    a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a0.record()
    for _ in range(args.steps):
        w.run(q, pool, out=out)
    a1.record()
    torch.cuda.synchronize(dev)
    attn_ms = a0.elapsed_time(a1) / args.steps
    pairs = W.causal_pairs(meta)
    flops = 4.0 * D * HQ * pairs
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            pk = json.load(f)
        peak, peak_kind = float(pk["bf16_tflops_sustained"]), "measured (sustained bf16 matmul)"
    except Exception:
        peak, peak_kind = 1400.0, "fallback"
    tf = flops / (attn_ms * 1e-3) / 1e12
    line = {
        "metric": "prefill_tokens_per_s", "value": n / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "dtype": "bf16",
        "data": "synthetic",
        "config": {"workload": f"chunked prefill mix: {meta.batch} requests, {n} query tokens, causal "
                               f"({'BRLE mask' if args.prefill_brle else 'boolean custom mask' if mask is not None else 'native causal flag'}), "
                               "32q/8kv heads, D128, bf16, page16", "pool_pages": num_pages},
        "clocks": sampler.summary(),
        "roofline": {"bound": "tensor", "kernel": "prefill_tc2_kernel (two query heads per CTA)", "achieved": tf, "peak": peak,
                     "unit": "TFLOP/s", "frac": tf / peak, "peak_source": peak_kind, "traffic": None,
                     "flops_causal_exact": flops, "ms_per_launch": attn_ms},
        "mask_plan": mask_plan,
        "device_error_word": ops.device_error(dev),
    }
    return line


def run_prefill(args):
    print(json.dumps(prefill_leg(args)), flush=True)


def prefill_subrecord(dev):
    """The `prefill` sub-record of the headline line: the chunked-prefill mix with the native causal flag, in a
    loop long enough (about half a second of attention launches) for the sustained-clock regime the
    tensor-core peak is quoted in."""
    import types

    a = types.SimpleNamespace(prefill_scale=1.0, pages=32768, prefill_mask=False, prefill_brle=False, warmup=10,
                              steps=500)
    line = prefill_leg(a)
    return {"workload": line["config"]["workload"], "tokens_per_s": line["value"], "ms_per_step": line["ms_per_step"],
            "ms_per_launch": line["roofline"]["ms_per_launch"], "launches_timed": a.steps,
            "roofline": line["roofline"], "clocks": line["clocks"], "device_error_word": line["device_error_word"]}


# ---------------------------------------------------------------------------------------------
# secondary workload: 70B-shaped decode with eviction churn, KV heads sharded over the ranks
# ---------------------------------------------------------------------------------------------
def decode70b_leg(world, rank, dev, steps, warmup, join="peer", graph=False, batch=256, num_pages=None,
                  group_world=None, shard_of=1):
    """One timed leg of the 70B-shaped workload.  `world` ranks share the heads (world == 1: all heads on this
    GPU, no join).  Returns a dict of raw figures; every rank of the group must call it together when
    world > 1.  64 q / 8 kv heads, D128, bf16, `batch` requests with lognormal contexts; every 32 steps 20 % of
    the requests are evicted, their pages recycled and the slots refilled with 1024-token contexts written
    through the RoPE + append kernel.  `shard_of` > 1 (one GPU only): the head counts one rank of that many
    would hold, with no join - the per-GPU shape of the sharded step, for profiling."""
    import torch.distributed as dist

    from pie_b200 import ops, parallel
    from pie_b200 import workloads as W

    cfg = W.CONFIG5
    B, D = batch, cfg.head_dim
    hq, hkv = cfg.num_qo_heads // (world * shard_of), cfg.num_kv_heads // (world * shard_of)
    num_pages = num_pages or cfg.num_pages
    reqs = W.config5_requests(B, 5, num_pages)

    def t(x):
        return torch.from_numpy(np.ascontiguousarray(x)).to(dev)

    # the schedule is identical on every rank (seeded): per step the page table, per churn the refill lists
    plan = []
    for s in range(steps + warmup):
        refill = None
        if s > 0 and s % 32 == 0:
            victims = W.eviction_victims(B, s)
            for r in victims:
                reqs.evict(r, 1024)
            idx, ptr, last = reqs.csr()
            qo = np.zeros(B + 1, np.int64)
            for r in victims:
                qo[r + 1] = 1024
            qo = np.cumsum(qo).astype(np.int32)
            pos = np.tile(np.arange(1024, dtype=np.int32), len(victims))
            refill = dict(indices=t(idx), indptr=t(ptr), last=t(last), qo=t(qo), pos=t(pos), n=int(qo[-1]))
        m = W.decode_steps(reqs, 1)[0]
        plan.append(dict(meta=m, indices=t(m.kv_indices), indptr=t(m.kv_indptr), last=t(m.kv_last_page_len),
                         pos=t(m.pos_ids), refill=refill))
    pool = W.randn((num_pages, 2, 16, hkv, D), 100 + rank, cfg.dtype, 0.5, device=dev)
    qkv = W.randn((4, B, (hq + 2 * hkv) * D), 200 + rank, cfg.dtype, 0.5, device=dev)
    kv_refill = W.randn((2, (int(round(B * 0.2)) + 1) * 1024, hkv, D), 300 + rank, cfg.dtype, 0.5, device=dev)
    out = torch.empty((B, hq, D), dtype=cfg.dtype, device=dev)
    gather = torch.empty((world, B, hq, D), dtype=cfg.dtype, device=dev)
    ws = torch.zeros(128 << 20, dtype=torch.uint8, device=dev)
    rope = ops.RopeConfig()
    w = ops.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")
    launches = [0]
    peers = None
    if world > 1 and join == "peer":
        peers = parallel.PeerOutputs(B, cfg.num_qo_heads, D, cfg.dtype, dev)

    def step(i, counted=False):
        pl = plan[i]
        rf = pl["refill"]
        if rf is not None:
            seq = ops.get_seq_lens(rf["indptr"], rf["last"], 16)
            bi, kp = ops.get_batch_indices_positions(rf["qo"], seq, rf["n"])
            ops.rope_append_paged_kv_cache(None, kv_refill[0, : rf["n"]], kv_refill[1, : rf["n"]], rf["pos"], bi, kp,
                                           pool, rf["indices"], rf["indptr"], rf["last"], rope)
            launches[0] += 3
        x = qkv[i % 4]
        q = x[:, : hq * D].view(B, hq, D)
        k = x[:, hq * D: (hq + hkv) * D].view(B, hkv, D)
        v = x[:, (hq + hkv) * D:].view(B, hkv, D)
        w.plan(pl["indptr"], pl["indices"], pl["last"], hq, hkv, D, 16, q_data_type=cfg.dtype)
        if peers is not None:
            launches[0] += 2  # the fused step and the flag wait
            return w.run_fused_peer(q, k, v, pl["pos"], pool, peers, rope, counted=counted)
        o = w.run_fused(q, k, v, pl["pos"], pool, rope, out=out)
        launches[0] += 1
        return parallel.allgather_heads(o, gather_buffer=gather) if world > 1 else o

    def barrier():
        # device idle first: the barrier's own NCCL kernel would otherwise run (and spin) beside the
        # timed kernels and take an SM away from a grid that fills all of them
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    g = None
    launch_mode = "eager, one fused kernel per step"
    # The pool, the inputs and the zeroed workspace were made on the default stream, and `side` is not ordered
    # behind it: without this, a first step on `side` can read a workspace that is not zero yet (recycled
    # allocator memory holds whatever the previous leg left there).
    torch.cuda.synchronize(dev)
    side = torch.cuda.Stream(device=dev)
    use_graph = graph and (peers is not None or world == 1)  # the NCCL join stays eager
    if use_graph:
        # all timed steps (and their refills) in ONE graph: the device paces itself, no host jitter between
        # steps.  With the peer-store join the step number lives in device memory (counted mode).
        with torch.cuda.stream(side):
            for i in range(warmup):
                step(i, counted=True)
        side.synchronize()
        barrier()
        launches[0] = 0
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=side):
            for i in range(steps):
                step(warmup + i, counted=True)
        with torch.cuda.stream(side):
            g.replay()  # one untimed replay: graph upload
        if peers is not None:
            peers.advance(steps)
        side.synchronize()
        launch_mode = "CUDA graph of all timed steps"
    else:
        for i in range(warmup):
            step(i)
    barrier()
    if g is None:
        launches[0] = 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(dev.index or 0)
    with sampler:
        barrier()
        if g is not None:
            with torch.cuda.stream(side):
                e0.record(side)
                g.replay()
                e1.record(side)
            if peers is not None:
                peers.advance(steps)
        else:
            e0.record()
            for i in range(steps):
                step(warmup + i)
            e1.record()
        barrier()
    ms = e0.elapsed_time(e1)
    if world > 1:
        tt = torch.tensor([ms], dtype=torch.float64, device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms = float(tt.item())
    # attention kernel alone on a mid-run table (per-GPU bytes)
    mid = plan[warmup + steps // 2]
    x = qkv[0]
    q = x[:, : hq * D].view(B, hq, D)
    w.plan(mid["indptr"], mid["indices"], mid["last"], hq, hkv, D, 16, q_data_type=cfg.dtype)
    for _ in range(3):
        w.run(q, pool, out=out)
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0.record()
    for _ in range(20):
        w.run(q, pool, out=out)
    k1.record()
    torch.cuda.synchronize(dev)
    kern_ms = k0.elapsed_time(k1) / 20
    tokens = int(mid["meta"].seq_lens.astype(np.int64).sum())
    kern_bytes = tokens * 2 * hkv * D * 2 + B * 2 * hq * D * 2 + 4 * (len(mid["meta"].kv_indices) + 2 * B + 1)
    errw = ops.device_error(dev)
    if peers is not None:
        peers.close()
    del pool, qkv, kv_refill, ws, w
    torch.cuda.empty_cache()
    return dict(B=B, hq=hq, hkv=hkv, num_pages=num_pages, ms=ms, steps=steps, warmup=warmup, kern_ms=kern_ms,
                kern_bytes=kern_bytes, tokens=tokens, launches=launches[0], launch_mode=launch_mode,
                clocks=sampler.summary(), err=errw, peer=peers is not None)


def measure_head_sharded(world, rank, dev, steps=48, warmup=4):
    """The `head_sharded` sub-record of the headline line: the 70B-shaped decode step with the KV heads split
    over all `world` ranks, joined by the decode kernel's own peer stores and, for comparison, by an NCCL
    all-gather; plus the same step unsharded on rank 0's GPU alone, which is what strong scaling is quoted
    against.  At world == 1 it is the unsharded step."""
    import torch.distributed as dist

    peak, peak_kind = load_peaks()

    def roof(r):
        ach = r["kern_bytes"] / (r["kern_ms"] * 1e-3) / 1e9
        return {"bound": "hbm", "kernel": f"decode_tma_kernel<bf16, {r['hkv']} kv heads> (attention only, per GPU)",
                "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak, "peak_source": peak_kind,
                "bytes_per_launch": r["kern_bytes"], "us_per_launch": r["kern_ms"] * 1e3}

    rec = {"workload": "llama3-70b-shaped decode layer with eviction: 64q/8kv heads, D128, bf16, page16, 256 requests, "
                       "lognormal ctx (median 2048), 20% evicted + refilled every 32 steps", "steps": steps,
           "warmup": warmup, "scaling": "strong"}
    if world == 1:
        r = decode70b_leg(1, 0, dev, steps, warmup)
        rec.update({"n_gpus": 1, "join": "none (all heads on one GPU)", "tokens_per_s": r["B"] * steps / (r["ms"] * 1e-3),
                    "ms_per_step": r["ms"] / steps, "per_gpu_kernel_us": r["kern_ms"] * 1e3, "roofline": roof(r),
                    "strong_scaling_vs_1gpu": 1.0, "launch": r["launch_mode"], "device_error_word": r["err"]})
        return rec
    peer = decode70b_leg(world, rank, dev, steps, warmup, join="peer")
    peer_graph = decode70b_leg(world, rank, dev, steps, warmup, join="peer", graph=True)
    nccl = decode70b_leg(world, rank, dev, steps, warmup, join="nccl")
    # the unsharded step on rank 0 alone (the other ranks wait at the barrier with an idle GPU)
    one = None
    if rank == 0:
        one = decode70b_leg(1, 0, dev, steps, warmup)
    torch.cuda.synchronize(dev)
    dist.barrier()
    if rank != 0:
        return None
    best = min(peer["ms"], peer_graph["ms"])
    tps = peer["B"] * steps / (best * 1e-3)
    tps1 = one["B"] * steps / (one["ms"] * 1e-3)
    rec.update({"n_gpus": world, "join": "peer (decode kernel stores its heads to every GPU over NVLink, flag + bounded wait)",
                "tokens_per_s": tps, "ms_per_step": best / steps,
                "eager_ms_per_step": peer["ms"] / steps, "graph_ms_per_step": peer_graph["ms"] / steps,
                "nccl_ms_per_step": nccl["ms"] / steps, "peer_vs_nccl": nccl["ms"] / best,
                "per_gpu_kernel_us": peer["kern_ms"] * 1e3, "roofline": roof(peer),
                "one_gpu_tokens_per_s": tps1, "one_gpu_ms_per_step": one["ms"] / steps,
                "strong_scaling_vs_1gpu": tps / tps1, "strong_scaling_efficiency": tps / tps1 / world,
                "kv_heads_per_gpu": peer["hkv"], "clocks": peer["clocks"],
                "device_error_word": peer["err"] or nccl["err"] or one["err"]})
    return rec


def run_decode70b(args):
    """`--workload decode70b`: one leg of the head-sharded workload as a line of its own (`--join peer|nccl`,
    `--graph`)."""
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        # a collective that a failed rank never joins gives up after five minutes, not the default ten
        dist.init_process_group("nccl", device_id=torch.device("cuda", local), timeout=datetime.timedelta(seconds=300))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    B = args.requests if args.requests != 64 else 256
    if args.shard_of > 1 and world > 1:
        raise SystemExit("--shard-of emulates one rank's shape on ONE GPU")
    r = decode70b_leg(world, rank, dev, args.steps, args.warmup, join=args.join, graph=args.graph, batch=B,
                      num_pages=args.pages if args.pages != 32768 else None, shard_of=args.shard_of)
    peak, peak_kind = load_peaks()
    achieved = r["kern_bytes"] / (r["kern_ms"] * 1e-3) / 1e9
    if rank == 0:
        print(json.dumps({
            "metric": METRIC, "value": B * r["steps"] / (r["ms"] * 1e-3), "unit": UNIT, "n_gpus": world,
            "steps": r["steps"], "warmup": r["warmup"], "ms_per_step": r["ms"] / r["steps"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "llama3-70b-shaped decode layer with eviction: 64q/8kv heads, D128, bf16, page16, "
                                   f"{B} requests, lognormal ctx, 20% evicted+refilled every 32 steps",
                       "parallelism": (f"the shape one of {args.shard_of} ranks holds, alone on one GPU, no join; "
                                       if args.shard_of > 1 else "") +
                                      f"KV heads sharded x{world * args.shard_of} ({r['hkv']} kv / {r['hq']} q heads per GPU), " + (
                           "outputs stored to every GPU by the decode kernel (NVLink peer stores + flags)"
                           if r["peer"] else ("no join" if world == 1 else "NCCL all-gather of attention outputs")),
                       "pool_pages": r["num_pages"],
                       "l2": "inputs larger than L2; no flush", "launch": r["launch_mode"]},
            "clocks": r["clocks"], "gpu_launches": r["launches"],
            "roofline": {"bound": "hbm", "kernel": "decode_tma_kernel (attention only, per GPU)", "achieved": achieved,
                         "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_source": peak_kind,
                         "traffic": None, "bytes_per_launch": r["kern_bytes"], "us_per_launch": r["kern_ms"] * 1e3,
                         "cached_tokens": r["tokens"]},
            "device_error_word": r["err"]}), flush=True)
    if world > 1:
        dist.destroy_process_group()


# ---------------------------------------------------------------------------------------------
# secondary workload: beam search with shared prefix pages and copy-on-write of the partial page
# ---------------------------------------------------------------------------------------------
def beam_leg():
    """16 prefixes of 1024 tokens, each forked into 4 beams that share the prefix pages; 64 decode steps;
    every 8 steps the 2 best beams of a group (seeded random score) survive and fork again: full pages are
    shared by reference count, a partially filled last page is copied (copy_pages_kernel), losers' private
    pages return to the free list.

    Timed path: page tables, reference counts and the free list live on the device
    (pie_b200.pages.DevicePageTable); a step is [page-table advance, CSR gather, fused RoPE + append +
    attention] and a fork step adds [release, fork, page copy].  The whole 64-step run, from an empty page
    table, is ONE CUDA graph; nothing is uploaded while it runs.  Beside it: the same run with the page
    bookkeeping in Python and the tables uploaded every step (what a host-side page manager costs)."""
    from pie_b200 import ops, pages
    from pie_b200 import workloads as W

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    cfg = W.CONFIG2
    HQ, HKV, D = cfg.num_qo_heads, cfg.num_kv_heads, cfg.head_dim
    groups, beams, prefix, steps, every = 16, 4, 1024, 64, 8
    num_pages = 8192
    B = groups * beams
    pool = W.randn((num_pages, 2, 16, HKV, D), 400, cfg.dtype, 0.5, device=dev)
    qkv = W.randn((4, B, (HQ + 2 * HKV) * D), 401, cfg.dtype, 0.5, device=dev)
    out = torch.empty((B, HQ, D), dtype=cfg.dtype, device=dev)
    ws = torch.zeros(64 << 20, dtype=torch.uint8, device=dev)
    rope = ops.RopeConfig()
    rng = np.random.default_rng(4)
    plan = {}
    for i in range(steps):
        if i % every == every - 1:
            losers, parents, children = [], [], []
            for g in range(groups):
                order = rng.permutation(beams)
                keep = [g * beams + int(j) for j in order[:2]]
                lose = [g * beams + int(j) for j in order[2:]]
                losers += lose
                parents += keep
                children += lose
            plan[i] = (losers, parents, children)

    def split(x):
        return (x[:, : HQ * D].view(B, HQ, D), x[:, HQ * D: (HQ + HKV) * D].view(B, HKV, D),
                x[:, (HQ + HKV) * D:].view(B, HKV, D))

    def i32(x):
        return torch.tensor(list(x), dtype=torch.int32, device=dev)

    # ---- host-side bookkeeping, tables uploaded every step ------------------------------------------
    w = ops.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")
    host = torch.empty(4 * B + 2 + num_pages, dtype=torch.int32).pin_memory()
    devbuf = torch.empty_like(host, device=dev)
    cp_host = torch.empty(3 * B, dtype=torch.int32).pin_memory()
    cp_dev = torch.empty_like(cp_host, device=dev)
    stats = dict(copies=0, copy_bytes=0, freed=0, unique_tokens=0, logical_tokens=0)

    def host_run(count):
        pp = pages.PagePool(num_pages)
        ctxs = {}
        for g in range(groups):
            root = pages.KvPageList(pp, 16)
            root.grow(prefix)
            ctxs[g * beams] = root
            for j in range(1, beams):
                ctxs[g * beams + j], _ = root.fork_cow()  # 1024 tokens = 64 full pages: shared, nothing to copy
        mid_meta = None
        for i in range(steps):
            flat = [ctxs[s_] for s_ in range(B)]
            pos = np.fromiter((c.total_tokens for c in flat), dtype=np.int32, count=B)
            for c in flat:
                c.grow(1)
            idx, ptr, last = pages.build_csr(flat)
            n = len(idx)
            hv = host.numpy()
            hv[: B + 1] = ptr
            hv[B + 1: 2 * B + 1] = last
            hv[2 * B + 1: 3 * B + 1] = pos
            hv[4 * B + 2: 4 * B + 2 + n] = idx
            devbuf[: 4 * B + 2 + n].copy_(host[: 4 * B + 2 + n], non_blocking=True)
            mv = views(devbuf, B)
            q, k, v = split(qkv[i % 4])
            w.plan(mv["indptr"], mv["indices"][:n], mv["last"], HQ, HKV, D, 16, q_data_type=cfg.dtype)
            w.run_fused(q, k, v, mv["pos"], pool, rope, out=out)
            if i == steps // 2:
                mid_meta = (ptr.copy(), idx.copy(), last.copy())
            if count:
                stats["logical_tokens"] += int(pos.sum()) + B
                stats["unique_tokens"] += 16 * len(set(idx.tolist()))
            if i in plan:
                losers, parents, children = plan[i]
                for s_ in losers:
                    f = ctxs[s_].release()
                    if count:
                        stats["freed"] += len(f)
                cps = []
                for p_, c_ in zip(parents, children):
                    ctxs[c_], cp = ctxs[p_].fork_cow()
                    if cp is not None:
                        cps.append(cp)
                if cps:
                    m = len(cps)
                    arr = np.array(cps, dtype=np.int32).T.reshape(-1)  # src..., dst..., valid...
                    cp_host[: 3 * m].copy_(torch.from_numpy(arr))
                    cp_dev[: 3 * m].copy_(cp_host[: 3 * m], non_blocking=True)
                    ops.copy_kv_pages(pool, cp_dev[:m], cp_dev[m: 2 * m], cp_dev[2 * m: 3 * m])
                    if count:
                        stats["copies"] += m
                        stats["copy_bytes"] += int(sum(2 * c[2] * 2 * HKV * D * 2 for c in cps))
        return mid_meta

    host_run(False)
    torch.cuda.synchronize(dev)
    h0, h1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0 = time.perf_counter()
    h0.record()
    mid_meta = host_run(True)
    h1.record()
    torch.cuda.synchronize(dev)
    host_wall_ms = (time.perf_counter() - t0) * 1e3
    host_ms = h0.elapsed_time(h1)

    # ---- device-resident page tables: the whole run as one CUDA graph --------------------------------
    dpt = pages.DevicePageTable(num_pages, B, 128, max_batch=B)
    roots = i32(g * beams for g in range(groups))
    kid_parents = i32(g * beams for g in range(groups) for _ in range(beams - 1))
    kids = i32(g * beams + j for g in range(groups) for j in range(1, beams))
    all_slots = i32(range(B))
    dplan = {i: tuple(i32(x) for x in v) for i, v in plan.items()}
    wd = ops.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD", use_cuda_graph=True,
                                                paged_kv_indptr_buffer=dpt.kv_indptr[: B + 1],
                                                paged_kv_indices_buffer=dpt.kv_indices,
                                                paged_kv_last_page_len_buffer=dpt.kv_last_page_len[:B])
    launches = [0]

    def device_run():
        from pie_b200._lib import lib, check
        check(lib.piekv_pagestate_init(dpt.state.data_ptr(), dpt.state.numel() * 4, num_pages, B, 128, 16,
                                       torch.cuda.current_stream(dev).cuda_stream), "pagestate_init")
        dpt.grow(roots, prefix, csr=False)
        dpt.fork(kid_parents, kids)
        launches[0] += 3
        for i in range(steps):
            indptr, indices, last, pos = dpt.grow(all_slots, 1)
            q, k, v = split(qkv[i % 4])
            wd.plan(indptr, indices, last, HQ, HKV, D, 16, q_data_type=cfg.dtype)
            wd.run_fused(q, k, v, pos, pool, rope, out=out)
            launches[0] += 3
            if i in dplan:
                losers, parents, children = dplan[i]
                dpt.release(losers)
                src, dst, val = dpt.fork(parents, children)
                ops.copy_kv_pages(pool, src, dst, val)
                launches[0] += 3

    torch.cuda.synchronize(dev)  # tables and buffers above were made on the default stream
    side = torch.cuda.Stream(device=dev)
    with torch.cuda.stream(side):
        device_run()  # eager once: warm-up
    side.synchronize()
    launches[0] = 0
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        device_run()
    with torch.cuda.stream(side):
        graph.replay()
    side.synchronize()
    reps = 5
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(side):
        e0.record(side)
        for _ in range(reps):
            graph.replay()
        e1.record(side)
    side.synchronize()
    ms = e0.elapsed_time(e1) / reps
    # the fused attention launch alone, on the mid-run table, for scale
    ptr, idx, last = mid_meta
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    w.plan(t(ptr), t(idx), t(last), HQ, HKV, D, 16, q_data_type=cfg.dtype)
    q, k, v = split(qkv[0])
    posm = torch.zeros(B, dtype=torch.int32, device=dev)
    for _ in range(3):
        w.run_fused(q, k, v, posm, pool, rope, out=out)
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0.record()
    for _ in range(50):
        w.run_fused(q, k, v, posm, pool, rope, out=out)
    k1.record()
    torch.cuda.synchronize(dev)
    fused_us = k0.elapsed_time(k1) / 50 * 1e3
    return {
        "metric": METRIC, "value": B * steps / (ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": steps, "warmup": 1,
        "ms_per_step": ms / steps, "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "beam search page sharing: 16 prefixes x 1024 tokens x 4 beams, fork top-2 every 8 "
                               "steps, copy-on-write of the partial last page; 32q/8kv heads, D128, bf16, page16",
                   "host": "none inside the timed region: page tables, reference counts and the free list are "
                           "advanced on the device; the 64-step run (from an empty table) is one CUDA graph"},
        "gpu_launches": launches[0],
        "fused_kernel_us": fused_us, "step_over_fused_kernel": ms / steps * 1e3 / fused_us,
        "host_tables_ms_per_step": host_ms / steps, "host_tables_wall_ms_per_step": host_wall_ms / steps,
        "page_copies": stats["copies"], "page_copy_bytes": stats["copy_bytes"], "pages_recycled": stats["freed"],
        "logical_kv_bytes_per_step": stats["logical_tokens"] * 4096 // steps,
        "unique_page_kv_bytes_per_step": stats["unique_tokens"] * 4096 // steps,
        "device_error_word": ops.device_error(dev)}


def qkv_rows(dev, prefill_only=False):
    """The QKV projection of the prefill mix (config 3's 20480 tokens, hidden 4096, 32q/8kv heads) with RoPE +
    append, as the library GEMM followed by `rope_append_paged_kv_cache` and as the one fused tcgen05 kernel
    (`qkv_rope_append_paged_kv_cache`); plus (unless `prefill_only`) a decode-sized batch."""
    from pie_b200 import ops
    from pie_b200 import workloads as W

    cfg = W.CONFIG2
    HQ, HKV, D = cfg.num_qo_heads, cfg.num_kv_heads, cfg.head_dim
    hidden = 4096
    peak_tf, peak_kind = load_peaks_tensor()
    t = lambda x: torch.from_numpy(np.ascontiguousarray(x)).to(dev)
    rows = []

    def timed(fn, reps):
        for _ in range(3):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1) / reps

    w = W.randn(((HQ + 2 * HKV) * D, hidden), 601, cfg.dtype, hidden ** -0.5, device=dev)
    rope = ops.RopeConfig()
    cases = [("prefill mix, 20480 tokens", W.config3_meta(num_pages=8192), 20)]
    if not prefill_only:
        cases.append(("decode batch, 64 tokens", W.decode_steps(W.config2_requests(), 1)[0], 50))
    for label, meta, reps in cases:
        n = meta.nnz if hasattr(meta, "nnz") else meta.batch
        pool = W.randn((32768 if n == 64 else 8192, 2, 16, HKV, D), 600, cfg.dtype, 0.5, device=dev)
        x = W.randn((n, hidden), 602, cfg.dtype, 1.0, device=dev)
        qo, indptr, indices, last, pos = t(meta.qo_indptr), t(meta.kv_indptr), t(meta.kv_indices), \
            t(meta.kv_last_page_len), t(meta.pos_ids)
        seq = ops.get_seq_lens(indptr, last, 16)
        bi, kp = ops.get_batch_indices_positions(qo, seq, n)

        def separate():
            qkv = torch.nn.functional.linear(x, w)
            q = qkv[:, : HQ * D].view(n, HQ, D)
            k = qkv[:, HQ * D: (HQ + HKV) * D].view(n, HKV, D)
            v = qkv[:, (HQ + HKV) * D:].view(n, HKV, D)
            ops.rope_append_paged_kv_cache(q, k, v, pos, bi, kp, pool, indices, indptr, last, rope)

        q_out = torch.empty((n, HQ, D), dtype=cfg.dtype, device=dev)

        def fused():
            ops.qkv_rope_append_paged_kv_cache(x, w, pos, bi, kp, pool, indices, indptr, HQ, HKV, rope=rope, q_out=q_out)

        gemm_only = timed(lambda: torch.nn.functional.linear(x, w), reps)
        sep = timed(separate, reps)
        fus = timed(fused, reps)
        flops = 2.0 * n * hidden * (HQ + 2 * HKV) * D
        rows.append({"case": label, "tokens": n, "flop": flops,
                     "library_gemm_ms": gemm_only, "library_gemm_plus_rope_append_ms": sep, "fused_ms": fus,
                     "fused_tflops": flops / fus / 1e9, "library_gemm_tflops": flops / gemm_only / 1e9,
                     "fused_frac_of_peak": flops / fus / 1e9 / peak_tf, "fused_vs_separate": sep / fus,
                     "peak_source": peak_kind})
        del pool, x, q_out
    del w
    torch.cuda.empty_cache()
    return rows, peak_tf


def qkv_subrecord(dev):
    """The `qkv` sub-record of the headline line: the fused projection + RoPE + append kernel on the prefill
    mix, next to the library GEMM followed by the separate kernel."""
    from pie_b200 import ops

    rows, peak_tf = qkv_rows(dev, prefill_only=True)
    r = rows[0]
    return {"workload": "QKV projection + RoPE + append of the prefill mix: 20480 tokens, hidden 4096, 32q/8kv heads, "
                        "D128, bf16, page16",
            "kernel": "qkv_rope_append_kernel (tcgen05 GEMM, RoPE + append in the epilogue)",
            "ms_per_launch": r["fused_ms"], "library_gemm_ms": r["library_gemm_ms"],
            "library_gemm_plus_rope_append_ms": r["library_gemm_plus_rope_append_ms"],
            "roofline": {"bound": "tensor", "achieved": r["fused_tflops"], "peak": peak_tf, "unit": "TFLOP/s",
                         "frac": r["fused_frac_of_peak"], "peak_source": r["peak_source"]},
            "device_error_word": ops.device_error(dev)}


def run_qkv(args):
    """`--workload qkv`: see `qkv_rows`."""
    from pie_b200 import ops

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    rows, peak_tf = qkv_rows(dev)
    print(json.dumps({"workload": "QKV projection + RoPE + append, hidden 4096, 32q/8kv heads, D128, bf16, page16",
                      "peak_TFLOPs": peak_tf, "rows": rows, "device_error_word": ops.device_error(dev)}), flush=True)


# ---------------------------------------------------------------------------------------------
# secondary workload: output projection with the sum over the ranks in its epilogue
# ---------------------------------------------------------------------------------------------
def measure_oproj(world, rank, dev, steps=40, warmup=5, cases=None, shard_of=1):
    """The `oproj` sub-record: the row-parallel output projection of a 70B-shaped layer (hidden 8192, 64 query
    heads x 128 split over the ranks) with the all-reduce and the residual add in the kernel's epilogue
    (`piekv_oproj_allreduce`), next to what the reference does with library calls: matmul, NCCL all-reduce,
    residual add.  Eight layers' weight shards are used in turn so that a launch does not find its weights in
    L2.  Times are CUDA events around `steps` launches, max over ranks."""
    import torch.distributed as dist

    from pie_b200 import ops
    from pie_b200 import workloads as W
    from pie_b200.parallel import PeerReduce

    hidden, k_full, layers = 8192, 8192, 8
    kl = k_full // (world * shard_of)   # shard_of > 1: the shape one of that many ranks holds, no exchange
    dt = torch.bfloat16
    ws = [W.randn((hidden, kl), 900 + l, dt, 0.02, device=dev) for l in range(layers)]
    peak_tf, peak_tf_kind = load_peaks_tensor()
    peak_bw, peak_bw_kind = load_peaks()
    cases = cases or (("decode", 256), ("prefill", 8192))
    n_max = max(n for _, n in cases)
    pr = PeerReduce(n_max, hidden, dt, dev)
    pr16 = PeerReduce(n_max, hidden, dt, dev, partial_sums="storage") if world > 1 else None

    def over_ranks(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(fn):
        for i in range(warmup):
            fn(i)
        torch.cuda.synchronize(dev)
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(steps):
            fn(warmup + i)
        e1.record()
        torch.cuda.synchronize(dev)
        return over_ranks(e0.elapsed_time(e1) / steps)

    rows = []
    for name, n in cases:
        a = W.randn((n, kl), 910, dt, 0.5, device=dev)
        res = W.randn((n, hidden), 911, dt, 1.0, device=dev)

        def fused(i):
            return pr.oproj(a, ws[i % layers], res)

        def fused16(i):
            return pr16.oproj(a, ws[i % layers], res)

        def library(i):
            y = torch.matmul(a, ws[i % layers].t())
            if world > 1:
                dist.all_reduce(y)
            return res + y

        def library_matmul(i):
            return torch.matmul(a, ws[i % layers].t())

        got = fused(0).clone()
        want = library(0)
        torch.cuda.synchronize(dev)
        diff = (got.float() - want.float()).abs().max().item()
        ms_f = timed(fused)
        ms_l = timed(library)
        ms_g = timed(library_matmul)
        flops = 2.0 * n * hidden * kl
        w_bytes = hidden * kl * 2 + n * kl * 2 + 2 * n * hidden * 2
        row = {"case": name, "rows": n, "k_local": kl, "fused_ms": ms_f, "library_ms": ms_l,
               "library_matmul_alone_ms": ms_g, "fused_vs_library": ms_l / ms_f,
               "fused_tflops_per_gpu": flops / ms_f / 1e9, "max_abs_diff_to_library": diff}
        if n <= 1024:
            ach = w_bytes / (ms_f * 1e-3) / 1e9
            row["roofline"] = {"bound": "hbm", "achieved": ach, "peak": peak_bw, "unit": "GB/s", "frac": ach / peak_bw,
                               "peak_source": peak_bw_kind, "bytes_per_launch": w_bytes,
                               "note": "weight shard + rows in + residual in + rows out; the exchange is not counted"}
        else:
            ach = flops / ms_f / 1e9
            row["roofline"] = {"bound": "tensor", "achieved": ach, "peak": peak_tf, "unit": "TFLOP/s",
                               "frac": ach / peak_tf, "peak_source": peak_tf_kind}
        if world > 1:
            # fp32 partial sums to the owners + rounded rows to every rank, per rank and launch
            row["nvlink_bytes_out_per_gpu"] = int(n * hidden * 4 * (world - 1) / world + n * hidden * 2 * (world - 1) / world)
            # the same kernel with the partial sums rounded to bf16 on their way (an all-reduce's bytes)
            got16 = fused16(0).clone()
            torch.cuda.synchronize(dev)
            row["partials_16bit_max_abs_diff_to_library"] = (got16.float() - want.float()).abs().max().item()
            row["partials_16bit_fused_ms"] = timed(fused16)
            row["partials_16bit_fused_vs_library"] = ms_l / row["partials_16bit_fused_ms"]
        rows.append(row)
    err = ops.device_error(dev)
    pr.close()
    if pr16 is not None:
        pr16.close()
    if rank != 0:
        return None
    return {"workload": f"o_proj of a llama3-70b-shaped layer: hidden {hidden}, {k_full // 128} query heads x 128 over "
                        f"{world} rank(s), bf16; residual added; 8 layers' weights in turn",
            "kernel": "oproj_reduce_kernel (tcgen05 GEMM; fp32 partial sums over NVLink peer stores, summed in rank "
                      "order by the tile's owner, one rounding, rows stored to every rank)",
            "library": "torch.matmul + NCCL all_reduce + residual add" if world > 1 else "torch.matmul + residual add",
            "n_gpus": world, "steps": steps, "warmup": warmup, "rows": rows, "device_error_word": err}


def run_oproj(args):
    """`--workload oproj`: see `measure_oproj`; one rank per GPU under torchrun."""
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=300))
    rec = measure_oproj(world, rank, dev, steps=args.steps, warmup=args.warmup, shard_of=args.shard_of)
    if rank == 0:
        print(json.dumps(rec), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_copy(args):
    """`--workload copy`: the page-copy kernel (copy-on-write of forked pages) and the RoPE + append kernel
    alone, with CUDA events: achieved bytes/s (read + written) against the measured HBM copy bandwidth."""
    from pie_b200 import ops
    from pie_b200 import workloads as W

    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    cfg = W.CONFIG2
    HQ, HKV, D = cfg.num_qo_heads, cfg.num_kv_heads, cfg.head_dim
    num_pages = 16384
    peak, peak_kind = load_peaks()
    pool = W.randn((num_pages, 2, 16, HKV, D), 500, cfg.dtype, 0.5, device=dev)
    rows = []

    def timed(fn, reps=50):
        for _ in range(5):
            fn()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize(dev)
        return e0.elapsed_time(e1) / reps * 1e3

    perm = torch.randperm(num_pages, generator=torch.Generator().manual_seed(9)).to(torch.int32)
    for pairs, valid in ((32, 8), (32, 16), (512, 16), (4096, 16)):
        src = perm[:pairs].to(dev)
        dst = perm[num_pages // 2: num_pages // 2 + pairs].to(dev)
        val = torch.full((pairs,), valid, dtype=torch.int32, device=dev)
        us = timed(lambda: ops.copy_kv_pages(pool, src, dst, val))
        nbytes = 2 * pairs * 2 * valid * HKV * D * 2
        rows.append({"kernel": "copy_pages_kernel", "pairs": pairs, "valid_tokens": valid, "bytes": nbytes,
                     "us": us, "GBps": nbytes / us / 1e3, "frac_of_peak": nbytes / us / 1e3 / peak})
    # RoPE + append of a prefill-sized batch (config 3: 20480 tokens)
    meta = W.config3_meta(num_pages=8192)
    n = meta.nnz
    t = lambda x: torch.from_numpy(np.ascontiguousarray(x)).to(dev)
    qkv = W.randn((n, (HQ + 2 * HKV) * D), 501, cfg.dtype, 0.5, device=dev)
    q = qkv[:, : HQ * D].view(n, HQ, D)
    k = qkv[:, HQ * D: (HQ + HKV) * D].view(n, HKV, D)
    v = qkv[:, (HQ + HKV) * D:].view(n, HKV, D)
    qo, indptr, indices, last, pos = t(meta.qo_indptr), t(meta.kv_indptr), t(meta.kv_indices), \
        t(meta.kv_last_page_len), t(meta.pos_ids)
    seq = ops.get_seq_lens(indptr, last, 16)
    bi, kp = ops.get_batch_indices_positions(qo, seq, n)
    rope = ops.RopeConfig()
    us = timed(lambda: ops.rope_append_paged_kv_cache(q, k, v, pos, bi, kp, pool[:8192], indices, indptr, last, rope), 30)
    nbytes = n * ((HQ + 2 * HKV) * D * 2 + HQ * D * 2 + 2 * HKV * D * 2)
    rows.append({"kernel": "rope_append_tokens_kernel", "tokens": n, "bytes": nbytes, "us": us,
                 "GBps": nbytes / us / 1e3, "frac_of_peak": nbytes / us / 1e3 / peak})
    us = timed(lambda: ops.append_paged_kv_cache(k, v, bi, kp, pool[:8192], indices, indptr, last), 30)
    nbytes = n * (2 * 2 * HKV * D * 2)
    rows.append({"kernel": "append_tokens_warp_kernel (append only)", "tokens": n, "bytes": nbytes, "us": us,
                 "GBps": nbytes / us / 1e3, "frac_of_peak": nbytes / us / 1e3 / peak})
    print(json.dumps({"workload": "page copy and RoPE + append kernels alone, 32q/8kv heads, D128, bf16, page16",
                      "peak_GBps": peak, "peak_source": peak_kind, "rows": rows,
                      "device_error_word": ops.device_error(dev)}), flush=True)


def run_beam(args):
    print(json.dumps(beam_leg()), flush=True)


def beam_subrecord(dev):
    """The `beam` sub-record of the headline line (beam search with shared prefix pages)."""
    line = beam_leg()
    keep = ("ms_per_step", "fused_kernel_us", "step_over_fused_kernel", "host_tables_ms_per_step",
            "host_tables_wall_ms_per_step", "gpu_launches", "page_copies", "page_copy_bytes", "pages_recycled",
            "logical_kv_bytes_per_step", "unique_page_kv_bytes_per_step", "device_error_word")
    rec = {"workload": line["config"]["workload"], "tokens_per_s": line["value"], "steps": line["steps"]}
    rec.update({k: line[k] for k in keep})
    rec["host"] = line["config"]["host"]
    return rec


# ---------------------------------------------------------------------------------------------
# CPU arms
# ---------------------------------------------------------------------------------------------
def load_workloads_standalone():
    """pie_b200/workloads.py loaded by file path: it needs only numpy and torch, and importing it through the
    package would map libpiekv.so into a process whose job is to time the CPU path."""
    import importlib.util

    name = "_piekv_workloads_standalone"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "pie_b200", "workloads.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


class CpuPath:
    """The reference path on host cores: the CPU oracle in the reference's op order
    (RoPE -> append -> decode attention, pie/src/pie_worker/model/llama3.py:654-689)."""

    def __init__(self, num_pages: int = 32768, seed: int = 1):
        from oracle import paged_kv_ref as R

        W = load_workloads_standalone()
        self.R, self.W = R, W
        self.cfg = W.CONFIG2
        torch.set_num_threads(os.cpu_count() or 1)
        self.cores = torch.get_num_threads()
        reqs = W.config2_requests(seed=seed, num_pages=num_pages)
        self.metas = W.decode_steps(reqs, 64)
        cfg = self.cfg
        g = torch.Generator().manual_seed(7)
        self.pool = torch.empty(cfg.pool_shape(), dtype=cfg.dtype)
        # filling 2 GiB with Gaussian noise on the CPU takes a while; uniform noise of the same scale is
        # enough for timing (values do not change the work)
        self.pool.view(torch.int16).random_(0x3C00, 0x3F80, generator=g)  # bf16 bit patterns in [2^-7, 1)
        self.q = W.randn((64, cfg.num_qo_heads, cfg.head_dim), 1, cfg.dtype, 0.5)
        self.k = W.randn((64, cfg.num_kv_heads, cfg.head_dim), 2, cfg.dtype, 0.5)
        self.v = W.randn((64, cfg.num_kv_heads, cfg.head_dim), 3, cfg.dtype, 0.5)
        self.inv = R.rope_inv_freq(cfg.head_dim, cfg.rope_theta, "llama31", cfg.rope_scale)

    def step(self, i: int, nreq: int = 64) -> int:
        """One decode step over the first `nreq` requests; returns tokens processed."""
        R = self.R
        m = self.metas[i % len(self.metas)]
        c, s = R.rope_cos_sin(m.pos_ids[:nreq], self.inv)
        q = R.apply_rope(self.q[:nreq], c, s)
        k = R.apply_rope(self.k[:nreq], c, s)
        ptr = m.kv_indptr[: nreq + 1]
        seq = R.get_seq_lens(ptr, m.kv_last_page_len[:nreq], 16)
        bi, pos = R.get_batch_indices_positions(m.qo_indptr[: nreq + 1], seq, nreq)
        R.append_paged_kv_cache(k, self.v[:nreq], bi, pos, self.pool, m.kv_indices, ptr)
        R.decode_attention(q, self.pool, ptr, m.kv_indices, m.kv_last_page_len[:nreq])
        return nreq


def cpu_baseline(sample_steps: int = 0, sample_s: float = 20.0):
    path = CpuPath()
    path.step(0)
    t0 = time.perf_counter()
    path.step(1)
    one = time.perf_counter() - t0
    n = sample_steps or max(1, min(64, int(sample_s / max(one, 1e-3))))
    t0 = time.perf_counter()
    tokens = 0
    for i in range(n):
        tokens += path.step(2 + i)
    dt = time.perf_counter() - t0
    return {"value": tokens / dt, "unit": UNIT, "cores": path.cores, "kind": "port",
            "sample": f"{n} full decode steps of the workload (64 requests each) on the CPU oracle, "
                      f"torch CPU with {path.cores} threads; {dt:.1f} s"}


def run_reference(args):
    """`--impl reference`: the reference's path on the host cores.  The reference has no CPU (or in-repo
    CUDA) implementation of this path, so the timed code is the CPU restatement under oracle/ ("port")."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank != 0:
        return
    path = CpuPath()
    steps, warmup = args.steps, args.warmup
    path.step(0)
    t0 = time.perf_counter()
    path.step(1)
    one = time.perf_counter() - t0
    # bound the whole run to about two minutes: each step processes a sample of the 64 requests
    limit_s = 120.0
    nreq = 64
    if one * (steps + warmup) > limit_s:
        nreq = max(1, min(64, int(64 * limit_s / (one * (steps + warmup)))))
    for i in range(min(warmup, 3)):
        path.step(i, nreq)
    t0 = time.perf_counter()
    tokens = 0
    for i in range(steps):
        tokens += path.step(warmup + i, nreq)
    dt = time.perf_counter() - t0
    value = tokens / dt
    sample = (f"each step = the first {nreq} of 64 requests of the workload's decode step "
              f"(RoPE + append + paged decode attention) on the CPU oracle, {path.cores} torch threads")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": steps,
        "warmup": warmup, "ms_per_step": dt / steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": headline_config(path.W, 64, world, 32768, steps, warmup),
        "sample": sample,
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": path.cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_flashinfer(args):
    """Black-box comparator: the reference's CUDA dependency (FlashInfer, whatever version the box has)
    driven through the call sequence of pie/src/pie_worker/model/llama3.py:660-689,745-791 on the headline
    workload.  Never read, linked or copied - only called and timed."""
    import flashinfer

    from pie_b200 import workloads as W

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = W.CONFIG2
    B, HQ, HKV, D = 64, cfg.num_qo_heads, cfg.num_kv_heads, cfg.head_dim
    steps, warmup = args.steps, args.warmup
    horizon = min(HORIZON, steps + warmup)
    metas = build_steps(0, horizon)

    def t(x):
        return torch.from_numpy(np.ascontiguousarray(x)).to(dev)

    tabs = [dict(indptr=t(m.kv_indptr), indices=t(m.kv_indices), last=t(m.kv_last_page_len), pos=t(m.pos_ids),
                 qo=t(m.qo_indptr)) for m in metas]
    pool = W.randn(cfg.pool_shape(), 100, cfg.dtype, cfg.value_scale, device=dev)
    qkv = W.randn((8, B, (HQ + 2 * HKV) * D), 200, cfg.dtype, cfg.value_scale, device=dev)
    ws = torch.zeros(128 << 20, dtype=torch.uint8, device=dev)
    w = flashinfer.BatchDecodeWithPagedKVCacheWrapper(ws, "NHD")

    def step(i, plan=True):
        tb = tabs[i % horizon]
        x = qkv[i % 8]
        q = x[:, : HQ * D].view(B, HQ, D)
        k = x[:, HQ * D: (HQ + HKV) * D].view(B, HKV, D)
        v = x[:, (HQ + HKV) * D:].view(B, HKV, D)
        seq = flashinfer.get_seq_lens(tb["indptr"], tb["last"], 16)
        bi, kp = flashinfer.get_batch_indices_positions(tb["qo"], seq, B)
        if plan:
            w.plan(indptr=tb["indptr"], indices=tb["indices"], last_page_len=tb["last"], num_qo_heads=HQ,
                   num_kv_heads=HKV, head_dim=D, page_size=16, pos_encoding_mode="NONE", q_data_type=cfg.dtype)
        flashinfer.apply_llama31_rope_pos_ids_inplace(q=q, k=k, pos_ids=tb["pos"], rope_scale=8.0, rope_theta=5e5,
                                                      low_freq_factor=1.0, high_freq_factor=4.0, old_context_len=8192)
        flashinfer.append_paged_kv_cache(append_key=k, append_value=v, batch_indices=bi, positions=kp,
                                         paged_kv_cache=pool, kv_indices=tb["indices"], kv_indptr=tb["indptr"],
                                         kv_last_page_len=tb["last"], kv_layout="NHD")
        return w.run(q, pool)

    for i in range(warmup):
        step(i)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps):
        step(warmup + i)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1)
    # attention kernel alone on one table
    mid = (warmup + steps // 2) % horizon
    tb = tabs[mid]
    w.plan(indptr=tb["indptr"], indices=tb["indices"], last_page_len=tb["last"], num_qo_heads=HQ, num_kv_heads=HKV,
           head_dim=D, page_size=16, pos_encoding_mode="NONE", q_data_type=cfg.dtype)
    q = qkv[0][:, : HQ * D].view(B, HQ, D)
    for _ in range(5):
        w.run(q, pool)
    k0, k1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    k0.record()
    for _ in range(100):
        w.run(q, pool)
    k1.record()
    torch.cuda.synchronize()
    kern_ms = k0.elapsed_time(k1) / 100
    m = metas[mid]
    tokens = int(m.seq_lens.astype(np.int64).sum())
    kern_bytes = tokens * 2 * HKV * D * 2 + B * 2 * HQ * D * 2 + 4 * (len(m.kv_indices) + 2 * B + 1)
    peak, peak_kind = load_peaks()
    print(json.dumps({
        "impl": "flashinfer", "version": flashinfer.__version__, "metric": METRIC, "value": B * steps / (ms * 1e-3),
        "unit": UNIT, "n_gpus": 1, "steps": steps, "warmup": warmup, "ms_per_step": ms / steps,
        "higher_is_better": True, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": WORKLOAD, "launch": "eager: get_seq_lens, get_batch_indices_positions, plan, rope, "
                                                   "append, run per step (the reference's per-step sequence)"},
        "roofline": {"bound": "hbm", "kernel": "BatchDecodeWithPagedKVCacheWrapper.run", "achieved":
                     kern_bytes / (kern_ms * 1e-3) / 1e9, "peak": peak, "unit": "GB/s",
                     "frac": kern_bytes / (kern_ms * 1e-3) / 1e9 / peak, "peak_source": peak_kind,
                     "us_per_launch": kern_ms * 1e3, "bytes_per_launch": kern_bytes}}), flush=True)


def run_flashinfer_prefill(args):
    """Black-box comparator for the chunked-prefill mix: FlashInfer's BatchPrefillWithPagedKVCacheWrapper with its
    native causal flag on the same metadata and tensor shapes (called and timed only)."""
    import flashinfer

    from pie_b200 import workloads as W

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    cfg = W.CONFIG3
    HQ, HKV, D = cfg.num_qo_heads, cfg.num_kv_heads, cfg.head_dim
    num_pages = 8192
    meta = W.config3_meta(num_pages=num_pages)
    n = meta.nnz

    def t(x):
        return torch.from_numpy(np.ascontiguousarray(x)).to(dev)

    pool = W.randn((num_pages, 2, 16, HKV, D), 300, cfg.dtype, 0.5, device=dev)
    q = W.randn((n, HQ, D), 301, cfg.dtype, 0.5, device=dev)
    ws = torch.zeros(256 << 20, dtype=torch.uint8, device=dev)
    w = flashinfer.BatchPrefillWithPagedKVCacheWrapper(ws, "NHD")
    w.plan(qo_indptr=t(meta.qo_indptr), paged_kv_indptr=t(meta.kv_indptr), paged_kv_indices=t(meta.kv_indices),
           paged_kv_last_page_len=t(meta.kv_last_page_len), num_qo_heads=HQ, num_kv_heads=HKV, head_dim_qk=D,
           page_size=16, causal=True, q_data_type=cfg.dtype)
    for _ in range(args.warmup):
        w.run(q, pool)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        w.run(q, pool)
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / args.steps
    flops = 4.0 * D * HQ * W.causal_pairs(meta)
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            peak = float(json.load(f)["bf16_tflops_sustained"])
    except Exception:
        peak = 1400.0
    tf = flops / (ms * 1e-3) / 1e12
    print(json.dumps({"impl": "flashinfer", "version": flashinfer.__version__, "metric": "prefill_tokens_per_s",
                      "value": n / (ms * 1e-3), "unit": "tokens/s", "n_gpus": 1, "steps": args.steps,
                      "warmup": args.warmup, "ms_per_step": ms, "dtype": "bf16", "data": "synthetic",
                      "config": {"workload": f"chunked prefill mix: {meta.batch} requests, {n} query tokens, native "
                                             "causal flag, attention only (no RoPE / append)"},
                      "roofline": {"bound": "tensor", "kernel": "BatchPrefillWithPagedKVCacheWrapper.run",
                                   "achieved": tf, "peak": peak, "unit": "TFLOP/s", "frac": tf / peak,
                                   "flops_causal_exact": flops, "ms_per_launch": ms}}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference", "flashinfer"])
    ap.add_argument("--cpu-steps", type=int, default=0, help="CPU-baseline sample size in steps (0 = ~20 s)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg (profiling runs)")
    ap.add_argument("--requests", type=int, default=64, help="requests per GPU (default: the workload's 64)")
    ap.add_argument("--pages", type=int, default=32768, help="pool pages (default: the workload's 32768)")
    ap.add_argument("--kernel-reps", type=int, default=100, help="launches timed for the roofline figure")
    ap.add_argument("--workload", default="decode", choices=["decode", "prefill", "decode70b", "beam", "copy", "qkv", "oproj"],
                    help="decode: the headline decode layer; prefill: the chunked-prefill mix (tensor-core bound)")
    ap.add_argument("--prefill-scale", type=float, default=1.0, help="fraction of the 8+8 requests of the prefill mix")
    ap.add_argument("--prefill-mask", action="store_true", help="prefill: pass the reference-form boolean mask")
    ap.add_argument("--graph", action="store_true",
                    help="decode70b: capture all timed steps in one CUDA graph (peer-store join or one GPU; the "
                         "NCCL join stays eager)")
    ap.add_argument("--shard-of", type=int, default=1, choices=[1, 2, 4, 8],
                    help="decode70b on one GPU: the head counts one of this many ranks would hold (profiling)")
    ap.add_argument("--join", default="peer", choices=["peer", "nccl"],
                    help="decode70b on several GPUs: how the head-sharded outputs are joined")
    ap.add_argument("--pdl", type=int, default=3, choices=[0, 1, 2, 3],
                    help="decode: programmatic dependent launch mode of the timed steps (see PIEKV_OPT_PDL)")
    ap.add_argument("--min-timed-ms", type=float, default=250.0,
                    help="decode: replay the captured graph of --steps steps until the timed region lasts this long")
    ap.add_argument("--no-sub", action="store_true",
                    help="decode: skip the secondary workloads' sub-records (head_sharded, oproj, prefill, beam, qkv)")
    ap.add_argument("--prefill-brle", action="store_true",
                    help="prefill: pass the mask as BRLE runs (wire form), expanded to bits on the device")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        run_reference(args)
    elif args.impl == "flashinfer":
        if args.workload == "prefill":
            run_flashinfer_prefill(args)
        else:
            run_flashinfer(args)
    elif args.workload == "prefill":
        run_prefill(args)
    elif args.workload == "decode70b":
        run_decode70b(args)
    elif args.workload == "beam":
        run_beam(args)
    elif args.workload == "copy":
        run_copy(args)
    elif args.workload == "qkv":
        run_qkv(args)
    elif args.workload == "oproj":
        run_oproj(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
