#!/usr/bin/env python
"""Benchmark of the fused score + top-k pass.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Default workload `c3` is the configuration the headline metric is quoted on: q8 cosine, 10,000,000 candidates x
768 (int8 codes + one f32 scale per row, 7.72 GB), one f16 query per step, k = 10.  A step is one pass of the
hot path over all candidates for one query batch.  With N GPUs the rows are sharded (strong scaling: the rows
are split), each rank scans its shard and the per-shard lists are all-gathered (NCCL) and merged on every rank.
Other workloads (`--workload`) are the remaining benchmark configurations (batched f16 dot, q8 at query batch 256,
q4 l2 nearest neighbours, embed + score), used for profiles and parity at size; they print the same JSON line.

Prints ONE JSON line.  `value` is measured with candidates and queries resident in HBM (CUDA events on the
launching stream, max over ranks); `e2e` goes through the host-buffer C-ABI call (queries copied H2D from pinned
memory and ids/scores copied D2H inside the timed region, candidates resident as bound parameters).
`--impl reference` times the CPU restatement of the reference's Go host path (the oracle) on this box's cores.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time
from dataclasses import dataclass

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_QUERY_SET = 64  # distinct resident query batches cycled through the steps (fewer for large batches)


@dataclass
class Workload:
    name: str
    layout: str
    metric: str
    rows: int
    cols: int
    nq: int
    k: int
    smallest: bool = False
    normalise: bool = True
    note: str = ""
    embed: tuple = ()  # (vocab, dim, seq): queries come from the embedding front end instead of a query set
    embed_order: int = 0  # 0: normalize(mean_pool(x @ P)); 1: mean_pool(normalize(x @ P)), every token row projected

    def row_bytes(self) -> float:
        """Algorithmic bytes per candidate row and pass: stored codes + the per-row values the metric reads."""
        if self.layout == "q8":
            return self.cols + 4 + (0 if self.metric == "cosine" else 4) - (4 if self.metric == "dot" else 0)
        if self.layout == "q4":
            return self.cols / 2 + self.cols / 16 + (0 if self.metric == "dot" else 4)
        extra = 4 if self.metric == "cosine" else 0
        return 2 * self.cols + extra

    def describe(self) -> str:
        order = "smallest" if self.smallest else "largest"
        front = (f"embed(tokens i32[{self.nq},{self.embed[2]}], table f16[{self.embed[0]},{self.embed[1]}], projection "
                 f"f16[{self.embed[1]},{self.cols}], {'normalize, masked mean_pool' if self.embed_order else 'masked mean_pool, normalize'}) -> ") if self.embed else ""
        return (f"{front}{self.layout} {self.metric} {self.rows / 1e6:g}M x {self.cols}, {self.nq} "
                f"quer{'y' if self.nq == 1 else 'ies'} per pass, k={self.k} {order}")


WORKLOADS = {
    "c1": Workload("c1", "q8", "cosine", 10_000, 128, 1, 10, note="CPU-runnable select configuration"),
    "c2": Workload("c2", "f16", "dot", 1_000_000, 384, 64, 100, note="batched f16 dot"),
    "c3": Workload("c3", "q8", "cosine", 10_000_000, 768, 1, 10, note="headline: single-query q8 cosine at scale"),
    "c3q256": Workload("c3q256", "q8", "cosine", 10_000_000, 768, 256, 10, note="q8 cosine at scale, query batch 256"),
    "c4": Workload("c4", "q4", "l2_distance", 12_500_000, 256, 1, 1000, smallest=True, normalise=False,
                   note="one GPU's share (1/8) of the 100M x 256 q4 set"),
    "c4x8": Workload("c4x8", "q4", "l2_distance", 100_000_000, 256, 1, 1000, smallest=True, normalise=False,
                     note="the whole 100M x 256 q4 set (14.4 GB), meant to be sharded over 8 GPUs"),
    "c4x8q32": Workload("c4x8q32", "q4", "l2_distance", 100_000_000, 256, 32, 1000, smallest=True, normalise=False,
                        note="the whole 100M x 256 q4 set, query batch 32"),
    "c4q32": Workload("c4q32", "q4", "l2_distance", 12_500_000, 256, 32, 1000, smallest=True, normalise=False,
                      note="one GPU's share (1/8) of the 100M x 256 q4 set, query batch 32"),
    "c5": Workload("c5", "q8", "dot", 5_000_000, 384, 128, 50, embed=(32000, 384, 128),
                   note="end to end: token batch -> embedding front end -> q8 dot score + top-k, queries never leave the device"),
    "c5n": Workload("c5n", "q8", "dot", 5_000_000, 384, 128, 50, embed=(32000, 384, 128), embed_order=1,
                    note="as c5 with the normalize-first step order: every token row is projected (tensor cores), normalised, then pooled"),
}
METRIC_NAME = "q8 cosine score+topk queries/s at 10M x 768 candidates (k=10, 1 query per pass)"


def _peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return 6650.0, "fallback (earlier pool measurement)"


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons during the timed region."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap,clocks.mem")

    def __init__(self, gpu_index: int):
        self.gpu, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "20", "-i", str(self.gpu)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
            time.sleep(0.3)  # let the first samples arrive before the timed region starts
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def stop(self, t_begin: float, t_end: float) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.1)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, power, mem = [], [], set(), [], []
        inside = [ln for (t, ln) in self.lines if t_begin <= t <= t_end + 0.05] or [ln for (_, ln) in self.lines]
        for ln in inside:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
                power.append(float(f[3]))
                if len(f) > 9:
                    mem.append(float(f[9]))
            except ValueError:
                continue
            for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(name)
        sm.sort()
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "power_w_max": max(power) if power else None,
                "mem_mhz_min": min(mem) if mem else None}


# ------------------------------------------------------------------------------------------------------------
_SAMPLE_CACHE = {}


def _cpu_sample(wl: Workload, sample_rows: int, nsets: int):
    """First `sample_rows` rows of the seeded set, de-quantised to f32 (the layout the reference holds), and the
    query batches -- the same values the GPU arm scores (same seeds, same generator)."""
    import numpy as np
    import torch

    import oracle
    from manta_b200 import synth

    key = (wl.name, sample_rows)
    if key in _SAMPLE_CACHE:
        return _SAMPLE_CACHE[key]
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    x = synth.rows_f16(0, sample_rows, wl.cols, normalise=wl.normalise, device=dev).float().cpu().numpy()
    if wl.embed:
        # the token batches themselves; cpu_reference_pass embeds them inside its timed region
        nsets = min(nsets, 2)
        table, proj = synth.embed_weights_f16(wl.embed[0], wl.embed[1], wl.cols, device=dev)
        tokens, mask = synth.token_batches(nsets, wl.nq, wl.embed[2], wl.embed[0], device=dev)
        q = (table.float().cpu().numpy(), proj.float().cpu().numpy(), tokens.cpu().numpy(), mask.cpu().numpy())
    else:
        q = synth.queries_f16(nsets * wl.nq, wl.cols, normalise=wl.normalise, device=dev).float().cpu().numpy().reshape(nsets, wl.nq, wl.cols)
    if wl.layout == "q8":
        docs = oracle.unpack_q8_rows(*oracle.pack_q8_rows(x))
    elif wl.layout == "q4":
        docs = oracle.unpack_q4_b32(*oracle.pack_q4_b32(x))
    else:
        docs = np.ascontiguousarray(x)
    _SAMPLE_CACHE[key] = (docs, q)
    return docs, q


def cpu_reference_pass(wl: Workload, sample_rows: int, threads: int, steps: int, warmup: int, nsets: int):
    """Times the oracle (C restatement of the score builtin + full-sort topKTensor) on the bounded sample;
    returns (queries/s extrapolated to wl.rows rows, seconds per sample pass, ids of the last pass)."""
    import numpy as np

    import oracle

    oracle.set_threads(threads)
    docs, queries = _cpu_sample(wl, sample_rows, nsets)
    last, times, front = None, [], []
    for i in range(warmup + steps):
        t0 = time.perf_counter()
        if wl.embed:
            table, proj, tokens, mask = queries
            j = i % tokens.shape[0]
            q = oracle.half_to_float(oracle.float_to_half(oracle.embed_pooled(table, proj, tokens[j], mask[j], wl.embed_order)))
        else:
            q = queries[i % nsets]
        tq = time.perf_counter()
        scores = oracle.SCORE_FNS[wl.metric](q, docs)
        last = oracle.topk(scores, min(wl.k, sample_rows), wl.smallest)
        t1 = time.perf_counter()
        if i >= warmup:
            times.append(t1 - tq)
            front.append(tq - t0)
    sec = sum(times) / len(times)
    front_sec = sum(front) / len(front)  # the embedding front end does not grow with the candidate rows
    qps = wl.nq / (front_sec + sec * (wl.rows / sample_rows))
    sec += front_sec
    return qps, sec, np.asarray(last)


def _sample_rows_for(wl: Workload) -> int:
    # about 1 GB of f32 rows for small batches, never fewer than 100,000 rows (the parity spot check runs on the same
    # sample), at most the whole set; the timed CPU work stays in the 10-30 s range
    return int(min(wl.rows, max(100_000, 250_000_000 // wl.cols // max(1, wl.nq // 4))))


def run_reference(args, wl: Workload):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle

    threads = os.cpu_count() or 1
    sample_rows = _sample_rows_for(wl)
    nsets = max(1, min(N_QUERY_SET, 4096 // wl.nq))
    t0 = time.perf_counter()
    # every step is one pass over the bounded sample; the run is capped so that it ends within a few minutes
    steps = max(1, min(args.steps, 10))
    warm = max(1, min(args.warmup, 2))
    qps, sec, _ = cpu_reference_pass(wl, sample_rows, threads, steps, warm, nsets)
    factor = wl.rows / sample_rows
    line = {
        "impl": "reference", "metric": METRIC_NAME if wl.name == "c3" else f"{wl.describe()} queries/s",
        "value": qps, "unit": "queries/s", "n_gpus": args.gpus, "steps": steps, "warmup": warm,
        "steps_requested": args.steps, "warmup_requested": args.warmup,
        "ms_per_step": wl.nq / qps * 1e3, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f64 accumulate / f32 result" if wl.metric != "dot" else "f32",
        "data": "synthetic",
        "config": {"workload": wl.describe(), "rows": wl.rows, "cols": wl.cols, "k": wl.k, "queries_per_step": wl.nq,
                   "layout": "f32 rows as the reference holds them (the same values the packed set de-quantises to)",
                   "where": "host cores"},
        "extrapolated": factor != 1.0, "extrapolation_factor": factor, "sample_rows": sample_rows,
        "sample_seconds_per_pass": sec, "sample_ms_per_step_measured": sec * 1e3,
        "cpu_baseline": {"value": qps, "unit": "queries/s", "cores": threads, "kind": "port",
                         "sample": f"{sample_rows} of {wl.rows} rows per step as f32, {steps} timed steps after {warm} warm-up "
                                   f"(at most 10 / 2 whatever was asked, to stay within minutes), {sec:.3f} s measured per "
                                   f"sample pass; score builtin + full-sort topKTensor restated in C with OpenMP over rows; "
                                   f"queries/s and ms_per_step extrapolated x{factor:g} to the full row count; the Go "
                                   f"toolchain is unavailable so the reference itself cannot run"},
        "e2e": {"value": qps, "unit": "queries/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0, "oracle_threads": oracle.num_threads(), "wall_s": time.perf_counter() - t0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------------------
def run_ours(args, wl: Workload):
    import numpy as np
    import torch

    from manta_b200 import native, sharding, synth

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the hot path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        # stdout carries the one JSON line: whatever the communicator set-up prints there (NCCL's version banner) is sent
        # to stderr for the duration of the set-up
        sys.stdout.flush()
        saved_stdout = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
            dist.barrier()   # the first collective creates the communicator
        finally:
            sys.stdout.flush()
            os.dup2(saved_stdout, 1)
            os.close(saved_stdout)
    native.load()
    # One "lane" = a runtime (stream + scratch) with its own result buffers.  With more than one GPU two lanes
    # alternate steps, so that the selection, the all-gather and the merge of one step overlap the scan of the
    # next (independent queries; throughput, not latency).  A single GPU runs one lane.
    n_lanes = args.lanes if args.lanes > 0 else (2 if world > 1 else 1)
    nq, k = wl.nq, wl.k
    nsets = max(1, min(N_QUERY_SET, 4096 // nq))
    if wl.embed:
        nsets = 8

    class Lane:
        def __init__(self):
            self.rt = native.Runtime(local_rank)
            self.stream = torch.cuda.ExternalStream(self.rt.stream)
            with torch.cuda.stream(self.stream):
                # ids and scores of a rank share one buffer so that a single all-gather carries both
                self.d_pair, self.d_ids, self.d_scores = sharding.new_pair(nq, k, "cuda")
                self.d_q = torch.empty((nq, wl.cols), dtype=torch.float16, device="cuda") if wl.embed else None
                if world > 1:
                    self.g_pair = torch.empty((world, 2, nq, k), dtype=torch.int32, device="cuda")
                    self.g_ids, self.g_scores, _, self.g_stride = sharding.merge_args(self.g_pair, nq, k)
                    self.m_ids = torch.empty((nq, k), dtype=torch.int32, device="cuda")
                    self.m_scores = torch.empty((nq, k), dtype=torch.float32, device="cuda")
            self.stream.synchronize()
            self.px = None
            if world > 1 and args.exchange == "peer":
                self.px = sharding.PeerExchange.try_create(self.rt, dist, nq, k)  # None on every rank if any rank cannot map its peers
                if self.px is None:
                    args.exchange = "nccl (peer mapping unavailable)"

        def merge(self, sync):
            if self.px is not None:
                self.px.merge(self.d_ids, self.d_scores, nq, k, self.m_ids, self.m_scores, smallest=wl.smallest, sync=sync)
                return
            with torch.cuda.stream(self.stream):
                sharding.gather_pairs(self.d_pair, self.g_pair, dist)
            self.rt.topk_merge_device(self.g_ids, self.g_scores, world, nq, k, self.m_ids, self.m_scores, smallest=wl.smallest,
                                      sync=sync, list_stride=self.g_stride)

    lanes = [Lane() for _ in range(n_lanes)]
    rt, stream = lanes[0].rt, lanes[0].stream

    r0, r1 = sharding.shard_bounds(wl.rows, rank, world)
    data, scales = synth.packed_candidates(rt, wl.layout, r0, r1, wl.cols, normalise=wl.normalise)
    cands = rt.bind(wl.layout, data, scales, row_base=r0, rows=r1 - r0, cols=wl.cols)
    emb = None
    with torch.cuda.stream(stream):
        if wl.embed:
            vocab, dim, seq = wl.embed
            table, proj = synth.embed_weights_f16(vocab, dim, wl.cols)
            d_tokens, d_mask = synth.token_batches(nsets, nq, seq, vocab)
        else:
            d_queries = synth.queries_f16(nsets * nq, wl.cols, normalise=wl.normalise).view(nsets, nq, wl.cols)
    stream.synchronize()
    if wl.embed:
        emb = rt.bind_embedder(table.cpu().numpy().view(np.uint16), proj.cpu().numpy().view(np.uint16))
        h_tokens = d_tokens.cpu().pin_memory().numpy()
        h_mask = d_mask.cpu().pin_memory().numpy()
    else:
        h_queries = d_queries.cpu().numpy().view(np.uint16)
    d_ids, d_scores, d_pair = lanes[0].d_ids, lanes[0].d_scores, lanes[0].d_pair
    if world > 1:
        g_pair, g_ids, g_scores, g_stride = lanes[0].g_pair, lanes[0].g_ids, lanes[0].g_scores, lanes[0].g_stride
        m_ids, m_scores = lanes[0].m_ids, lanes[0].m_scores

    def step_device(i):
        ln = lanes[i % n_lanes]
        if wl.embed:
            ln.rt.embed_device(emb, d_tokens[i % nsets], d_mask[i % nsets], nq, wl.embed[2], ln.d_q, normalize_then_pool=bool(wl.embed_order), sync=False)
            dq = ln.d_q
        else:
            dq = d_queries[i % nsets]
        if ln.px is not None:  # shard pass, exchange over peer memory and merge as one stream-ordered chain
            ln.px.score_topk_merge(cands, wl.metric, dq, nq, k, ln.m_ids, ln.m_scores, smallest=wl.smallest, sync=False)
            return
        ln.rt.score_topk_device(cands, wl.metric, dq, nq, k, ln.d_ids, ln.d_scores, smallest=wl.smallest, sync=False)
        if world > 1:
            ln.merge(False)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing ------------------------------------------------------------------
    def warm_up():
        """Runs the warm-up steps; returns the first error text (None if every lane finished cleanly)."""
        problem = None
        for i in range(max(args.warmup, n_lanes)):
            step_device(i)
        for ln in lanes:
            try:
                ln.rt.synchronize()  # raises if a warm-up pass overflowed its pool or a peer's list never arrived
            except native.MantaError as exc:
                problem = problem or str(exc)
        return problem

    problem = warm_up()
    if world > 1 and any(ln.px is not None for ln in lanes):
        # If the peer exchange misbehaved on ANY rank, every rank drops it and the run continues over NCCL.
        bad = torch.tensor([1 if problem else 0], dtype=torch.int32, device="cuda")
        dist.all_reduce(bad, op=dist.ReduceOp.MAX)
        if int(bad.item()):
            for ln in lanes:
                try:
                    ln.px.close()
                except native.MantaError:
                    pass
                ln.px = None
            args.exchange = "nccl (the peer exchange failed during warm-up: %s)" % (problem or "on another rank")
            problem = warm_up()
    if problem:
        raise SystemExit("bench.py: warm-up failed: " + problem)
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # The scan kernel is timed by CUDA events inside the timed region when one lane runs; with two lanes the lanes'
    # kernels overlap, so the per-kernel time is taken from a single-lane pass after the timed region instead.
    profile_inside = n_lanes == 1
    if profile_inside:
        rt.profile(True)
    barrier()  # after the sampler's start-up delay, so that all ranks enter the timed region together
    launches0 = native.kernel_launch_count()
    t_begin = time.perf_counter()
    repeat_ms = []
    launches = 0
    for rep in range(max(1, args.repeats)):
        # One repeat = one independent measurement of the timed region: `warmup` untimed steps, then exactly `steps`
        # steps between a barrier + synchronize on both sides, CUDA events on the stream.  Repeats are a quarter of a
        # second apart, so that one does not inherit the power / thermal state the previous one left.
        if rep > 0:
            time.sleep(0.25)
            for i in range(max(args.warmup, n_lanes)):
                step_device(i)
            barrier()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record(stream)
        for i in range(args.steps):
            step_device(rep * args.steps + i)
        for ln in lanes[1:]:  # the closing event waits for every lane
            done = torch.cuda.Event()
            done.record(ln.stream)
            stream.wait_event(done)
        ev1.record(stream)
        barrier()
        for ln in lanes:
            ln.rt.synchronize()
        if rep == 0:
            launches = native.kernel_launch_count() - launches0
        repeat_ms.append(ev0.elapsed_time(ev1))
    t_end = time.perf_counter()
    scan_ms, scan_passes = rt.scan_time() if profile_inside else (0.0, 0)
    rt.profile(False)
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None
    if not profile_inside:
        lanes[0].rt.profile(True)
        for i in range(min(args.steps, 20)):
            ln = lanes[0]
            if wl.embed:
                ln.rt.embed_device(emb, d_tokens[i % nsets], d_mask[i % nsets], nq, wl.embed[2], ln.d_q, normalize_then_pool=bool(wl.embed_order), sync=False)
            dq1 = ln.d_q if wl.embed else d_queries[i % nsets]
            if ln.px is not None:
                ln.px.score_topk_merge(cands, wl.metric, dq1, nq, k, ln.m_ids, ln.m_scores, smallest=wl.smallest, sync=False)
            else:
                ln.rt.score_topk_device(cands, wl.metric, dq1, nq, k, ln.d_ids, ln.d_scores, smallest=wl.smallest, sync=False)
                ln.merge(False)
        scan_ms, scan_passes = lanes[0].rt.scan_time()
        lanes[0].rt.profile(False)
        barrier()
    t = torch.tensor(repeat_ms + [scan_ms / max(scan_passes, 1)], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    repeat_ms = [float(x) for x in t[:-1]]
    scan_ms_per_pass = float(t[-1])
    # the value comes from the median repeat (each repeat is `steps` steps, max over ranks)
    order_ms = sorted(repeat_ms)
    total_ms = order_ms[len(order_ms) // 2]
    total_steps = args.steps * len(repeat_ms)
    last = lanes[(total_steps - 1) % n_lanes]
    final_ids = (last.m_ids if world > 1 else last.d_ids).cpu().numpy().copy()
    stats_device = rt.stats()

    # ---- sharded runs over the peer exchange check themselves against the NCCL path (one extra, untimed step) -------
    exchange_verified = None
    if world > 1 and lanes[0].px is not None:
        ln = lanes[0]
        step_no = total_steps + 7
        dq_chk = None
        if wl.embed:
            ln.rt.embed_device(emb, d_tokens[step_no % nsets], d_mask[step_no % nsets], nq, wl.embed[2], ln.d_q, normalize_then_pool=bool(wl.embed_order), sync=False)
            dq_chk = ln.d_q
        else:
            dq_chk = d_queries[step_no % nsets]
        ln.px.score_topk_merge(cands, wl.metric, dq_chk, nq, k, ln.m_ids, ln.m_scores, smallest=wl.smallest, sync=True)
        peer_ids, peer_scores = ln.m_ids.cpu().numpy().copy(), ln.m_scores.cpu().numpy().copy()
        ln.rt.score_topk_device(cands, wl.metric, dq_chk, nq, k, ln.d_ids, ln.d_scores, smallest=wl.smallest, sync=False)
        with torch.cuda.stream(ln.stream):
            sharding.gather_pairs(ln.d_pair, ln.g_pair, dist)
        ln.rt.topk_merge_device(ln.g_ids, ln.g_scores, world, nq, k, ln.m_ids, ln.m_scores, smallest=wl.smallest, sync=True,
                                list_stride=ln.g_stride)
        same = bool(np.array_equal(peer_ids, ln.m_ids.cpu().numpy()) and np.array_equal(peer_scores, ln.m_scores.cpu().numpy()))
        flag = torch.tensor([1 if same else 0], dtype=torch.int32, device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        exchange_verified = bool(int(flag.item()))
        if not exchange_verified:
            raise SystemExit("bench.py: the peer exchange and the NCCL path disagree on the merged top-k")

    # ---- end to end through the host-buffer ABI call ------------------------------------------------
    # Sharded: every lane has its own pinned host buffers and staging buffers; steps alternate between the lanes, and
    # a step's result is read (its lane synchronised) while the next step is already on the other lane, so that the
    # selection, exchange and merge of one step overlap the scan of the next -- like the device-timed loop.  Every step's
    # host-to-device and device-to-host copies stay inside the timed region.
    hbs = []  # released before the streams they used
    if world > 1:
        for ln in lanes:
            hb = {}
            with torch.cuda.stream(ln.stream):
                if wl.embed:
                    hb["tokens"] = torch.from_numpy(h_tokens)
                    hb["mask"] = torch.from_numpy(h_mask)
                    hb["s_tokens"] = torch.empty((nq, wl.embed[2]), dtype=torch.int32, device="cuda")
                    hb["s_mask"] = torch.empty((nq, wl.embed[2]), dtype=torch.int32, device="cuda")
                    hb["s_q"] = torch.empty((nq, wl.cols), dtype=torch.float16, device="cuda")
                else:
                    hb["queries"] = torch.from_numpy(h_queries.view(np.int16)).pin_memory()
                    hb["s_q"] = torch.empty((nq, wl.cols), dtype=torch.int16, device="cuda")
                hb["ids"] = torch.empty((nq, k), dtype=torch.int32).pin_memory()
                hb["scores"] = torch.empty((nq, k), dtype=torch.float32).pin_memory()
            ln.stream.synchronize()
            hbs.append(hb)
        hb = None  # the list holds the only references: hbs.clear() below must release the pinned buffers

    def enqueue_host_step(i):
        """Upload, shard pass, exchange + merge, download of step i on lane i % n_lanes; returns the lane index."""
        li = i % n_lanes
        ln, hb = lanes[li], hbs[li]
        with torch.cuda.stream(ln.stream):
            if wl.embed:
                hb["s_tokens"].copy_(hb["tokens"][i % nsets], non_blocking=True)
                hb["s_mask"].copy_(hb["mask"][i % nsets], non_blocking=True)
            else:
                hb["s_q"].copy_(hb["queries"][i % nsets], non_blocking=True)
        if wl.embed:
            ln.rt.embed_device(emb, hb["s_tokens"], hb["s_mask"], nq, wl.embed[2], hb["s_q"], normalize_then_pool=bool(wl.embed_order), sync=False)
        if ln.px is not None:
            # the merge writes the step's ids and scores straight into the pinned host buffers (device-addressable memory):
            # the same bytes cross PCIe, without a copy operation behind the kernel
            ln.px.score_topk_merge(cands, wl.metric, hb["s_q"], nq, k, hb["ids"], hb["scores"], smallest=wl.smallest, sync=False)
        else:
            ln.rt.score_topk_device(cands, wl.metric, hb["s_q"], nq, k, ln.d_ids, ln.d_scores, smallest=wl.smallest, sync=False)
            ln.merge(False)
            with torch.cuda.stream(ln.stream):
                hb["ids"].copy_(ln.m_ids, non_blocking=True)
                hb["scores"].copy_(ln.m_scores, non_blocking=True)
        return li

    def finish_host_step(li):
        lanes[li].rt.synchronize()  # also raises if the pass overflowed its pool or a list never arrived
        return hbs[li]["ids"].numpy(), hbs[li]["scores"].numpy()

    def host_steps(first, count):
        if world == 1:
            for i in range(first, first + count):
                if wl.embed:
                    rt.embed_score_topk(emb, cands, h_tokens[i % nsets], h_mask[i % nsets], wl.metric, k, smallest=wl.smallest,
                                        normalize_then_pool=bool(wl.embed_order))
                else:
                    rt.score_topk(cands, wl.metric, h_queries[i % nsets], k, smallest=wl.smallest)
            return
        pending = []
        for i in range(first, first + count):
            pending.append(enqueue_host_step(i))
            if len(pending) == n_lanes:  # the oldest step's lane is needed again: read its result first
                finish_host_step(pending.pop(0))
        while pending:
            finish_host_step(pending.pop(0))

    host_steps(0, args.warmup)
    barrier()
    t0 = time.perf_counter()
    host_steps(args.warmup, args.steps)
    barrier()
    e2e_s = time.perf_counter() - t0
    te = torch.tensor([e2e_s], dtype=torch.float64, device="cuda")
    if world > 1:
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
    e2e_s = float(te[0])

    # The sharded end-to-end steps deliver their results in pinned host buffers: one more step (untimed) must hand back
    # exactly what the device-resident path returns for the same queries.
    e2e_verified = None
    if world > 1 and lanes[0].px is not None and not wl.embed:
        j = args.warmup + args.steps
        ids_h, sc_h = finish_host_step(enqueue_host_step(j))
        ids_h, sc_h = ids_h.copy(), sc_h.copy()
        ln = lanes[j % n_lanes]
        ln.px.score_topk_merge(cands, wl.metric, d_queries[j % nsets], nq, k, ln.m_ids, ln.m_scores, smallest=wl.smallest, sync=True)
        same = bool(np.array_equal(ids_h, ln.m_ids.cpu().numpy()) and np.array_equal(sc_h, ln.m_scores.cpu().numpy()))
        flag = torch.tensor([1 if same else 0], dtype=torch.int32, device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        e2e_verified = bool(int(flag.item()))
        if not e2e_verified:
            raise SystemExit("bench.py: the end-to-end step and the device-resident step disagree")

    # ---- CPU baseline + parity spot check on the same bounded sample (rank 0, N=1) ----------------------
    cpu = None
    parity = None
    if rank == 0 and world == 1 and not args.no_cpu:
        sample_rows = _sample_rows_for(wl)
        threads = os.cpu_count() or 1
        qps, sec, ref_ids = cpu_reference_pass(wl, sample_rows, threads, 3, 1, nsets)
        qps1 = cpu_reference_pass(wl, sample_rows, 1, 1, 0, nsets)[0] if nq <= 4 else None  # bounded: small batches only
        cpu = {"value": qps, "unit": "queries/s", "cores": threads, "kind": "port",
               "sample": f"first {sample_rows} of {wl.rows} rows as f32 per pass, 3 timed passes after 1 warm-up, "
                         f"C restatement of the score builtin + full-sort topKTensor with OpenMP over rows; queries/s "
                         f"extrapolated x{wl.rows / sample_rows:g}; single thread (the reference's own threading): "
                         + (f"{qps1:.4f} queries/s" if qps1 is not None else "not timed for this batch size"),
               "single_thread_value": qps1, "sample_seconds_per_pass": sec, "extrapolated": wl.rows != sample_rows}
        sub = rt.bind(wl.layout, data[:sample_rows], None if scales is None else scales[:sample_rows], row_base=0,
                      rows=sample_rows, cols=wl.cols)
        kk = min(k, sample_rows)
        if wl.embed:  # the CPU pass cycles through two token batches; its last pass used batch 3 % 2
            ids, sc = rt.embed_score_topk(emb, sub, h_tokens[1], h_mask[1], wl.metric, kk, smallest=wl.smallest,
                                          normalize_then_pool=bool(wl.embed_order))
        else:
            ids, sc = rt.score_topk(sub, wl.metric, h_queries[(1 + 3 - 1) % nsets], kk, smallest=wl.smallest)
        # the comparison rule of tests/helpers.py: ids equal to topKTensor's except across score gaps below twice the
        # tolerance, returned scores within tolerance of the oracle's
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import oracle
        from helpers import EMBED_FLOOR, FLOOR, REL_TOL, topk_parity_report

        docs_f32, q_sets = _cpu_sample(wl, sample_rows, nsets)
        if wl.embed:
            table, proj, tokens, mask = q_sets
            q_chk = oracle.half_to_float(oracle.float_to_half(oracle.embed_pooled(table, proj, tokens[1], mask[1], wl.embed_order)))
        else:
            q_chk = q_sets[(1 + 3 - 1) % nsets]
        floor = EMBED_FLOOR if wl.embed else FLOOR  # the embedded queries themselves differ from the CPU's in a few f16 roundings
        parity = topk_parity_report(wl.metric, q_chk, docs_f32, np.asarray(ids).reshape(nq, kk), np.asarray(sc).reshape(nq, kk), kk,
                                    wl.smallest, floor=floor)
        parity.update({"sample_rows": sample_rows, "rel_tol": REL_TOL, "floor": floor,
                       "ids_equal_fraction": float((np.asarray(ids).reshape(nq, kk) == ref_ids.reshape(nq, kk)).mean())})
        sub.unbind()

    if rank == 0:
        peak, peak_src = _peaks()
        shard_rows = r1 - r0
        algo_bytes = shard_rows * wl.row_bytes()
        achieved = algo_bytes / (scan_ms_per_pass * 1e-3) / 1e9
        # DRAM traffic per launch is not read live: it is the dram__bytes_read + dram__bytes_write of one ncu capture of
        # the same kernel on a 2 M-row case (1.5521e9 B read + 4.0e6 B written for 2e6 rows), scaled by rows -- every row
        # is read exactly once, so traffic grows in proportion.
        traffic, traffic_source = None, None
        if wl.layout == "q8" and wl.metric == "cosine" and wl.cols == 768 and nq == 1:
            traffic = shard_rows * (1.552110e9 + 4.0e6) / 2e6
            traffic_source = "from_profile: profiles/stream_scan_q8_cosine_2Mx768.md (ncu, 2 M rows), scaled by rows; not measured in this run"
        value = args.steps * nq / (total_ms * 1e-3)
        line = {
            "metric": METRIC_NAME if wl.name == "c3" else f"{wl.describe()} queries/s",
            "value": value, "unit": "queries/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": total_ms / args.steps,
            "repeats": {"count": len(repeat_ms), "ms_per_step": [x / args.steps for x in repeat_ms],
                        "median_ms_per_step": total_ms / args.steps, "min_ms_per_step": min(repeat_ms) / args.steps,
                        "max_ms_per_step": max(repeat_ms) / args.steps,
                        "note": "each repeat is an independent measurement (warm-up steps, then exactly `steps` timed steps between "
                                "barriers), 0.25 s apart; value is the median repeat"}, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": {"q8": "int8 x int8 -> int32 (two int8 query planes), f32 epilogue",
                      "q4": "int4 x int8 -> int32 per block, f32 across blocks", "f16": "f16 x f16 -> f32"}[wl.layout],
            "data": "synthetic",
            "config": {"workload": wl.describe(), "rows": wl.rows, "cols": wl.cols, "k": k, "queries_per_step": nq,
                       "layout": wl.layout, "shards": world, "note": wl.note, "lanes": n_lanes,
                       "exchange": (args.exchange if world > 1 else None), "exchange_equals_nccl_path": exchange_verified, "e2e_equals_device_path": e2e_verified,
                       "l2": f"inputs larger than L2: {algo_bytes / 1e9:.3f} GB scanned per pass and GPU" if algo_bytes > 2.5e8
                             else "inputs smaller than L2 (latency-bound configuration, not a roofline point)"},
            "candidates_dim_per_s": value * wl.rows * wl.cols,
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic, "traffic_source": traffic_source, "peak_source": peak_src,
                         "kernel": "mma_scan_kernel (mma.cu, tcgen05)" if stats_device["mma_passes"] else "stream_scan_kernel (stream_scan.cuh)",
                         "kernel_ms": scan_ms_per_pass,
                         "kernel_ms_source": "CUDA events around the scan kernel inside the timed region" if profile_inside else
                                             "CUDA events around the scan kernel in a single-lane pass after the timed region (two lanes overlap inside it)", "algorithmic_bytes_per_launch": algo_bytes,
                         "frac_of_nominal_8TBs": achieved / 8000.0},
            "e2e": {"value": args.steps * nq / e2e_s, "unit": "queries/s", "h2d_bytes_per_step": (2 * nq * wl.embed[2] * 4) if wl.embed else nq * wl.cols * 2,
                    "d2h_bytes_per_step": nq * k * 8, "ms_per_step": e2e_s / args.steps * 1e3,
                    "note": "host-buffer C-ABI call per step; candidates stay bound (resident) as plan parameters"
                            if world == 1 else "inputs from pinned host memory, results to pinned host memory, one synchronisation per "
                            "step, steps alternating over the lanes (upload, shard pass, " + ("peer-store exchange fused with the merge" if str(args.exchange) == "peer"
                                                            else "NCCL all-gather, merge") + ", download on one stream)"},
            "gpu_launches": int(launches), "clocks": clocks, "cpu_baseline": cpu, "parity_check": parity,
            "result_checksum": int(np.asarray(final_ids, dtype=np.int64).sum()),
            "stats": rt.stats(),
        }
        print(json.dumps(line), flush=True)
    torch.cuda.synchronize()
    for ln in lanes:
        if ln.px is not None:
            ln.px.close()
    hbs.clear()
    if wl.embed:
        h_tokens = h_mask = None  # pinned: released while the streams that read them still exist
    import gc

    gc.collect()
    cands.unbind()
    if emb is not None:
        rt.unbind_embedder(emb)
    for ln in lanes:
        ln.rt.close()
    if world > 1:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c3", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline / parity spot check")
    ap.add_argument("--rows", type=int, default=0, help="override the workload's row count (smaller cases for profiling)")
    ap.add_argument("--cols", type=int, default=0, help="override the workload's row width")
    ap.add_argument("--nq", type=int, default=0, help="override the workload's query batch")
    ap.add_argument("--k", type=int, default=0, help="override the workload's k")
    ap.add_argument("--metric", default="", choices=["", "dot", "cosine", "l2_distance"], help="override the workload's metric")
    ap.add_argument("--smallest", action="store_true", help="select the k smallest scores instead of the k largest")
    ap.add_argument("--exchange", default="peer", choices=["nccl", "peer"],
                    help="sharded runs: how the per-shard lists meet (NCCL all-gather + merge, or peer stores over NVLink fused "
                         "with the merge)")
    ap.add_argument("--repeats", type=int, default=5, help="timed repeats of `steps` steps; the value is the median repeat")
    ap.add_argument("--lanes", type=int, default=0,
                    help="runtimes alternating steps (0: one on a single GPU, two when sharded so that merge and scan overlap)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    wl = WORKLOADS[args.workload]
    if args.rows:
        wl.rows = args.rows
    if args.cols:
        wl.cols = args.cols
    if args.nq:
        wl.nq = args.nq
    if args.k:
        wl.k = args.k
    if args.metric:
        wl.metric = args.metric
    if args.smallest:
        wl.smallest = True
    if args.impl == "reference":
        run_reference(args, wl)
    else:
        run_ours(args, wl)


if __name__ == "__main__":
    main()
