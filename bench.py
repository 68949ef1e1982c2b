#!/usr/bin/env python
"""Benchmark of the sampler hot path: rows sampled per second at V = 151936 on the row-partitioned serving
batch (1024 rows per GPU, temperature 0.7, top_k 50, top_p 0.95, min_p 0.02, repeat_penalty 1.15 over a 256-id
window), seeded synthetic logits.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--rows R] [--sweep]

One JSON line on stdout (rank 0).  `value` = rows/s with the logits resident in HBM (CUDA events on the launch
stream, max over ranks); `e2e` = the same through the host-buffer entry point, host->device copy of the logits
and device->host copy of the ids inside the timed region; `roofline` = algorithmic bytes (4 * V per row) over
the measured launch duration against the measured HBM copy peak; `cpu_baseline` = the reference's own CPU
sampler on this box's host cores.  Under torchrun every rank samples its own 1024 rows (no collective on the
data path: rows are independent), so scaling is weak.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

VOCAB = 151936
NCU_DRAM_BYTES_PER_ROW = 631_340  # (368.10 MB read + 5.65 MB written) / 592 rows, 128-thread build; algorithmic: 4 * V = 607_744
FALLBACK_HBM_GBS = 6650.0  # earlier measurement on this pool, used only if MEASURED_PEAKS.json is absent


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            return float(json.load(open(path))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons of one GPU while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.samples = []
        self.proc = None
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                 "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) >= 6:
                self.samples.append(parts)

    def stop(self):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()
        sm = [int(s[0]) for s in self.samples if s[0].isdigit()]
        mx = [int(s[1]) for s in self.samples if s[1].isdigit()]
        reasons = []
        for name, col in (("hw_slowdown", 2), ("hw_thermal_slowdown", 3), ("sw_thermal_slowdown", 4), ("sw_power_cap", 5)):
            if any(s[col].lower().startswith("active") for s in self.samples):
                reasons.append(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm)}


def cpu_reference(wl, seconds_of_work: float = 10.0):
    """The reference CPU sampler (qp::Sampler compiled into oracle/_ref) fanned over all host threads on the
    bench workload's rows; falls back to the single-threaded C restatement when that build is absent."""
    from oracle import Oracle, Ref

    rows = wl.rows
    if Ref.available():
        threads = Ref.hardware_threads()
        best = None
        done = 0.0
        reps = 0
        while done < seconds_of_work and reps < 50:
            r = Ref.sample_rows(wl.params, wl.logits, wl.history, wl.hist_len, threads=threads)
            sec = r["seconds"]
            best = sec if best is None else min(best, sec)
            done += sec * threads
            reps += 1
        return {"value": rows / best, "unit": "rows/s", "cores": threads, "kind": "reference",
                "sample": f"{rows} rows of the bench workload, best of {reps} passes over all host threads"}
    n = min(rows, 64)
    t0 = time.perf_counter()
    Oracle.sample_rows(wl.params[:n], wl.logits[:n], wl.history[:n], wl.hist_len[:n])
    sec = time.perf_counter() - t0
    return {"value": n / sec, "unit": "rows/s", "cores": 1, "kind": "port",
            "sample": f"first {n} rows of the bench workload, one pass, one thread"}


def run_reference(args, rank, world):
    if rank != 0:
        return
    from oracle import Ref
    from qpack_b200 import synth

    wl = synth.serving_batch(rows=args.rows, vocab=VOCAB)
    if not Ref.available():
        base = cpu_reference(wl, 5.0)
        sec = args.rows / base["value"]
        cores, kind = base["cores"], base["kind"]
        ms = sec * 1e3
    else:
        threads = Ref.hardware_threads()
        for _ in range(args.warmup):
            Ref.sample_rows(wl.params, wl.logits, wl.history, wl.hist_len, threads=threads)
        t = 0.0
        for _ in range(args.steps):
            t += Ref.sample_rows(wl.params, wl.logits, wl.history, wl.hist_len, threads=threads)["seconds"]
        ms = t / args.steps * 1e3
        cores, kind = threads, "reference"
    value = args.rows / (ms * 1e-3)
    line = {
        "impl": "reference", "metric": "rows sampled/sec at V=151936", "value": value, "unit": "rows/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "row-partitioned serving batch (config 4)", "rows_per_gpu": args.rows, "vocab": VOCAB,
                   "history": 256, "note": "reference CPU sampler on the host cores of rank 0, one step = all rows"},
        "cpu_baseline": {"value": value, "unit": "rows/s", "cores": cores, "kind": kind,
                         "sample": f"{args.rows} rows per step, {args.steps} steps"},
        "e2e": {"value": value, "unit": "rows/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def graph_latency_us(bs, torch, x, h, iters=50):
    """Device time of one call: CUDA-graph replay of `iters` back-to-back launches, divided by iters."""
    s = torch.cuda.Stream()
    out = torch.empty(x.shape[0], dtype=torch.int32, device=x.device)
    with torch.cuda.stream(s):
        for _ in range(3):
            bs.sample(x, h, out=out)
        s.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            for _ in range(iters):
                bs.sample(x, h, out=out)
        g.replay()
        s.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(s)
        g.replay()
        e1.record(s)
        s.synchronize()
    return e0.elapsed_time(e1) / iters * 1e3


def run_ours(args, rank, world, local_rank):
    import torch

    from qpack_b200 import synth
    from qpack_b200.sampler import BatchSampler

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA GPU: the sampler has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod

        dist = dist_mod
        dist.init_process_group("nccl", device_id=dev)

    rows = args.rows
    wl = synth.serving_batch(rows=rows, vocab=VOCAB, seed=4 + rank)
    h_logits = torch.from_numpy(wl.logits).pin_memory()
    h_hist = torch.from_numpy(wl.history).pin_memory()
    d_logits = h_logits.to(dev, non_blocking=True)
    d_hist = h_hist.to(dev, non_blocking=True)
    out = torch.empty(rows, dtype=torch.int32, device=dev)
    bs = BatchSampler(rows, local_rank)
    bs.set_params(wl.params)
    stream = torch.cuda.current_stream(dev)

    def barrier():
        torch.cuda.synchronize(dev)
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- device-resident throughput ----
    for _ in range(max(args.warmup, 3)):
        bs.sample(d_logits, d_hist, out=out)
    bs.check()
    clocks = ClockSampler(local_rank)
    if rank == 0:
        clocks.start()
        time.sleep(0.3)
    barrier()
    # The K timed steps are captured once into a CUDA graph (K kernel nodes, one per step) and replayed: a serving
    # loop launches its decode step that way, and it keeps host launch gaps out of the device time.  One untimed
    # replay first uploads the graph.
    side = torch.cuda.Stream(dev)
    side.wait_stream(stream)
    launches0 = bs.launches
    with torch.cuda.stream(side):
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(args.steps):
                bs.sample(d_logits, d_hist, out=out)
        launches = bs.launches - launches0
        graph.replay()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    # the 622 MB of logits per step exceed the 126 MB L2, so every step streams from HBM
    with torch.cuda.stream(side):
        e0.record(side)
        graph.replay()
        e1.record(side)
    barrier()
    bs.check()
    ms = e0.elapsed_time(e1) / args.steps
    clock_info = clocks.stop() if rank == 0 else None

    # ---- end to end through the host-buffer entry point ----
    ids_host = np.empty(rows, np.int32)
    bs.set_params(wl.params)
    e2e_steps = max(2, min(args.steps, 5))
    bs.sample_host(wl_logits_np(h_logits), wl.history, None, out=ids_host)
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        bs.sample_host(wl_logits_np(h_logits), wl.history, None, out=ids_host)
    torch.cuda.synchronize(dev)
    e2e_ms = (time.perf_counter() - t0) / e2e_steps * 1e3

    t = torch.tensor([ms, e2e_ms], dtype=torch.float64, device=dev)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e_ms = float(t[0]), float(t[1])

    extra = {}
    if rank == 0:
        # single-row latency (device time, the row stays in L2) and the batch sweep
        bs1 = BatchSampler(rows, local_rank)
        bs1.set_params(wl.params)
        extra["b1_latency_us"] = round(graph_latency_us(bs1, torch, d_logits[:1], d_hist[:1]), 2)
        if args.sweep:
            sweep = {}
            for b in (1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024):
                if b <= rows:
                    us = graph_latency_us(bs1, torch, d_logits[:b], d_hist[:b], iters=20)
                    sweep[str(b)] = {"us": round(us, 1), "rows_per_s": round(b / us * 1e6), "gbs": round(b * 4 * VOCAB / us / 1e3, 1),
                                     "regime": "hbm" if b * 4 * VOCAB > 126e6 else "l2"}
            extra["sweep"] = sweep
        bs1.close()

    # ---- vocabulary-sharded step (config 5), N > 1 only: latency-bound, reported by phase ----
    if dist is not None:
        sh = bench_vocab_sharded(torch, dist, dev, local_rank, rank, world, graph=args.sharded_graph)
        if rank == 0:
            extra["vocab_sharded"] = sh

    if rank == 0:
        peak, peak_kind = measured_peak()
        bytes_per_launch = rows * 4 * VOCAB
        achieved = bytes_per_launch / (ms * 1e-3) / 1e9
        # DRAM bytes per launch: dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this kernel on a
        # 592-row case of the same workload (profiles/stream_rows_kernel_serving_batch.md), scaled by rows
        traffic = NCU_DRAM_BYTES_PER_ROW * rows
        line = {
            "metric": "rows sampled/sec at V=151936", "value": rows * world / (ms * 1e-3), "unit": "rows/s", "n_gpus": world,
            "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": "row-partitioned serving batch (config 4)", "rows_per_gpu": rows, "vocab": VOCAB,
                       "history": 256, "params": "T0.7 top_k50 top_p0.95 min_p0.02 rp1.15",
                       "l2": "inputs (622 MB per GPU) larger than L2, no flush needed", "parallelism": f"rows x{world}",
                       "launch": "the K steps replayed as one CUDA graph of K kernel launches"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": traffic, "peak_source": peak_kind, "frac_of_8000": achieved / 8000.0,
                         "kernel": "stream_rows_kernel<MODE_SAMPLE>"},
            "cpu_baseline": cpu_reference(wl, args.cpu_seconds),
            "e2e": {"value": rows * world / (e2e_ms * 1e-3), "unit": "rows/s", "h2d_bytes_per_step": int(wl.logits.nbytes + wl.history.nbytes),
                    "d2h_bytes_per_step": int(ids_host.nbytes), "ms_per_step": e2e_ms},
            "gpu_launches": int(launches),
            "clocks": clock_info,
        }
        line.update(extra)
        print(json.dumps(line), flush=True)
    bs.close()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def bench_vocab_sharded(torch, dist, dev, local_rank, rank, world, iters=30, graph=False):
    """Config 5 over the ranks of this run: 128 rows, V = 151936 split into contiguous column shards, local top-64
    per shard -> one all-gather -> merge, filter and draw.  Device time per phase (CUDA events on the current
    stream, max over ranks); every rank must end up with the same ids."""
    from qpack_b200 import synth
    from qpack_b200.distributed import gather_candidates, vocab_shard
    from qpack_b200.sampler import BatchSampler

    wl = synth.sharded_batch(rows=128, vocab=VOCAB)
    c0, c1 = vocab_shard(VOCAB, world, rank)
    per_max = max(vocab_shard(VOCAB, world, r)[1] - vocab_shard(VOCAB, world, r)[0] for r in range(world))
    x = torch.from_numpy(np.ascontiguousarray(wl.logits[:, c0:c1])).to(dev)
    bs = BatchSampler(128, local_rank)
    bs.set_params(wl.params)
    slots = bs.cand_slots(VOCAB, per_max)
    stream = torch.cuda.current_stream(dev)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]
    acc = np.zeros(3)
    ids = None
    for it in range(iters + 3):
        ev[0].record(stream)
        local = bs.local_candidates(x, VOCAB, c0, slots)
        ev[1].record(stream)
        allc = gather_candidates(local)
        ev[2].record(stream)
        ids = bs.merge_sample(allc, VOCAB)
        ev[3].record(stream)
        torch.cuda.synchronize(dev)
        if it >= 3:
            acc += [ev[i].elapsed_time(ev[i + 1]) * 1e3 for i in range(3)]
    # the same step, ten times over, captured in one CUDA graph (kernel -> all-gather -> kernel, no host in between)
    graph_us = None
    try:
        if not graph:
            raise RuntimeError("not requested (--sharded-graph)")
        side = torch.cuda.Stream(dev)
        side.wait_stream(stream)
        with torch.cuda.stream(side):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=side):
                for _ in range(10):
                    ids_g = bs.merge_sample(gather_candidates(bs.local_candidates(x, VOCAB, c0, slots)), VOCAB)
            g.replay()
            side.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(side)
            g.replay()
            e1.record(side)
            side.synchronize()
            graph_us = e0.elapsed_time(e1) * 1e3 / 10
    except Exception as exc:  # capture of the collective is not available: the per-phase numbers stand alone
        graph_us = None
        if graph:
            sys.stderr.write(f"vocab-sharded graph capture skipped: {exc}\n")
    bs.check()
    bs.close()
    gt = torch.tensor([graph_us if graph_us is not None else -1.0], dtype=torch.float64, device=dev)
    dist.all_reduce(gt, op=dist.ReduceOp.MAX)
    graph_us = float(gt.item()) if float(gt.item()) > 0 else None
    t = torch.tensor(acc / iters, dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    same = ids.to(torch.int64).clone()
    dist.broadcast(same, src=0)
    agree = torch.tensor([int(torch.equal(same, ids.to(torch.int64)))], device=dev)
    dist.all_reduce(agree, op=dist.ReduceOp.MIN)
    us = [float(v) for v in t]
    return {"rows": 128, "vocab": VOCAB, "shards": world, "local_topk_us": round(us[0], 1), "all_gather_us": round(us[1], 1),
            "merge_draw_us": round(us[2], 1), "rows_per_s": round(128 / (sum(us) * 1e-6)),
            "all_gather_bytes_sent_per_rank": int(128 * slots * 8), "ranks_agree": bool(int(agree.item())),
            "step_us_in_one_graph": None if graph_us is None else round(graph_us, 1)}


def wl_logits_np(pinned):
    return pinned.numpy()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--rows", type=int, default=1024)
    ap.add_argument("--sweep", action="store_true")
    ap.add_argument("--sharded-graph", action="store_true", dest="sharded_graph",
                    help="N > 1: also time the vocabulary-sharded step captured in one CUDA graph (NCCL inside the capture)")
    ap.add_argument("--cpu-seconds", type=float, default=10.0, dest="cpu_seconds")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
    else:
        run_ours(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
