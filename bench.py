#!/usr/bin/env python
"""Benchmark of the tile-sparse hot path on B200.

One "step" is one pass of the masked GEMMs of a BERT-base encoder layer (QKV, attention output,
FFN1, FFN2; batch 32 x sequence 128 = 4096 rows) over one batch of synthetic activations, fp16
inputs with fp32 accumulation, tile-wise sparsity 75 % at G = 128.  The metric is the kept-FLOP
rate  2*M*sum_t K_t*N_t / time;  the speed-up over cuBLAS dense on the same shapes is reported
beside it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Launched under torchrun for N > 1 (one rank per GPU): every rank runs the same layer on its own
batch (no data-path collective), timing is the max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "kept_flop_tflops_tw75_g128"
UNIT = "TFLOP/s"
GEMMS = ("qkv", "attn_out", "ffn1", "ffn2")
M_ROWS = 4096
SPARSITY = 75.0
G = 128
L2_BYTES = 126 * 1024 * 1024


def load_peaks() -> dict:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


# ------------------------------------------------------------------------------------------------
# Clock sampling during the timed region (read-only NVML queries)
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {
        0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
        0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
        0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting",
    }

    def __init__(self, torch_device_index: int):
        self.samples, self.reasons = [], set()
        self.max_mhz = None
        self._stop = threading.Event()
        self._thread = None
        self._h = None
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(torch_device_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            try:
                self._h = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            except Exception:
                self._h = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            self._nv = pynvml
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:
            self._h = None

    def _poll(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                bits = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
                for b, name in self.REASONS.items():
                    if bits & b and name != "gpu_idle":
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.005)

    def start(self):
        if self._h is not None:
            self._thread = threading.Thread(target=self._poll, daemon=True)
            self._thread.start()

    def stop(self) -> dict:
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
        med = int(np.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------------
# Workload
# ------------------------------------------------------------------------------------------------
def make_kept_lists(name: str, K: int, N: int, W, masks: str):
    """Per-tile kept-row lists for one weight matrix at 75 % tile-wise sparsity."""
    from tilesparsity_b200 import synth
    n_tiles = (N + G - 1) // G
    if masks == "random":
        keep = int(round(K * (1 - SPARSITY / 100.0) / 8)) * 8
        return synth.random_kept_lists(K, n_tiles, keep, synth.BERT_SEEDS[name] + 100)
    from tilesparsity_b200 import masks as tsm
    res = tsm.build_mask("tw1", [W.abs()], SPARSITY, G)
    return res.tiles[0].lists()


def build_workload(device, masks: str, n_sets: int):
    import torch
    from tilesparsity_b200 import TWLayer, synth
    work = []
    for name in GEMMS:
        A, W = synth.bert_gemm(name, M_ROWS)
        K, N = W.shape
        Wd = torch.from_numpy(W).to(device)
        lists = make_kept_lists(name, K, N, Wd, masks)
        layer = TWLayer.from_lists(Wd, lists, None, G, torch.float16)
        At = torch.from_numpy(np.ascontiguousarray(A.T)).to(device=device, dtype=torch.float16)
        g = {"name": name, "K": K, "N": N, "layer": layer, "W16": Wd.to(torch.float16),
             "At": [At] + [At.clone() for _ in range(n_sets - 1)],
             "Ct": [torch.zeros((N, M_ROWS), dtype=torch.float16, device=device) for _ in range(n_sets)],
             "A_rm": [At.t().contiguous() for _ in range(n_sets)],
             "C_rm": [torch.empty((M_ROWS, N), dtype=torch.float16, device=device) for _ in range(n_sets)]}
        g["kept_flops"] = layer.stats()["kept_flops_per_row"] * M_ROWS
        g["dense_flops"] = 2 * M_ROWS * K * N
        g["alg_bytes"] = layer.algorithmic_bytes(M_ROWS)
        work.append(g)
    return work


def time_loop(fn, steps: int, warmup: int, barrier=None, graph_span: int = 0):
    """fn(i) enqueues step i; returns elapsed milliseconds of `steps` steps on the current stream.

    With graph_span > 0 the steps are captured once into a CUDA graph of `graph_span` consecutive
    steps (fn must be periodic in i with that period) and the graph is replayed steps/graph_span
    times, so the host's launch path is not part of the measurement.
    """
    import torch
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    graph = None
    if graph_span > 0:
        assert steps % graph_span == 0
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(graph_span):
                fn(i)
        graph.replay()
        torch.cuda.synchronize()
    if barrier is not None:
        barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    if graph is not None:
        for _ in range(steps // graph_span):
            graph.replay()
    else:
        for i in range(steps):
            fn(warmup + i)
    e1.record()
    torch.cuda.synchronize()
    if barrier is not None:
        barrier()
    return e0.elapsed_time(e1)


def cpu_reference_pass(sample_steps: int, budget_s: float, masks: str = "tw1"):
    """The reference's CPU path for the same step: NumPy `A @ (W * mask)` per GEMM on fp32
    (Pruning/BERT/utils/modeling.py:992-1007) with the masks of the CPU oracle's tw1
    (Pruning/VGG/prune_algo.py:113-148).  The mask build is timed separately."""
    from oracle import masked_gemm as og
    from oracle import tw_masks as om
    from tilesparsity_b200 import synth
    from tilesparsity_b200.tiles import tiles_from_lists, tiles_from_mask
    items, kept, t_mask = [], 0, 0.0
    for name in GEMMS:
        A, W = synth.bert_gemm(name, M_ROWS)
        K, N = W.shape
        if masks == "random":
            keep = int(round(K * (1 - SPARSITY / 100.0) / 8)) * 8
            lists = synth.random_kept_lists(K, (N + G - 1) // G, keep, synth.BERT_SEEDS[name] + 100)
            ts = tiles_from_lists(K, N, G, lists)
            mask = ts.dense_mask()
        else:
            t0 = time.perf_counter()
            mask = om.tw1([np.abs(W)], SPARSITY, G)[0]
            t_mask += time.perf_counter() - t0
            ts = tiles_from_mask(mask, G)
        items.append((A, W, mask))
        kept += ts.kept_flops_per_row() * M_ROWS
    og.masked_matmul_dense(*items[1])  # warm the BLAS threads
    times = []
    t_start = time.perf_counter()
    for _ in range(max(1, sample_steps)):
        t0 = time.perf_counter()
        for A, W, mask in items:
            og.masked_matmul_dense(A, W, mask)
        times.append(time.perf_counter() - t0)
        if time.perf_counter() - t_start > budget_s:
            break
    try:
        from threadpoolctl import threadpool_info
        cores = max([p.get("num_threads", 1) for p in threadpool_info()] + [1])
    except Exception:
        cores = os.cpu_count() or 1
    t = float(np.median(times))
    # one step with the BLAS pool limited to a single thread, for a per-core figure
    t_one = None
    try:
        from threadpoolctl import threadpool_limits
        with threadpool_limits(limits=1):
            t0 = time.perf_counter()
            for A, W, mask in items:
                og.masked_matmul_dense(A, W, mask)
            t_one = time.perf_counter() - t0
    except Exception:
        t_one = None
    return {"value": kept / t / 1e12, "seconds_per_step": t, "steps_run": len(times), "cores": int(cores),
            "kept_flops": kept, "mask_build_seconds": t_mask,
            "value_one_thread": (kept / t_one / 1e12) if t_one else None}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    r = cpu_reference_pass(args.steps, budget_s=90.0, masks=args.masks)
    sample = (f"{r['steps_run']} full steps (4 GEMMs, M={M_ROWS}) of numpy fp32 A@(W*mask) on the host, "
              f"median; requested steps={args.steps}")
    line = {
        "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": r["seconds_per_step"] * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "impl": "reference",
        "config": {"workload": f"bert_base_layer_m{M_ROWS}_tw75_g{G}", "gemms": list(GEMMS), "masks": args.masks},
        "cpu_baseline": {"value": r["value"], "unit": UNIT, "cores": r["cores"], "kind": "port", "sample": sample,
                         "value_one_thread": r["value_one_thread"], "host_cpus": os.cpu_count()},
        "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_ours(args):
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the tile-sparse kernels have no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    barrier = None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        barrier = dist.barrier
    peaks = load_peaks()

    step_bytes = 0
    n_sets = 4
    work = build_workload(device, args.masks, n_sets)
    step_bytes = sum(g["alg_bytes"] for g in work)
    footprint = n_sets * sum(g["At"][0].numel() * 2 + g["Ct"][0].numel() * 2 for g in work)

    def step(i):
        s = i % n_sets
        for g in work:
            g["layer"].masked_gemm(g["At"][s], out=g["Ct"][s])

    def dense_step(i):
        s = i % n_sets
        for g in work:
            torch.matmul(g["A_rm"][s], g["W16"], out=g["C_rm"][s])

    span = 0 if args.no_graph else n_sets
    steps = args.steps if span == 0 else max(span, args.steps // span * span)
    args.steps = steps
    sampler = ClockSampler(local_rank)
    time_loop(step, 4, max(3, args.warmup), barrier)  # settle clocks and caches before sampling
    sampler.start()
    ms = time_loop(step, steps, max(3, args.warmup), barrier, span)
    clocks = sampler.stop()
    for g in work:
        g["layer"].check()
    ms_t = torch.tensor([ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(ms_t, op=dist.ReduceOp.MAX)
    ms_max = float(ms_t.item())
    kept_flops_step = sum(g["kept_flops"] for g in work)
    value = world * kept_flops_step * args.steps / (ms_max * 1e-3) / 1e12

    # Per-GEMM timings, cuBLAS dense on the same shapes, end-to-end through host buffers (rank 0).
    per_gemm, ms_dense, e2e, cpu, grouped = [], None, None, None, None
    if rank == 0:
        sub_steps = max(48, min(args.steps, 480) // 4 * 4)
        tot_masked = 0.0
        for g in work:
            t_m = time_loop(lambda i, g=g: g["layer"].masked_gemm(g["At"][i % n_sets], out=g["Ct"][i % n_sets]),
                            sub_steps, 5, None, span) / sub_steps
            t_d = time_loop(lambda i, g=g: torch.matmul(g["A_rm"][i % n_sets], g["W16"], out=g["C_rm"][i % n_sets]),
                            sub_steps, 5, None, span) / sub_steps
            sched = g["layer"].schedule_stats(M_ROWS)
            tot_masked += t_m
            per_gemm.append({"name": g["name"], "K": g["K"], "N": g["N"], "us": t_m * 1e3, "dense_us": t_d * 1e3,
                             "speedup_vs_cublas_dense": t_d / t_m,
                             "kept_tflops": g["kept_flops"] / (t_m * 1e-3) / 1e12,
                             "dense_tflops": g["dense_flops"] / (t_d * 1e-3) / 1e12,
                             "gbs": g["alg_bytes"] / (t_m * 1e-3) / 1e9,
                             "ctas": sched["n_ctas"], "units": sched["n_units"], "balance": round(sched["balance"], 4)})
        ms_dense = time_loop(dense_step, sub_steps, 5, None, span) / sub_steps

        # The four GEMMs of this benchmark do not depend on each other, so they can also run as ONE
        # tile-wise sparse layer: block-structured weights, activations stacked [sum K][M], outputs
        # stacked [sum N][M] (TWLayer.grouped).  Same kernel, same results; one launch instead of four.
        # Reported beside the headline, which keeps the four launches a real layer needs.
        from tilesparsity_b200 import TWLayer
        glayer, k_off, n_off = TWLayer.grouped([g["W16"] for g in work], [g["layer"].tiles for g in work], torch.float16)
        gAt = [torch.cat([g["At"][s] for g in work], dim=0).contiguous() for s in range(n_sets)]
        gCt = [torch.zeros((int(n_off[-1]), M_ROWS), dtype=torch.float16, device=device) for _ in range(n_sets)]
        glayer.masked_gemm(gAt[0], out=gCt[0])
        same = all(torch.equal(gCt[0][n_off[i]:n_off[i + 1]], g["layer"].masked_gemm(g["At"][0]))
                   for i, g in enumerate(work))
        ms_grouped = time_loop(lambda i: glayer.masked_gemm(gAt[i % n_sets], out=gCt[i % n_sets]),
                               sub_steps, 5, None, span) / sub_steps
        grouped = {"ms_per_step": ms_grouped, "value": kept_flops_step / (ms_grouped * 1e-3) / 1e12, "unit": UNIT,
                   "speedup_vs_cublas_dense": ms_dense / ms_grouped, "identical_to_separate_launches": bool(same),
                   "what": "the four GEMMs as one block-structured tile-wise layer over stacked activations and "
                           "outputs (TWLayer.grouped): one launch; valid because they are independent here"}
        glayer.close()
        del gAt, gCt

        # mask construction for the four weight matrices (tw1, 75 %), timed end to end on the GPU
        mask_build = None
        if args.masks == "tw1":
            from tilesparsity_b200 import masks as tsm
            scores = [g["W16"].float().abs() for g in work]
            for sc in scores:
                tsm.build_mask("tw1", [sc], SPARSITY, G)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            reps = 5
            for _ in range(reps):
                for sc in scores:
                    tsm.build_mask("tw1", [sc], SPARSITY, G)
            torch.cuda.synchronize()
            dt = (time.perf_counter() - t0) / reps
            nbytes = sum(sc.numel() * 4 + sc.numel() for sc in scores)   # scores read once, dense masks written
            mask_build = {"seconds": dt, "bytes": int(nbytes), "gbs": nbytes / dt / 1e9,
                          "what": "ts_build_tw_mask(tw1) on the 4 weight matrices, host-synchronous call, wall clock"}

        # end to end: pinned host activations in, host outputs back, through ts_masked_gemm_host_async
        hA = [torch.empty((g["K"], M_ROWS), dtype=torch.float16).pin_memory() for g in work]
        hC = [torch.empty((g["N"], M_ROWS), dtype=torch.float16).pin_memory() for g in work]
        for h, g in zip(hA, work):
            h.copy_(g["At"][0].cpu())

        def e2e_step(i):
            # the four GEMMs are independent: each call queues its copy-in / GEMM / copy-out pipeline
            # and returns; the timing loop's stream resumes when every output is on the host
            for g, a, c in zip(work, hA, hC):
                g["layer"].masked_gemm_host(a, c, wait=False)
            for g in work:
                g["layer"].host_wait()

        e2e_steps = max(5, min(args.steps, 30))
        ms_e2e = time_loop(e2e_step, e2e_steps, 3) / e2e_steps
        e2e = {"value": kept_flops_step / (ms_e2e * 1e-3) / 1e12, "unit": UNIT,
               "h2d_bytes_per_step": int(sum(h.numel() * 2 for h in hA)),
               "d2h_bytes_per_step": int(sum(h.numel() * 2 for h in hC)),
               "ms_per_step": ms_e2e, "n_gpus_timed": 1,
               "what": "ts_masked_gemm_host_async per GEMM (pinned host buffers, 4 column blocks each, copies of "
                       "different GEMMs overlap), one wait per step"}
        if world == 1:
            r = cpu_reference_pass(8, budget_s=25.0, masks=args.masks)
            cpu = {"value": r["value"], "unit": UNIT, "cores": r["cores"], "kind": "port",
                   "sample": f"{r['steps_run']} full steps of numpy fp32 A@(W*mask), 4 GEMMs at M={M_ROWS}, median",
                   "seconds_per_step": r["seconds_per_step"], "mask_build_seconds": r["mask_build_seconds"],
                   "value_one_thread": r["value_one_thread"], "host_cpus": os.cpu_count()}

    if rank == 0:
        t_launch = (sum(p["us"] for p in per_gemm) / len(per_gemm)) * 1e-6
        bytes_launch = step_bytes / len(work)
        achieved = bytes_launch / t_launch / 1e9
        traffic = None
        tp = os.path.join(ROOT, "profiles", "masked_gemm_traffic.json")
        if os.path.exists(tp):
            with open(tp) as f:
                traffic = json.load(f).get("dram_bytes_per_launch")
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms_max / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"bert_base_layer_m{M_ROWS}_tw75_g{G}", "gemms": list(GEMMS),
                       "masks": args.masks, "accumulate": "f32",
                       "launch": "host launches" if args.no_graph else f"CUDA graph of {n_sets} steps, replayed",
                       "l2": f"activations and outputs rotate over {n_sets} buffer sets "
                             f"({footprint / 2**20:.0f} MiB > {L2_BYTES / 2**20:.0f} MiB L2)",
                       "parallelism": f"dp{world}"},
            "speedup_vs_cublas_dense": (ms_dense / (ms_max / args.steps)) if ms_dense else None,
            "cublas_dense_ms_per_step": ms_dense,
            "tensor_frac_of_measured_peak": value / world / peaks["bf16_tflops"],
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "traffic": traffic, "peak_source": peaks["source"],
                         "kernel": "masked_gemm_kernel", "bytes_per_launch": bytes_launch,
                         "us_per_launch": t_launch * 1e6},
            "cpu_baseline": cpu,
            "mask_build": mask_build,
            "grouped_single_launch": grouped,
            "e2e": e2e,
            "gpu_launches": len(work) * args.steps,
            "clocks": clocks,
            "per_gemm": per_gemm,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run_square(args):
    """Tile-sharded strong-scaling run: M = N = K = --size, bf16, tile-wise 75 % with per-tile kept-row
    counts skewed ~Beta(2,5); the column tiles are sharded across the ranks by kept FLOPs
    (tilesparsity_b200.sharding), every rank holds At and computes its own slab of Ct; with
    --gather nccl the slabs are all-gathered over NCCL inside the timed region; with --gather fused the
    GEMM's epilogue stores every kept row into all ranks' buffers (peer-mapped memory over NVLink)."""
    import torch
    import torch.distributed as dist
    from tilesparsity_b200 import sharding, synth
    from tilesparsity_b200.tiles import tiles_from_lists

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    barrier = None
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
        barrier = dist.barrier
    n = args.size
    nt = (n + G - 1) // G
    counts = synth.beta_skewed_counts(n, nt, 1 - SPARSITY / 100.0, 5000 + int(np.log2(n)))
    g = synth.rng(5000 + int(np.log2(n)))
    lists = [np.sort(g.choice(n, size=int(c), replace=False)).astype(np.int32) for c in counts]
    ts = tiles_from_lists(n, n, G, lists)
    gen = torch.Generator(device=device).manual_seed(1234)
    W = torch.randn((n, n), generator=gen, device=device, dtype=torch.float32)
    shard = sharding.ShardedTWLayer(W, ts, rank, world, torch.bfloat16)
    del W
    n_sets = max(2, min(4, (3 * L2_BYTES) // (n * n * 2) + 1))
    At = [torch.randn((n, n), generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16) for _ in range(n_sets)]
    Ct = [torch.zeros((shard.plan.n_pad, n), dtype=torch.bfloat16, device=device) for _ in range(n_sets)]
    full = torch.empty((world * shard.plan.n_pad, n), dtype=torch.bfloat16, device=device) if args.gather == "nccl" else None
    fused = shard.make_gather_buffer(n) if (args.gather == "fused" and world > 1) else None

    def step(i):
        s = i % n_sets
        if fused is not None:
            shard.masked_gemm_allgather(At[s], fused[0], fused[1])
            return
        shard.masked_gemm(At[s], out=Ct[s])
        if args.gather == "nccl" and world > 1:
            dist.all_gather_into_tensor(full, Ct[s])

    sampler = ClockSampler(local_rank)
    time_loop(step, 2, max(3, args.warmup), barrier)
    sampler.start()
    ms = time_loop(step, args.steps, max(3, args.warmup), barrier)
    clocks = sampler.stop()
    shard.layer.check()
    ms_t = torch.tensor([ms], dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(ms_t, op=dist.ReduceOp.MAX)
    kept = ts.kept_flops_per_row() * n
    value = kept * args.steps / (float(ms_t.item()) * 1e-3) / 1e12
    if rank == 0:
        peaks = load_peaks()
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": max(3, args.warmup), "ms_per_step": float(ms_t.item()) / args.steps, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": f"square_{n}_tw75_g{G}_beta25", "gather": args.gather,
                           "parallelism": f"tile-sharded x{world}", "shard_balance": round(shard.plan.balance(), 4),
                           "l2": f"activations rotate over {n_sets} buffers of {n * n * 2 / 2**20:.0f} MiB"},
                "tensor_frac_of_measured_peak": value / world / peaks["bf16_tflops_sustained"],
                "gpu_launches": args.steps, "clocks": clocks}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--masks", choices=["tw1", "random"], default="tw1",
                    help="tw1: the reference's tile-wise masks of the synthetic weights, built on the GPU; "
                         "random: the perf driver's random per-tile row subsets")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from the host instead of replaying a CUDA graph")
    ap.add_argument("--workload", choices=["bert", "square"], default="bert",
                    help="bert: the headline BERT-base layer step; square: tile-sharded M=N=K=--size strong scaling")
    ap.add_argument("--size", type=int, default=16384)
    ap.add_argument("--gather", choices=["none", "nccl", "fused"], default="none",
                    help="square workload: all-gather Ct inside the timed region, with NCCL after the GEMM or "
                         "by the GEMM's epilogue storing into the peers' buffers")
    args = ap.parse_args()
    if args.workload == "square" and args.impl == "ours":
        if args.steps == 2000:
            args.steps = 20
        run_square(args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
