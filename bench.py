#!/usr/bin/env python
"""Benchmark of the tile-sparse hot path on B200.

One "step" is one pass of the masked GEMMs of a BERT-base encoder layer (QKV, attention output,
FFN1, FFN2; batch 32 x sequence 128 = 4096 rows) over one batch of synthetic activations, fp16
inputs with fp32 accumulation, tile-wise sparsity 75 % at G = 128.  The metric is the kept-FLOP
rate  2*M*sum_t K_t*N_t / time;  the speed-up over cuBLAS dense on the same shapes is reported
beside it.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

The timed region of K steps is repeated (at least 50 times, about 0.4 s in total); `ms_per_step` is
the median over the repeats, the spread is reported, and the clocks are sampled across all repeats.
Before anything is timed every GEMM's output is compared with the CPU oracle (`verified`).

Launched under torchrun for N > 1 (one rank per GPU): every rank runs the same layer on its own
batch (no data-path collective, weak scaling; timing is the max over ranks), and the line also
carries a `tile_sharded` block: the 16384-square layer with its column tiles sharded over the ranks
by kept FLOPs, without a gather, with the gather fused into the GEMM's epilogue (peer stores over
NVLink) and with NCCL's all-gather, next to one GPU running the whole layer.

Other workloads of the benchmark configurations (one JSON line per row, one GPU):

    python bench.py --workload vgg|lstm|square|bert_sweep|masks|readme
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
MIN_REPEATS = 50
TIMED_SECONDS = 0.4


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
        s = self.samples
        return {"sm_mhz": int(np.median(s)) if s else None, "sm_mhz_min": int(min(s)) if s else None,
                "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": len(s)}


# ------------------------------------------------------------------------------------------------
# Timing
# ------------------------------------------------------------------------------------------------
class StepRunner:
    """Enqueues `steps` consecutive steps of fn(i) on the current stream, from CUDA graphs when
    graph_span > 0 (fn must be periodic in i with that period): one graph of graph_span steps replayed
    steps // graph_span times and one of the remaining steps, so exactly `steps` steps run."""

    def __init__(self, fn, steps: int, graph_span: int = 0):
        import torch
        self.fn, self.steps, self.span = fn, steps, graph_span
        self.main = self.tail = None
        if graph_span > 0:
            torch.cuda.synchronize()
            if steps >= graph_span:
                self.main = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self.main):
                    for i in range(graph_span):
                        fn(i)
            if steps % graph_span:
                self.tail = torch.cuda.CUDAGraph()
                with torch.cuda.graph(self.tail):
                    for i in range(steps % graph_span):
                        fn(i)
            torch.cuda.synchronize()

    def run(self):
        if self.span > 0:
            for _ in range(self.steps // self.span):
                self.main.replay()
            if self.tail is not None:
                self.tail.replay()
        else:
            for i in range(self.steps):
                self.fn(i)


def timed_repeats(fn, steps: int, warmup: int, repeats: int, barrier=None, graph_span: int = 0) -> list:
    """Milliseconds of `steps` steps, `repeats` times: CUDA events on the current stream, a barrier and
    a device synchronisation on both sides of every repeat."""
    import torch
    for i in range(warmup):
        fn(i)
    torch.cuda.synchronize()
    runner = StepRunner(fn, steps, graph_span)
    runner.run()
    torch.cuda.synchronize()
    out = []
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(repeats):
        if barrier is not None:
            barrier()
        torch.cuda.synchronize()
        e0.record()
        runner.run()
        e1.record()
        torch.cuda.synchronize()
        out.append(e0.elapsed_time(e1))
    if barrier is not None:
        barrier()
    return out


def time_us(fn, steps: int, warmup: int = 5, graph_span: int = 0, repeats: int = 5) -> float:
    """Median microseconds per step."""
    ms = timed_repeats(fn, steps, warmup, repeats, None, graph_span)
    return float(np.median(ms)) / steps * 1e3


def max_over_ranks(values, device, world):
    import torch
    import torch.distributed as dist
    t = torch.tensor(values, dtype=torch.float64, device=device)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return t.cpu().numpy()


# ------------------------------------------------------------------------------------------------
# The reference's CPU path
# ------------------------------------------------------------------------------------------------
def cpu_reference_pass(sample_steps: int, budget_s: float, masks: str = "tw1"):
    """The reference's CPU path for the same step: NumPy `A @ (W * mask)` per GEMM on fp32
    (Pruning/BERT/utils/modeling.py:992-1007) with the masks of the CPU oracle's tw1
    (Pruning/VGG/prune_algo.py:113-148), on every host core the BLAS pool can use.  A launcher such
    as torchrun exports OMP_NUM_THREADS=1 to its children; the pool is therefore sized explicitly.
    The mask build is timed separately."""
    from threadpoolctl import threadpool_limits
    from oracle import masked_gemm as og
    from oracle import tw_masks as om
    from tilesparsity_b200 import synth
    from tilesparsity_b200.tiles import tiles_from_lists, tiles_from_mask
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
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
    times = []
    with threadpool_limits(limits=cores):
        og.masked_matmul_dense(*items[1])  # warm the BLAS threads
        t_start = time.perf_counter()
        for _ in range(max(1, sample_steps)):
            t0 = time.perf_counter()
            for A, W, mask in items:
                og.masked_matmul_dense(A, W, mask)
            times.append(time.perf_counter() - t0)
            if time.perf_counter() - t_start > budget_s:
                break
    t = float(np.median(times))
    with threadpool_limits(limits=1):     # one step on a single thread, for a per-core figure
        t0 = time.perf_counter()
        for A, W, mask in items:
            og.masked_matmul_dense(A, W, mask)
        t_one = time.perf_counter() - t0
    return {"value": kept / t / 1e12, "seconds_per_step": t, "steps_run": len(times), "cores": int(cores),
            "kept_flops": kept, "mask_build_seconds": t_mask, "value_one_thread": kept / t_one / 1e12}


def run_reference(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    r = cpu_reference_pass(args.steps, budget_s=90.0, masks=args.masks)
    sample = (f"{r['steps_run']} full steps (4 GEMMs, M={M_ROWS}) of numpy fp32 A@(W*mask) on {r['cores']} host "
              f"threads, median; requested steps={args.steps}")
    line = {
        "metric": METRIC, "value": r["value"], "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": r["seconds_per_step"] * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "impl": "reference",
        "config": {"workload": f"bert_base_layer_m{M_ROWS}_tw75_g{G}", "gemms": list(GEMMS), "masks": args.masks},
        "cpu_baseline": {"value": r["value"], "unit": UNIT, "cores": r["cores"], "kind": "port", "sample": sample,
                         "value_one_thread": r["value_one_thread"], "host_cpus": os.cpu_count()},
        "e2e": {"value": r["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "CPU throughput of one host, whatever --gpus says: the same number of host cores serves every N",
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# Headline workload: the BERT-base layer step
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


def verify_workload(work) -> dict:
    """Every GEMM of the step against the CPU oracle (compaction form, StreamMaskedGEMM/perf/
    basic_nn.cu:450-503) on the same 16-bit-rounded inputs, outside the timed region."""
    from oracle import masked_gemm as og
    worst, bad = 0.0, 0
    for g in work:
        out = g["layer"].masked_gemm(g["At"][0], out=g["Ct"][0]).float().cpu().numpy()
        g["layer"].check()
        ref = og.masked_matmul_compacted(g["At"][0].float().cpu().numpy(), g["W16"].float().cpu().numpy(),
                                         g["layer"].tiles)
        worst = max(worst, og.max_rel_error(out, ref))
        bad += og.elementwise_violations(out, ref, rtol=1e-2, floor=1e-3)
    return {"verified": bool(worst <= 1e-2 and bad == 0), "max_rel_err": worst, "elementwise_violations": bad,
            "checker": "oracle.masked_gemm.masked_matmul_compacted, bounds 1e-2 (matrix) and 1e-2|ref|+1e-3 rms (element)"}


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

    n_sets = 4
    work = build_workload(device, args.masks, n_sets)
    step_bytes = sum(g["alg_bytes"] for g in work)
    footprint = n_sets * sum(g["At"][0].numel() * 2 + g["Ct"][0].numel() * 2 for g in work)
    check = verify_workload(work) if rank == 0 else None
    if check is not None and not check["verified"]:
        raise RuntimeError(f"masked GEMM output differs from the oracle: {check}")

    def step(i):
        s = i % n_sets
        for g in work:
            g["layer"].masked_gemm(g["At"][s], out=g["Ct"][s])

    def dense_step(i):
        s = i % n_sets
        for g in work:
            torch.matmul(g["A_rm"][s], g["W16"], out=g["C_rm"][s])

    span = 0 if args.no_graph else n_sets
    warm = max(3, args.warmup)
    # settle clocks and caches, and size the number of repeats from a first estimate of the step
    est = float(np.median(timed_repeats(step, args.steps, warm, 3, barrier, span))) / args.steps * 1e-3
    repeats = int(max(MIN_REPEATS, min(5000, np.ceil(TIMED_SECONDS / max(est * args.steps, 1e-9)))))
    repeats = int(max_over_ranks([repeats], device, world)[0])
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms = timed_repeats(step, args.steps, warm, repeats, barrier, span)
    clocks = sampler.stop()
    for g in work:
        g["layer"].check()
    ms = max_over_ranks(ms, device, world)                      # per repeat: the slowest rank
    ms_med = float(np.median(ms))
    kept_flops_step = sum(g["kept_flops"] for g in work)
    value = world * kept_flops_step * args.steps / (ms_med * 1e-3) / 1e12

    # end to end on every rank: pinned host activations in, host outputs back, through
    # ts_masked_gemm_host_async
    hA = [torch.empty((g["K"], M_ROWS), dtype=torch.float16).pin_memory() for g in work]
    hC = [[torch.empty((g["N"], M_ROWS), dtype=torch.float16).pin_memory() for g in work] for _ in range(2)]
    for h, g in zip(hA, work):
        h.copy_(g["At"][0].cpu())
    e2e_steps = max(5, min(args.steps, 30))

    def e2e_step_serial(i):
        # the four GEMMs are independent: each call queues its copy-in / GEMM / copy-out pipeline
        # and returns; the timing loop's stream resumes when every output of the step is on the host
        for g, a, c in zip(work, hA, hC[i % 2]):
            g["layer"].masked_gemm_host(a, c, wait=False)
        for g in work:
            g["layer"].host_wait()

    def e2e_step(i):
        # steps queued back to back: the next step's copy-in runs under this step's copy-out (a layer's
        # staging buffers are handed over by events inside the library); outputs alternate between two
        # host buffer sets; the timing loop's stream waits once, for the last step of the region
        for g, a, c in zip(work, hA, hC[i % 2]):
            g["layer"].masked_gemm_host(a, c, wait=False)
        if i % e2e_steps == e2e_steps - 1:
            for g in work:
                g["layer"].host_wait()

    ms_serial = max_over_ranks(timed_repeats(e2e_step_serial, e2e_steps, 3, 5, barrier), device, world)
    ms_serial = float(np.median(ms_serial)) / e2e_steps
    ms_e2e = max_over_ranks(timed_repeats(e2e_step, e2e_steps, e2e_steps, 5, barrier), device, world)
    ms_e2e = float(np.median(ms_e2e)) / e2e_steps
    e2e = {"value": world * kept_flops_step / (ms_e2e * 1e-3) / 1e12, "unit": UNIT,
           "h2d_bytes_per_step": int(world * sum(h.numel() * 2 for h in hA)),
           "d2h_bytes_per_step": int(world * sum(h.numel() * 2 for h in hC[0])),
           "ms_per_step": ms_e2e, "ms_per_step_one_step_in_flight": ms_serial, "n_gpus_timed": world,
           "what": "ts_masked_gemm_host_async per GEMM (pinned host buffers in and out, contiguous copies), steps "
                   "queued back to back so that one step's copy-out runs under the next step's copy-in, one wait "
                   "at the end of the timed region; every rank moves its own batch, max over ranks"}
    if rank == 0:
        from oracle import masked_gemm as og
        ref = og.masked_matmul_compacted(hA[1].float().numpy(), work[1]["W16"].float().cpu().numpy(), work[1]["layer"].tiles)
        e2e["verified"] = bool(og.max_rel_error(hC[0][1].float().numpy(), ref) <= 1e-2 and
                               og.max_rel_error(hC[1][1].float().numpy(), ref) <= 1e-2)

    # Per-GEMM timings, cuBLAS dense on the same shapes, mask build, CPU baseline (rank 0).
    per_gemm, ms_dense, cpu, grouped, mask_build = [], None, None, None, None
    if rank == 0:
        sub_steps = 48
        for g in work:
            t_m = time_us(lambda i, g=g: g["layer"].masked_gemm(g["At"][i % n_sets], out=g["Ct"][i % n_sets]),
                          sub_steps, 5, span, 9)
            t_d = time_us(lambda i, g=g: torch.matmul(g["A_rm"][i % n_sets], g["W16"], out=g["C_rm"][i % n_sets]),
                          sub_steps, 5, span, 9)
            sched = g["layer"].schedule_stats(M_ROWS)
            per_gemm.append({"name": g["name"], "K": g["K"], "N": g["N"], "us": t_m, "dense_us": t_d,
                             "speedup_vs_cublas_dense": t_d / t_m,
                             "kept_tflops": g["kept_flops"] / t_m / 1e6,
                             "dense_tflops": g["dense_flops"] / t_d / 1e6,
                             "gbs": g["alg_bytes"] / t_m / 1e3,
                             "hbm_frac": g["alg_bytes"] / t_m / 1e3 / peaks["hbm_gbs"],
                             "ctas": sched["n_ctas"], "units": sched["n_units"], "balance": round(sched["balance"], 4)})
        ms_dense = time_us(dense_step, sub_steps, 5, span, 9) * 1e-3

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
        ms_grouped = time_us(lambda i: glayer.masked_gemm(gAt[i % n_sets], out=gCt[i % n_sets]), sub_steps, 5, span, 9) * 1e-3
        grouped = {"ms_per_step": ms_grouped, "value": kept_flops_step / (ms_grouped * 1e-3) / 1e12, "unit": UNIT,
                   "speedup_vs_cublas_dense": ms_dense / ms_grouped, "identical_to_separate_launches": bool(same),
                   "what": "the four GEMMs as one block-structured tile-wise layer over stacked activations and "
                           "outputs (TWLayer.grouped): one launch; valid because they are independent here"}
        glayer.close()
        del gAt, gCt

        # mask construction for the four weight matrices (tw1, 75 %), timed end to end on the GPU
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
        if world == 1:
            r = cpu_reference_pass(8, budget_s=25.0, masks=args.masks)
            cpu = {"value": r["value"], "unit": UNIT, "cores": r["cores"], "kind": "port",
                   "sample": f"{r['steps_run']} full steps of numpy fp32 A@(W*mask), 4 GEMMs at M={M_ROWS}, median",
                   "seconds_per_step": r["seconds_per_step"], "mask_build_seconds": r["mask_build_seconds"],
                   "value_one_thread": r["value_one_thread"], "host_cpus": os.cpu_count()}

    sharded = None
    if world > 1:
        for g in work:
            g["layer"].close()
        del work, hA, hC
        torch.cuda.empty_cache()
        sharded = tile_sharded_block(args, device, rank, world)

    if rank == 0:
        t_launch = sum(p["us"] for p in per_gemm) / len(per_gemm) * 1e-6
        bytes_launch = step_bytes / len(GEMMS)
        achieved = bytes_launch / t_launch / 1e9
        traffic = None
        tp = os.path.join(ROOT, "profiles", "masked_gemm_traffic.json")
        if os.path.exists(tp):
            with open(tp) as f:
                traffic = json.load(f).get("dram_bytes_per_launch")
        per_step = ms / args.steps
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": warm, "ms_per_step": ms_med / args.steps, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": {"workload": f"bert_base_layer_m{M_ROWS}_tw75_g{G}", "gemms": list(GEMMS),
                       "masks": args.masks, "accumulate": "f32",
                       "launch": "host launches" if args.no_graph else f"CUDA graph of {n_sets} steps, replayed",
                       "l2": f"activations and outputs rotate over {n_sets} buffer sets "
                             f"({footprint / 2**20:.0f} MiB > {L2_BYTES / 2**20:.0f} MiB L2)",
                       "parallelism": f"dp{world}"},
            "repeats": {"n": int(len(ms)), "ms_per_step_median": float(np.median(per_step)),
                        "ms_per_step_min": float(per_step.min()), "ms_per_step_max": float(per_step.max()),
                        "ms_per_step_p10": float(np.percentile(per_step, 10)),
                        "ms_per_step_p90": float(np.percentile(per_step, 90))},
            "verified": check["verified"], "max_rel_err": check["max_rel_err"], "verification": check,
            "speedup_vs_cublas_dense": (ms_dense / (ms_med / args.steps)) if ms_dense else None,
            "cublas_dense_ms_per_step": ms_dense,
            "tensor_frac_of_measured_peak": value / world / peaks["bf16_tflops"],
            "step_hbm_frac": step_bytes / (ms_med / args.steps * 1e-3) / 1e9 / peaks["hbm_gbs"],
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": achieved / peaks["hbm_gbs"], "traffic": traffic, "peak_source": peaks["source"],
                         "kernel": "masked_gemm_kernel", "bytes_per_launch": bytes_launch,
                         "us_per_launch": t_launch * 1e6},
            "cpu_baseline": cpu,
            "mask_build": mask_build,
            "grouped_single_launch": grouped,
            "e2e": e2e,
            "gpu_launches": len(GEMMS) * args.steps * int(len(ms)),
            "clocks": clocks,
            "per_gemm": per_gemm,
        }
        if sharded is not None:
            line["tile_sharded"] = sharded
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
# Tile-sharded square layer (strong scaling over the GPUs of one box)
# ------------------------------------------------------------------------------------------------
def square_layer(n: int, device):
    """M = N = K = n, tile-wise 75 % with per-tile kept-row counts ~ Beta(2,5), seeded."""
    import torch
    from tilesparsity_b200 import synth
    from tilesparsity_b200.tiles import tiles_from_lists
    nt = (n + G - 1) // G
    counts = synth.beta_skewed_counts(n, nt, 1 - SPARSITY / 100.0, 5000 + int(np.log2(n)))
    g = synth.rng(5000 + int(np.log2(n)))
    lists = [np.sort(g.choice(n, size=int(c), replace=False)).astype(np.int32) for c in counts]
    ts = tiles_from_lists(n, n, G, lists)
    gen = torch.Generator(device=device).manual_seed(1234)
    W = torch.randn((n, n), generator=gen, device=device, dtype=torch.float32)
    return ts, W, gen


def sharded_outputs_match(n: int, device, rank: int, world: int) -> dict:
    """On a small square: the gathered and re-assembled output of the tile-sharded layer, by NCCL
    and by the fused epilogue stores (twice in a row on the same buffer), must equal the unsharded
    layer's output bit for bit on every rank."""
    import torch
    import torch.distributed as dist
    from tilesparsity_b200 import TWLayer, sharding
    ts, W, gen = square_layer(n, device)
    At = torch.randn((n, n), generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16)
    full = TWLayer(ts, torch.bfloat16, device)
    full.pack(W)
    ref = full.masked_gemm(At)
    shard = sharding.ShardedTWLayer(W, ts, rank, world, torch.bfloat16)
    ok_nccl = torch.equal(shard.assemble(shard.all_gather(shard.masked_gemm(At))), ref)
    buf, handle = shard.make_gather_buffer(n)
    ok_fused = True
    for scale in (1.0, 0.5):
        out = shard.masked_gemm_allgather(At * scale, buf, handle)
        ok_fused = ok_fused and torch.equal(shard.assemble(out), full.masked_gemm(At * scale))
    has_mc = shard.has_multicast(handle)
    ok_mc = True
    if has_mc:
        for scale in (2.0, 1.0):
            out = shard.masked_gemm_allgather(At * scale, buf, handle, multicast=True)
            ok_mc = ok_mc and torch.equal(shard.assemble(out), full.masked_gemm(At * scale))
    torch.cuda.synchronize()
    flags = torch.tensor([int(ok_nccl), int(ok_fused), int(ok_mc), int(has_mc)], device=device)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    full.close()
    shard.close()
    del buf, handle
    return {"nccl": bool(flags[0].item()), "fused": bool(flags[1].item()),
            "fused_multicast": bool(flags[2].item()) if flags[3].item() else None, "size": n}


def tile_sharded_block(args, device, rank: int, world: int, n: int = 16384, steps: int = 20):
    import torch
    import torch.distributed as dist
    from tilesparsity_b200 import TWLayer, sharding
    check = sharded_outputs_match(2048, device, rank, world)
    ts, W, gen = square_layer(n, device)
    shard = sharding.ShardedTWLayer(W, ts, rank, world, torch.bfloat16)
    one_gpu_ms = None
    n_sets = 2
    At = [torch.randn((n, n), generator=gen, device=device, dtype=torch.float32).to(torch.bfloat16) for _ in range(n_sets)]
    if rank == 0:
        full_layer = TWLayer(ts, torch.bfloat16, device)
        full_layer.pack(W)
        Cfull = torch.zeros((n, n), dtype=torch.bfloat16, device=device)
        one_gpu_ms = float(np.median(timed_repeats(lambda i: full_layer.masked_gemm(At[i % n_sets], out=Cfull),
                                                   steps, 3, 3))) / steps
        full_layer.close()
        del Cfull
    del W
    torch.cuda.empty_cache()
    dist.barrier()
    Ct = [torch.zeros((shard.plan.n_pad, n), dtype=torch.bfloat16, device=device) for _ in range(n_sets)]
    full = torch.empty((world * shard.plan.n_pad, n), dtype=torch.bfloat16, device=device)
    buf, handle = shard.make_gather_buffer(n)

    def run(mode):
        def step(i):
            s = i % n_sets
            if mode in ("fused", "fused_mc"):
                shard.masked_gemm_allgather(At[s], buf, handle, multicast=(mode == "fused_mc"))
                return
            shard.masked_gemm(At[s], out=Ct[s])
            if mode == "nccl":
                dist.all_gather_into_tensor(full, Ct[s])
        ms = max_over_ranks(timed_repeats(step, steps, 3, 5, dist.barrier), device, world)
        return float(np.median(ms)) / steps

    t_none, t_fused, t_nccl = run("none"), run("fused"), run("nccl")
    t_mc = run("fused_mc") if (check["fused_multicast"] is not None) else None
    shard.layer.check()
    kept = ts.kept_flops_per_row() * n
    out_bytes = int(sum(shard.plan.n_local)) * n * 2
    inbound = out_bytes * (world - 1) / world
    res = None
    if rank == 0:
        res = {"workload": f"square_{n}_tw75_g{G}_beta25", "dtype": "bf16", "scaling": "strong", "steps": steps,
               "one_gpu_ms": one_gpu_ms, "none_ms": t_none, "fused_ms": t_fused, "nccl_ms": t_nccl,
               "efficiency_none": one_gpu_ms / (world * t_none), "efficiency_fused": one_gpu_ms / (world * t_fused),
               "efficiency_nccl": one_gpu_ms / (world * t_nccl),
               "kept_tflops_none": kept / (t_none * 1e-3) / 1e12, "kept_tflops_fused": kept / (t_fused * 1e-3) / 1e12,
               "shard_balance": round(shard.plan.balance(), 4),
               "gather_inbound_bytes_per_gpu": int(inbound),
               "gather_floor_ms_at_770GBs": inbound / 770e9 * 1e3,
               "fused_frac_of_nvlink_floor": (inbound / 770e9 * 1e3) / t_fused,
               "fused_multicast_ms": t_mc,
               "efficiency_fused_multicast": (one_gpu_ms / (world * t_mc)) if t_mc else None,
               "fused_multicast_frac_of_nvlink_floor": ((inbound / 770e9 * 1e3) / t_mc) if t_mc else None,
               "binding": "with the gather: inbound bytes per GPU over NVLink; without: tensor cores / L2",
               "verified": bool(check["nccl"] and check["fused"] and check["fused_multicast"] is not False),
               "verification": check,
               "l2": f"activations rotate over {n_sets} buffers of {n * n * 2 / 2**20:.0f} MiB"}
    shard.close()
    return res


def run_square(args):
    """`--workload square`: one configuration of the tile-sharded strong-scaling run as a line of its
    own (M = N = K = --size, --gather none|nccl|fused); at one GPU the unsharded layer."""
    import torch
    import torch.distributed as dist
    from tilesparsity_b200 import sharding

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
    check = sharded_outputs_match(min(n, 2048), device, rank, world) if world > 1 else None
    ts, W, gen = square_layer(n, device)
    shard = sharding.ShardedTWLayer(W, ts, rank, world, torch.bfloat16)
    Wt = W.t().contiguous().to(torch.bfloat16) if world == 1 else None    # for the cuBLAS dense line
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
    sampler.start()
    ms = max_over_ranks(timed_repeats(step, args.steps, max(3, args.warmup), 7, barrier), device, world)
    clocks = sampler.stop()
    shard.layer.check()
    ms_med = float(np.median(ms))
    kept = ts.kept_flops_per_row() * n
    value = kept * args.steps / (ms_med * 1e-3) / 1e12
    dense_ms = None
    if Wt is not None:
        Cd = torch.empty((n, n), dtype=torch.bfloat16, device=device)
        dense_ms = float(np.median(timed_repeats(lambda i: torch.matmul(Wt, At[i % n_sets], out=Cd), args.steps,
                                                 max(3, args.warmup), 5))) / args.steps
    if rank == 0:
        peaks = load_peaks()
        line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
                "warmup": max(3, args.warmup), "ms_per_step": ms_med / args.steps, "higher_is_better": True,
                "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": f"square_{n}_tw75_g{G}_beta25", "gather": args.gather,
                           "parallelism": f"tile-sharded x{world}", "shard_balance": round(shard.plan.balance(), 4),
                           "l2": f"activations rotate over {n_sets} buffers of {n * n * 2 / 2**20:.0f} MiB"},
                "tensor_frac_of_measured_peak": value / world / peaks["bf16_tflops_sustained"],
                "cublas_dense_ms_per_step": dense_ms,
                "speedup_vs_cublas_dense": (dense_ms / (ms_med / args.steps)) if dense_ms else None,
                "verified": None if check is None else bool(check["nccl"] and check["fused"]),
                "gpu_launches": args.steps * len(ms), "clocks": clocks}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


# ------------------------------------------------------------------------------------------------
# The other benchmark configurations on one GPU: one JSON line per row
# ------------------------------------------------------------------------------------------------
def sweep_case(name, M, K, N, dtype, layer_fn, iters, note="", w_scale=0.02, relu_inputs=False):
    import torch
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev).manual_seed(sum(name.encode()) + K + N)
    W = torch.randn((K, N), generator=gen, device=dev, dtype=torch.float32) * w_scale
    layer, kept_flops_per_row, extra = layer_fn(W)
    per_set = (K * M + N * M) * 2
    n_sets = int(max(2, min(8, (2 * L2_BYTES) // per_set + 1)))
    At = []
    for _ in range(n_sets):
        a = torch.randn((K, M), generator=gen, device=dev, dtype=torch.float32)
        At.append((a.clamp_min(0) if relu_inputs else a).to(dtype))
    Ct = [torch.zeros((N, M), dtype=dtype, device=dev) for _ in range(n_sets)]
    Wt = W.t().contiguous().to(dtype)
    steps = max(n_sets, iters // n_sets * n_sets)
    t_m = time_us(lambda i: layer.masked_gemm(At[i % n_sets], out=Ct[i % n_sets]), steps, n_sets, n_sets)
    t_d = time_us(lambda i: torch.matmul(Wt, At[i % n_sets], out=Ct[i % n_sets]), steps, n_sets, n_sets)
    kept = kept_flops_per_row * M
    peaks = load_peaks()
    row = {"config": name, "M": M, "K": K, "N": N, "dtype": str(dtype).split(".")[-1], "masked_us": round(t_m, 2),
           "cublas_dense_us": round(t_d, 2), "speedup_vs_cublas_dense": round(t_d / t_m, 3),
           "kept_tflops": round(kept / t_m / 1e6, 1), "dense_tflops": round(2.0 * M * K * N / t_d / 1e6, 1),
           "tensor_frac_of_measured_peak": round(kept / t_m / 1e6 / peaks["bf16_tflops"], 3),
           "kept_fraction": round(kept / (2.0 * M * K * N), 4), "buffer_sets": n_sets, "note": note, **extra}
    print(json.dumps(row), flush=True)
    layer.close()
    return row


def conv_case(name, B, H, W, cin, cout, algo, sparsity, g1, iters, note=""):
    """A 3 x 3 convolution as an implicit masked GEMM (no im2col matrix): input planes packed from NHWC,
    the GEMM over the padded pixel space, the output brought back to NHWC; each part timed, next to
    cuDNN's dense convolution through torch on the same NHWC (channels-last) tensors."""
    import torch
    from tilesparsity_b200 import ConvTWLayer, build_mask, masks
    dev = torch.device("cuda", torch.cuda.current_device())
    gen = torch.Generator(device=dev).manual_seed(3001)
    w = torch.randn((3, 3, cin, cout), generator=gen, device=dev, dtype=torch.float32) * float(np.sqrt(2.0 / (9 * cin)))
    res = build_mask(algo, masks.img2col_forward([w]), sparsity, G, g1)
    layer = ConvTWLayer(w, res.tiles[0], torch.bfloat16)
    n_sets = 4
    xs = [torch.randn((B, H, W, cin), generator=gen, device=dev, dtype=torch.float32).clamp_min(0).to(torch.bfloat16)
          for _ in range(n_sets)]
    planes, geo = layer.pack_input(xs[0])
    pl = [planes] + [torch.empty_like(planes) for _ in range(n_sets - 1)]
    cts = [torch.zeros((cout, geo["m_padded"]), dtype=torch.bfloat16, device=dev) for _ in range(n_sets)]
    ys = [torch.empty((B, H, W, cout), dtype=torch.bfloat16, device=dev) for _ in range(n_sets)]
    for i in range(n_sets):
        layer.pack_input(xs[i], pl[i])
    steps = max(n_sets, iters // n_sets * n_sets)
    t_pack = time_us(lambda i: layer.pack_input(xs[i % n_sets], pl[i % n_sets]), steps, n_sets, n_sets)
    t_gemm = time_us(lambda i: layer.masked_conv(pl[i % n_sets], geo, out=cts[i % n_sets]), steps, n_sets, n_sets)
    t_unpack = time_us(lambda i: layer.unpack_output(cts[i % n_sets], geo, ys[i % n_sets]), steps, n_sets, n_sets)
    # inside a chain of convolutions the input comes from the previous layer's padded-space output
    # (ts_conv_repack) and the output stays there: neither pack nor unpack
    chain_ok = cin == cout
    t_repack = t_chain = None
    if chain_ok:
        t_repack = time_us(lambda i: layer.repack_input(cts[i % n_sets], geo, pl[(i + 1) % n_sets]), steps, n_sets, n_sets)

        def chained(i):
            s = i % n_sets
            layer.repack_input(cts[s], geo, pl[s])
            layer.masked_conv(pl[s], geo, out=cts[(s + 1) % n_sets])
        t_chain = time_us(chained, steps, n_sets, n_sets)
        for i in range(n_sets):
            layer.pack_input(xs[i], pl[i])

    def whole(i):
        s = i % n_sets
        layer.pack_input(xs[s], pl[s])
        layer.masked_conv(pl[s], geo, out=cts[s])
        layer.unpack_output(cts[s], geo, ys[s])
    t_all = time_us(whole, steps, n_sets, n_sets)
    # dense convolution by cuDNN on channels-last tensors (the same memory layout as NHWC)
    xc = [x.permute(0, 3, 1, 2) for x in xs]
    wc = w.permute(3, 2, 0, 1).contiguous(memory_format=torch.channels_last).to(torch.bfloat16)
    t_dense = time_us(lambda i: torch.nn.functional.conv2d(xc[i % n_sets], wc, padding=1), steps, n_sets, n_sets)
    kept = res.tiles[0].kept_flops_per_row() * B * H * W
    alg = layer.algorithmic_bytes(B, H, W)
    peaks = load_peaks()
    row = {"config": name, "B": B, "H": H, "W": W, "cin": cin, "cout": cout, "dtype": "bfloat16",
           "pack_us": round(t_pack, 2), "gemm_us": round(t_gemm, 2), "unpack_us": round(t_unpack, 2),
           "conv_us": round(t_all, 2), "cudnn_dense_us": round(t_dense, 2), "speedup_vs_cudnn_dense": round(t_dense / t_all, 3),
           "repack_us": round(t_repack, 2) if t_repack else None,
           "chained_conv_us": round(t_chain, 2) if t_chain else None,
           "chained_speedup_vs_cudnn_dense": round(t_dense / t_chain, 3) if t_chain else None,
           "kept_tflops": round(kept / t_all / 1e6, 1), "kept_tflops_gemm_only": round(kept / t_gemm / 1e6, 1),
           "algorithmic_bytes": alg, "gbs_on_algorithmic_bytes": round(alg / t_all / 1e3, 1),
           "padded_pixels_over_pixels": round(geo["m_padded"] / (B * H * W), 3),
           "tensor_frac_of_measured_peak": round(kept / t_all / 1e6 / peaks["bf16_tflops"], 3),
           "kept_fraction": round(kept / (2.0 * B * H * W * 9 * cin * cout), 4), "tiles": res.tiles[0].n_tiles, "note": note}
    print(json.dumps(row), flush=True)
    layer.close()
    return row


def run_sweep(args):
    """The benchmark configurations other than the headline, and the perf driver's own shapes."""
    import torch
    from tilesparsity_b200 import TEWLayer, TWLayer, build_mask, synth
    torch.cuda.set_device(0)
    want = args.workload

    def tw_layer(sparsity, dtype, algo="tw1", g1=None):
        def fn(W):
            res = build_mask(algo, [W.abs()], sparsity, G, g1)
            layer = TWLayer(res.tiles[0], dtype, W.device)
            layer.pack(W)
            return layer, res.tiles[0].kept_flops_per_row(), {"tiles": res.tiles[0].n_tiles}
        return fn

    if want == "bert_sweep":
        for sp in (50.0, 75.0, 90.0):
            for nm, (K, N) in synth.BERT_BASE_LAYER.items():
                sweep_case(f"bert_{nm}_tw{int(sp)}", M_ROWS, K, N, torch.float16, tw_layer(sp, torch.float16), args.iters)
        for nm in ("ffn1", "ffn2"):
            K, N = synth.BERT_BASE_LAYER[nm]
            sweep_case(f"bert_{nm}_type2_75", M_ROWS, K, N, torch.float16, tw_layer(75.0, torch.float16, "bert_type2"),
                       args.iters, "per-tile percentile: equal kept rows per tile")
    elif want == "vgg":
        he = float(np.sqrt(2.0 / 4608))
        sweep_case("vgg16_conv5_tw2_75", 12544, 4608, 512, torch.bfloat16, tw_layer(75.0, torch.bfloat16, "tw2"),
                   args.iters, "tw2 at 75 %: 50 % of columns x 50 % of rows per tile; GEMM over an im2col-sized matrix",
                   he, True)
        sweep_case("vgg16_conv5_c10_k75", 12544, 4608, 512, torch.bfloat16,
                   tw_layer(75.0, torch.bfloat16, "tw_cols_rows", 10.0), args.iters,
                   "10 % of columns pruned, then 75 % of the rows of every tile; GEMM over an im2col-sized matrix",
                   he, True)
        conv_case("vgg16_conv5_implicit_tw2_75", 64, 14, 14, 512, 512, "tw2", 75.0, None, args.iters,
                  "the convolution itself: NHWC in, NHWC out, no im2col matrix")
        conv_case("vgg16_conv5_implicit_c10_k75", 64, 14, 14, 512, 512, "tw_cols_rows", 75.0, 10.0, args.iters,
                  "the convolution itself: NHWC in, NHWC out, no im2col matrix")
    elif want == "lstm":
        def tew(W):
            res = build_mask("tw1m", [W.abs()], 75.0, G, 1.5, want_residual=True)
            layer = TEWLayer(W, res.tiles[0], res.residuals[0], torch.float16)
            return layer, res.tiles[0].kept_flops_per_row() + 2 * layer.nnz, {"residual_nnz": layer.nnz}
        sweep_case("nmt_lstm_tew_75_1.5", 6400, 2048, 4096, torch.float16, tew, args.iters, "", 0.0577)
        sweep_case("nmt_lstm_tw1_75", 6400, 2048, 4096, torch.float16, tw_layer(75.0, torch.float16), args.iters, "", 0.0577)
    elif want == "masks":
        for algo, K, N, sp, g1 in [("tw1", 768, 3072, 75.0, None), ("tw1", 2048, 4096, 75.0, None),
                                    ("tw1", 8192, 8192, 75.0, None), ("tw2", 4608, 512, 75.0, None),
                                    ("tw2", 8192, 8192, 75.0, None), ("tw1m", 2048, 4096, 75.0, 1.5)]:
            dev = torch.device("cuda", 0)
            gen = torch.Generator(device=dev).manual_seed(K * 31 + N)
            W = (torch.randn((K, N), generator=gen, device=dev, dtype=torch.float32) * 0.02).abs()
            build_mask(algo, [W], sp, G, g1)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            reps = 5
            for _ in range(reps):
                res = build_mask(algo, [W], sp, G, g1)
            torch.cuda.synchronize()
            dt = (time.perf_counter() - t0) / reps
            passes = {"tw1": 1, "tw2": 2, "tw1m": 2, "tw2m": 3}[algo]
            nbytes = K * N * (4 * passes + 1)
            print(json.dumps({"config": f"mask_{algo}_{K}x{N}", "K": K, "N": N, "sparsity": sp, "seconds": round(dt, 6),
                              "bytes": nbytes, "gbs": round(nbytes / dt / 1e9, 1),
                              "density": round(float(res.masks[0].float().mean()), 4)}), flush=True)
    elif want == "readme":
        # the shapes the reference's README quotes for a V100 (StreamMaskedGEMM/README.md:14-27):
        # M = 12800, 768 / 3072 wide, half of the columns and half of the rows kept
        from tilesparsity_b200 import stream_gemm
        for M, N, K, Np, Kp in [(12800, 768, 768, 384, 384), (12800, 3072, 768, 1536, 384), (12800, 768, 3072, 384, 1536)]:
            r = stream_gemm.run(M, N, K, Np, Kp, torch.float16, iters=100, out=sys.stderr)
            print(json.dumps({"config": f"readme_{M}x{N}x{K}_{Np}_{Kp}", **{k: r[k] for k in
                              ("M", "N", "K", "N_pruned", "K_pruned", "dense_us", "stream_us", "speedup", "kept_tflops",
                               "errors", "errors_reference_rule")}}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--masks", choices=["tw1", "random"], default="tw1",
                    help="tw1: the reference's tile-wise masks of the synthetic weights, built on the GPU; "
                         "random: the perf driver's random per-tile row subsets")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from the host instead of replaying a CUDA graph")
    ap.add_argument("--workload", choices=["bert", "square", "bert_sweep", "vgg", "lstm", "masks", "readme"], default="bert",
                    help="bert: the headline BERT-base layer step; square: tile-sharded M=N=K=--size strong scaling; "
                         "the others: further benchmark configurations on one GPU, one JSON line per row")
    ap.add_argument("--size", type=int, default=16384)
    ap.add_argument("--iters", type=int, default=200, help="timed launches per row of the single-GPU sweeps")
    ap.add_argument("--gather", choices=["none", "nccl", "fused"], default="none",
                    help="square workload: all-gather Ct inside the timed region, with NCCL after the GEMM or "
                         "by the GEMM's epilogue storing into the peers' buffers")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    elif args.workload == "square":
        if args.steps == 200:
            args.steps = 20
        run_square(args)
    elif args.workload == "bert":
        run_ours(args)
    else:
        run_sweep(args)


if __name__ == "__main__":
    main()
