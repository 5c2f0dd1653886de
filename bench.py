"""Benchmark of the B200 execution path on the reference's headline configurations.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c2|c5|c1] [--impl reference]

A step is one pass of the hot path over one batch of seeded synthetic input.  The default
workload is ResNet-50 v1.5, f32 graph, batch 32 (TF32 tensor-core contractions); `c5` is the
QLinearConv INT8 ResNet-50 at a global batch of 1024 split over the GPUs of the run, `c1` the INT8 MLP, `c3` the InSwapper-shaped f32
generator at batch 16, `c4` the BERT-base-shaped dynamic-INT8 encoder at 64 x 128 tokens (tokens/s).  With N > 1 (launched by
torchrun, one rank per GPU) every rank holds a full weight replica and runs its own batch:
the path shards along the batch only, there is no data-path collective; the scaling is weak (per-GPU
batch fixed) except for `c5`, whose global batch is fixed (strong).

One JSON line is printed by rank 0:
  value      images/s (rows/s for c1) with inputs resident in HBM, device time from CUDA events on
             the launching stream, max over ranks; L2 is flushed between timed steps
  e2e        the same metric through the public call (oxb200_run) with pinned HOST buffers:
             host-to-device copy of the batch, the run, device-to-host copy of the result
  roofline   the tensor-core contraction kernel: algorithmic ops of its launches / their summed
             CUDA-event durations, against the measured peak
  cpu_baseline  the CPU oracle (a port of the reference's CPU operators) timed on this host's
             cores on a bounded sample of the same workload
  int8       (default workload, one GPU) the INT8 half of the headline metric measured in the same run:
             the QLinearConv ResNet-50 at batch 1024, images/s and the contraction kernel's TOP/s
             against twice the measured bf16 rate

`--impl reference` times that CPU port alone on all host threads (the reference itself is a Rust
project and cannot be built in this environment).
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

WORKLOADS = {
    "c2": dict(name="resnet50_v1.5_f32_b32", metric="images_per_s", unit="images/s", dtype="tf32", batch=32),
    # global batch 1024 split over the GPUs of the run (BASELINE.json configs[4]): 1024 / N images per GPU
    "c5": dict(name="resnet50_qlinearconv_int8_b1024_global", metric="images_per_s", unit="images/s", dtype="i8", batch=1024, global_batch=True),
    "c1": dict(name="int8_mlp_64x1024-4096-4096-1024", metric="rows_per_s", unit="rows/s", dtype="i8", batch=64),
    "c3": dict(name="inswapper128_shaped_f32_b16", metric="images_per_s", unit="images/s", dtype="tf32", batch=16),
    "c4": dict(name="bert_base_dynamic_int8_b64_s128", metric="tokens_per_s", unit="tokens/s", dtype="i8", batch=64, per_item=128),
}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return dict(hbm_gbs=p["hbm_gbs"], bf16=p["bf16_tflops"], bf16_sustained=p["bf16_tflops_sustained"], source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


# DRAM bytes (read + written) per launch of the tensor-core kernel, averaged over the launches of one
# step: dram__bytes_read.sum + dram__bytes_write.sum from the ncu launch lists summarised under profiles/
# (launch_list_resnet50_f32_b32.md, launch_list_resnet50_int8_b1024.md).  None: not captured.
NCU_TRAFFIC_PER_LAUNCH = {"c2": 43.35e6, "c5": 351.83e6, "c1": None, "c3": None, "c4": None}


def build_workload(key, batch):
    from oxionnx_b200 import models
    if key == "c2":
        return models.build_resnet50_f32(batch=batch)
    if key == "c5":
        return models.build_resnet50_qlinear(batch=batch)
    if key == "c3":
        return models.build_inswapper_f32(batch=batch)
    if key == "c4":
        return models.build_bert_dynamic_int8(batch=batch)
    return models.build_int8_mlp(rows=batch)


class ClockSampler:
    """nvidia-smi clocks and throttle reasons sampled while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits",
                                          "-lms", "100"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        time.sleep(0.15)
        self.proc.terminate()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ts, line in self.lines:
            if not (t0 - 0.05 <= ts <= t1 + 0.15):
                continue
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 8:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[4:8]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["no samples inside the timed region"])
        return dict(sm_mhz=statistics.median(sm), sm_max_mhz=max(mx), reasons=sorted(reasons), samples=len(sm))


def pinned_array(shape, lib):
    n = int(np.prod(shape))
    ptr = lib.oxb200_host_alloc(n * 4)
    if not ptr:
        raise RuntimeError("pinned allocation failed")
    arr = np.ctypeslib.as_array(ctypes.cast(ptr, ctypes.POINTER(ctypes.c_float)), shape=(n,)).reshape(shape)
    return arr, ptr


def cpu_baseline(key, graph_builder_batch, sample, threads):
    """The CPU oracle on `sample` units of the workload with `threads` host threads."""
    import oracle
    graph, weights, feeds, _ = build_workload(key, sample)
    f = feeds(sample) if key != "c1" else feeds()
    oracle.set_threads(threads)
    oracle.set_float_accum(1)
    t0 = time.time()
    oracle.run_graph(graph, weights, f, keep_all=False)
    dt = time.time() - t0
    oracle.set_float_accum(0)
    oracle.set_threads(1)
    return sample * WORKLOADS[key].get("per_item", 1) / dt, dt


def int8_companion(args, local_rank, flush_l2, peaks):
    """The INT8 half of the headline metric, measured in the same run: the QLinearConv ResNet-50 at batch
    1024 (the configuration's global batch on one GPU), inputs resident, L2 flushed between steps; images/s
    and the contraction kernel's TOP/s."""
    from oxionnx_b200.session import Session
    key = "c5"
    w = WORKLOADS[key]
    batch = w["batch"]
    graph, weights, feeds, info = build_workload(key, batch)
    sess = Session.builder().with_device(local_rank).with_profiling(True).with_kernel_path(args.kernel_path).with_cuda_graph(args.cuda_graph != 0).build_from_graph(graph, weights)
    sess.upload(feeds(batch, "c5_companion"))
    for _ in range(3):
        sess.run_resident(1)
    steps = min(args.steps, 10)
    sess.ctx.set_profiling(False)
    total_ms = 0.0
    for _ in range(steps):
        flush_l2()
        total_ms += sess.run_resident(1)
    sess.ctx.set_profiling(True)
    conv_ms, conv_ops = 0.0, 0.0
    for _ in range(steps):
        flush_l2()
        sess.run_resident(1)
        for s in sess.steps():
            if s["ms"] >= 0 and s["kernel"].startswith("umma"):
                conv_ms += s["ms"]
                conv_ops += s["work"]
    sess.close()
    tops = conv_ops / (conv_ms / 1000.0) / 1e12 if conv_ms > 0 else 0.0
    peak = 2.0 * peaks["bf16_sustained"]
    return {"workload": w["name"], "value": batch * steps / (total_ms / 1000.0), "unit": "images/s", "steps": steps, "ms_per_step": total_ms / steps,
            "contraction_tops": tops, "peak_tops": peak, "frac": tops / peak, "peak_basis": f"2 x bf16_tflops_sustained of {peaks['source']}",
            "traffic": NCU_TRAFFIC_PER_LAUNCH[key]}


def run_reference(args, rank, world):
    """The reference arm: the CPU port of the reference's operators, all host threads."""
    if rank != 0:
        return
    w = WORKLOADS[args.workload]
    cores = os.cpu_count() or 1
    sample = {"c2": 2, "c5": 1, "c1": 64, "c3": 1, "c4": 1}[args.workload]
    times = []
    for i in range(args.warmup + args.steps):
        v, dt = cpu_baseline(args.workload, w["batch"], sample, cores)
        if i >= args.warmup:
            times.append(dt)
        if sum(times) > 150:
            break
    steps = len(times)
    value = sample * w.get("per_item", 1) * steps / sum(times)
    line = {
        "impl": "reference", "metric": w["metric"], "value": value, "unit": w["unit"], "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup,
        "ms_per_step": 1000.0 * sum(times) / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32" if args.workload in ("c2", "c3") else "i64",
        "data": "synthetic", "config": {"workload": w["name"], "sample": f"{sample} {w['unit'].split('/')[0]} per step"},
        "cpu_baseline": {"value": value, "unit": w["unit"], "cores": cores, "kind": "port",
                         "sample": f"{sample} {w['unit'].split('/')[0]} per step through the CPU oracle; the Rust reference cannot be built here"},
        "e2e": {"value": value, "unit": w["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=0, help="per-GPU batch (default: the configuration's)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-int8", action="store_true", help="skip the INT8 ResNet-50 companion measurement of the default workload")
    ap.add_argument("--kernel-path", default="auto", choices=["auto", "direct"])
    ap.add_argument("--cuda-graph", type=int, default=-1,
                    help="1: replay the planned step list as one CUDA graph (OXIONNX_CUDA_GRAPH); default: on, except for the six-launch MLP "
                         "(c1), where a graph launch costs more than the launches it replaces")
    args = ap.parse_args()
    if args.cuda_graph < 0:
        args.cuda_graph = 0 if args.workload == "c1" else 1
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return

    dist = None
    torch = None
    if world > 1:
        import torch
        import torch.distributed as dist
        torch.cuda.set_device(local_rank)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from oxionnx_b200 import _ffi
    from oxionnx_b200.session import Session
    lib = _ffi.lib()
    w = WORKLOADS[args.workload]
    batch = args.batch or (max(w["batch"] // world, 1) if w.get("global_batch") else w["batch"])
    graph, weights, feeds, info = build_workload(args.workload, batch)
    f = feeds(batch, f"{args.workload}_in_rank{rank}") if args.workload != "c1" else feeds()
    sess = Session.builder().with_device(local_rank).with_profiling(True).with_kernel_path(args.kernel_path).with_cuda_graph(args.cuda_graph != 0).build_from_graph(graph, weights)

    # pinned host staging for the end-to-end leg
    feeds_pinned, pinned_ptrs = {}, []
    for in_name in graph.input_names:
        host_in, in_ptr = pinned_array(f[in_name].shape, lib)
        host_in[...] = f[in_name]
        feeds_pinned[in_name] = host_in
        pinned_ptrs.append(in_ptr)
    sess.ensure_planned(feeds_pinned)

    # L2 flush between timed steps: a 256 MiB memset (L2 is 126 MB)
    import torch
    torch.cuda.set_device(local_rank)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=f"cuda:{local_rank}")

    def flush_l2():
        flush.zero_()
        torch.cuda.synchronize()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident leg ----
    sess.upload(feeds_pinned)
    for _ in range(args.warmup):
        sess.run_resident(1)
    c0 = sess.cuda_cache_counters()
    sampler = ClockSampler(int(os.environ.get("CUDA_VISIBLE_DEVICES", "").split(",")[local_rank]) if os.environ.get("CUDA_VISIBLE_DEVICES") else local_rank)
    if rank == 0:  # one sampler per job: eight nvidia-smi loops would compete with the ranks' launch threads
        sampler.start()
    barrier()
    t_begin = time.time()
    # the timed K steps run without per-kernel events (an event record between two launches keeps the second
    # from being scheduled while the first drains) ...
    sess.ctx.set_profiling(False)
    step_ms = []
    for _ in range(args.steps):
        flush_l2()
        step_ms.append(sess.run_resident(1))
    c1 = sess.cuda_cache_counters()
    # ... and the same K steps again with a CUDA-event pair around every kernel, for the roofline figures
    sess.ctx.set_profiling(True)
    prof_ms = 0.0
    conv_ms, conv_ops, conv_launches = 0.0, 0.0, 0
    glue_ms, glue_bytes = 0.0, 0.0
    for _ in range(args.steps):
        flush_l2()
        prof_ms += sess.run_resident(1)
        for s in sess.steps():
            if s["ms"] < 0:
                continue
            if s["kernel"].startswith("umma"):
                conv_ms += s["ms"]
                conv_ops += s["work"]
                conv_launches += 1
            elif s["work_is_bytes"]:
                glue_ms += s["ms"]
                glue_bytes += s["work"]
    barrier()
    t_end = time.time()
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None
    sess.ctx.set_profiling(False)
    total_ms = sum(step_ms)
    if dist is not None:
        t = torch.tensor([total_ms], dtype=torch.float64, device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    per_item = w.get("per_item", 1)  # tokens per sequence for the encoder, 1 otherwise
    value = world * batch * per_item * args.steps / (total_ms / 1000.0)

    # ---- end-to-end leg: pinned host buffers through the public pipelined call (submit / collect): every step
    # uploads its inputs from pinned host memory and reads its result back; the upload of step i+1 overlaps
    # the run of step i.  Timed on the host from the first submit to the last collect, inside barriers.
    out = sess.run(feeds_pinned)
    sess.run_pipelined([feeds_pinned] * 3)
    barrier()
    t0 = time.perf_counter()
    pending = 0
    for _ in range(args.steps):
        sess.submit(feeds_pinned)
        pending += 1
        if pending == 2:
            out = sess.collect()
            pending -= 1
    while pending:
        out = sess.collect()
        pending -= 1
    if torch.cuda.is_available():
        torch.cuda.synchronize()
    e2e_total = (time.perf_counter() - t0) * 1000.0
    barrier()
    if dist is not None:
        t = torch.tensor([e2e_total], dtype=torch.float64, device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_total = float(t.item())
    e2e_value = world * batch * per_item * args.steps / (e2e_total / 1000.0)
    h2d = int(sum(v.size for v in feeds_pinned.values()) * 4)
    d2h = int(sum(v.size for v in out.values()) * 4)

    if rank == 0:
        peaks = measured_peaks()
        kind = w["dtype"]
        # TF32 runs at half, INT8 at twice the measured dense bf16 rate (architectural ratios); the kernels
        # are timed inside a long step, so the sustained figure is the denominator.
        factor = {"tf32": 0.5, "i8": 2.0}[kind]
        peak = peaks["bf16_sustained"] * factor
        achieved = (conv_ops / (conv_ms / 1000.0) / 1e12) if conv_ms > 0 else 0.0
        roofline = {
            "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TOP/s" if kind == "i8" else "TFLOP/s",
            "frac": achieved / peak if peak else None, "traffic": NCU_TRAFFIC_PER_LAUNCH.get(args.workload),
            "traffic_note": "DRAM bytes per launch from the committed ncu launch list (profiles/), not measured in this run",
            "kernel": "umma_conv_kernel (tcgen05 implicit GEMM)", "launches_per_step": conv_launches // max(args.steps, 1),
            "avg_launch_ms": conv_ms / max(conv_launches, 1), "share_of_step": conv_ms / prof_ms if prof_ms > 0 else None,
            "timed_in": "a second pass of the same K steps with a CUDA-event pair around every kernel (ms_per_step %.3f there)" % (prof_ms / max(args.steps, 1)),
            "peak_basis": f"{factor} x bf16_tflops_sustained of {peaks['source']} ({peaks['bf16_sustained']})",
            "glue_gbs": (glue_bytes / (glue_ms / 1000.0) / 1e9) if glue_ms > 0 else None, "hbm_peak_gbs": peaks["hbm_gbs"],
        }
        line = {
            "metric": w["metric"], "value": value, "unit": w["unit"], "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "strong" if (w.get("global_batch") and not args.batch) else "weak", "vs_baseline": None, "dtype": kind,
            "data": "synthetic",
            "config": {"workload": w["name"], "per_gpu_batch": batch, "global_batch": batch * world, "parallelism": f"batch-sharded replicas x{world}, no collective",
                       "l2": "flushed between timed steps (256 MiB memset)", "algorithmic_ops_per_step": info["ops"], "kernel_path": args.kernel_path,
                       "cuda_graph": bool(args.cuda_graph)},
            "clocks": dict(clocks, window="the timed K steps and the profiled K steps that follow them"),
            "e2e": {"value": e2e_value, "unit": w["unit"], "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "ms_per_step": e2e_total / args.steps,
                    "call": "oxb200_run_submit / oxb200_run_collect, two runs in flight, L2 not flushed between steps (the uploads replace the flush)"},
            "gpu_launches": int(c1["kernel_launches"] - c0["kernel_launches"]),
            "launch_mix": {"umma": int(c1["umma_launches"] - c0["umma_launches"]), "direct": int(c1["simt_launches"] - c0["simt_launches"]),
                           "glue": int(c1["glue_launches"] - c0["glue_launches"])},
            "roofline": roofline,
        }
        if args.workload == "c2" and world == 1 and not args.no_int8:
            line["int8"] = int8_companion(args, local_rank, flush_l2, peaks)
        if not args.no_cpu_baseline and world == 1:
            sample = {"c2": 2, "c5": 1, "c1": 64, "c3": 1, "c4": 1}[args.workload]
            cores = os.cpu_count() or 1
            v, dt = cpu_baseline(args.workload, batch, sample, cores)
            line["cpu_baseline"] = {"value": v, "unit": w["unit"], "cores": cores, "kind": "port",
                                    "sample": f"{sample} {w['unit'].split('/')[0]} through the CPU oracle in {dt:.1f} s"}
        print(json.dumps(line), flush=True)
    for ptr in pinned_ptrs:
        lib.oxb200_host_free(ptr)
    sess.close()
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
