"""Benchmark of the B200 execution path on the reference's headline configurations.

  python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c5|c2|c1|c3|c4] [--impl reference]
  python bench.py --layer "i8|f32 N C H W OC K STRIDE PAD"        (one contraction layer in isolation)
  python bench.py --layer "dql ROWS COLS"                         (DynamicQuantizeLinear of a [ROWS, COLS] activation)

A step is one pass of the hot path over one batch of seeded synthetic input.  The default
workload is `c5`: the QLinearConv INT8 ResNet-50 at a GLOBAL batch of 1024 images split over the
GPUs of the run (1024 / N images per GPU, strong scaling), the configuration the headline metric
("images/s per B200 and on 8 x B200; INT8 TOPS as a fraction of dense peak") is quoted on.  `c2`
is ResNet-50 v1.5 as an f32 graph at batch 32 (TF32 contractions), `c1` the INT8 MLP, `c3` the
InSwapper-shaped f32 generator at batch 16, `c4` the BERT-base-shaped dynamic-INT8 encoder at
64 x 128 tokens (tokens/s); those keep their batch per GPU (weak scaling).  With N > 1 (launched
by torchrun, one rank per GPU) every rank holds a full weight replica and runs its own shard:
the path shards along the batch only, there is no data-path collective.

One JSON line is printed by rank 0:
  value         images/s (rows/s for c1, tokens/s for c4) with inputs resident in HBM, device time from
                CUDA events on the launching stream, max over ranks; L2 is flushed between timed steps
  e2e           the same metric through the public pipelined call (oxb200_run_submit / _collect) with
                pinned HOST buffers: host-to-device copy of the batch, the run, device-to-host copy of
                the result, every step; `e2e_u8_feed` (c5) is the same with the image declared and fed
                as u8 lanes, a quarter of the upload
  roofline      the tensor-core contraction kernel: algorithmic ops of its launches / their summed
                CUDA-event durations, against the measured peak (cuBLAS-derived, and this library's own
                tcgen05 issue-rate probe beside it)
  cpu_baseline  the CPU oracle -- a restatement of the reference's CPU operators, float contractions by
                its im2col + blocked-sgemm algorithm -- timed on this host's cores on a bounded sample
  f32           (default workload, one GPU) ResNet-50 f32 at batch 32 measured in the same run

`--impl reference` times that CPU restatement alone on all host threads (the reference itself is a
Rust project and cannot be built in this environment).
"""
import argparse
import ctypes
import hashlib
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
    # global batch 1024 split over the GPUs of the run: 1024 / N images per GPU
    "c5": dict(name="resnet50_qlinearconv_int8_b1024_global", metric="images_per_s", unit="images/s", dtype="i8", batch=1024, global_batch=True),
    "c2": dict(name="resnet50_v1.5_f32_b32", metric="images_per_s", unit="images/s", dtype="tf32", batch=32),
    "c1": dict(name="int8_mlp_64x1024-4096-4096-1024", metric="rows_per_s", unit="rows/s", dtype="i8", batch=64),
    "c3": dict(name="inswapper128_shaped_f32_b16", metric="images_per_s", unit="images/s", dtype="tf32", batch=16),
    "c4": dict(name="bert_base_dynamic_int8_b64_s128", metric="tokens_per_s", unit="tokens/s", dtype="i8", batch=64, per_item=128),
}
# units the CPU baseline runs per sample (about 10-30 s of CPU work each)
CPU_SAMPLE = {"c2": 4, "c5": 8, "c1": 64, "c3": 1, "c4": 1}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            p = json.load(fh)
        return dict(hbm_gbs=p["hbm_gbs"], bf16=p["bf16_tflops"], bf16_sustained=p["bf16_tflops_sustained"], source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


def kernel_source_sha():
    """Identity of the tensor-core kernel sources: recorded next to captured DRAM traffic, so that a figure taken
    from another version of the kernel is not reported for this one."""
    h = hashlib.sha256()
    csrc = os.path.join(ROOT, "oxionnx_b200", "csrc")
    for name in ("umma_kernel.cuh", "umma_launch.cuh", "kernels_umma.cu", "umma_i8.cu", "umma_tf32.cu", "umma_f16.cu"):
        with open(os.path.join(csrc, name), "rb") as fh:
            h.update(fh.read())
    return h.hexdigest()[:16]


def captured_traffic(key):
    """DRAM bytes (read + written) per launch of the tensor-core kernel from an ncu capture of this workload, or
    None when no capture exists for the present kernel sources."""
    path = os.path.join(ROOT, "profiles", "traffic.json")
    if not os.path.exists(path):
        return None, "no capture recorded", None
    with open(path) as fh:
        table = json.load(fh)
    rec = table.get(key)
    if not rec:
        return None, "no capture recorded for this workload", None
    if rec.get("kernel_sha16") != kernel_source_sha():
        return None, "the recorded capture is of other kernel sources (%s)" % rec.get("kernel_sha16"), None
    return rec["dram_bytes_per_launch"], rec.get("note", ""), rec.get("batch")


def build_workload(key, batch, typed_input=False):
    from oxionnx_b200 import models
    if key == "c2":
        return models.build_resnet50_f32(batch=batch)
    if key == "c5":
        return models.build_resnet50_qlinear(batch=batch, typed_input=typed_input)
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


def pinned_like(array, lib):
    """A page-locked host copy of `array` (same element type)."""
    ptr = lib.oxb200_host_alloc(max(array.nbytes, 1))
    if not ptr:
        raise RuntimeError("pinned allocation failed")
    ctype = {1: ctypes.c_uint8, 4: ctypes.c_float}[array.dtype.itemsize]
    flat = np.ctypeslib.as_array(ctypes.cast(ptr, ctypes.POINTER(ctype)), shape=(array.size,))
    out = flat.view(array.dtype).reshape(array.shape)
    out[...] = array
    return out, ptr


def cpu_run(key, sample, threads, float_mode=2):
    """The CPU oracle on `sample` units of the workload with `threads` host threads.  Float contractions run the
    reference's algorithm (im2col blocks + blocked sgemm); the integer operators are the reference's loops, split
    over independent outputs when threads > 1 (bit-identical)."""
    import oracle
    graph, weights, feeds, _ = build_workload(key, sample)
    f = feeds(sample) if key != "c1" else feeds()
    oracle.set_threads(threads)
    oracle.set_float_accum(float_mode)
    t0 = time.time()
    oracle.run_graph(graph, weights, f, keep_all=False)
    dt = time.time() - t0
    oracle.set_float_accum(0)
    oracle.set_threads(1)
    return sample * WORKLOADS[key].get("per_item", 1) / dt, dt


def cpu_baseline_record(key, cores):
    """Variant B (every core) as the value; for the integer configurations also variant A, the reference's own
    threading for those operators: one thread."""
    w = WORKLOADS[key]
    sample = CPU_SAMPLE[key]
    unit = w["unit"].split("/")[0]
    v, dt = cpu_run(key, sample, cores)
    rec = {"value": v, "unit": w["unit"], "cores": cores, "kind": "port",
           "variant": "all cores: the reference's arithmetic split over independent outputs" if w["dtype"] == "i8"
                      else "the reference's algorithm and threading: im2col in blocks of at most 64 MiB + blocked sgemm (8x8 FMA tile), jobs or row bands over all cores",
           "sample": f"{sample} {unit} through the CPU oracle in {dt:.1f} s, scaled linearly to the unit"}
    if w["dtype"] == "i8" and key in ("c5", "c1"):
        v1, dt1 = cpu_run(key, sample, 1)
        rec["faithful"] = {"value": v1, "cores": 1, "note": f"the reference runs its integer operators on one thread (naive i64 loops); {sample} {unit} in {dt1:.1f} s"}
    return rec


def run_reference(args, rank):
    """The reference arm: the CPU restatement of the reference's operators, all host threads."""
    if rank != 0:
        return
    w = WORKLOADS[args.workload]
    cores = os.cpu_count() or 1
    sample = CPU_SAMPLE[args.workload]
    times = []
    for i in range(args.warmup + args.steps):
        _, dt = cpu_run(args.workload, sample, cores)
        if i >= args.warmup:
            times.append(dt)
        if sum(times) > 150:
            break
    steps = len(times)
    value = sample * w.get("per_item", 1) * steps / sum(times)
    unit = w["unit"].split("/")[0]
    line = {
        "impl": "reference", "metric": w["metric"], "value": value, "unit": w["unit"], "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup,
        "ms_per_step": 1000.0 * sum(times) / steps, "higher_is_better": True, "scaling": "strong" if w.get("global_batch") else "weak", "vs_baseline": None,
        "dtype": "f32" if args.workload in ("c2", "c3") else "i64", "data": "synthetic",
        "config": {"workload": w["name"], "sample": f"{sample} {unit} per step", "same_config": False,
                   "note": "each step is a bounded sample of the workload; the value is per unit, i.e. scaled linearly to the full batch"},
        "cpu_baseline": {"value": value, "unit": w["unit"], "cores": cores, "kind": "port",
                         "sample": f"{sample} {unit} per step through the CPU oracle (float contractions: the reference's im2col + blocked-sgemm algorithm; "
                                   "integer operators: its loops split over the cores); the Rust reference cannot be built here"},
        "e2e": {"value": value, "unit": w["unit"], "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_layer(spec, iters, pairs):
    """One contraction layer between two cheap glue nodes, so that its operands are device-resident activations as
    inside a network; prints the kernel the planner chose, its best CUDA-event time and the algorithmic rate."""
    from oxionnx_b200.graph import Graph, Node
    from oxionnx_b200.session import Session
    kind = spec[0]
    if kind == "dql":  # "dql ROWS COLS": DynamicQuantizeLinear of a [ROWS, COLS] activation
        rows, cols = int(spec[1]), int(spec[2])
        nodes = [Node("Relu", "pre", ["x"], ["x1"], {}), Node("DynamicQuantizeLinear", "dq", ["x1"], ["y", "s", "z"], {})]
        sess = Session.builder().with_profiling(True).build_from_graph(Graph(nodes=nodes, input_names=["x"], output_names=["s", "z"]), {})
        sess.upload({"x": np.random.default_rng(0).standard_normal((rows, cols)).astype(np.float32)})
        for _ in range(3):
            sess.run_resident(1)
        best = {}
        for _ in range(iters):
            sess.run_resident(1)
            for s in sess.steps():
                if s["node"] == "dq":
                    best[s["kernel"]] = min(best.get(s["kernel"], 1e9), s["ms"])
        for kname, ms in best.items():
            print(f"{kname}: best {ms * 1000:.1f} us  {rows * cols * 4 / (ms / 1e3) / 1e12:.2f} TB/s of input")
        sess.close()
        return
    n, c, h, w, oc, k, stride, pad = [int(a) for a in spec[1:9]]
    rng = np.random.default_rng(0)
    if kind == "f32":
        weights = {"w": (rng.standard_normal((oc, c, k, k)) * 0.05).astype(np.float32), "b": rng.standard_normal(oc).astype(np.float32)}
        nodes = [Node("Relu", "pre", ["x"], ["x1"], {}),
                 Node("Conv", "conv", ["x1", "w", "b"], ["y"], {"strides": [stride, stride], "pads": [pad] * 4, "activation": "relu"}),
                 Node("GlobalAveragePool", "gap", ["y"], ["z"], {})]
        x = rng.standard_normal((n, c, h, w)).astype(np.float32)
    else:
        weights = {"w": rng.integers(-127, 128, (oc, c, k, k)).astype(np.float32), "ws": rng.uniform(0.001, 0.01, oc).astype(np.float32),
                   "wz": np.zeros(oc, np.float32), "b": rng.integers(-1000, 1000, oc).astype(np.float32), "xs": np.float32([0.02]),
                   "z0": np.float32([0]), "ys": np.float32([0.5]), "qs": np.float32([0.02])}
        nodes = [Node("QuantizeLinear", "q", ["x", "qs", "z0"], ["xq"], {}),
                 Node("QLinearConv", "conv", ["xq", "xs", "z0", "w", "ws", "wz", "ys", "z0", "b"], ["yq"],
                      {"strides": [stride, stride], "pads": [pad] * 4}),
                 Node("Relu", "r", ["yq"], ["yr"], {}),
                 Node("DequantizeLinear", "dq", ["yr", "ys", "z0"], ["yd"], {}),
                 Node("GlobalAveragePool", "gap", ["yd"], ["z"], {})]
        x = np.abs(rng.standard_normal((n, c, h, w))).astype(np.float32)
    graph = Graph(nodes=nodes, input_names=["x"], output_names=["z"])
    sess = Session.builder().with_profiling(True).with_tuning(cta_pairs=pairs).build_from_graph(graph, weights)
    sess.upload({"x": x})
    for _ in range(3):
        sess.run_resident(1)
    best, desc, work = 1e9, "", 0.0
    for _ in range(iters):
        sess.run_resident(1)
        for s in sess.steps():
            if s["node"] == "conv" and not s["work_is_bytes"] and 0 <= s["ms"] < best:
                best, desc, work = s["ms"], s["kernel"], s["work"]
    print(f"{desc}: best {best * 1000:.1f} us  {work / (best / 1e3) / 1e12:.1f} T/s")
    sess.close()


def measure(args, key, batch, local_rank, world, dist, torch, lib, flush_l2, barrier, sample_clocks):
    """Device-resident and end-to-end throughput of workload `key` at `batch` units per GPU."""
    from oxionnx_b200.session import Session
    w = WORKLOADS[key]
    rank = int(os.environ.get("RANK", "0"))
    graph, weights, feeds, info = build_workload(key, batch)
    f = feeds(batch, f"{key}_in_rank{rank}") if key != "c1" else feeds()
    graph_on = args.cuda_graph != 0 if args.cuda_graph >= 0 else key != "c1"
    sess = Session.builder().with_device(local_rank).with_profiling(True).with_kernel_path(args.kernel_path).with_cuda_graph(graph_on).build_from_graph(graph, weights)
    pinned, ptrs = {}, []
    for name in graph.input_names:
        pinned[name], ptr = pinned_like(f[name], lib)
        ptrs.append(ptr)
    sess.ensure_planned(pinned)

    # ---- device-resident leg ----
    sess.upload(pinned)
    for _ in range(args.warmup):
        sess.run_resident(1)
    c0 = sess.cuda_cache_counters()
    sampler = None
    if sample_clocks and rank == 0:  # one sampler per job: eight nvidia-smi loops would compete with the ranks' launch threads
        visible = os.environ.get("CUDA_VISIBLE_DEVICES")
        sampler = ClockSampler(int(visible.split(",")[local_rank]) if visible else local_rank)
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
    prof_ms, conv_ms, conv_ops, conv_launches, glue_ms, glue_bytes = 0.0, 0.0, 0.0, 0, 0.0, 0.0
    conv_algo_bytes = 0.0
    conv_layers = []  # (ops, algorithmic bytes) of every contraction launch of one step: the layer-wise bound below
    slowest = {}
    umma_kernels = set()
    for _ in range(args.steps):
        flush_l2()
        prof_ms += sess.run_resident(1)
        for s in sess.steps():
            if s["ms"] < 0:
                continue
            if s["kernel"].startswith("umma"):
                fam0 = s["kernel"].split()[0]
                umma_kernels.add("umma_chain_kernel (cooperative tcgen05 chain of quantised linears)" if fam0 == "umma_i8_chain" else
                                 ("umma_attention_kernel (tcgen05 scores + softmax + context)" if fam0 == "umma_attention" else
                                  "umma_conv_kernel (tcgen05 implicit GEMM)"))
                conv_ms += s["ms"]
                conv_ops += s["work"]
                conv_launches += 1
                conv_algo_bytes += s["bytes"]
                if _ == 0:
                    conv_layers.append((s["work"], s["bytes"]))
            elif s["work_is_bytes"]:
                glue_ms += s["ms"]
                glue_bytes += s["work"]
            fam = s["kernel"].split()[0]
            slowest[fam] = slowest.get(fam, 0.0) + s["ms"]
    barrier()
    t_end = time.time()
    clocks = sampler.stop(t_begin, t_end) if sampler else None
    sess.ctx.set_profiling(False)
    from oxionnx_b200.shard import max_over_ranks
    total_ms = max_over_ranks(sum(step_ms), world, device=f"cuda:{local_rank}")  # the slowest rank's device time
    per_item = w.get("per_item", 1)  # tokens per sequence for the encoder, 1 otherwise
    value = world * batch * per_item * args.steps / (total_ms / 1000.0)

    # ---- end-to-end leg: pinned host buffers through the public pipelined call (submit / collect): every step
    # uploads its inputs from pinned host memory and reads its result back; the upload of step i+1 overlaps
    # the run of step i.  Timed on the host from the first submit to the last collect, inside barriers.
    def pipelined(session, fd):
        out = session.run(fd)
        session.run_pipelined([fd] * 3)
        barrier()
        t0 = time.perf_counter()
        pending = 0
        for _ in range(args.steps):
            session.submit(fd)
            pending += 1
            if pending == 2:
                out = session.collect()
                pending -= 1
        while pending:
            out = session.collect()
            pending -= 1
        torch.cuda.synchronize()
        elapsed = (time.perf_counter() - t0) * 1000.0
        barrier()
        elapsed = max_over_ranks(elapsed, world, device=f"cuda:{local_rank}")
        return elapsed, out

    e2e_total, out = pipelined(sess, pinned)
    e2e = {"value": world * batch * per_item * args.steps / (e2e_total / 1000.0), "unit": w["unit"],
           "h2d_bytes_per_step": int(sum(v.nbytes for v in pinned.values())), "d2h_bytes_per_step": int(sum(v.size for v in out.values()) * 4),
           "ms_per_step": e2e_total / args.steps,
           "call": "oxb200_run_submit / oxb200_run_collect, two runs in flight, f32 lanes, L2 not flushed between steps (the uploads replace the flush)"}
    counters = dict(gpu_launches=int(c1["kernel_launches"] - c0["kernel_launches"]),
                    launch_mix={"umma": int(c1["umma_launches"] - c0["umma_launches"]), "direct": int(c1["simt_launches"] - c0["simt_launches"]),
                                "glue": int(c1["glue_launches"] - c0["glue_launches"])})
    peak_probe = None
    if rank == 0:
        try:
            peak_probe = sess.ctx.probe_tensor_peak("i8" if w["dtype"] == "i8" else "tf32") / 1e12
        except Exception as exc:  # the probe is a report, not the measurement
            peak_probe = None
            print(f"tensor-peak probe failed: {exc}", file=sys.stderr)
    sess.close()
    for ptr in ptrs:
        lib.oxb200_host_free(ptr)

    e2e_u8 = None
    if key == "c5":
        # the same network with the image declared and fed as u8 lanes (a quarter of the upload)
        g8, w8, f8, _ = build_workload(key, batch, typed_input=True)
        fd8 = f8(batch, f"{key}_in_rank{rank}")
        s8 = Session.builder().with_device(local_rank).with_kernel_path(args.kernel_path).with_cuda_graph(graph_on).build_from_graph(g8, w8)
        p8, ptrs8 = {}, []
        for name in g8.input_names:
            p8[name], ptr = pinned_like(fd8[name], lib)
            ptrs8.append(ptr)
        t8, out8 = pipelined(s8, p8)
        e2e_u8 = {"value": world * batch * args.steps / (t8 / 1000.0), "unit": w["unit"], "h2d_bytes_per_step": int(sum(v.nbytes for v in p8.values())),
                  "d2h_bytes_per_step": int(sum(v.size for v in out8.values()) * 4), "ms_per_step": t8 / args.steps,
                  "note": "input declared u8 (oxb200_value_info.dtype) and fed as typed lanes; its QuantizeLinear is then the caller's"}
        s8.close()
        for ptr in ptrs8:
            lib.oxb200_host_free(ptr)

    peaks = measured_peaks()
    kind = w["dtype"]
    # TF32 runs at half, INT8 at twice the measured dense bf16 rate (architectural ratios); the kernels
    # are timed inside a long step, so the sustained figure is the denominator.
    factor = {"tf32": 0.5, "i8": 2.0}[kind]
    peak = peaks["bf16_sustained"] * factor
    achieved = (conv_ops / (conv_ms / 1000.0) / 1e12) if conv_ms > 0 else 0.0
    traffic, traffic_note, traffic_batch = captured_traffic(key)
    if traffic is not None and traffic_batch and traffic_batch != batch:
        # the capture was taken at another batch: activations dominate the traffic and grow with the batch, the
        # weights (25.5 MB in 54 launches for the INT8 network) do not; scale by the units one launch processes
        traffic = traffic * batch / traffic_batch
        traffic_note += f" -- scaled by {batch}/{traffic_batch} to this run's per-GPU batch"
    # A network is a mix of layers, each with its own roofline: a layer cannot take less than the longer of its
    # operations at the tensor peak and its algorithmic bytes (operands, weights and result once) at the measured
    # copy bandwidth.  The sum of those per-layer floors against the measured contraction time says how far the
    # kernel is from what this layer mix allows; `frac` above is the plain tensor-pipe fraction.
    floor_ms = sum(max(ops / (peak * 1e12), nbytes / (peaks["hbm_gbs"] * 1e9)) for ops, nbytes in conv_layers) * 1000.0
    conv_ms_per_step = conv_ms / max(args.steps, 1)
    hbm_bound_layers = sum(1 for ops, nbytes in conv_layers if nbytes / (peaks["hbm_gbs"] * 1e9) > ops / (peak * 1e12))
    roofline = {
        "layerwise": {"floor_ms_per_step": floor_ms, "measured_ms_per_step": conv_ms_per_step,
                      "frac": floor_ms / conv_ms_per_step if conv_ms_per_step > 0 else None,
                      "hbm_bound_layers": hbm_bound_layers, "layers": len(conv_layers),
                      "algorithmic_bytes_per_launch": conv_algo_bytes / max(conv_launches, 1),
                      "rule": "sum over the contraction launches of max(ops / tensor peak, algorithmic bytes / measured copy bandwidth)"},
        "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TOP/s" if kind == "i8" else "TFLOP/s",
        "frac": achieved / peak if peak else None, "traffic": traffic, "traffic_note": traffic_note,
        "kernel": " + ".join(sorted(umma_kernels)) or "umma_conv_kernel (tcgen05 implicit GEMM)", "launches_per_step": conv_launches // max(args.steps, 1),
        "avg_launch_ms": conv_ms / max(conv_launches, 1), "share_of_step": conv_ms / prof_ms if prof_ms > 0 else None,
        "timed_in": "a second pass of the same K steps with a CUDA-event pair around every kernel (ms_per_step %.3f there)" % (prof_ms / max(args.steps, 1)),
        "peak_basis": f"{factor} x bf16_tflops_sustained of {peaks['source']} ({peaks['bf16_sustained']})",
        "frac_of_burst": achieved / (peaks["bf16"] * factor),
        "tcgen05_issue_rate_peak": peak_probe, "frac_of_issue_rate_peak": (achieved / peak_probe) if peak_probe else None,
        "glue_gbs": (glue_bytes / (glue_ms / 1000.0) / 1e9) if glue_ms > 0 else None, "hbm_peak_gbs": peaks["hbm_gbs"],
        "time_by_kernel_family_ms_per_step": {k2: v / max(args.steps, 1) for k2, v in sorted(slowest.items(), key=lambda kv: -kv[1])[:6]},
    }
    line = {
        "metric": w["metric"], "value": value, "unit": w["unit"], "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total_ms / args.steps, "higher_is_better": True,
        "scaling": "strong" if (w.get("global_batch") and not args.batch) else "weak", "vs_baseline": None, "dtype": kind, "data": "synthetic",
        "config": {"workload": w["name"], "per_gpu_batch": batch, "global_batch": batch * world, "parallelism": f"batch-sharded replicas x{world}, no collective",
                   "l2": "flushed between timed steps (256 MiB memset)", "algorithmic_ops_per_step": info["ops"], "kernel_path": args.kernel_path,
                   "cuda_graph": bool(graph_on)},
        "e2e": e2e, "roofline": roofline,
    }
    line.update(counters)
    if clocks is not None:
        line["clocks"] = dict(clocks, window="the timed K steps and the profiled K steps that follow them")
    if e2e_u8 is not None:
        line["e2e_u8_feed"] = e2e_u8
    return line


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="c5", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--batch", type=int, default=0, help="per-GPU batch (default: the configuration's)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-companion", action="store_true", help="skip the f32 ResNet-50 measurement that accompanies the default workload on one GPU")
    ap.add_argument("--kernel-path", default="auto", choices=["auto", "direct"])
    ap.add_argument("--cuda-graph", type=int, default=-1,
                    help="1: replay the planned step list as one CUDA graph (OXIONNX_CUDA_GRAPH); default: on, except for the six-launch MLP "
                         "(c1), where a graph launch costs more than the launches it replaces")
    ap.add_argument("--layer", default=None, help='time one layer: "i8|f32 N C H W OC K STRIDE PAD"')
    ap.add_argument("--layer-iters", type=int, default=5)
    ap.add_argument("--cta-pairs", default="auto", choices=["auto", "never", "always"], help="--layer only: the CTA-pair form of the kernel")
    args = ap.parse_args()

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.layer:
        run_layer(args.layer.split(), args.layer_iters, args.cta_pairs)
        return
    if args.impl == "reference":
        run_reference(args, rank)
        return
    args.warmup = max(args.warmup, 3)

    import torch
    dist = None
    torch.cuda.set_device(local_rank)
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from oxionnx_b200 import _ffi
    lib = _ffi.lib()
    w = WORKLOADS[args.workload]
    batch = args.batch or (max(w["batch"] // world, 1) if w.get("global_batch") else w["batch"])

    # L2 flush between timed steps: a 256 MiB memset (L2 is 126 MB)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=f"cuda:{local_rank}")

    def flush_l2():
        flush.zero_()
        torch.cuda.synchronize()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    line = measure(args, args.workload, batch, local_rank, world, dist, torch, lib, flush_l2, barrier, True)
    if rank == 0:
        if args.workload == "c5" and world == 1 and not args.no_companion:
            # ResNet-50 as an f32 graph at batch 32 (TF32 contractions), the float half of the headline metric, in the same run
            comp_args = argparse.Namespace(**vars(args))
            comp_args.steps = max(args.steps, 20)
            c = measure(comp_args, "c2", WORKLOADS["c2"]["batch"], local_rank, 1, None, torch, lib, flush_l2, lambda: torch.cuda.synchronize(), False)
            line["f32"] = {"workload": c["config"]["workload"], "value": c["value"], "unit": c["unit"], "ms_per_step": c["ms_per_step"], "steps": c["steps"],
                           "e2e": c["e2e"], "roofline": c["roofline"], "gpu_launches": c["gpu_launches"]}
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline_record(args.workload, os.cpu_count() or 1)
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
