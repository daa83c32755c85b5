#!/usr/bin/env python
"""Benchmark of the quantized-operator hot path: MobileNetV2-int8 images/s through dl::Model on N B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--batch B]

One step = one forward pass of the MobileNetV2-1.0 classifier (224x224x3 int8 input, 70-node graph, random int8
per-channel weights; synthetic, see esp-dl_b200/zoo.py) over a GLOBAL batch of B = 1024 images, sharded evenly over the
ranks ("scaling": "strong" - the configuration the workload is stated on: batch 1024 across 1/2/4/8 GPUs).  Ranks hold
a replica of the weights and their own B/N images (the units are independent, no data-path collective); the only
exchange is the gather of the [B,1000] int8 logits over NCCL at the end of a step.  Prints ONE JSON line on rank 0.

  value      images/s with the input batch already resident in HBM (CUDA events around K graph replays, max over ranks)
  e2e        images/s through dl::Model::submit()/wait() with pinned HOST buffers: H2D of the images, forward, D2H of the
             logits; `copy_ceiling` is the same loop with the copies only (no kernels)
  weak       (N > 1) the same two measurements with B images PER GPU, i.e. replicas at the single-GPU batch
  roofline   for the kernel with the largest share of the step: algorithmic bytes of the modules it runs / their summed
             device time, both per step, against the measured HBM copy bandwidth
  ops        (N = 1) the operator configurations of the workload, each through the C ABI with CUDA events and the L2
             flushed between launches: int8 and int16 Gemm 4096x1024x1024, a large int8 Gemm, the 3x3 conv 56x56x64->64
             at batch 1 and 1024 (tera-operations/s against the tensor peak), the inverted-residual block at batch 256
             and the 640x640 detector at batch 512 (ms per step)
  nsharded   (N > 1) the N-sharded Gemm: bit-exactness against the single-rank product on every rank, and its times
  cpu_baseline / --impl reference: the same network on the host cores (see _cpu_images_per_s)
"""
import argparse
import ctypes as C
import json
import os
import subprocess
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402

import __graft_entry__ as entry  # noqa: E402


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--batch", type=int, default=1024, help="global batch per step (sharded over the GPUs)")
    ap.add_argument("--no-ops", action="store_true", help="skip the operator configurations (ops block)")
    ap.add_argument("--cpu-images", type=int, default=0, help="images in the CPU sample (0 = sized to ~20 s)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    return ap.parse_args()


TRAFFIC_RATIO_GEMM_TC = 0.87  # gemm_tc_kernel, 401408x128x768: 313.2 MB DRAM for 359.8 MB algorithmic (the output tail is still in L2)
TRAFFIC_RATIO_DW = 1.034      # dw3x3_dp4a_kernel, 256x112x112x96: 637.4 MB DRAM for 616.6 MB algorithmic


# ------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clock and clock-event (throttle) reasons of one GPU while the timed region runs: NVML read-only
    queries from a thread of this process every few milliseconds (nothing is set or reset)."""

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.sm, self.reason_bits, self.max_mhz = [], 0, None
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(self.gpu)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
        except Exception:  # no NVML: the clocks record stays empty
            self._nvml = None
            return
        self._thread = threading.Thread(target=self._loop, daemon=True)
        self._thread.start()

    def _loop(self):
        n = self._nvml
        while not self._stop.is_set():
            try:
                self.sm.append(float(n.nvmlDeviceGetClockInfo(self._h, n.NVML_CLOCK_SM)))
                self.reason_bits |= int(n.nvmlDeviceGetCurrentClocksEventReasons(self._h))
            except Exception:
                break
            self._stop.wait(0.005)

    def stop(self):
        self._stop.set()
        if self._thread:
            self._thread.join(timeout=2)
        reasons = []
        n = self._nvml
        if n is not None:
            names = {"hw_slowdown": "nvmlClocksEventReasonHwSlowdown", "hw_thermal_slowdown": "nvmlClocksEventReasonHwThermalSlowdown",
                     "sw_thermal_slowdown": "nvmlClocksEventReasonSwThermalSlowdown", "sw_power_cap": "nvmlClocksEventReasonSwPowerCap"}
            legacy = {"hw_slowdown": "nvmlClocksThrottleReasonHwSlowdown", "hw_thermal_slowdown": "nvmlClocksThrottleReasonHwThermalSlowdown",
                      "sw_thermal_slowdown": "nvmlClocksThrottleReasonSwThermalSlowdown", "sw_power_cap": "nvmlClocksThrottleReasonSwPowerCap"}
            for key in names:
                bit = getattr(n, names[key], None) or getattr(n, legacy[key], 0)
                if bit and (self.reason_bits & int(bit)):
                    reasons.append(key)
        return {"sm_mhz": float(np.median(self.sm)) if self.sm else None, "sm_max_mhz": self.max_mhz, "reasons": sorted(reasons),
                "samples": len(self.sm)}


# ------------------------------------------------------------------------------------------ workload
def build_network(per_tensor=False):
    entry._package()
    from espdl_b200 import zoo
    g = zoo.mobilenet_v2(seed=5)
    if per_tensor:
        # same topology, shapes and weights; one filter exponent per layer (the reference's generic C epilogue has
        # no per-channel branch): every per-channel exponent vector is replaced by its first entry
        g.initializers = [(n, a, ([e[0]] if e is not None and len(e) > 1 else e)) for n, a, e in g.initializers]
    fd, path = tempfile.mkstemp(suffix=".espdl", prefix="mbv2_")
    os.close(fd)
    g.save(path)
    return path


def module_traffic(parsed, batch):
    """Algorithmic bytes per module for a batch: every input and output tensor once, weights once."""
    shapes = {v["name"]: v["shape"] for v in list(parsed["value_info"].values()) + parsed["inputs"] + parsed["outputs"]}
    rows = []
    for node in parsed["nodes"]:
        b = 0
        macs = 0
        for name in node["inputs"]:
            if name in parsed["initializers"]:
                t = parsed["initializers"][name]
                b += int(np.prod(t["dims"])) * t["data"].dtype.itemsize
            elif name in shapes:
                b += int(np.prod(shapes[name])) * batch
        for name in node["outputs"]:
            b += int(np.prod(shapes[name])) * batch
        kind = node["op_type"]
        if kind in ("Conv", "Gemm"):
            w = parsed["initializers"][node["inputs"][1]]["dims"]
            out = shapes[node["outputs"][0]]
            group = node["attrs"].get("group", 1)
            macs = int(np.prod(out)) * batch * w[0] * w[1] * (1 if group != 1 else w[2])
            if group != 1:
                kind = "depthwise"
            elif w[0] == 1 and w[1] == 1:
                kind = "pointwise_tc"
            else:
                kind = "conv_simt"
        rows.append(dict(name=node["name"], kind=kind, bytes=b, macs=macs))
    return rows


# ------------------------------------------------------------------------------------------ CPU legs
def _cpu_images_per_s(kind, images, seconds=12.0):
    """Times the network on the host cores: chunks of `images` images, repeated until `seconds` of work are done
    (a bounded sample of the step's batch).  Returns (images/s, threads, elapsed s, images done).
    kind "reference": the reference's own operators (oracle/_ref, built from its sources), per-tensor filter exponents.
    kind "port": the plain-C restatement (oracle/), per-channel exponents as in the GPU run.  Both use OpenMP over images / rows."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    entry._package()
    import checkers
    import graph_oracle
    from espdl_b200 import espdl_file
    path = build_network(per_tensor=(kind == "reference"))
    parsed = espdl_file.read(path)
    os.unlink(path)
    rng = np.random.default_rng(7)
    x = rng.integers(-128, 128, size=(images, 224, 224, 3), dtype=np.int8)
    backend = checkers.ref() if kind == "reference" else checkers.oracle()
    cores = backend.ref_num_threads() if kind == "reference" else backend.oracle_num_threads()
    graph_oracle.run_graph(parsed, {"input": x[:max(1, images // 4)]}, backend=kind)  # warm the caches and the thread pool
    done, t0 = 0, time.perf_counter()
    while True:
        graph_oracle.run_graph(parsed, {"input": x}, backend=kind)
        done += images
        dt = time.perf_counter() - t0
        if dt >= seconds:
            break
    return done / dt, cores, dt, done


def reference_arm(args, rank):
    if rank != 0:
        return
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    entry._package()
    import checkers
    kind = "reference" if checkers.have_ref() else "port"
    cores_guess = os.cpu_count() or 1
    images = args.cpu_images or max(cores_guess, 16)
    vals = []
    cores = 1
    total = args.warmup + args.steps
    per_step = max(2.0, min(12.0, 200.0 / total))  # seconds of host work per step; the whole run stays within a few minutes
    done = images
    for i in range(total):
        v, cores, dt, done = _cpu_images_per_s(kind, images, seconds=per_step)
        if i >= args.warmup:
            vals.append(v)
    value = float(np.mean(vals)) if vals else v
    sample = (f"{done} images per step (chunks of {images}) through the reference's own dl::module operators compiled for the host "
              f"(MobileNetV2 topology and shapes of the GPU run, per-tensor filter exponents: its generic C epilogue has no "
              f"per-channel branch), OpenMP over images") if kind == "reference" else \
             f"{done} images per step (chunks of {images}) through the plain-C oracle port (per-channel exponents), OpenMP over output rows"
    line = {"impl": "reference", "metric": "images/s MobileNetV2-int8", "value": value, "unit": "images/s", "n_gpus": args.gpus,
            "steps": len(vals), "warmup": args.warmup, "ms_per_step": 1000.0 * done / value, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "s8", "data": "synthetic",
            "config": {"workload": "mobilenet_v2_1.0_224_int8", "images_per_step": done},
            "cpu_baseline": {"value": value, "unit": "images/s", "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------ GPU arm
def bind_to_gpu_numa_node(gpu_index):
    """Pins this process (and so the first-touch placement of its pinned host buffers) to the CPUs NVML reports as
    local to the GPU.  Read-only NVML query plus sched_setaffinity of this process; returns the CPU count or None."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
        words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, words)
        cpus = {64 * i + b for i, w in enumerate(mask) for b in range(64) if (int(w) >> b) & 1}
        cpus &= set(os.sched_getaffinity(0))
        if cpus:
            os.sched_setaffinity(0, cpus)
            return len(cpus)
    except Exception:
        pass
    return None


class Timed:
    """One model at a given per-GPU batch with the two measurements of the benchmark."""

    def __init__(self, path, batch, local_rank, rank, world, global_batch):
        import torch
        from espdl_b200 import abi, model
        self.torch, self.abi, self.L = torch, abi, abi.load()
        self.world, self.rank, self.local_rank, self.batch, self.global_batch = world, rank, local_rank, batch, global_batch
        self.m = model.Model(path, batch=batch, device=local_rank)
        self.inp, self.out = self.m.inputs[0], self.m.outputs[0]
        rng = np.random.default_rng(1000 + rank)
        self.inp.array[...] = rng.integers(-128, 128, size=self.inp.shape, dtype=np.int8)
        self.stream = self.m.stream
        self.torch_stream = torch.cuda.ExternalStream(self.stream)
        self.logits_dev, self.gathered = None, None
        if world > 1:
            out = self.out

            class _Ext:  # a torch view of the model's device output buffer, so NCCL reads it in place
                __cuda_array_interface__ = {"shape": out.shape, "typestr": "|i1", "data": (out.device_ptr, False), "version": 2}
            self.logits_dev = torch.as_tensor(_Ext(), device=f"cuda:{local_rank}")
            self.gathered = torch.empty((world * out.shape[0],) + tuple(out.shape[1:]), dtype=torch.int8, device=f"cuda:{local_rank}")
        launches0 = self.L.espdl_b200_launch_count()
        self.m.run()  # one full pass through the public API first: uploads the inputs and captures the CUDA graph
        self.launches_per_step = (self.L.espdl_b200_launch_count() - launches0) // 2  # the capture pass enqueues every kernel twice

    def barrier(self):
        if self.world > 1:
            import torch.distributed as dist
            dist.barrier()
        self.torch.cuda.synchronize()

    def gather(self):
        if self.world > 1:
            from espdl_b200 import sharding
            with self.torch.cuda.stream(self.torch_stream):
                sharding.gather_logits(self.logits_dev, self.world * self.batch, out=self.gathered)

    def max_over_ranks(self, ms):
        if self.world > 1:
            import torch.distributed as dist
            t = self.torch.tensor([ms], device=f"cuda:{self.local_rank}")
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def device_timed(self, steps, warmup, sampler=None):
        """images/s with the inputs resident: CUDA events on the model's stream around `steps` graph replays."""
        L, abi = self.L, self.abi
        for _ in range(warmup):
            self.m.run_device(sync=False)
            self.gather()
        abi.check(L.espdl_b200_stream_sync(self.stream), "warm-up")
        ev0, ev1 = C.c_void_p(), C.c_void_p()
        L.espdl_b200_event_create(C.byref(ev0))
        L.espdl_b200_event_create(C.byref(ev1))
        if sampler:
            sampler.start()
        self.barrier()
        L.espdl_b200_event_record(ev0, self.stream)
        for _ in range(steps):
            self.m.run_device(sync=False)
            self.gather()
        L.espdl_b200_event_record(ev1, self.stream)
        ms = C.c_float()
        abi.check(L.espdl_b200_event_elapsed_ms(ev0, ev1, C.byref(ms)), "event_elapsed")
        abi.check(L.espdl_b200_stream_sync(self.stream), "timed region")
        self.barrier()
        clocks = sampler.stop() if sampler else None
        L.espdl_b200_event_destroy(ev0)
        L.espdl_b200_event_destroy(ev1)
        total_ms = self.max_over_ranks(float(ms.value))
        return self.world * self.batch * steps / (total_ms / 1000.0), total_ms / steps, clocks

    def end_to_end(self, steps):
        """images/s through Model::submit()/wait(): submit() copies the step's images from the pinned host buffer to the
        device and enqueues the pass, wait() returns when the logits of the oldest step are back in host memory.  One
        step is kept in flight, so the upload of step i+1 overlaps the execution of step i; every step's host->device
        and device->host copies happen inside the timed region."""
        m = self.m
        for _ in range(2):  # warm-up: the first submit() creates the second stream and the staging buffers
            m.submit()
            m.wait()
        self.barrier()
        t0 = time.perf_counter()
        for i in range(steps):
            m.submit()
            if i >= 1:
                m.wait()
                self.gather()
        m.wait()
        self.gather()
        if self.world > 1:
            self.torch_stream.synchronize()
        self.barrier()
        ms = self.max_over_ranks((time.perf_counter() - t0) * 1000.0)
        return self.world * self.batch * steps / (ms / 1000.0)

    def copy_ceiling(self, steps):
        """The end-to-end loop with the copies alone: the same pinned host buffers and byte counts, upload and read-back
        on two streams of the library, no kernels.  What the host link alone allows, in images/s."""
        L, abi = self.L, self.abi
        up, down = C.c_void_p(), C.c_void_p()
        abi.check(L.espdl_b200_stream_create(C.byref(up)), "stream")
        abi.check(L.espdl_b200_stream_create(C.byref(down)), "stream")
        staging = C.c_void_p()
        abi.check(L.espdl_b200_arena_alloc(self.inp.nbytes, C.byref(staging)), "arena_alloc")
        src = self.inp.array.ctypes.data
        dst = self.out.array.ctypes.data
        for _ in range(2):
            L.espdl_b200_upload(staging, src, self.inp.nbytes, up)
            L.espdl_b200_download(dst, self.out.device_ptr, self.out.nbytes, down)
        L.espdl_b200_stream_sync(up)
        L.espdl_b200_stream_sync(down)
        self.barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            L.espdl_b200_upload(staging, src, self.inp.nbytes, up)
            L.espdl_b200_download(dst, self.out.device_ptr, self.out.nbytes, down)
        L.espdl_b200_stream_sync(up)
        L.espdl_b200_stream_sync(down)
        self.barrier()
        ms = self.max_over_ranks((time.perf_counter() - t0) * 1000.0)
        L.espdl_b200_arena_free(staging)
        L.espdl_b200_stream_destroy(up)
        L.espdl_b200_stream_destroy(down)
        return self.world * self.batch * steps / (ms / 1000.0)

    def close(self):
        self.m.close()


def roofline_of(m, parsed, batch):
    """Roofline of the kernel with the largest share of the step, from per-module CUDA-event times measured now (eager
    launches on the model's stream)."""
    prof = m.profile()
    traffic = {tr["name"]: tr for tr in module_traffic(parsed, batch)}
    executed = {name for (_, _, _, name) in prof}
    # an Add that the model folded into the conv before it (espdl_conv_desc::residual) has no launch of its own:
    # the conv then also reads the Add's other input and writes the Add's output instead of its own
    shapes = {v["name"]: v["shape"] for v in list(parsed["value_info"].values()) + parsed["inputs"] + parsed["outputs"]}
    for node in parsed["nodes"]:
        if node["op_type"] == "Add" and node["name"] not in executed:
            for prod in parsed["nodes"]:
                if prod["name"] in executed and prod["op_type"] == "Conv" and prod["outputs"][0] in node["inputs"]:
                    traffic[prod["name"]]["bytes"] += int(np.prod(shapes[node["outputs"][0]])) * batch
    # a depthwise conv that the model fused into the pointwise conv behind it (one launch, named after the pointwise conv)
    # has no launch of its own either: that launch reads the depthwise conv's input and filter instead of the tensor between
    # the two, which never exists
    for node in parsed["nodes"]:
        if node["op_type"] == "Conv" and node["name"] not in executed and node["attrs"].get("group", 1) != 1:
            for cons in parsed["nodes"]:
                if cons["name"] in executed and cons["op_type"] == "Conv" and cons["inputs"][0] == node["outputs"][0]:
                    hidden = int(np.prod(shapes[node["outputs"][0]])) * batch
                    t = traffic[cons["name"]]
                    t["bytes"] += traffic[node["name"]]["bytes"] - 2 * hidden
                    t["macs"] += traffic[node["name"]]["macs"]
                    t["kind"] = "depthwise_pointwise_fused"
    by_kind = {}
    for (idx, typ, us, name) in prof:
        tr = traffic[name]
        k = by_kind.setdefault(tr["kind"], dict(us=0.0, bytes=0, macs=0, launches=0))
        k["us"] += us
        k["bytes"] += tr["bytes"]
        k["macs"] += tr["macs"]
        k["launches"] += 1
    total_us = sum(k["us"] for k in by_kind.values())
    dom_kind = max(by_kind, key=lambda k: by_kind[k]["us"])
    dom = by_kind[dom_kind]
    peaks = measured_peaks()
    peak = float(peaks.get("hbm_gbs", 6650.0))
    achieved = dom["bytes"] / (dom["us"] * 1e-6) / 1e9
    kernel_names = {"pointwise_tc": "gemm_tc_kernel", "depthwise": "dw3x3_tma_kernel", "conv_simt": "stem_tc_kernel",
                    "depthwise_pointwise_fused": "dwpw_kernel"}
    # DRAM bytes moved per algorithmic byte, from one profiler capture of each kernel on a layer larger than L2
    # (profiles/): the launches of a step differ in shape, so the per-launch traffic is that ratio applied to
    # the average algorithmic bytes of a launch.
    dram_per_algorithmic = {"pointwise_tc": TRAFFIC_RATIO_GEMM_TC, "depthwise": TRAFFIC_RATIO_DW}
    bytes_per_launch = dom["bytes"] / dom["launches"]
    ratio = dram_per_algorithmic.get(dom_kind)
    return {"bound": "hbm", "kernel": kernel_names.get(dom_kind, dom_kind), "achieved": achieved, "peak": peak, "unit": "GB/s",
            "frac": achieved / peak, "traffic": None if ratio is None else bytes_per_launch * ratio,
            "traffic_note": "bytes per launch: average algorithmic bytes of a launch x the DRAM/algorithmic ratio of one ncu capture",
            "peak_source": "measured" if peaks else "fallback",
            "launches_per_step": dom["launches"], "algorithmic_bytes_per_launch": bytes_per_launch,
            "avg_launch_us": dom["us"] / dom["launches"],
            "share_of_step_time": dom["us"] / total_us,
            "per_kind_us": {k: round(v["us"], 1) for k, v in by_kind.items()},
            "per_kind_frac_of_peak": {k: round(v["bytes"] / (v["us"] * 1e-6) / 1e9 / peak, 3) for k, v in by_kind.items() if v["us"] > 0}}


def measured_peaks():
    try:
        return json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except (OSError, ValueError):
        return {}


def ops_block(local_rank):
    """The operator configurations through the C ABI (CUDA events, L2 flushed between launches) and the two other network
    configurations through dl::Model (CUDA-graph replays).  Tensor-core fractions are against twice the measured bf16 burst
    (the int8 rate of the same tensor cores; MEASURED_PEAKS.json has no int8 figure) and, for context, the nominal 4.5 POPS."""
    from espdl_b200 import abi, model, opbench, zoo
    peaks = measured_peaks()
    peak = 2.0 * float(peaks.get("bf16_tflops", 1590.0))
    peak_source = "2 x measured bf16 burst (MEASURED_PEAKS.json)" if peaks else "2 x fallback bf16 burst (1590 TFLOP/s)"
    dev = opbench.Dev(local_rank)
    ops = {}
    cases = [("gemm_s8_4096x1024x1024", (1, 1, 4096, 1024, 1024, 1, 1, 0, 8)),
             ("gemm_s16_4096x1024x1024", (1, 1, 4096, 1024, 1024, 1, 1, 0, 16)),
             ("gemm_s8_65536x1024x1024", (1, 1, 65536, 1024, 1024, 1, 1, 0, 8)),
             ("gemm_s8_65536x2048x2048", (1, 1, 65536, 2048, 2048, 1, 1, 0, 8)),
             ("conv3x3_s8_1x56x56x64_64", (1, 56, 56, 64, 64, 3, 1, 0, 8)),
             ("conv3x3_s8_1024x56x56x64_64", (1024, 56, 56, 64, 64, 3, 1, 0, 8)),
             ("conv3x3_s8_256x80x80x128_128", (256, 80, 80, 128, 128, 3, 1, 0, 8))]
    for name, spec in cases:
        ms, tops, gbs, algo = opbench.run_case(dev, spec, 10, 3, abi.KERNEL_AUTO)
        work = tops * (4.0 if spec[8] == 16 else 1.0)  # an int16 product runs as four int8 products on the tensor cores
        ops[name] = {"us": round(ms * 1000.0, 2), "tops": round(tops, 1), "frac_of_peak": round(work / peak, 4),
                     "frac_of_nominal_4500": round(work / 4500.0, 4), "gb_s": round(gbs, 1)}
    ops["peak_tops"] = peak
    ops["peak_source"] = peak_source
    ops["int16_note"] = "int16 fractions count the four int8 tensor-core products one int16 product needs"
    # the inverted-residual block at batch 256 and the detector at 640x640, batch 512: ms per step, CUDA-graph replays
    topo = os.path.join(ROOT, "tests", "golden", "yolo11n_640_topology.json")
    nets = [("mbv2_block_256x112x112x32", zoo.inverted_residual_block(seed=4), 256, 20)]
    if os.path.exists(topo):
        nets.append(("yolo11n_640_batch512", zoo.yolo11n_640(topo, seed=6), 512, 5))
    for name, g, batch, steps in nets:
        fd, path = tempfile.mkstemp(suffix=".espdl", prefix="ops_")
        os.close(fd)
        g.save(path)
        m = model.Model(path, batch=batch, device=local_rank)
        os.unlink(path)
        for t in m.inputs:
            t.array[...] = np.random.default_rng(5).integers(-128, 128, size=t.shape, dtype=np.int8)
        L = abi.load()
        launches0 = L.espdl_b200_launch_count()
        m.run()
        launches = (L.espdl_b200_launch_count() - launches0) // 2
        for _ in range(3):
            m.run_device(sync=False)
        abi.check(L.espdl_b200_stream_sync(m.stream), "warm-up")
        ev0, ev1 = C.c_void_p(), C.c_void_p()
        L.espdl_b200_event_create(C.byref(ev0))
        L.espdl_b200_event_create(C.byref(ev1))
        L.espdl_b200_event_record(ev0, m.stream)
        for _ in range(steps):
            m.run_device(sync=False)
        L.espdl_b200_event_record(ev1, m.stream)
        ms = C.c_float()
        abi.check(L.espdl_b200_event_elapsed_ms(ev0, ev1, C.byref(ms)), "event_elapsed")
        ops[name] = {"ms_per_step": round(ms.value / steps, 3), "images_per_s": round(batch * steps / (ms.value / 1000.0), 1),
                     "launches_per_step": int(launches), "arena_mb": round(m.arena_bytes / 1e6, 1)}
        L.espdl_b200_event_destroy(ev0)
        L.espdl_b200_event_destroy(ev1)
        m.close()
    return ops


def nsharded_block(local_rank, rank, world):
    """The N-sharded Gemm on this run's ranks: gather mode (int8, int16) and peer-store mode (int8) against the product one
    rank computes alone with the same kernels - bit for bit, on every rank - and the time of each (CUDA events, max over
    ranks, median of five)."""
    import torch
    import torch.distributed as dist
    from espdl_b200 import abi, sharding
    L = abi.load()
    res = {"world": world}
    ok_all = True
    # a group of this rank alone, for the single-rank product (every rank takes part in the creation of every group)
    alone = None
    for r in range(world):
        grp = dist.new_group([r])
        if r == rank:
            alone = grp
    for tag, np_dt, m_rows, k, n, e_in, e_w, e_out in (("s8", np.int8, 8192, 1024, 4096, -7, (-9, -6), -4), ("s16", np.int16, 2048, 512, 1024, -14, (-15, -15), -11)):
        rng = np.random.default_rng(77)  # the same arrays on every rank
        info = np.iinfo(np_dt)
        w = rng.integers(info.min // 2, info.max // 2 + 1, size=(n, k), dtype=np_dt)
        bias = rng.integers(-4096, 4096, size=n).astype(np.int32 if np_dt == np.int8 else np.int64)
        ew = rng.integers(e_w[0], e_w[1] + 1, size=n).astype(np.int32) if np_dt == np.int8 else int(e_w[0])
        x = torch.from_numpy(rng.integers(info.min // 2, info.max // 2 + 1, size=(m_rows, k), dtype=np_dt)).cuda()
        one = sharding.NShardedGemm(w, bias, e_in, ew, e_out, group=alone)   # this rank alone: the whole filter
        want = one.forward(x).clone()
        modes = ["gather", "peer"] if np_dt == np.int8 else ["gather"]
        for mode in modes:
            g = sharding.NShardedGemm(w, bias, e_in, ew, e_out, mode=mode)
            got = g.forward(x).clone()
            torch.cuda.synchronize()
            same = bool(torch.equal(got, want))
            flag = torch.tensor([1 if same else 0], device=f"cuda:{local_rank}")
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            ok = bool(flag.item())
            ok_all &= ok
            times = []
            for _ in range(5):
                dist.barrier()
                torch.cuda.synchronize()
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                g.forward(x)
                e1.record()
                torch.cuda.synchronize()
                t = torch.tensor([e0.elapsed_time(e1)], device=f"cuda:{local_rank}")
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                times.append(float(t.item()))
            res[f"{tag}_{mode}"] = {"bit_exact_on_every_rank": ok, "ms": round(float(np.median(times)), 4), "shape": [m_rows, k, n]}
            g.close()
        times = []
        for _ in range(5):
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            one.forward(x)
            e1.record()
            torch.cuda.synchronize()
            times.append(e0.elapsed_time(e1))
        res[f"{tag}_one_gpu_ms"] = round(float(np.median(times)), 4)
        one.close()
    res["bit_exact"] = ok_all
    return res


def main():
    args = parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if rank == 0:
        # the host-core legs use every core: launchers such as torchrun export OMP_NUM_THREADS=1 for their children
        os.environ["OMP_NUM_THREADS"] = str(os.cpu_count() or 1)
    if args.impl == "reference":
        reference_arm(args, rank)
        return
    if args.warmup < 3:
        args.warmup = 3
    if args.batch % world:
        raise SystemExit(f"--batch {args.batch} is not a multiple of the {world} ranks")

    # The host-core baseline runs first, on rank 0, BEFORE any rank touches its GPU or joins the process group: the
    # other ranks then wait in the rendezvous (a blocking socket read), not in a collective that keeps their GPUs busy.
    cpu = None
    if rank == 0 and not args.no_cpu_baseline:
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        entry._package()
        import checkers
        kind = "reference" if checkers.have_ref() else "port"
        images = args.cpu_images or max(os.cpu_count() or 1, 16)
        v, cores, dt, done = _cpu_images_per_s(kind, images)
        cpu = {"value": v, "unit": "images/s", "cores": cores, "kind": kind,
               "sample": f"{done} images of the same network in {dt:.1f} s ("
                         + ("reference operators built from its sources, per-tensor filter exponents" if kind == "reference"
                            else "plain-C oracle port, per-channel exponents") + ", OpenMP)"}

    numa_cpus = bind_to_gpu_numa_node(local_rank) if world > 1 else None
    import torch
    import torch.distributed as dist
    torch.cuda.set_device(local_rank)
    stdout_fd = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # NCCL prints its version banner (and, with NCCL_DEBUG set, more) on the process's stdout when the communicator is
        # created; stdout carries the one JSON line, so file descriptor 1 points at stderr until that line is written
        os.environ.setdefault("NCCL_DEBUG_FILE", "/dev/stderr")
        sys.stdout.flush()
        stdout_fd = os.dup(1)
        os.dup2(2, 1)
        import datetime
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank), timeout=datetime.timedelta(minutes=20))

    entry._package()
    from espdl_b200 import abi, espdl_file
    path = build_network()
    parsed = espdl_file.read(path)
    per_gpu = args.batch // world
    e2e_steps = max(3, min(args.steps, 20))

    # headline: the global batch sharded over the ranks
    run = Timed(path, per_gpu, local_rank, rank, world, args.batch)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    value, ms_per_step, clocks = run.device_timed(args.steps, args.warmup, sampler)
    e2e_value = run.end_to_end(e2e_steps)
    ceiling = run.copy_ceiling(e2e_steps)
    roofline = roofline_of(run.m, parsed, per_gpu) if rank == 0 else None
    launches_per_step = run.launches_per_step
    h2d, d2h = run.inp.nbytes, run.out.nbytes
    run.close()

    weak = None
    nsharded = None
    if world > 1:
        # replicas at the single-GPU batch: per-GPU work fixed as N grows
        wrun = Timed(path, args.batch, local_rank, rank, world, args.batch * world)
        w_value, w_ms, _ = wrun.device_timed(args.steps, args.warmup)
        w_e2e = wrun.end_to_end(e2e_steps)
        w_ceiling = wrun.copy_ceiling(e2e_steps)
        weak = {"scaling": "weak", "batch_per_gpu": args.batch, "global_batch": args.batch * world, "value": w_value, "ms_per_step": w_ms,
                "e2e": w_e2e, "e2e_copy_ceiling": w_ceiling, "unit": "images/s",
                "h2d_bytes_per_step": wrun.inp.nbytes, "d2h_bytes_per_step": wrun.out.nbytes}
        wrun.close()
        try:
            nsharded = nsharded_block(local_rank, rank, world)
        except Exception as exc:  # the proof is reported, never allowed to take the headline down with it
            nsharded = {"error": f"{type(exc).__name__}: {exc}"[:300]}
    os.unlink(path)

    ops = None
    if rank == 0 and world == 1 and not args.no_ops:
        try:
            ops = ops_block(local_rank)
        except Exception as exc:
            ops = {"error": f"{type(exc).__name__}: {exc}"[:300]}

    result = None
    if rank == 0:
        result = {"metric": "images/s MobileNetV2-int8", "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps,
                  "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong",
                  "vs_baseline": None, "dtype": "s8", "data": "synthetic",
                  "config": {"workload": "mobilenet_v2_1.0_224_int8", "batch_per_gpu": per_gpu, "global_batch": args.batch,
                             "nodes": len(parsed["nodes"]),
                             "l2": f"per-step inputs ({h2d / 1e6:.0f} MB per GPU) and activations exceed the 126 MB L2" if h2d > 126e6 else
                                   f"per-step activations of {per_gpu} images per GPU (about {9.2 * per_gpu:.0f} MB written and read per pass) exceed the 126 MB L2",
                             "parallelism": f"global batch sharded over {world} replicas, logits all-gather" if world > 1 else "single GPU",
                             "numa_bound_cpus": numa_cpus},
                  "e2e": {"value": e2e_value, "unit": "images/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                          "steps": e2e_steps, "api": "dl::Model::submit()/wait(), one step in flight",
                          "copy_ceiling": ceiling, "copy_ceiling_note": "the same loop with the host<->device copies only (no kernels)"},
                  "gpu_launches": int(launches_per_step * args.steps), "launches_per_step": int(launches_per_step),
                  "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu}
        if weak is not None:
            result["weak"] = weak
        if nsharded is not None:
            result["nsharded"] = nsharded
        if ops is not None:
            result["ops"] = ops
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        if stdout_fd is not None:
            sys.stdout.flush()
            C.CDLL(None).fflush(None)  # what C libraries still hold for fd 1 goes to stderr too
            os.dup2(stdout_fd, 1)
            os.close(stdout_fd)
        print(json.dumps(result), flush=True)


if __name__ == "__main__":
    main()
