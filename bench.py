#!/usr/bin/env python
"""Benchmark of the quantized-operator hot path: MobileNetV2-int8 images/s through dl::Model on N B200s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--batch B]

One step = one forward pass of the MobileNetV2-1.0 classifier (224x224x3 int8 input, 70-node graph, random int8
per-channel weights; synthetic, see esp-dl_b200/zoo.py) over a batch of B images per GPU.  Ranks hold a replica of
the weights and their own B images (the units are independent, no data-path collective); the only exchange is the
gather of the [B,1000] int8 logits over NCCL at the end of a step.  Prints ONE JSON line on rank 0.

  value      images/s with the input batch already resident in HBM (CUDA events around K graph replays, max over ranks)
  e2e        images/s through dl::Model::run() with pinned HOST buffers: H2D of the images, forward, D2H of the logits
  roofline   for the dominant kernel (the tcgen05 pointwise-conv tile kernel): algorithmic bytes of the modules it
             runs / their summed device time, both per step, against the measured HBM copy bandwidth
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
    ap.add_argument("--batch", type=int, default=1024, help="images per GPU per step")
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
            "scaling": "weak", "vs_baseline": None, "dtype": "s8", "data": "synthetic",
            "config": {"workload": "mobilenet_v2_1.0_224_int8", "images_per_step": done},
            "cpu_baseline": {"value": value, "unit": "images/s", "cores": cores, "kind": kind, "sample": sample},
            "e2e": {"value": value, "unit": "images/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------ GPU arm
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
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    entry._package()
    from espdl_b200 import abi, espdl_file, model, sharding
    L = abi.load()
    path = build_network()
    parsed = espdl_file.read(path)
    m = model.Model(path, batch=args.batch, device=local_rank)
    os.unlink(path)
    inp, out = m.inputs[0], m.outputs[0]
    rng = np.random.default_rng(1000 + rank)
    inp.array[...] = rng.integers(-128, 128, size=inp.shape, dtype=np.int8)
    stream = m.stream
    torch_stream = torch.cuda.ExternalStream(stream)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # logits gather: the one exchange of the path (every rank ends up with all [world*B, 1000] logits)
    logits_dev = torch.empty(0)
    gathered = None
    if world > 1:
        # a torch view of the model's device output buffer, so NCCL reads it in place
        class _Ext:
            __cuda_array_interface__ = {"shape": out.shape, "typestr": "|i1", "data": (out.device_ptr, False), "version": 2}
        logits_dev = torch.as_tensor(_Ext(), device=f"cuda:{local_rank}")
        gathered = torch.empty((world * out.shape[0],) + tuple(out.shape[1:]), dtype=torch.int8, device=f"cuda:{local_rank}")

    def step_device():
        m.run_device(sync=False)
        if world > 1:
            with torch.cuda.stream(torch_stream):
                sharding.gather_logits(logits_dev, world * args.batch, out=gathered)

    # one full pass through the public API first: uploads the inputs and captures the CUDA graph
    launches0 = L.espdl_b200_launch_count()
    m.run()
    launches_per_step = (L.espdl_b200_launch_count() - launches0) // 2  # the capture pass enqueues every kernel twice
    for _ in range(args.warmup):
        step_device()
    abi.check(L.espdl_b200_stream_sync(stream), "warm-up")

    ev0, ev1 = C.c_void_p(), C.c_void_p()
    L.espdl_b200_event_create(C.byref(ev0))
    L.espdl_b200_event_create(C.byref(ev1))
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    barrier()
    L.espdl_b200_event_record(ev0, stream)
    for _ in range(args.steps):
        step_device()
    L.espdl_b200_event_record(ev1, stream)
    ms = C.c_float()
    abi.check(L.espdl_b200_event_elapsed_ms(ev0, ev1, C.byref(ms)), "event_elapsed")
    abi.check(L.espdl_b200_stream_sync(stream), "timed region")
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    total_ms = float(ms.value)
    if world > 1:
        t = torch.tensor([total_ms], device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    value = world * args.batch * args.steps / (total_ms / 1000.0)

    # end to end through the model's public API, host buffers in and out: Model::submit() copies the step's images
    # from the pinned host buffer to the device and enqueues the pass, Model::wait() returns when the logits of the
    # oldest step are back in host memory.  One step is kept in flight, so the upload of step i+1 overlaps the
    # execution of step i; every step's host->device and device->host copies happen inside the timed region.
    e2e_steps = max(3, min(args.steps, 20))
    for _ in range(2):  # warm-up: the first submit() creates the second stream and the staging buffers
        m.submit()
        m.wait()
    barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        m.submit()
        if i >= 1:
            m.wait()
            if world > 1:
                with torch.cuda.stream(torch_stream):
                    sharding.gather_logits(logits_dev, world * args.batch, out=gathered)
    m.wait()
    if world > 1:
        with torch.cuda.stream(torch_stream):
            sharding.gather_logits(logits_dev, world * args.batch, out=gathered)
        torch_stream.synchronize()
    barrier()
    e2e_ms = (time.perf_counter() - t0) * 1000.0
    if world > 1:
        t = torch.tensor([e2e_ms], device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = world * args.batch * e2e_steps / (e2e_ms / 1000.0)

    result = None
    if rank == 0:
        # roofline of the dominant kernel, from per-module CUDA-event times measured now (eager launches on the model's stream)
        prof = m.profile()
        traffic = {tr["name"]: tr for tr in module_traffic(parsed, args.batch)}
        executed = {name for (_, _, _, name) in prof}
        # an Add that the model folded into the conv before it (espdl_conv_desc::residual) has no launch of its own:
        # the conv then also reads the Add's other input and writes the Add's output instead of its own
        shapes = {v["name"]: v["shape"] for v in list(parsed["value_info"].values()) + parsed["inputs"] + parsed["outputs"]}
        for node in parsed["nodes"]:
            if node["op_type"] == "Add" and node["name"] not in executed:
                for prod in parsed["nodes"]:
                    if prod["name"] in executed and prod["op_type"] == "Conv" and prod["outputs"][0] in node["inputs"]:
                        traffic[prod["name"]]["bytes"] += int(np.prod(shapes[node["outputs"][0]])) * args.batch
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
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except OSError:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        achieved = dom["bytes"] / (dom["us"] * 1e-6) / 1e9
        kernel_names = {"pointwise_tc": "gemm_tc_kernel", "depthwise": "dw3x3_dp4a_kernel", "conv_simt": "stem_tc_kernel"}
        # DRAM bytes moved per algorithmic byte, from one profiler capture of each kernel on a layer larger than L2
        # (profiles/): the launches of a step differ in shape, so the per-launch traffic is that ratio applied to
        # the average algorithmic bytes of a launch.
        dram_per_algorithmic = {"pointwise_tc": TRAFFIC_RATIO_GEMM_TC, "depthwise": TRAFFIC_RATIO_DW}
        bytes_per_launch = dom["bytes"] / dom["launches"]
        ratio = dram_per_algorithmic.get(dom_kind)
        roofline = {"bound": "hbm", "kernel": kernel_names.get(dom_kind, dom_kind), "achieved": achieved, "peak": peak, "unit": "GB/s",
                    "frac": achieved / peak, "traffic": None if ratio is None else bytes_per_launch * ratio,
                    "traffic_note": "bytes per launch: average algorithmic bytes of a launch x the DRAM/algorithmic ratio of one ncu capture",
                    "peak_source": "measured" if peaks else "fallback",
                    "launches_per_step": dom["launches"], "algorithmic_bytes_per_launch": bytes_per_launch,
                    "avg_launch_us": dom["us"] / dom["launches"],
                    "share_of_step_time": dom["us"] / total_us,
                    "per_kind_us": {k: round(v["us"], 1) for k, v in by_kind.items()}}
        cpu = None
        if not args.no_cpu_baseline:
            sys.path.insert(0, os.path.join(ROOT, "tests"))
            import checkers
            kind = "reference" if checkers.have_ref() else "port"
            images = args.cpu_images or max(os.cpu_count() or 1, 16)
            v, cores, dt, done = _cpu_images_per_s(kind, images)
            cpu = {"value": v, "unit": "images/s", "cores": cores, "kind": kind,
                   "sample": f"{done} images of the same network in {dt:.1f} s ("
                             + ("reference operators built from its sources, per-tensor filter exponents" if kind == "reference"
                                else "plain-C oracle port, per-channel exponents") + ", OpenMP)"}
        result = {"metric": "images/s MobileNetV2-int8", "value": value, "unit": "images/s", "n_gpus": world, "steps": args.steps,
                  "warmup": args.warmup, "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak",
                  "vs_baseline": None, "dtype": "s8", "data": "synthetic",
                  "config": {"workload": "mobilenet_v2_1.0_224_int8", "batch_per_gpu": args.batch, "global_batch": args.batch * world,
                             "nodes": len(parsed["nodes"]), "l2": "per-step inputs (154 MB) and activations exceed the 126 MB L2",
                             "parallelism": f"replicas x{world}, logits all-gather" if world > 1 else "single GPU"},
                  "e2e": {"value": e2e_value, "unit": "images/s", "h2d_bytes_per_step": inp.nbytes, "d2h_bytes_per_step": out.nbytes,
                          "steps": e2e_steps, "api": "dl::Model::submit()/wait(), one step in flight"},
                  "gpu_launches": int(launches_per_step * args.steps), "launches_per_step": int(launches_per_step),
                  "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu}
    m.close()
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
