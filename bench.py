#!/usr/bin/env python
"""ResNet-50 v1 int8 inference throughput on N B200s (pure data parallelism, one process per GPU).

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --impl reference ...      # the reference arithmetic on the host cores (CPU oracle)

One step = one forward pass of the whole network over one batch of synthetic u8 images.  Rank 0 prints one JSON line.
`value` is measured with the batch resident in HBM (rotating over several resident batches so that no step finds its
input in L2); `e2e` includes, every step, the copy of a fresh batch from pinned host memory and the read-back of the
class probabilities.
"""
import argparse
import json
import os
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "ResNet-50 int8 images/s"
UNIT = "images/s"


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=256, help="images per GPU per step")
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--tune", type=int, default=1, help="1: pick tile shapes from on-device timings at build")
    ap.add_argument("--retune", action="store_true", help="ignore the tuning cache shipped with the package: time every tile shape on this device")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--cpu-sample", type=int, default=8, help="images in the CPU baseline sample")
    return ap.parse_args()


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p.get("hbm_gbs"), bf16_sustained=p.get("bf16_tflops_sustained"), bf16_burst=p.get("bf16_tflops"), source="measured")
    return dict(hbm_gbs=6650.0, bf16_sustained=1400.0, bf16_burst=1590.0, source="fallback")


class ClockSampler(threading.Thread):
    """SM clock and throttle reasons of one GPU while the timed region runs (NVML, read-only)."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.max_mhz, self._stop_evt = index, [], set(), None, threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {nv.nvmlClocksEventReasonHwSlowdown if hasattr(nv, "nvmlClocksEventReasonHwSlowdown") else 0x8: "hw_slowdown",
                 getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
                 getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
                 getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4): "sw_power_cap"}
        while not self._stop_evt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop_evt.wait(0.02)

    def finish(self):
        self._stop_evt.set()
        self.join(timeout=2)
        s = sorted(self.samples)
        return dict(sm_mhz=s[len(s) // 2] if s else None, sm_max_mhz=self.max_mhz, reasons=sorted(self.reasons), samples=len(s))


# dram__bytes_read.sum + dram__bytes_write.sum of the 53 conv_i8_tc launches of one network execution at batch 256, per image
# (one ncu capture on a B200; the algorithmic bytes of the same launches are 25.4 MB per image)
NCU_DRAM_BYTES_PER_IMAGE_CONV_TC = 18.27e6
NCU_TRAFFIC_BATCH = 256


def cpu_baseline(batch_images, threads=0):
    """The reference arithmetic on the host cores, on a bounded sample (whole ResNet-50, `batch_images` images): the
    convolutions run the reference's own kernel source compiled as C++ when oracle/_ref holds the prebuilt variants,
    otherwise the C restatement; `kind` says which."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import numpy as np
    import oracle_lib
    import oracle_net
    from cldnn_b200 import topologies
    spec = topologies.resnet50_int8(batch_images)
    lay = spec.input_layout
    x = np.random.default_rng(1).integers(0, 256, size=(lay.size.batch, lay.size.feature, lay.size.y, lay.size.x)).astype(np.uint8)
    cores = threads or oracle_lib.num_threads()
    stats = {}
    t0 = time.perf_counter()
    oracle_net.run(spec, {spec.input_id: x}, threads=cores, stats=stats, conv_impl="reference")
    dt = time.perf_counter() - t0
    nref = stats.get("reference_kernel_convs", 0)
    # "reference": all 53 convolutions ran the reference's own kernel source (fused_conv_eltwise_gpu_ref.cl compiled as C++);
    # pooling, the 2048x1000 inner product and softmax (0.05 % of the work) run the C restatement
    return dict(value=batch_images / dt, unit=UNIT, cores=cores, kind="reference" if nref >= 53 else "port",
                sample="full ResNet-50 v1 int8 forward, %d images of 224x224, %.1f s, %d convolutions on the reference kernel source" % (batch_images, dt, nref))


def shard_plan(global_images, world):
    """Images are independent units: rank r takes global_images // world, the remainder goes to the low ranks."""
    base, rem = divmod(global_images, world)
    return [base + (1 if r < rem else 0) for r in range(world)]


def max_over_ranks(ms, world, device="cpu"):
    """Device time of the slowest rank (no other collective exists on the path)."""
    if world == 1:
        return ms
    import torch
    import torch.distributed as dist
    t = torch.tensor([ms], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def whole_job_rate(images_per_rank, steps, ms):
    return sum(images_per_rank) * steps / (ms / 1e3)


def run_reference(args, rank):
    """--impl reference: the reference's arithmetic on the box's host cores (rank 0 only)."""
    if rank != 0:
        return
    vals = []
    for _ in range(args.warmup if args.warmup < 1 else 1):
        cpu_baseline(1)
    t0 = time.perf_counter()
    last = None
    for _ in range(args.steps):
        last = cpu_baseline(args.cpu_sample)
        vals.append(last["value"])
    dt = time.perf_counter() - t0
    value = args.steps * args.cpu_sample / dt
    line = {"impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": {"workload": "resnet50_v1_int8", "batch_per_step": args.cpu_sample, "image": 224,
                       "note": "the reference's convolution kernel source compiled for the host cores (no OpenCL device exists here); each step is a bounded sample"},
            "cpu_baseline": dict(last, value=value),
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def main():
    args = parse()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if args.impl == "reference":
        run_reference(args, rank)
        return

    import numpy as np
    import torch
    import torch.distributed as dist
    from cldnn_b200 import cldnn as cl
    from cldnn_b200 import topologies

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the engine has no CPU fallback (use --impl reference for the CPU arithmetic)")
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_DEBUG", "WARN")             # keep stdout to the one JSON line
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    B = args.batch
    peaks = read_peaks()
    spec = topologies.resnet50_int8(B)
    total_ops, per_layer = topologies.conv_ops(spec)            # per image

    def build(profiling):
        eng = cl.engine(local_rank, enable_profiling=profiling)
        topo, keep = spec.realise(eng)
        # tile shapes: start from the cache shipped with the package (tuned on a B200, keyed by SM count like the
        # reference's cache.json); shapes it does not know are timed on the device now and added to a scratch copy
        cache = os.path.join(ROOT, "gpurun_out", "tuning_cache_rank%d.json" % rank)
        os.makedirs(os.path.dirname(cache), exist_ok=True)
        shipped = os.path.join(ROOT, "cldnn_b200", "cache", "tuning_cache.json")
        if args.retune and not profiling and os.path.exists(cache):
            os.remove(cache)
        if not args.retune and not os.path.exists(cache) and os.path.exists(shipped):
            import shutil
            shutil.copyfile(shipped, cache)
        opts = cl.build_options(optimize_data=True, outputs=["prob"],
                                tuning=cl.tuning_mode.tuning_tune_and_cache if args.tune else cl.tuning_mode.tuning_disabled,
                                tuning_cache_path=cache)
        net = cl.network(eng, topo, opts)
        stream = torch.cuda.ExternalStream(eng.stream(), device=local_rank)
        x_dev = torch.empty((B, 3, 224, 224), dtype=torch.uint8, device="cuda")
        net.set_input_data(spec.input_id, cl.memory.attach(eng, spec.input_layout, x_dev.data_ptr()))
        return eng, net, stream, x_dev, keep

    eng, net, stream, x_dev, keep = build(False)
    gen = torch.Generator(device="cpu").manual_seed(1234 + rank)
    n_resident = 4                                                   # 4 x 38.5 MB at batch 256 > 126 MB of L2
    host = [torch.randint(0, 256, (B, 3, 224, 224), dtype=torch.uint8, generator=gen).pin_memory() for _ in range(n_resident)]
    resident = [h.cuda() for h in host]
    torch.cuda.synchronize()

    def step_resident(i):
        with torch.cuda.stream(stream):
            x_dev.copy_(resident[i % n_resident], non_blocking=True)
        net.execute()

    out_mem = None
    prob_host = torch.empty((B, 1000), dtype=torch.float32).pin_memory()

    # End to end through the public API: every step's images start in pinned host memory and its probabilities end there.
    # The host->device copy of step i+1 runs on a copy stream into one of two staging buffers while step i computes; the
    # network's bound input is refilled from the staging buffer by a device-to-device copy on the compute stream.
    copy_stream = torch.cuda.Stream(device=local_rank)
    staging = [torch.empty((B, 3, 224, 224), dtype=torch.uint8, device="cuda") for _ in range(2)]
    staged = [torch.cuda.Event() for _ in range(2)]       # host->device copy into staging[k] has finished
    consumed = [torch.cuda.Event() for _ in range(2)]     # staging[k] has been copied into the network input
    e2e_state = {"primed": -1}

    def _stage(i):
        k = i % 2
        with torch.cuda.stream(copy_stream):
            copy_stream.wait_event(consumed[k])
            staging[k].copy_(host[i % n_resident], non_blocking=True)
            staged[k].record(copy_stream)

    def step_e2e(i):
        if e2e_state["primed"] != i:                          # first step of a run: nothing was prefetched for it
            _stage(i)
        k = i % 2
        with torch.cuda.stream(stream):
            stream.wait_event(staged[k])
            x_dev.copy_(staging[k], non_blocking=True)
            consumed[k].record(stream)
        _stage(i + 1)                                         # next step's images travel while this step computes
        e2e_state["primed"] = i + 1
        net.execute()
        with torch.cuda.stream(stream):
            prob_host.copy_(prob_dev, non_blocking=True)

    # first execution builds the launches (and tunes); then find the output buffer
    step_resident(0)
    out_mem = net.get_output("prob")
    prob_dev = torch.empty(0)
    # view the network's output buffer as a torch tensor for the asynchronous read-back
    import ctypes
    class _Holder:  # minimal __cuda_array_interface__ provider
        def __init__(self, ptr, shape):
            self.__cuda_array_interface__ = {"shape": shape, "typestr": "<f4", "data": (ptr, False), "version": 3}
    prob_dev = torch.as_tensor(_Holder(out_mem.device_ptr(), (B, 1000)), device="cuda")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(step_fn, steps, warmup):
        for i in range(warmup):
            step_fn(i)
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            a.record(stream)
        for i in range(steps):
            step_fn(warmup + i)
        with torch.cuda.stream(stream):
            b.record(stream)
        torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        barrier()
        return max_over_ranks(ms, world, "cuda")

    sampler = ClockSampler(local_rank)
    sampler.start()
    ms = timed(step_resident, args.steps, max(args.warmup, 3))
    clocks = sampler.finish()
    ms_e2e = timed(step_e2e, args.steps, 3)
    launches_per_step = net.stats()["launches_per_execute"]

    # per-primitive device time (CUDA events around every launch on the engine's stream) for the roofline of the dominant kernel
    roof = None
    if rank == 0:
        del net
        engp, netp, streamp, x_devp, keepp = build(True)
        with torch.cuda.stream(streamp):
            x_devp.copy_(resident[0])
        for _ in range(3):
            netp.execute()
        acc = {}
        reps = 5
        for r in range(reps):
            with torch.cuda.stream(streamp):
                x_devp.copy_(resident[r % n_resident])
            netp.execute()
            for k, v in netp.profiling_info().items():
                acc[k] = acc.get(k, 0) + v
        info = {r["id"]: r for r in netp.primitives_info()}
        tc_ns = sum(v for k, v in acc.items() if info[k]["kernel"] == "conv_i8_tc") / reps
        all_ns = sum(acc.values()) / reps
        ops_by_id = {pid: ops for pid, kind, ops, shape in per_layer}
        tc_ops = sum(ops_by_id.get(k, 0) for k in acc if info[k]["kernel"] == "conv_i8_tc") * B
        k3_ns = sum(v for k, v in acc.items() if k.endswith("_b") and info[k]["kernel"] == "conv_i8_tc") / reps
        k3_ops = sum(ops_by_id.get(k, 0) for k in acc if k.endswith("_b")) * B
        int8_peak = 2.0 * peaks["bf16_sustained"]                    # TOPS; no int8 figure is measured on this pool
        achieved = tc_ops / tc_ns / 1e3                              # ops/ns = Gop/s; /1e3 -> TOPS
        roof = {"bound": "tensor", "kernel": "conv_i8_tc", "achieved": achieved, "peak": int8_peak, "unit": "TFLOP/s", "frac": achieved / int8_peak,
                "traffic": NCU_DRAM_BYTES_PER_IMAGE_CONV_TC * B if B == NCU_TRAFFIC_BATCH else None,
                "traffic_note": "dram read+write bytes of the conv_i8_tc launches of one step, from the ncu capture summarised in "
                                "profiles/conv_i8_tc_dram_traffic_b256.md (batch 256; not scaled to other batch sizes because the L2 share changes)",
                "peak_source": "2 x bf16_tflops_sustained of %s MEASURED_PEAKS (dense int8 : bf16 = 2 : 1)" % peaks["source"],
                "launches_per_step": sum(1 for k in acc if info[k]["kernel"] == "conv_i8_tc"),
                "share_of_step": tc_ns / all_ns,
                "conv3x3_tops": k3_ops / k3_ns / 1e3, "conv3x3_frac": k3_ops / k3_ns / 1e3 / int8_peak,
                "per_kernel_ms": {kern: sum(v for k, v in acc.items() if info[k]["kernel"] == kern) / reps / 1e6
                                  for kern in sorted(set(r["kernel"] for r in info.values() if r["kernel"]))}}

    per_rank = shard_plan(B * world, world)
    images = sum(per_rank) * args.steps
    value = whole_job_rate(per_rank, args.steps, ms)
    line = {"metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "u8", "data": "synthetic",
            "config": {"workload": "resnet50_v1_int8_b%d" % B, "batch_per_gpu": B, "global_batch": B * world, "image": 224, "parallelism": "dp%d" % world,
                       "l2": "each step reads a different one of %d resident batches (%.0f MB total > 126 MB L2); activations per step exceed L2" % (n_resident, n_resident * B * 3 * 224 * 224 / 1e6),
                       "ops_per_image": total_ops},
            "clocks": clocks,
            "e2e": {"value": images / (ms_e2e / 1e3), "unit": UNIT, "h2d_bytes_per_step": B * 3 * 224 * 224 * world, "d2h_bytes_per_step": B * 1000 * 4 * world,
                    "ms_per_step": ms_e2e / args.steps},
            "gpu_launches": int(launches_per_step) * args.steps}
    if rank == 0:
        line["roofline"] = roof
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(args.cpu_sample)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
