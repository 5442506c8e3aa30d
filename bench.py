#!/usr/bin/env python
"""Inference throughput of the benchmark configurations on N B200s (pure data parallelism, one process per GPU).

    python bench.py --gpus 1 --steps 20 --warmup 5                      # ResNet-50 v1 int8, batch 256 per GPU (the headline)
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...
    python bench.py --config mobilenet_v2_int8 | alexnet_fp16 | alexnet_int8 | vgg16_fp16 | vgg16_fp16_layers
    python bench.py --impl reference ...      # the reference arithmetic on the host cores (CPU oracle)

One step = one forward pass of the whole network over one batch of synthetic images.  Rank 0 prints one JSON line.
`value` is measured with the batch resident in HBM (rotating over several resident batches so that no step finds its
input in L2); `e2e` includes, every step, the copy of a fresh batch from pinned host memory and the read-back of the
class probabilities.  The timed region of K steps is repeated until at least --min-seconds have been measured; the line
reports the median repeat (and the fastest and slowest).  After the timed regions, outside them, rank 0 checks the very
network it timed against the CPU oracle on the first images of a batch (`parity`) and times every primitive on a
profiling engine (`per_primitive`, `roofline`).
"""
import argparse
import json
import os
import sys
import tempfile
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

UNIT = "images/s"

# name: (topology constructor name, default batch per GPU, metric, arithmetic type, images checked against the oracle)
CONFIGS = {
    "resnet50_int8": ("resnet50_int8", 256, "ResNet-50 int8 images/s", "u8", 8),
    "mobilenet_v2_int8": ("mobilenet_v2_int8", 128, "MobileNet-v2 int8 images/s", "u8", 8),
    "alexnet_int8": ("alexnet_int8", 256, "AlexNet int8 images/s", "u8", 8),
    "alexnet_fp16": ("alexnet_fp16", 256, "AlexNet fp16 images/s", "f16", 8),
    "vgg16_fp16": ("vgg16_fp16", 32, "VGG16 fp16 images/s", "f16", 1),
}
HBM_KERNELS = ("conv_i8_first", "conv_first_tc", "conv_i8_dw", "pooling_i8_byxf", "pooling_f16_byxf", "pooling_ref", "lrn_f16_byxf", "lrn_ref",
               "softmax", "eltwise_ref", "eltwise_byxf", "reorder_ref", "activation_ref", "concatenation")


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--batch", type=int, default=0, help="images per GPU per step (default: the configuration's own)")
    ap.add_argument("--config", default="resnet50_int8", choices=sorted(CONFIGS) + ["vgg16_fp16_layers"])
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--tune", type=int, default=1, help="1: pick tile shapes from on-device timings at build")
    ap.add_argument("--retune", action="store_true", help="ignore the tuning cache shipped with the package: time every tile shape on this device")
    ap.add_argument("--save-cache", default="", help="write the tuning cache this run ended with to this file")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU oracle leg (no cpu_baseline, no parity)")
    ap.add_argument("--cpu-sample", type=int, default=0, help="images in the CPU baseline / parity sample (default: per configuration)")
    ap.add_argument("--min-seconds", type=float, default=1.0, help="repeat the timed region of K steps until this much device time is measured")
    ap.add_argument("--table", default="", help="also write the per-primitive table as markdown to this file")
    return ap.parse_args()


def read_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p.get("hbm_gbs"), bf16_sustained=p.get("bf16_tflops_sustained"), bf16_burst=p.get("bf16_tflops"), source="measured")
    return dict(hbm_gbs=6650.0, bf16_sustained=1400.0, bf16_burst=1590.0, source="fallback")


def host_cores():
    """Cores this process may run on.  (OMP_NUM_THREADS is no guide: torchrun sets it to 1 for every rank.)"""
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return max(1, os.cpu_count() or 1)


class ClockSampler(threading.Thread):
    """SM clock and throttle reasons of the measured GPU while the timed regions run (NVML, read-only).  The NVML handle
    is resolved from the CUDA device's UUID / PCI address: NVML indices ignore CUDA_VISIBLE_DEVICES."""

    def __init__(self, cuda_index):
        super().__init__(daemon=True)
        self.samples, self.reasons, self.max_mhz, self._stop_evt, self.how = [], set(), None, threading.Event(), None
        try:
            import pynvml
            import torch
            pynvml.nvmlInit()
            self.nv = pynvml
            prop = torch.cuda.get_device_properties(cuda_index)
            self.h = None
            try:
                u = str(prop.uuid)
                self.h = pynvml.nvmlDeviceGetHandleByUUID((u if u.startswith("GPU-") else "GPU-" + u).encode())
                self.how = "uuid"
            except Exception:
                try:
                    bus = "%08x:%02x:%02x.0" % (prop.pci_domain_id, prop.pci_bus_id, prop.pci_device_id)
                    self.h = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
                    self.how = "pci"
                except Exception:
                    self.h = pynvml.nvmlDeviceGetHandleByIndex(cuda_index)
                    self.how = "index"
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def run(self):
        if self.nv is None:
            return
        nv = self.nv
        names = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}
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
        return dict(sm_mhz=s[len(s) // 2] if s else None, sm_min_mhz=s[0] if s else None, sm_max_mhz=self.max_mhz, reasons=sorted(self.reasons),
                    samples=len(s), device_by=self.how)


# dram__bytes_read.sum + dram__bytes_write.sum of the 53 conv_i8_tc launches of one ResNet-50 execution at batch 256, per image
# (one ncu capture on a B200; the algorithmic bytes of the same launches are 25.4 MB per image)
NCU_DRAM_BYTES_PER_IMAGE_CONV_TC = 18.27e6
NCU_TRAFFIC_BATCH = 256


def make_spec(config, batch):
    from cldnn_b200 import topologies
    return getattr(topologies, CONFIGS[config][0])(batch)


def synthetic_images(spec, n, seed):
    """u8 images uniform in [0, 255] or fp16 images N(0, 1), as the configuration says, in the caller's bfyx layout."""
    import numpy as np
    from cldnn_b200 import cldnn as cl
    lay = spec.input_layout
    shape = (n, lay.size.feature, lay.size.y, lay.size.x)
    rng = np.random.default_rng(seed)
    if lay.data_type == cl.data_types.u8:
        return rng.integers(0, 256, size=shape, dtype=np.int64).astype(np.uint8)
    return rng.standard_normal(shape).astype(np.float16)


def oracle_forward(config, x, threads=0):
    """The reference arithmetic on the host cores for the images `x` of `config`: the convolutions run the reference's own
    kernel source compiled as C++ when oracle/_ref holds the prebuilt variants, otherwise the C restatement.
    Returns (outputs by id, seconds, convolutions that ran the reference's source, convolutions in all)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_net
    spec = make_spec(config, x.shape[0])
    stats = {}
    t0 = time.perf_counter()
    out = oracle_net.run(spec, {spec.input_id: x}, threads=threads or host_cores(), stats=stats, conv_impl="reference",
                         fuse_activations=config == "mobilenet_v2_int8")
    dt = time.perf_counter() - t0
    nconv = sum(1 for p in spec.prims if p.kind in ("convolution", "fused_conv_eltwise"))
    return out, dt, stats.get("reference_kernel_convs", 0), nconv


def cpu_baseline_record(config, images, dt, nref, nconv, cores):
    # "reference": every convolution ran the reference's own kernel source (fused_conv_eltwise_gpu_ref.cl compiled as C++);
    # pooling, inner products and softmax (well under 1 % of the work) run the C restatement
    return dict(value=images / dt, unit=UNIT, cores=cores, kind="reference" if nref >= nconv else "port",
                sample="full %s forward, %d images, %.1f s, %d of %d convolutions on the reference kernel source" % (config, images, dt, nref, nconv))


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
    config = args.config if args.config in CONFIGS else "vgg16_fp16"
    sample = args.cpu_sample or CONFIGS[config][4]
    cores = host_cores()
    spec1 = make_spec(config, 1)
    for _ in range(1 if args.warmup > 0 else 0):
        oracle_forward(config, synthetic_images(spec1, 1, 1), cores)
    x = synthetic_images(spec1, sample, 1)
    t0 = time.perf_counter()
    last = None
    for _ in range(args.steps):
        _, dt, nref, nconv = oracle_forward(config, x, cores)
        last = cpu_baseline_record(config, sample, dt, nref, nconv, cores)
    dt = time.perf_counter() - t0
    value = args.steps * sample / dt
    line = {"impl": "reference", "metric": CONFIGS[config][2], "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": CONFIGS[config][3], "data": "synthetic",
            "config": {"workload": config, "batch_per_step": sample,
                       "note": "the reference's convolution kernel source compiled for the host cores (no OpenCL device exists here); each step is a bounded sample"},
            "cpu_baseline": dict(last, value=value),
            "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def primitive_table(spec, info_rows, times_ns, batch, peaks):
    """Per executed primitive: kernel, tile choice, device time, and the achieved rate against the roofline that bounds it.
    Operations: 2 x multiply-adds of the direct form (padding taps counted); bytes: every input, constant and output once."""
    import numpy as np
    from cldnn_b200 import topologies
    _, per_layer = topologies.conv_ops(spec)
    ops_by_id = {pid: ops for pid, kind, ops, shape in per_layer}
    inputs, wbytes = topologies.primitive_inputs(spec), topologies.weight_bytes(spec)
    info = {r["id"]: r for r in info_rows}
    absorbed = {}                                               # id fused away -> the primitive that now computes it
    for r in info_rows:
        for f in r["fused"]:
            absorbed[f] = r["id"]
    dt_bytes = lambda code: max(1, code & 0x0f)

    def out_bytes(pid):
        r = info.get(absorbed.get(pid, pid))
        if r is None:                                           # the network input
            lay = spec.input_layout
            return batch * lay.size.feature * lay.size.y * lay.size.x * dt_bytes(int(lay.data_type))
        return int(np.prod(r["dims"])) * dt_bytes(r["data_type"])

    rows = []
    for pid, ns in times_ns.items():
        r = info[pid]
        group = [pid] + r["fused"]
        ops = sum(ops_by_id.get(g, 0) for g in group) * batch
        ext_in = []
        for g in group:
            for i in inputs.get(g, []):
                if i not in group and absorbed.get(i, i) != pid and i not in ext_in:
                    ext_in.append(i)
        if not ext_in and pid.endswith("_to_byxf_af32"):
            ext_in = [pid[:-len("_to_byxf_af32")]]
        if not ext_in and pid.endswith("_from_byxf_af32"):
            ext_in = [pid[:-len("_from_byxf_af32")]]
        nbytes = sum(out_bytes(i) for i in ext_in) + sum(wbytes.get(g, 0) for g in group) + out_bytes(pid)
        row = {"id": pid, "type": r["type"], "kernel": r["kernel"], "tune": r["tune"], "out": list(r["dims"]), "us": ns / 1e3, "mbytes": nbytes / 1e6,
               "gbs": nbytes / ns, "hbm_frac": nbytes / ns / peaks["hbm_gbs"]}
        if ops:
            row["gop"] = ops / 1e9
            row["tops"] = ops / ns / 1e3
        rows.append(row)
    return rows


def table_markdown(title, rows, peaks_note):
    out = ["# " + title, "", peaks_note, "",
           "| primitive | kernel | tune | output (b,f,y,x) | us | Gop | TOPS | of tensor peak | MB | GB/s | of HBM |", "|---|---|---|---|---|---|---|---|---|---|---|"]
    for r in rows:
        out.append("| %s | %s | %d | %s | %.1f | %s | %s | %s | %.1f | %.0f | %.2f |" % (
            r["id"], r["kernel"], r["tune"], "x".join(str(v) for v in r["out"]), r["us"], "%.1f" % r["gop"] if "gop" in r else "",
            "%.0f" % r["tops"] if "tops" in r else "", "%.2f" % r["tensor_frac"] if "tensor_frac" in r else "", r["mbytes"], r["gbs"], r["hbm_frac"]))
    return "\n".join(out) + "\n"


def run_vgg_layers(args, peaks):
    """The layer benchmark of the reference's Winograd kernels: the 13 3x3 layers of VGG16 at batch 32, fp16, direct tensor-core kernel against the Winograd
    F(2x2, 3x3) path, each on its best tile shape; TFLOP/s on the direct form's operation count for both."""
    import ctypes as C
    import numpy as np
    from cldnn_b200 import abi, engine as eng, topologies
    batch = args.batch or 32
    E = eng.Engine(0)
    rng = np.random.default_rng(16)
    f16_peak = E.tensor_peak(abi.F16, 256)
    rows = []

    def best_of(kernel, p, args_for, runs=20):
        k = E.kernel(kernel)
        if not k.supports(p):
            return None
        # one workspace for every tile shape / variant of the kernel: the largest any of them asks for
        tunes, sb = [], C.c_size_t()
        need = 0
        for tune in range(1 if k.tune_count(p) > 1 else 0, k.tune_count(p)):
            q = abi.ConvParams.from_buffer_copy(bytes(p))
            q.tune = tune
            if not k.supports(q):
                continue
            E.lib.cldnn_b200_kernel_scratch_bytes(k.handle, C.byref(q), C.sizeof(q), C.byref(sb))
            need = max(need, sb.value)
            tunes.append(q)
        sb = C.c_size_t(need)
        scratch = E.alloc(need) if need else None
        best = None
        for q in tunes:
            tune = q.tune
            pr = k.prepare(q, args_for(scratch))
            ns = pr.time_ns(3, runs)
            pr.destroy()
            if best is None or ns < best[0]:
                best = (ns, tune, sb.value)
        if scratch is not None:
            scratch.free()
        return best

    for name, cin, cout, size in topologies.vgg16_conv_layers():
        planar = cin <= 4                                           # the image layer: planar input read in place
        p = abi.ConvParams()
        p.in_, n_in = abi.tensor(abi.F16, batch, cin, size, size, "bfyx" if planar else "byxf", 1 if planar else 16)
        p.out, n_out = abi.tensor(abi.F16, batch, cout, size, size, "byxf", 16)
        abi.set_weights(p, abi.F16, 1, cout, cin, 3, 3, "oiyx" if planar else "oyxi", *(() if planar else (16,)))
        p.stride_x = p.stride_y = p.dil_x = p.dil_y = 1
        p.pad_x = p.pad_y = 1
        p.bias_dtype, p.act = abi.F32, abi.ACT_RELU
        p.eltw_stride_x = p.eltw_stride_y = 1
        p.i_qf = p.o_qf = 1.0
        cs = cin if planar else -(-cin // 16) * 16
        x = np.zeros(n_in, dtype=np.float16)
        if planar:
            x[:] = rng.standard_normal(n_in).astype(np.float16)
            w = (rng.standard_normal(cout * cin * 9) * np.sqrt(2.0 / (cin * 9))).astype(np.float16)
        else:
            x.reshape(batch, size, size, cs)[..., :cin] = rng.standard_normal((batch, size, size, cin)).astype(np.float16)
            wp = np.zeros((cout, 3, 3, cs), dtype=np.float16)
            wp[..., :cin] = (rng.standard_normal((cout, 3, 3, cin)) * np.sqrt(2.0 / (cin * 9))).astype(np.float16)
            w = wp.reshape(-1)
        bias = (rng.standard_normal(cout) * 0.05).astype(np.float32)
        mx, mw, mb, mo = E.upload(x), E.upload(w), E.upload(bias), E.alloc(n_out * 2)
        flops = 2.0 * batch * size * size * cout * cin * 9
        res = {"layer": name, "features_in": cin, "features_out": cout, "map": size, "gflop": flops / 1e9}
        for kernel in (("conv_first_tc",) if planar else ("conv_f16_tc", "conv_f16_winograd")):
            b = best_of(kernel, p, lambda scratch: eng.make_args(input0=mx, output=mo, weights=mw, bias=mb, scratch=scratch))
            if b:
                res[kernel] = {"us": b[0] / 1e3, "tune": b[1], "tflops": flops / b[0] / 1e3, "of_f16_peak": flops / b[0] / 1e3 / f16_peak, "scratch_mb": b[2] / 1e6}
        assert E.device_status() == 0
        rows.append(res)
        for m in (mx, mw, mb, mo):
            m.free()
    direct_us = sum(r.get("conv_f16_tc", r.get("conv_first_tc"))["us"] for r in rows)
    best_us = sum(min(v["us"] for k, v in r.items() if isinstance(v, dict)) for r in rows)
    total = sum(r["gflop"] for r in rows)
    value = total / best_us * 1e3
    line = {"metric": "VGG16 fp16 conv sweep TFLOP/s (best of direct and Winograd per layer, direct-form operation count)", "value": value, "unit": "TFLOP/s",
            "n_gpus": 1, "steps": 20, "warmup": 3, "ms_per_step": best_us / 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16", "data": "synthetic", "config": {"workload": "vgg16_fp16_layers_b%d" % batch, "batch": batch, "l2": "every layer's tensors exceed L2 except the 14x14 stage"},
            "direct_tflops": total / direct_us * 1e3, "winograd_wins": [r["layer"] for r in rows if "conv_f16_winograd" in r and r["conv_f16_winograd"]["us"] < r["conv_f16_tc"]["us"]],
            "roofline": {"bound": "tensor", "kernel": "conv_f16_tc", "achieved": value, "peak": f16_peak, "unit": "TFLOP/s", "frac": value / f16_peak,
                         "peak_source": "tcgen05 kind::f16 N=256 micro-kernel on this device (cldnn_b200_tensor_peak); cuBLAS bf16 burst of MEASURED_PEAKS: %s" % peaks["bf16_burst"],
                         "traffic": None},
            "layers": rows, "gpu_launches": int(E.launch_count())}
    print(json.dumps(line), flush=True)
    E.close()


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
    from cldnn_b200 import abi
    from cldnn_b200 import cldnn as cl
    from cldnn_b200 import topologies

    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the engine has no CPU fallback (use --impl reference for the CPU arithmetic)")
    peaks = read_peaks()
    if args.config == "vgg16_fp16_layers":
        if rank == 0:
            run_vgg_layers(args, peaks)
        return
    torch.cuda.set_device(local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("NCCL_DEBUG", "WARN")             # keep stdout to the one JSON line
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    config = args.config
    _, default_batch, metric, dtype, parity_images = CONFIGS[config]
    B = args.batch or default_batch
    spec = make_spec(config, B)
    total_ops, per_layer = topologies.conv_ops(spec)            # per image
    lay = spec.input_layout
    in_shape = (B, lay.size.feature, lay.size.y, lay.size.x)
    in_torch = torch.uint8 if lay.data_type == cl.data_types.u8 else torch.float16
    in_bytes = int(np.prod(in_shape)) * (1 if in_torch == torch.uint8 else 2)
    out_ids = list(spec.outputs)                                # class probabilities first, then the logits

    # tile shapes: start from the cache shipped with the package (tuned on a B200, keyed by SM count like the reference's
    # cache.json); shapes it does not know are timed on the device now and added to a private scratch copy
    workdir = tempfile.mkdtemp(prefix="cldnn_b200_bench_")
    cache = os.path.join(workdir, "tuning_cache_rank%d.json" % rank)
    shipped = os.path.join(ROOT, "cldnn_b200", "cache", "tuning_cache.json")
    if not args.retune and os.path.exists(shipped):
        import shutil
        shutil.copyfile(shipped, cache)

    def build(profiling):
        eng = cl.engine(local_rank, enable_profiling=profiling)
        topo, keep = spec.realise(eng)
        opts = cl.build_options(optimize_data=True, outputs=out_ids,
                                tuning=cl.tuning_mode.tuning_tune_and_cache if args.tune else cl.tuning_mode.tuning_disabled,
                                tuning_cache_path=cache)
        net = cl.network(eng, topo, opts)
        stream = torch.cuda.ExternalStream(eng.stream(), device=local_rank)
        x_dev = torch.empty(in_shape, dtype=in_torch, device="cuda")
        net.set_input_data(spec.input_id, cl.memory.attach(eng, spec.input_layout, x_dev.data_ptr()))
        return eng, net, stream, x_dev, keep

    eng, net, stream, x_dev, keep = build(False)
    n_resident = max(4, -(-3 * 126_000_000 // (2 * in_bytes)))       # the resident batches together exceed L2 (126 MB)
    n_resident = min(n_resident, 16)
    host = [torch.from_numpy(synthetic_images(spec, B, 1234 + 100 * rank + i)).pin_memory() for i in range(n_resident)]
    resident = [h.cuda() for h in host]
    torch.cuda.synchronize()

    def step_resident(i):
        with torch.cuda.stream(stream):
            x_dev.copy_(resident[i % n_resident], non_blocking=True)
        net.execute()

    # End to end through the public API: every step's images start in pinned host memory and its probabilities end there.
    # The host->device copy of step i+1 runs on a copy stream into one of two staging buffers while step i computes; the
    # network's bound input is refilled from the staging buffer by a device-to-device copy on the compute stream.
    copy_stream = torch.cuda.Stream(device=local_rank)
    staging = [torch.empty(in_shape, dtype=in_torch, device="cuda") for _ in range(2)]
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

    # first execution builds the launches (and tunes); then view the output buffer as a torch tensor for the read-back
    step_resident(0)
    out_mem = net.get_output(out_ids[0])
    out_lay = out_mem.get_layout()
    out_np = out_lay.np_dtype()
    n_out = out_lay.size.batch * out_lay.size.feature * out_lay.size.y * out_lay.size.x

    class _Holder:  # minimal __cuda_array_interface__ provider
        def __init__(self, ptr, shape, typestr):
            self.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (ptr, False), "version": 3}
    prob_dev = torch.as_tensor(_Holder(out_mem.device_ptr(), (n_out,), np.dtype(out_np).str), device="cuda")
    prob_host = torch.empty((n_out,), dtype=prob_dev.dtype).pin_memory()
    out_bytes = n_out * prob_dev.element_size()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed_once(step_fn, steps, first):
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            a.record(stream)
        for i in range(steps):
            step_fn(first + i)
        with torch.cuda.stream(stream):
            b.record(stream)
        torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        barrier()
        return max_over_ranks(ms, world, "cuda")

    def timed(step_fn, steps, warmup, min_seconds):
        """Warm up, then time regions of exactly `steps` steps until `min_seconds` of device time have been measured
        (every rank sees the same max-over-ranks times, so every rank repeats the same number of regions)."""
        for i in range(warmup):
            step_fn(i)
        times, n = [], warmup
        while True:
            times.append(timed_once(step_fn, steps, n))
            n += steps
            if sum(times) >= min_seconds * 1e3 or len(times) >= 200:
                break
        s = sorted(times)
        return s[len(s) // 2], s[0], s[-1], len(s)

    warm = max(args.warmup, 3)
    sampler = ClockSampler(local_rank)
    sampler.start()
    ms, ms_min, ms_max, reps = timed(step_resident, args.steps, warm, args.min_seconds)
    clocks = sampler.finish()
    ms_e2e, e2e_min, e2e_max, e2e_reps = timed(step_e2e, args.steps, 3, args.min_seconds)
    launches_per_step = net.stats()["launches_per_execute"]

    roof = parity = cpu = None
    table = []
    if rank == 0:
        # ---- parity of the very network that was timed: its first images against the CPU oracle (outside the timed regions)
        n_par = 0 if args.no_cpu_baseline else min(args.cpu_sample or parity_images, B)
        if n_par:
            with torch.cuda.stream(stream):
                x_dev.copy_(resident[0], non_blocking=True)
            net.execute()
            got = {o: net.get_output(o).to_numpy() for o in out_ids}
            want, dt_cpu, nref, nconv = oracle_forward(config, host[0][:n_par].numpy())
            cpu = cpu_baseline_record(config, n_par, dt_cpu, nref, nconv, host_cores())
            parity = {"images": n_par, "batch": B, "against": "CPU oracle (%s)" % cpu["kind"]}
            ok = True
            for o in out_ids:
                w, g = want[o], got[o][:n_par]
                if w.dtype.kind in "iu":
                    bad = int((w != g).sum())
                    parity["%s_mismatches" % o] = bad
                    parity["%s_distinct_values" % o] = int(len(np.unique(w)))
                    ok &= bad == 0
                else:
                    w32, g32 = w.astype(np.float32), g.astype(np.float32)
                    scale = float(np.abs(w32).max())
                    rel = float(np.abs(g32 - w32).max() / scale) if scale > 0 else 0.0
                    parity["%s_max_rel" % o] = rel
                    # integer networks: the float tail (softmax of exact logits) differs by exp() rounding only; fp16: 1e-2
                    ok &= rel <= (1e-4 if dtype == "u8" else 1e-2)
            parity["ok"] = bool(ok)
        # ---- per-primitive device time (CUDA events around every launch on the engine's stream, profiling engine, same
        # tuned build) for the roofline of the dominant kernel
        del net
        engp, netp, streamp, x_devp, keepp = build(True)
        with torch.cuda.stream(streamp):
            x_devp.copy_(resident[0])
        for _ in range(3):
            netp.execute()
        acc, nrep = {}, 5
        for r in range(nrep):
            with torch.cuda.stream(streamp):
                x_devp.copy_(resident[r % n_resident])
            netp.execute()
            for k, v in netp.profiling_info().items():
                acc[k] = acc.get(k, 0) + v
        times_ns = {k: v / nrep for k, v in acc.items()}
        info_rows = netp.primitives_info()
        table = primitive_table(spec, info_rows, times_ns, B, peaks)
        half = dtype == "f16"
        tc_kernel = "conv_f16_tc" if half else "conv_i8_tc"
        from cldnn_b200 import engine as seam             # the engine seam: measured tensor peak of this device
        seam_eng = seam.Engine(local_rank)
        peak_measured = seam_eng.tensor_peak(abi.F16 if half else abi.I8, 256)
        seam_eng.close()
        peak_assumed = (1.0 if half else 2.0) * peaks["bf16_sustained"]
        for r in table:
            if "tops" in r and r["kernel"] not in HBM_KERNELS:
                r["tensor_frac"] = r["tops"] / peak_measured
                r["tensor_frac_vs_bf16"] = r["tops"] / peak_assumed
        tc = [r for r in table if r["kernel"] == tc_kernel]
        tc_us, tc_ops = sum(r["us"] for r in tc), sum(r.get("gop", 0) for r in tc)
        all_us = sum(r["us"] for r in table)
        k3 = [r for r in tc if r["id"].endswith("_b")]
        achieved = tc_ops / tc_us * 1e3 if tc_us else 0.0           # Gop / us = 1e15 op/s = 1000 TOPS
        per_kernel = {}
        for r in table:
            d = per_kernel.setdefault(r["kernel"], {"ms": 0.0, "launches": 0, "mbytes": 0.0})
            d["ms"] += r["us"] / 1e3
            d["launches"] += 1
            d["mbytes"] += r["mbytes"]
        for kname, d in per_kernel.items():
            d["share"] = d["ms"] * 1e3 / all_us
            if kname in HBM_KERNELS:
                d["gbs"] = d["mbytes"] / d["ms"]                    # MB / ms = GB/s
                d["hbm_frac"] = d["gbs"] / peaks["hbm_gbs"]
        roof = {"bound": "tensor", "kernel": tc_kernel, "achieved": achieved, "peak": peak_assumed, "unit": "TFLOP/s", "frac": achieved / peak_assumed,
                "peak_source": "%s x bf16_tflops_sustained of %s MEASURED_PEAKS (of %s)" % ("1" if half else "2", peaks["source"], peaks["source"]),
                "tensor_peak_measured": peak_measured, "frac_of_tensor_peak_measured": achieved / peak_measured,
                "tensor_peak_measured_how": "cldnn_b200_tensor_peak: tcgen05.mma M128 N256, operands resident in shared memory, all SMs, CUDA events",
                "traffic": NCU_DRAM_BYTES_PER_IMAGE_CONV_TC * B if (config == "resnet50_int8" and B == NCU_TRAFFIC_BATCH) else None,
                "traffic_note": "dram read+write bytes of the conv_i8_tc launches of one step, from the ncu capture summarised in "
                                "profiles/conv_i8_tc_dram_traffic_b256.md (ResNet-50 at batch 256 only; not scaled, because the L2 share changes)",
                "launches_per_step": len(tc), "share_of_step": tc_us / all_us if all_us else None,
                "per_kernel": per_kernel}
        if k3:
            k3_tops = sum(r["gop"] for r in k3) / sum(r["us"] for r in k3) * 1e3
            roof.update({"conv3x3_tops": k3_tops, "conv3x3_frac": k3_tops / peak_assumed, "conv3x3_frac_of_tensor_peak_measured": k3_tops / peak_measured})
        if args.table:
            note = ("%s, batch %d, 1 x B200; CUDA events around every primitive on a profiling engine (launches serialised: shares, not the step time). "
                    "Tensor fractions against the measured tcgen05 peak of this device (%.0f T%s/s); 2 x bf16 sustained of MEASURED_PEAKS would be %.0f. "
                    "HBM fractions against %.0f GB/s (%s).  Command: `python bench.py --config %s --table <file>`."
                    % (config, B, peak_measured, "FLOP" if half else "OP", peak_assumed, peaks["hbm_gbs"], peaks["source"], config))
            with open(args.table, "w") as f:
                f.write(table_markdown("%s per-primitive table (batch %d)" % (config, B), table, note))
        if args.save_cache and os.path.exists(cache):
            import shutil
            shutil.copyfile(cache, args.save_cache)

    per_rank = shard_plan(B * world, world)
    images = sum(per_rank) * args.steps
    value = whole_job_rate(per_rank, args.steps, ms)
    line = {"metric": metric, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": warm,
            "ms_per_step": ms / args.steps, "ms_per_step_min": ms_min / args.steps, "ms_per_step_max": ms_max / args.steps, "timed_regions": reps,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype, "data": "synthetic",
            "config": {"workload": "%s_b%d" % (config, B), "batch_per_gpu": B, "global_batch": B * world, "image": lay.size.x, "parallelism": "dp%d" % world,
                       "l2": "each step reads a different one of %d resident batches (%.0f MB total > 126 MB L2)" % (n_resident, n_resident * in_bytes / 1e6),
                       "ops_per_image": total_ops, "timing": "median of %d regions of %d steps (>= %.1f s of device time in all)" % (reps, args.steps, args.min_seconds)},
            "clocks": clocks,
            "e2e": {"value": images / (ms_e2e / 1e3), "unit": UNIT, "h2d_bytes_per_step": in_bytes * world, "d2h_bytes_per_step": out_bytes * world,
                    "ms_per_step": ms_e2e / args.steps, "ms_per_step_min": e2e_min / args.steps, "ms_per_step_max": e2e_max / args.steps, "timed_regions": e2e_reps},
            "gpu_launches": int(launches_per_step) * args.steps}
    if rank == 0:
        line["roofline"] = roof
        line["parity"] = parity
        if cpu is not None and world == 1:
            line["cpu_baseline"] = cpu
        line["per_primitive"] = table
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()
    if rank == 0 and parity is not None and not parity["ok"]:
        raise SystemExit("bench.py: the timed network differs from the CPU oracle: %s" % json.dumps(parity))


if __name__ == "__main__":
    main()
