"""Benchmark of the BatchNorm / Adam / BiasAdd+activation path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the workload over one batch of synthetic input:

  workload resnet50_bn_train_bf16_b256 (N >= 1)
      FusedBatchNormV3 (training) over ResNet-50's 53 BatchNorm layers, then
      FusedBatchNormGradV3 over the same layers in reverse order; bf16 NHWC
      activations at batch 256 per GPU, fp32 statistics.  With N > 1 every
      layer is a cross-replica BatchNorm: the per-channel sums are all-reduced
      with NCCL between the statistics pass and the element-wise pass (weak
      scaling: the per-GPU batch is fixed).

Rank 0 prints ONE JSON line.  `value` is Gelem/s over all GPUs with inputs
resident in HBM (every layer has its own x and dy, 10.8 GB per GPU, so no input
is re-read from L2 between launches); `e2e` is the same metric through the
public op API with pinned host buffers, copies inside the timed region;
`roofline` describes the dominant kernel, `ops` every op of the path
(Adam, BiasAdd chains and the single-layer BatchNorm configurations) at N = 1;
`cpu_baseline` is the CPU oracle timed on this machine's host cores.

`--impl reference` times the CPU restatement of the reference path (the
reference's own kernels need its vendor toolchain and TensorFlow, neither of
which can be installed here) on a bounded sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import tempfile
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

# (count, H, W, C) of ResNet-50's 53 BatchNorm layers at 224x224 input.
RESNET50_BN = [(1, 112, 112, 64), (6, 56, 56, 64), (4, 56, 56, 256), (8, 28, 28, 128),
               (5, 28, 28, 512), (12, 14, 14, 256), (7, 14, 14, 1024), (6, 7, 7, 512),
               (4, 7, 7, 2048)]
BATCH = 256
EPS = 1e-3
# DRAM bytes per launch from an ncu capture (the summary under profiles/ names
# the command): 822.2 MB read + 376.4 MB written for 1233.1 MB algorithmic.
# The whole step: sum over its 318 launches, one single-pass capture per metric with
# L2 left as the previous kernel left it (profiles/resnet50_bn_step_launch_list.md).
NCU_TRAFFIC_BYTES = {"bn_grad_apply_bf16_256x56x56x256": 1198591488,
                     "resnet50_bn_step": 37391728896}
# One-directional rate of a cudaMemcpyAsync between two B200 of one NVSwitch
# node, as measured by `bench.py --probe peer_copy` (nominal 900 GB/s).
PEER_COPY_GBS = 770.0
# HBM3e bandwidth NVIDIA quotes for the part (8 TB/s); fractions against it ride
# along with the fractions against the measured copy bandwidth.
NOMINAL_HBM_GBS = 8000.0
WORKLOAD = "resnet50_bn_train_bf16_b256"
METRIC = "bn_fwd_grad_throughput"
UNIT = "Gelem/s"


def layer_list():
    out = []
    for count, h, w, c in RESNET50_BN:
        out += [(h, w, c)] * count
    return out


def workload_config():
    """The description of the workload that both arms print, key for key."""
    layers = layer_list()
    elems = 2 * sum(BATCH * h * w * c for (h, w, c) in layers)       # forward + gradient
    sum_s = sum(BATCH * h * w * c * 2 for (h, w, c) in layers)      # bytes of all x
    return {"workload": WORKLOAD, "layers": len(layers), "batch_per_gpu": BATCH,
            "layout": "NHWC", "stats_dtype": "f32",
            "elements_per_step_per_gpu": elems,
            "algorithmic_bytes_per_step_per_gpu": 5 * sum_s,   # 2*S forward + 3*S gradient
            "l2": "inputs exceed the last-level cache between reuses (GPU arm: one x and "
                  "dy per layer, 10.8 GB per GPU; CPU arm: one x and dy per distinct "
                  "shape, 2.7 GB)"}


def measured_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        try:
            return float(json.load(open(p))["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


# ------------------------------------------------------------ clock sampler --

class ClockSampler:
    """SM clock and throttle reasons while the timed region runs: a thread that
    reads NVML every few milliseconds (read-only queries), so that even a timed
    region of a fraction of a second is covered; `nvidia-smi -lms` is the
    fall-back when the NVML binding is missing."""
    FIELDS = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    # NVML clocks-event-reason bits (nvml.h).
    REASONS = ((0x8, "hw_slowdown"), (0x40, "hw_thermal_slowdown"),
               (0x20, "sw_thermal_slowdown"), (0x4, "sw_power_cap"))

    def __init__(self, gpu_index):
        self.gpu = gpu_index
        self.proc = None
        self.path = None
        self.thread = None
        self.samples = []      # (time, sm_mhz, reason_bits)
        self.max_mhz = None
        self._stop = False

    def _nvml_loop(self, nv, handle):
        while not self._stop:
            try:
                mhz = nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)
                try:
                    bits = nv.nvmlDeviceGetCurrentClocksEventReasons(handle)
                except Exception:
                    bits = nv.nvmlDeviceGetCurrentClocksThrottleReasons(handle)
                self.samples.append((time.time(), float(mhz), int(bits)))
            except Exception:
                pass
            time.sleep(0.004)

    def start(self):
        try:
            import threading
            import pynvml as nv
            nv.nvmlInit()
            handle = nv.nvmlDeviceGetHandleByIndex(self.gpu)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._nvml_loop, args=(nv, handle),
                                           daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", "50"],
                stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self, t_begin=None, t_end=None):
        """Summary of the samples whose timestamp lies in [t_begin, t_end]
        (epoch seconds; all samples when not given)."""
        import datetime
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        if self.thread is not None:
            self._stop = True
            self.thread.join(timeout=2)
            picked = [x for x in self.samples
                      if t_begin is None or t_begin - 0.005 <= x[0] <= t_end + 0.005]
            if not picked:          # a window shorter than one sampling period
                picked = self.samples[-3:]
            if picked:
                out["sm_mhz"] = float(np.median([x[1] for x in picked]))
                out["sm_max_mhz"] = self.max_mhz
                out["samples"] = len(picked)
                bits = 0
                for x in picked:
                    bits |= x[2]
                out["reasons"] = sorted(name for bit, name in self.REASONS if bits & bit)
            out["source"] = "nvml"
            return out
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [s.strip() for s in line.split(",")]
                if len(f) < 9:
                    continue
                try:
                    if t_begin is not None:
                        ts = datetime.datetime.strptime(
                            f[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                        if ts < t_begin - 0.05 or ts > t_end + 0.05:
                            continue
                    sm.append(float(f[1]))
                    mx.append(float(f[2]))
                except ValueError:
                    continue
                for name, val in zip(names, f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(name)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out["sm_mhz"] = float(np.median(sm))
            out["sm_max_mhz"] = float(max(mx))
            out["samples"] = len(sm)
        out["reasons"] = sorted(reasons)
        out["source"] = "nvidia-smi"
        return out


# ------------------------------------------------------------------ ours ----

def finish(torch, dist, world):
    """Leaves a multi-rank run: every rank drains its GPU, meets the others at
    a barrier and exits at once.  The process group is not torn down
    collectively: tearing down NCCL communicators that captured CUDA graphs
    still reference has hung, and nothing is in flight at this point."""
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(0)


def arm_watchdog(seconds):
    """Ends the process if the run has not finished after `seconds` (a hung
    collective must not hold the GPUs)."""
    import threading

    def bail():
        sys.stderr.write("bench.py: watchdog fired after %d s\n" % seconds)
        sys.stderr.flush()
        os._exit(3)

    t = threading.Timer(seconds, bail)
    t.daemon = True
    t.start()
    return t


def run_ours(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus %d needs torchrun with %d ranks" % (args.gpus, args.gpus))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the kernels have no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    arm_watchdog(args.watchdog)
    if world > 1:
        # Plain peer-to-peer rings: the exchanged messages are a few KiB, and a
        # rank never sits bound to an NVLink multicast object.
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)

    import tensorflow_musa_extension_b200 as pkg
    from tensorflow_musa_extension_b200 import raw_ops
    from tensorflow_musa_extension_b200.cross_replica import SyncBatchNorm

    pkg.load_plugin()
    lib = raw_ops._lib()
    layers = layer_list()
    st = torch.cuda.current_stream()

    # ---- device-resident inputs: one x and one dy per layer, outputs shared
    # per shape.  bf16 values drawn once on the device (x ~ N(0,1),
    # dy ~ N(0, 1e-2)), seed 4 + rank.
    gen = torch.Generator(device=dev)
    gen.manual_seed(4 + rank)
    xs, dys, scales, offsets = [], [], [], []
    out_y, out_dx = {}, {}
    for (h, w, c) in layers:
        rows = BATCH * h * w
        x = torch.empty(rows, c, device=dev, dtype=torch.bfloat16)
        x.normal_(0, 1, generator=gen)
        dy = torch.empty(rows, c, device=dev, dtype=torch.bfloat16)
        dy.normal_(0, 1e-2, generator=gen)
        xs.append(x)
        dys.append(dy)
        scales.append(torch.empty(c, device=dev).uniform_(0.5, 1.5, generator=gen))
        offsets.append(torch.empty(c, device=dev).normal_(0, 0.1, generator=gen))
        if (rows, c) not in out_y:
            out_y[(rows, c)] = torch.empty_like(x)
            out_dx[(rows, c)] = torch.empty_like(x)
    n_layers = len(layers)
    elems_per_pass = sum(x.numel() for x in xs)
    elems_per_step = 2 * elems_per_pass          # forward + gradient
    sum_s = sum(x.numel() * 2 for x in xs)       # bytes of all x
    algo_bytes_step = 5 * sum_s                  # 2*S forward + 3*S gradient

    # N > 1: the per-channel sums are exchanged by a peer-memory kernel fused
    # into the launch chain; --sync nccl keeps the NCCL all-reduce instead.
    exchange = None
    sync_kind = "none (1 GPU)"
    if world > 1:
        sync_kind = "nccl all-reduce of 2*C(+1) fp32 per layer and pass"
        if args.sync in ("peer", "peer_fused", "peer_kernel"):
            from tensorflow_musa_extension_b200.cross_replica import PeerExchange
            try:
                exchange = PeerExchange(dist.group.WORLD, 2 * max(c for (_, _, c) in layers) + 1,
                                        dev)
                sync_kind = ("peer-memory exchange inside the finalize kernel (NVLink stores "
                             "into every replica, bounded wait, rank-ordered merge) of "
                             "2*C(+1) fp32 per layer and pass")
            except Exception as e:  # not one node / no peer access
                if rank == 0:
                    print("peer exchange unavailable (%r): using NCCL" % (e,), file=sys.stderr)
    bns = [SyncBatchNorm(c, eps=EPS, dtype=torch.bfloat16, device=dev,
                         max_rows=BATCH * h * w, group=(dist.group.WORLD if world > 1 else None),
                         exchange=exchange)
           for (h, w, c) in layers]
    if args.sync == "peer_kernel":
        for b in bns:
            b.fuse_exchange = False
    elif args.sync == "peer_fused":
        for b in bns:
            b.fuse_exchange = True
    if exchange is not None and not bns[0].fuse_exchange:
        sync_kind = ("peer-memory exchange kernel (NVLink stores into every replica, bounded "
                     "wait, rank-ordered merge) of 2*C(+1) fp32 per layer and pass")

    def step():
        for i in range(n_layers):
            bns[i].forward(xs[i], scales[i], offsets[i], out_y[tuple(xs[i].shape)])
        for i in reversed(range(n_layers)):
            bns[i].backward(dys[i], xs[i], scales[i], out_dx[tuple(xs[i].shape)])

    if world == 1 and args.force_split != "off":
        # Diagnostic: the cross-replica launch chain with a single replica, with
        # ("exchange") or without ("bare") the exchange kernel.
        if args.force_split == "exchange":
            from tensorflow_musa_extension_b200.cross_replica import PeerExchange
            exchange = PeerExchange(None, 2 * max(c for (_, _, c) in layers) + 1, dev)
        for b in bns:
            b.force_split = True
            b.exchange = exchange
        sync_kind = "split launch chain on one replica (%s)" % args.force_split
    if args.profile_step:
        # One eager pass and nothing else: the target of an ncu launch list.
        step()
        finish(torch, dist, world)
        return

    # Kernels per step, counted by the library itself over one eager step
    # (three per pass - statistics, finalize, element-wise - or two where the
    # element-wise kernel adds the partial rows itself; a collective-library
    # exchange adds launches that are not this library's and are not counted).
    step()
    torch.cuda.synchronize()
    launched = lib.MusaKernelsLaunchCount()
    step()
    torch.cuda.synchronize()
    launches_per_step = lib.MusaKernelsLaunchCount() - launched

    parity = None
    if world > 1:
        parity = check_multi_gpu_parity(torch, dist, world, rank, dev, exchange,
                                        dist.group.WORLD, args.adam_multicast)
        if rank == 0 and not (parity[0] and parity[1] in (True, None)):
            print(json.dumps({"error": "multi-GPU parity check failed", "sync_parity": parity[0],
                              "adam_shard_parity": parity[1], "detail": parity[2]}), flush=True)
        if not (parity[0] and parity[1] in (True, None)):
            torch.cuda.synchronize()
            dist.barrier()
            sys.stdout.flush()
            os._exit(4)

    # Warm up eagerly, then capture the step in a CUDA graph (the launchers
    # neither allocate nor synchronise, so a step is a pure launch sequence).
    for _ in range(2):
        step()
    torch.cuda.synchronize()
    graph = None
    if not args.no_graph:
        try:
            g = torch.cuda.CUDAGraph()
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                step()
                with torch.cuda.graph(g, stream=side):
                    step()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            graph = g
        except Exception as e:  # capture unsupported: time eager launches
            if rank == 0:
                print("graph capture failed, timing eager launches: %r" % (e,),
                      file=sys.stderr)
            graph = None

    def run_step():
        if graph is not None:
            graph.replay()
        else:
            step()

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    sampler = ClockSampler(local_rank if "CUDA_VISIBLE_DEVICES" not in os.environ else
                           int(os.environ["CUDA_VISIBLE_DEVICES"].split(",")[local_rank]))
    if rank == 0:
        sampler.start()   # nvidia-smi needs a moment to start: begin before the warm-up
    for _ in range(max(args.warmup, 3)):
        run_step()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin = time.time()
    e0.record()
    for _ in range(args.steps):
        run_step()
    e1.record()
    barrier()
    t_end = time.time()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None
    if exchange is not None:
        st = exchange.status()
        if st != 0:
            raise SystemExit("peer exchange: a wait for replica %d ran out" % (st - 1))
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_per_step = ms / args.steps
    value = world * elems_per_step / (ms_per_step * 1e-3) / 1e9

    # ---- end to end: pinned host buffers through the public op API
    e2e = None if args.skip_e2e else \
        measure_e2e(torch, dist, raw_ops, layers, world, rank, dev, args)

    result = None
    if rank == 0:
        peak, peak_kind = measured_peak()
        result = {
            "metric": METRIC, "value": round(value, 3), "unit": UNIT,
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
            "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic",
            "config": workload_config(),
            "run": {"sync": sync_kind,
                    "launch": "cuda graph replay" if graph is not None else "eager"},
            "step_algorithmic_gbs_per_gpu": round(algo_bytes_step / (ms_per_step * 1e-3) / 1e9, 1),
            "step_frac_of_peak": round(algo_bytes_step / (ms_per_step * 1e-3) / 1e9 / peak, 4),
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
            "e2e": e2e,
        }
    if world == 1:
        # Free the workload before the per-op section allocates its own inputs.
        del xs, dys, out_y, out_dx, bns, graph
        torch.cuda.empty_cache()
        ops, roof = (None, None) if args.skip_ops else \
            measure_ops(torch, lib, raw_ops, dev, args)
        if roof is not None:
            # The whole step beside the kernel: fraction of peak by algorithmic
            # bytes, and the DRAM bytes a step really moves (ncu, per step).
            roof["step_frac"] = result["step_frac_of_peak"]
            roof["traffic_step"] = NCU_TRAFFIC_BYTES.get("resnet50_bn_step")
            roof["algorithmic_bytes_step"] = algo_bytes_step
        result["roofline"] = roof
        result["ops"] = ops
        result["cpu_baseline"] = None if args.skip_cpu else \
            cpu_baseline(budget_s=args.cpu_seconds)
    else:
        adam = None if args.skip_ops else \
            measure_adam_sharded(torch, dist, world, rank, dev, exchange, args)
        if rank == 0:
            result["roofline"] = None
            result["cpu_baseline"] = None
            result["adam_sharded"] = adam
            result["sync_parity"] = parity[0]
            result["adam_shard_parity"] = parity[1]
            result["parity_detail"] = parity[2]
    if rank == 0:
        print(json.dumps(result), flush=True)
    finish(torch, dist, world)


def measure_e2e(torch, dist, raw_ops, layers, world, rank, dev, args):
    """The same step through the public ops with HOST buffers: every layer's x
    and dy start in pinned host memory, y / dx and the statistics are read back
    to the host, all inside the timed region.  The ops are driven through the
    package's staging pipeline (upload, compute and download streams), so the
    PCIe transfers of neighbouring layers overlap the kernels and each other;
    x stays on the device between a layer's forward and its gradient.
    `blocking` is the same step with one blocking op call per layer."""
    import collections
    from tensorflow_musa_extension_b200.staging import StagedPipeline
    shapes = sorted({(BATCH * h * w, c) for (h, w, c) in layers})
    gen = torch.Generator()
    gen.manual_seed(40 + rank)
    host = {}
    for rows, c in shapes:
        # One pinned x / dy per shape; values as in the device-resident run.
        x = torch.empty(rows, c, dtype=torch.bfloat16).normal_(0, 1, generator=gen).pin_memory()
        dy = torch.empty(rows, c, dtype=torch.bfloat16).normal_(0, 1e-2, generator=gen).pin_memory()
        host[(rows, c)] = (x, dy)
    par = {c: (torch.empty(c).uniform_(0.5, 1.5, generator=gen).pin_memory(),
               torch.empty(c).normal_(0, 0.1, generator=gen).pin_memory())
           for c in sorted({c for (_, _, c) in layers})}
    empty = torch.empty(0)
    from tensorflow_musa_extension_b200 import cross_replica as cr
    group = dist.group.WORLD if world > 1 else None
    depth = args.e2e_depth
    pipe = StagedPipeline(dev, depth=depth)

    def step():
        pending = collections.deque()

        def collect(limit):
            while len(pending) > limit:
                call = pending.popleft()
                call.result()          # host tensors: y / dx and the statistics
                call.release()

        fwd = []
        for (h, w, c) in layers:
            x, _ = host[(BATCH * h * w, c)]
            s, o = par[c]
            if world > 1:
                call = pipe.submit(cr.sync_batch_norm_forward, x, s, o, EPS, group)
            else:
                call = pipe.submit(raw_ops.FusedBatchNormV3, x, s, o, empty, empty, epsilon=EPS)
            fwd.append(call)
            pending.append(call)
            collect(depth)
        for (h, w, c), f in zip(reversed(layers), reversed(fwd)):
            _, dy = host[(BATCH * h * w, c)]
            s, _ = par[c]
            if world > 1:
                call = pipe.submit(cr.sync_batch_norm_backward, dy, f.input(0), s, f.output(3),
                                   f.output(4), EPS, group)
            else:
                call = pipe.submit(raw_ops.FusedBatchNormGradV3, dy, f.input(0), s, f.output(3),
                                   f.output(4), None, epsilon=EPS)
            pending.append(call)
            collect(depth)
        collect(0)

    def step_blocking():
        saved = []
        for (h, w, c) in layers:
            x, _ = host[(BATCH * h * w, c)]
            s, o = par[c]
            out = raw_ops.FusedBatchNormV3(x, s, o, empty, empty, epsilon=EPS)
            saved.append((out[3], out[4]))
        for (h, w, c), (mean, var) in zip(reversed(layers), reversed(saved)):
            x, dy = host[(BATCH * h * w, c)]
            s, _ = par[c]
            raw_ops.FusedBatchNormGradV3(dy, x, s, mean, var, None, epsilon=EPS)

    def timed(fn, steps):
        fn()  # warm up: staging pools and allocator growth
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            fn()
        torch.cuda.synchronize()
        dt = time.perf_counter() - t0
        if world > 1:
            t = torch.tensor([dt], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dt = float(t.item())
        return dt / steps

    elems = 2 * sum(BATCH * h * w * c for (h, w, c) in layers)
    tensor_bytes = sum(BATCH * h * w * c * 2 for (h, w, c) in layers)
    steps = max(1, min(args.steps, args.e2e_steps))
    sec = timed(step, steps)
    pipe.close()
    out = {"value": round(world * elems / sec / 1e9, 3), "unit": UNIT,
           "h2d_bytes_per_step": 2 * tensor_bytes,   # x (forward), dy (gradient)
           "d2h_bytes_per_step": 2 * tensor_bytes,   # y, dx
           "steps": steps, "ms_per_step": round(sec * 1e3, 2), "pipeline_depth": depth,
           "api": ("staging.StagedPipeline.submit(" +
                   ("raw_ops.FusedBatchNormV3 / FusedBatchNormGradV3" if world == 1 else
                    "cross_replica.sync_batch_norm_forward / _backward") +
                   ") on pinned host tensors")}
    if world == 1:
        sec_b = timed(step_blocking, 1)
        out["blocking"] = {"value": round(elems / sec_b / 1e9, 3), "ms_per_step": round(sec_b * 1e3, 2),
                           "h2d_bytes_per_step": 3 * tensor_bytes, "d2h_bytes_per_step": 2 * tensor_bytes,
                           "api": "one blocking raw_ops call per layer (x uploaded again for the gradient)"}
    return out


def _gather_rows(torch, dist, t, world):
    parts = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(parts, t.contiguous())
    return torch.cat(parts, 0)


def check_multi_gpu_parity(torch, dist, world, rank, dev, exchange, group,
                           with_multicast=False):
    """Before anything is timed at N > 1: one small cross-replica BatchNorm
    layer (forward + gradient, bf16 and fp32) and three steps of the
    range-sharded Adam, each compared with the CPU oracle on the WHOLE problem
    (the concatenated batch; the unsharded vector) at the tolerances of the
    single-GPU parity tests.  The oracle is the checker here, never the thing
    measured.  Returns (sync_ok, adam_ok, details); every rank gets the same
    verdict."""
    from oracle import np_ref
    from tensorflow_musa_extension_b200 import cross_replica as cr
    import ml_dtypes
    details = {}
    rows, c = 4096, 256

    def host_block(r, np_dt):
        rng = np.random.default_rng(9000 + r)
        x = (rng.standard_normal((rows, c), dtype=np.float32) * 2.0 + 0.5).astype(np_dt)
        dy = (rng.standard_normal((rows, c), dtype=np.float32) * 1e-2).astype(np_dt)
        return x, dy

    def to_dev(a):
        if a.dtype == ml_dtypes.bfloat16:
            return torch.from_numpy(a.view(np.int16)).view(torch.bfloat16).to(dev)
        return torch.from_numpy(a).to(dev)

    def rms(a):
        a = np.asarray(a, np.float64)
        return float(np.sqrt(np.mean(a * a))) or 1.0

    def worst(got, want, rtol):
        """Largest |got - want| / (rtol * (|want| + rms(want))): <= 1 passes."""
        g = got.detach().float().cpu().numpy().astype(np.float64)
        w = np.asarray(want).astype(np.float64)
        return float(np.max(np.abs(g - w) / (rtol * (np.abs(w) + rms(w)))))

    sync_ok = True
    prng = np.random.default_rng(77)
    scale = prng.uniform(0.5, 1.5, c).astype(np.float32)
    offset = prng.normal(0, 0.1, c).astype(np.float32)
    for name, t_dt, np_dt, rtol in (("bf16", torch.bfloat16, ml_dtypes.bfloat16, 2e-2),
                                    ("f32", torch.float32, np.float32, 1e-4)):
        x, dy = host_block(rank, np_dt)
        bn = cr.SyncBatchNorm(c, eps=EPS, dtype=t_dt, device=dev, max_rows=rows, group=group,
                              exchange=exchange)
        tx, tdy = to_dev(x), to_dev(dy)
        y, dx = torch.empty_like(tx), torch.empty_like(tx)
        ts, to = torch.from_numpy(scale).to(dev), torch.from_numpy(offset).to(dev)
        bn.forward(tx, ts, to, y)
        bn.backward(tdy, tx, ts, dx)
        torch.cuda.synchronize()
        all_y = _gather_rows(torch, dist, y, world)
        all_dx = _gather_rows(torch, dist, dx, world)
        blocks = [host_block(r, np_dt) for r in range(world)]
        gx = np.concatenate([b[0] for b in blocks], 0)
        gdy = np.concatenate([b[1] for b in blocks], 0)
        want = np_ref.fused_batch_norm(gx, scale, offset, epsilon=EPS)
        wg = np_ref.fused_batch_norm_grad(gdy, gx, scale, want[3], want[4], EPS)
        errs = {"y": worst(all_y, want[0], rtol),
                "batch_mean": worst(bn.batch_mean, want[1], 1e-4),
                "batch_var": worst(bn.batch_var, want[2], 1e-4),
                "saved_mean": worst(bn.saved_mean, want[3], 1e-4),
                "saved_var": worst(bn.saved_var, want[4], 1e-4),
                "dx": worst(all_dx, wg[0], rtol),
                "dscale": worst(bn.dscale, wg[1], 1e-4),
                "doffset": worst(bn.doffset, wg[2], 1e-4)}
        details["syncbn_" + name] = {k: round(v, 4) for k, v in errs.items()}
        sync_ok = sync_ok and all(v <= 1.0 for v in errs.values())
        del bn

    adam_ok = None
    if exchange is not None:
        adam_ok = True
        n = 1_000_003
        # (multicast transport?, gradient dtype): the fp32 op, and the mixed
        # op (fp32 state, bf16 gradient) through the same fused kernel.
        variants = [(False, torch.float32), (False, torch.bfloat16)]
        if with_multicast:
            variants.insert(0, (True, torch.float32))
        for want_multicast, gdt in variants:
            arng = np.random.default_rng(31)
            var0 = arng.normal(0, 0.05, n).astype(np.float32)
            pv = cr.PeerVector(group, n, dev, multicast=want_multicast)
            if want_multicast and not pv.multicast_ptr:
                details["adam_shard_multicast"] = "no multicast mapping on this node"
                pv.close()
                continue
            pv.tensor.copy_(torch.from_numpy(var0).to(dev))
            torch.cuda.synchronize()
            dist.barrier()
            opt = cr.FusedShardedAdam(pv, exchange,
                                      transport="multicast" if want_multicast else "stores")
            ev, em, evv = var0.copy(), np.zeros(n, np.float32), np.zeros(n, np.float32)
            for step in range(1, 4):
                g = arng.normal(0, 1e-3, n).astype(np.float32)
                tg = torch.from_numpy(g).to(gdt)
                g = tg.float().numpy()          # what the kernel sees, widened
                ev, em, evv = np_ref.apply_adam(ev, em, evv, 0.9 ** step, 0.999 ** step, 1e-3,
                                                0.9, 0.999, 1e-7, g)
                opt.step(tg.to(dev), 1e-3, 0.9 ** step, 0.999 ** step)
            torch.cuda.synchronize()
            dist.barrier()
            got = pv.tensor.cpu().numpy().astype(np.float64)
            err = float(np.max(np.abs(got - ev) / (1e-8 + 1e-5 * np.abs(ev))))
            label = opt.transport + ("" if gdt == torch.float32 else "_bf16_grad")
            details["adam_shard_%s_worst_over_tolerance" % label] = round(err, 4)
            adam_ok = adam_ok and err <= 1.0
            opt.close()
            dist.barrier()
            pv.close()
    flags = torch.tensor([1.0 if sync_ok else 0.0, 1.0 if adam_ok in (True, None) else 0.0],
                         device=dev)
    dist.all_reduce(flags, op=dist.ReduceOp.MIN)
    sync_ok = bool(flags[0].item() > 0.5)
    if adam_ok is not None:
        adam_ok = bool(flags[1].item() > 0.5)
    return sync_ok, adam_ok, details


def measure_adam_sharded(torch, dist, world, rank, dev, exchange, args):
    """ResourceApplyAdam over the 25,557,032-parameter vector, sharded by
    contiguous range over the replicas, two ways: update + NCCL all-gather of
    the updated weights, and the fused update-and-broadcast kernel (peer
    stores) + one-float exchange.  Strong scaling: the vector is fixed."""
    from tensorflow_musa_extension_b200 import cross_replica as cr
    n = 25_557_032
    peak, _ = measured_peak()
    # Peer-copy rate per direction and GPU (profiles/peer_copy_bandwidth.md has the
    # command that measures it: `bench.py --probe peer_copy`).
    nvlink_gbs = PEER_COPY_GBS
    hyper = dict(lr=1e-3, b1p=0.9 ** 10, b2p=0.999 ** 10)
    gen = torch.Generator(device=dev)
    gen.manual_seed(3)
    out = {}

    def timed(step_fn, label):
        for _ in range(5):
            step_fn()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        iters = 50
        a.record()
        for _ in range(iters):
            step_fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        hbm = 28.0 * n / world
        # Bytes every GPU has to RECEIVE over NVLink (the other replicas'
        # ranges) - with unicast stores also what it sends; a multicast store
        # sends less but cannot receive less.
        link = 4.0 * n / world * (world - 1)
        bound_ms = max(hbm / (peak * 1e9), link / (nvlink_gbs * 1e9)) * 1e3
        out[label] = {"ms_per_step": round(ms, 4), "gelem_per_s": round(n / (ms * 1e-3) / 1e9, 2),
                      "hbm_bytes_per_gpu": int(hbm), "nvlink_bytes_in_per_gpu": int(link),
                      "bound_ms": round(bound_ms, 4), "frac_of_bound": round(bound_ms / ms, 3)}

    # (a) update, then NCCL all-gather in place
    var = torch.empty(n, device=dev).normal_(0, 0.05, generator=gen)
    opt = cr.ShardedAdam(var, dist.group.WORLD)
    shard = opt.hi - opt.lo
    grads = [torch.empty(max(shard, 1), device=dev).normal_(0, 1e-3, generator=gen)
             for _ in range(4)]
    k = [0]

    def step_nccl():
        k[0] += 1
        opt.step(grads[k[0] % 4][:shard], hyper["lr"], hyper["b1p"], hyper["b2p"])

    timed(step_nccl, "update_then_nccl_all_gather")
    del opt, var

    # (b) fused forms over peer memory: the update kernel stores into every
    # replica ("stores"), or copy engines carry finished chunks to the peers
    # while the next chunk updates ("copies").  Each is replayed from a CUDA
    # graph (the step is a fixed launch sequence), eager when capture fails.
    if exchange is not None:
        variants = [("fused_update_and_peer_broadcast", "stores", 1),
                    ("update_and_copy_engine_broadcast_2_chunks", "copies", 2)]
        if args.adam_multicast:
            variants.append(("fused_update_and_multicast_store", "multicast", 1))
        for label, transport, chunks in variants:
            pv = fopt = None
            try:
                pv = cr.PeerVector(dist.group.WORLD, n, dev, multicast=(transport == "multicast"))
                if transport == "multicast" and not pv.multicast_ptr:
                    out[label] = {"unavailable": "no multicast mapping on this node"}
                    pv.close()
                    pv = None
                    continue
                pv.tensor.normal_(0, 0.05, generator=gen)
                fopt = cr.FusedShardedAdam(pv, exchange, transport=transport, chunks=chunks)
                fshard = fopt.hi - fopt.lo
                fgrad = torch.empty(max(fshard, 1), device=dev).normal_(0, 1e-3, generator=gen)

                def step_peer():
                    fopt.step(fgrad[:fshard], hyper["lr"], hyper["b1p"], hyper["b2p"])

                runner = step_peer
                launch = "eager"
                try:
                    g = torch.cuda.CUDAGraph()
                    side = torch.cuda.Stream()
                    side.wait_stream(torch.cuda.current_stream())
                    with torch.cuda.stream(side):
                        step_peer()
                        with torch.cuda.graph(g, stream=side):
                            step_peer()
                    torch.cuda.current_stream().wait_stream(side)
                    torch.cuda.synchronize()
                    runner = g.replay
                    launch = "cuda graph replay"
                except Exception as e:  # noqa: BLE001
                    if rank == 0:
                        print("adam graph capture failed (%s): %r" % (label, e), file=sys.stderr)
                timed(runner, label)
                out[label]["launch"] = launch
                out[label]["transport"] = transport
                st = exchange.status()
                if st != 0:
                    out[label]["error"] = "wait for replica %d ran out" % (st - 1)
                # every replica must hold the same vector
                check = pv.tensor[::4099].double().sum().reshape(1)
                lo_hi = check.clone()
                dist.all_reduce(lo_hi, op=dist.ReduceOp.MAX)
                out[label]["replicas_identical"] = bool((lo_hi == check).all().item())
            except Exception as e:  # noqa: BLE001
                out[label] = {"unavailable": repr(e)}
            torch.cuda.synchronize()
            dist.barrier()
            if fopt is not None:
                fopt.close()
            if pv is not None:
                pv.close()
    out["config"] = "ResourceApplyAdam fp32, 25,557,032 parameters, contiguous ranges, strong scaling"
    return out


def time_launch(torch, fn, iters, flush=None):
    """Median device time of fn() in ms (CUDA events on the current stream);
    `flush` runs before every timed launch, outside the events."""
    for _ in range(3):
        if flush is not None:
            flush()
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(iters):
        if flush is not None:
            flush()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        b.synchronize()
        times.append(a.elapsed_time(b))
    return float(np.median(times))


def time_stream(torch, fn, iters):
    """Average device time of fn() in ms over `iters` back-to-back launches
    (one pair of CUDA events around the run)."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    b.synchronize()
    return a.elapsed_time(b) / iters


def measure_ops(torch, lib, raw_ops, dev, args):
    """Per-op device timings at N = 1 for every configuration of the path, each
    with its algorithmic bytes, and the roofline entry of the dominant kernel
    of the headline workload.  L2 is flushed (a 512 MB write) before every
    timed launch of the configurations whose inputs fit in L2."""
    peak, peak_kind = measured_peak()
    st = torch.cuda.current_stream().cuda_stream
    flush_buf = torch.empty(512 << 20, dtype=torch.uint8, device=dev)
    flush_src = torch.ones(64 << 20, dtype=torch.float32, device=dev)
    flush_dst = torch.empty(1, dtype=torch.float32, device=dev)

    def flush():
        # Write 512 MB (evicts everything), then read 256 MB of other data so
        # that the dirty lines of the write are back in HBM before the timed
        # launch starts; otherwise their write-back lands inside it.
        flush_buf.fill_(1)
        torch.sum(flush_src, dim=(0,), out=flush_dst[0])

    iters = 20
    ops = {}

    def both(fn):
        """(median time of a launch timed on its own, average time of a launch
        in a run of back-to-back launches) for inputs larger than L2."""
        return time_launch(torch, fn, iters), time_stream(torch, fn, iters)

    def entry(name, ms, algo_bytes, elems, note):
        ms_stream = None
        if isinstance(ms, tuple):
            ms, ms_stream = ms
        gbs = algo_bytes / (ms * 1e-3) / 1e9
        ops[name] = {"ms": round(ms, 4), "algorithmic_bytes": algo_bytes,
                     "achieved_gbs": round(gbs, 1), "frac_of_peak": round(gbs / peak, 4),
                     "frac_of_nominal": round(gbs / NOMINAL_HBM_GBS, 4),
                     "gelem_per_s": round(elems / (ms * 1e-3) / 1e9, 2), "note": note}
        if ms_stream is not None:
            # The same launch as one of a run of back-to-back launches (how it
            # runs inside a training step): no ramp-up / drain per launch.
            ops[name]["ms_back_to_back"] = round(ms_stream, 4)
            ops[name]["frac_back_to_back"] = round(
                algo_bytes / (ms_stream * 1e-3) / 1e9 / peak, 4)

    # Adam, config 4: fp32 N = 25,557,032 (715.6 MB per step: beyond L2).
    n = 25_557_032
    var = torch.randn(n, device=dev) * 0.05
    m = torch.randn(n, device=dev) * 1e-4
    v = torch.rand(n, device=dev) * 1e-6
    g = torch.randn(n, device=dev) * 1e-3
    alpha = 1e-3 * np.sqrt(1 - 0.999 ** 10) / (1 - 0.9 ** 10)
    ms = both(lambda: lib.LaunchResourceApplyAdamFloat(
        var.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(), 0.9, 0.999, 1e-7,
        alpha, n, st))
    entry("adam_f32_25.6M", ms, 28 * n, n, "inputs exceed L2")
    # The other streaming optimizers at the same size (same kernel template).
    ms = both(lambda: lib.LaunchResourceApplyNadam_Float(
        var.data_ptr(), m.data_ptr(), v.data_ptr(), g.data_ptr(), 0.9 ** 10, 0.999 ** 10,
        1e-3, 0.9, 0.999, 1e-7, n, st))
    entry("nadam_f32_25.6M", ms, 28 * n, n, "inputs exceed L2")
    ms = both(lambda: lib.LaunchFusedResourceApplyRMSProp_Float(
        var.data_ptr(), v.data_ptr(), m.data_ptr(), g.data_ptr(), 1e-3, 0.9, 0.9, 1e-7,
        n, st))
    entry("rmsprop_f32_25.6M", ms, 28 * n, n, "inputs exceed L2")
    ms = both(lambda: lib.LaunchResourceApplyGradientDescentFloat(
        var.data_ptr(), g.data_ptr(), 1e-3, n, st))
    entry("sgd_f32_25.6M", ms, 12 * n, n, "inputs exceed L2")
    gb = g.to(torch.bfloat16)
    ms = both(lambda: lib.LaunchResourceApplyGradientDescentFloatBFloat16(
        var.data_ptr(), gb.data_ptr(), 1e-3, n, st))
    entry("sgd_f32_bf16grad_25.6M", ms, 10 * n, n, "inputs exceed L2")
    del var, m, v, g, gb

    # BiasAdd chains, config 3: fp16 [65536, 1024] (268 MB per launch).
    x = torch.randn(65536, 1024, device=dev, dtype=torch.float16)
    b = (torch.randn(1024, device=dev) * 0.1).half()
    y = torch.empty_like(x)
    for name, act in (("bias_relu_f16", 1), ("bias_swish_f16", 2)):
        ms = both(lambda: lib.LaunchBiasAct_F16(
            x.data_ptr(), b.data_ptr(), y.data_ptr(), 65536, 1024, 1, act, st))
        entry(name, ms, 4 * x.numel(), x.numel(), "inputs exceed L2")
    # Backward of the chain at the same shape: gradients and features in,
    # backprops out (6 B/elem); the un-fused pair reads backprops once more.
    db = torch.empty(1024, device=dev, dtype=torch.float16)
    need = lib.BiasGradWorkspaceBytes(65536, 1024, 1, 2)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
    gr = torch.randn_like(x)
    ms = both(lambda: lib.LaunchBiasAddReluGrad_F16(
        gr.data_ptr(), x.data_ptr(), y.data_ptr(), db.data_ptr(), 65536, 1024, 1,
        ws.data_ptr(), need, st))
    entry("bias_relu_grad_fused_f16", ms, 6 * x.numel(), x.numel(), "inputs exceed L2")
    ms = both(lambda: lib.LaunchReluGrad_F16(
        gr.data_ptr(), x.data_ptr(), y.data_ptr(), x.numel(), st))
    entry("relu_grad_f16", ms, 6 * x.numel(), x.numel(), "inputs exceed L2")
    ms = time_launch(torch, lambda: lib.LaunchBiasAddGrad_F16(
        y.data_ptr(), db.data_ptr(), 65536, 1024, 1, ws.data_ptr(), need, st), iters, flush)
    # One input (134 MB) is about the size of L2: the back-to-back run
    # alternates between two inputs.
    turn = [0]

    def alternate():
        src = (y, gr)[turn[0] & 1]
        turn[0] += 1
        lib.LaunchBiasAddGrad_F16(src.data_ptr(), db.data_ptr(), 65536, 1024, 1,
                                  ws.data_ptr(), need, st)

    entry("bias_add_grad_f16", (ms, time_stream(torch, alternate, iters)), 2 * x.numel(),
          x.numel(), "L2 flushed before each launch; back-to-back over two alternating inputs")
    del x, y, gr

    # Row normalisations at the chain's shape, bf16 [65536, 1024] (S = 134 MB).
    rows, n = 65536, 1024
    x = (torch.randn(rows, n, device=dev) * 3 + 1).to(torch.bfloat16)
    dy = torch.randn(rows, n, device=dev).to(torch.bfloat16)
    y = torch.empty_like(x)
    y2 = torch.empty_like(x)
    gam = torch.ones(n, device=dev, dtype=torch.bfloat16)
    bet = torch.zeros(n, device=dev, dtype=torch.bfloat16)
    dgam, dbet = torch.empty_like(gam), torch.empty_like(bet)
    inv = torch.empty(rows, device=dev, dtype=torch.bfloat16)
    need = lib.LayerNormGradWorkspaceBytes(rows, n)
    ws = torch.empty(max(need, 16), dtype=torch.uint8, device=dev)
    s_bytes = x.numel() * 2
    ms = both(lambda: lib.LaunchLayerNorm_BF16(
        x.data_ptr(), gam.data_ptr(), bet.data_ptr(), y.data_ptr(), None, None, rows, n, 1e-5,
        st))
    entry("layer_norm_bf16", ms, 2 * s_bytes, x.numel(), "inputs exceed L2")
    ms = both(lambda: lib.LaunchLayerNormGrad_BF16(
        dy.data_ptr(), x.data_ptr(), gam.data_ptr(), y.data_ptr(), dgam.data_ptr(),
        dbet.data_ptr(), rows, n, 1e-5, ws.data_ptr(), need, st))
    entry("layer_norm_grad_bf16", ms, 3 * s_bytes, x.numel(), "inputs exceed L2")
    ms = both(lambda: lib.LaunchRmsNormBFloat16(
        x.data_ptr(), gam.data_ptr(), y.data_ptr(), y2.data_ptr(), inv.data_ptr(), rows, n,
        1e-5, st))
    entry("rms_norm_bf16", ms, 3 * s_bytes, x.numel(), "inputs exceed L2")
    ms = both(lambda: lib.LaunchRmsNormGradDxBFloat16(
        x.data_ptr(), inv.data_ptr(), gam.data_ptr(), dy.data_ptr(), y.data_ptr(), rows, n, st))
    entry("rms_norm_grad_dx_bf16", ms, 3 * s_bytes, x.numel(), "inputs exceed L2")
    del x, dy, y, y2

    # BatchNorm single layers: config 1 (fp32) and config 2 (fp16, bf16).
    # The last entry is config 2 in NCHW ([256, 256, 28, 28]: outer 256, inner 784).
    for name, shape, dt, sfx in (("cfg1_f32", (32 * 56 * 56, 64), torch.float32, "F32"),
                                 ("cfg2_f16", (256 * 28 * 28, 256), torch.float16, "F16"),
                                 ("cfg2_bf16", (256 * 28 * 28, 256), torch.bfloat16, "BF16"),
                                 ("cfg2_bf16_nchw", (256, 256, 784), torch.bfloat16, "BF16")):
        inner = shape[2] if len(shape) == 3 else 1
        rows, c = shape[0], shape[1]
        x = (torch.randn(rows, c * inner, device=dev) * 3 + 1).to(dt)
        dy = (torch.randn(rows, c * inner, device=dev) * 1e-2).to(dt)
        y = torch.empty_like(x)
        sc = torch.rand(c, device=dev) + 0.5
        of = torch.randn(c, device=dev) * 0.1
        stats = [torch.empty(c, device=dev) for _ in range(6)]
        need = lib.BnWorkspaceBytes(rows, c, inner)
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        fwd = getattr(lib, "LaunchBnFwdTrain_" + sfx)
        bwd = getattr(lib, "LaunchBnGrad_" + sfx)
        s_bytes = x.numel() * x.element_size()
        ms = time_launch(torch, lambda: fwd(
            x.data_ptr(), sc.data_ptr(), of.data_ptr(), None, None, y.data_ptr(),
            stats[0].data_ptr(), stats[1].data_ptr(), stats[2].data_ptr(),
            stats[3].data_ptr(), rows, c, inner, EPS, 1.0, ws.data_ptr(), need, st),
            iters, flush)
        entry("bn_fwd_" + name, ms, 2 * s_bytes, x.numel(), "L2 flushed before each launch")
        ms = time_launch(torch, lambda: bwd(
            dy.data_ptr(), x.data_ptr(), sc.data_ptr(), stats[2].data_ptr(),
            stats[3].data_ptr(), y.data_ptr(), stats[4].data_ptr(), stats[5].data_ptr(),
            rows, c, inner, EPS, True, ws.data_ptr(), need, st), iters, flush)
        entry("bn_grad_" + name, ms, 3 * s_bytes, x.numel(), "L2 flushed before each launch")
        del x, dy, y

    # The nine layer shapes of the headline workload, one launch each (bf16,
    # batch 256): whole-op time, forward and gradient.
    for (_, h, w, c) in RESNET50_BN:
        rows = BATCH * h * w
        x = torch.randn(rows, c, device=dev).to(torch.bfloat16)
        dy = (torch.randn(rows, c, device=dev) * 1e-2).to(torch.bfloat16)
        y = torch.empty_like(x)
        sc = torch.rand(c, device=dev) + 0.5
        of = torch.randn(c, device=dev) * 0.1
        stats = [torch.empty(c, device=dev) for _ in range(6)]
        need = lib.BnWorkspaceBytes(rows, c, 1)
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        s_bytes = x.numel() * 2
        tag = "r50_%dx%dx%d_bf16" % (h, w, c)
        ms = time_launch(torch, lambda: lib.LaunchBnFwdTrain_BF16(
            x.data_ptr(), sc.data_ptr(), of.data_ptr(), None, None, y.data_ptr(),
            stats[0].data_ptr(), stats[1].data_ptr(), stats[2].data_ptr(),
            stats[3].data_ptr(), rows, c, 1, EPS, 1.0, ws.data_ptr(), need, st), iters, flush)
        entry("bn_fwd_" + tag, ms, 2 * s_bytes, x.numel(), "L2 flushed before each launch")
        ms = time_launch(torch, lambda: lib.LaunchBnGrad_BF16(
            dy.data_ptr(), x.data_ptr(), sc.data_ptr(), stats[2].data_ptr(),
            stats[3].data_ptr(), y.data_ptr(), stats[4].data_ptr(), stats[5].data_ptr(),
            rows, c, 1, EPS, True, ws.data_ptr(), need, st), iters, flush)
        entry("bn_grad_" + tag, ms, 3 * s_bytes, x.numel(), "L2 flushed before each launch")
        del x, dy, y

    # Dominant kernel of the headline workload: the gradient element-wise pass
    # (reads dy and x, writes dx: 3 * S per launch), timed alone on the largest
    # ResNet-50 layer, [256, 56, 56, 256] bf16 (S = 411 MB).
    rows, c = BATCH * 56 * 56, 256
    x = torch.randn(rows, c, device=dev).to(torch.bfloat16)
    dy = (torch.randn(rows, c, device=dev) * 1e-2).to(torch.bfloat16)
    dx = torch.empty_like(x)
    sc = torch.rand(c, device=dev) + 0.5
    mean = torch.zeros(c, device=dev)
    varc = torch.ones(c, device=dev)
    sums = torch.zeros(2 * c, device=dev)
    ds, do = torch.empty(c, device=dev), torch.empty(c, device=dev)
    s_bytes = x.numel() * 2
    ms, ms_stream = both(lambda: lib.LaunchBnGradApplyFromSums(
        2, dy.data_ptr(), x.data_ptr(), sc.data_ptr(), mean.data_ptr(), varc.data_ptr(),
        sums.data_ptr(), float(rows), dx.data_ptr(), None, None, rows, c, 1, EPS, st))
    achieved = 3 * s_bytes / (ms * 1e-3) / 1e9
    roof = {"bound": "hbm", "kernel": "BnApplyLastKernel<bf16, grad>",
            "case": "[256,56,56,256] bf16, 3*S = %d bytes per launch" % (3 * s_bytes),
            "achieved": round(achieved, 1), "peak": peak, "peak_kind": peak_kind,
            "unit": "GB/s", "frac": round(achieved / peak, 4), "ms": round(ms, 4),
            "frac_of_nominal": round(achieved / NOMINAL_HBM_GBS, 4),
            "nominal_gbs": NOMINAL_HBM_GBS, "traffic": None}
    roof["ms_back_to_back"] = round(ms_stream, 4)
    roof["frac_back_to_back"] = round(3 * s_bytes / (ms_stream * 1e-3) / 1e9 / peak, 4)
    # The whole op this kernel belongs to (statistics + element-wise pass).
    roof["op"] = "bn_grad_r50_56x56x256_bf16"
    roof["op_frac"] = ops["bn_grad_r50_56x56x256_bf16"]["frac_of_peak"]
    roof["traffic"] = NCU_TRAFFIC_BYTES["bn_grad_apply_bf16_256x56x56x256"]
    roof["traffic_source"] = ("ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch of this "
                              "kernel and case (profiles/bn_grad_apply_bf16_256x56x56x256_ncu_full.md)")
    return ops, roof


# ------------------------------------------------------------- CPU arms -----

def _bf16_normal(rng, shape, std):
    import ml_dtypes
    return (rng.standard_normal(shape, dtype=np.float32) * std).astype(ml_dtypes.bfloat16)


def cpu_workload(batch, seed=4):
    from oracle import c_ref
    # A multi-rank launcher pins OMP_NUM_THREADS=1 for its workers; the CPU arm
    # is one job on this host and takes every core it is allowed to run on.
    if os.environ.get("OMP_NUM_THREADS") == "1" and "LOCAL_RANK" in os.environ:
        c_ref.set_num_threads(len(os.sched_getaffinity(0)))
    rng = np.random.default_rng(seed)
    data = {}
    for (_, h, w, c) in RESNET50_BN:
        rows = batch * h * w
        data[(h, w, c)] = (_bf16_normal(rng, (rows, c), 1.0), _bf16_normal(rng, (rows, c), 1e-2),
                           rng.uniform(0.5, 1.5, c).astype(np.float32),
                           rng.normal(0, 0.1, c).astype(np.float32))
    layers = layer_list()

    def step():
        saved = []
        for key in layers:
            x, _, s, o = data[key]
            out = c_ref.bn_fwd_train(x, s, o, EPS)
            saved.append((out[3], out[4]))
        for key, (mean, var) in zip(reversed(layers), reversed(saved)):
            x, dy, s, _ = data[key]
            c_ref.bn_grad(dy, x, s, mean, var, EPS)

    elems = 2 * sum(batch * h * w * c for (h, w, c) in layers)
    return step, elems, c_ref.num_threads()


def cpu_baseline(budget_s=15.0):
    """The CPU oracle (C, all host threads) on the stated workload: the same 53
    layers forward + gradient at batch 256, as many whole passes as fit the
    time budget (at least one)."""
    step, elems, cores = cpu_workload(BATCH)
    step()
    t0 = time.perf_counter()
    n = 0
    while True:
        step()
        n += 1
        if time.perf_counter() - t0 > budget_s or n >= 20:
            break
    dt = time.perf_counter() - t0
    return {"value": round(elems * n / dt / 1e9, 4), "unit": UNIT, "cores": cores,
            "kind": "port",
            "sample": "the whole step (53 layers fwd+grad at batch %d), %d passes after one "
                      "warm-up pass" % (BATCH, n)}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    step, elems, cores = cpu_workload(BATCH)
    warm = max(1, min(args.warmup, 3))
    for _ in range(warm):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    ms = dt / args.steps * 1e3
    val = round(elems * args.steps / dt / 1e9, 4)
    sample = "the whole step (53 layers fwd+grad at batch %d), %d timed passes" % (
        BATCH, args.steps)
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT,
        "n_gpus": args.gpus, "steps": args.steps, "warmup": warm,
        "ms_per_step": round(ms, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(),
        "run": {"sync": "none (host cores)", "launch": "one process, %d OpenMP threads" % cores},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port",
                         "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": "CPU restatement of the reference path (oracle/cpu_ref.c): the reference's "
                "own kernels need the MUSA toolchain, muDNN and TensorFlow 2.6.1, none of "
                "which can be installed here",
    }), flush=True)


def run_probe(args):
    """Measurements of the machine that the bounds quoted beside the results
    rest on (not part of the timed benchmark):
      peer_copy  one-directional cudaMemcpyAsync rate between two GPUs, and the
                 rate per GPU when every GPU sends a block to every other GPU at
                 once (the traffic pattern of the range-sharded Adam); N >= 2
      pcie       pinned host <-> device copy rates per GPU, one direction at a
                 time and both at once, with all N ranks copying simultaneously
                 (the bound of the end-to-end leg)"""
    import ctypes
    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    arm_watchdog(args.watchdog)
    if world > 1:
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
    import tensorflow_musa_extension_b200 as pkg
    from tensorflow_musa_extension_b200 import raw_ops
    from tensorflow_musa_extension_b200 import cross_replica as cr
    pkg.load_plugin()
    lib = raw_ops._lib()

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def timed_ms(fn, iters):
        """Max over ranks of the device time of `iters` calls of fn()."""
        for _ in range(2):
            fn()
        sync_all()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(iters):
            fn()
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / iters], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    out = {"probe": args.probe, "n_gpus": world}
    if args.probe == "peer_copy":
        if world < 2:
            raise SystemExit("--probe peer_copy needs at least two ranks")
        n = 64 << 20                               # floats: 256 MB per replica
        pv = cr.PeerVector(dist.group.WORLD, n, dev, multicast=False)
        src = torch.empty(n, device=dev).normal_()
        main = torch.cuda.current_stream()
        # (a) one pair, one direction: rank 0 -> rank 1, everybody else idle.
        nbytes = n * 4

        def one_way():
            if rank == 0:
                raw_ops._check(lib.MusaPeerCopyAsync(pv.replica_ptrs[1], src.data_ptr(), nbytes,
                                                     main.cuda_stream), "MusaPeerCopyAsync")

        ms = timed_ms(one_way, 10)
        out["one_pair_one_direction_gbs"] = round(nbytes / (ms * 1e-3) / 1e9, 1)
        # (b) every GPU sends a block to every other GPU at once, one copy per
        # peer on its own stream (block = 1 / world of the buffer).
        block = n // world
        sides = [torch.cuda.Stream() for _ in range(world - 1)]

        def all_to_all():
            ev = torch.cuda.Event()
            ev.record(main)
            for k in range(1, world):
                q = (rank + k) % world
                st = sides[k - 1]
                st.wait_event(ev)
                dst = pv.replica_ptrs[q] + rank * block * 4
                raw_ops._check(lib.MusaPeerCopyAsync(dst, src.data_ptr() + rank * block * 4,
                                                     block * 4, st.cuda_stream),
                               "MusaPeerCopyAsync")
            for st in sides:
                main.wait_stream(st)

        ms = timed_ms(all_to_all, 10)
        out["all_to_all_block_mb"] = round(block * 4 / 1e6, 1)
        out["all_to_all_egress_gbs_per_gpu"] = round((world - 1) * block * 4 / (ms * 1e-3) / 1e9, 1)
        sync_all()
        pv.close()
    elif args.probe == "pcie":
        nbytes = 1 << 30
        h_up = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
        h_down = torch.empty(nbytes, dtype=torch.uint8).pin_memory()
        d_up = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        d_down = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        s_up, s_down = torch.cuda.Stream(), torch.cuda.Stream()
        main = torch.cuda.current_stream()

        def up():
            d_up.copy_(h_up, non_blocking=True)

        def down():
            h_down.copy_(d_down, non_blocking=True)

        def both():
            s_up.wait_stream(main)
            s_down.wait_stream(main)
            with torch.cuda.stream(s_up):
                d_up.copy_(h_up, non_blocking=True)
            with torch.cuda.stream(s_down):
                h_down.copy_(d_down, non_blocking=True)
            main.wait_stream(s_up)
            main.wait_stream(s_down)

        for name, fn in (("h2d", up), ("d2h", down), ("both_each_way", both)):
            ms = timed_ms(fn, 5)
            out[name + "_gbs_per_gpu"] = round(nbytes / (ms * 1e-3) / 1e9, 1)
        out["note"] = ("all %d ranks copy at the same time; rates are per GPU and direction, "
                       "from the slowest rank" % world)
        out["host_cores"] = len(os.sched_getaffinity(0))
    else:
        raise SystemExit("unknown --probe " + args.probe)
    if rank == 0:
        print(json.dumps(out), flush=True)
    finish(torch, dist, world)


def run_profile_case(args):
    """Small fixed launch sequences for `ncu` captures (one kernel family per
    case, inputs beyond L2, a few hundred MB on the device):
      bn      FusedBatchNorm forward + gradient, bf16 [256,28,28,256], twice
      bnsmall the same on bf16 [256,28,28,128] (S = 51 MB, inside L2)
      bnbig   gradient element-wise pass alone, bf16 [256,56,56,256], twice
      adam    ResourceApplyAdam fp32, 25,557,032 parameters, twice
      bias    Relu(BiasAdd) and x*sigmoid(x+b), fp16 [65536,1024], twice each
      biasgrad  fused ReluGrad+BiasAddGrad, ReluGrad, BiasAddGrad, fp16 [65536,1024]
      optim   Nadam, RMSProp, gradient descent fp32, 25,557,032 parameters
      rownorm LayerNorm fwd/grad and RMSNorm fwd/grad, bf16 [65536,1024]"""
    import torch
    import tensorflow_musa_extension_b200 as pkg
    from tensorflow_musa_extension_b200 import raw_ops
    pkg.load_plugin()
    lib = raw_ops._lib()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(0)
    st = torch.cuda.current_stream().cuda_stream
    case = args.profile_case
    if case in ("bn", "bnbig", "bnsmall"):
        rows, c = {"bn": (256 * 28 * 28, 256), "bnbig": (256 * 56 * 56, 256),
                   "bnsmall": (256 * 28 * 28, 128)}[case]
        x = torch.randn(rows, c, device=dev).to(torch.bfloat16)
        dy = (torch.randn(rows, c, device=dev) * 1e-2).to(torch.bfloat16)
        out = torch.empty_like(x)
        sc = torch.rand(c, device=dev) + 0.5
        of = torch.randn(c, device=dev) * 0.1
        stats = [torch.empty(c, device=dev) for _ in range(6)]
        sums = torch.zeros(2 * c, device=dev)
        need = lib.BnWorkspaceBytes(rows, c, 1)
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        for _ in range(2):
            if case != "bnbig":
                lib.LaunchBnFwdTrain_BF16(
                    x.data_ptr(), sc.data_ptr(), of.data_ptr(), None, None, out.data_ptr(),
                    stats[0].data_ptr(), stats[1].data_ptr(), stats[2].data_ptr(),
                    stats[3].data_ptr(), rows, c, 1, EPS, 1.0, ws.data_ptr(), need, st)
                lib.LaunchBnGrad_BF16(
                    dy.data_ptr(), x.data_ptr(), sc.data_ptr(), stats[2].data_ptr(),
                    stats[3].data_ptr(), out.data_ptr(), stats[4].data_ptr(),
                    stats[5].data_ptr(), rows, c, 1, EPS, True, ws.data_ptr(), need, st)
            else:
                stats[2].zero_()
                stats[3].fill_(1.0)
                lib.LaunchBnGradApplyFromSums(
                    2, dy.data_ptr(), x.data_ptr(), sc.data_ptr(), stats[2].data_ptr(),
                    stats[3].data_ptr(), sums.data_ptr(), float(rows), out.data_ptr(), None,
                    None, rows, c, 1, EPS, st)
    elif case == "adam":
        n = 25_557_032
        var = torch.randn(n, device=dev) * 0.05
        m = torch.randn(n, device=dev) * 1e-4
        v = torch.rand(n, device=dev) * 1e-6
        g = torch.randn(n, device=dev) * 1e-3
        for _ in range(2):
            lib.LaunchResourceApplyAdamFloat(var.data_ptr(), m.data_ptr(), v.data_ptr(),
                                             g.data_ptr(), 0.9, 0.999, 1e-7, 3e-4, n, st)
    elif case == "bias":
        x = torch.randn(65536, 1024, device=dev, dtype=torch.float16)
        b = (torch.randn(1024, device=dev) * 0.1).half()
        y = torch.empty_like(x)
        for _ in range(2):
            for act in (1, 2):
                lib.LaunchBiasAct_F16(x.data_ptr(), b.data_ptr(), y.data_ptr(), 65536, 1024,
                                      1, act, st)
    elif case == "biasgrad":
        x = torch.relu(torch.randn(65536, 1024, device=dev, dtype=torch.float16))
        g = torch.randn_like(x)
        y = torch.empty_like(x)
        db = torch.empty(1024, device=dev, dtype=torch.float16)
        need = lib.BiasGradWorkspaceBytes(65536, 1024, 1, 2)
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        for _ in range(2):
            lib.LaunchBiasAddReluGrad_F16(g.data_ptr(), x.data_ptr(), y.data_ptr(), db.data_ptr(),
                                          65536, 1024, 1, ws.data_ptr(), need, st)
            lib.LaunchReluGrad_F16(g.data_ptr(), x.data_ptr(), y.data_ptr(), x.numel(), st)
            lib.LaunchBiasAddGrad_F16(y.data_ptr(), db.data_ptr(), 65536, 1024, 1, ws.data_ptr(),
                                      need, st)
    elif case == "optim":
        n = 25_557_032
        var = torch.randn(n, device=dev) * 0.05
        m = torch.randn(n, device=dev) * 1e-4
        v = torch.rand(n, device=dev) * 1e-6
        g = torch.randn(n, device=dev) * 1e-3
        for _ in range(2):
            lib.LaunchResourceApplyNadam_Float(var.data_ptr(), m.data_ptr(), v.data_ptr(),
                                               g.data_ptr(), 0.9 ** 10, 0.999 ** 10, 1e-3, 0.9,
                                               0.999, 1e-7, n, st)
            lib.LaunchFusedResourceApplyRMSProp_Float(var.data_ptr(), v.data_ptr(), m.data_ptr(),
                                                      g.data_ptr(), 1e-3, 0.9, 0.9, 1e-7, n, st)
            lib.LaunchResourceApplyGradientDescentFloat(var.data_ptr(), g.data_ptr(), 1e-3, n, st)
    elif case == "rownorm":
        rows, n = 65536, 1024
        x = (torch.randn(rows, n, device=dev) * 3 + 1).to(torch.bfloat16)
        dy = torch.randn(rows, n, device=dev).to(torch.bfloat16)
        y, y2 = torch.empty_like(x), torch.empty_like(x)
        gam = torch.ones(n, device=dev, dtype=torch.bfloat16)
        bet = torch.zeros(n, device=dev, dtype=torch.bfloat16)
        dgam, dbet = torch.empty_like(gam), torch.empty_like(bet)
        inv = torch.empty(rows, device=dev, dtype=torch.bfloat16)
        need = lib.LayerNormGradWorkspaceBytes(rows, n)
        ws = torch.empty(need, dtype=torch.uint8, device=dev)
        for _ in range(2):
            lib.LaunchLayerNorm_BF16(x.data_ptr(), gam.data_ptr(), bet.data_ptr(), y.data_ptr(),
                                     None, None, rows, n, 1e-5, st)
            lib.LaunchLayerNormGrad_BF16(dy.data_ptr(), x.data_ptr(), gam.data_ptr(), y.data_ptr(),
                                         dgam.data_ptr(), dbet.data_ptr(), rows, n, 1e-5,
                                         ws.data_ptr(), need, st)
            lib.LaunchRmsNormBFloat16(x.data_ptr(), gam.data_ptr(), y.data_ptr(), y2.data_ptr(),
                                      inv.data_ptr(), rows, n, 1e-5, st)
            lib.LaunchRmsNormGradDxBFloat16(x.data_ptr(), inv.data_ptr(), gam.data_ptr(),
                                            dy.data_ptr(), y.data_ptr(), rows, n, st)
    else:
        raise SystemExit("unknown --profile-case " + case)
    torch.cuda.synchronize()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-graph", action="store_true", help="time eager launches")
    ap.add_argument("--e2e-depth", type=int, default=6,
                    help="calls in flight in the staging pipeline of the end-to-end leg")
    ap.add_argument("--e2e-steps", type=int, default=2)
    ap.add_argument("--skip-e2e", action="store_true")
    ap.add_argument("--skip-ops", action="store_true")
    ap.add_argument("--skip-cpu", action="store_true")
    ap.add_argument("--profile-step", action="store_true",
                    help="run one eager pass of the workload and exit (ncu target)")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--watchdog", type=int, default=600,
                    help="seconds after which a run that has not finished is ended")
    ap.add_argument("--sync", default="peer", choices=["peer", "peer_fused", "peer_kernel", "nccl"],
                    help="N > 1: how the per-channel values cross the replicas: peer-memory "
                         "exchange (peer: run by the finalize kernel up to 4 replicas, by its "
                         "own kernel beyond; peer_fused / peer_kernel force one), or an NCCL "
                         "collective")
    ap.add_argument("--adam-multicast", action="store_true",
                    help="N > 1: also check and time the NVSwitch-multicast transport of the "
                         "sharded Adam step (torch symmetric memory)")
    ap.add_argument("--force-split", default="off", choices=["off", "bare", "exchange"],
                    help="N = 1 diagnostic: run the cross-replica launch chain anyway")
    ap.add_argument("--profile-case", default=None,
                    help="run a small fixed launch sequence and exit (ncu target): "
                         "bn | bnsmall | bnbig | adam | bias | biasgrad | optim | rownorm")
    ap.add_argument("--probe", default=None, choices=["peer_copy", "pcie"],
                    help="measure a machine rate that a quoted bound rests on, and exit")
    args = ap.parse_args()
    if args.probe:
        run_probe(args)
        return
    if args.profile_case:
        run_profile_case(args)
        return
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
