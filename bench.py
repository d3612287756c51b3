#!/usr/bin/env python
"""Benchmark of the conv hot path: 3x3 layer sweep, forward + deltaX + deltaW, fp32 NHWC.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--math 3xtf32|tf32]

One step = one pass over the four layers of the sweep (56x56x64, 28x28x128, 14x14x256, 7x7x512;
batch 256 per GPU, stride 1, pad 1): conv3D, dconv3D_deltaX and dconv3D_deltaW of each layer, 12
contractions of 59.19 GFLOP.  With N > 1 (launched by torch.distributed.run, one rank per GPU) every
rank works on its own batch-256 shard (weak scaling) and the deltaW of each layer is summed over the
ranks with an NCCL all-reduce.  Rank 0 prints one JSON line.

`value` is device-timed throughput with inputs resident in HBM; `e2e` runs the same step through the
operator API from pinned HOST buffers, host<->device copies inside the timed region.  Inputs are
seeded synthetic tensors (ReLU(N(0,1)) activations, He-normal weights, N(0,1) output gradients).

--impl reference times the reference's own CPU loops (compiled from the reference checkout into
oracle/_ref when that was possible, else the C restatement in oracle/) on the host cores, on a
bounded sample of the same workload.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised under
# profiles/ (kernel, launch shape, math mode) -> bytes
NCU_TRAFFIC = {
    ("conv_halo_kernel", "fwd_56x56x64", "3xtf32"): 368.6e6,   # profiles/conv_halo_fwd_3xtf32.md
    ("conv_halo_kernel", "dx_56x56x64", "3xtf32"): 368.6e6,    # same kernel and shape as the forward launch
    ("conv_halo_kernel", "fwd_14x14x256", "3xtf32"): 90.3e6,
    ("conv_halo_kernel", "fwd_28x28x128", "tf32"): 158.2e6,
    ("conv_halo_pair_kernel", "fwd_28x28x128", "3xtf32"): 164.2e6,   # profiles/conv_halo_pair_fwd_3xtf32.md
    ("conv_halo_pair_kernel", "dx_28x28x128", "3xtf32"): 164.2e6,    # same kernel and shape as the forward launch
    ("conv_halo_pair_kernel", "fwd_7x7x512", "3xtf32"): 47.1e6,
    ("conv_halo_pair_kernel", "dx_7x7x512", "3xtf32"): 47.1e6,
    ("conv_dw_halo_kernel", "dw_56x56x64", "3xtf32"): 415.5e6,  # profiles/conv_dw_halo_3xtf32.md
    ("conv_dw_halo_kernel", "dw_28x28x128", "3xtf32"): 209.7e6,
}

METRIC = "conv fwd+deltaX+deltaW throughput, 3x3 layer sweep (batch 256 per GPU)"
UNIT = "TFLOP/s"
OPS = ("fwd", "dx", "dw")


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--math", default="3xtf32", choices=["3xtf32", "tf32"])
    ap.add_argument("--batch", type=int, default=None, help="per-GPU batch (default 256)")
    ap.add_argument("--cpu-sample-batch", type=int, default=2)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--streams", type=int, default=3, choices=[1, 3],
                    help="3: forward, deltaX and deltaW of a layer go to three streams (graph branches), so the tail of one kernel overlaps the start of another")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel eagerly instead of replaying a CUDA graph of the step")
    ap.add_argument("--only-layer", type=int, default=None, help="profiling aid: run one sweep layer")
    ap.add_argument("--only-op", default=None, choices=list(OPS), help="profiling aid: run one contraction")
    return ap.parse_args()


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], bf16=p["bf16_tflops"], bf16_sustained=p["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, bf16=1590.0, bf16_sustained=1400.0, source="fallback")


# ---------------------------------------------------------------------------------------------------
# CPU arm: the reference's own loops on the host cores
# ---------------------------------------------------------------------------------------------------

def cpu_threads():
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


class CpuArm:
    """Runs fwd + deltaX + deltaW of every sweep layer at a small batch on the host.

    kind "reference": the reference's C++ loops (CONV_3D_NAIVE, deconv3D_deltaX_img2col,
    deconv3D_deltaW_img2col2 of its test.cuh files) from oracle/_ref, one call per channel slice,
    the slices spread over all host threads.  kind "port": the OpenMP C restatement in oracle/.
    """

    def __init__(self, batch):
        import numpy as np
        import oracle as O
        from __graft_entry__ import submodule
        self.np, self.O = np, O
        synth = submodule("synth")
        self.synth = synth
        self.batch = batch
        self.threads = cpu_threads()
        self.kind = "reference" if O.ref_lib() is not None else "port"
        self.layers = []
        for hw, c in synth.SWEEP_LAYERS:
            X, W, dY = synth.sweep_layer(hw, c, batch=batch, seed=1)
            entry = dict(hw=hw, c=c, X=X, W=W, dY=dY)
            if self.kind == "reference":
                n_sl = min(self.threads, c // 4)
                bounds = [(i * c // n_sl, (i + 1) * c // n_sl) for i in range(n_sl)]
                entry["slices"] = bounds
                entry["W_oc"] = [np.ascontiguousarray(W[a:b]) for a, b in bounds]
                entry["W_ic"] = [np.ascontiguousarray(W[..., a:b]) for a, b in bounds]
                entry["dY_oc"] = [np.ascontiguousarray(dY[..., a:b]) for a, b in bounds]
            self.layers.append(entry)
        self.flops = sum(3 * synth.conv_flops(batch, hw, hw, c, 3, 3, c) for hw, c in synth.SWEEP_LAYERS)

    def _pool_map(self, fn, items):
        from concurrent.futures import ThreadPoolExecutor
        with ThreadPoolExecutor(max_workers=self.threads) as ex:
            return list(ex.map(fn, items))

    def step(self):
        O = self.O
        for L in self.layers:
            hw, X, W, dY = L["hw"], L["X"], L["W"], L["dY"]
            if self.kind == "reference":
                self._pool_map(lambda w: O.ref_CONV_3D_NAIVE(X, w, 1, 1, 1, 1), L["W_oc"])
                self._pool_map(lambda w: O.ref_deconv3D_deltaX_img2col(dY, w, hw, hw, 1, 1, 1, 1), L["W_ic"])
                self._pool_map(lambda d: O.ref_deconv3D_deltaW_img2col2(X, d, 3, 3, 1, 1, 1, 1), L["dY_oc"])
            else:
                O.conv3D_naive(X, W, 1, 1, 1, 1, threads=self.threads)
                O.deconv3D_deltaX_img2col(dY, W, hw, hw, 1, 1, 1, 1, threads=self.threads)
                O.deconv3D_deltaW_img2col2(X, dY, 3, 3, 1, 1, 1, 1, threads=self.threads)

    def describe(self):
        return "all 4 sweep layers x (fwd, deltaX, deltaW) at batch %d instead of 256 (the loops are linear in the batch)" % self.batch


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    arm = CpuArm(args.cpu_sample_batch)
    for _ in range(max(args.warmup, 0)):
        arm.step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        arm.step()
    dt = time.perf_counter() - t0
    val = arm.flops * args.steps / dt / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "3x3 s1 p1 layer sweep (56x56x64, 28x28x128, 14x14x256, 7x7x512), fwd+deltaX+deltaW",
                   "batch_per_gpu": 256, "sample": arm.describe()},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": arm.threads, "kind": arm.kind, "sample": arm.describe()},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# ---------------------------------------------------------------------------------------------------
# GPU arm
# ---------------------------------------------------------------------------------------------------

class ClockSampler:
    """SM clock, power and clock-event reasons of one GPU, sampled while the timed region runs.

    Reads NVML every 10 ms from a thread (queries only; nothing is set); falls back to an
    `nvidia-smi -lms 200` child process when the NVML binding is missing.
    """

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, uuid):
        self.uuid = uuid
        self.proc = None
        self.lines = []
        self.samples = []      # (sm_mhz, power_w, reasons bitmask)
        self.nvml = None
        self.stop_flag = threading.Event()

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.handle = pynvml.nvmlDeviceGetHandleByUUID(self.uuid) if self.uuid else pynvml.nvmlDeviceGetHandleByIndex(0)
            self.sm_max = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
            self.nvml = pynvml
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        cmd = ["nvidia-smi", "--query-gpu=" + self.FIELDS, "--format=csv,noheader,nounits", "-lms", "200"]
        if self.uuid:
            cmd += ["-i", self.uuid]
        try:
            self.proc = subprocess.Popen(cmd, stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _poll(self):
        n = self.nvml
        while not self.stop_flag.is_set():
            try:
                sm = n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)
                pw = n.nvmlDeviceGetPowerUsage(self.handle) / 1000.0
                rs = n.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                self.samples.append((float(sm), pw, int(rs)))
            except Exception:
                pass
            time.sleep(0.01)

    def _pump(self):
        for ln in self.proc.stdout:
            self.lines.append(ln.strip())

    def stop(self):
        if self.nvml is not None:
            self.stop_flag.set()
            self.thread.join(timeout=2)
            n = self.nvml
            names = (("hw_slowdown", n.nvmlClocksEventReasonHwSlowdown),
                     ("hw_thermal_slowdown", n.nvmlClocksEventReasonHwThermalSlowdown),
                     ("sw_thermal_slowdown", n.nvmlClocksEventReasonSwThermalSlowdown),
                     ("sw_power_cap", n.nvmlClocksEventReasonSwPowerCap),
                     ("hw_power_brake", n.nvmlClocksEventReasonHwPowerBrakeSlowdown))
            reasons = sorted({nm for (_, _, r) in self.samples for nm, bit in names if r & bit})
            sm = [x[0] for x in self.samples]
            return {"sm_mhz": statistics.median(sm) if sm else None, "sm_min_mhz": min(sm) if sm else None,
                    "sm_max_mhz": float(self.sm_max),
                    "power_w_max": max((x[1] for x in self.samples), default=None), "samples": len(sm),
                    "source": "nvml, 10 ms", "reasons": reasons}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, smax, reasons, power = [], [], set(), []
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for ln in self.lines:
            parts = [p.strip() for p in ln.split(",")]
            if len(parts) < 7:
                continue
            try:
                sm.append(float(parts[0])); smax.append(float(parts[1])); power.append(float(parts[2]))
            except ValueError:
                continue
            for nm, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "power_w_max": max(power) if power else None, "samples": len(sm), "source": "nvidia-smi, 200 ms",
                "reasons": sorted(reasons)}


def run_ours(args):
    import numpy as np
    import torch
    import torch.distributed as dist
    from __graft_entry__ import submodule

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    lib = submodule("lib")
    synth = submodule("synth")
    base = submodule("engine").CudaFloat32EngineBase()
    lib.set_math_mode(args.math)
    B = args.batch or synth.SWEEP_BATCH
    peaks = measured_peaks()

    # ---- resident tensors ----
    layers = []
    sweep = synth.SWEEP_LAYERS if args.only_layer is None else [synth.SWEEP_LAYERS[args.only_layer]]
    ops = OPS if args.only_op is None else (args.only_op,)
    for hw, c in sweep:
        Xh, Wh, dYh = synth.sweep_layer(hw, c, batch=B, seed=rank)
        Wh = synth.sweep_layer(hw, c, batch=1, seed=0)[1]  # weights are replicated: same seed on every rank
        L = dict(hw=hw, c=c,
                 X=torch.from_numpy(Xh).to(dev), W=torch.from_numpy(Wh).to(dev), dY=torch.from_numpy(dYh).to(dev),
                 Y=torch.empty((B, hw, hw, c), device=dev), dX=torch.empty((B, hw, hw, c), device=dev),
                 dW=torch.empty((c, 3, 3, c), device=dev), Xh=Xh, Wh=Wh, dYh=dYh,
                 flops=synth.conv_flops(B, hw, hw, c, 3, 3, c))
        layers.append(L)
    step_flops = sum(len(ops) * L["flops"] for L in layers)
    comm_stream = torch.cuda.Stream() if world > 1 else None
    # the deltaW tensors of all layers are views of one flat buffer: one collective per step.  It runs
    # after the last kernel: an all-reduce that overlaps the persistent conv kernels takes SMs from
    # them, and a one-CTA-per-SM kernel that finds SMs busy runs those CTAs as a second wave.
    bucket = submodule("sharding").GradientBucket([L["dW"].numel() for L in layers], dev)
    for i, L in enumerate(layers):
        L["dW"] = bucket.view(i, L["dW"].shape)

    def run_op(L, op):
        hw, c = L["hw"], L["c"]
        if op == "fwd":
            base.conv3D(L["Y"], hw, hw, L["X"], hw, hw, L["W"], 3, 3, B, c, c, 1, 1, 1, 1)
        elif op == "dx":
            base.dconv3D_deltaX(L["dX"], hw, hw, L["dY"], hw, hw, L["W"], 3, 3, B, c, c, 1, 1, 1, 1)
        else:
            base.dconv3D_deltaW(L["dW"], 3, 3, L["X"], hw, hw, L["dY"], hw, hw, B, c, c, 1, 1, 1, 1)

    op_streams = [torch.cuda.Stream() for _ in range(2)] if args.streams == 3 else []

    def compute(events=None):
        if op_streams and events is None and len(ops) == 3:
            # the three contractions of a layer are independent: one stream each (the library keeps a
            # workspace per stream).  Every kernel fills the GPU, so only their tails overlap.
            cur = torch.cuda.current_stream()
            fork = torch.cuda.Event(); fork.record(cur)
            for s_ in op_streams:
                s_.wait_event(fork)
            for L in layers:
                run_op(L, "fwd")
                with torch.cuda.stream(op_streams[0]):
                    run_op(L, "dx")
                with torch.cuda.stream(op_streams[1]):
                    run_op(L, "dw")
            for s_ in op_streams:
                cur.wait_stream(s_)
            return
        for li, L in enumerate(layers):
            for op in ops:
                if events is not None:
                    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
                    e0.record()
                run_op(L, op)
                if events is not None:
                    e1.record()
                    events.append((li, op, e0, e1, lib.last_algo()))

    def reduce_gradients():
        if world > 1 and "dw" in ops and os.environ.get("BENCH_AR", "full") != "none":
            dist.all_reduce(bucket.flat, op=dist.ReduceOp.SUM)

    def step(events=None):
        if os.environ.get("BENCH_AR", "full") not in ("layer", "tiny"):
            compute(events)
            reduce_gradients()
            return
        works = []
        for li, L in enumerate(layers):
            for op in ops:
                if events is not None:
                    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
                    e0.record()
                run_op(L, op)
                if events is not None:
                    e1.record()
                    events.append((li, op, e0, e1, lib.last_algo()))
            if world > 1 and "dw" in ops and os.environ.get("BENCH_AR", "full") == "layer":
                ready = torch.cuda.Event(); ready.record()
                with torch.cuda.stream(comm_stream):
                    comm_stream.wait_event(ready)
                    works.append(dist.all_reduce(L["dW"], op=dist.ReduceOp.SUM, async_op=True))
        for w in works:
            w.wait()
        if world > 1 and "dw" in ops:
            mode = os.environ.get("BENCH_AR", "full")
            if mode == "full":
                dist.all_reduce(bucket.flat, op=dist.ReduceOp.SUM)
            elif mode == "tiny":
                dist.all_reduce(bucket.flat[:4], op=dist.ReduceOp.SUM)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing ----
    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    # The 24 kernel launches of a step are captured once into a CUDA graph and replayed: the tensor
    # maps and shapes of a training step do not change, and the replay removes the launch gaps
    # between the 0.1-0.4 ms kernels.  The collective stays outside the graph.
    graph, launches_per_step, graph_error = None, None, None
    if not args.no_graph and os.environ.get("BENCH_AR", "full") in ("full", "none"):
        try:
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                compute()
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize()
            gobj = torch.cuda.CUDAGraph()
            n0 = lib.launch_count()
            with torch.cuda.graph(gobj, stream=side):
                compute()
            launches_per_step = lib.launch_count() - n0
            for _ in range(3):
                gobj.replay(); reduce_gradients()
            torch.cuda.synchronize()
            if lib.device_status() != 0:
                raise RuntimeError("kernel status %d after graph replay" % lib.device_status())
            graph = gobj
        except Exception as e:  # fall back to eager launches, and say so in the JSON line
            graph = None
            graph_error = str(e).splitlines()[0][:200]
            torch.cuda.synchronize()
        barrier()
    uuid = None
    try:
        uuid = "GPU-" + str(torch.cuda.get_device_properties(dev).uuid)
    except Exception:
        pass
    sampler = ClockSampler(uuid) if rank == 0 else None
    if sampler:
        sampler.start()
    launches0 = lib.launch_count()
    events = []
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    if graph is not None:
        for _ in range(args.steps):
            graph.replay()
            reduce_gradients()
    else:
        for _ in range(args.steps):
            step(events)
    t1.record()
    barrier()
    ms_total = t0.elapsed_time(t1)
    launches = launches_per_step * args.steps if graph is not None else lib.launch_count() - launches0
    if graph is not None:
        # per-op times for the roofline come from a few eager steps outside the timed region
        step([])   # single-stream warm-up: the library keeps one workspace per stream
        for _ in range(8):
            step(events)
        torch.cuda.synchronize()
    clocks = sampler.stop() if sampler else None
    status = lib.device_status()
    if status != 0:
        raise SystemExit("bench.py: kernel status word %d: %s" % (status, lib.last_error()))
    if world > 1:
        t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / args.steps
    value = world * step_flops / (ms_step * 1e-3) / 1e12

    # per-kernel time from the CUDA events of the timed region; the roofline is reported for the
    # kernel with the largest share, on its longest-running launch shape
    KERNELS = {"halo": "conv_halo_kernel", "halo_row": "conv_halo_kernel", "halo_tap": "conv_halo_kernel",
               "halo_pair_row": "conv_halo_pair_kernel", "halo_pair_tap": "conv_halo_pair_kernel",
               "igemm": "conv_igemm_kernel", "dw_halo": "conv_dw_halo_kernel", "dw": "conv_dw_kernel",
               "simt": "conv_*_simt"}
    fam, per_op = {}, {}
    for li, op, e0, e1, algo in events:
        ms = e0.elapsed_time(e1)
        kname = KERNELS.get(algo, algo)
        f = fam.setdefault(kname, dict(ms=0.0, flops=0.0, n=0))
        f["ms"] += ms; f["flops"] += layers[li]["flops"]; f["n"] += 1
        k = "%s_%dx%dx%d" % (op, layers[li]["hw"], layers[li]["hw"], layers[li]["c"])
        e = per_op.setdefault(k, dict(ms=[], flops=layers[li]["flops"], kernel=kname, li=li, op=op))
        e["ms"].append(ms)
    dom = max(fam, key=lambda k: fam[k]["ms"])
    heavy = max((k for k in per_op if per_op[k]["kernel"] == dom), key=lambda k: statistics.mean(per_op[k]["ms"]))
    h = per_op[heavy]
    hl = layers[h["li"]]
    tf32_peak = peaks["bf16_sustained"] / 2.0
    achieved = h["flops"] / (statistics.mean(h["ms"]) * 1e-3) / 1e12
    alg_bytes = synth.conv_bytes(B, hl["hw"], hl["hw"], hl["c"], hl["hw"], hl["hw"], hl["c"], 3, 3)
    roofline = {
        "bound": "tensor", "kernel": dom, "launch": heavy, "achieved": achieved, "peak": tf32_peak, "unit": "TFLOP/s",
        "frac": achieved / tf32_peak,
        "traffic": NCU_TRAFFIC.get((dom, heavy, args.math)),
        "algorithmic_bytes": alg_bytes,
        "peak_source": "%s bf16 sustained %.1f TFLOP/s / 2 (dense TF32 rate is half the bf16 rate)" % (
            peaks["source"], peaks["bf16_sustained"]),
        "note": "3xTF32 issues three MMAs per product, so its useful-FLOP ceiling is peak/3" if args.math == "3xtf32" else "plain TF32",
        "time_share": fam[dom]["ms"] / max(sum(f["ms"] for f in fam.values()), 1e-9),
        "kernel_time_shares": {k: round(v["ms"] / max(sum(f["ms"] for f in fam.values()), 1e-9), 3) for k, v in fam.items()},
    }
    per_op_tflops = {k: v["flops"] / (statistics.mean(v["ms"]) * 1e-3) / 1e12 for k, v in per_op.items()}

    # ---- end to end from pinned host buffers ----
    e2e = None
    if not args.no_e2e and args.only_layer is None and args.only_op is None:
        e2e = run_e2e(args, torch, dist, dev, world, layers, run_op, step_flops, B, comm_stream)

    # ---- CPU baseline (rank 0, single GPU runs only) ----
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        arm = CpuArm(args.cpu_sample_batch)
        arm.step()  # warm the caches and the thread pool
        reps, t_cpu = 0, 0.0
        c0 = time.perf_counter()
        while True:
            arm.step(); reps += 1
            t_cpu = time.perf_counter() - c0
            if t_cpu > 10.0 or reps >= 20:
                break
        cpu = {"value": arm.flops * reps / t_cpu / 1e12, "unit": UNIT, "cores": arm.threads, "kind": arm.kind,
               "sample": arm.describe() + ", %d passes in %.1f s" % (reps, t_cpu)}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "tf32x3 (fp32-faithful split)" if args.math == "3xtf32" else "tf32",
            "data": "synthetic",
            "config": {"workload": "3x3 s1 p1 layer sweep (56x56x64, 28x28x128, 14x14x256, 7x7x512), fwd+deltaX+deltaW",
                       "batch_per_gpu": B, "global_batch": B * world, "math": args.math,
                       "parallelism": "batch-sharded x%d, deltaW all-reduce" % world if world > 1 else "single GPU",
                       "l2": "inputs larger than L2 (%.2f GB of tensors per step)" % (
                           sum(4.0 * (2 * L["X"].numel() + 2 * L["Y"].numel() + 2 * L["W"].numel()) for L in layers) / 1e9),
                       "launch": ("CUDA graph of the step's kernels, replayed" if graph is not None else "eager launches") +
                                 (", forward / deltaX / deltaW on three streams" if op_streams else "")},
            "roofline": roofline, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": int(launches), "clocks": clocks,
            "per_op_tflops": {k: round(v, 1) for k, v in per_op_tflops.items()},
        }
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_e2e(args, torch, dist, dev, world, layers, run_op, step_flops, B, comm_stream):
    """Same step through the operator API with HOST buffers: every step copies that step's X,
    deltaY and W from pinned host memory, runs the twelve contractions and copies Y, deltaX and
    deltaW back to pinned host memory.  Copies run on their own streams and the device tensors are
    double-buffered, so that uploads, kernels and downloads of neighbouring layers and steps overlap;
    the clock stops when the last step's results are on the host."""
    pin = lambda a: torch.from_numpy(a).pin_memory()
    for L in layers:
        L["Xp"], L["Wp"], L["dYp"] = pin(L["Xh"]), pin(L["Wh"]), pin(L["dYh"])
        L["Yp"] = torch.empty(L["Y"].shape, dtype=torch.float32).pin_memory()
        L["dXp"] = torch.empty(L["dX"].shape, dtype=torch.float32).pin_memory()
        L["dWp"] = torch.empty(L["dW"].shape, dtype=torch.float32).pin_memory()
    h2d = sum(4 * (L["Xp"].numel() + L["Wp"].numel() + L["dYp"].numel()) for L in layers)
    d2h = sum(4 * (L["Yp"].numel() + L["dXp"].numel() + L["dWp"].numel()) for L in layers)
    s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
    main = torch.cuda.current_stream()
    # two sets of device tensors: the uploads of step i+1 run while step i computes and downloads
    dev_keys = ("X", "W", "dY", "Y", "dX", "dW")
    sets = [layers, [dict(L, **{k: torch.empty_like(L[k]) for k in dev_keys}) for L in layers]]
    consumed = [None, None]    # main-stream event: the kernels that read/wrote this set are done
    downloaded = [None, None]  # s_out event: this set's results have reached the host
    counter = [0]

    def step():
        s = counter[0] & 1
        counter[0] += 1
        cur = sets[s]
        ins = []
        with torch.cuda.stream(s_in):
            if consumed[s] is not None:
                s_in.wait_event(consumed[s])
            for L in cur:
                L["X"].copy_(L["Xp"], non_blocking=True)
                L["W"].copy_(L["Wp"], non_blocking=True)
                L["dY"].copy_(L["dYp"], non_blocking=True)
                ev = torch.cuda.Event(); ev.record(s_in); ins.append(ev)
        if downloaded[s] is not None:
            main.wait_event(downloaded[s])
        for L, ev in zip(cur, ins):
            main.wait_event(ev)
            for op in OPS:
                run_op(L, op)
            if world > 1:
                w = dist.all_reduce(L["dW"], op=dist.ReduceOp.SUM, async_op=True)
                w.wait()
            done = torch.cuda.Event(); done.record(main)
            with torch.cuda.stream(s_out):
                s_out.wait_event(done)
                L["Yp"].copy_(L["Y"], non_blocking=True)
                L["dXp"].copy_(L["dX"], non_blocking=True)
                L["dWp"].copy_(L["dW"], non_blocking=True)
        consumed[s] = torch.cuda.Event(); consumed[s].record(main)
        downloaded[s] = torch.cuda.Event(); downloaded[s].record(s_out)

    steps = max(3, min(args.steps, 10))
    for _ in range(2):
        step()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
    t0.record()
    for _ in range(steps):
        step()
    main.wait_stream(s_out)   # the last step's results are on the host when the clock stops
    t1.record()
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    ms = t0.elapsed_time(t1)
    if world > 1:
        t = torch.tensor([ms], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    ms_step = ms / steps
    return {"value": world * step_flops / (ms_step * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": int(h2d),
            "d2h_bytes_per_step": int(d2h), "ms_per_step": ms_step, "steps": steps}


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
