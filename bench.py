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

# dram__bytes_read.sum + dram__bytes_write.sum per launch, from one ncu capture of each kernel at the
# benchmark's batch: (kernel, launch shape, math mode) -> bytes
NCU_TRAFFIC = {
    ("conv_halo_kernel", "fwd_56x56x64", "3xtf32"): 368.6e6,
    ("conv_halo_kernel", "dx_56x56x64", "3xtf32"): 368.6e6,    # same kernel and shape as the forward launch
    ("conv_halo_kernel", "fwd_14x14x256", "3xtf32"): 90.3e6,
    ("conv_halo_kernel", "fwd_28x28x128", "tf32"): 158.2e6,
    ("conv_halo_pair_kernel", "fwd_28x28x128", "3xtf32"): 164.2e6,
    ("conv_halo_pair_kernel", "dx_28x28x128", "3xtf32"): 164.2e6,    # same kernel and shape as the forward launch
    ("conv_halo_pair_kernel", "fwd_7x7x512", "3xtf32"): 47.1e6,
    ("conv_halo_pair_kernel", "dx_7x7x512", "3xtf32"): 47.1e6,
    ("conv_dw_halo_kernel", "dw_56x56x64", "3xtf32"): 415.5e6,
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
    ap.add_argument("--repeats", type=int, default=7, help="timed regions of --steps steps each; the median is reported")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="skip the TF32, Winograd, cu32 and config-3 sub-records")
    ap.add_argument("--no-peak", action="store_true", help="skip the in-run measurement of the TF32 matmul peak")
    ap.add_argument("--no-cu32", action="store_true")
    ap.add_argument("--no-config3", action="store_true")
    ap.add_argument("--config3-only", action="store_true",
                    help="profiling aid: run only the ResNet-18 conv stack (with --no-graph: eager launches) and print its record")
    ap.add_argument("--neighbours-only", action="store_true",
                    help="profiling aid: run only the batched matrix products and the pooling operators and print their record")
    ap.add_argument("--config3-batch", type=int, default=None,
                    help="global batch of the ResNet-18 stack (default 512); 64 on one GPU shows the per-GPU compute of the 8-GPU case")
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


def measure_tf32_peak(torch, dev, seconds=2.0):
    """Dense TF32 tensor-core throughput of this GPU, measured the way MEASURED_PEAKS.json measured
    bf16: torch.matmul on 8192^3 fp32 operands with TF32 allowed (a cuBLAS GEMM; the yardstick, not the
    product), best of 10 single calls ("burst") and back to back for `seconds` ("sustained")."""
    old = torch.backends.cuda.matmul.allow_tf32
    torch.backends.cuda.matmul.allow_tf32 = True
    try:
        n = 8192
        a = torch.randn((n, n), device=dev)
        b = torch.randn((n, n), device=dev)
        c = torch.empty((n, n), device=dev)
        flops = 2.0 * n ** 3
        for _ in range(3):
            torch.matmul(a, b, out=c)
        torch.cuda.synchronize()
        best = None
        for _ in range(10):
            e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
            e0.record(); torch.matmul(a, b, out=c); e1.record()
            torch.cuda.synchronize()
            ms = e0.elapsed_time(e1)
            best = ms if best is None else min(best, ms)
        reps = max(10, int(seconds * 1e3 / best))
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            torch.matmul(a, b, out=c)
        e1.record()
        torch.cuda.synchronize()
        sustained_ms = e0.elapsed_time(e1) / reps
        return {"burst": flops / (best * 1e-3) / 1e12, "sustained": flops / (sustained_ms * 1e-3) / 1e12,
                "how": "torch.matmul fp32 8192^3 with allow_tf32: best of 10 (burst), %d calls back to back (sustained)" % reps}
    finally:
        torch.backends.cuda.matmul.allow_tf32 = old


KERNELS = {"halo": "conv_halo_kernel", "halo_row": "conv_halo_kernel", "halo_tap": "conv_halo_kernel",
           "halo_pair_row": "conv_halo_pair_kernel", "halo_pair_tap": "conv_halo_pair_kernel",
           "igemm": "conv_igemm_kernel", "dw_halo": "conv_dw_halo_kernel", "dw": "conv_dw_kernel",
           "simt": "conv_*_simt"}


class Sweep:
    """The 3x3 layer sweep resident in HBM: tensors, the step, its CUDA graph and the timing loops."""

    def __init__(self, args, env):
        torch, synth, dev = env["torch"], env["synth"], env["dev"]
        self.args, self.env = args, env
        self.B = args.batch or synth.SWEEP_BATCH
        self.layers = []
        sweep = synth.SWEEP_LAYERS if args.only_layer is None else [synth.SWEEP_LAYERS[args.only_layer]]
        self.ops = OPS if args.only_op is None else (args.only_op,)
        B = self.B
        for hw, c in sweep:
            Xh, Wh, dYh = synth.sweep_layer(hw, c, batch=B, seed=env["rank"])
            Wh = synth.sweep_layer(hw, c, batch=1, seed=0)[1]  # weights are replicated: same seed on every rank
            L = dict(hw=hw, c=c,
                     X=torch.from_numpy(Xh).to(dev), W=torch.from_numpy(Wh).to(dev), dY=torch.from_numpy(dYh).to(dev),
                     Y=torch.empty((B, hw, hw, c), device=dev), dX=torch.empty((B, hw, hw, c), device=dev),
                     dW=torch.empty((c, 3, 3, c), device=dev), Xh=Xh, Wh=Wh, dYh=dYh,
                     flops=synth.conv_flops(B, hw, hw, c, 3, 3, c))
            self.layers.append(L)
        self.step_flops = sum(len(self.ops) * L["flops"] for L in self.layers)
        # the deltaW tensors of all layers are views of one flat buffer: one collective per step
        self.bucket = env["sharding"].GradientBucket([L["dW"].numel() for L in self.layers], dev)
        for i, L in enumerate(self.layers):
            L["dW"] = self.bucket.view(i, L["dW"].shape)
        self.op_streams = [torch.cuda.Stream() for _ in range(2)] if args.streams == 3 else []
        self.graph = None
        self.graph_has_allreduce = False
        self.graph_error = None
        self.launches_per_step = None

    def run_op(self, L, op):
        base, B = self.env["base"], self.B
        hw, c = L["hw"], L["c"]
        if op == "fwd":
            base.conv3D(L["Y"], hw, hw, L["X"], hw, hw, L["W"], 3, 3, B, c, c, 1, 1, 1, 1)
        elif op == "dx":
            base.dconv3D_deltaX(L["dX"], hw, hw, L["dY"], hw, hw, L["W"], 3, 3, B, c, c, 1, 1, 1, 1)
        else:
            base.dconv3D_deltaW(L["dW"], 3, 3, L["X"], hw, hw, L["dY"], hw, hw, B, c, c, 1, 1, 1, 1)

    def compute(self, events=None):
        torch, lib = self.env["torch"], self.env["lib"]
        if self.op_streams and events is None and len(self.ops) == 3:
            # the three contractions of a layer are independent: one stream each (the library keeps a
            # scratch block per stream).  Every kernel fills the GPU, so only their tails overlap.
            cur = torch.cuda.current_stream()
            fork = torch.cuda.Event(); fork.record(cur)
            for s_ in self.op_streams:
                s_.wait_event(fork)
            for L in self.layers:
                self.run_op(L, "fwd")
                with torch.cuda.stream(self.op_streams[0]):
                    self.run_op(L, "dx")
                with torch.cuda.stream(self.op_streams[1]):
                    self.run_op(L, "dw")
            for s_ in self.op_streams:
                cur.wait_stream(s_)
            return
        for li, L in enumerate(self.layers):
            for op in self.ops:
                if events is not None:
                    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
                    e0.record()
                self.run_op(L, op)
                if events is not None:
                    e1.record()
                    events.append((li, op, e0, e1, lib.last_algo()))

    def reduce_gradients(self):
        if self.env["world"] > 1 and "dw" in self.ops and os.environ.get("BENCH_AR", "full") != "none":
            self.env["dist"].all_reduce(self.bucket.flat, op=self.env["dist"].ReduceOp.SUM)

    def step(self, events=None):
        self.compute(events)
        self.reduce_gradients()

    def capture(self):
        """Captures the step's kernel launches - and, with several ranks, the all-reduce that follows them -
        into one CUDA graph: the tensor maps and shapes of a training step do not change, and a replay
        leaves neither launch gaps between the 0.1-0.4 ms kernels nor a host gap before the collective."""
        torch, lib = self.env["torch"], self.env["lib"]
        self.graph, self.graph_error = None, None
        with_ar = self.env["world"] > 1 and os.environ.get("BENCH_GRAPH_AR", "1") != "0"
        for attempt in ((True, False) if with_ar else (False,)):
            try:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    self.compute()
                    if attempt:
                        self.reduce_gradients()
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                gobj = torch.cuda.CUDAGraph()
                n0 = lib.launch_count()
                with torch.cuda.graph(gobj, stream=side):
                    self.compute()
                    if attempt:
                        self.reduce_gradients()
                self.launches_per_step = lib.launch_count() - n0
                for _ in range(3):
                    gobj.replay()
                    if not attempt:
                        self.reduce_gradients()
                torch.cuda.synchronize()
                st = lib.device_status()
                if st != 0:
                    raise RuntimeError("kernel status %d after graph replay" % st)
                self.graph, self.graph_has_allreduce = gobj, attempt
                return
            except Exception as e:  # fall back (collective outside the graph, then eager launches), and say so
                self.graph = None
                self.graph_error = str(e).splitlines()[0][:200]
                torch.cuda.synchronize()

    def replay_or_step(self, events=None):
        if self.graph is not None:
            self.graph.replay()
            if not self.graph_has_allreduce:
                self.reduce_gradients()
        else:
            self.step(events)

    def timed(self, steps, repeats, barrier):
        """`repeats` timed regions of exactly `steps` steps each, every region bracketed by a barrier and a
        device synchronisation on both sides; per region the max over ranks.  Returns ms per step of every region."""
        torch, dist, world, dev = self.env["torch"], self.env["dist"], self.env["world"], self.env["dev"]
        out = []
        for _ in range(repeats):
            barrier()
            t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(steps):
                self.replay_or_step()
            t1.record()
            barrier()
            ms = t0.elapsed_time(t1)
            if world > 1:
                t = torch.tensor([ms], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            out.append(ms / steps)
        return out

    def per_op_events(self, passes=8):
        torch = self.env["torch"]
        events = []
        self.compute([])   # single-stream warm-up: the library keeps one scratch block per stream
        for _ in range(passes):
            self.compute(events)
        torch.cuda.synchronize()
        per_op = {}
        for li, op, e0, e1, algo in events:
            L = self.layers[li]
            k = "%s_%dx%dx%d" % (op, L["hw"], L["hw"], L["c"])
            e = per_op.setdefault(k, dict(ms=[], flops=L["flops"], kernel=KERNELS.get(algo, algo), li=li, op=op))
            e["ms"].append(e0.elapsed_time(e1))
        return per_op


def check_allreduce(env, sweep):
    """Before anything is timed: every rank's partial deltaW of one layer is gathered, summed in double
    precision and compared with what the all-reduce over the bucket left in that layer's view."""
    torch, dist, world = env["torch"], env["dist"], env["world"]
    if world == 1 or "dw" not in sweep.ops:
        return None
    li = len(sweep.layers) - 1
    L = sweep.layers[li]
    sweep.run_op(L, "dw")
    torch.cuda.synchronize()
    part = L["dW"].clone()
    parts = [torch.empty_like(part) for _ in range(world)]
    dist.all_gather(parts, part)
    want = torch.stack([p.double() for p in parts]).sum(0)
    scale = torch.stack([p.double().abs() for p in parts]).sum(0)
    sweep.compute()
    sweep.reduce_gradients()
    torch.cuda.synchronize()
    got = sweep.bucket.view(li, L["dW"].shape).double()
    bad = float(((got - want).abs() - 1e-6 * scale).max())
    return "ok" if bad <= 0 else "MISMATCH (excess %.3e)" % bad


class Config3:
    """The conv stack of the reference's CIFAR-10 ResNet-18 (20 unbiased convolutions, Net.java:24-77),
    global batch 512 split evenly over the ranks (strong scaling): per step forward, deltaX and deltaW of
    every layer on the rank's shard, the 50 MB of weight gradients summed over the ranks by one all-reduce
    of a flat bucket the deltaW kernels write into.  Activations between the layers (batch norm, LeakyReLU,
    the residual adds) are not part of this path: every layer runs on seeded synthetic inputs of its shape."""

    def __init__(self, env, global_batch):
        torch, synth, dev, world, rank = env["torch"], env["synth"], env["dev"], env["world"], env["rank"]
        self.env = env
        self.global_batch = global_batch
        lo, hi = env["sharding"].shard_bounds(global_batch, rank, world)
        self.n = hi - lo
        g = torch.Generator(device=dev).manual_seed(1234 + rank)
        gw = torch.Generator(device=dev).manual_seed(99)
        self.layers = []
        for (IH, IC, OC, F, s, p) in synth.RESNET18_CONVS:
            OH = (IH + 2 * p - F) // s + 1
            X = torch.randn((self.n, IH, IH, IC), device=dev, generator=g).relu_() if IC > 4 else torch.rand((self.n, IH, IH, IC), device=dev, generator=g)
            if IC == 4:
                X[..., 3] = 0          # 3 colour planes padded to 4
            W = torch.randn((OC, F, F, IC), device=dev, generator=gw) * (2.0 / (F * F * IC)) ** 0.5
            dY = torch.randn((self.n, OH, OH, OC), device=dev, generator=g)
            self.layers.append(dict(IH=IH, IC=IC, OC=OC, F=F, s=s, p=p, OH=OH, X=X, W=W, dY=dY,
                                    Y=torch.empty((self.n, OH, OH, OC), device=dev), dX=torch.empty_like(X)))
        self.bucket = env["sharding"].GradientBucket([L["W"].numel() for L in self.layers], dev)
        for i, L in enumerate(self.layers):
            L["dW"] = self.bucket.view(i, L["W"].shape)
        self.flops = sum(3 * synth.conv_flops(global_batch, L["OH"], L["OH"], L["OC"], L["F"], L["F"], L["IC"]) for L in self.layers)
        self.streams = [torch.cuda.Stream() for _ in range(2)]
        # Weight-side transforms (lo plane of W for the forward pass, transposed planes for deltaX) depend on W
        # only: like a training loop after its optimizer step, the step enqueues them for all layers on a side
        # stream into blocks of its own, off the critical path of the forward and backward chains.
        self.prepare = os.environ.get("BENCH_C3_PREP", "1") != "0"
        self.ops = os.environ.get("BENCH_C3_OPS", "fwd,dx,dw").split(",")     # analysis aid: a subset of the three chains
        self.prep_stream = torch.cuda.Stream()
        base = env["base"]
        for L in self.layers:
            geo = (L["F"], L["F"], self.n, L["IH"], L["IH"], L["OH"], L["OH"], L["IC"], L["OC"], L["s"], L["s"], L["p"], L["p"])
            L["geo"] = geo
            L["pf"] = base.prepare_weights("forward", L["W"], *geo) if self.prepare else None
            L["pd"] = base.prepare_weights("deltaX", L["W"], *geo) if self.prepare else None
        # The gradient bucket is reduced in pieces, in backward order, on a communication stream, each piece as
        # soon as the deltaW kernels that fill it have run (layers are contiguous in the bucket).
        self.comm_stream = torch.cuda.Stream()
        n_chunks = max(1, int(os.environ.get("BENCH_C3_AR_BUCKETS", "4"))) if world > 1 else 1
        self.chunks = self.bucket.pieces(n_chunks)       # (first layer, last layer + 1) in backward order

    def chunk_view(self, lo, hi):
        return self.bucket.piece_view(lo, hi)

    def compute(self, with_reduce=False):
        torch, base, n, dist = self.env["torch"], self.env["base"], self.n, self.env["dist"]
        cur = torch.cuda.current_stream()
        fork = torch.cuda.Event(); fork.record(cur)
        for s_ in self.streams + [self.prep_stream]:
            s_.wait_event(fork)
        ready_f, ready_d = {}, {}
        if self.prepare:
            with torch.cuda.stream(self.prep_stream):
                for i, L in enumerate(self.layers):
                    if L["pf"] is not None:
                        base.prepare_weights_into(L["pf"], "forward", L["W"], *L["geo"], stream=self.prep_stream)
                        ready_f[i] = torch.cuda.Event(); ready_f[i].record(self.prep_stream)
                for i in range(len(self.layers) - 1, -1, -1):
                    L = self.layers[i]
                    if L["pd"] is not None:
                        base.prepare_weights_into(L["pd"], "deltaX", L["W"], *L["geo"], stream=self.prep_stream)
                        ready_d[i] = torch.cuda.Event(); ready_d[i].record(self.prep_stream)
        for i, L in enumerate(self.layers):
            if "fwd" not in self.ops:
                break
            a = (L["IH"], L["IH"])
            if i in ready_f:
                cur.wait_event(ready_f[i])
            base.conv3D_prepared(L["Y"], L["OH"], L["OH"], L["X"], *a, L["W"], L["F"], L["F"], n, L["IC"], L["OC"], L["s"], L["s"], L["p"], L["p"], L["pf"])
        chunk_end = {lo: (lo, hi) for lo, hi in self.chunks}
        for i in range(len(self.layers) - 1, -1, -1):
            L = self.layers[i]
            a = (L["IH"], L["IH"])
            with torch.cuda.stream(self.streams[0]):
                if i in ready_d:
                    self.streams[0].wait_event(ready_d[i])
                if "dx" in self.ops:
                    base.dconv3D_deltaX_prepared(L["dX"], *a, L["dY"], L["OH"], L["OH"], L["W"], L["F"], L["F"], n, L["IC"], L["OC"], L["s"], L["s"], L["p"], L["p"], L["pd"])
            with torch.cuda.stream(self.streams[1]):
                if "dw" in self.ops:
                    base.dconv3D_deltaW(L["dW"], L["F"], L["F"], L["X"], *a, L["dY"], L["OH"], L["OH"], n, L["IC"], L["OC"], L["s"], L["s"], L["p"], L["p"])
                if with_reduce and i in chunk_end and self.env["world"] > 1:
                    done = torch.cuda.Event(); done.record(self.streams[1])
                    self.comm_stream.wait_event(done)
                    with torch.cuda.stream(self.comm_stream):
                        dist.all_reduce(self.chunk_view(*chunk_end[i]), op=dist.ReduceOp.SUM)
        for s_ in self.streams + [self.prep_stream] + ([self.comm_stream] if with_reduce else []):
            cur.wait_stream(s_)

    def reduce(self):
        if self.env["world"] > 1:
            self.env["dist"].all_reduce(self.bucket.flat, op=self.env["dist"].ReduceOp.SUM)

    def check_reduce(self):
        """The bucket after the chunked, overlapped all-reduce against the double-precision sum of the per-rank
        partial gradients of two layers (first and last), gathered before anything is timed."""
        torch, dist, world = self.env["torch"], self.env["dist"], self.env["world"]
        if world == 1:
            return None
        self.compute(with_reduce=False)
        torch.cuda.synchronize()
        want = {}
        for i in (0, len(self.layers) - 1):
            part = self.layers[i]["dW"].clone()
            parts = [torch.empty_like(part) for _ in range(world)]
            dist.all_gather(parts, part)
            want[i] = (torch.stack([p.double() for p in parts]).sum(0), torch.stack([p.double().abs() for p in parts]).sum(0))
        self.compute(with_reduce=True)
        torch.cuda.synchronize()
        bad = max(float(((self.layers[i]["dW"].double() - w).abs() - 1e-6 * sc).max()) for i, (w, sc) in want.items())
        return "ok" if bad <= 0 else "MISMATCH (excess %.3e)" % bad

    def run(self, steps, repeats, barrier, use_graph=True):
        torch, lib, dist, world, dev = self.env["torch"], self.env["lib"], self.env["dist"], self.env["world"], self.env["dev"]
        for _ in range(3):
            self.compute(with_reduce=True)
        torch.cuda.synchronize()
        ar_check = self.check_reduce()
        graph, in_graph, err, launches = None, False, None, None
        with_ar = world > 1 and os.environ.get("BENCH_GRAPH_AR", "1") != "0"
        for attempt in (() if not use_graph else (True, False) if with_ar else (False,)):
            try:
                side = torch.cuda.Stream()
                side.wait_stream(torch.cuda.current_stream())
                with torch.cuda.stream(side):
                    self.compute(with_reduce=attempt)
                torch.cuda.current_stream().wait_stream(side)
                torch.cuda.synchronize()
                gobj = torch.cuda.CUDAGraph()
                n0 = lib.launch_count()
                with torch.cuda.graph(gobj, stream=side):
                    self.compute(with_reduce=attempt)
                launches = lib.launch_count() - n0
                gobj.replay()
                torch.cuda.synchronize()
                graph, in_graph = gobj, attempt
                break
            except Exception as e:
                err = str(e).splitlines()[0][:200]
                torch.cuda.synchronize()

        def one():
            if graph is not None:
                graph.replay()
                if not in_graph:
                    self.reduce()
            else:
                self.compute(with_reduce=True)
        for _ in range(3):
            one()
        if launches is None:
            n0 = lib.launch_count(); self.compute(with_reduce=True); launches = lib.launch_count() - n0
        regions = []
        for _ in range(repeats):
            barrier()
            t0 = torch.cuda.Event(enable_timing=True); t1 = torch.cuda.Event(enable_timing=True)
            t0.record()
            for _ in range(steps):
                one()
            t1.record()
            barrier()
            ms = t0.elapsed_time(t1)
            if world > 1:
                t = torch.tensor([ms], device=dev, dtype=torch.float64)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            regions.append(ms / steps)
        status = lib.device_status()
        ms_step = statistics.median(regions)
        return {"workload": "ResNet-18 conv stack (20 convolutions of the reference's CIFAR-10 net) on 32x32x3 images, "
                            "forward + deltaX + deltaW of every layer, deltaW all-reduced",
                "global_batch": self.global_batch, "batch_per_gpu": self.n, "scaling": "strong",
                "ms_per_step": ms_step, "img_s": self.global_batch / (ms_step * 1e-3), "tflops": self.flops / (ms_step * 1e-3) / 1e12,
                "ms_per_step_regions": [round(x, 4) for x in regions], "steps_per_region": steps,
                "gpu_launches_per_step": int(launches), "allreduce_bytes": int(self.bucket.flat.numel() * 4) if world > 1 else 0,
                "launch": ("CUDA graph" + (" incl. the all-reduce" if in_graph else "") if graph is not None else "eager launches"),
                "allreduce": ("%d pieces in backward order on a communication stream, overlapped with the remaining kernels" % len(self.chunks)
                              if world > 1 and (in_graph or graph is None) else ("one piece after the step" if world > 1 else None)),
                "weight_transforms": "prepared on a side stream into caller-owned blocks" if self.prepare else "inside every call",
                "allreduce_check": ar_check, "graph_error": err, "kernel_status": status}


def cu32_baseline(env, sweep, iters=3):
    """The reference's own cu32 SIMT kernels, rebuilt for sm_100 from its checkout (oracle/_ref/libcu32_*.so,
    test infrastructure), on the four sweep layers of this run: forward, deltaX and deltaW through the
    reference's JNI natives in its engine's call order, device time between synchronisations."""
    torch = env["torch"]
    try:
        from oracle import cu32_ref
        if not cu32_ref.available():
            return {"unavailable": "oracle/_ref/libcu32_*.so are not built (they need the reference checkout at build time)"}
        R = cu32_ref.Cu32Reference()
        total, per_op = 0.0, {}
        for L in sweep.layers:
            hw, c = L["hw"], L["c"]
            calls = (("fwd", lambda: R.conv3D(L["X"], L["W"], 1, 1, 1, 1)),
                     ("dx", lambda: R.dconv3D_deltaX(L["dY"], L["W"], hw, hw, 1, 1, 1, 1)),
                     ("dw", lambda: R.dconv3D_deltaW(L["X"], L["dY"], 3, 3, 1, 1, 1, 1)))
            for op, f in calls:
                f()
                torch.cuda.synchronize()
                t0 = time.perf_counter()
                for _ in range(iters):
                    f()       # every call ends with a device synchronisation
                ms = (time.perf_counter() - t0) / iters * 1e3
                total += ms
                per_op["%s_%dx%dx%d" % (op, hw, hw, c)] = round(L["flops"] / (ms * 1e-3) / 1e12, 2)
        return {"ms_per_step": total, "value": sweep.step_flops / (total * 1e-3) / 1e12, "unit": UNIT, "per_op_tflops": per_op,
                "kind": "the reference's cu32 kernels (fp32 FFMA) compiled for sm_100, same GPU, same tensors",
                "timing": "wall clock between device synchronisations, %d calls per contraction, allocations of the harness included" % iters}
    except Exception as e:
        return {"unavailable": "cu32 baseline failed: %s" % str(e).splitlines()[0][:160]}


def run_ours(args):
    import numpy as np  # noqa: F401
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
        # NCCL announces its version on stdout when the first communicator comes up; the line of this program is the
        # only thing that belongs there, so file descriptor 1 points at stderr until that has happened
        sys.stdout.flush()
        saved = os.dup(1)
        os.dup2(2, 1)
        try:
            dist.init_process_group("nccl", device_id=dev)
            warm = torch.zeros(1, device=dev)
            dist.all_reduce(warm)
            torch.cuda.synchronize()
        finally:
            sys.stdout.flush()
            os.dup2(saved, 1)
            os.close(saved)

    lib = submodule("lib")
    synth = submodule("synth")
    env = dict(torch=torch, dist=dist, world=world, rank=rank, dev=dev, lib=lib, synth=synth,
               sharding=submodule("sharding"), base=submodule("engine").CudaFloat32EngineBase())
    lib.set_math_mode(args.math)
    peaks = measured_peaks()
    extras = not args.no_extras and args.only_layer is None and args.only_op is None

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    if args.neighbours_only:
        rec = neighbour_ops(env) if rank == 0 else None
        if rank == 0:
            print(json.dumps({"metric": "batched matrix products and pooling (profiling aid)", "n_gpus": world, "neighbours": rec}))
        if world > 1:
            dist.destroy_process_group()
        return
    if args.config3_only:
        rec = Config3(env, args.config3_batch or synth.RESNET18_BATCH).run(args.steps, args.repeats, barrier, use_graph=not args.no_graph)
        if rank == 0:
            print(json.dumps({"metric": "ResNet-18 conv stack step (profiling aid)", "value": rec["img_s"], "unit": "img/s",
                              "n_gpus": world, "steps": args.steps, "config3": rec}))
        if world > 1:
            dist.destroy_process_group()
        return
    sweep = Sweep(args, env)
    B = sweep.B
    warm = max(args.warmup, 3)
    for _ in range(warm):
        sweep.step()
    barrier()
    ar_check = check_allreduce(env, sweep)
    if not args.no_graph and os.environ.get("BENCH_AR", "full") in ("full", "none"):
        sweep.capture()
        barrier()
    for _ in range(warm):
        sweep.replay_or_step()
    uuid = None
    try:
        uuid = "GPU-" + str(torch.cuda.get_device_properties(dev).uuid)
    except Exception:
        pass
    sampler = ClockSampler(uuid) if rank == 0 else None
    if sampler:
        sampler.start()
    launches0 = lib.launch_count()
    regions = sweep.timed(args.steps, args.repeats, barrier)
    eager_launches = lib.launch_count() - launches0
    clocks = sampler.stop() if sampler else None
    per_op = sweep.per_op_events()
    status = lib.device_status()
    if status != 0:
        raise SystemExit("bench.py: kernel status word %d: %s" % (status, lib.last_error()))
    ms_step = statistics.median(regions)
    value = world * sweep.step_flops / (ms_step * 1e-3) / 1e12
    launch_desc = ("CUDA graph of the step's kernels%s, replayed" % (" and its all-reduce" if sweep.graph_has_allreduce else "")
                   if sweep.graph is not None else "eager launches")
    launch_desc += ", forward / deltaX / deltaW on three streams" if sweep.op_streams else ""
    headline_graph_error = sweep.graph_error
    launches = sweep.launches_per_step * args.steps if sweep.graph is not None else eager_launches // max(args.repeats, 1)

    # ---- measured TF32 peak of this GPU (the roofline's denominator) ----
    tf32_peak = measure_tf32_peak(torch, dev) if not args.no_peak else None

    # per-kernel time from per-op CUDA events; the roofline is reported for the kernel with the largest
    # share of the step, on its longest-running launch shape
    fam = {}
    for k, v in per_op.items():
        f = fam.setdefault(v["kernel"], dict(ms=0.0, n=0))
        f["ms"] += statistics.mean(v["ms"]); f["n"] += 1
    fam_total = max(sum(f["ms"] for f in fam.values()), 1e-9)
    dom = max(fam, key=lambda k: fam[k]["ms"])
    heavy = max((k for k in per_op if per_op[k]["kernel"] == dom), key=lambda k: statistics.mean(per_op[k]["ms"]))
    h = per_op[heavy]
    hl = sweep.layers[h["li"]]
    launch_ms = statistics.mean(h["ms"])
    achieved = h["flops"] / (launch_ms * 1e-3) / 1e12
    # a launch timed alone, well under a second, with the SM clock at its maximum meets the burst figure;
    # anything else the sustained one
    at_max = bool(clocks and clocks.get("sm_mhz") and clocks.get("sm_max_mhz") and clocks["sm_mhz"] >= 0.97 * clocks["sm_max_mhz"])
    if tf32_peak is not None:
        use_burst = at_max and launch_ms < 1000.0
        peak = tf32_peak["burst"] if use_burst else tf32_peak["sustained"]
        peak_source = "measured in this run: %s; %s figure (SM clock %s its maximum during the timed region)" % (
            tf32_peak["how"], "burst" if use_burst else "sustained", "at" if at_max else "below")
    else:
        peak = peaks["bf16"] / 2.0
        peak_source = "%s bf16 burst %.1f TFLOP/s / 2 (dense TF32 rate is half the bf16 rate)" % (peaks["source"], peaks["bf16"])
    alg_bytes = synth.conv_bytes(B, hl["hw"], hl["hw"], hl["c"], hl["hw"], hl["hw"], hl["c"], 3, 3)
    roofline = {
        "bound": "tensor", "kernel": dom, "launch": heavy, "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
        "frac": achieved / peak, "traffic": NCU_TRAFFIC.get((dom, heavy, args.math)), "algorithmic_bytes": alg_bytes,
        "peak_source": peak_source,
        "note": "3xTF32 issues three MMAs per product, so its useful-FLOP ceiling is peak/3" if args.math == "3xtf32" else "plain TF32",
        "time_share": fam[dom]["ms"] / fam_total,
        "kernel_time_shares": {k: round(v["ms"] / fam_total, 3) for k, v in fam.items()},
        "step_frac_of_peak": value / world / peak,
    }
    per_op_tflops = {k: v["flops"] / (statistics.mean(v["ms"]) * 1e-3) / 1e12 for k, v in per_op.items()}

    # ---- the same sweep in plain TF32 (the opt-in mode the 60 %-of-peak target is stated in) ----
    tf32 = None
    if extras and args.math == "3xtf32":
        lib.set_math_mode("tf32")
        for _ in range(3):
            sweep.step()
        if sweep.graph is not None:
            sweep.capture()
        for _ in range(3):
            sweep.replay_or_step()
        r2 = sweep.timed(args.steps, max(3, args.repeats // 2), barrier)
        po = sweep.per_op_events()
        ms2 = statistics.median(r2)
        pk = tf32_peak["burst"] if tf32_peak else peaks["bf16"] / 2.0
        tf32 = {"ms_per_step": ms2, "value": world * sweep.step_flops / (ms2 * 1e-3) / 1e12, "unit": UNIT,
                "ms_per_step_regions": [round(x, 4) for x in r2],
                "per_op_tflops": {k: round(v["flops"] / (statistics.mean(v["ms"]) * 1e-3) / 1e12, 1) for k, v in po.items()},
                "forward_frac_of_tf32_peak": {k: round(v["flops"] / (statistics.mean(v["ms"]) * 1e-3) / 1e12 / pk, 3)
                                              for k, v in po.items() if k.startswith("fwd")},
                "peak": pk, "peak_kind": "burst (single launches timed alone)", "kernel_status": lib.device_status()}
        if tf32_peak:
            # the per-op times above come from passes that follow seconds of continuous load (clocks at the power cap):
            # the like-for-like yardstick is the matmul peak sustained under the same cap; the burst figure is the stricter one
            tf32["forward_frac_of_tf32_peak_sustained"] = {
                k: round(v["flops"] / (statistics.mean(v["ms"]) * 1e-3) / 1e12 / tf32_peak["sustained"], 3)
                for k, v in po.items() if k.startswith("fwd")}
            tf32["peak_sustained"] = tf32_peak["sustained"]
        lib.set_math_mode(args.math)
        for _ in range(2):
            sweep.step()
        if sweep.graph is not None:
            sweep.capture()

    # ---- Winograd F(2,3) forward variant, per layer ----
    wino = None
    if extras:
        wino = {}
        try:
            for mode in ((args.math, "tf32") if args.math == "3xtf32" else (args.math,)):
                lib.set_math_mode(mode)
                lib.set_algo("winograd")
                for L in sweep.layers:
                    for _ in range(2):
                        sweep.run_op(L, "fwd")
                    e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
                    e0.record()
                    for _ in range(5):
                        sweep.run_op(L, "fwd")
                    e1.record(); torch.cuda.synchronize()
                    wino["fwd_%dx%dx%d_%s" % (L["hw"], L["hw"], L["c"], mode)] = round(L["flops"] / (e0.elapsed_time(e1) / 5 * 1e-3) / 1e12, 1)
        finally:
            lib.set_algo("auto")
            lib.set_math_mode(args.math)
        wino["note"] = "TFLOP/s credited with the direct convolution's FLOPs; AUTO never selects this variant"

    # ---- operators next to the convolutions: batched matrix products and pooling (rank 0, single GPU runs only) ----
    neighbours = neighbour_ops(env) if (extras and rank == 0 and world == 1) else None

    # ---- the reference's own GPU kernels on the same tensors (rank 0, single GPU runs only) ----
    cu32 = cu32_baseline(env, sweep) if (extras and rank == 0 and world == 1 and not args.no_cu32) else None

    # ---- end to end from pinned host buffers ----
    e2e = None
    if not args.no_e2e and args.only_layer is None and args.only_op is None:
        e2e = run_e2e(args, torch, dist, dev, world, sweep.layers, sweep.run_op, sweep.step_flops, B, None)

    # ---- config 3: ResNet-18 conv stack, global batch 512, strong scaling ----
    config3 = None
    if extras and not args.no_config3:
        sweep.graph = None
        c3 = Config3(env, args.config3_batch or synth.RESNET18_BATCH)
        config3 = c3.run(max(10, args.steps), max(3, args.repeats), barrier)

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
            "warmup": warm, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "tf32x3 (fp32-faithful split)" if args.math == "3xtf32" else "tf32",
            "data": "synthetic",
            "config": {"workload": "3x3 s1 p1 layer sweep (56x56x64, 28x28x128, 14x14x256, 7x7x512), fwd+deltaX+deltaW",
                       "batch_per_gpu": B, "global_batch": B * world, "math": args.math,
                       "parallelism": "batch-sharded x%d, deltaW all-reduce" % world if world > 1 else "single GPU",
                       "l2": "inputs larger than L2 (%.2f GB of tensors per step)" % (
                           sum(4.0 * (2 * L["X"].numel() + 2 * L["Y"].numel() + 2 * L["W"].numel()) for L in sweep.layers) / 1e9),
                       "launch": launch_desc,
                       "timing": "median of %d timed regions of %d steps each (CUDA events, max over ranks)" % (args.repeats, args.steps)},
            "ms_per_step_regions": [round(x, 4) for x in regions],
            "roofline": roofline, "tf32_peak": tf32_peak, "cpu_baseline": cpu, "cu32_baseline": cu32, "e2e": e2e,
            "gpu_launches": int(launches), "clocks": clocks,
            "per_op_tflops": {k: round(v, 1) for k, v in per_op_tflops.items()},
            "tf32": tf32, "winograd": wino, "neighbours": neighbours, "config3": config3, "allreduce_check": ar_check,
            "graph_error": headline_graph_error,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        # graphs that captured the all-reduce must be gone, and every rank done, before the communicator goes
        sweep.graph = None
        import gc
        gc.collect()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        dist.destroy_process_group()


def neighbour_ops(env):
    """Batched matrix products (Cuda_batchMatMul) and pooling (Cuda_pool2D / Cuda_upool2D) through the same library:
    CUDA events over 20 calls each after 3 warm-up calls, device tensors resident.  Products: the shape of the
    reference's own table (batch 32 x 8, N = M = 128, K = 256) in TFLOP/s; pooling: the max pool after an ImageNet
    stem (256 x 112 x 112 x 64, 3x3 s2 p1) and its gradient as algorithmic bytes per second against the measured
    copy bandwidth."""
    from __graft_entry__ import submodule
    torch, lib = env["torch"], env["lib"]
    E = submodule("engine").Engine()
    dev = env["dev"]

    def timed(f, iters=20):
        for _ in range(3):
            f()
        torch.cuda.synchronize()
        e0 = torch.cuda.Event(enable_timing=True); e1 = torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(iters):
            f()
        e1.record(); torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters

    out = {}
    try:
        g = torch.Generator(device=dev); g.manual_seed(11)
        Bt, N, M, K = 256, 128, 128, 256
        A = torch.randn((Bt, N, K), device=dev, generator=g); Bm = torch.randn((Bt, K, M), device=dev, generator=g)
        A1 = torch.randn((Bt, K, N), device=dev, generator=g); B2 = torch.randn((Bt, M, K), device=dev, generator=g)
        fl = 2.0 * Bt * N * M * K
        bm = {"shape": "batch 256, N = M = 128, K = 256", "unit": "TFLOP/s"}
        for name, f in (("batchMatMul", lambda: E.batchMatMul(A, Bm)), ("batchMatMulT1", lambda: E.batchMatMulT1(A1, Bm)),
                        ("batchMatMulT2", lambda: E.batchMatMulT2(A, B2))):
            ms = timed(f)
            bm[name] = {"ms": round(ms, 4), "tflops": round(fl / ms / 1e9, 1), "algo": lib.last_algo()}
        out["batch_matmul"] = bm
        del A, Bm, A1, B2
        X = torch.randn((256, 112, 112, 64), device=dev, generator=g)
        win = (3, 3, 2, 2, 1, 1)
        Y = E.pool2D_max(X, *win)
        dY = torch.randn(Y.shape, device=dev, generator=g)
        xb, yb = 4.0 * X.numel(), 4.0 * Y.numel()
        peak = measured_peaks()["hbm_gbs"]
        pl = {"shape": "256 x 112 x 112 x 64, 3x3 s2 p1", "unit": "GB/s of algorithmic bytes", "hbm_peak_gbs": peak}
        for name, f, nbytes in (("pool2D_max", lambda: E.pool2D_max(X, *win), xb + yb),
                                ("pool2D_avg", lambda: E.pool2D_avg(X, *win), xb + yb),
                                ("upool2D_max", lambda: E.upool2D_max(dY, Y, X, *win), 2 * xb + 2 * yb),
                                ("upool2D_avg", lambda: E.upool2D_avg(dY, 112, 112, *win), xb + yb)):
            ms = timed(f)
            gbs = nbytes / ms / 1e6
            pl[name] = {"ms": round(ms, 4), "gbs": round(gbs, 0), "frac_of_hbm_peak": round(gbs / peak, 3)}
        out["pool"] = pl
        out["kernel_status"] = lib.device_status()
    except Exception as e:      # a sub-record must not take the headline down with it
        out["error"] = "%s: %s" % (type(e).__name__, str(e)[:200])
    return out


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
