"""Benchmark of the deformable-conv3d hot path.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--mode auto|fp32|bf16x3|bf16] [--impl reference]

One "step" is one pass of the hot path over one batch of synthetic input: forward plus full
backward (all five gradients) of the modulated deformable conv3d layer of the headline
configuration -- B=2 clips per GPU, Cin=Cout=512, T=8, H=30, W=54, 3x3x3, pad 1, 8 deformable
groups, offsets ~ N(0, 2 voxels), mask = sigmoid(N(0,1)), Kaiming-normal weights, fp32 tensors.
With N > 1 (launched by torchrun, one rank per GPU) every rank owns its own clips (weak scaling,
no data-path collective) and only grad_weight/grad_bias are all-reduced over NCCL inside the step.

Prints ONE JSON line (rank 0).  `value` = contraction TFLOP/s of the whole job with inputs
resident in HBM (3 x 2*B*V*Cout*Cin*K flops per step: forward, dcol and dW contractions);
`e2e` = the same metric with host buffers (pinned H2D of the step's inputs, D2H of its results,
inside the timed region); `roofline` describes the dominant kernel phase as timed by the
library's own CUDA events during the timed steps; `cpu_baseline` is the CPU restatement of the
reference algorithm (oracle/) on a bounded sample of the same workload.

`--impl reference` times the UNMODIFIED reference op on the same inputs with the same protocol: its compiled
CUDA extension from baseline/_ref (the reference has no CPU implementation of this op) -- every rank on its own
clips, grad_weight all-reduced, device-timed value and host-buffer `e2e` like the line above; the CPU
restatement (oracle/) is timed beside it on rank 0 and reported as `cpu_baseline`.  Only when that extension
cannot be loaded or there is no GPU does the arm fall back to the CPU restatement alone (rank 0), saying why.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOAD = dict(name="C2 modulated deformable conv3d 512->512, 8x30x54, 3x3x3 pad 1, G=8, B=2 clips/GPU, fwd+bwd",
                B=2, Cin=512, Cout=512, dims=(8, 30, 54), k=3, pad=1, G=8, offset_std=2.0)
METRIC = "deform_conv3d_layer_fwd_bwd_tflops"
UNIT = "TFLOP/s"


def fwd_flops(B, Cin, Cout, V, K, groups=1):
    return 2.0 * B * V * Cout * (Cin // groups) * K


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        return dict(hbm_gbs=p["hbm_gbs"], tensor_burst=p["bf16_tflops"], tensor_sustained=p["bf16_tflops_sustained"],
                    source="measured")
    return dict(hbm_gbs=6650.0, tensor_burst=1590.0, tensor_sustained=1400.0, source="fallback")


def make_inputs(seed, wl, B=None, dims=None):
    """Seeded synthetic inputs generated on the host in fp32 (same bits for CPU and GPU paths)."""
    from tests._util import make_problem
    p = make_problem(seed, B or wl["B"], wl["Cin"], wl["Cout"], dims or wl["dims"], k=wl["k"], padding=wl["pad"],
                     G=wl["G"], dtype=np.float32, offset_std=wl["offset_std"])
    p["bias"] = np.zeros_like(p["bias"])
    return p


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons; `summary(t0, t1)` keeps the samples that arrived
    inside the timed window (host clock)."""

    FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.gpu_index, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True, bufsize=1)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def wait_for_samples(self, n=2, timeout=5.0):
        t0 = time.time()
        while self.proc is not None and len(self.lines) < n and time.time() - t0 < timeout:
            time.sleep(0.05)

    def stop(self):
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()

    def summary(self, t0, t1):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

        def collect(lo, hi):
            sm, mx, reasons, power = [], None, set(), []
            for ts, ln in self.lines:
                if not (lo <= ts <= hi):
                    continue
                f = [x.strip() for x in ln.split(",")]
                if len(f) < 9:
                    continue
                try:
                    sm.append(float(f[1])); mx = float(f[2]); power.append(float(f[3]))
                except ValueError:
                    continue
                for nm, val in zip(names, f[5:9]):
                    if val.lower().startswith("active"):
                        reasons.add(nm)
            return sm, mx, reasons, power

        sm, mx, reasons, power = collect(t0, t1 + 0.06)
        window = "timed region"
        if len(sm) < 2:   # very short timed region: fall back to everything sampled under load
            sm, mx, reasons, power = collect(0, float("inf"))
            window = "warm-up + timed region (timed region shorter than the sampling period)"
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power) if power else None, "window": window}


# ---- CPU arm (oracle) ----------------------------------------------------------------------------

SAMPLE_LADDER = [(8, 30), (4, 30), (2, 30), (2, 15), (2, 8), (2, 4)]


def cpu_step(orc, p):
    kw = dict(stride=1, padding=1, dilation=1, groups=1, offset_groups=WORKLOAD["G"])
    orc.deform_conv3d_fwd(p["x"], p["geo"], p["mask"], p["weight"], p["bias"], **kw)
    orc.deform_conv3d_bwd(p["gy"], p["x"], p["geo"], p["mask"], p["weight"], True, **kw)


def cpu_arm(steps, warmup, budget_s):
    """Times the oracle (forward + backward) on a slab of one clip of the workload, picked from a
    ladder so that warmup+steps fit the time budget.  Returns (TFLOP/s, ms per step, sample text)."""
    from oracle import oracle as orc
    wl = WORKLOAD
    # all host cores, whatever OMP_NUM_THREADS the launcher exported (torchrun sets 1 for its ranks)
    avail = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    cores = orc.set_threads(avail)
    probe = make_inputs(5, wl, B=1, dims=(2, 4, wl["dims"][2]))
    cpu_step(orc, probe)
    t0 = time.perf_counter(); cpu_step(orc, probe); tp = time.perf_counter() - t0
    per_voxel = tp / (2 * 4 * wl["dims"][2])
    target = budget_s / max(1, steps + warmup)
    d, h = SAMPLE_LADDER[-1]
    for dd, hh in SAMPLE_LADDER:
        if per_voxel * dd * hh * wl["dims"][2] <= target:
            d, h = dd, hh
            break
    p = make_inputs(6, wl, B=1, dims=(d, h, wl["dims"][2]))
    for _ in range(warmup):
        cpu_step(orc, p)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_step(orc, p)
    dt = (time.perf_counter() - t0) / steps
    V = d * h * wl["dims"][2]
    flops = 3 * fwd_flops(1, wl["Cin"], wl["Cout"], V, 27)
    sample = (f"1 clip, {d}x{h}x{wl['dims'][2]} slab of the workload volume (same channels, groups, kernel), "
              f"fwd+bwd, fp32, OpenMP on {cores} threads")
    return flops / dt / 1e12, dt * 1e3, sample, cores


def run_reference_arm(args):
    """The reference's own implementation of the path.  Its op is CUDA-only (every tensor is checked with
    is_cuda, ops/dconv-native/csrc/ops/dconv_gpu_common.h:32-36), so the like-for-like arm is its compiled
    extension on the same GPU(s); the CPU restatement is the fallback and the `cpu_baseline` figure."""
    rank = int(os.environ.get("RANK", "0"))
    why = None
    try:
        import torch
        from tests import _reference
        if not torch.cuda.is_available():
            why = "no CUDA device"
        elif _reference.load("dconv_native") is None:
            why = "baseline/_ref (the reference's compiled extension) is absent or does not import"
    except Exception as exc:                                  # pragma: no cover
        why = f"{type(exc).__name__}: {exc}"
    if why is None:
        return run_gpu_arm(args, impl="reference")
    if rank != 0:
        return
    val, ms, sample, cores = cpu_arm(args.steps, args.warmup, budget_s=150.0)
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": {"workload": WORKLOAD["name"], "l2": "host run"},
        "cpu_baseline": {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
        "note": f"reference CUDA op not usable here ({why}); this line times the CPU restatement of its algorithm (oracle/)",
    }
    print(json.dumps(line), flush=True)


# ---- GPU arm ---------------------------------------------------------------------------------------

# dram__bytes_read.sum + dram__bytes_write.sum of ONE launch, from ncu captures of this workload at full size
# (None where no capture has been taken).  TRAFFIC_SOURCE names the capture; kernels changed after it keep their
# entry only if the change cannot alter DRAM traffic.
TRAFFIC_SOURCE = "ncu --set full capture of this bench's C2 step, one launch per kernel, both math modes"
TRAFFIC_PER_LAUNCH = {       # (phase, math mode) -> DRAM read + write bytes of one launch
    # the forward keeps its operand tiles for the weight gradient (sample cache): + 0.72 / 1.44 GB written
    ("fwd_sm100_fused", "bf16"): 0.411e9 + 0.762e9, ("fwd_sm100_fused", "auto"): 1.560e9 + 1.648e9,
    ("fwd_sm100_fused", "bf16x3"): 1.560e9 + 1.648e9,
    ("bwd_sample_grad", "bf16"): 1.603e9 + 0.137e9, ("bwd_sample_grad", "auto"): 1.630e9 + 0.137e9,
    ("bwd_sample_grad", "bf16x3"): 1.630e9 + 0.137e9,
    ("bwd_dcol_sm100", "bf16"): 0.112e9 + 1.383e9, ("bwd_dcol_sm100", "auto"): 0.634e9 + 1.393e9,
    ("bwd_dcol_sm100", "bf16x3"): 0.634e9 + 1.393e9,
    ("bwd_dw_sm100_saved", "bf16"): 0.781e9 + 0.004e9, ("bwd_dw_sm100_saved", "auto"): 1.530e9 + 0.004e9,
    ("bwd_dw_sm100_saved", "bf16x3"): 1.530e9 + 0.004e9,
    # gather route of the weight gradient (sample cache off)
    ("bwd_dw_sm100", "bf16"): 0.430e9 + 0.073e9, ("bwd_dw_sm100", "auto"): 0.592e9 + 0.127e9,
    ("bwd_dw_sm100", "bf16x3"): 0.592e9 + 0.127e9,
}
# The sampling-gradient kernel's real limiter: every live corner of every sample adds 64 fp32 channels into the
# L2-resident grad_input accumulator.  payload_bytes = corners inside the volume for the benchmark's offsets
# (5.69 of 8 per sample on average at sigma = 2 voxels, D = 8) x 5.6 M samples x 256 B; rate = what
# red.global.add.v4.f32 sustains on this part for exactly this access pattern (microbenchmark, 11.5 GB in 1.69 ms).
SCATTER = {"payload_bytes": 5.687 * 2 * 8 * 27 * 12960 * 256, "rate_gbs": 6773.0,
           "source": "d2conv3d_b200/csrc/microbench/l2_rates.cu on a B200 of this pool"}

PHASE_WORK = {
    # phase name -> (bound, key of the algorithmic work of one launch)
    "fwd_sm100_fused": ("tensor", "F"), "fwd_generic": ("tensor", "F"),
    "bwd_dcol_sm100": ("tensor", "F"), "bwd_dcol_generic": ("tensor", "F"),
    "bwd_dw_sm100": ("tensor", "F"), "bwd_dw_sm100_saved": ("tensor", "F"), "bwd_dw_generic": ("tensor", "F"),
    "bwd_sample_grad": ("hbm", "sample_grad_bytes"),
    "bwd_coord_grad_generic": ("hbm", "coord_bytes"), "bwd_col2im_generic": ("hbm", "col2im_bytes"),
}


def time_reference_cuda_op(host, w, bias, wl, F):
    """The reference's own CUDA op (unmodified sources built into baseline/_ref), same inputs, same GPU:
    the kernel to beat.  Its kernels launch on the legacy default stream, so every measurement is
    bracketed by device-wide synchronisation.  Returns None when the build is absent."""
    import torch
    from tests import _reference
    ref = _reference.load("dconv_native")
    if ref is None:
        return None
    try:
        torch.backends.cuda.matmul.allow_tf32 = False
        dev = w.device
        x, off, mask, gy = (host[k].to(dev) for k in ("x", "geo", "mask", "gy"))
        ts = [t.detach().clone().requires_grad_() for t in (x, off, mask, w, bias)]
        torch.cuda.reset_peak_memory_stats()

        def one():
            for t in ts:
                t.grad = None
            torch.cuda.synchronize()
            e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
            e[0].record()
            y = ref.deform_conv3d(*ts, 1, wl["pad"], 1, 1, wl["G"])
            e[1].record()
            y.backward(gy)
            e[2].record()
            torch.cuda.synchronize()
            return e[0].elapsed_time(e[1]), e[1].elapsed_time(e[2])

        for _ in range(2):
            one()
        runs = [one() for _ in range(5)]
        fwd = statistics.median(r[0] for r in runs)
        bwd = statistics.median(r[1] for r in runs)
        return {"fwd_ms": fwd, "bwd_ms": bwd, "ms_per_step": fwd + bwd, "value": 3 * F / ((fwd + bwd) * 1e-3) / 1e12,
                "unit": UNIT, "peak_mem_gb": torch.cuda.max_memory_allocated() / 1e9,
                "what": "unmodified reference dconv_native (im2col + cuBLAS fp32, allow_tf32=False), median of 5"}
    except Exception as exc:  # the reference op is outside our control; report instead of failing the bench
        return {"error": f"{type(exc).__name__}: {exc}"}


def bind_to_gpu_numa_node(local_rank):
    """Pins this process to the CPUs that NVML reports as nearest to its GPU (read-only query), BEFORE any pinned
    host buffer is allocated, so that the buffers land on that NUMA node and N ranks do not all stream through
    one socket's memory.  Returns a short description for the JSON line."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(local_rank)
        n_words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, n_words)
        cpus = {64 * i + b for i, w in enumerate(mask) for b in range(64) if (w >> b) & 1}
        allowed = os.sched_getaffinity(0)
        cpus &= allowed
        if cpus:
            os.sched_setaffinity(0, cpus)
            return f"{len(cpus)} CPUs near GPU {local_rank} (NVML affinity)"
        return "NVML affinity empty: unchanged"
    except Exception as exc:
        return f"unchanged ({type(exc).__name__})"


def run_gpu_arm(args, impl="ours"):
    """One step = forward + full backward of the C2 layer on every rank's own clips; with N > 1 the parameter
    gradients are all-reduced (NCCL) inside the step.  impl = "ours": this library; impl = "reference": the
    reference's compiled CUDA op from baseline/_ref, same inputs, same timing protocol."""
    import torch
    import torch.distributed as dist

    import d2conv3d_b200
    from d2conv3d_b200 import _lib, dconv_native, sharding

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.gpus != world:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch N>1 with torchrun (one rank per GPU)")
    affinity = bind_to_gpu_numa_node(local_rank)
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    ours = impl == "ours"
    _lib.lib()
    wl = WORKLOAD
    peaks = measured_peaks()
    if ours:
        d2conv3d_b200.set_math_mode(args.mode)
        op = lambda *t: dconv_native.deform_conv3d(*t, 1, wl["pad"], 1, 1, wl["G"])
    else:
        from tests import _reference
        ref = _reference.load("dconv_native")
        torch.backends.cuda.matmul.allow_tf32 = False          # the reference's cuBLAS path in plain fp32
        op = lambda *t: ref.deform_conv3d(*t, 1, wl["pad"], 1, 1, wl["G"])

    p = make_inputs(1002 + rank, wl)
    # ONE pinned buffer per direction: the four inputs of a step are slices of `host_in` (and of one device
    # buffer), so a step's upload is a single copy
    keys = ("x", "geo", "mask", "gy")
    sizes = [p[k].size for k in keys]
    offs = np.concatenate([[0], np.cumsum([(n + 63) // 64 * 64 for n in sizes])])      # 256-byte aligned slices
    host_in = torch.empty(int(offs[-1]), dtype=torch.float32).pin_memory()
    for k, o, n in zip(keys, offs, sizes):
        host_in[int(o):int(o) + n].copy_(torch.from_numpy(p[k]).reshape(-1))

    def views(flat):
        return {k: flat[int(o):int(o) + n].view(p[k].shape) for k, o, n in zip(keys, offs, sizes)}

    dev_in = views(host_in.to(dev))
    x, off, mask, gy = (dev_in[k] for k in keys)
    w = torch.from_numpy(make_inputs(1002, wl)["weight"]).to(dev)      # weights replicated across ranks
    bias = torch.zeros(wl["Cout"], device=dev)
    for t in (x, off, mask, w, bias):
        t.requires_grad_(True)
    V = wl["dims"][0] * wl["dims"][1] * wl["dims"][2]
    F = fwd_flops(wl["B"], wl["Cin"], wl["Cout"], V, 27)
    s = 4
    coord_bytes = s * (wl["B"] * wl["Cin"] * 27 * V + wl["B"] * wl["Cin"] * V + 2 * wl["B"] * wl["G"] * 4 * 27 * V)
    col2im_bytes = s * (wl["B"] * wl["Cin"] * 27 * V + wl["B"] * wl["G"] * 4 * 27 * V + wl["B"] * wl["Cin"] * V)
    # fused offset/mask-gradient + scatter: dcol read once, x read, offsets+mask read, their gradients and grad_x written
    sample_grad_bytes = s * (wl["B"] * wl["Cin"] * 27 * V + 2 * wl["B"] * wl["Cin"] * V + 2 * wl["B"] * wl["G"] * 4 * 27 * V)
    work = {"F": F, "coord_bytes": coord_bytes, "col2im_bytes": col2im_bytes, "sample_grad_bytes": sample_grad_bytes}

    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)      # 256 MB > 126 MB L2
    s_main = torch.cuda.current_stream()
    s_coll = torch.cuda.Stream() if world > 1 else None

    def reduce_param_grads(wt, bt):
        """All-reduce of grad_weight + grad_bias as one bucket.  This library: issued from a side stream that
        waits only for the event the backward records when the parameter gradients are final (they are computed
        first), so the collective runs under the data-side backward; the compute stream joins at the end of the
        step.  Reference op: no such event, the collective follows the backward (what DDP does for a
        single-bucket model)."""
        if world == 1:
            return
        ev = dconv_native._ops.params_ready_event() if ours else None
        finish = sharding.all_reduce_param_grads_overlapped([wt.grad, bt.grad], ev, s_coll)
        finish()

    def step():
        for t in (x, off, mask, w, bias):
            t.grad = None
        y = op(x, off, mask, w, bias)
        y.backward(gy)
        reduce_param_grads(w, bias)
        return y

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- N > 1: the all-reduced parameter gradients against the single-GPU full-batch gradient -------------
    allreduce_check = None
    if world > 1:
        step()
        torch.cuda.synchronize()
        got_w, got_b = w.grad.clone(), bias.grad.clone()
        if rank == 0:
            want_w, want_b = torch.zeros_like(w), torch.zeros_like(bias)
            for r in range(world):                       # every rank's clips, one rank after the other, on this GPU
                q = p if r == 0 else make_inputs(1002 + r, wl)
                ts = [torch.from_numpy(q[k]).to(dev).requires_grad_(k != "gy") for k in keys]
                wr, br = w.detach().clone().requires_grad_(), bias.detach().clone().requires_grad_()
                op(ts[0], ts[1], ts[2], wr, br).backward(ts[3])
                want_w += wr.grad; want_b += br.grad
                del ts, q
            torch.cuda.synchronize()
            ew = float((got_w - want_w).abs().max() / want_w.abs().max())
            eb = float((got_b - want_b).abs().max() / want_b.abs().max())
            bound = 1e-4 if (not ours or args.mode != "bf16") else 2e-2
            allreduce_check = {"status": "ok" if max(ew, eb) <= bound else "MISMATCH", "grad_weight_rel_err": ew,
                               "grad_bias_rel_err": eb, "bound": bound,
                               "what": f"all-reduced gradients of {world} ranks vs the sum over the same {world * wl['B']} "
                                       "clips evaluated on one GPU"}
            del want_w, want_b
        dist.barrier()

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        flush.zero_()
        step()
    barrier()
    if rank == 0:
        sampler.wait_for_samples()

    def timed_steps(n, with_phases):
        if with_phases:
            _lib.profile_read()
            _lib.profile_enable(True)
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
        barrier()
        t0 = time.time()
        for i in range(n):
            flush.zero_()                      # L2 flush between timed iterations, outside the event pair
            ev[i][0].record()
            step()
            ev[i][1].record()
        barrier()
        t1 = time.time()
        phases = None
        if with_phases:
            _lib.profile_enable(False)
            phases = _lib.profile_read()
        tt = torch.tensor([sum(a.elapsed_time(b) for a, b in ev)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item()) / n, phases, t0, t1

    launches0 = _lib.launch_count()
    ms_per_step, phases, t_start, t_end = timed_steps(args.steps, ours)
    launches = _lib.launch_count() - launches0
    clocks = None
    if rank == 0:
        sampler.stop()
        clocks = sampler.summary(t_start, t_end)
    if ours:
        _lib.device_status()               # raises if a bounded device-side wait gave up
    value = 3 * F * world / (ms_per_step * 1e-3) / 1e12

    # ---- end-to-end with host buffers: pinned H2D of the step's inputs, D2H of its results ----
    # Every step copies its own inputs up (ONE copy: the packed input buffer) and its own results down (into ONE
    # packed pinned buffer; the five results are separate device tensors, so five slice copies).  The copies of
    # neighbouring steps run on two copy streams (the link is full duplex) behind the compute stream, with
    # double-buffered device inputs and pinned host outputs, as a training loop with a prefetching loader would.
    # grad_weight is identical on every rank after the all-reduce: only rank 0 reads it back.
    out_keys = ("y", "gx", "goff", "gmask") + (("gw",) if rank == 0 else ())
    out_like = {"y": gy, "gx": x, "goff": off, "gmask": mask, "gw": w}
    out_sizes = [out_like[k].numel() for k in out_keys]
    out_offs = np.concatenate([[0], np.cumsum([(n + 63) // 64 * 64 for n in out_sizes])])
    host_out = [torch.empty(int(out_offs[-1]), dtype=torch.float32).pin_memory() for _ in range(2)]
    ins = [torch.empty_like(host_in, device=dev) for _ in range(2)]
    h2d = host_in.numel() * 4
    d2h = sum(out_sizes) * 4
    s_up, s_down = torch.cuda.Stream(), torch.cuda.Stream()

    def e2e_run(n, compute=True):
        up_done = [torch.cuda.Event() for _ in range(2)]
        comp_done = [torch.cuda.Event() for _ in range(2)]
        down_done = [torch.cuda.Event() for _ in range(2)]
        stand_in = None
        if not compute:      # copy-only run: the same bytes move, no kernel of the layer runs
            stand_in = {"y": gy, "gx": x.detach(), "goff": off.detach(), "gmask": mask.detach(), "gw": w.detach()}

        def upload(i):
            cur = i & 1
            with torch.cuda.stream(s_up):
                if i >= 2:
                    s_up.wait_event(comp_done[cur])          # step i-2 no longer reads this input buffer
                ins[cur].copy_(host_in, non_blocking=True)
                up_done[cur].record(s_up)

        upload(0)
        for i in range(n):
            cur = i & 1
            if i + 1 < n:
                upload(i + 1)
            s_main.wait_event(up_done[cur])
            if compute:
                v = views(ins[cur])
                xs, os_, ms_ = (v[k].detach().requires_grad_(True) for k in ("x", "geo", "mask"))
                w.grad = None
                bias.grad = None
                y = op(xs, os_, ms_, w, bias)
                y.backward(v["gy"])
                reduce_param_grads(w, bias)
                res = {"y": y.detach(), "gx": xs.grad, "goff": os_.grad, "gmask": ms_.grad, "gw": w.grad}
            else:
                res = stand_in
            comp_done[cur].record(s_main)
            with torch.cuda.stream(s_down):
                s_down.wait_event(comp_done[cur])
                if i >= 2:
                    s_down.wait_event(down_done[cur])        # host buffer of step i-2 is free again
                for k, o, nn_ in zip(out_keys, out_offs, out_sizes):
                    host_out[cur][int(o):int(o) + nn_].copy_(res[k].reshape(-1), non_blocking=True)
                    res[k].record_stream(s_down)
                down_done[cur].record(s_down)
        s_main.wait_stream(s_down)
        s_main.wait_stream(s_up)

    def e2e_time(n, compute):
        e2e_run(2, compute)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        e2e_run(n, compute)
        e1.record()
        barrier()
        te = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        return float(te.item()) / n

    e2e = None
    if not args.no_e2e:
        # as many steps as the device-timed run (at most 50): the first upload and the last download are not hidden by
        # anything, so a short run overstates the per-step cost (10 steps: +0.8 ms per step)
        e2e_steps = max(2, min(args.steps, 50))
        e2e_ms = e2e_time(e2e_steps, True)
        copy_ms = e2e_time(e2e_steps, False)
        e2e = {"value": 3 * F * world / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "h2d_bytes_per_step": h2d,
               "d2h_bytes_per_step": d2h, "ms_per_step": e2e_ms, "steps": e2e_steps,
               "copy_only_ms": copy_ms,
               "copy_only_note": "the same uploads and downloads per step with no kernel of the layer in between: "
                                 "what the host link sustains with all ranks copying at once",
               "host_buffers": f"one packed pinned buffer per direction, allocated after binding to {affinity}",
               "overlap": "copies of neighbouring steps on two copy streams behind the compute stream"}

    # ---- the single-pass bf16 mode (looser stated parity bound) on the same inputs, as a second figure ----
    bf16_mode = None
    main_mode = _lib.get_math_mode()
    if ours and main_mode != "bf16" and not args.no_bf16_mode:
        d2conv3d_b200.set_math_mode("bf16")
        n2 = max(1, min(args.steps, 20))
        for _ in range(3):
            flush.zero_()
            step()
        ms2, ph2, _, _ = timed_steps(n2, True)
        agg2 = {}
        for name, ms in ph2:
            agg2[name] = agg2.get(name, 0.0) + ms / n2
        bf16_mode = {"ms_per_step": ms2, "value": 3 * F * world / (ms2 * 1e-3) / 1e12, "unit": UNIT, "steps": n2,
                     "parity": "output <= 1e-2, gradients <= 2e-2 of scale (stated bound of this mode)",
                     "phases": {k: {"ms_avg": round(v, 4),
                                    **({"frac_of_peak": round(F / (v * 1e-3) / 1e12 / peaks["tensor_sustained"], 4)}
                                       if PHASE_WORK.get(k, ("", ""))[0] == "tensor" else
                                       {"frac_of_peak": round(work[PHASE_WORK[k][1]] / (v * 1e-3) / 1e9 / peaks["hbm_gbs"], 4)}
                                       if k in PHASE_WORK else {})}
                                for k, v in agg2.items()}}
        d2conv3d_b200.set_math_mode(main_mode)
        _lib.device_status()

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "data": "synthetic", "tensor_dtype": "f32",
        "config": {"workload": wl["name"], "l2": "256 MB buffer written between timed iterations",
                   "collective": ("all-reduce of grad_weight+grad_bias as one bucket (NCCL)" +
                                  (", issued when the weight gradient is done, under the data-side backward" if ours else
                                   ", after the backward")) if world > 1 else "none"},
        "clips_per_s": wl["B"] * world / (ms_per_step * 1e-3),
        "e2e": e2e, "clocks": clocks,
    }
    if allreduce_check is not None:
        line["allreduce_check"] = allreduce_check["status"]
        line["allreduce_check_detail"] = allreduce_check
    if ours:
        # ---- roofline of the dominant kernel phase (library events over the timed steps) ----
        agg = {}
        for name, ms in phases:
            a = agg.setdefault(name, [0, 0.0])
            a[0] += 1; a[1] += ms

        def phase_roofline(name, avg_ms, launches_per_step=1.0):
            # avg_ms: the phase's time per STEP (a phase may be more than one launch: the fp32-parity mode runs
            # the gradient-column contraction as two accumulating launches); work[key] is per step as well
            if name not in PHASE_WORK:
                return None
            bound, key = PHASE_WORK[name]
            if bound == "tensor":
                achieved, peak, unit = work[key] / (avg_ms * 1e-3) / 1e12, peaks["tensor_sustained"], "TFLOP/s"
            else:
                achieved, peak, unit = work[key] / (avg_ms * 1e-3) / 1e9, peaks["hbm_gbs"], "GB/s"
            r = {"kernel": name, "bound": bound, "achieved": achieved, "peak": peak, "unit": unit,
                 "frac": achieved / peak, "traffic": TRAFFIC_PER_LAUNCH.get((name, _lib.get_math_mode())),
                 "traffic_source": TRAFFIC_SOURCE,
                 "ms_per_launch": avg_ms / launches_per_step, "launches_per_step": launches_per_step,
                 "peak_source": peaks["source"] + (" (bf16 dense, sustained)" if bound == "tensor" else " (copy)")}
            if name == "bwd_sample_grad":
                # what actually bounds this kernel: fp32 vector reductions into the L2-resident grad_input
                # accumulator; the payload and the sustained rate of such reductions are measured, see SCATTER
                r["second_bound"] = {"what": "fp32 red.global.add.v4 payload into L2", "payload_bytes": SCATTER["payload_bytes"],
                                     "measured_rate_gbs": SCATTER["rate_gbs"],
                                     "floor_ms": SCATTER["payload_bytes"] / SCATTER["rate_gbs"] / 1e6,
                                     "frac": SCATTER["payload_bytes"] / SCATTER["rate_gbs"] / 1e6 / (avg_ms / launches_per_step),
                                     "source": SCATTER["source"]}
            return r

        phase_summary = {}
        for n, (c, t) in agg.items():
            phase_summary[n] = {"launches": c, "ms_total": round(t, 4), "ms_avg": round(t / args.steps, 4)}
            r = phase_roofline(n, t / args.steps, c / args.steps)
            if r:
                phase_summary[n]["frac_of_peak"] = round(r["frac"], 4)
        roofline = None
        candidates = [n for n in agg if n in PHASE_WORK]
        if candidates:
            dom = max(candidates, key=lambda n: agg[n][1])
            roofline = phase_roofline(dom, agg[dom][1] / args.steps, agg[dom][0] / args.steps)
        mode = _lib.get_math_mode()
        line.update({
            "dtype": {"bf16": "bf16", "fp32": "f32"}.get(mode, "bf16x3"), "math_mode": mode,
            "parity": ("1e-4 of scale vs the fp32 reference (bf16 hi/lo split of both operands, fp32 accumulate)"
                       if mode in ("auto", "bf16x3") else
                       "1e-4 of scale (FMA pipe)" if mode == "fp32" else
                       "output <= 1e-2, gradients <= 2e-2 of scale (stated bound of this mode)"),
            "gpu_launches": int(launches), "roofline": roofline, "phases": phase_summary, "bf16_mode": bf16_mode,
        })
        if world == 1 and not args.no_cpu_baseline:
            val, ms, sample, cores = cpu_arm(1, 1, budget_s=40.0)
            line["cpu_baseline"] = {"value": val, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample,
                                    "ms_per_sample_step": ms}
        else:
            line["cpu_baseline"] = None
        if world == 1 and not args.no_reference_gpu:
            host = {k: torch.from_numpy(p[k]) for k in keys}
            line["reference_cuda_op"] = time_reference_cuda_op(host, w, bias, wl, F)
        if world == 1 and args.secondary:
            del x, off, mask, gy, dev_in, ins, host_out
            torch.cuda.empty_cache()
            line["secondary"] = secondary_summary(args)
    else:
        # the reference arm: its kernels are not this library's, so no launch count of ours
        val, ms, sample, cores = cpu_arm(1, 1, budget_s=40.0) if not args.no_cpu_baseline else (None, None, None, None)
        line.update({
            "impl": "reference", "dtype": "f32", "gpu_launches": 0,
            "what": "unmodified reference dconv_native (im2col + cuBLAS fp32, allow_tf32=False) from baseline/_ref, "
                    f"{world} rank(s) x {wl['B']} clips, same inputs / flush / events as the other arm",
            "peak_mem_gb": torch.cuda.max_memory_allocated() / 1e9,
            "cpu_baseline": None if val is None else {"value": val, "unit": UNIT, "cores": cores, "kind": "port",
                                                      "sample": sample, "ms_per_sample_step": ms,
                                                      "note": "the reference has no CPU implementation of this op; this is "
                                                              "the CPU restatement of its algorithm (oracle/), for context"},
        })
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def secondary_summary(args):
    """Forward / backward milliseconds and fraction of the measured peak of the secondary configurations, in the
    headline line's math mode and in bf16 mode, so that one record carries them (each as `--workload NAME` would
    print it, fewer steps)."""
    import d2conv3d_b200
    out = {}
    for name in ("c3-xyz", "c4-depthwise", "c4-md", "c5-e1-train"):
        modes = [args.mode] if name == "c4-depthwise" or args.mode == "bf16" else [args.mode, "bf16"]
        try:
            for mode, r in measure_extra_workload(name, modes, steps=5, warmup=3).items():
                out[f"{name}/{mode}"] = {"fwd_ms": round(r["fwd_ms"], 4), "bwd_ms": round(r["bwd_ms"], 4),
                                         "fwd_frac": round(r["fwd"]["frac_of_measured_peak"], 4),
                                         "bwd_frac": round(r["bwd"]["frac_of_measured_peak"], 4), "unit": r["fwd"]["unit"]}
        except Exception as exc:
            out[name] = {"error": f"{type(exc).__name__}: {exc}"}
    d2conv3d_b200.set_math_mode(args.mode)
    return out


EXTRA_WORKLOADS = {
    # benchmark configuration 1: the plumbing / correctness layer (launch-latency bound at this size)
    "c1": dict(kind="deform", B=1, Cin=64, Cout=64, dims=(4, 16, 16), G=1, offset_std=1.0),
    # benchmark configuration 3: dynamic-dilation conv3d, one field shared by all taps, optional 27-channel mask
    "c3-xyz": dict(kind="dyndil", mode="xyz", B=4, Cin=256, Cout=256, dims=(8, 60, 108), G=1),
    "c3-xy": dict(kind="dyndil", mode="xy", B=4, Cin=256, Cout=256, dims=(8, 60, 108), G=1),
    "c3-x": dict(kind="dyndil", mode="x", B=4, Cin=256, Cout=256, dims=(8, 60, 108), G=1),
    # benchmark configuration 4: depthwise 3x3x3 of an ir-CSN bottleneck, then the modulated deformable 1024->256 stage
    "c4-depthwise": dict(kind="depthwise", B=8, C=1024, dims=(8, 30, 54)),
    "c4-md": dict(kind="deform", B=8, Cin=1024, Cout=256, dims=(8, 30, 54), G=8),
    # benchmark configuration 5 (decoder inference): the xyz dynamic-dilated 256->256 conv of a refine block at the
    # stride-4 pyramid level, one clip, 8 offset groups (32 channels per group), forward only
    "c5-e1": dict(kind="dyndil", mode="xyz", B=1, Cin=256, Cout=256, dims=(8, 120, 214), G=8, fwd_only=True),
    # the same layer with its backward (decoder training)
    "c5-e1-train": dict(kind="dyndil", mode="xyz", B=1, Cin=256, Cout=256, dims=(8, 120, 214), G=8),
}


def run_decoder_workload(args):
    """Benchmark configuration 5: decoder inference on synthetic ir-CSN features, clips sharded over the ranks with no
    collective (one process per GPU under torchrun; one rank otherwise).  Every rank pushes its share of the 32
    clips through the decoder one clip at a time (forward only, no_grad); rank 0 prints clips/s of the whole job
    from the slowest rank's CUDA-event time."""
    import torch
    import torch.distributed as dist

    import d2conv3d_b200
    from d2conv3d_b200 import _lib, decoder

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    _lib.lib()
    d2conv3d_b200.set_math_mode(args.mode)
    torch.manual_seed(1005)
    net = decoder.Decoder().to(dev).eval()
    for m in net.modules():                          # non-trivial deformation: random predictor weights
        if hasattr(m, "deform_params"):
            torch.nn.init.normal_(m.deform_params.weight, std=0.02)
    total_clips = args.clips
    mine = decoder_share(total_clips, rank, world)
    g = torch.Generator().manual_seed(1005 + rank)
    feats = [torch.relu(torch.randn(s, generator=g)).to(dev) for s in decoder.pyramid_shapes(1)]

    def one_clip():
        with torch.no_grad():
            return net(*feats)

    for _ in range(2):
        one_clip()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    launches0 = _lib.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(mine):
        out = one_clip()
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    _lib.device_status()
    if rank == 0:
        print(json.dumps({
            "workload": "c5-decoder", "metric": "decoder_inference_clips_per_s", "value": total_clips / (float(ms.item()) * 1e-3),
            "unit": "clips/s", "n_gpus": world, "clips": total_clips, "clips_per_rank": mine,
            "ms_per_clip": float(ms.item()) / mine, "math_mode": _lib.get_math_mode(), "scaling": "strong",
            "deformable_layers": net.converted, "gpu_launches_per_clip": (_lib.launch_count() - launches0) // max(1, mine),
            "output_shape": list(out.shape), "data": "synthetic ReLU(N(0,1)) features, random-init decoder",
            "config": {"features": [list(s) for s in decoder.pyramid_shapes(total_clips)],
                       "decoder": "GC bridge + 3 refine blocks, xyz dilation-field + mask conv3d 3x3x3, Cout 256, 8 offset groups",
                       "collective": "none"}}), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_block_workload(args):
    """ir-CSN stage-4 bottleneck block (1024 -> 256 -> depthwise 3x3x3 -> 1024) at 8x30x54, B = 8, forward +
    backward in training mode: the depthwise kernels measured where the reference uses them; the 1x1x1
    convolutions and batch norms are cuDNN / PyTorch."""
    import torch

    from d2conv3d_b200 import _lib
    from d2conv3d_b200.backbone import IrBottleneck3d

    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    _lib.lib()
    torch.manual_seed(1004)
    blk = IrBottleneck3d(1024, 256).to(dev).train()
    x = torch.randn(8, 1024, 8, 30, 54, device=dev, requires_grad=True)
    gy = torch.randn(8, 1024, 8, 30, 54, device=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def one():
        x.grad = None
        blk.zero_grad(set_to_none=True)
        flush.zero_()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record(); y = blk(x); e[1].record(); y.backward(gy); e[2].record()
        torch.cuda.synchronize()
        return e[0].elapsed_time(e[1]), e[1].elapsed_time(e[2])

    for _ in range(max(3, args.warmup)):
        one()
    _lib.profile_read(); _lib.profile_enable(True)
    runs = [one() for _ in range(args.steps)]
    _lib.profile_enable(False)
    ph = {}
    for k, v in _lib.profile_read():
        ph[k] = ph.get(k, 0.0) + v / args.steps
    f_ms = statistics.median(r[0] for r in runs)
    b_ms = statistics.median(r[1] for r in runs)
    print(json.dumps({
        "workload": "c4-block", "config": "ir-CSN bottleneck 1024->256->1024, depthwise 3x3x3 on 256 channels, B=8, 8x30x54, train mode",
        "steps": args.steps, "fwd_ms": f_ms, "bwd_ms": b_ms, "clips_per_s_fwd_bwd": 8 / ((f_ms + b_ms) * 1e-3),
        "depthwise_ms_per_step": {k: round(v, 4) for k, v in ph.items()},
        "depthwise_share": sum(ph.values()) / (f_ms + b_ms)}), flush=True)


def decoder_share(total, rank, world):
    """Clips of rank `rank`: contiguous shares, the first `total % world` ranks take one more."""
    return total // world + (1 if rank < total % world else 0)


def measure_extra_workload(name, modes, steps, warmup):
    """Secondary configurations: forward / backward milliseconds from CUDA events (median over `steps`), contraction
    TFLOP/s or GB/s against the measured peaks, for each math mode of `modes` on the same tensors.  Returns
    {mode: the dict that `--workload NAME --mode MODE` prints}."""
    import torch

    import d2conv3d_b200
    from d2conv3d_b200 import _lib, dconv_native, fast_depthwise_conv3d
    from tests._util import make_problem

    wl = EXTRA_WORKLOADS[name]
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    _lib.lib()
    peaks = measured_peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    V = wl["dims"][0] * wl["dims"][1] * wl["dims"][2]

    if wl["kind"] == "depthwise":
        g = torch.Generator().manual_seed(1004)
        x = torch.randn((wl["B"], wl["C"]) + wl["dims"], generator=g).to(dev).requires_grad_()
        w = (torch.randn((wl["C"], 1, 3, 3, 3), generator=g) * 0.1).to(dev).requires_grad_()
        gy = torch.randn((wl["B"], wl["C"]) + wl["dims"], generator=g).to(dev)
        fwd = lambda: fast_depthwise_conv3d._ops.depthwise_separable_conv3d(x, w, None, 1, 1, 1)
        params = [x, w]
        work_f = 2 * 4 * wl["B"] * wl["C"] * V      # bytes: read x, write y
        work_b = 3 * 4 * wl["B"] * wl["C"] * V      # read grad_out + x, write grad_x
        unit, peak = "GB/s", peaks["hbm_gbs"]
    else:
        p = make_problem(1003, wl["B"], wl["Cin"], wl["Cout"], wl["dims"], k=3, padding=1, G=wl["G"],
                         dtype=np.float32, offset_std=wl.get("offset_std", 2.0), field_mode=wl.get("mode"))
        ts = [torch.from_numpy(p[k]).to(dev).requires_grad_() for k in ("x", "geo", "mask", "weight", "bias")]
        gy = torch.from_numpy(p["gy"]).to(dev)
        del p
        if wl["kind"] == "dyndil":
            fwd = lambda: dconv_native.dyn_dilated_conv3d(*ts, wl["mode"], 1, 1, 1, 1, wl["G"])
        else:
            fwd = lambda: dconv_native.deform_conv3d(*ts, 1, 1, 1, 1, wl["G"])
        params = ts
        work_f = fwd_flops(wl["B"], wl["Cin"], wl["Cout"], V, 27)
        work_b = 2 * work_f
        unit, peak = "TFLOP/s", peaks["tensor_sustained"]

    def one():
        for t in params:
            t.grad = None
        flush.zero_()
        e = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
        e[0].record()
        if wl.get("fwd_only"):
            with torch.no_grad():      # an inference layer: nothing is kept for a backward
                y = fwd()
        else:
            y = fwd()
        e[1].record()
        if not wl.get("fwd_only"):
            y.backward(gy)
        e[2].record()
        torch.cuda.synchronize()
        return e[0].elapsed_time(e[1]), max(e[1].elapsed_time(e[2]), 1e-9)

    out = {}
    scale = 1e9 if unit == "GB/s" else 1e12
    for mode in modes:
        d2conv3d_b200.set_math_mode(mode)
        for _ in range(max(3, warmup)):
            one()
        runs = [one() for _ in range(steps)]
        f_ms = statistics.median(r[0] for r in runs)
        b_ms = statistics.median(r[1] for r in runs)
        _lib.device_status()
        out[mode] = {
            "workload": name, "config": wl, "math_mode": _lib.get_math_mode(), "steps": steps,
            "fwd_ms": f_ms, "bwd_ms": b_ms, "clips_per_s_fwd_bwd": wl["B"] / ((f_ms + b_ms) * 1e-3),
            "fwd": {"achieved": work_f / (f_ms * 1e-3) / scale, "unit": unit, "frac_of_measured_peak": work_f / (f_ms * 1e-3) / scale / peak},
            "bwd": {"achieved": work_b / (b_ms * 1e-3) / scale, "unit": unit, "frac_of_measured_peak": work_b / (b_ms * 1e-3) / scale / peak},
            "note": "times include operand staging and (backward) all gradients; L2 flushed between iterations",
        }
    return out


def run_extra_workload(args):
    print(json.dumps(measure_extra_workload(args.workload, [args.mode], args.steps, args.warmup)[args.mode]), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--mode", default="auto", choices=["auto", "fp32", "bf16x3", "bf16"],
                    help="math mode of the timed steps; auto = fp32-parity tensor-core mode (bf16x3) where it applies")
    ap.add_argument("--no-bf16-mode", action="store_true", help="skip the second figure in the single-pass bf16 mode")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-reference-gpu", action="store_true")
    ap.add_argument("--no-keep-samples", action="store_true",
                    help="the forward keeps nothing for the backward (d2conv3d_b200.set_keep_samples(False)): the weight "
                         "gradient gathers and blends its samples again, as the reference does")
    ap.add_argument("--no-secondary", dest="secondary", action="store_false",
                    help="skip the `secondary` key (c3-xyz, c4-depthwise, c4-md, c5-e1-train, a few steps each)")
    ap.add_argument("--clips", type=int, default=32, help="c5-decoder: clips of the whole job")
    ap.add_argument("--workload", default="c2", choices=["c2", "c4-block", "c5-decoder"] + sorted(EXTRA_WORKLOADS),
                    help="c2 = the headline line (default); the others print a secondary line for one GPU")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.no_keep_samples:
        import d2conv3d_b200
        d2conv3d_b200.set_keep_samples(False)
    if args.impl == "reference":
        run_reference_arm(args)
    elif args.workload == "c5-decoder":
        run_decoder_workload(args)
    elif args.workload == "c4-block":
        run_block_workload(args)
    elif args.workload != "c2":
        run_extra_workload(args)
    else:
        run_gpu_arm(args)


if __name__ == "__main__":
    main()
