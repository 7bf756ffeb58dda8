#!/usr/bin/env python
"""Benchmark of the Fastmax hot path:  python bench.py --gpus N --steps K --warmup W [--impl reference]

Workload (BASELINE config 2, the configuration the headline metric is quoted on): Fastmax order 2, causal,
B=8, H=16, N=4096, D=Dv=64, bf16 inputs with fp32 accumulation, q,k,v ~ N(0,1), temperature 8*sqrt(D);
one step = forward + backward over the whole batch.  Inputs are seeded synthetic tensors (the reference's
datasets are not available offline).

Multi-GPU: every (batch, head) is independent, so each rank processes its own B=8 batch with no data-path
collective (weak scaling); the job's throughput is all ranks' tokens over the slowest rank's time.

The printed JSON line carries: value (device-resident inputs, CUDA events), e2e (through the public operator
with pinned HOST buffers, copies inside the timed region), roofline of the dominant kernel, per-kernel times,
the CPU baseline (the oracle's restatement of the reference's factorised algorithm on the host cores) and the
SM clocks sampled during the timed region.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B, H, N, D, order, causal, dtype, input scale)
    "cfg2_bf16_causal_p2_B8_H16_N4096_D64": (8, 16, 4096, 64, 2, True, "bf16", 1.0),
    # profiling case: same per-CTA work as config 2, a few GB on the device, inputs (134 MB) larger than L2
    "prof_bf16_causal_p2_B4_H16_N4096_D64": (4, 16, 4096, 64, 2, True, "bf16", 1.0),
    # the config-2 shape without a mask: the moment build over all keys, then the apply over all queries (and the
    # matching backward), on the same tensor-memory scans
    "nc_bf16_noncausal_p2_B8_H16_N4096_D64": (8, 16, 4096, 64, 2, False, "bf16", 1.0),
    "ncprof_bf16_noncausal_p2_B4_H16_N4096_D64": (4, 16, 4096, 64, 2, False, "bf16", 1.0),
    # one long causal sequence with few heads in bf16 / D=64 (config 3's shape at the tensor-memory engine's dtype and
    # head dim): the library cuts it into segments so that the scans still cover the GPU
    "long_bf16_causal_p2_B1_H8_N131072_D64": (1, 8, 131072, 64, 2, True, "bf16", 1.0),
    # BASELINE config 3: one long causal sequence, cut into contiguous pieces across the ranks (strong scaling)
    "cfg3_f32_causal_p2_B1_H8_N131072_D32": (1, 8, 131072, 32, 2, True, "f32", 1.0),
    # BASELINE config 4: order 1, non-causal, wide batch, forward (run with --mode fwd): HBM-bound
    "cfg4_bf16_noncausal_p1_B64_H12_N1024_D64": (64, 12, 1024, 64, 1, False, "bf16", 0.5),
    # config 2's shape with narrower heads (bf16): zero-padded to 64 on the tensor-memory kernels
    "d32_bf16_causal_p2_B8_H16_N4096_D32": (8, 16, 4096, 32, 2, True, "bf16", 1.0),
    # incremental decoding: one new token per (batch, head) per step against the carried state (N = prefix length is
    # irrelevant to the cost; 512 head states = 330 MB, larger than L2)
    "decode_bf16_p2_B32_H16_D64": (32, 16, 1, 64, 2, True, "bf16", 1.0),
    # the q / k normalisation stage alone (forward of one tensor and its backward), config-2 sized: HBM-bound
    "norm_bf16_B8_H16_N4096_D64": (8, 16, 4096, 64, 2, True, "bf16", 1.0),
}
SEQUENCE_SHARDED = {"cfg3_f32_causal_p2_B1_H8_N131072_D32"}
NORMALIZE = {"norm_bf16_B8_H16_N4096_D64"}
DECODE = {"decode_bf16_p2_B32_H16_D64"}
DEFAULT = "cfg2_bf16_causal_p2_B8_H16_N4096_D64"
def dram_traffic():
    """dram__bytes_read.sum + dram__bytes_write.sum per launch of the scan kernels, from the machine-readable record
    written with the ncu capture (profiles/dram_traffic.json: kernel -> bytes per launch, the head-tokens of the
    captured workload and the summary file that documents the capture).  bench.py scales by head-tokens."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        with open(path) as f:
            return json.load(f)["kernels"]
    except (OSError, KeyError, ValueError):
        return {}


DRAM_TRAFFIC = dram_traffic()
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


# The contract is ONE JSON line on stdout.  Native libraries write there too (NCCL prints its version banner on file
# descriptor 1 when the process group comes up), so descriptor 1 is pointed at stderr for the whole run and the
# result line goes to a private copy of the original stdout.
_RESULT_FD = None


def claim_stdout():
    global _RESULT_FD
    if _RESULT_FD is None:
        sys.stdout.flush()
        _RESULT_FD = os.dup(1)
        os.dup2(2, 1)


def emit(line):
    if _RESULT_FD is None:
        print(json.dumps(line), flush=True)
    else:
        os.write(_RESULT_FD, (json.dumps(line) + "\n").encode())


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        p["_source"] = "measured"
        return p
    p = dict(FALLBACK_PEAKS)
    p["_source"] = "fallback"
    return p


def algorithmic_flops(B, H, N, D, order):
    """U = 2 B H N M (Dv+1), M = 1 + D + D^2 (order 2) or 1 + D: one GEMM pass over all tokens with the full
    D^2 feature map.  forward = 2U (moment build + apply), backward = 4U (dq, dS, dk, dv)."""
    M = 1 + D + (D * D if order == 2 else 0)
    return 2.0 * B * H * N * M * (D + 1)


def executed_units(D, order):
    """Feature rows the kernels actually contract over (8x8 block-symmetric packing of x (x) x)."""
    nb = D // 8
    return (64 * nb * (nb + 1) // 2 if order == 2 else 0) + D + 1


class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU while the timed region runs (NVML every 5 ms in a thread;
    `nvidia-smi -lms` when the NVML binding is missing).  Reading the settings changes nothing on the GPU."""

    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index):
        self.index = index
        self.samples = []
        self.reasons = set()
        self.max_mhz = None
        self.stop_flag = threading.Event()
        self.thread = None
        self.proc = None

    def _nvml_loop(self, nv, handle):
        while not self.stop_flag.is_set():
            try:
                self.samples.append(float(nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(handle)) if hasattr(nv, "nvmlDeviceGetCurrentClocksEventReasons") \
                    else int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(handle))
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(0.005)

    def start(self):
        try:
            import pynvml as nv

            nv.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(vis.split(",")[self.index]) if vis and vis.split(",")[self.index].isdigit() else self.index
            handle = nv.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._nvml_loop, args=(nv, handle), daemon=True)
            self.thread.start()
            return
        except Exception:
            self.thread = None
        try:
            q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
                 "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + q,
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._smi_loop, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _smi_loop(self):
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                self.samples.append(float(parts[0]))
                self.max_mhz = float(parts[1])
            except ValueError:
                continue
            for nm, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    self.reasons.add(nm)

    def stop(self):
        self.stop_flag.set()
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
        if self.thread is not None:
            self.thread.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "samples": 0, "reasons": ["no clock samples"]}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz, "samples": len(self.samples),
                "reasons": sorted(self.reasons)}


# ----------------------------------------------------------------------------------------------------
# CPU arm: the oracle's restatement of the reference's factorised algorithm, on the host cores
# ----------------------------------------------------------------------------------------------------
def cpu_sample(workload, n_sample=512, heads=1):
    """Times forward+backward of the factorised CPU algorithm (cumsum of per-token moments, the
    reference's attention_mechanisms implementation) on `heads` heads of n_sample tokens, one head after the
    other, with the workload's D, order and mask.  Memory of that algorithm is O(N D^3) per head, which bounds
    the tokens of a head; the number of heads sets how long the sample runs.
    Returns (seconds, head-tokens processed, threads)."""
    import torch

    from oracle import fastmax_oracle as orc

    B, H, N, D, order, causal, dtype, scale = WORKLOADS[workload]
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    poly = orc.Poly(1.0, 1.0, 0.5, 1.0 / (8.0 * math.sqrt(D)), order)
    total = 0.0
    for _ in range(heads):
        q, k, v, do = (torch.randn(1, 1, n_sample, D, generator=g) * scale for _ in range(4))
        if dtype == "bf16":
            q, k, v, do = (t.bfloat16().float() for t in (q, k, v, do))
        t0 = time.perf_counter()
        orc.fastmax_factorized_fwd_bwd(q, k, v, do, causal, poly)
        total += time.perf_counter() - t0
    return total, heads * n_sample, threads


def cpu_sample_text(workload, n_sample, heads):
    B, H, N, D, order, causal, dtype, scale = WORKLOADS[workload]
    return (f"factorised {'causal' if causal else 'non-causal'} order-{order} forward+backward (torch CPU, autograd) on "
            f"{heads} of {B * H} heads, {n_sample} of {N} tokens each, D={D}; head-tokens / H = metric tokens")


REFERENCE_EINOPS = os.path.join(ROOT, "oracle", "_ref", "fastattention_einops.py")


def reference_einops():
    """The reference's own CPU implementation (attention_mechanisms/fastattention_einops.py, placed unmodified under
    oracle/_ref/ by baseline/vendor_reference.py), or None when it has not been placed."""
    if not os.path.exists(REFERENCE_EINOPS):
        return None
    import importlib.util

    name = "fastmax_reference_einops"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, REFERENCE_EINOPS)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def cpu_sample_reference(workload, n_sample=512, heads=1):
    """Forward + backward of the reference's einops Fastmax (its factorised forward and hand-derived factorised
    backward, fastattention_einops.py:42-182) on `heads` heads of n_sample tokens, one after the other.
    Returns (seconds, head-tokens, threads)."""
    import torch

    ein = reference_einops()
    B, H, N, D, order, causal, dtype, scale = WORKLOADS[workload]
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    total = 0.0
    for _ in range(heads):
        q, k, v, do = (torch.randn(1, 1, n_sample, D, generator=g) * scale for _ in range(4))
        if dtype == "bf16":
            q, k, v, do = (t.bfloat16().float() for t in (q, k, v, do))
        q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
        t0 = time.perf_counter()
        o = ein.fastmax(q, k, v, mask=causal, normalize_term=8, tensors_normalized=False, p=order)
        o.backward(do)
        total += time.perf_counter() - t0
    return total, heads * n_sample, threads


def config1_record(torch, dev):
    """BASELINE config 1 exactly (order 2, no mask, float32, B2 H4 N256 D32, q, k, v ~ N(0,1) from seed 0, upstream
    gradient of ones), the one configuration the reference's CPU code runs whole: its forward + backward time on the
    host cores, this library's on the GPU (through the C ABI), and the largest max-normalised difference between the
    two sets of results (o, dq, dk, dv): the reference itself as the checker, on this machine."""
    from reproducing_fastmax_results_b200 import _lib

    ein = reference_einops()
    if ein is None:
        return None
    B, H, N, D = 2, 4, 256, 32
    torch.manual_seed(0)
    q, k, v = (torch.randn(B, H, N, D) for _ in range(3))
    do = torch.ones(B, H, N, D)
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)

    def ref_step():
        qq, kk, vv = (t.clone().requires_grad_(True) for t in (q, k, v))
        o = ein.fastmax(qq, kk, vv, mask=False, normalize_term=8, tensors_normalized=False, p=2)
        o.backward(do)
        return o.detach(), qq.grad, kk.grad, vv.grad

    ref_step()
    t0 = time.perf_counter()
    reps = 5
    for _ in range(reps):
        ref = ref_step()
    cpu_ms = (time.perf_counter() - t0) / reps * 1e3
    qd, kd, vd, dod = (t.to(dev) for t in (q, k, v, do))
    inv_temp = 1.0 / (8.0 * math.sqrt(D))

    def gpu_step():
        o, g, _ = _lib.forward(qd, kd, vd, False, inv_temp, order=2)
        return (o,) + tuple(_lib.backward(qd, kd, vd, o, g, dod, False, inv_temp, order=2)[:3])

    for _ in range(5):
        got = gpu_step()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(50):
        gpu_step()
    b.record()
    torch.cuda.synchronize()
    gpu_ms = a.elapsed_time(b) / 50
    err = max(float((x.cpu().double() - r.double()).abs().max() / r.double().abs().max()) for x, r in zip(got, ref))
    return {"config": "order 2, no mask, float32, B2 H4 N256 D32, forward + backward, upstream gradient of ones",
            "reference_cpu_ms": cpu_ms, "cores": threads, "gpu_ms": gpu_ms,
            "reference_cpu_ktokens_per_s": B * N / cpu_ms, "gpu_ktokens_per_s": B * N / gpu_ms,
            "max_normalised_difference": err, "tolerance": 1e-4}


def config4_record(torch, dev):
    """BASELINE config 4 exactly (order 1, no mask, B64 H12 N1024 D64, bfloat16 values, forward only): the reference's
    einops forward on the host cores (on the bf16-rounded inputs, in float32), this library's forward on the GPU
    through the C ABI, and the max-normalised difference of the outputs (bfloat16 tolerance)."""
    from reproducing_fastmax_results_b200 import _lib

    ein = reference_einops()
    if ein is None:
        return None
    B, H, N, D = 64, 12, 1024, 64
    g = torch.Generator().manual_seed(0)
    q, k, v = ((torch.randn(B, H, N, D, generator=g) * 0.5).bfloat16() for _ in range(3))
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    qf, kf, vf = q.float(), k.float(), v.float()
    with torch.no_grad():
        ref = ein.fastmax(qf, kf, vf, mask=False, normalize_term=8, tensors_normalized=False, p=1)
        t0 = time.perf_counter()
        reps = 3
        for _ in range(reps):
            ein.fastmax(qf, kf, vf, mask=False, normalize_term=8, tensors_normalized=False, p=1)
        cpu_ms = (time.perf_counter() - t0) / reps * 1e3
    qd, kd, vd = (t.to(dev) for t in (q, k, v))
    inv_temp = 1.0 / (8.0 * math.sqrt(D))
    for _ in range(5):
        o, _, _ = _lib.forward(qd, kd, vd, False, inv_temp, order=1)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(50):
        _lib.forward(qd, kd, vd, False, inv_temp, order=1)
    b.record()
    torch.cuda.synchronize()
    gpu_ms = a.elapsed_time(b) / 50
    err = float((o.float().cpu().double() - ref.double()).abs().max() / ref.double().abs().max())
    return {"config": "order 1, no mask, bfloat16 values, B64 H12 N1024 D64, forward only",
            "reference_cpu_ms": cpu_ms, "cores": threads, "gpu_ms": gpu_ms,
            "reference_cpu_mtokens_per_s": B * N / cpu_ms / 1e3, "gpu_mtokens_per_s": B * N / gpu_ms / 1e3,
            "max_normalised_difference": err, "tolerance": 2e-2}


def score_function_sample(workload, n_sample=256):
    """Second CPU figure: the reference's other CPU implementation (attention_mechanisms/score_function.py, autograd
    backward) on one head of n_sample tokens of the workload.  Returns a record or None when the file is not placed."""
    import importlib.util

    import torch

    path = os.path.join(os.path.dirname(REFERENCE_EINOPS), "score_function.py")
    if not os.path.exists(path):
        return None
    name = "fastmax_reference_score_function"
    if name in sys.modules:
        mod = sys.modules[name]
    else:
        spec = importlib.util.spec_from_file_location(name, path)
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
    B, H, N, D, order, causal, dtype, scale = WORKLOADS[workload]
    threads = os.cpu_count() or 1
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(0)
    q, k, v, do = (torch.randn(1, 1, n_sample, D, generator=g) * scale for _ in range(4))
    if dtype == "bf16":
        q, k, v, do = (t.bfloat16().float() for t in (q, k, v, do))
    q.requires_grad_(True), k.requires_grad_(True), v.requires_grad_(True)
    t0 = time.perf_counter()
    o = mod.fastmax(q, k, v, mask=causal, denum_term=8, normalize=0, p=order)
    o.backward(do)
    sec = time.perf_counter() - t0
    return {"value": (n_sample / H) / sec / 1e6, "unit": "Mtokens/s", "cores": threads, "seconds": sec,
            "sample": f"the reference's score_function.fastmax (mask={causal}, p={order}, denum_term=8) forward + autograd "
                      f"backward on 1 of {B * H} heads, {n_sample} of {N} tokens, D={D}; head-tokens / H = metric tokens"}


def cpu_baseline_record(workload, n_sample, heads):
    """CPU figure for the JSON line: the reference's einops code when it is present (kind "reference"), with the oracle's
    restatement as a second figure; the restatement alone (kind "port") otherwise."""
    B, H, N, D, order, causal, dtype, scale = WORKLOADS[workload]
    cpu_sample(workload, min(n_sample, 256), 1)  # page the CPU kernels in
    sec_p, ht_p, threads = cpu_sample(workload, n_sample, heads if reference_einops() is None else max(1, heads // 4))
    port = {"value": (ht_p / H) / sec_p / 1e6, "unit": "Mtokens/s", "cores": threads, "kind": "port", "seconds": sec_p,
            "sample": cpu_sample_text(workload, n_sample, ht_p // n_sample)}
    if reference_einops() is None:
        return port
    ref_heads = max(1, heads // 12)
    cpu_sample_reference(workload, 64, 1)
    sec, ht, threads = cpu_sample_reference(workload, n_sample, ref_heads)
    return {"value": (ht / H) / sec / 1e6, "unit": "Mtokens/s", "cores": threads, "kind": "reference", "seconds": sec,
            "sample": f"the reference's fastattention_einops.fastmax (mask={causal}, p={order}, normalize_term=8) forward + backward "
                      f"on {ref_heads} of {B * H} heads, {n_sample} of {N} tokens each, D={D} (its memory is O(N D^3) per head); "
                      "head-tokens / H = metric tokens",
            "port": port}


def bind_host_near_gpu(torch, index):
    """Pins this process to the CPU cores that sit on the GPU's PCIe root (sysfs local_cpulist), so that the pinned
    host buffers it allocates afterwards are first touched on that NUMA node.  Returns the core list or None."""
    try:
        props = torch.cuda.get_device_properties(index)
        bdf = "%04x:%02x:%02x.0" % (props.pci_domain_id, props.pci_bus_id, props.pci_device_id)
        with open(f"/sys/bus/pci/devices/{bdf}/local_cpulist") as f:
            text = f.read().strip()
        cores = set()
        for part in text.split(","):
            if "-" in part:
                a, b = part.split("-")
                cores.update(range(int(a), int(b) + 1))
            elif part:
                cores.add(int(part))
        allowed = os.sched_getaffinity(0)
        cores &= allowed
        if cores and cores != allowed:
            os.sched_setaffinity(0, cores)
            return text
    except Exception:
        pass
    return None


def run_reference_arm(args):
    """`--impl reference`: the reference's CPU implementation of the path timed on the host, rank 0 only: its own
    fastattention_einops.py when present under oracle/_ref/, else the oracle's restatement (kind "port")."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    B, H, N, D, order, causal, dtype, scale = WORKLOADS[args.workload]
    use_ref = reference_einops() is not None
    n_sample = args.ref_tokens if use_ref else args.cpu_tokens
    heads = 1 if use_ref else args.ref_heads
    sample = cpu_sample_reference if use_ref else cpu_sample
    for _ in range(min(args.warmup, 1)):
        sample(args.workload, n_sample, 1)
    times = []
    threads = 1
    head_tokens = heads * n_sample
    for _ in range(args.steps):
        t, head_tokens, threads = sample(args.workload, n_sample, heads)
        times.append(t)
    sec = sum(times) / len(times)
    # metric tokens carry all H heads: one head of n_sample tokens is n_sample / H metric tokens
    value = (head_tokens / H) / sec / 1e6
    text = (f"fastattention_einops.fastmax forward + backward, {heads} of {B * H} heads x {n_sample} of {N} tokens per step"
            if use_ref else cpu_sample_text(args.workload, n_sample, heads))
    line = {
        "impl": "reference",
        "metric": "fastmax_fwd_bwd_mtokens_per_s", "value": value, "unit": "Mtokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "sample": f"{heads} head(s) x {n_sample} tokens per step"},
        "cpu_baseline": {"value": value, "unit": "Mtokens/s", "cores": threads, "kind": "reference" if use_ref else "port",
                         "seconds": sec, "sample": text},
        "e2e": {"value": value, "unit": "Mtokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    emit(line)
    return 0


# ----------------------------------------------------------------------------------------------------
# GPU arm, sequence-sharded workload: every rank owns N/world consecutive tokens of all heads; the ranks
# exchange the moment states (forward: exclusive prefix, backward: exclusive suffix) with one all_gather each.
# ----------------------------------------------------------------------------------------------------
def _exact_rows_fp64(torch, q_rows, rows, k, v, inv_temp, o_rows=None, g_rows=None, do_rows=None):
    """Exact float64 evaluation on the device of sampled causal query rows (global positions `rows`) against ALL keys
    k, v (b, h, N, d): returns o rows, and dq rows when o/g/dO rows are given.  O(N d) per row, no N x N matrix."""
    kd, vd = k.double(), v.double()
    qd = q_rows.double()                                                  # (b, h, r, d)
    s = torch.einsum("bhrd,bhnd->bhrn", qd, kd) * inv_temp
    vis = (torch.arange(k.shape[2], device=k.device)[None, :] <= rows[:, None]).double()
    a = (1.0 + s + 0.5 * s * s) * vis
    g = a.sum(-1)
    o = torch.einsum("bhrn,bhnd->bhrd", a, vd) / g[..., None]
    if do_rows is None:
        return o, None
    dod = do_rows.double()
    dog = dod / g[..., None]
    dg = -(dod * o).sum(-1) / g
    da = torch.einsum("bhrd,bhnd->bhrn", dog, vd) + dg[..., None]
    ds = da * (1.0 + s) * vis
    return o, torch.einsum("bhrn,bhnd->bhrd", ds, kd) * inv_temp


def _exact_cols_fp64(torch, k_cols, v_cols, cols, q, o, g, do, inv_temp):
    """Exact float64 dk, dv of sampled key positions `cols` against ALL queries (b, h, N, d)."""
    qd, od, dod, gd = q.double(), o.double(), do.double(), g.double()
    kd, vd = k_cols.double(), v_cols.double()
    s = torch.einsum("bhnd,bhcd->bhnc", qd, kd) * inv_temp
    vis = (cols[None, :] <= torch.arange(q.shape[2], device=q.device)[:, None]).double()
    a = (1.0 + s + 0.5 * s * s) * vis
    dog = dod / gd[..., None]
    dg = -(dod * od).sum(-1) / gd
    da = torch.einsum("bhnd,bhcd->bhnc", dog, vd) + dg[..., None]
    ds = da * (1.0 + s) * vis
    dk = torch.einsum("bhnc,bhnd->bhcd", ds, qd) * inv_temp
    dv = torch.einsum("bhnc,bhnd->bhcd", a, dog)
    return dk, dv


def measure_sequence_sharded(workload, steps, warmup, torch, dist, dev, rank, world, check=True):
    """Forward + backward of one long causal sequence cut into `world` contiguous pieces (strong scaling): ms per
    step (max over ranks), the time inside the two all_gathers, per-kernel times, and the largest max-normalised
    error of sampled rows of o, dq, dk, dv on any rank against an exact float64 evaluation on the device."""
    from reproducing_fastmax_results_b200 import _lib, sequence_parallel as sp

    B, H, N, D, order, causal, dtype_name, scale = WORKLOADS[workload]
    dtype = torch.bfloat16 if dtype_name == "bf16" else torch.float32
    n_local = N // world
    inv_temp = 1.0 / (8.0 * math.sqrt(D))
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    q, k, v, do = ((torch.randn(B, H, n_local, D, device=dev, generator=gen) * scale).to(dtype) for _ in range(4))
    eng = sp.CudaEngine(inv_temp, p=order)
    lib = _lib.load()

    def step():
        o, g, prefix = sp.forward(eng, q, k, v)
        return (o, g) + tuple(sp.backward(eng, q, k, v, o, g, do, prefix))

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        step()
    barrier()
    sampler = ClockSampler(torch.cuda.current_device())
    if rank == 0:
        sampler.start()
    launches0 = lib.fastmax_launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(steps):
        step()
    ev1.record()
    barrier()
    launches = lib.fastmax_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ev0.elapsed_time(ev1)], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / steps
    # the exchange alone: both all_gathers of a step on states of the real size, device-timed
    exchange_ms = 0.0
    if dist is not None:
        st = eng.key_state(k, v)
        for _ in range(2):
            sp.exclusive_prefix(st), sp.exclusive_suffix(st)
        barrier()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record()
        for _ in range(steps):
            sp.exclusive_prefix(st), sp.exclusive_suffix(st)
        a1.record()
        barrier()
        te = torch.tensor([a0.elapsed_time(a1)], device=dev, dtype=torch.float64)
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
        exchange_ms = float(te.item()) / steps
    _lib.profile(True)
    for _ in range(steps):
        step()
    torch.cuda.synchronize()
    _lib.profile(False)
    kernels = {name: {"ms_per_launch": ms / cnt, "launches_per_step": cnt / steps, "ms_per_step": ms / steps}
               for name, (ms, cnt) in _lib.profile_collect().items()}
    def parity_error():
        o, g, dq, dk, dv = step()
        full = []
        for x in (q, k, v, do, o, g):
            if dist is None:
                full.append(x)
            else:
                parts = [torch.empty_like(x) for _ in range(world)]
                dist.all_gather(parts, x.contiguous())
                full.append(torch.cat(parts, dim=2))
        fq, fk, fv, fdo, fo, fg = full
        sg = torch.Generator(device=dev).manual_seed(99)
        local = torch.randint(0, n_local, (6,), device=dev, generator=sg)
        local = torch.cat([local, torch.tensor([0, n_local - 1], device=dev)])
        rows = local + rank * n_local
        o_ref, dq_ref = _exact_rows_fp64(torch, q[:, :, local], rows, fk, fv, inv_temp, o[:, :, local], g[:, :, local],
                                         do[:, :, local])
        dk_ref, dv_ref = _exact_cols_fp64(torch, k[:, :, local], v[:, :, local], rows, fq, fo, fg, fdo, inv_temp)
        # max-normalised against the largest magnitude of the WHOLE local tensor (rows alone may sit near zero)
        def err(x, ref, whole):
            return float(((x.double() - ref).abs().max() / whole.double().abs().max()).item())
        e = max(err(o[:, :, local], o_ref, o), err(dq[:, :, local], dq_ref, dq), err(dk[:, :, local], dk_ref, dk),
                err(dv[:, :, local], dv_ref, dv))
        te = torch.tensor([e], device=dev, dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        return float(te.item()), int(rows.numel())

    parity = None
    if check:
        e, nrows = parity_error()
        parity = {"max_normalised_error_all_ranks": e, "tolerance": 1e-4 if dtype_name == "f32" else 2e-2,
                  "rows_per_rank": nrows,
                  "how": "sampled rows of o, dq and sampled key positions of dk, dv on every rank against an exact float64 "
                         "row evaluation over the gathered sequence, on the device"}
    medium = None
    if check and dtype == torch.float32:
        # the same float32 step after torch.set_float32_matmul_precision("medium"): the pieces run on bfloat16 copies on the
        # tensor-memory kernels (32-wide heads zero-padded to 64), the exchanged states stay float32; bfloat16 tolerance
        saved_precision = torch.get_float32_matmul_precision()
        torch.set_float32_matmul_precision("medium")
        try:
            for _ in range(2):
                step()
            barrier()
            ev0.record()
            for _ in range(steps):
                step()
            ev1.record()
            barrier()
            tm = torch.tensor([ev0.elapsed_time(ev1)], device=dev, dtype=torch.float64)
            if dist is not None:
                dist.all_reduce(tm, op=dist.ReduceOp.MAX)
            _lib.profile_collect()
            _lib.profile(True)
            step()
            torch.cuda.synchronize()
            _lib.profile(False)
            kinds = sorted(_lib.profile_collect())
            e, _ = parity_error()
            medium = {"ms_per_step": float(tm.item()) / steps, "max_normalised_error_all_ranks": e, "tolerance": 2e-2,
                      "engines": kinds}
        finally:
            torch.set_float32_matmul_precision(saved_precision)
    rows_state = (64 * (D // 8) * (D // 8 + 1) // 2) + D + 1
    return {"ms_per_step": ms_step, "value": B * N / (ms_step * 1e-3) / 1e6, "unit": "Mtokens/s", "exchange_ms_per_step": exchange_ms,
            "state_bytes_per_rank": B * H * rows_state * (D + 4) * 4, "tokens_per_rank": n_local, "kernels": kernels,
            "gpu_launches": int(launches), "clocks": clocks, "parity": parity, "engines": sorted(kernels),
            "medium_matmul_precision": medium}


def run_sequence_sharded(args, torch, dist, dev, rank, world):
    B, H, N, D, order, causal, dtype_name, scale = WORKLOADS[args.workload]
    r = measure_sequence_sharded(args.workload, args.steps, args.warmup, torch, dist, dev, rank, world)
    ms_step, value, kernels = r["ms_per_step"], r["value"], r["kernels"]
    if rank == 0:
        pk = peaks()
        U = algorithmic_flops(B, H, N, D, order)
        m_full = 1 + D + (D * D if order == 2 else 0)
        executed = 6.0 * U * executed_units(D, order) / m_full / world  # per rank (the exchange replaces no flops)
        line = {
            "metric": "fastmax_fwd_bwd_mtokens_per_s", "value": value, "unit": "Mtokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": dtype_name + " inputs, f32 accumulate", "data": "synthetic",
            "config": {"workload": args.workload, "batch": B, "heads": H, "seq_len": N, "tokens_per_rank": r["tokens_per_rank"],
                       "head_dim": D, "order": order, "causal": causal,
                       "parallelism": f"sequence pieces over {world} rank(s); all_gather of {r['state_bytes_per_rank']} state bytes per rank, "
                                      "once forward (exclusive prefix) and once backward (exclusive suffix)",
                       "l2": "inputs exceed the 126 MB L2 at 1-2 ranks; no explicit flush"},
            "roofline": {"kernel": "whole step (fp32 CUDA-core engine)", "bound": "tensor",
                         "achieved": executed / (ms_step * 1e-3) / 1e12, "peak": pk["bf16_tflops_sustained"] / 2.0,
                         "unit": "TFLOP/s", "frac": executed / (ms_step * 1e-3) / 1e12 / (pk["bf16_tflops_sustained"] / 2.0),
                         "peak_source": pk["_source"] + " bf16 sustained / 2 (TF32 runs at half the bf16 rate; no TF32 peak was measured)",
                         "note": "executed flops of one rank over the step time; the fp32 engine runs on the FFMA pipe because "
                                 "TF32 operands miss the 1e-4 tolerance", "traffic": None},
            "exchange_ms_per_step": r["exchange_ms_per_step"], "parity": r["parity"],
            "kernels": kernels, "cpu_baseline": None, "e2e": None, "gpu_launches": r["gpu_launches"], "clocks": r["clocks"],
        }
        emit(line)
    if dist is not None:
        dist.destroy_process_group()
    return 0


# ----------------------------------------------------------------------------------------------------
# GPU arm, decoding workload: one fastmax_decode_step per step; every rank decodes its own batch (weak scaling)
# ----------------------------------------------------------------------------------------------------
def run_decode(args, torch, dist, dev, rank, world):
    from reproducing_fastmax_results_b200 import _lib

    B, H, _, D, order, causal, dtype_name, scale = WORKLOADS[args.workload]
    dtype = torch.bfloat16 if dtype_name == "bf16" else torch.float32
    inv_temp = 1.0 / (8.0 * math.sqrt(D))
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    ntok = 16
    q, k, v = ((torch.randn(B, H, ntok, D, device=dev, generator=gen) * scale).to(dtype) for _ in range(3))
    state = _lib.new_state(B, H, D, order, dev)
    out = torch.empty(B, H, D, device=dev, dtype=dtype)
    lib = _lib.load()
    counter = [0]

    def step():
        t = counter[0] % ntok
        counter[0] += 1
        _lib.decode_step(q[:, :, t], k[:, :, t], v[:, :, t], state, inv_temp, order=order, out=out)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(torch.cuda.current_device())
    if rank == 0:
        sampler.start()
    launches0 = lib.fastmax_launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    launches = lib.fastmax_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ev0.elapsed_time(ev1)], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    # the same steps replayed from a CUDA graph (what a generation loop would do): no host launch gaps
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(ntok):
            step()
    reps = max(1, args.steps // ntok)
    graph.replay()
    torch.cuda.synchronize()
    g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    g0.record()
    for _ in range(reps):
        graph.replay()
    g1.record()
    torch.cuda.synchronize()
    ms_graph = g0.elapsed_time(g1) / (reps * ntok)
    if rank == 0:
        pk = peaks()
        state_bytes = state.numel() * 4
        gbs = 2.0 * state_bytes / (ms_step * 1e-3) / 1e9
        line = {
            "metric": "fastmax_decode_mtokens_per_s", "value": world * B / (ms_step * 1e-3) / 1e6, "unit": "Mtokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": dtype_name + " tokens, f32 state", "data": "synthetic",
            "config": {"workload": args.workload, "batch_per_gpu": B, "heads": H, "head_dim": D, "order": order,
                       "parallelism": f"batch sharding, {world} rank(s), no collective",
                       "l2": f"the states ({state_bytes >> 20} MiB per rank) exceed the 126 MB L2; no explicit flush"},
            "roofline": {"kernel": "decode_step", "bound": "hbm", "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / pk["hbm_gbs"], "peak_source": pk["_source"],
                         "note": "algorithmic bytes = one read and one write of every head's state; launch gaps between "
                                 "the back-to-back steps are inside the time",
                         "traffic": 604.3e6 * state_bytes / 329.9e6, "traffic_source": "profiles/ncu_decode_step.md",
                         "cuda_graph": {"ms_per_step": ms_graph, "achieved": 2.0 * state_bytes / (ms_graph * 1e-3) / 1e9,
                                        "frac": 2.0 * state_bytes / (ms_graph * 1e-3) / 1e9 / pk["hbm_gbs"]}},
            "cpu_baseline": None, "e2e": None, "gpu_launches": int(launches), "clocks": clocks,
        }
        emit(line)
    if dist is not None:
        dist.destroy_process_group()
    return 0


# ----------------------------------------------------------------------------------------------------
# GPU arm, normalisation workload: y = lim (x - mean_d x) / max_token ||x - mean_d x|| of one tensor and its backward
# ----------------------------------------------------------------------------------------------------
def run_normalize(args, torch, dist, dev, rank, world):
    from reproducing_fastmax_results_b200 import _lib

    B, H, N, D, order, causal, dtype_name, scale = WORKLOADS[args.workload]
    dtype = torch.bfloat16 if dtype_name == "bf16" else torch.float32
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    x, dy = ((torch.randn(B, H, N, D, device=dev, generator=gen) * scale).to(dtype) for _ in range(2))
    lib = _lib.load()

    def step():
        y, stats = _lib.normalize_forward(x)
        return _lib.normalize_backward(y, dy, stats)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(torch.cuda.current_device())
    if rank == 0:
        sampler.start()
    launches0 = lib.fastmax_launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    launches = lib.fastmax_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ev0.elapsed_time(ev1)], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    _lib.profile(True)
    for _ in range(args.steps):
        step()
    torch.cuda.synchronize()
    _lib.profile(False)
    kernels = {name: {"ms_per_launch": ms / cnt, "launches_per_step": cnt / args.steps, "ms_per_step": ms / args.steps}
               for name, (ms, cnt) in _lib.profile_collect().items()}
    if rank == 0:
        pk = peaks()
        nbytes = x.numel() * x.element_size()
        bytes_alg = 5 * nbytes   # forward: read x, write y; backward: read y and dy, write dx
        gbs = bytes_alg / (ms_step * 1e-3) / 1e9
        emit({
            "metric": "fastmax_normalize_fwd_bwd_mtokens_per_s", "value": world * B * N / (ms_step * 1e-3) / 1e6,
            "unit": "Mtokens/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype_name + " tensors, f32 statistics",
            "data": "synthetic",
            "config": {"workload": args.workload, "batch_per_gpu": B, "heads": H, "seq_len": N, "head_dim": D,
                       "parallelism": f"batch x head sharding, {world} rank(s), no collective",
                       "l2": "x, y, dy, dx are %d MB each; no explicit flush" % (nbytes >> 20)},
            "roofline": {"kernel": "normalize forward + backward (%s)" % ", ".join(sorted(kernels)), "bound": "hbm",
                         "achieved": gbs, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"],
                         "peak_source": pk["_source"],
                         "note": "algorithmic bytes: forward reads x and writes y, backward reads y and dy and writes dx; the "
                                 "second read of x by the forward's statistics pass is not algorithmic", "traffic": None},
            "kernels": kernels, "cpu_baseline": None, "e2e": None, "gpu_launches": int(launches), "clocks": clocks,
        })
    if dist is not None:
        dist.destroy_process_group()
    return 0


# ----------------------------------------------------------------------------------------------------
# GPU arm, BASELINE config 5: the REFERENCE's transformer (transformer/model.py, vendored unmodified but for the one
# documented edit, see baseline/vendor_reference.py) trained on seeded random token ids; the attention operator under
# it is this library.  Data parallel over the ranks with torch DDP (gradient all-reduce over NCCL), weak scaling.
# ----------------------------------------------------------------------------------------------------
CFG5 = dict(out_dim=50257, max_tokens=1024, d_model=512, d_mlp=2048, heads_per_block=8, num_blocks=6, dropout_rate=0.0,
            use_masking=True, vocab_size=50257, fastmax=True, p=2)


def measure_cfg5(torch, dist, dev, rank, world, steps=5, warmup=3, batch=16, seq=1024):
    import contextlib

    from baseline import reference_model
    import reproducing_fastmax_results_b200 as pkg
    from reproducing_fastmax_results_b200 import _lib

    if not reference_model.available():
        return {"unavailable": "baseline/_ref/transformer is not populated (python baseline/vendor_reference.py <reference>)"}
    model = reference_model.load()
    out = {"model": "reference transformer/model.py Transformer(%s)" % ", ".join(f"{k}={v}" for k, v in CFG5.items()),
           "batch_per_replica": batch, "seq_len": seq, "optimizer": "AdamW lr 3e-4", "scaling": "weak",
           "data": "seeded uniform-random token ids, targets = ids shifted by one"}
    lib = _lib.load()
    variants = {
        # the model exactly as the reference runs it: float32, its own autograd Function over fastmax_cuda.forwardpass
        "f32_reference_function": dict(autocast=False, swap=False, medium=False),
        # the same unmodified float32 model after torch.set_float32_matmul_precision("medium"), PyTorch's switch that lets
        # float32 matmuls (the model's Linear layers included) compute in bfloat16: forwardpass / backwardpass then run
        # the attention on the tensor-memory kernels through bfloat16 copies
        "f32_reference_function_medium_matmul_precision": dict(autocast=False, swap=False, medium=True),
        # same call site (model.py:303), module-level fastmax_custom replaced by this package's zero-copy FastMax,
        # bf16 autocast: q, k, v reach the tensor-memory kernels as strided bf16 views
        "bf16_autocast_zero_copy": dict(autocast=True, swap=True, medium=False),
    }
    if world > 1:
        # the collective alone: one all-reduce of a tensor as large as the model's gradients, nothing else running
        buf = torch.zeros(70944337, device=dev)
        for _ in range(2):
            dist.all_reduce(buf)
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(5):
            dist.all_reduce(buf)
        b.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(b) / 5], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ar_ms = float(t.item())
        out["allreduce_alone"] = {"bytes": 4 * buf.numel(), "ms": ar_ms,
                                  "bus_gbs": 2.0 * (world - 1) / world * 4 * buf.numel() / (ar_ms * 1e-3) / 1e9}
        del buf
    for vname, vcfg in variants.items():
        torch.manual_seed(0)
        net = model.Transformer(**CFG5).to(dev)
        nparams = sum(p.numel() for p in net.parameters())
        ddp = net
        if world > 1:
            from torch.nn.parallel import DistributedDataParallel as DDP

            ddp = DDP(net, device_ids=[dev.index])
        opt = torch.optim.AdamW(net.parameters(), lr=3e-4)
        gen = torch.Generator(device=dev).manual_seed(rank)
        ids = torch.randint(0, CFG5["vocab_size"], (batch, seq + 1), device=dev, generator=gen)
        saved = model.fastmax_custom
        saved_precision = torch.get_float32_matmul_precision()
        if vcfg["swap"]:
            model.fastmax_custom = pkg.fastmax_custom
        if vcfg["medium"]:
            torch.set_float32_matmul_precision("medium")
        try:
            def step(sync=True):
                # sync=False: the same step on the bare module (no DDP hooks, no gradient all-reduce): the replicas
                # drift apart, so it is only used for the last timing of a variant
                fwd = ddp if sync else net
                with torch.autocast("cuda", dtype=torch.bfloat16, enabled=vcfg["autocast"]):
                    logits = fwd(ids[:, :-1])
                loss = torch.nn.functional.cross_entropy(logits.float().reshape(-1, logits.shape[-1]), ids[:, 1:].reshape(-1))
                opt.zero_grad(set_to_none=True)
                loss.backward()
                opt.step()
                return loss

            def timed(n, sync=True):
                if dist is not None:
                    dist.barrier()
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(n):
                    loss = step(sync)
                b.record()
                if dist is not None:
                    dist.barrier()
                torch.cuda.synchronize()
                t = torch.tensor([a.elapsed_time(b)], device=dev, dtype=torch.float64)
                if dist is not None:
                    dist.all_reduce(t, op=dist.ReduceOp.MAX)
                return float(t.item()) / n, float(loss.detach())

            import io

            with contextlib.redirect_stdout(io.StringIO()):   # the reference prints a dtype notice per call under bf16
                loss0 = float(step().detach())
                for _ in range(warmup - 1):
                    step()
                l0 = lib.fastmax_launch_count()
                ms, loss1 = timed(steps)
                launches = lib.fastmax_launch_count() - l0
                _lib.profile_collect()
                _lib.profile(True)
                step()
                torch.cuda.synchronize()
                _lib.profile(False)
                prof = _lib.profile_collect()
                ms_nosync = None
                if world > 1:
                    step(sync=False)
                    ms_nosync = timed(steps, sync=False)[0]
            lib_ms = sum(m for m, _ in prof.values())
            out[vname] = {
                "value": world * batch * seq / (ms * 1e-3), "unit": "tokens/s", "ms_per_step": ms, "parameters": nparams,
                "loss_first_step": loss0, "loss_last_step": loss1, "library_launches_per_step": launches / steps,
                "library_ms_per_step": lib_ms, "library_share_of_step": lib_ms / ms,
                "library_kernels": {k: round(m, 4) for k, (m, _) in sorted(prof.items())},
                "gradient_allreduce": None if world == 1 else {
                    "bytes_per_step": 4 * nparams, "ms_per_step_without_gradient_sync": ms_nosync,
                    "exposed_ms_per_step": ms - ms_nosync,
                    "note": "DDP buckets the all-reduce under the backward pass; exposed = step time minus the same step "
                            "of the bare module (no DDP hooks, no all-reduce), timed right after"},
            }
        finally:
            model.fastmax_custom = saved
            torch.set_float32_matmul_precision(saved_precision)
        del net, ddp, opt
        torch.cuda.empty_cache()
    return out


def measure_cfg2_strong(torch, dist, dev, rank, world, steps=10, warmup=3):
    """The FIXED config-2 problem (B8 H16 N4096 D64 bf16, causal, order 2) split over the ranks by batch (128 / world
    heads each, no collective): strong scaling, device-timed, max over ranks."""
    from reproducing_fastmax_results_b200 import _lib

    B, H, N, D, order, causal, dtype_name, scale = WORKLOADS[DEFAULT]
    if B % world:
        return {"unavailable": f"batch {B} does not divide over {world} ranks"}
    b = B // world
    gen = torch.Generator(device=dev).manual_seed(4321 + rank)
    q, k, v, do = ((torch.randn(b, H, N, D, device=dev, generator=gen) * scale).bfloat16() for _ in range(4))
    inv_temp = 1.0 / (8.0 * math.sqrt(D))

    def step():
        o, g, _ = _lib.forward(q, k, v, causal, inv_temp, order=order)
        return _lib.backward(q, k, v, o, g, do, causal, inv_temp, order=order)

    for _ in range(warmup):
        step()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        step()
    e.record()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(e)], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item()) / steps
    _lib.profile_collect()
    _lib.profile(True)
    step()
    torch.cuda.synchronize()
    _lib.profile(False)
    return {"ms_per_step": ms, "value": B * N / (ms * 1e-3) / 1e6, "unit": "Mtokens/s", "scaling": "strong",
            "heads_per_rank": b * H, "engines": sorted(_lib.profile_collect())}


def measure_reference_boundary(torch, dist, dev, rank, world, steps=3, warmup=1):
    """Config 2's shape through the reference's own boundary, per rank (weak): float32 (b, h, n, d) tensors into
    `FASTMultiHeadAttention_Function` (the twin of transformer/model.py:14-74: reshape, permute to (n, b*h, d) with
    copies, `fastmax_cuda.forwardpass` / `backwardpass`, permute back), forward + backward.  float32 puts the call on
    the CUDA-core engine; the figure says what a caller gets who changes nothing but the import."""
    from reproducing_fastmax_results_b200.attention import FASTMultiHeadAttention_Function

    B, H, N, D, order, causal, _, scale = WORKLOADS[DEFAULT]
    gen = torch.Generator(device=dev).manual_seed(99 + rank)
    q, k, v = ((torch.randn(B, H, N, D, device=dev, generator=gen) * scale).requires_grad_(True) for _ in range(3))
    do = torch.randn(B, H, N, D, device=dev, generator=gen) * scale
    noise = torch.zeros(B, H, N, D, device=dev)
    rpe = torch.zeros(2 * N - 1, D, device=dev)
    temperature = 8.0 * math.sqrt(D)

    def step():
        for t in (q, k, v):
            t.grad = None
        o = FASTMultiHeadAttention_Function.apply(q, k, v, noise, rpe, causal, 0.0, False, temperature, 1.0, 1.0, 0.5, 1.0, order)
        o.backward(do)

    for _ in range(warmup):
        step()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        step()
    e.record()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([a.elapsed_time(e)], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item()) / steps
    # the same calls after torch.set_float32_matmul_precision("medium"): forwardpass / backwardpass may compute in bfloat16
    saved_precision = torch.get_float32_matmul_precision()
    torch.set_float32_matmul_precision("medium")
    try:
        for _ in range(2):
            step()
        torch.cuda.synchronize()
        a.record()
        for _ in range(10):
            step()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([a.elapsed_time(e)], device=dev, dtype=torch.float64)
        if dist is not None:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_medium = float(t.item()) / 10
    finally:
        torch.set_float32_matmul_precision(saved_precision)
    return {"ms_per_step": ms, "value": world * B * N / (ms * 1e-3) / 1e6, "unit": "Mtokens/s", "scaling": "weak", "dtype": "f32",
            "api": "FASTMultiHeadAttention_Function.apply + backward: the reference wrapper's permutes and copies around "
                   "fastmax_cuda.forwardpass / backwardpass (float32 contract, CUDA-core engine)",
            "medium_matmul_precision": {"ms_per_step": ms_medium, "value": world * B * N / (ms_medium * 1e-3) / 1e6,
                                        "note": "same float32 tensors and calls after torch.set_float32_matmul_precision('medium'): "
                                                "the extension converts q, k, v and the upstream gradient to bfloat16 and runs the "
                                                "tensor-memory kernels (bfloat16 tolerance, not float32 parity)"}}


def other_workloads(args, torch, dist, dev, rank, world):
    """Bounded extra measurements reported beside the headline (same process group, after its timed region)."""
    out = {}
    legs = [("cfg2_strong", lambda: measure_cfg2_strong(torch, dist, dev, rank, world)),
            ("cfg3", lambda: measure_sequence_sharded("cfg3_f32_causal_p2_B1_H8_N131072_D32", 3, 3, torch, dist, dev, rank, world)),
            ("cfg5", lambda: measure_cfg5(torch, dist, dev, rank, world)),
            ("cfg2_reference_boundary_f32", lambda: measure_reference_boundary(torch, dist, dev, rank, world))]
    for name, fn in legs:
        t0 = time.perf_counter()
        try:
            out[name] = fn()
        except Exception as e:   # a leg that fails is reported, the headline line still goes out
            out[name] = {"error": f"{type(e).__name__}: {e}"[:400]}
        if isinstance(out[name], dict):
            out[name]["wall_s"] = round(time.perf_counter() - t0, 2)
        torch.cuda.empty_cache()
    return out


# ----------------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default=DEFAULT, choices=sorted(WORKLOADS))
    ap.add_argument("--cpu-tokens", type=int, default=512, help="tokens per head of the bounded CPU-baseline sample")
    ap.add_argument("--cpu-heads", type=int, default=24, help="heads of the CPU-baseline sample (about 10 s of CPU work)")
    ap.add_argument("--ref-heads", type=int, default=6, help="--impl reference: heads per step (a few seconds each)")
    ap.add_argument("--ref-tokens", type=int, default=256,
                    help="--impl reference on the reference's einops code: tokens of the one head per step (seconds each; its "
                         "time and memory grow linearly with the tokens, so tokens/s does not depend on this)")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-other", action="store_true", help="skip the other_workloads legs (cfg2 strong scaling, cfg3, cfg5)")
    ap.add_argument("--no-tensor-cores", action="store_true", help="force the CUDA-core kernels")
    ap.add_argument("--mode", default="fwd_bwd", choices=["fwd_bwd", "fwd"],
                    help="fwd: time the forward call only (profiling aid; the headline metric is fwd_bwd)")
    args = ap.parse_args()
    claim_stdout()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = max(args.warmup, 1)
    if args.impl == "reference":
        return run_reference_arm(args)

    import torch

    from reproducing_fastmax_results_b200 import _lib
    import reproducing_fastmax_results_b200 as pkg

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        import datetime

        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=300))

    if args.workload in SEQUENCE_SHARDED:
        return run_sequence_sharded(args, torch, dist, dev, rank, world)
    if args.workload in DECODE:
        return run_decode(args, torch, dist, dev, rank, world)
    if args.workload in NORMALIZE:
        return run_normalize(args, torch, dist, dev, rank, world)
    B, H, N, D, order, causal, dtype_name, scale = WORKLOADS[args.workload]
    dtype = torch.bfloat16 if dtype_name == "bf16" else torch.float32
    inv_temp = 1.0 / (8.0 * math.sqrt(D))
    flags = _lib.FLAG_NO_TENSOR_CORES if args.no_tensor_cores else 0
    gen = torch.Generator(device=dev).manual_seed(1234 + rank)
    q, k, v, do = ((torch.randn(B, H, N, D, device=dev, generator=gen) * scale).to(dtype) for _ in range(4))
    lib = _lib.load()

    def step():
        # a fresh holder per step: within the step the backward takes the forward's per-segment key moments (calls that
        # are cut into segments; the default workload is not), nothing is carried from one step to the next
        km = _lib.KeyMoments()
        o, g, _ = _lib.forward(q, k, v, causal, inv_temp, order=order, flags=flags, key_moments=km)
        if args.mode == "fwd":
            return o
        return _lib.backward(q, k, v, o, g, do, causal, inv_temp, order=order, flags=flags, key_moments=km)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(torch.cuda.current_device())
    if rank == 0:
        sampler.start()
    launches0 = lib.fastmax_launch_count()
    ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    ev0.record()
    for _ in range(args.steps):
        step()
    ev1.record()
    barrier()
    ms_total = ev0.elapsed_time(ev1)
    launches = lib.fastmax_launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms_total], device=dev, dtype=torch.float64)
    if dist is not None:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / args.steps
    tokens_per_step = B * N * world
    value = tokens_per_step / (ms_step * 1e-3) / 1e6

    # ---- per-kernel device times (same steps again, launches bracketed by events) ----
    _lib.profile(True)
    for _ in range(args.steps):
        step()
    torch.cuda.synchronize()
    _lib.profile(False)
    prof = _lib.profile_collect()
    kernels = {name: {"ms_per_launch": ms / cnt, "launches_per_step": cnt / args.steps, "ms_per_step": ms / args.steps}
               for name, (ms, cnt) in prof.items()}
    total_kernel_ms = sum(kk["ms_per_step"] for kk in kernels.values())
    for kk in kernels.values():
        kk["share"] = kk["ms_per_step"] / total_kernel_ms if total_kernel_ms else 0.0
    pk = peaks()
    U = algorithmic_flops(B, H, N, D, order)
    # Work units per launch, in passes over all tokens (one pass = U flops with the full D^2 feature map):
    #   algorithmic: what the reference's formulation needs (forward 2, dq 1, dS + dk 2, dv 1: 6 per step);
    #   executed:    contraction passes the kernel really runs, over the block-symmetric feature rows (x 0.569):
    #                every scan recomputes its state (apply/dphi + update = 2 passes).
    units_alg = {"scan_fwd": 2.0, "tc_scan_fwd": 2.0, "scan_bwd_q": 1.0, "tc_scan_bwd_q": 1.0, "scan_bwd_kv": 3.0,
                 "tc_scan_bwd_kv": 2.0, "tc_scan_bwd_dv": 1.0, "moments_kv": 1.0, "moments_qg": 1.0, "tc_moments": 1.0}
    units_exec = {"tc_scan_fwd": 2.0, "tc_scan_bwd_q": 2.0, "tc_scan_bwd_kv": 2.0, "tc_scan_bwd_dv": 2.0}
    m_full = 1 + D + (D * D if order == 2 else 0)
    ratio_exec = executed_units(D, order) / m_full

    def counted_flops(name):
        """min(algorithmic, executed) flops of one launch: never credits more than the hardware did."""
        alg = units_alg.get(name, 0.0) * U
        ex = units_exec.get(name, units_alg.get(name, 0.0)) * U * (ratio_exec if name.startswith("tc_") else 1.0)
        return min(alg, ex), alg

    dominant = max(kernels, key=lambda n: kernels[n]["ms_per_step"]) if kernels else None
    roofline = None
    if dominant is not None:
        counted, alg = counted_flops(dominant)
        per_launch = 1.0 / max(kernels[dominant]["launches_per_step"], 1e-9)
        dur_s = kernels[dominant]["ms_per_launch"] * 1e-3
        peak = pk["bf16_tflops_sustained"]
        achieved = counted * per_launch / dur_s / 1e12
        roofline = {
            "kernel": dominant, "bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
            "frac": achieved / peak, "peak_source": pk["_source"] + " (sustained cuBLAS bf16: kernel timed inside a long step)",
            "full_d2_equivalent": alg * per_launch / dur_s / 1e12,
            "note": "achieved = min(algorithmic, executed) flops of the launch / its CUDA-event time: executed counts the "
                    "block-symmetric feature rows (0.569 of D^2+D+1) the kernel contracts over, twice (state rebuild + "
                    "apply or dphi); full_d2_equivalent is the rate the reference's D^2 formulation would need",
            "traffic": DRAM_TRAFFIC.get(dominant, {}).get("bytes_per_launch") and
                       DRAM_TRAFFIC[dominant]["bytes_per_launch"] * (B * H * N) / DRAM_TRAFFIC[dominant]["head_tokens"],
            "traffic_source": DRAM_TRAFFIC.get(dominant, {}).get("source"),
        }
    if order == 1:   # 33 flop per byte: bound by HBM; the whole call against its algorithmic bytes
        esz = 2 if dtype_name == "bf16" else 4
        bytes_alg = (4 if args.mode == "fwd" else 12) * B * H * N * D * esz + 4 * B * H * N
        gbs = bytes_alg / (ms_step / world * 1e-3) / 1e9 if world == 1 else bytes_alg / (ms_step * 1e-3) / 1e9
        roofline = {"kernel": "whole call (%s)" % ", ".join(sorted(kernels)), "bound": "hbm", "achieved": gbs,
                    "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": gbs / pk["hbm_gbs"], "peak_source": pk["_source"],
                    "note": "algorithmic bytes of the call (read q, k, v; write o and g) per rank / step time", "traffic": None}
    step_counted = sum(counted_flops(n)[0] * kernels[n]["launches_per_step"] for n in kernels)
    whole = {
        "flops_alg_per_step": 6.0 * U,
        "flops_counted_per_step": step_counted,
        "tflops_counted": step_counted / (ms_step * 1e-3) / 1e12,
        "frac_of_peak": step_counted / (ms_step * 1e-3) / 1e12 / pk["bf16_tflops_sustained"],
        "tflops_full_d2_equivalent": 6.0 * U / (ms_step * 1e-3) / 1e12,
    }

    # ---- end to end: public operator, pinned host buffers, H2D + D2H inside the timed region ----
    e2e = None
    if not args.no_e2e and args.mode == "fwd_bwd":
        all_cores = os.sched_getaffinity(0)
        numa = bind_host_near_gpu(torch, local_rank)   # first touch of the pinned buffers on the GPU's NUMA node
        hq, hk, hv, hdo = (x.cpu().pin_memory() for x in (q, k, v, do))
        ho = torch.zeros_like(hq).pin_memory()
        hdq, hdk, hdv = (torch.zeros_like(hq).pin_memory() for _ in range(3))
        os.sched_setaffinity(0, all_cores)
        temperature = 8.0 * math.sqrt(D)

        def e2e_step():
            dq_, dk_, dv_ = (x.to(dev, non_blocking=True) for x in (hq, hk, hv))
            ddo = hdo.to(dev, non_blocking=True)
            dq_.requires_grad_(True), dk_.requires_grad_(True), dv_.requires_grad_(True)
            o = pkg.FastMax.apply(dq_, dk_, dv_, None, None, causal, 0.0, False, temperature, 1.0, 1.0, 0.5, 1.0, order)
            o.backward(ddo)
            ho.copy_(o.detach(), non_blocking=True)
            hdq.copy_(dq_.grad, non_blocking=True)
            hdk.copy_(dk_.grad, non_blocking=True)
            hdv.copy_(dv_.grad, non_blocking=True)

        from reproducing_fastmax_results_b200.host_pipeline import HostFastmax

        host_op = HostFastmax(mask=causal, temperature=temperature, p=order, device=dev)

        def e2e_pipelined():
            host_op.forward_backward(hq, hk, hv, hdo, ho, hdq, hdk, hdv)

        def time_e2e(fn):
            for _ in range(max(1, min(args.warmup, 3))):
                fn()
            barrier()
            n = max(3, min(args.steps, 10))
            a, b2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(n):
                fn()
            b2.record()
            barrier()
            tt = torch.tensor([a.elapsed_time(b2)], device=dev, dtype=torch.float64)
            if dist is not None:
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            return float(tt.item()) / n, n

        single_ms, _ = time_e2e(e2e_step)
        e2e_ms, e2e_steps = time_e2e(e2e_pipelined)
        nbytes = q.numel() * q.element_size()
        e2e = {"value": tokens_per_step / (e2e_ms * 1e-3) / 1e6, "unit": "Mtokens/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": 4 * nbytes, "d2h_bytes_per_step": 4 * nbytes, "steps": e2e_steps,
               "api": "reproducing_fastmax_results_b200.host_pipeline.HostFastmax.forward_backward: pinned host q,k,v,dO in; "
                      "o,dq,dk,dv out to pinned host; batch slices pipelined over copy-in / compute / copy-out streams",
               "host_cores": numa or "unchanged",
               "single_call": {"value": tokens_per_step / (single_ms * 1e-3) / 1e6, "ms_per_step": single_ms,
                               "api": "FastMax.apply + backward on the whole batch between one copy-in and one copy-out"}}

    cpu = None
    if rank == 0 and not args.no_cpu and world == 1:   # the CPU leg runs at N = 1 only
        cpu = cpu_baseline_record(args.workload, args.cpu_tokens, args.cpu_heads)
        if args.workload == DEFAULT:
            try:
                cpu["config1"] = config1_record(torch, dev)
            except Exception as e:   # reported, never fatal for the headline line
                cpu["config1"] = {"error": f"{type(e).__name__}: {e}"[:300]}
            try:
                cpu["config4"] = config4_record(torch, dev)
            except Exception as e:
                cpu["config4"] = {"error": f"{type(e).__name__}: {e}"[:300]}
            try:
                cpu["score_function"] = score_function_sample(args.workload)
            except Exception as e:
                cpu["score_function"] = {"error": f"{type(e).__name__}: {e}"[:300]}

    input_mb = 4 * q.numel() * q.element_size() >> 20
    others = None
    if args.workload == DEFAULT and args.mode == "fwd_bwd" and not args.no_other and not args.no_tensor_cores:
        del q, k, v, do
        torch.cuda.empty_cache()
        others = other_workloads(args, torch, dist, dev, rank, world)

    if rank == 0:
        line = {
            "metric": "fastmax_fwd_bwd_mtokens_per_s" if args.mode == "fwd_bwd" else "fastmax_fwd_mtokens_per_s",
            "value": value, "unit": "Mtokens/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": dtype_name + " inputs, f32 accumulate", "data": "synthetic",
            "config": {"workload": args.workload, "batch_per_gpu": B, "heads": H, "seq_len": N, "head_dim": D,
                       "order": order, "causal": causal, "parallelism": f"batch x head sharding, {world} rank(s), no collective",
                       "l2": "inputs (%d MB) + workspace exceed the 126 MB L2; no explicit flush"
                             % input_mb},
            "roofline": roofline, "whole_step": whole, "kernels": kernels, "cpu_baseline": cpu, "e2e": e2e,
            "gpu_launches": int(launches), "clocks": clocks, "other_workloads": others,
        }
        emit(line)
    if dist is not None:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
