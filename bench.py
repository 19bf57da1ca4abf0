#!/usr/bin/env python
"""Benchmark of the quantized-linear hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

A step is one pass of the workload over one batch of seeded synthetic input:

  c2_mlp (default)  the Qwen-Image-shaped FP8 MLP: X bf16 [4352,3072]; up W e4m3 [12288,3072] with
                    per-row scales and GELU-tanh in the epilogue; down W e4m3 [3072,12288] with the
                    residual X added in the epilogue. Two fl_fp8_linear calls per step.
  c1_linear         one FP8 linear, X [4096,3072] x W [3072,3072] + bias.
  c3_nvfp4_qkv      the NVFP4 fused-QKV GEMM, X [4352,3072] x W [9216,3072].

`value` is whole-job TFLOP/s (2*M*N*K per GEMM, nothing else counted) with operands resident in
HBM; `e2e` is the same metric through the C ABI with the step's activation copied from pinned host
memory and the result copied back inside the timed region. With N > 1 every rank runs its own
batch (weights replicated, no collective in the data path): weak scaling.

Prints one JSON line on rank 0.
"""
from __future__ import annotations

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

METRIC = "quantized GEMM TFLOP/s"
UNIT = "TFLOP/s"

WORKLOADS = {
    # name: (m, list of (n, k)), description
    "c2_mlp": dict(m=4352, gemms=[(12288, 3072), (3072, 12288)], kind="fp8",
                   desc="FP8 MLP 4352x3072 -> 12288 (GELU-tanh) -> 3072 (+residual)"),
    "c1_linear": dict(m=4096, gemms=[(3072, 3072)], kind="fp8", desc="FP8 linear 4096x3072x3072 + bias"),
    "c3_nvfp4_qkv": dict(m=4352, gemms=[(9216, 3072)], kind="nvfp4", desc="NVFP4 fused-QKV 4352x9216x3072"),
    # handled by run_mmdit(): the whole 60-block denoise step, metric "ms per MMDiT denoise step"
    "c4_mmdit_step": dict(m=2 * 4352, gemms=[], kind="fp8",
                          desc="60-block MMDiT denoise step, hidden 3072, 24x128 heads, MLP 12288, 256+4096 tokens, batch 2"),
    # handled by run_skinny(): the reference's own decode benchmark shape (docs/fp8.md:225-244), one
    # 16-bit activation row against an e4m3 weight through the unchanged fl_fp8_matmul; HBM-bound
    "skinny_decode": dict(m=1, gemms=[(16384, 3072)], kind="fp8_upcast",
                          desc="fl_fp8_matmul 1x16384x3072, fp16 activation x e4m3 weight, one scale"),
    # handled by run_legacy(): the reference's own entry point and benchmark shapes
    # (flint/cuda/gemm_fp8_cutlass_test.cc:365-406): a half activation that is NOT narrowed against an
    # e4m3 weight with one scale and a bias, through the unchanged fl_fp8_matmul_add
    "legacy_fp8_matmul": dict(m=4096, gemms=[(12288, 3072)], kind="fp8_upcast",
                              desc="fl_fp8_matmul_add 4096x12288x3072, fp16 activation x e4m3 weight, one scale, bias"),
    # handled by run_attention(): the denoise step's joint attention through fl_attention
    "attention_step": dict(m=2 * 4352, gemms=[], kind="bf16",
                           desc="fl_attention 2 x 24 heads x 4352 tokens x 128, bf16, no mask (the denoise step's attention)"),
}

NOMINAL_PEAK = {"fp8": 4500.0, "nvfp4": 9000.0}   # dense TFLOP/s, NVIDIA's B200 figures
PEAK_MULT = {"fp8": 2.0, "nvfp4": 4.0}            # relative to the measured bf16 cuBLAS throughput
FALLBACK_BF16_TFLOPS = 1590.0

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, copied from the
# committed ncu captures (profiles/); a bench run measures none of this itself, and the line says
# so (`traffic_source`). None until a capture of that workload exists.
NCU_TRAFFIC_SOURCE = {
    "c2_mlp": "profiles/gemm_tn_kernel_fp8_c2_mlp.md",
    "legacy_fp8_matmul": "profiles/gemm_tn_kernel_mixed_legacy_fp8_matmul.md",
    "c1_linear": "profiles/gemm_tn_kernel_fp8_c2_mlp.md",
    "c3_nvfp4_qkv": "profiles/gemm_tn_kernel_nvfp4_c3_qkv.md",
    "skinny_decode": "profiles/fewrow_tc_kernel_decode_16x16384x3072.md",
    "skinny_decode_linear": "profiles/fewrow_q8_kernel_decode_16x16384x3072.md",
    "attention_step": "profiles/attention_kernel_denoise_step.md",
}


def traffic_fields(workload):
    src = NCU_TRAFFIC_SOURCE.get(workload)
    return {"traffic": NCU_TRAFFIC_BYTES.get(workload),
            "traffic_source": (f"an earlier ncu capture summarised in {src}; not measured by this run" if src else None)}


NCU_TRAFFIC_BYTES = {
    "c2_mlp": (51.9e6 + 64.5e6 + 169.5e6 + 14.9e6) / 2,  # mean of the up and the down launch
    "c1_linear": 22.1e6,                                 # the bf16 output stays dirty in L2
    "c3_nvfp4_qkv": 24.0e6 + 25.5e6,
    "skinny_decode": 50.47e6 + 0.01e6,                   # the weight once; the result stays in L2
    "skinny_decode_linear": 50.48e6,                     # the same through fl_fp8_linear (the product's launch)
    "attention_step": 160.5e6 + 32.7e6,                  # q, k, v once (K and V re-reads hit L2); the output partly stays in L2
}


def flops_per_step(wl, m=None):
    m = wl["m"] if m is None else m
    return sum(2.0 * m * n * k for (n, k) in wl["gemms"])


def algorithmic_bytes_per_step(wl):
    """Each operand once: X (bf16), W (1 B or 0.5+1/16 B), scales, Y (bf16), residual/bias."""
    m = wl["m"]
    total = 0.0
    for (n, k) in wl["gemms"]:
        wbytes = n * k * (1.0 if wl["kind"] == "fp8" else 0.5 + 1.0 / 16.0)
        total += m * k * 2 + wbytes + n * 4 + m * n * 2
    if len(wl["gemms"]) == 2:
        total += m * wl["gemms"][1][0] * 2  # the residual read
    return total


class ClockSampler(threading.Thread):
    """Samples SM clock, power and throttle reasons through NVML (read-only) while the timed
    region runs; falls back to polling nvidia-smi where NVML cannot be imported."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")
    NAMES = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]

    def __init__(self, index: int):
        super().__init__(daemon=True)
        self.index = index
        self.samples = []  # (sm_mhz, max_mhz, watts, set of reason names)
        self.stop_flag = threading.Event()
        self.nvml = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = index
            if visible:
                ids = [v for v in visible.split(",") if v.strip() != ""]
                if index < len(ids) and ids[index].strip().isdigit():
                    phys = int(ids[index])
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
        except Exception:
            self.nvml = None

    def _sample_nvml(self):
        n = self.nvml
        sm = n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)
        mx = n.nvmlDeviceGetMaxClockInfo(self.handle, n.NVML_CLOCK_SM)
        watts = n.nvmlDeviceGetPowerUsage(self.handle) / 1000.0
        try:
            mask = n.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
        except Exception:
            mask = n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
        bits = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4}
        self.samples.append((float(sm), float(mx), watts, {k for k, b in bits.items() if mask & b}))

    def _sample_smi(self):
        out = subprocess.run(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                              "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
        parts = [p.strip() for p in out.strip().split(",")]
        if len(parts) >= 7:
            reasons = {nm for i, nm in enumerate(self.NAMES) if parts[3 + i].lower().startswith("active")}
            self.samples.append((float(parts[0]), float(parts[1]), float(parts[2]), reasons))

    def run(self):
        while not self.stop_flag.is_set():
            try:
                if self.nvml is not None:
                    self._sample_nvml()
                else:
                    self._sample_smi()
            except Exception:
                pass
            self.stop_flag.wait(0.02)

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        watts = [s[2] for s in self.samples]
        cut = statistics.median(watts)
        loaded = [s[0] for s in self.samples if s[2] >= cut] or [s[0] for s in self.samples]
        reasons = sorted(set().union(*[s[3] for s in self.samples]))
        return {"sm_mhz": statistics.median(loaded), "sm_max_mhz": max(s[1] for s in self.samples),
                "reasons": reasons, "samples": len(self.samples), "power_w_max": max(watts)}


def bind_by_nvml_affinity(bus):
    """Where sysfs names no NUMA node for the GPU (a virtual machine), the driver may still know the
    CPUs nearest to it: NVML's ideal CPU set for the device, read only, intersected with the CPUs
    this process may use."""
    allowed_now = set(os.sched_getaffinity(0))
    try:
        import pynvml
        pynvml.nvmlInit()
        try:
            handle = pynvml.nvmlDeviceGetHandleByPciBusId(bus.encode())
            words = pynvml.nvmlDeviceGetCpuAffinity(handle, (max(allowed_now) // 64) + 1)
        finally:
            pynvml.nvmlShutdown()
        cpus = {64 * i + b for i, w in enumerate(words) for b in range(64) if (int(w) >> b) & 1}
        allowed = cpus & allowed_now
        if not allowed or allowed == allowed_now:
            return f"the GPU reports no NUMA node and the driver's ideal CPU set does not narrow this process's {len(allowed_now)} CPUs; not bound"
        os.sched_setaffinity(0, allowed)
        return f"pinned buffers allocated from the driver's ideal CPU set for the GPU ({len(allowed)} of {len(allowed_now)} CPUs)"
    except Exception as e:
        return f"the GPU reports no NUMA node; not bound ({len(allowed_now)} CPUs, NVML: {type(e).__name__})"


def bind_to_gpu_numa_node(local_index):
    """Best effort: runs this process on the CPUs of the NUMA node its GPU hangs off, so that the
    page-locked buffers allocated afterwards are local to the GPU's PCIe root (eight ranks copying
    through one socket's memory is what limits end-to-end scaling). Returns a short description."""
    try:
        import torch
        props = torch.cuda.get_device_properties(local_index)
        bus = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{bus}/numa_node") as f:
            node = int(f.read().strip())
        if node < 0:
            return bind_by_nvml_affinity(bus)
        with open(f"/sys/devices/system/node/node{node}/cpulist") as f:
            text = f.read().strip()
        cpus = set()
        for part in text.split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & set(os.sched_getaffinity(0))
        if not allowed:
            return f"NUMA node {node} has no CPU this process may use; not bound"
        os.sched_setaffinity(0, allowed)
        return f"pinned buffers allocated from NUMA node {node} ({len(allowed)} CPUs), the GPU's own"
    except Exception as e:  # no sysfs, no permission: the run goes on unbound
        return f"not bound ({type(e).__name__})"


def measured_peaks(clocks=None):
    """(bf16 TFLOP/s, HBM GB/s, label). The bf16 figure is the burst one for a kernel timed at full
    clock and the sustained one when the clock record of the timed region shows the run sitting
    under the power cap (median SM clock below 0.9 of the maximum with sw_power_cap active), which
    is how the sustained figure itself was measured."""
    capped = bool(clocks) and "sw_power_cap" in (clocks.get("reasons") or []) and \
        (clocks.get("sm_mhz") or 0) < 0.9 * (clocks.get("sm_max_mhz") or 1)
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        burst = float(d.get("bf16_tflops", FALLBACK_BF16_TFLOPS))
        if capped and d.get("bf16_tflops_sustained"):
            return float(d["bf16_tflops_sustained"]), float(d.get("hbm_gbs", 6650.0)), "measured, sustained (power-capped run)"
        return burst, float(d.get("hbm_gbs", 6650.0)), "measured, burst"
    return FALLBACK_BF16_TFLOPS, 6650.0, "fallback"


# ------------------------------------------------------------------------------------------------
# the reference arm: the reference's own CPU float32 GEMM over dequantised operands
# ------------------------------------------------------------------------------------------------

def cpu_reference_step_factory(wl, rows):
    """Builds a closure that runs one bounded-sample step on the host cores and returns nothing.
    The product is fl_matmul of the reference's CPU build when it was compiled (kind "reference"),
    else the C port of the oracle (kind "port")."""
    import numpy as np
    from oracle import oracle as O
    O.lib()
    kind = "reference" if O.have_ref() else "port"
    rng = np.random.default_rng(0)
    x = O.narrow(rng.standard_normal((rows, wl["gemms"][0][1])).astype(np.float32), wl["kind"] != "fp8_upcast")
    weights = []
    for (n, k) in wl["gemms"]:
        w = (rng.standard_normal((n, k)) * 0.02).astype(np.float32)
        if wl["kind"] == "fp8_upcast":
            codes, scale = O.quantize_fp8_tensor(w)
            weights.append((O.decode_e4m3(codes), scale))
        elif wl["kind"] == "fp8":
            codes, scales = O.quantize_fp8_rows(w)
            weights.append((O.decode_e4m3(codes), scales))
        else:
            codes, sf, g = O.quantize_nvfp4_weight(w)
            weights.append((O.decode_nvfp4(codes, sf), g))

    def step():
        if wl["kind"] == "fp8_upcast":
            (wdec, scale), = weights
            acc = O.gemm_f32_nt(O.widen(x, False), wdec, kind)
            O.epilogue(acc, None, None, float(scale[0]), None, None, O.ACT_NONE, False)
        elif wl["kind"] == "fp8":
            cur = x
            for i, (wdec, scales) in enumerate(weights):
                xc, xs = O.quantize_fp8_act(cur, True)
                acc = O.gemm_f32_nt(O.decode_e4m3(xc), wdec, kind)
                last = i == len(weights) - 1
                act = O.ACT_GELU_TANH if (len(weights) == 2 and i == 0) else O.ACT_NONE
                res = x if (len(weights) == 2 and last) else None
                cur = O.epilogue(acc, xs, scales, 1.0, None, res, act, True)
        else:
            (wdec, g), = weights
            xc, xsf = O.quantize_nvfp4_act(x, True)
            acc = O.gemm_f32_nt(O.decode_nvfp4(xc, xsf), wdec, kind)
            O.epilogue(acc, None, None, float(g[0]), None, None, O.ACT_NONE, True)

    cores = os.cpu_count() or 1
    try:
        cores = len(os.sched_getaffinity(0))
    except Exception:
        pass
    return step, kind, cores


def run_reference(args, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torchrun pins every rank to one OpenMP thread; the reference arm is rank 0 alone with all the
    # host cores it may use, so say so before the reference's library starts its OpenMP runtime.
    try:
        os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))
    except Exception:
        os.environ.pop("OMP_NUM_THREADS", None)
    rows = min(wl["m"], args.reference_rows)
    step, kind, cores = cpu_reference_step_factory(wl, rows)
    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = time.perf_counter() - t0
    ms = dt * 1e3 / args.steps
    value = flops_per_step(wl, rows) / (ms * 1e-3) / 1e12
    sample = f"{rows} of {wl['m']} rows per step, whole step on the host (quantise, fp32 GEMM, epilogue)"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "what": wl["desc"], "sample": sample},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# our arm
# ------------------------------------------------------------------------------------------------

def run_ours(args, wl):
    import torch
    from libwaifu_b200 import flint as F

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    F.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if not F.fp8_available():
        raise RuntimeError("the CUDA path is unavailable on this device; there is no fallback")

    bf = F.DType.BFLOAT16
    m = wl["m"]
    sets = args.rotate
    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)

    def wrap(t, dt, shape=None):
        return F.Tensor.from_device_ptr(t.data_ptr(), tuple(shape or t.shape), dt, keepalive=t)

    # operand sets that rotate so that no operand survives in L2 from one step to the next
    operand_sets = []
    for _ in range(sets):
        x = torch.randn(m, wl["gemms"][0][1], device="cuda", dtype=torch.bfloat16, generator=gen)
        layers = []
        for (n, k) in wl["gemms"]:
            w = torch.randn(n, k, device="cuda", dtype=torch.float32, generator=gen) * 0.02
            if wl["kind"] == "fp8":
                codes, scales = F.quantize_fp8_rows(wrap(w, F.DType.FLOAT))
                layers.append((codes, scales))
            else:
                codes, sf, g = F.quantize_nvfp4(wrap(w, F.DType.FLOAT))
                layers.append((codes, sf, g))
            F.synchronize()
            del w
        bias = None
        if args.workload == "c1_linear":
            b = torch.randn(wl["gemms"][0][0], device="cuda", dtype=torch.bfloat16, generator=gen) * 0.01
            bias = wrap(b, bf)
        operand_sets.append((wrap(x, bf), layers, bias))
    outs = [F.Tensor.empty((m, n), bf) for (n, _) in wl["gemms"]]

    nsplit = args.parallel in ("nsplit", "nsplit_push", "nsplit_fp8", "nsplit_fp8_nccl")

    def build_split(mode):
        """Strong scaling of one MLP: every rank holds a slice of each weight's output channels and
        multiplies the whole activation by it. `mode` says how H and Y reach every rank:
          nsplit       NCCL all-gathers of the 16-bit slices;
          nsplit_push  the GEMMs' epilogues write their column blocks into every rank's full-width H
                       and Y over NVLink (peer-mapped storage);
          nsplit_fp8   H crosses as e4m3 codes: the up GEMM's epilogue leaves the rows' maxima, the
                       library's exchange kernel makes them the whole rows' over peer-mapped
                       mailboxes, a quantise-and-scatter kernel writes the codes to every rank, the
                       down GEMM reads codes and scatters Y; the same exchange kernel is the barrier
                       after each scatter (no library collective inside the step);
          nsplit_fp8_nccl  the same with NCCL all-reduces in place of the exchange kernel.
        The 16-bit push orders the ranks with a one-element all-reduce on the stream after each
        scatter. Returns the step and the tensor the result lands in."""
        from libwaifu_b200 import sharding
        (n_up, k_up), (n_dn, k_dn) = wl["gemms"]
        up_a, up_b = sharding.column_shard(n_up, world, rank, 128)
        dn_a, dn_b = sharding.column_shard(n_dn, world, rank, 128)
        up_sizes = sharding.column_sizes(n_up, world, 128)
        dn_sizes = sharding.column_sizes(n_dn, world, 128)
        g2 = torch.Generator(device="cuda").manual_seed(77)
        g3 = torch.Generator(device="cuda").manual_seed(4321 + rank)
        x_t = torch.randn(m, k_up, device="cuda", dtype=torch.bfloat16, generator=g2)
        x_cols_t = x_t[:, dn_a:dn_b].contiguous()
        w_up = torch.randn(up_b - up_a, k_up, device="cuda", dtype=torch.float32, generator=g3) * 0.02
        w_dn = torch.randn(dn_b - dn_a, k_dn, device="cuda", dtype=torch.float32, generator=g3) * 0.02
        up_q = F.quantize_fp8_rows(wrap(w_up, F.DType.FLOAT))
        dn_q = F.quantize_fp8_rows(wrap(w_dn, F.DType.FLOAT))
        F.synchronize()
        del w_up, w_dn
        h_loc_t = torch.empty(m, up_b - up_a, device="cuda", dtype=torch.bfloat16)
        x_w, x_cols_w, h_loc_w = wrap(x_t, bf), wrap(x_cols_t, bf), wrap(h_loc_t, bf)
        if mode == "nsplit":
            h_t = torch.empty(m, n_up, device="cuda", dtype=torch.bfloat16)
            y_loc_t = torch.empty(m, dn_b - dn_a, device="cuda", dtype=torch.bfloat16)
            y_t = torch.empty(m, n_dn, device="cuda", dtype=torch.bfloat16)
            h_w, y_loc_w = wrap(h_t, bf), wrap(y_loc_t, bf)

            def split_step():
                F.fp8_linear(x_w, up_q[0], up_q[1], None, None, F.ACT_GELU_TANH, h_loc_w)
                sharding.all_gather_columns(dist, h_loc_t, up_sizes, h_t)
                F.fp8_linear(h_w, dn_q[0], dn_q[1], None, x_cols_w, F.ACT_NONE, y_loc_w)
                sharding.all_gather_columns(dist, y_loc_t, dn_sizes, y_t)
            return split_step, wrap(y_t, bf), x_w, (h_t, y_t, y_loc_t)

        # memory of its own (not the pool's): the only kind another process can map
        h_dtype = F.DType.FP8E4M3 if mode.startswith("nsplit_fp8") else bf
        h_own = F.Tensor.empty((m, n_up), h_dtype, hint=F.AllocHint.WEIGHT)
        y_own = F.Tensor.empty((m, n_dn), bf, hint=F.AllocHint.WEIGHT)
        handles = [None] * world
        dist.all_gather_object(handles, (F.ipc_export(h_own), F.ipc_export(y_own)))
        h_dests, y_dests = [h_own], [y_own]
        for r in range(world):
            if r != rank:
                h_dests.append(F.ipc_import(handles[r][0], (m, n_up), h_dtype))
                y_dests.append(F.ipc_import(handles[r][1], (m, n_dn), bf))
        flag = torch.zeros(1, device="cuda", dtype=torch.float32)
        if mode == "nsplit_push":
            def split_step():
                F.fp8_linear_scatter(x_w, up_q[0], up_q[1], h_dests, up_a, None, None, F.ACT_GELU_TANH)
                dist.all_reduce(flag)
                F.fp8_linear_scatter(h_own, dn_q[0], dn_q[1], y_dests, dn_a, None, x_cols_w, F.ACT_NONE)
                dist.all_reduce(flag)
            return split_step, y_own, x_w, (h_dests, y_dests, flag)

        amax_t = torch.zeros(m, device="cuda", dtype=torch.float32)
        scales_t = torch.zeros(m, device="cuda", dtype=torch.float32)
        amax_w, scales_w = wrap(amax_t, F.DType.FLOAT), wrap(scales_t, F.DType.FLOAT)

        def all_gather_handles(mine):
            every = [None] * world
            dist.all_gather_object(every, mine)
            return every

        group = F.PeerGroup(rank, world, m, all_gather_handles)
        if mode == "nsplit_fp8_nccl":
            def split_step():
                F.fp8_linear_amax(x_w, up_q[0], up_q[1], amax_w, None, None, F.ACT_GELU_TANH, h_loc_w)
                dist.all_reduce(amax_t, op=dist.ReduceOp.MAX)
                F.fp8_quantize_scatter(h_loc_w, amax_w, h_dests, up_a, scales_w)
                dist.all_reduce(flag)
                F.fp8_linear_quantized_scatter(h_own, scales_w, dn_q[0], dn_q[1], y_dests, dn_a, None, x_cols_w, F.ACT_NONE)
                dist.all_reduce(flag)
        else:
            def split_step():
                F.fp8_linear_amax(x_w, up_q[0], up_q[1], amax_w, None, None, F.ACT_GELU_TANH, h_loc_w)
                group.exchange(amax_w)       # the rows' maxima over all ranks
                F.fp8_quantize_scatter(h_loc_w, amax_w, h_dests, up_a, scales_w)
                group.exchange()             # every rank's codes have landed
                F.fp8_linear_quantized_scatter(h_own, scales_w, dn_q[0], dn_q[1], y_dests, dn_a, None, x_cols_w, F.ACT_NONE)
                group.exchange()             # every rank's block of Y has landed
        return split_step, y_own, x_w, (h_dests, y_dests, flag, amax_t, scales_t, h_loc_t, group)

    SPLIT_WORDS = {
        "nsplit": "NCCL all-gather of H and Y in 16 bits",
        "nsplit_push": "epilogues push H and Y (16 bits) to peers over NVLink",
        "nsplit_fp8": "H crosses as e4m3 codes (row maxima and barriers by the library's exchange kernel over peer mailboxes, "
                      "quantise-and-scatter kernel), the down GEMM's epilogue pushes Y",
        "nsplit_fp8_nccl": "H crosses as e4m3 codes (row maxima and barriers by NCCL all-reduces, quantise-and-scatter kernel), "
                           "the down GEMM's epilogue pushes Y",
    }
    if nsplit:
        if not (wl["kind"] == "fp8" and len(wl["gemms"]) == 2 and dist is not None):
            raise SystemExit("--parallel nsplit* needs the c2_mlp workload and more than one GPU")
        nsplit_step, split_result, x_w, split_keep = build_split(args.parallel)

    def step(i, x_override=None, alloc=False):
        """One step on operand set i. `alloc`: the outputs are allocated by the call, as the
        reference's wrapper allocates `out` for every linear (waifu/src/flint/functional.rs:655-680),
        and the last one is returned; otherwise they land in buffers made once."""
        if nsplit:
            nsplit_step()
            return None
        x, layers, bias = operand_sets[i % sets]
        if x_override is not None:
            x = x_override
        o = [None] * len(layers) if alloc else outs
        if x_override is not None and x.shape[0] != m and not alloc:
            raise ValueError("a row chunk needs per-call outputs")
        if wl["kind"] == "nvfp4":
            codes, sf, g = layers[0]
            return F.nvfp4_linear(x, codes, sf, g, None, None, F.ACT_NONE, o[0])
        if len(layers) == 2:
            h = F.fp8_linear(x, layers[0][0], layers[0][1], None, None, F.ACT_GELU_TANH, o[0])
            return F.fp8_linear(h, layers[1][0], layers[1][1], None, x, F.ACT_NONE, o[1])
        return F.fp8_linear(x, layers[0][0], layers[0][1], bias, None, F.ACT_NONE, o[0])

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if dist is None:
            return ms
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- device-resident timing ----------------------------------------------------------------
    for i in range(args.warmup):
        step(i)
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    launches0 = F.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        step(args.warmup + i)
    e1.record()
    barrier()
    ms_total = e0.elapsed_time(e1)
    launches = F.launch_count() - launches0
    F.synchronize()
    ms_step = max_over_ranks(ms_total / args.steps)
    work_units = 1 if nsplit else world  # nsplit: one MLP shared by all ranks (strong scaling)
    value = work_units * flops_per_step(wl) / (ms_step * 1e-3) / 1e12

    # ---- the same K steps again with every GEMM launch bracketed by its own events -------------
    # (kept out of the region above: an event between two kernels stops the second from starting
    # its prologue under the first one's tail, which the steady-state figure should include)
    F.gemm_timing(True)
    F.gemm_timing_read()
    for i in range(args.steps):
        step(args.warmup + i)
    gemm_ms, gemm_launches = F.gemm_timing_read()
    F.gemm_timing(False)
    sampler.stop_flag.set()
    sampler.join(timeout=5)

    # ---- the same K steps with every output allocated by its call (the reference wrapper's way) ----
    alloc_check = None
    if not nsplit:
        for i in range(3):
            step(i, alloc=True)
        barrier()
        e0.record()
        for i in range(args.steps):
            step(args.warmup + i, alloc=True)
        e1.record()
        barrier()
        alloc_ms = max_over_ranks(e0.elapsed_time(e1) / args.steps)
        alloc_check = {"ms_per_step": alloc_ms, "value": work_units * flops_per_step(wl) / (alloc_ms * 1e-3) / 1e12,
                       "ratio_to_preallocated": ms_step / alloc_ms,
                       "what": "out allocated per call by fl_tensor_data_create (stream-ordered pool) and destroyed after, "
                               "as waifu/src/flint/functional.rs:655-680 does"}

    # ---- a second of back-to-back steps: the power-capped regime a 20-step region cannot show ------
    sustained = None
    if not nsplit and args.sustained_seconds > 0:
        n_sus = max(args.steps, int(args.sustained_seconds * 1e3 / ms_step) + 1)
        sus_sampler = ClockSampler(local)
        sus_sampler.start()
        barrier()
        e0.record()
        for i in range(n_sus):
            step(i)
        e1.record()
        barrier()
        sus_ms = max_over_ranks(e0.elapsed_time(e1) / n_sus)
        F.gemm_timing(True)
        F.gemm_timing_read()
        for i in range(n_sus):
            step(i)
        sus_gemm_ms, sus_gemm_launches = F.gemm_timing_read()
        F.gemm_timing(False)
        sus_sampler.stop_flag.set()
        sus_sampler.join(timeout=5)
        sus_clocks = sus_sampler.summary()
        sus_bf16, _, sus_kind = measured_peaks(sus_clocks)
        sus_tflops = flops_per_step(wl) * n_sus / (sus_gemm_ms * 1e-3) / 1e12 if sus_gemm_ms > 0 else None
        sustained = {"steps": n_sus, "ms_per_step": sus_ms, "value": work_units * flops_per_step(wl) / (sus_ms * 1e-3) / 1e12,
                     "achieved": sus_tflops, "peak": PEAK_MULT[wl["kind"]] * sus_bf16,
                     "frac": sus_tflops / (PEAK_MULT[wl["kind"]] * sus_bf16) if sus_tflops else None,
                     "frac_of_nominal": sus_tflops / NOMINAL_PEAK[wl["kind"]] if sus_tflops else None,
                     "peak_source": f"{PEAK_MULT[wl['kind']]:.0f} x bf16 cuBLAS, of {sus_kind}", "launches": sus_gemm_launches,
                     "clocks": sus_clocks}

    # ---- end to end through the C ABI with host buffers ----------------------------------------
    # The step's rows are cut into chunks and pipelined: every chunk's upload is started at once
    # (fl_transfer_async: page-locked memory, the upload stream), chunk j's linears wait for chunk
    # j's upload only (fl_transfer_wait), run while chunk j+1 is still crossing, and hand their
    # result to the download stream (fl_sm100_transfer_to_host_async) while chunk j+1 computes.
    # The host waits once, for the last download. Every device tensor of the step -- the uploaded
    # rows, H, Y -- is allocated by the call that produces it and destroyed at the end of the step.
    k0 = wl["gemms"][0][1]
    n_last = wl["gemms"][-1][0]
    affinity = os.sched_getaffinity(0)
    bind_note = bind_to_gpu_numa_node(local)
    depth = 1 if nsplit else max(1, args.e2e_depth)   # steps in flight: page-locked buffers each way
    host_xs = [F.Tensor.empty((m, k0), bf, F.Device.CUDA_HOST) for _ in range(depth)]
    host_ys = [F.Tensor.empty((m, n_last), bf, F.Device.CUDA_HOST) for _ in range(depth)]
    os.sched_setaffinity(0, affinity)  # only the allocation (and its first touch) needed the binding
    result = split_result if nsplit else None
    import ctypes
    import numpy as np
    for j, hx_t in enumerate(host_xs):
        p = ctypes.c_void_p()
        F.check(F.lib().fl_tensor_data_get_host_ptr(hx_t._data, ctypes.byref(p)))
        hx = np.ctypeslib.as_array(ctypes.cast(p.value, ctypes.POINTER(ctypes.c_uint16)), shape=(m * k0,))
        hx[:] = (np.random.default_rng(7 + rank + 100 * j).standard_normal(m * k0).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    ops = F.operators()
    chunks = 1 if nsplit else max(1, min(args.e2e_chunks, m // 128))
    bounds = [min(m, ((m * c // chunks) + 255) // 256 * 256) for c in range(chunks)] + [m]  # whole 256-row tiles
    bounds[0] = 0
    bounds = sorted(set(bounds))
    chunks = len(bounds) - 1
    x_chunks = [[hx_t.view_as((bounds[c + 1] - bounds[c], k0), (k0, 1), bounds[c] * k0) for c in range(chunks)] for hx_t in host_xs]
    y_chunks = [[hy_t.view_as((bounds[c + 1] - bounds[c], n_last), (n_last, 1), bounds[c] * n_last) for c in range(chunks)]
                for hy_t in host_ys]

    def e2e_issue(i):
        """Starts step i: every chunk's upload at once, chunk j's linears behind chunk j's upload
        only, its result handed to the download stream. Returns what the step's end waits for."""
        if nsplit:
            F.check(F.lib().fl_transfer(ops, host_xs[0].raw(), x_w.raw()))
            step(i)
            F.check(F.lib().fl_transfer(ops, result.raw(), host_ys[0].raw()))  # synchronises
            return None
        uploads = [F.transfer_async(xc) for xc in x_chunks[i % depth]]
        downloads, alive = [], []
        for c in range(chunks):
            xd, pending = uploads[c]
            pending.wait()
            y = step(i, x_override=xd, alloc=True)
            downloads.append(F.transfer_to_host_async(y, y_chunks[i % depth][c]))
            alive.append((xd, y))
        return downloads, alive

    def e2e_finish(token):
        """The host has step i's result: its downloads are complete (in order on their stream)."""
        if token is not None:
            for d in reversed(token[0]):
                d.wait_sync()

    def e2e_run(n_steps):
        # Two steps in flight: step i + 1 is started (its uploads cross while step i computes and
        # step i - 1's result goes back) before the host waits for step i's result, as a caller with
        # a queue of requests would; each step's copies, both ways, are inside the timed region.
        in_flight = []
        for i in range(n_steps):
            in_flight.append(e2e_issue(i))
            if len(in_flight) >= depth:
                e2e_finish(in_flight.pop(0))
        while in_flight:
            e2e_finish(in_flight.pop(0))

    e2e_steps = max(4, min(args.steps, 20))
    e2e_run(3)
    barrier()
    e0.record()
    e2e_run(e2e_steps)
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1) / e2e_steps)
    e2e_value = work_units * flops_per_step(wl) / (e2e_ms * 1e-3) / 1e12
    # the same with one step at a time (the host waits for a step's result before it starts the next)
    e2e_serial_ms = None
    if not nsplit:
        depth_keep, depth = depth, 1
        e2e_run(2)
        barrier()
        e0.record()
        e2e_run(e2e_steps)
        e1.record()
        barrier()
        e2e_serial_ms = max_over_ranks(e0.elapsed_time(e1) / e2e_steps)
        depth = depth_keep

    # ---- roofline of the dominant kernel (the tcgen05 GEMM), from its own events ---------------
    clocks = sampler.summary()
    bf16_peak, hbm_peak, peak_kind = measured_peaks(clocks)
    peak = PEAK_MULT[wl["kind"]] * bf16_peak
    gemm_tflops = (flops_per_step(wl) / (world if nsplit else 1)) * args.steps / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None
    roofline = {
        "bound": "tensor", "kernel": "gemm_tn_kernel", "achieved": gemm_tflops, "peak": peak, "unit": UNIT,
        "frac": (gemm_tflops / peak) if gemm_tflops else None,
        "peak_source": f"{PEAK_MULT[wl['kind']]:.0f} x bf16 cuBLAS, of {peak_kind}",
        "frac_of_nominal": (gemm_tflops / NOMINAL_PEAK[wl["kind"]]) if gemm_tflops else None,
        "nominal_peak": NOMINAL_PEAK[wl["kind"]],
        "launches": gemm_launches, "avg_launch_ms": gemm_ms / gemm_launches if gemm_launches else None,
        **traffic_fields(args.workload), "algorithmic_bytes_per_step": algorithmic_bytes_per_step(wl),
        "sustained": sustained,
    }

    # ---- CPU baseline on a bounded sample (rank 0, N = 1 only) ---------------------------------
    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        rows = min(m, args.reference_rows)
        cstep, kind, cores = cpu_reference_step_factory(wl, rows)
        cstep()
        best = None
        for _ in range(3):
            t0 = time.perf_counter()
            cstep()
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        cpu_baseline = {"value": flops_per_step(wl, rows) / best / 1e12, "unit": UNIT, "cores": cores, "kind": kind,
                        "sample": f"{rows} of {m} rows, whole step on the host, best of 3"}

    # ---- the same MLP once more, split over the ranks by output channel (strong scaling) ----------
    strong = None
    if dist is not None and not nsplit and wl["kind"] == "fp8" and len(wl["gemms"]) == 2 and not args.no_strong_scaling:
        del operand_sets[1:]
        try:
            split_step, _, _, split_keep = build_split("nsplit_fp8")
            for _ in range(max(3, args.warmup)):
                split_step()
            barrier()
            e0.record()
            for _ in range(args.steps):
                split_step()
            e1.record()
            barrier()
            split_ms = max_over_ranks(e0.elapsed_time(e1) / args.steps)
            strong = {"ms_per_step": split_ms, "one_gpu_ms_per_step": ms_step, "speedup_over_one_gpu": ms_step / split_ms,
                      "value": flops_per_step(wl) / (split_ms * 1e-3) / 1e12, "unit": UNIT, "rows": m,
                      "how": f"one MLP of {m} rows, weights split by output channel x{world}: {SPLIT_WORDS['nsplit_fp8']}; "
                             "bit-identical to the unsplit MLP; one_gpu_ms_per_step is this run's own step (every rank the whole MLP)"}
        except Exception as e:  # the weak-scaling line above stands on its own (what fails here fails on every rank alike)
            strong = {"error": f"{type(e).__name__}: {e}"[:300]}

    if rank == 0:
        touched = sets * (m * k0 * 2 + sum(n * k * (1 if wl["kind"] == "fp8" else 0.5625) for (n, k) in wl["gemms"]))
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "strong" if nsplit else "weak",
            "vs_baseline": None,
            "dtype": "e4m3" if wl["kind"] == "fp8" else "e2m1", "data": "synthetic",
            "config": {"workload": args.workload, "what": wl["desc"], "m_per_gpu": m,
                       "parallelism": (f"weights split by output channel x{world}, {SPLIT_WORDS[args.parallel]}"
                                       if nsplit else f"batch-sharded x{world}, weights replicated, no collective"),
                       "l2": f"{sets} rotating operand sets ({touched / 1e6:.0f} MB of inputs) > 126 MB L2",
                       "accumulate": "fp32", "out": "bf16"},
            "e2e": {"value": e2e_value, "unit": UNIT, "ms_per_step": e2e_ms, "h2d_bytes_per_step": m * k0 * 2,
                    "d2h_bytes_per_step": m * n_last * 2, "steps": e2e_steps, "chunks": chunks,
                    "steps_in_flight": depth, "one_step_at_a_time_ms": e2e_serial_ms,
                    "how": "rows in chunks: uploads on a copy stream (fl_transfer_async), linears per chunk behind "
                           "fl_transfer_wait, downloads on a second copy stream; outputs allocated per call; the next step is "
                           "started before the host waits for a step's result (steps_in_flight page-locked buffers each way); "
                           "one_step_at_a_time_ms is the same with one step in flight",
                    "host_memory": bind_note},
            "per_call_alloc": alloc_check,
            "strong_scaling": strong,
            "gpu_launches": launches,
            "clocks": sampler.summary(),
            "roofline": roofline,
            "cpu_baseline": cpu_baseline,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def mmdit_cpu_sample(steps_hint=1):
    """The CPU side of the c4 workload on a bounded sample: one block of the sixty on one of the two
    classifier-free-guidance rows (4352 tokens) at the benchmark's widths, plus the linears around
    the blocks for that row, through the oracle's restated quantisers with the reference's own CPU
    fl_matmul and fl_attention (oracle/_ref) doing the products where that library was built.
    Blocks and batch rows cost the same each, so a step is (block x 60 + outer) x 2.
    Returns (closure that runs the sample and returns (block seconds, outer seconds), kind, cores, text)."""
    import torch
    from oracle import oracle as O
    from oracle.mmdit_oracle import OracleBackend
    from libwaifu_b200.mmdit import MMDiT, MMDiTConfig
    O.lib()
    kind = "reference" if O.have_ref() else "port"
    cfg = MMDiTConfig(blocks=1, batch=1)
    model = MMDiT(cfg, OracleBackend(O), seed=0, cpu_init=True)
    g = torch.Generator().manual_seed(3)
    tokens = torch.randn(1, cfg.image_tokens, cfg.latent_channels, generator=g).bfloat16()
    context = torch.randn(1, cfg.text_tokens, cfg.context_size, generator=g).bfloat16()
    sinusoid = torch.randn(1, cfg.timestep_embed_dim, generator=g).bfloat16()

    def sample():
        with torch.no_grad():
            t0 = time.perf_counter()
            x, emb = model.embed(tokens, context, sinusoid)
            t1 = time.perf_counter()
            x = model.blocks(x, emb)
            t2 = time.perf_counter()
            model.final(x, emb)
            t3 = time.perf_counter()
        return t2 - t1, (t1 - t0) + (t3 - t2)

    cores = os.cpu_count() or 1
    try:
        cores = len(os.sched_getaffinity(0))
    except Exception:
        pass
    text = ("1 of 60 blocks and the outer linears on 1 of the 2 batch rows (4352 tokens) at the benchmark's widths, "
            "whole sample on the host (quantisers, fp32 GEMMs, fp32 attention, norms); a step is (block x 60 + outer) x 2")
    return sample, kind, cores, text


def run_mmdit_reference(args):
    """The reference arm of c4_mmdit_step: the CPU sample above, timed per step and extrapolated."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    try:
        os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))
    except Exception:
        os.environ.pop("OMP_NUM_THREADS", None)
    sample, kind, cores, text = mmdit_cpu_sample()
    for _ in range(args.warmup):
        sample()
    block_s = outer_s = 0.0
    t0 = time.perf_counter()
    for _ in range(args.steps):
        b, o = sample()
        block_s += b
        outer_s += o
    sample_ms = (time.perf_counter() - t0) * 1e3 / args.steps
    step_ms = (block_s * 60 + outer_s) * 2 / args.steps * 1e3
    line = {
        "impl": "reference", "metric": "ms per MMDiT denoise step", "value": step_ms, "unit": "ms", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sample_ms, "higher_is_better": False, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "c4_mmdit_step", "what": WORKLOADS["c4_mmdit_step"]["desc"], "sample": text,
                   "extrapolated": "value = (block time x 60 + outer time) x 2 from the timed sample; ms_per_step is the sample's own time"},
        "cpu_baseline": {"value": step_ms, "unit": "ms", "cores": cores, "kind": kind, "sample": text},
        "e2e": {"value": step_ms, "unit": "ms", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def run_mmdit(args):
    """The C4 workload: ms per denoise step of the 60-block MMDiT, every linear on the FP8 path and
    every kernel of a block this library's own (fl_attention included; torch's attention is timed
    beside it as a yardstick). N > 1: every rank runs its own batch."""
    import torch
    from libwaifu_b200 import flint as F
    from libwaifu_b200.mmdit import MMDiT, MMDiTConfig, FlintBackend

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    F.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist_mod
        dist = dist_mod
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    cfg = MMDiTConfig()
    if args.blocks:
        cfg.blocks = args.blocks
    backend = FlintBackend(args.attention)
    model = MMDiT(cfg, backend, seed=0)
    g = torch.Generator(device="cuda").manual_seed(1 + rank)
    tokens = torch.randn(cfg.batch, cfg.image_tokens, cfg.latent_channels, device="cuda", dtype=torch.bfloat16, generator=g)
    context = torch.randn(cfg.batch, cfg.text_tokens, cfg.context_size, device="cuda", dtype=torch.bfloat16, generator=g)
    sinusoid = torch.randn(cfg.batch, cfg.timestep_embed_dim, device="cuda", dtype=torch.bfloat16, generator=g)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(steps):
            model.step(tokens, context, sinusoid)
        e1.record()
        barrier()
        return e0.elapsed_time(e1) / steps

    with torch.no_grad():
        for _ in range(args.warmup):
            model.step(tokens, context, sinusoid)
        barrier()
        sampler = ClockSampler(local)
        sampler.start()
        launches0 = F.launch_count()
        ms = timed(args.steps)
        launches = F.launch_count() - launches0
        F.gemm_timing(True)
        F.gemm_timing_read()
        model.step(tokens, context, sinusoid)
        gemm_ms, gemm_launches = F.gemm_timing_read()
        F.gemm_timing(False)
        sampler.stop_flag.set()
        sampler.join(timeout=5)
        # the other attention kernel beside it, a few steps
        other = "sdpa" if args.attention == "flint" else "flint"
        backend.attention_kernel = other
        model.step(tokens, context, sinusoid)
        other_ms = timed(max(2, min(args.steps, 3)))
        backend.attention_kernel = args.attention
        # end to end: latent tokens, prompt states and sinusoid from pinned host memory, the velocity back
        host_in = [t.cpu().pin_memory() for t in (tokens, context, sinusoid)]
        hy = torch.empty(cfg.batch, cfg.image_tokens, cfg.latent_channels, dtype=torch.bfloat16).pin_memory()
        for _ in range(2):
            model.step(*[t.cuda(non_blocking=True) for t in host_in])
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        e2e_steps = max(2, min(args.steps, 5))
        for _ in range(e2e_steps):
            y = model.step(*[t.cuda(non_blocking=True) for t in host_in])
            hy.copy_(y, non_blocking=False)
        e1.record()
        barrier()
        e2e_ms = e0.elapsed_time(e1) / e2e_steps
    if dist is not None:
        t = torch.tensor([ms, e2e_ms, other_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, e2e_ms, other_ms = float(t[0]), float(t[1]), float(t[2])
    bf16_peak, _, peak_kind = measured_peaks(sampler.summary())
    gemm_tflops = cfg.gemm_flops() / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sample, kind, cores, text = mmdit_cpu_sample()
        best = None
        for _ in range(2):
            b, o = sample()
            step_ms = (b * 60 + o) * 2 * 1e3
            best = step_ms if best is None else min(best, step_ms)
        cpu_baseline = {"value": best, "unit": "ms", "cores": cores, "kind": kind, "sample": text + "; best of 2"}

    if rank == 0:
        names = {"flint": "fl_attention (this library), bf16", "sdpa": "torch SDPA (a library kernel), bf16"}
        line = {
            "metric": "ms per MMDiT denoise step", "value": ms, "unit": "ms", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": False, "scaling": "weak", "vs_baseline": None,
            "dtype": "e4m3", "data": "synthetic",
            "config": {"workload": "c4_mmdit_step", "what": WORKLOADS["c4_mmdit_step"]["desc"], "blocks": cfg.blocks,
                       "parallelism": f"batch-sharded x{world} (each rank its own CFG pair), weights replicated",
                       "l2": f"{cfg.blocks} blocks x 170 MB of FP8 weights stream through the 126 MB L2 every step",
                       "attention": names[args.attention],
                       "yardstick": {"attention": names[other], "ms_per_step": other_ms},
                       "outside_the_path": "the SiLU of the embeddings and the RMS norm of the prompt's 512 rows (torch)"},
            "e2e": {"value": e2e_ms, "unit": "ms", "h2d_bytes_per_step": int(sum(t.numel() for t in host_in) * 2),
                    "d2h_bytes_per_step": int(hy.numel() * 2), "steps": e2e_steps},
            "gpu_launches": launches,
            "clocks": sampler.summary(),
            "roofline": {"bound": "tensor", "kernel": "gemm_tn_kernel", "achieved": gemm_tflops, "peak": 2.0 * bf16_peak,
                         "unit": UNIT, "frac": gemm_tflops / (2.0 * bf16_peak) if gemm_tflops else None,
                         "peak_source": f"2 x bf16 cuBLAS, of {peak_kind}", "launches": gemm_launches,
                         "gemm_ms_per_step": gemm_ms, "gemm_share_of_step": gemm_ms / ms if ms else None,
                         "traffic": None},
            "cpu_baseline": cpu_baseline,
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.barrier()
        dist.destroy_process_group()


def run_skinny(args):
    """The skinny_decode workload: one activation row against a weight too large for L2, through
    fl_fp8_matmul. Every rank runs its own replica (the path does not shard at one row). The
    roofline is HBM: each call has to read the weight once."""
    import ctypes
    import numpy as np
    import torch
    from libwaifu_b200 import flint as F
    wl = dict(WORKLOADS["skinny_decode"])
    if args.rows:  # (up to 64 rows; up to 32 through fl_fp8_linear)
        wl["m"] = args.rows
        wl["desc"] = wl["desc"] + f" [{args.rows} rows]"
    linear = args.decode_entry == "fp8_linear"
    if linear:
        wl["kind"] = "fp8"
        wl["desc"] = wl["desc"].replace("fl_fp8_matmul", "fl_fp8_linear").replace(
            "fp16 activation x e4m3 weight, one scale", "bf16 activation quantised per token x e4m3 weight, channel scales")
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    torch.cuda.set_device(local)
    F.set_device(local)
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist = dist_mod
    m = wl["m"]
    (n, k), = wl["gemms"]
    sets = 4  # 4 x 50 MB of weights in rotation: nothing a call reads is left in the 126 MB L2
    gen = torch.Generator(device="cuda").manual_seed(rank)

    def wrap(t, dt):
        return F.Tensor.from_device_ptr(t.data_ptr(), tuple(t.shape), dt, keepalive=t)

    act_torch, act_dt = (torch.bfloat16, F.DType.BFLOAT16) if linear else (torch.float16, F.DType.FLOAT16)
    xs = [torch.randn(m, k, device="cuda", dtype=act_torch, generator=gen) for _ in range(sets)]
    ws = []
    for _ in range(sets):
        w = torch.randn(n, k, device="cuda", dtype=torch.float32, generator=gen) * 0.02
        codes, _ = F.quantize_fp8_rows(wrap(w, F.DType.FLOAT))  # e4m3 codes of a Gaussian weight
        ws.append(codes)
        del w
    F.synchronize()
    scale = wrap(torch.full((1,), 0.02 / 448.0 * 4.0, device="cuda", dtype=torch.float32), F.DType.FLOAT)
    channel_scales = wrap(torch.full((n,), 0.02 / 448.0 * 4.0, device="cuda", dtype=torch.float32), F.DType.FLOAT)
    out = F.Tensor.empty((m, n), act_dt)
    x_w = [wrap(x, act_dt) for x in xs]
    L = F.lib()

    def step(i, x_override=None):
        x = x_override if x_override is not None else x_w[i % sets]
        if linear:
            F.check(L.fl_fp8_linear(x.raw(), ws[i % sets].raw(), channel_scales.raw(), None, None, 0, out.raw()))
        else:
            F.check(L.fl_fp8_matmul(x.raw(), ws[i % sets].raw(), scale.raw(), out.raw()))

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if dist is None:
            return ms
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for i in range(args.warmup):
        step(i)
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    launches0 = F.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        step(args.warmup + i)
    e1.record()
    barrier()
    ms_step = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    launches = F.launch_count() - launches0
    F.synchronize()
    sampler.stop_flag.set()
    sampler.join(timeout=5)
    value = world * flops_per_step(wl) / (ms_step * 1e-3) / 1e12

    # end to end: the row from pinned host memory, the result row back to the host
    host_x = F.Tensor.empty((m, k), act_dt, F.Device.CUDA_HOST)
    host_y = F.Tensor.empty((m, n), act_dt, F.Device.CUDA_HOST)
    dev_x = F.Tensor.empty((m, k), act_dt)
    p = ctypes.c_void_p()
    F.check(L.fl_tensor_data_get_host_ptr(host_x._data, ctypes.byref(p)))
    hx = np.ctypeslib.as_array(ctypes.cast(p.value, ctypes.POINTER(ctypes.c_uint16)), shape=(m * k,))
    hx[:] = np.random.default_rng(7 + rank).standard_normal(m * k).astype(np.float16).view(np.uint16)
    if linear:  # (the same bits read as bfloat16 are finite values as well)
        hx[:] &= 0xbfff
    ops = F.operators()

    def e2e_step(i):
        F.check(L.fl_transfer(ops, host_x.raw(), dev_x.raw()))
        step(i, x_override=dev_x)
        F.check(L.fl_transfer(ops, out.raw(), host_y.raw()))  # synchronises

    e2e_steps = max(3, min(args.steps, 200))
    for i in range(3):
        e2e_step(i)
    barrier()
    e0.record()
    for i in range(e2e_steps):
        e2e_step(i)
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1) / e2e_steps)

    _, hbm_peak, peak_kind = measured_peaks()
    alg_bytes = n * k + m * k * 2 + m * n * 2 + (n * 4 if linear else 4)
    achieved = alg_bytes / (ms_step * 1e-3) / 1e9
    traffic = traffic_fields("skinny_decode")
    if linear:
        traffic = traffic_fields("skinny_decode_linear")
    if linear:  # (the routes of fl_sm100_few_rows_route: 33 rows and more go to the tile kernel)
        kernel_name = "fewrow_q8_kernel" if m <= 32 else "gemm_tn_kernel"
    else:
        kernel_name = "fewrow_tc_kernel" if m <= 64 else "gemm_tn_kernel"
    roofline = {"bound": "hbm", "kernel": kernel_name, "achieved": achieved,
                "peak": hbm_peak, "unit": "GB/s",
                "frac": achieved / hbm_peak, "peak_source": f"stream copy, of {peak_kind}", "launches": launches,
                "avg_launch_ms": ms_step, **traffic,
                "algorithmic_bytes_per_step": alg_bytes,
                "note": ("two launches per step (the rows' quantiser, then the product); the time is the step time of the "
                         "back-to-back timed region" if linear else
                         "one launch per step; the launch time is the step time of the back-to-back timed region")}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cstep, kind, cores = cpu_reference_step_factory(wl, m)
        cstep()
        best = None
        for _ in range(5):
            t0 = time.perf_counter()
            cstep()
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        cpu_baseline = {"value": flops_per_step(wl) / best / 1e12, "unit": UNIT, "cores": cores, "kind": kind,
                        "sample": "the whole call (widen, fp32 GEMM, scale) on the host, best of 5"}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "e4m3 x e4m3 -> f32 accumulate" if linear else "f16 x e4m3 -> f32 accumulate", "data": "synthetic",
            "config": {"workload": "skinny_decode", "what": wl["desc"], "parallelism": f"replicas{world}",
                       "l2": f"{sets} rotating weights of {n * k / 1e6:.0f} MB, larger than L2 together",
                       "published": "the reference reports 130.6 us for this shape on an RTX 5060 Ti (docs/fp8.md), other hardware"},
            "e2e": {"value": world * flops_per_step(wl) / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": m * k * 2, "d2h_bytes_per_step": m * n * 2},
            "gpu_launches": launches, "roofline": roofline, "cpu_baseline": cpu_baseline, "clocks": sampler.summary(),
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def run_legacy(args):
    """The legacy_fp8_matmul workload: flint's own fl_fp8_matmul_add (fp16 activation kept in half,
    e4m3 weight widened inside the kernel, one fp32 scale, a bias pre-expanded to the product's
    shape as the Rust wrapper hands it over) on the reference's benchmark shapes. Tensor-bound on
    the 16-bit tcgen05 kind: the roofline is the measured bf16 GEMM throughput. Every rank runs
    its own batch of rows."""
    import ctypes
    import numpy as np
    import torch
    from libwaifu_b200 import flint as F
    wl = dict(WORKLOADS["legacy_fp8_matmul"])
    if args.rows:
        wl["m"] = args.rows
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    torch.cuda.set_device(local)
    F.set_device(local)
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist = dist_mod
    f16 = F.DType.FLOAT16
    gen = torch.Generator(device="cuda").manual_seed(rank)
    L = F.lib()

    def wrap(t, dt):
        return F.Tensor.from_device_ptr(t.data_ptr(), tuple(t.shape), dt, keepalive=t)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if dist is None:
            return ms
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def make(m, n, k, sets):
        xs = [wrap(torch.randn(m, k, device="cuda", dtype=torch.float16, generator=gen), f16) for _ in range(sets)]
        ws = []
        for _ in range(sets):
            w = torch.randn(n, k, device="cuda", dtype=torch.float32, generator=gen) * 0.02
            codes, _ = F.quantize_fp8_rows(wrap(w, F.DType.FLOAT))
            ws.append(codes)
            del w
        F.synchronize()
        scale = wrap(torch.full((1,), 0.02 * 4.0 / 448.0, device="cuda", dtype=torch.float32), F.DType.FLOAT)
        bias = wrap(torch.randn(n, device="cuda", dtype=torch.float16, generator=gen) * 0.01, f16)
        out = F.Tensor.empty((m, n), f16)
        expanded = F._broadcast_to(bias, out)  # a zero-stride view, waifu/src/flint/functional.rs:80-108,698

        def call(i):
            F.check(L.fl_fp8_matmul_add(xs[i % sets].raw(), ws[i % sets].raw(), scale.raw(), expanded.raw(), out.raw()))
        return call, out, (xs, ws, scale, bias, expanded)

    def time_calls(call, warmup, steps):
        for i in range(warmup):
            call(i)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for i in range(steps):
            call(warmup + i)
        e1.record()
        barrier()
        return max_over_ranks(e0.elapsed_time(e1) / steps)

    m = wl["m"]
    (n, k), = wl["gemms"]
    call, out, keep = make(m, n, k, args.rotate)
    sampler = ClockSampler(local)
    sampler.start()
    launches0 = F.launch_count()
    ms_step = time_calls(call, max(args.warmup, 3), args.steps)
    launches = F.launch_count() - launches0
    F.gemm_timing(True)
    F.gemm_timing_read()
    for i in range(args.steps):
        call(i)
    gemm_ms, gemm_launches = F.gemm_timing_read()
    F.gemm_timing(False)
    sampler.stop_flag.set()
    sampler.join(timeout=5)
    flops = 2.0 * m * n * k
    value = world * flops / (ms_step * 1e-3) / 1e12

    others = {}
    for (m2, n2, k2) in [(256, 3072, 3072), (4096, 3072, 3072)]:
        c2, _, keep2 = make(m2, n2, k2, 4)
        t = time_calls(c2, 3, max(20, min(args.steps, 200)))
        others[f"{m2}x{n2}x{k2}"] = {"ms": t, "tflops": 2.0 * m2 * n2 * k2 / (t * 1e-3) / 1e12}
        del c2, keep2

    # end to end: the activation from pinned host memory, the product back
    host_x = F.Tensor.empty((m, k), f16, F.Device.CUDA_HOST)
    host_y = F.Tensor.empty((m, n), f16, F.Device.CUDA_HOST)
    p = ctypes.c_void_p()
    F.check(L.fl_tensor_data_get_host_ptr(host_x._data, ctypes.byref(p)))
    hx = np.ctypeslib.as_array(ctypes.cast(p.value, ctypes.POINTER(ctypes.c_uint16)), shape=(m * k,))
    hx[:] = np.random.default_rng(7 + rank).standard_normal(m * k).astype(np.float16).view(np.uint16)
    xs, ws, scale, bias, expanded = keep

    def e2e_step(i):
        xd, pending = F.transfer_async(host_x)
        pending.wait()
        F.check(L.fl_fp8_matmul_add(xd.raw(), ws[i % len(ws)].raw(), scale.raw(), expanded.raw(), out.raw()))
        F.transfer_to_host_async(out, host_y).wait_sync()

    e2e_ms = time_calls(e2e_step, 2, max(3, min(args.steps, 20)))

    bf16_peak, _, peak_kind = measured_peaks(sampler.summary())
    achieved = flops * args.steps / (gemm_ms * 1e-3) / 1e12 if gemm_ms > 0 else None
    roofline = {"bound": "tensor", "kernel": "gemm_tn_kernel (16-bit kind, e4m3 weight widened in shared memory)",
                "achieved": achieved, "peak": bf16_peak, "unit": UNIT, "frac": achieved / bf16_peak if achieved else None,
                "peak_source": f"bf16 cuBLAS, of {peak_kind}", "launches": gemm_launches,
                "avg_launch_ms": gemm_ms / gemm_launches if gemm_launches else None, "traffic": None,
                "algorithmic_bytes_per_step": m * k * 2 + n * k + m * n * 2 + n * 2 + 4}

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        rows = min(m, args.reference_rows)
        cstep, kind, cores = cpu_reference_step_factory(wl, rows)
        cstep()
        best = None
        for _ in range(3):
            t0 = time.perf_counter()
            cstep()
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        cpu_baseline = {"value": 2.0 * rows * n * k / best / 1e12, "unit": UNIT, "cores": cores, "kind": kind,
                        "sample": f"{rows} of {m} rows, the whole call (widen, fp32 GEMM, scale) on the host, best of 3"}
    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f16 x e4m3 -> f32 accumulate", "data": "synthetic",
            "config": {"workload": "legacy_fp8_matmul", "what": wl["desc"], "parallelism": f"batch-sharded x{world}",
                       "l2": f"{args.rotate} rotating operand sets", "other_shapes": others,
                       "published": "the reference reports 44-46 TFLOP/s for these shapes on an RTX 5060 Ti (docs/fp8.md), other hardware"},
            "e2e": {"value": world * flops / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": m * k * 2, "d2h_bytes_per_step": m * n * 2},
            "gpu_launches": launches, "roofline": roofline, "cpu_baseline": cpu_baseline, "clocks": sampler.summary(),
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def run_attention(args):
    """The attention_step workload: the denoise step's joint attention (batch 2, 24 heads of 128,
    4352 tokens, no mask) through fl_attention on q, k, v laid out as the fused projection leaves
    them, (batch, tokens, 3, heads, head_dim), the result token-major. Every rank runs its own
    batch (rows shard with no exchange). Tensor-bound: 4 N h L^2 D flops against the measured bf16
    GEMM throughput. Four sets of operands in rotation keep a call's inputs out of L2."""
    import torch
    from libwaifu_b200 import flint as F
    wl = WORKLOADS["attention_step"]
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    torch.cuda.set_device(local)
    F.set_device(local)
    if world > 1:
        import torch.distributed as dist_mod
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local))
        dist = dist_mod
    n, h, L, d = 2, 24, 4352, 128
    sets = 4  # 4 x 160 MB
    gen = torch.Generator(device="cuda").manual_seed(rank)
    qkvs = [torch.randn(n, L, 3, h, d, device="cuda", dtype=torch.bfloat16, generator=gen) for _ in range(sets)]
    out = torch.empty(n, L, h, d, device="cuda", dtype=torch.bfloat16)

    def view(t5, i):
        part = t5[:, :, i].transpose(1, 2)
        return F.Tensor.from_device_ptr(part.data_ptr(), tuple(part.shape), F.DType.BFLOAT16, keepalive=t5,
                                        stride=tuple(part.stride()), numel=t5.numel())

    ops_in = [[view(t, i) for i in range(3)] for t in qkvs]
    o = out.transpose(1, 2)
    out_v = F.Tensor.from_device_ptr(o.data_ptr(), tuple(o.shape), F.DType.BFLOAT16, keepalive=out, stride=tuple(o.stride()),
                                     numel=out.numel())

    def step(i):
        q, k, v = ops_in[i % sets]
        F.attention(q, k, v, F.MaskType.NONE, 0, out_v)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if dist is None:
            return ms
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    for i in range(args.warmup):
        step(i)
    barrier()
    sampler = ClockSampler(local)
    sampler.start()
    launches0 = F.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for i in range(args.steps):
        step(args.warmup + i)
    e1.record()
    barrier()
    ms_step = max_over_ranks(e0.elapsed_time(e1) / args.steps)
    launches = F.launch_count() - launches0
    sampler.stop_flag.set()
    sampler.join(timeout=5)
    flops = 4.0 * n * h * L * L * d
    value = world * flops / (ms_step * 1e-3) / 1e12

    # end to end: q, k, v from pinned host memory, the result back to the host
    host_in = torch.empty(n, L, 3, h, d, dtype=torch.bfloat16).pin_memory()
    host_in.copy_(qkvs[0].cpu())
    host_out = torch.empty(n, L, h, d, dtype=torch.bfloat16).pin_memory()
    e2e_steps = max(3, min(args.steps, 20))

    def e2e_step():
        qkvs[0].copy_(host_in, non_blocking=True)
        step(0)
        host_out.copy_(out, non_blocking=True)
        torch.cuda.synchronize()

    for _ in range(2):
        e2e_step()
    barrier()
    e0.record()
    for _ in range(e2e_steps):
        e2e_step()
    e1.record()
    barrier()
    e2e_ms = max_over_ranks(e0.elapsed_time(e1) / e2e_steps)

    bf16_peak, _, peak_kind = measured_peaks(sampler.summary())
    achieved = flops / (ms_step * 1e-3) / 1e12
    roofline = {"bound": "tensor", "kernel": "attention2_kernel", "achieved": achieved, "peak": bf16_peak, "unit": "TFLOP/s",
                "frac": achieved / bf16_peak, "peak_source": f"bf16 cuBLAS, of {peak_kind}", "launches": launches,
                "avg_launch_ms": ms_step, **traffic_fields("attention_step"),
                "algorithmic_bytes_per_step": 4 * n * h * L * d * 2,
                "note": "one launch per step (the two-tile kernel reads v as it lies): the step time is the kernel's"}
    if rank == 0:
        line = {
            "metric": METRIC.replace("quantized GEMM", "attention"), "value": value, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16 -> f32 accumulate", "data": "synthetic",
            "config": {"workload": "attention_step", "what": wl["desc"], "parallelism": f"batch-sharded x{world}",
                       "l2": f"{sets} rotating operand sets of 160 MB, larger than L2"},
            "e2e": {"value": world * flops / (e2e_ms * 1e-3) / 1e12, "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int(host_in.numel() * 2), "d2h_bytes_per_step": int(host_out.numel() * 2)},
            "gpu_launches": launches, "roofline": roofline, "cpu_baseline": None, "clocks": sampler.summary(),
        }
        print(json.dumps(line), flush=True)
    if dist is not None:
        dist.destroy_process_group()


def run_attention_reference(args):
    """The reference arm of attention_step: the reference's own CPU fl_attention (float32, the
    composition of flint/operators.cc:148-230) on a bounded sample of the workload, all host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    try:
        os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))
    except Exception:
        os.environ.pop("OMP_NUM_THREADS", None)
    import numpy as np
    sys.path.insert(0, ROOT)
    from oracle import oracle as O
    wl = WORKLOADS["attention_step"]
    line = {"impl": "reference", "config": {"workload": "attention_step", "what": wl["desc"]}}
    if not O.have_ref():
        line["unavailable"] = "the reference's CPU library (oracle/_ref) is not built here"
        print(json.dumps(line), flush=True)
        return
    heads, q_len, kv_len, d = 4, 1088, 4352, 128
    rng = np.random.default_rng(0)
    q = rng.standard_normal((1, heads, q_len, d)).astype(np.float32)
    k = rng.standard_normal((1, heads, kv_len, d)).astype(np.float32)
    v = rng.standard_normal((1, heads, kv_len, d)).astype(np.float32)
    R = O.ref()
    for _ in range(args.warmup):
        R.attention(q, k, v, False)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        R.attention(q, k, v, False)
    ms = (time.perf_counter() - t0) * 1e3 / args.steps
    value = 4.0 * heads * q_len * kv_len * d / (ms * 1e-3) / 1e12
    cores = len(os.sched_getaffinity(0))
    sample = f"{heads} of 48 (batch, head) pairs, {q_len} of 4352 queries over all 4352 keys per step, float32"
    line.update({
        "metric": METRIC.replace("quantized GEMM", "attention"), "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "reference", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    })
    line["config"]["sample"] = sample
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=1000)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2_mlp", choices=sorted(WORKLOADS))
    ap.add_argument("--rotate", type=int, default=3, help="operand sets rotated through to defeat L2 reuse")
    ap.add_argument("--rows", type=int, default=None, help="override the workload's row count (for small profile captures)")
    ap.add_argument("--decode-entry", default="fp8_matmul", choices=["fp8_matmul", "fp8_linear"],
                    help="skinny_decode: the reference's fl_fp8_matmul (16-bit rows) or fl_fp8_linear (rows quantised per token)")
    ap.add_argument("--reference-rows", type=int, default=1088, help="rows of the bounded CPU sample")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--e2e-chunks", type=int, default=4, help="row chunks the end-to-end step is pipelined in")
    ap.add_argument("--sustained-seconds", type=float, default=1.0,
                    help="length of the extra back-to-back loop behind roofline.sustained (0: skip it)")
    ap.add_argument("--parallel", default="batch", choices=["batch", "nsplit", "nsplit_push", "nsplit_fp8", "nsplit_fp8_nccl"],
                    help="batch: rows sharded, no collective (weak scaling; at N > 1 the line also carries a "
                         "strong_scaling object from the nsplit_fp8 form); nsplit*: one MLP with its weights split by "
                         "output channel (strong scaling): NCCL all-gathers / epilogue pushes in 16 bits / H gathered as e4m3 codes")
    ap.add_argument("--e2e-depth", type=int, default=2, help="end-to-end leg: steps in flight (page-locked buffers each way)")
    ap.add_argument("--no-strong-scaling", action="store_true", help="leave the strong_scaling object out of a batch run at N > 1")
    ap.add_argument("--blocks", type=int, default=None, help="c4_mmdit_step: run this many blocks instead of 60")
    ap.add_argument("--attention", default="flint", choices=["sdpa", "flint"],
                    help="c4_mmdit_step: this library's fl_attention (the reported number), or torch's attention; "
                         "the other one is timed beside it as a yardstick")
    args = ap.parse_args()
    if args.workload == "skinny_decode" and args.impl == "ours":
        args.warmup = max(args.warmup, 3)
        if args.steps == 1000:
            args.steps = 20000  # 20 us a step: long enough for the clock sampler to see the run
        return run_skinny(args)
    if args.workload == "legacy_fp8_matmul" and args.impl == "ours":
        if args.steps == 1000:
            args.steps = 200
        return run_legacy(args)
    if args.workload == "attention_step" and args.impl == "reference":
        if args.steps == 1000:
            args.steps = 3
        return run_attention_reference(args)
    if args.workload == "attention_step" and args.impl == "ours":
        args.warmup = max(args.warmup, 3)
        if args.steps == 1000:
            args.steps = 50
        return run_attention(args)
    if args.workload == "c4_mmdit_step" and args.impl == "ours":
        if args.steps == 1000:
            args.steps = 10
        return run_mmdit(args)
    if args.workload == "c4_mmdit_step" and args.impl == "reference":
        if args.steps == 1000:
            args.steps = 3
        return run_mmdit_reference(args)
    wl = dict(WORKLOADS[args.workload])
    if args.rows:
        wl["m"] = args.rows
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args, wl)
    else:
        run_ours(args, wl)


if __name__ == "__main__":
    main()
