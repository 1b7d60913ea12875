#!/usr/bin/env python
"""Benchmark of the poplin contraction path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one pass of the hot path (one convolution / matrix product call)
over one batch of synthetic input.  The default workload is the ResNet 3x3
forward convolution the metric is quoted on; the other named configurations
can be selected with --workload, and by default each of them is also timed
in the same process with a bounded step count and reported under
"workloads" (ms per step, TFLOP/s, roofline, clocks, parity check).  One JSON
line is printed by rank 0.

  value      TFLOP/s with inputs resident in HBM (2 x MACs, products with
             padding not counted, as the reference's getFwdFlops does), timed
             with CUDA events on the launching stream, max over ranks.  The
             steps are replayed from a CUDA graph holding one library call per
             rotating buffer set (--no-graph: one call per step), so that the
             host's per-launch cost does not pace microsecond kernels.
  e2e        the same metric through the host-buffer C ABI calls: every step
             uploads its inputs from pinned host memory, runs and downloads its
             result, all inside the timed region; steps alternate between two
             contexts so one step's download overlaps the next one's upload.
  roofline   achieved vs the measured bf16 burst peak (tensor bound) or the
             measured copy bandwidth (HBM bound) of MEASURED_PEAKS.json.
  cpu_baseline  the reference's own CPU model (oracle/_ref when built, else the
             C restatement) timed on the host cores on a bounded sample.

  parity_check  a sample of what the timed loop computed, compared with the CPU
             oracle after the timed region (same tolerance as the tests).

With N > 1 (launched under torchrun) every rank runs the same per-GPU
workload on its own shard of a batch N times larger (weak scaling; the path
needs no collective in the forward pass).  The line then also carries "wu":
the weight update of the 3x3 128-channel layer, whose per-rank gradients are
summed inside the library's reduction kernel over NVLink peer memory (the one
collective of the path), checked against the process group's all-reduce, with
the same rank's update without the collective timed beside it; and
"strong_scaling": the two largest configurations sharded over the ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import numpy as np  # noqa: E402

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# Dense fp8 (e4m3) peak, measured on this pool's B200s the way MEASURED_PEAKS.json
# measures bf16: torch._scaled_mm on 8192^3, best of 10 (burst) and back to back
# for 4 s (sustained); see profiles/fp8_peak.md.
FP8_PEAK_TFLOPS = {"burst": 3151.1, "sustained": 2587.6,
                   "source": "of measured (torch._scaled_mm e4m3 8192^3, burst; profiles/fp8_peak.md)"}

# name -> description of one call.  kind conv: ConvParams kwargs + pass; kind gemm: m, k, n.
WORKLOADS = {
    "conv3x3_fwd_n32_56x56_c64": dict(kind="conv", pass_="fwd", bound="tensor",
                                      params=dict(batch=32, field=[56, 56], kernel=[3, 3], in_chans=64,
                                                  out_chans=64, padding=1)),
    "conv3x3_fwd_n256_28x28_c128": dict(kind="conv", pass_="fwd", bound="tensor",
                                        params=dict(batch=256, field=[28, 28], kernel=[3, 3], in_chans=128,
                                                    out_chans=128, padding=1)),
    "conv3x3_bwd_n256_28x28_c128": dict(kind="conv", pass_="bwd", bound="tensor",
                                        params=dict(batch=256, field=[28, 28], kernel=[3, 3], in_chans=128,
                                                    out_chans=128, padding=1)),
    "conv3x3_wu_n256_28x28_c128": dict(kind="conv", pass_="wu", bound="tensor",
                                       params=dict(batch=256, field=[28, 28], kernel=[3, 3], in_chans=128,
                                                   out_chans=128, padding=1)),
    "conv1x1_s2_fwd_n256_56x56_c256_c512": dict(kind="conv", pass_="fwd", bound="hbm",
                                                params=dict(batch=256, field=[56, 56], kernel=[1, 1],
                                                            in_chans=256, out_chans=512, stride=2)),
    "conv7x7_s2_fwd_n256_224x224_c3_c64": dict(kind="conv", pass_="fwd", bound="hbm",
                                               params=dict(batch=256, field=[224, 224], kernel=[7, 7],
                                                           in_chans=3, out_chans=64, padding=3, stride=2)),
    # batch normalisation of the 3x3 layer's output, forward: statistics, whiten, scale and shift
    "batchnorm_fwd_n32_56x56_c64": dict(kind="norm", bound="hbm", batch=32, field=[56, 56], chans=64),
    "matmul_fp16_512x1024x1024": dict(kind="gemm", m=512, k=1024, n=1024, quarter=False, bound="tensor"),
    "matmul_fp16_8192": dict(kind="gemm", m=8192, k=8192, n=8192, quarter=False, bound="tensor"),
    "matmul_fp8_8192": dict(kind="gemm", m=8192, k=8192, n=8192, quarter=True, bound="tensor"),
}
DEFAULT_WORKLOAD = "conv3x3_fwd_n32_56x56_c64"

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel,
# from the ncu captures summarised under profiles/ (absent = not captured).
# Outputs smaller than the 126 MB L2 are still dirty in L2 when the kernel
# ends, so their write-back does not show in the kernel's own DRAM write count.
NCU_DRAM_TRAFFIC_BYTES = {
    "conv3x3_fwd_n32_56x56_c64": 12995328,
    "conv3x3_fwd_n256_28x28_c128": 51744768 + 13427520,
    "conv3x3_bwd_n256_28x28_c128": 51750000 + 13090000,
    "conv3x3_wu_n256_28x28_c128": 105509248 + 4087936,
    "conv1x1_s2_fwd_n256_56x56_c256_c512": 103111168 + 153707456,
    "conv7x7_s2_fwd_n256_224x224_c3_c64": 114367232 + 358181632,   # the implicit-GEMM kernel of the two (the fold adds 77.1 + 56.1 MB)
    "batchnorm_fwd_n32_56x56_c64": 2 * 12850000,                   # column sums + the normalising pass (outputs stay in L2)
    "matmul_fp16_512x1024x1024": 3220000,
    "matmul_fp16_8192": 1074835000 + 128641408,
    "matmul_fp8_8192": 344460000 + 119442500,
}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        try:
            with open(path) as f:
                d = json.load(f)
            return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
        except Exception:
            pass
    return dict(FALLBACK_PEAKS), "fallback"


# --------------------------------------------------------------------------- clocks

class ClockSampler:
    """Samples SM clocks and throttle reasons during the timed region: NVML
    polled from a thread every few milliseconds (the timed region of a small
    layer lasts only milliseconds), nvidia-smi at 100 ms as the fallback.
    Read-only: nothing about the GPU is changed."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, device_index: int):
        self.rows = []
        self.proc = None
        self.device_index = device_index
        self.nvml = None
        self.samples = []      # (sm_mhz, reasons bitmask)
        self.stop_flag = False

    def start(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nvml = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(self.device_index)
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._poll, daemon=True)
            self.thread.start()
            return
        except Exception:
            self.nvml = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-i", str(self.device_index), "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _poll(self):
        n = self.nvml
        while not self.stop_flag:
            try:
                mhz = float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                try:
                    reasons = int(n.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                except Exception:
                    reasons = int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                self.samples.append((mhz, reasons))
            except Exception:
                pass
            time.sleep(0.002)

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append(line.strip())

    def stop(self):
        if self.nvml is not None:
            self.stop_flag = True
            self.thread.join(timeout=2)
            n = self.nvml
            names = {"hw_slowdown": getattr(n, "nvmlClocksThrottleReasonHwSlowdown", 0x8),
                     "hw_thermal_slowdown": getattr(n, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40),
                     "sw_thermal_slowdown": getattr(n, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20),
                     "sw_power_cap": getattr(n, "nvmlClocksThrottleReasonSwPowerCap", 0x4)}
            reasons = sorted(k for k, bit in names.items() if any(r & bit for _, r in self.samples))
            sm = [m for m, _ in self.samples]
            try:
                n.nvmlShutdown()
            except Exception:
                pass
            return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": self.max_mhz,
                    "reasons": reasons, "samples": len(sm), "source": "nvml, 2 ms poll"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        for row in self.rows:
            f = [c.strip() for c in row.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"),
                                 f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons), "samples": len(sm),
                "source": "nvidia-smi, 100 ms"}


# --------------------------------------------------------------------------- workload state

def workload_plan(spec):
    """What the library's planner chooses for a workload (host-side arithmetic:
    no device is touched), as both arms report it in `config.plan`."""
    from poplibs_b200 import capi
    if spec["kind"] == "norm":
        pixels = spec["batch"] * int(np.prod(spec["field"]))
        return {"kernel": "norm column sums + element-wise maps", "bytes": 4 * 2 * pixels * spec["chans"]}
    if spec["kind"] == "conv":
        p = capi.ConvParams.make(**spec["params"])
        pass_id = {"bwd": capi.PASS_TRAINING_BWD, "wu": capi.PASS_TRAINING_WU}.get(
            spec["pass_"], capi.PASS_TRAINING_FWD)
        return capi.conv_plan(p, pass_id).as_dict()
    q = spec["quarter"]
    desc = capi.MatmulDesc.make(spec["m"], spec["k"], spec["n"], input_type=capi.QUARTER if q else capi.HALF,
                                transpose_b=q, scale_a=-3 if q else 0, scale_b=-2 if q else 0)
    return capi.matmul_plan(desc).as_dict()


class Workload:
    """Device-resident rotating buffer sets (so that consecutive steps do not
    find their inputs in L2) and, for the workload the headline is quoted on,
    pinned host copies for the end-to-end leg."""

    def __init__(self, name, spec, ctx, device, rank=0, world=1, sets_bytes_target=300 << 20, force_sets=0,
                 host_copies=True, allreduce="auto"):
        import torch
        from poplibs_b200 import capi
        self.name, self.spec, self.ctx, self.capi = name, spec, ctx, capi
        self.rank, self.world, self.device = rank, world, device
        g = torch.Generator(device=device).manual_seed(1234 + rank)
        self.kind = spec["kind"]
        self.sharded = None
        self.allreduce = None

        def uniform(shape, scale=1.0):
            return ((torch.rand(shape, generator=g, device=device) * 2 - 1) * scale).half()
        if self.kind == "norm":
            shape = (spec["batch"], *spec["field"], spec["chans"])
            self.pixels, self.chans = int(np.prod(shape[:-1])), spec["chans"]
            proto = {"x": uniform(shape).add_(0.25), "gamma": uniform((self.chans,)).abs_().add_(0.5),
                     "beta": uniform((self.chans,))}
            self.flops = 0
            # the activations are read twice (statistics, normalise), the whitened ones and the output written
            self.plan = workload_plan(spec)
            per_set = 3 * 2 * self.pixels * self.chans
            out_shape = shape
        elif self.kind == "conv":
            p = capi.ConvParams.make(**spec["params"])
            self.p = p
            kw = spec["params"]
            of = p.output_field()
            ci, co = p.in_chans_per_group, p.out_chans_per_group
            self.flops = 2 * p.macs()
            self.x_shape = (p.batch, *kw["field"], ci)
            self.y_shape = (p.batch, *of, co)
            self.w_shape = (*kw["kernel"], co, ci)
            bound = 1.0 / np.sqrt(ci * int(np.prod(kw["kernel"])))
            self.pass_ = spec["pass_"]
            proto = {"x": uniform(self.x_shape), "w": uniform(self.w_shape, bound), "dy": uniform(self.y_shape)}
            if world > 1 and self.pass_ == "wu":
                from poplibs_b200 import parallel
                # weak scaling: every rank holds one full per-GPU batch of the layer
                glob = dict(kw, batch=kw["batch"] * world)
                peer = allreduce != "nccl"
                try:
                    self.sharded = parallel.ShardedConv(ctx, glob, rank, world, peer_allreduce=peer,
                                                        allreduce_mode=allreduce if peer else "auto")
                    self.allreduce = (f"library kernels over NVLink peer memory ({self.sharded.peer.mode})"
                                      if peer else "nccl all_reduce + cast")
                except Exception as e:  # symmetric memory unavailable: the process group's all-reduce
                    self.sharded = parallel.ShardedConv(ctx, glob, rank, world)
                    self.allreduce = f"nccl all_reduce + cast (peer memory unavailable: {type(e).__name__})"
            self.plan = workload_plan(spec)
            per_set = 2 * (int(np.prod(self.x_shape)) + int(np.prod(self.y_shape)))
            out_shape = {"fwd": self.y_shape, "bwd": self.x_shape, "wu": self.w_shape}[self.pass_]
        else:
            m, k, n = spec["m"], spec["k"], spec["n"]
            self.quarter = spec["quarter"]
            self.desc = capi.MatmulDesc.make(m, k, n, input_type=capi.QUARTER if self.quarter else capi.HALF,
                                             transpose_b=self.quarter,
                                             scale_a=-3 if self.quarter else 0, scale_b=-2 if self.quarter else 0)
            self.flops = 2 * m * k * n
            self.plan = workload_plan(spec)
            if self.quarter:
                a = torch.randn((m, k), generator=g, device=device).mul_(8).to(torch.float8_e4m3fn).view(torch.uint8)
                b = torch.randn((n, k), generator=g, device=device).mul_(4).to(torch.float8_e4m3fn).view(torch.uint8)
            else:
                a = torch.randn((m, k), generator=g, device=device).half()
                b = torch.randn((k, n), generator=g, device=device).half()
            proto = {"a": a, "b": b}
            per_set = a.numel() * a.element_size() + b.numel() * b.element_size() + 2 * m * n
            out_shape = (m, n)
        self.bytes = self.plan["bytes"]
        self.nsets = int(max(2, min(16, -(-sets_bytes_target // max(per_set, 1)))))
        if force_sets > 0:
            self.nsets = force_sets
        self.dev = []
        for i in range(self.nsets):
            d = proto if i == 0 else {k: v.clone() for k, v in proto.items()}
            d["out"] = torch.empty(out_shape, dtype=torch.float16, device=device)
            if self.kind == "norm":
                d["white"] = torch.empty(out_shape, dtype=torch.float16, device=device)
                d["mean"] = torch.empty(self.chans, dtype=torch.float16, device=device)
                d["inv"] = torch.empty(self.chans, dtype=torch.float16, device=device)
                d["power"] = torch.empty(self.chans, dtype=torch.float32, device=device)
            if self.kind == "conv" and self.pass_ == "wu":
                d["out32"] = torch.empty(out_shape, dtype=torch.float32, device=device)
            self.dev.append(d)
        self.host = self.host_out = None
        self.e2e_ctx = None
        if host_copies and self.has_e2e():
            # end-to-end leg: pinned inputs, two contexts (streams) and two pinned output buffers,
            # allocated from the CPUs next to the GPU so that the pages land in that NUMA node's memory
            previous = capi.bind_host_to_device(device.index)
            self.host_binding = ("page-locked buffers allocated on the GPU's NUMA node" if previous is not None
                                 else "none (no other node, or the platform does not say)")
            try:
                self.host = {k: v.cpu().pin_memory() for k, v in proto.items() if self._is_input(k)}
                self.host_out = [torch.empty(out_shape, dtype=torch.float16).pin_memory() for _ in range(2)]
                for t in self.host_out:
                    t.zero_()   # touch the pages here
            finally:
                if previous is not None:
                    os.sched_setaffinity(0, previous)
            self.h2d_bytes = sum(v.numel() * v.element_size() for v in self.host.values())
            self.d2h_bytes = self.host_out[0].numel() * 2
        self.launches_per_step = 1
        torch.cuda.synchronize()

    def _is_input(self, key):
        if self.kind == "gemm":
            return key in ("a", "b")
        return key in {"fwd": ("x", "w"), "bwd": ("dy", "w"), "wu": ("x", "dy")}[self.pass_]

    def step(self, i):
        d = self.dev[i % self.nsets]
        if self.kind == "norm":
            H, c, n = self.capi.HALF, self.chans, self.pixels
            self.ctx.norm_statistics(H, d["x"], n, c, 1e-3, 1.0, d["mean"], d["inv"], d["power"])
            self.ctx.norm_normalise(H, d["x"], d["mean"], d["inv"], d["gamma"], d["beta"], n, c, d["white"],
                                    d["out"])
        elif self.kind == "gemm":
            self.ctx.matmul(self.desc, d["a"], d["b"], None, d["out"])
        elif self.pass_ == "fwd":
            self.ctx.conv_fwd(self.p, d["x"], d["w"], d["out"])
        elif self.pass_ == "bwd":
            self.ctx.conv_bwd(self.p, d["dy"], d["w"], d["out"])
        elif self.sharded is None:
            self.ctx.conv_wu(self.p, d["x"], d["dy"], d["out"], d["out32"])
        else:
            # per-rank batch reduced locally and summed over the ranks: the one collective of the path
            self.sharded.wu(d["x"], d["dy"], d["out"], d["out32"])

    def step_local(self, i):
        """The weight update of this rank's batch alone (no sum over ranks)."""
        d = self.dev[i % self.nsets]
        self.ctx.conv_wu(self.p, d["x"], d["dy"], d["out"], d["out32"])

    def check_allreduce(self):
        """One untimed step of the multi-GPU weight update compared with (a) the
        per-rank gradients gathered and added in rank order with fp32 adds, which
        the library's sum must equal bit for bit on every rank, and (b) the process
        group's own all-reduce, whose order of additions is NCCL's (ring / tree):
        agreement to the last place or two of fp32."""
        import torch
        import torch.distributed as dist
        d = self.dev[0]
        local = torch.empty_like(d["out32"])
        self.ctx.conv_wu(self.p, d["x"], d["dy"], None, local)
        self.ctx.synchronize()
        gathered = [torch.empty_like(local) for _ in range(self.world)]
        dist.all_gather(gathered, local)
        ordered = gathered[0].clone()
        for g in gathered[1:]:
            ordered += g
        nccl = local.clone()
        dist.all_reduce(nccl)
        self.sharded.wu(d["x"], d["dy"], d["out"], d["out32"])
        self.ctx.synchronize()
        torch.cuda.synchronize()
        ok = torch.tensor([int(torch.equal(ordered, d["out32"]) and torch.equal(ordered.half(), d["out"]))],
                          device=local.device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        return {"equals_rank_order_sum_on_every_rank": bool(ok.item()),
                "max_abs_diff_vs_nccl": float((nccl - d["out32"]).abs().max().item()),
                "max_abs": float(nccl.abs().max().item())}

    def step_e2e(self, i):
        """One end-to-end step: pinned host inputs -> device -> kernel -> pinned
        host output, through the host-buffer entry points.  Steps alternate
        between two library contexts (streams), so one step's download overlaps
        the next one's upload; a context is synchronised before it is reused,
        i.e. the result of step i - 2 is complete on the host by then."""
        c = self.e2e_ctx[i & 1]
        c.synchronize()
        out = self.host_out[i & 1]
        if self.kind == "gemm":
            c.matmul_host(self.desc, self.host["a"], self.host["b"], None, out, sync=False)
        else:
            c.conv_fwd_host(self.p, self.host["x"], self.host["w"], out, sync=False)

    def has_e2e(self):
        return self.kind == "gemm" or (self.kind == "conv" and self.pass_ == "fwd")

    # ---- correctness evidence carried by the bench line ------------------------------
    def parity_check(self):
        """Compares a sample of what the timed loop left in buffer set 0 with the
        CPU oracle (the checker; outside every timed region), under the
        tolerance the tests use: relative 1e-3 (half) / 5e-2 (quarter),
        absolute max(1e-5, 2.5e-4 * rms(expected))."""
        import torch
        import common as T
        import oracle
        d = self.dev[0]
        rel = T.REL_TOL_QUARTER if self.spec.get("quarter") else T.REL_TOL_HALF
        if self.kind == "norm":
            # the whole tensor: statistics from the model, the output from the device's own statistics
            to_bcf = lambda t: t.float().cpu().numpy().reshape(self.spec["batch"], -1, self.chans).transpose(0, 2, 1)  # noqa: E731
            x = to_bcf(d["x"]).astype(np.float64)
            mean, inv = oracle.norm_statistics(x, 1e-3)
            bad_stats = int(oracle.check_is_close(d["inv"].float().cpu().numpy(), inv, 5e-3, 1e-5)[0] +
                            oracle.check_is_close(d["mean"].float().cpu().numpy(), mean, 2e-3, 1e-4)[0])
            want, _ = oracle.norm_normalise(x, d["gamma"].float().cpu().numpy(), d["beta"].float().cpu().numpy(),
                                            d["mean"].float().cpu().numpy(), d["inv"].float().cpu().numpy())
            got = to_bcf(d["out"])
            rel = 4e-3   # two roundings to half (whitened, then scaled and shifted)
            what = f"all {got.size} outputs; statistics outside tolerance: {bad_stats}"
        elif self.kind == "gemm":
            m = self.spec["m"]
            rows = sorted({0, m // 3, (2 * m) // 3, m - 1})
            a = d["a"][rows]
            if self.quarter:
                av = a.view(torch.float8_e4m3fn).float().cpu().numpy()
                bv = d["b"].view(torch.float8_e4m3fn).float().cpu().numpy()
                want = oracle.gemm(av, bv, transpose_b=True) * 2.0 ** -5
            else:
                want = oracle.gemm(a.float().cpu().numpy(), d["b"].float().cpu().numpy())
            got = d["out"][rows].float().cpu().numpy()
            what = f"{len(rows)} rows of the product"
        else:
            p, kw = self.p, self.spec["params"]
            pick = [0, p.batch - 1] if p.batch > 1 else [0]
            sub = self.capi.ConvParams.make(**{**kw, "batch": len(pick)})
            spec = T.spec_from_params(sub)
            nchw = lambda t: t.permute(0, 3, 1, 2).float().cpu().numpy()       # noqa: E731
            w = d["w"].permute(2, 3, 0, 1)[None].float().cpu().numpy() if self.pass_ != "wu" else None
            if self.pass_ == "fwd":
                want = oracle.conv_fwd(spec, nchw(d["x"][pick]), w)
                got = nchw(d["out"][pick])
                what = f"{len(pick)} images of the output"
            elif self.pass_ == "bwd":
                want = oracle.conv_bwd(spec, nchw(d["dy"][pick]), w)
                got = nchw(d["out"][pick])
                what = f"{len(pick)} images of the input gradient"
            else:
                # the gradient sums over the whole batch: the oracle is run on a
                # two-image batch, through the same entry point
                x, dy = d["x"][pick].contiguous(), d["dy"][pick].contiguous()
                g32 = torch.empty(self.w_shape, dtype=torch.float32, device=self.device)
                self.ctx.conv_wu(sub, x, dy, None, g32)
                self.ctx.synchronize()
                want = oracle.conv_wu(spec, nchw(x), nchw(dy))[0]
                got = g32.permute(2, 3, 0, 1)[None].cpu().numpy()
                what = f"weight gradient of a {len(pick)}-image batch (same entry point)"
        got = np.asarray(got, dtype=np.float64)
        want = np.asarray(want, dtype=np.float64).reshape(got.shape)
        rms = float(np.sqrt(np.mean(want * want))) if want.size else 0.0
        # (normalisation: outputs near zero carry the rounding of the whitened value, so the floor is rel * rms)
        abs_tol = max(T.ABS_TOL, (rel if self.kind == "norm" else 2.5e-4) * rms)
        bad, _, _ = oracle.check_is_close(got, want, rel, abs_tol)
        strict_bad, _, _ = oracle.check_is_close(got, want, rel, T.ABS_TOL)
        return {"sample": what, "elements": int(got.size), "bad": int(bad), "rel_tol": rel, "abs_tol": abs_tol,
                "passing_only_by_rms_floor": int(strict_bad - bad),
                "worst_abs_err_over_rms": float(np.abs(got - want).max() / rms) if rms else 0.0}

# --------------------------------------------------------------------------- CPU arm

def cpu_reference_rate(name, spec, budget_s=12.0):
    """TFLOP/s of the reference's CPU model on this host, on a bounded sample
    of the workload, all host cores in use (one slice of the sample per
    thread; the models are single-threaded and pure).  Returns a dict."""
    import oracle
    from oracle import ConvSpec
    use_ref = oracle.have_ref()
    cores = os.cpu_count() or 1
    threads = max(1, min(cores, 64))
    r = np.random.default_rng(99)

    def run_parallel(fn, nslices):
        errs = []

        def body(i):
            try:
                fn(i)
            except Exception as e:  # pragma: no cover
                errs.append(e)
        ts = [threading.Thread(target=body, args=(i,)) for i in range(nslices)]
        t0 = time.perf_counter()
        for t in ts:
            t.start()
        for t in ts:
            t.join()
        if errs:
            raise errs[0]
        return time.perf_counter() - t0

    if spec["kind"] == "conv":
        kw = dict(spec["params"])
        pass_ = spec["pass_"]

        def make(batch):
            nd = len(kw["field"])
            pad = kw.get("padding", 0)
            return ConvSpec.simple(batch, kw["field"], kw["kernel"], kw["in_chans"], kw["out_chans"],
                                   padding=pad, stride=kw.get("stride", 1))
        one = make(1)
        xs, ws, ys = oracle._shapes(one)
        x, w, dy = r.uniform(-1, 1, xs), r.uniform(-1, 1, ws), r.uniform(-1, 1, ys)

        def call(_):
            if pass_ == "fwd":
                oracle.conv_fwd(one, x, w, threads=1, use_ref=use_ref)
            elif pass_ == "bwd":
                oracle.conv_bwd(one, dy, w, threads=1, use_ref=use_ref)
            else:
                oracle.conv_wu(one, x, dy, threads=1, use_ref=use_ref)
        t1 = run_parallel(call, 1)                     # calibration: one image on one core
        rounds = int(max(1, min(8, budget_s / max(t1 * 1.3, 1e-3))))
        images = 0
        elapsed = 0.0
        for _ in range(rounds):
            elapsed += run_parallel(call, threads)
            images += threads
        flops = 2 * one.macs() * images
        sample = f"{images} images of the layer (one per thread per round, {rounds} round(s))"
    else:
        m, k, n = spec["m"], spec["k"], spec["n"]
        rows = max(1, min(m, int(2.0e9 * budget_s / 12.0 / max(k * n, 1) / 1)))  # ~bounded MACs per thread
        rows = max(1, min(rows, 16))
        a = r.uniform(-1, 1, (rows, k))
        b = r.uniform(-1, 1, (k, n))

        def call(_):
            oracle.gemm(a, b, threads=1, use_ref=use_ref)
        elapsed = run_parallel(call, threads)
        flops = 2 * rows * k * n * threads
        sample = f"{rows} rows of A per thread x full B ({threads} threads)"
    return {"value": flops / elapsed / 1e12, "unit": "TFLOP/s", "cores": threads,
            "kind": "reference" if use_ref else "port", "sample": sample}


# --------------------------------------------------------------------------- main

# steps of the additional workloads timed in the same process (bounded so that
# the default run stays within minutes)
EXTRA_STEPS = {"matmul_fp16_8192": 50, "matmul_fp8_8192": 50, "conv7x7_s2_fwd_n256_224x224_c3_c64": 100}
EXTRA_STEPS_DEFAULT = 200
WU_WORKLOAD = "conv3x3_wu_n256_28x28_c128"


def roofline_of(name, spec, flops, nbytes, ms_per_step, peaks, peak_src):
    per_launch_s = ms_per_step * 1e-3
    if spec["bound"] == "hbm":
        achieved, peak, unit = nbytes / per_launch_s / 1e9, peaks["hbm_gbs"], "GB/s"
        src = f"of {peak_src} (copy bandwidth)"
    elif spec.get("quarter"):
        achieved, peak, unit = flops / per_launch_s / 1e12, FP8_PEAK_TFLOPS["burst"], "TFLOP/s"
        src = FP8_PEAK_TFLOPS["source"]
    else:
        achieved, peak, unit = flops / per_launch_s / 1e12, peaks["bf16_tflops"], "TFLOP/s"
        src = f"of {peak_src} (burst)"
    extra = {}
    if spec["bound"] == "tensor" and ms_per_step > 0.2:
        # a kernel this long runs under the power cap within its own duration: also
        # against the sustained figure (MEASURED_PEAKS.json / the fp8 measurement)
        sustained = FP8_PEAK_TFLOPS["sustained"] if spec.get("quarter") else peaks["bf16_tflops_sustained"]
        extra = {"frac_of_sustained_peak": achieved / sustained, "sustained_peak": sustained}
    return {"bound": spec["bound"], "achieved": achieved, "peak": peak, "unit": unit, "frac": achieved / peak, **extra,
            "traffic": NCU_DRAM_TRAFFIC_BYTES.get(name), "peak_source": src,
            "algorithmic_flops_per_launch": flops, "algorithmic_bytes_per_launch": nbytes}


def measure_memory_mix(stream_bytes=1 << 29, reps=20):
    """TB/s of the library's streaming probe (plb_memory_mix_probe: one grid-stride
    kernel of 16-byte accesses) for mixes of read and write streams of 512 MB
    each, timed with CUDA events over `reps` launches after 3 warm-up launches.
    Prints one JSON line."""
    import torch
    from poplibs_b200 import capi
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = torch.cuda.Stream(device=dev)
    ctx = capi.Context(0, stream=stream.cuda_stream)
    src = torch.empty(stream_bytes, dtype=torch.uint8, device=dev)
    dst = torch.empty(4 * stream_bytes, dtype=torch.uint8, device=dev)
    src.random_(0, 255)
    out = {}
    for name, reads, writes in (("write_only", 0, 1), ("read_only", 1, 0), ("copy_1r_1w", 1, 1),
                                ("1r_2w", 1, 2), ("1r_4w", 1, 4)):
        for _ in range(3):
            ctx.memory_mix_probe(reads, writes, stream_bytes, src, dst)
        ctx.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        with torch.cuda.stream(stream):
            start.record()
            for _ in range(reps):
                ctx.memory_mix_probe(reads, writes, stream_bytes, src, dst)
            end.record()
        end.synchronize()
        out[name] = round((reads + writes) * stream_bytes * reps / (start.elapsed_time(end) * 1e-3) / 1e12, 3)
    print(json.dumps({"memory_mix_tb_per_s": out, "stream_bytes": stream_bytes, "reps": reps,
                      "kernel": "plb_memory_mix_probe (grid-stride, 16-byte accesses, 16 blocks of 512 threads per SM)"}))


def measure_fp8_peak(n=8192, sustained_s=4.0):
    """Dense e4m3 x e4m3 -> bf16 GEMM of the vendor library on n^3: best of 10
    launches (burst) and back to back for `sustained_s` seconds (sustained),
    SM clocks sampled during the sustained loop.  Read-only: no GPU setting is
    touched.  Prints one JSON line."""
    import torch
    dev = torch.device("cuda", 0)
    a = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
    b = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn).t()      # column-major right operand
    one = torch.ones((), device=dev, dtype=torch.float32)
    run = lambda: torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)  # noqa: E731
    for _ in range(5):
        run()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(10):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        run()
        e.record()
        e.synchronize()
        best = min(best, s.elapsed_time(e))
    sampler = ClockSampler(0)
    sampler.start()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    iters, t0 = 0, time.perf_counter()
    s.record()
    while time.perf_counter() - t0 < sustained_s:
        for _ in range(50):
            run()
        iters += 50
        torch.cuda.synchronize()
    e.record()
    e.synchronize()
    clocks = sampler.stop()
    flops = 2.0 * n ** 3
    print(json.dumps({"fp8_tflops": flops / (best * 1e-3) / 1e12,
                      "fp8_tflops_sustained": flops * iters / (s.elapsed_time(e) * 1e-3) / 1e12,
                      "how": f"torch._scaled_mm e4m3 x e4m3 -> bf16, {n}^3: best of 10 (burst), "
                             f"back to back for {sustained_s} s (sustained)", "clocks": clocks}))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true",
                    help="time only --workload (skip the other configurations, the multi-GPU weight "
                         "update and the strong-scaling shapes that are added to the line by default)")
    ap.add_argument("--no-graph", action="store_true",
                    help="time one library call per step instead of replaying CUDA graphs")
    ap.add_argument("--allreduce", default="auto", choices=["auto", "fused", "fused_all", "fused_owners", "oneshot", "rs", "nccl"],
                    help="how the multi-GPU weight update sums the per-rank gradients")
    ap.add_argument("--buffer-sets", type=int, default=0,
                    help="number of rotating buffer sets (default: enough to exceed L2; 1 = every step "
                         "re-reads the same, L2-resident, inputs: a diagnostic, not a bench value)")
    ap.add_argument("--measure-fp8-peak", action="store_true",
                    help="measure the dense fp8 (e4m3) peak of this GPU with the library GEMM "
                         "(torch._scaled_mm, 8192^3) and print it: the roofline denominator of the "
                         "fp8 workloads, not a result of this library")
    ap.add_argument("--measure-memory-mix", action="store_true",
                    help="measure what a streaming kernel of 16-byte accesses gets from the memory system "
                         "for several mixes of reads and writes (write only ... one read per four writes) "
                         "and print it: context for the fractions of the HBM-bound workloads")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.measure_fp8_peak:
        measure_fp8_peak()
        return
    if args.measure_memory_mix:
        measure_memory_mix()
        return

    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    spec = WORKLOADS[args.workload]
    metric = "conv/matMul TFLOP/s (fp16, fp8) at 1/2/4/8 B200; % of tensor-core peak"
    config = {"workload": args.workload, "plan": None, "per_gpu_batch": None,
              "l2": "rotating buffer sets larger than L2 (inputs of step i+1 are not those of step i)"}

    if args.impl == "reference":
        # The reference's own CPU implementation of the path on the host cores.
        if rank != 0:
            return
        steps = max(1, min(args.steps, 3))
        best = None
        t0 = time.perf_counter()
        for _ in range(steps):
            res = cpu_reference_rate(args.workload, spec, budget_s=6.0)
            best = res if best is None or res["value"] > best["value"] else best
        elapsed = time.perf_counter() - t0
        if spec["kind"] == "conv":
            config["per_gpu_batch"] = spec["params"]["batch"]
            config["global_batch"] = spec["params"]["batch"] * world
        # the same description of the workload as the library's arm gives (the
        # plan is host-side arithmetic; it needs the library, not a GPU)
        try:
            config["plan"] = workload_plan(spec)
        except (ImportError, OSError):
            config["plan"] = None
        line = {"impl": "reference", "metric": metric, "value": best["value"], "unit": "TFLOP/s",
                "n_gpus": args.gpus, "steps": steps, "warmup": 0, "ms_per_step": elapsed / steps * 1e3,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64",
                "data": "synthetic", "config": config, "cpu_baseline": best,
                "e2e": {"value": best["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0,
                        "d2h_bytes_per_step": 0}, "gpu_launches": 0}
        print(json.dumps(line))
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; the product has no CPU path "
                         "(use --impl reference for the CPU model)")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    from poplibs_b200 import capi

    # the library enqueues on a torch stream so that NCCL collectives (the
    # checker of the multi-GPU weight update) are ordered with the kernels
    stream = torch.cuda.Stream(device=device)
    ctx = capi.Context(local_rank, stream=stream.cuda_stream)
    peaks, peak_src = load_peaks()

    def barrier():
        torch.cuda.synchronize()
        ctx.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms):
        if world > 1:
            t = torch.tensor([ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    def timed(wl, step_fn, steps, warmup, use_graph):
        """Device time of exactly `steps` calls of step_fn.  With use_graph the
        steps are replayed from CUDA graphs, which takes the host's per-launch
        cost (argument marshalling, tensor-map encoding) out of a loop of
        microsecond kernels: up to 512 steps are one graph of `steps` nodes
        (buffer sets in rotation); more are one graph of wl.nsets consecutive
        steps replayed steps // nsets times plus one of the steps % nsets
        remaining steps.  Returns (ms, launches, graphed)."""
        with torch.cuda.stream(stream):
            for i in range(warmup):
                step_fn(i)
        barrier()
        graphs = None
        if use_graph:
            try:
                graphs = []
                replays, rest = divmod(steps, wl.nsets)
                for n, times in (((steps, 1), (0, 0)) if steps <= 512 else ((wl.nsets, replays), (rest, 1))):
                    if n == 0 or times == 0:
                        continue
                    g = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(g, stream=stream):
                        for i in range(n):
                            step_fn(i)
                    with torch.cuda.stream(stream):
                        g.replay()  # untimed: uploads the graph
                    graphs.append((g, times))
                barrier()
            except Exception as e:  # capture not possible: plain launches
                print(f"bench: CUDA graph capture failed ({type(e).__name__}: {e}); "
                      "timing plain launches", file=sys.stderr)
                graphs = None
                torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0 = ctx.launch_count()
        with torch.cuda.stream(stream):
            start.record()
            if graphs is not None:
                for g, times in graphs:
                    for _ in range(times):
                        g.replay()
            else:
                for i in range(steps):
                    step_fn(warmup + i)
            end.record()
        end.synchronize()
        barrier()
        ms = max_over_ranks(start.elapsed_time(end))
        launches = ctx.launch_count() - launches0
        if graphs is not None:
            launches += steps * wl.launches_per_step   # replayed kernels are not counted by the library
        return ms, launches, graphs is not None

    def count_launches(wl, step_fn):
        n0 = ctx.launch_count()
        with torch.cuda.stream(stream):
            step_fn(0)
        barrier()
        wl.launches_per_step = ctx.launch_count() - n0

    def timed_e2e(wl, steps, warmup):
        """Device time of `steps` end-to-end steps over the two e2e streams."""
        wl.e2e_ctx = [capi.Context(local_rank), capi.Context(local_rank)]
        for i in range(warmup):
            wl.step_e2e(i)
        for c in wl.e2e_ctx:
            c.synchronize()
        barrier()
        s_a, s_b = (torch.cuda.ExternalStream(c.stream, device=device) for c in wl.e2e_ctx)
        start, end_b, end = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        start.record(s_a)
        s_b.wait_event(start)
        for i in range(steps):
            wl.step_e2e(i)
        end_b.record(s_b)
        s_a.wait_event(end_b)
        end.record(s_a)
        end.synchronize()
        for c in wl.e2e_ctx:
            c.synchronize()
        barrier()
        return max_over_ranks(start.elapsed_time(end))

    def with_clocks(fn):
        sampler = ClockSampler(local_rank)
        if rank == 0:
            sampler.start()
        out = fn()
        return out, (sampler.stop() if rank == 0 else None)

    # ---- the workload the headline is quoted on ------------------------------------------
    wl = Workload(args.workload, spec, ctx, device, rank, world, force_sets=args.buffer_sets,
                  allreduce=args.allreduce)
    config["plan"] = wl.plan
    run = {"buffer_sets": wl.nsets}   # how this arm ran the workload (not part of its description)
    if args.buffer_sets > 0:
        config["l2"] = f"DIAGNOSTIC: {wl.nsets} buffer set(s) forced; inputs may stay in L2 between steps"
    if spec["kind"] == "conv":
        config["per_gpu_batch"] = spec["params"]["batch"]
        config["global_batch"] = spec["params"]["batch"] * world
    if wl.sharded is not None:
        run["allreduce"] = wl.allreduce
        run["allreduce_check"] = wl.check_allreduce()
    count_launches(wl, wl.step)
    # The multi-GPU weight update passes a step counter to its kernels, so its
    # steps cannot be replayed from a graph.
    use_graph = not args.no_graph and wl.sharded is None
    (ms, launches, graphed), clocks = with_clocks(lambda: timed(wl, wl.step, args.steps, args.warmup, use_graph))
    run["launch"] = ((f"one CUDA graph of {args.steps} steps, buffer sets in rotation" if args.steps <= 512
                         else f"CUDA graphs of {wl.nsets} steps (one per buffer set) and of the remaining "
                              f"{args.steps % wl.nsets}, replayed: exactly {args.steps} steps") if graphed
                        else "one library call per step")
    ms_per_step = ms / args.steps
    value = wl.flops * world / (ms_per_step * 1e-3) / 1e12
    parity = wl.parity_check() if rank == 0 else None

    e2e = None
    if wl.has_e2e() and wl.host is not None:
        e2e_steps = max(4, min(args.steps, 40))
        ms_e = timed_e2e(wl, e2e_steps, 3)
        e2e = {"value": wl.flops * world / (ms_e / e2e_steps * 1e-3) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": wl.h2d_bytes, "d2h_bytes_per_step": wl.d2h_bytes,
               "ms_per_step": ms_e / e2e_steps, "host_binding": wl.host_binding,
               "note": "one layer per call: 25.8 MB over PCIe per 7.2 GFLOP, bound by the host link"
               if args.workload == DEFAULT_WORKLOAD else None}
        wl.e2e_ctx = None
    roofline = roofline_of(args.workload, spec, wl.flops, wl.bytes, ms_per_step, peaks, peak_src)
    del wl
    torch.cuda.empty_cache()

    # ---- the other configurations, same process, bounded step counts -----------------------
    workloads = None
    if not args.no_extra and world == 1:
        workloads = {}
        for name, sp in WORKLOADS.items():
            if name == args.workload:
                continue
            try:
                w2 = Workload(name, sp, ctx, device, host_copies=False)
                count_launches(w2, w2.step)
                steps2 = EXTRA_STEPS.get(name, EXTRA_STEPS_DEFAULT)
                (ms2, _, g2), clk2 = with_clocks(lambda: timed(w2, w2.step, steps2, 5, not args.no_graph))
                per = ms2 / steps2
                workloads[name] = {"ms_per_step": per, "steps": steps2,
                                   "tflops": w2.flops / (per * 1e-3) / 1e12 if w2.flops else None,
                                   "roofline": roofline_of(name, sp, w2.flops, w2.bytes, per, peaks, peak_src),
                                   "clocks": clk2, "launches_per_step": w2.launches_per_step,
                                   "graphed": g2, "parity_check": w2.parity_check()}
                del w2
            except Exception as e:  # one configuration failing must not lose the line
                workloads[name] = {"error": f"{type(e).__name__}: {e}"}
            torch.cuda.empty_cache()

    # ---- multi-GPU: the one collective of the path, and the shapes the path shards ---------
    wu = strong = None
    if not args.no_extra and world > 1 and args.workload != WU_WORKLOAD:
        sp = WORKLOADS[WU_WORKLOAD]
        w3 = Workload(WU_WORKLOAD, sp, ctx, device, rank, world, host_copies=False, allreduce=args.allreduce)
        check = w3.check_allreduce()
        count_launches(w3, w3.step)
        steps3 = 300
        (ms_d, _, _), clk3 = with_clocks(lambda: timed(w3, w3.step, steps3, 10, False))
        ms_l, _, _ = timed(w3, w3.step_local, steps3, 10, False)
        wu = {"workload": WU_WORKLOAD, "per_gpu_batch": sp["params"]["batch"], "ms_per_step": ms_d / steps3,
              "tflops": w3.flops * world / (ms_d / steps3 * 1e-3) / 1e12, "allreduce": w3.allreduce,
              "allreduce_check": check, "local_ms_per_step": ms_l / steps3,
              "efficiency_vs_local": ms_l / ms_d, "launches_per_step": w3.launches_per_step, "clocks": clk3,
              "note": "weak scaling; local = the same rank's weight update without the sum over ranks, "
                      "timed in the same process (max over ranks)"}
        del w3
        torch.cuda.empty_cache()
        # strong scaling: the stated configurations sharded over the ranks (no collective)
        strong = {}
        from poplibs_b200 import parallel
        for name in ("conv3x3_fwd_n256_28x28_c128", "matmul_fp16_8192"):
            sp = dict(WORKLOADS[name])
            if sp["kind"] == "conv":
                b, e = parallel.shard_range(sp["params"]["batch"], rank, world)
                sp["params"] = dict(sp["params"], batch=e - b)
                total = 2 * capi.ConvParams.make(**WORKLOADS[name]["params"]).macs()
            else:
                b, e = parallel.shard_range(sp["m"], rank, world)
                sp["m"] = e - b
                total = 2 * WORKLOADS[name]["m"] * sp["k"] * sp["n"]
            w4 = Workload(name, sp, ctx, device, rank, 1, host_copies=False)
            count_launches(w4, w4.step)
            steps4 = EXTRA_STEPS.get(name, EXTRA_STEPS_DEFAULT)
            ms4, _, _ = timed(w4, w4.step, steps4, 5, not args.no_graph)
            strong[name] = {"per_gpu_share": e - b, "ms_per_step": ms4 / steps4,
                            "tflops_total": total / (ms4 / steps4 * 1e-3) / 1e12}
            del w4
            torch.cuda.empty_cache()

    if rank == 0:
        cpu = None
        if not args.no_cpu_baseline and world == 1:
            cpu = cpu_reference_rate(args.workload, spec)
        line = {"metric": metric, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f8e4m3" if spec.get("quarter") else "f16",
                "data": "synthetic", "config": config, "run": run, "clocks": clocks, "e2e": e2e,
                "gpu_launches": launches, "roofline": roofline, "cpu_baseline": cpu,
                "parity_check": parity}
        if workloads is not None:
            line["workloads"] = workloads
        if wu is not None:
            line["wu"] = wu
            line["strong_scaling"] = strong
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
