#!/usr/bin/env python
"""Benchmark of the poplin contraction path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

A step is one pass of the hot path (one convolution / matrix product call)
over one batch of synthetic input.  The default workload is the ResNet 3x3
forward convolution the metric is quoted on; the other named configurations
can be selected with --workload.  One JSON line is printed by rank 0.

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

With N > 1 (launched under torchrun) every rank runs the same per-GPU
workload on its own shard of a batch N times larger (weak scaling; the path
needs no collective in the forward pass; the weight update sums the per-rank
gradients with the library's all-reduce kernel over NVLink peer memory).
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
    "conv3x3_fwd_n32_56x56_c64": 12987392,
    "conv3x3_fwd_n256_28x28_c128": 51742720 + 10673664,
    "conv3x3_bwd_n256_28x28_c128": 51746048 + 10921728,
    "conv3x3_wu_n256_28x28_c128": 105506304 + 5284096,
    "conv1x1_s2_fwd_n256_56x56_c256_c512": 103098624 + 147304192,
    "conv7x7_s2_fwd_n256_224x224_c3_c64": 114623744 + 352808192,   # the implicit-GEMM kernel of the three
    "matmul_fp16_512x1024x1024": 3208192,
    "matmul_fp16_8192": 1096498000 + 126829568,
    "matmul_fp8_8192": 344297728 + 116545280,
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

class Workload:
    """Device-resident rotating buffer sets (so that consecutive steps do not
    find their inputs in L2) and pinned host copies for the end-to-end leg."""

    def __init__(self, name, spec, ctx, device, rank=0, world=1, sets_bytes_target=300 << 20, force_sets=0):
        import torch
        from poplibs_b200 import capi
        self.name, self.spec, self.ctx, self.capi = name, spec, ctx, capi
        self.rank, self.world = rank, world
        g = torch.Generator(device="cpu").manual_seed(1234)
        self.kind = spec["kind"]
        if self.kind == "conv":
            p = capi.ConvParams.make(**spec["params"])
            self.p = p
            kw = spec["params"]
            of = p.output_field()
            ci, co = p.in_chans_per_group, p.out_chans_per_group
            self.flops = 2 * p.macs()
            x_shape = (p.batch, *kw["field"], ci)
            y_shape = (p.batch, *of, co)
            w_shape = (*kw["kernel"], co, ci)
            bound = 1.0 / np.sqrt(ci * int(np.prod(kw["kernel"])))
            self.host = {
                "x": (torch.rand(x_shape, generator=g) * 2 - 1).half().pin_memory(),
                "w": ((torch.rand(w_shape, generator=g) * 2 - 1) * bound).half().pin_memory(),
                "dy": (torch.rand(y_shape, generator=g) * 2 - 1).half().pin_memory(),
            }
            self.pass_ = spec["pass_"]
            if world > 1:
                from poplibs_b200 import parallel
                # weak scaling: every rank holds one full per-GPU batch of the layer
                glob = dict(kw, batch=kw["batch"] * world)
                self.allreduce = "none (no collective on this pass)"
                ar = os.environ.get("PLB_BENCH_ALLREDUCE", "p2p")   # p2p | p2p_fused | p2p_oneshot | p2p_rs | nccl
                peer = self.pass_ == "wu" and ar.startswith("p2p")
                ar_mode = {"p2p_oneshot": "oneshot", "p2p_rs": "rs", "p2p_fused": "fused"}.get(ar, "auto")
                # PLB_BENCH_OVERLAP=1: the all-reduce of step i runs on a stream of its own, behind
                # step i + 1's kernels.  Off by default: the event between the kernels costs the
                # programmatic launch overlap, and the measured step is not shorter
                # (2 GPUs 57.1 vs 59.8 us, 8 GPUs 72.4 vs 68.8 us).
                overlap = peer and os.environ.get("PLB_BENCH_OVERLAP", "0") == "1"
                try:
                    self.sharded = parallel.ShardedConv(ctx, glob, rank, world, peer_allreduce=peer,
                                                        overlap_allreduce=overlap, allreduce_mode=ar_mode)
                    if self.pass_ == "wu":
                        self.allreduce = ((f"library kernel over NVLink peer memory ({self.sharded.peer.mode})"
                                           + (", overlapped with the next step on a second stream" if overlap else ""))
                                          if peer else "nccl all_reduce + cast")
                except Exception as e:  # symmetric memory unavailable: the process group's all-reduce
                    self.sharded = parallel.ShardedConv(ctx, glob, rank, world)
                    self.allreduce = f"nccl all_reduce + cast (peer memory unavailable: {type(e).__name__})"
            pass_id = {"bwd": capi.PASS_TRAINING_BWD, "wu": capi.PASS_TRAINING_WU}.get(
                self.pass_, capi.PASS_TRAINING_FWD)
            self.plan = capi.conv_plan(p, pass_id).as_dict()
            self.bytes = self.plan["bytes"]
            per_set = 2 * (int(np.prod(x_shape)) + int(np.prod(y_shape)))
            out_shape = {"fwd": y_shape, "bwd": x_shape, "wu": w_shape}[self.pass_]
        else:
            m, k, n = spec["m"], spec["k"], spec["n"]
            self.quarter = spec["quarter"]
            self.desc = capi.MatmulDesc.make(m, k, n, input_type=capi.QUARTER if self.quarter else capi.HALF,
                                             transpose_b=self.quarter,
                                             scale_a=-3 if self.quarter else 0, scale_b=-2 if self.quarter else 0)
            self.flops = 2 * m * k * n
            self.plan = capi.matmul_plan(self.desc).as_dict()
            self.bytes = self.plan["bytes"]
            if self.quarter:
                a = torch.randn((m, k), generator=g).mul_(8).to(torch.float8_e4m3fn).view(torch.uint8)
                b = torch.randn((n, k), generator=g).mul_(4).to(torch.float8_e4m3fn).view(torch.uint8)
            else:
                a = torch.randn((m, k), generator=g).half()
                b = torch.randn((k, n), generator=g).half()
            self.host = {"a": a.pin_memory(), "b": b.pin_memory()}
            per_set = a.numel() * a.element_size() + b.numel() * b.element_size() + 2 * m * n
            out_shape = (m, n)
        self.nsets = int(max(2, min(16, -(-sets_bytes_target // max(per_set, 1)))))
        if force_sets > 0:
            self.nsets = force_sets
        self.dev = []
        for _ in range(self.nsets):
            d = {k: v.to(device, non_blocking=False) for k, v in self.host.items()}
            d["out"] = torch.empty(out_shape, dtype=torch.float16, device=device)
            if self.kind == "conv" and self.pass_ == "wu":
                d["out32"] = torch.empty(out_shape, dtype=torch.float32, device=device)
            self.dev.append(d)
        # end-to-end leg: two contexts (streams) and two pinned output buffers
        self.host_out = [torch.empty(out_shape, dtype=torch.float16).pin_memory() for _ in range(2)]
        self.e2e_ctx = None
        self.h2d_bytes = sum(v.numel() * v.element_size() for k, v in self.host.items()
                             if self._is_input(k))
        self.d2h_bytes = self.host_out[0].numel() * 2
        torch.cuda.synchronize()

    def _is_input(self, key):
        if self.kind == "gemm":
            return True
        return key in {"fwd": ("x", "w"), "bwd": ("dy", "w"), "wu": ("x", "dy")}[self.pass_]

    def step(self, i):
        d = self.dev[i % self.nsets]
        if self.kind == "gemm":
            self.ctx.matmul(self.desc, d["a"], d["b"], None, d["out"])
        elif self.pass_ == "fwd":
            self.ctx.conv_fwd(self.p, d["x"], d["w"], d["out"])
        elif self.pass_ == "bwd":
            self.ctx.conv_bwd(self.p, d["dy"], d["w"], d["out"])
        elif self.world == 1:
            self.ctx.conv_wu(self.p, d["x"], d["dy"], d["out"], d["out32"])
        else:
            # per-rank batch reduced locally, then the one collective of the path
            self.sharded.wu(d["x"], d["dy"], d["out"], d["out32"])

    def check_allreduce(self):
        """One untimed step of the multi-GPU weight update compared with the
        process group's own all-reduce of the per-rank gradients."""
        import torch
        import torch.distributed as dist
        d = self.dev[0]
        local = torch.empty_like(d["out32"])
        self.ctx.conv_wu(self.p, d["x"], d["dy"], None, local)
        self.ctx.synchronize()
        dist.all_reduce(local)
        self.sharded.wu(d["x"], d["dy"], d["out"], d["out32"])
        self.ctx.synchronize()
        self.sync_comm()
        torch.cuda.synchronize()
        diff = float((local - d["out32"]).abs().max().item())
        scale = float(local.abs().max().item())
        return {"max_abs_diff_vs_nccl": diff, "max_abs": scale}

    def sync_comm(self):
        """Waits for the communication stream of an overlapped all-reduce (and checks its status)."""
        sharded = getattr(self, "sharded", None)
        if sharded is not None and sharded.peer is not None:
            sharded.peer.synchronize()

    def join_comm(self):
        """Orders the main stream after the latest overlapped all-reduce."""
        sharded = getattr(self, "sharded", None)
        if sharded is not None and sharded.peer is not None:
            sharded.peer.wait()

    def comm_launches(self):
        sharded = getattr(self, "sharded", None)
        if sharded is not None and sharded.peer is not None and sharded.peer.overlap:
            return sharded.peer.comm_ctx.launch_count()
        return 0

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
        elif self.pass_ == "fwd":
            c.conv_fwd_host(self.p, self.host["x"], self.host["w"], out, sync=False)
        else:
            raise RuntimeError("end-to-end leg is defined for the forward pass and matMul")

    def has_e2e(self):
        return self.kind == "gemm" or self.pass_ == "fwd"


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

def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=50)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-graph", action="store_true",
                    help="time one library call per step instead of replaying a CUDA graph")
    ap.add_argument("--buffer-sets", type=int, default=0,
                    help="number of rotating buffer sets (default: enough to exceed L2; 1 = every step "
                         "re-reads the same, L2-resident, inputs: a diagnostic, not a bench value)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

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
        flops_per_step = None
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

    # the library enqueues on a torch stream so that NCCL collectives (weight
    # update at N > 1) are ordered with the kernels without host synchronisation
    torch_stream = torch.cuda.Stream(device=device)
    ctx = capi.Context(local_rank, stream=torch_stream.cuda_stream)
    wl = Workload(args.workload, spec, ctx, device, rank, world, force_sets=args.buffer_sets)
    config["plan"] = wl.plan
    config["buffer_sets"] = wl.nsets
    if args.buffer_sets > 0:
        config["l2"] = f"DIAGNOSTIC: {wl.nsets} buffer set(s) forced; inputs may stay in L2 between steps"
    if world > 1 and spec["kind"] == "conv":
        config["allreduce"] = wl.allreduce
        if spec["pass_"] == "wu":
            config["allreduce_check"] = wl.check_allreduce()
    if spec["kind"] == "conv":
        config["per_gpu_batch"] = spec["params"]["batch"]
        config["global_batch"] = spec["params"]["batch"] * world
    stream = torch_stream

    def barrier():
        torch.cuda.synchronize()
        ctx.synchronize()
        wl.sync_comm()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(step_fn, steps, warmup, graph_sets=0):
        """Times `steps` calls of step_fn on the device.  With graph_sets = n the
        steps are replayed from a CUDA graph of n consecutive steps (one per
        rotating buffer set), which takes the host's per-launch cost (argument
        marshalling, tensor-map encoding) out of a loop of microsecond kernels."""
        with torch.cuda.stream(stream):
            for i in range(warmup):
                step_fn(i)
        barrier()
        graph = None
        if graph_sets:
            try:
                graph = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph, stream=stream):
                    for i in range(graph_sets):
                        step_fn(i)
                with torch.cuda.stream(stream):
                    graph.replay()  # untimed: uploads the graph
                barrier()
            except Exception as e:  # capture not possible: plain launches
                print(f"bench: CUDA graph capture failed ({type(e).__name__}: {e}); "
                      "timing plain launches", file=sys.stderr)
                graph = None
                torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        launches0, comm0 = ctx.launch_count(), wl.comm_launches()
        with torch.cuda.stream(stream):
            start.record()
            if graph is not None:
                replays, rest = divmod(steps, graph_sets)
                for _ in range(replays):
                    graph.replay()
                for i in range(rest):
                    step_fn(i)
            else:
                for i in range(steps):
                    step_fn(warmup + i)
            wl.join_comm()   # the last step's all-reduce belongs to the timed region
            end.record()
        end.synchronize()
        barrier()
        ms = start.elapsed_time(end)
        launches = ctx.launch_count() - launches0 + wl.comm_launches() - comm0
        if graph is not None:
            # replayed kernels are not counted by the library: add them
            launches += (steps // graph_sets) * graph_sets * wl.launches_per_step
        if world > 1:
            t = torch.tensor([ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms, launches, graph is not None

    def timed_e2e(steps, warmup):
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
        ms = start.elapsed_time(end)
        if world > 1:
            t = torch.tensor([ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # kernels per step, counted on one untimed step
    n0 = ctx.launch_count()
    with torch.cuda.stream(stream):
        wl.step(0)
    barrier()
    wl.launches_per_step = ctx.launch_count() - n0
    # The multi-GPU weight update passes a step counter to its all-reduce kernel,
    # so its steps cannot be replayed from a graph.
    use_graph = not args.no_graph and not (world > 1 and spec.get("pass_") == "wu")
    ms, launches, graphed = timed(wl.step, args.steps, args.warmup, wl.nsets if use_graph else 0)
    config["launch"] = (f"CUDA graph of {wl.nsets} steps (one per buffer set), replayed" if graphed
                        else "one library call per step")
    clocks = sampler.stop() if rank == 0 else None
    ms_per_step = ms / args.steps
    value = wl.flops * world / (ms_per_step * 1e-3) / 1e12

    e2e = None
    if wl.has_e2e():
        e2e_steps = max(4, min(args.steps, 40))
        ms_e = timed_e2e(e2e_steps, 3)
        e2e = {"value": wl.flops * world / (ms_e / e2e_steps * 1e-3) / 1e12, "unit": "TFLOP/s",
               "h2d_bytes_per_step": wl.h2d_bytes, "d2h_bytes_per_step": wl.d2h_bytes,
               "ms_per_step": ms_e / e2e_steps}

    if rank == 0:
        peaks, peak_src = load_peaks()
        per_launch_s = ms_per_step * 1e-3
        if spec["bound"] == "hbm":
            achieved = wl.bytes / per_launch_s / 1e9
            peak, unit = peaks["hbm_gbs"], "GB/s"
        else:
            achieved = wl.flops / per_launch_s / 1e12
            peak, unit = peaks["bf16_tflops"] * (2.0 if spec.get("quarter") else 1.0), "TFLOP/s"
        roofline = {"bound": spec["bound"], "achieved": achieved, "peak": peak, "unit": unit,
                    "frac": achieved / peak, "traffic": NCU_DRAM_TRAFFIC_BYTES.get(args.workload),
                    "peak_source": f"of {peak_src}" + (" (fp8 taken as 2 x the measured 16-bit burst peak)"
                                                        if spec.get("quarter") else " (burst)"),
                    "algorithmic_flops_per_launch": wl.flops, "algorithmic_bytes_per_launch": wl.bytes}
        cpu = None
        if not args.no_cpu_baseline and world == 1:
            cpu = cpu_reference_rate(args.workload, spec)
        line = {"metric": metric, "value": value, "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
                "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "dtype": "f8e4m3" if spec.get("quarter") else "f16",
                "data": "synthetic", "config": config, "clocks": clocks, "e2e": e2e,
                "gpu_launches": launches, "roofline": roofline, "cpu_baseline": cpu}
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
