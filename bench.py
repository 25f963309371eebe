"""Benchmark of the flash-attention hot path: TFLOP/s of one forward+backward step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config C3] [--impl ours|reference]

A "step" is one forward and one backward pass of the attention operator over one batch of
seeded synthetic tensors.  With N > 1 (launched under ``torch.distributed.run``, one rank per
GPU) every rank owns an independent batch of the same size — the path shards over
(batch, kv-head group) units with no collective — so scaling is weak and ``value`` is the
aggregate over all ranks.  FLOPs follow the reference's convention: forward
``4*B*Hq*S*S*D`` halved when causal, backward 2.5x forward
(benchmarks/test_attention.py:46,163).

Rank 0 prints ONE JSON line.  ``value`` is timed with CUDA events on tensors already resident
in HBM; ``e2e`` runs the same step through the public `mojo`-device operator API with pinned
HOST buffers, host<->device copies inside the timed region (headline: the batch pipelined in
pieces over three streams; ``e2e.single_call``: one call over the whole batch on one stream); ``roofline`` times the dominant
kernel (the backward dK/dV kernel) alone; ``cpu_baseline`` is the CPU oracle timed on the
host cores on a bounded slice of the same workload.
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

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "flash-attn fwd+bwd TFLOP/s (bf16, causal)"
NOMINAL_BF16_TFLOPS = 2250.0
FALLBACK_BF16_TFLOPS = 1590.0
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the backward dK/dV kernel on the
# C3 workload, from the ncu capture summarised in profiles/bwd_dkdv_kernel_C3.md.
BWD_DKDV_DRAM_TRAFFIC_BYTES = 395.2e6


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return float(d["bf16_tflops"]), float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "measured"
    except Exception:
        return FALLBACK_BF16_TFLOPS, 1400.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML while the timed region runs
    (falls back to polling nvidia-smi when NVML bindings are unavailable)."""

    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index = gpu_index
        self.clocks: list[float] = []
        self.max_clock = None
        self.reasons: set[str] = set()
        self._stop = threading.Event()
        self._thread = None
        self._nvml = None
        try:
            import pynvml

            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = gpu_index
            if visible:
                entry = visible.split(",")[gpu_index].strip()
                if entry.isdigit():
                    phys = int(entry)
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_clock = float(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
            self._nvml = pynvml
        except Exception:
            self._nvml = None

    def _sample_nvml(self):
        n = self._nvml
        self.clocks.append(float(n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM)))
        mask = n.nvmlDeviceGetCurrentClocksEventReasons(self._handle)
        for name, bit in (("hw_slowdown", n.nvmlClocksEventReasonHwSlowdown),
                          ("hw_thermal_slowdown", n.nvmlClocksEventReasonHwThermalSlowdown),
                          ("sw_thermal_slowdown", n.nvmlClocksEventReasonSwThermalSlowdown),
                          ("sw_power_cap", n.nvmlClocksEventReasonSwPowerCap)):
            if mask & bit:
                self.reasons.add(name)

    def _sample_smi(self):
        out = subprocess.run(
            ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits"],
            capture_output=True, text=True, timeout=5).stdout.strip()
        if not out:
            return
        s = [x.strip() for x in out.splitlines()[0].split(",")]
        self.clocks.append(float(s[0]))
        self.max_clock = float(s[1])
        for name, val in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], s[2:6]):
            if val.lower().startswith("active"):
                self.reasons.add(name)

    def _run(self):
        while not self._stop.is_set():
            try:
                if self._nvml is not None:
                    self._sample_nvml()
                else:
                    self._sample_smi()
            except Exception:
                pass
            self._stop.wait(0.002 if self._nvml is not None else 0.1)

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=10)

    def summary(self):
        return {
            "sm_mhz": statistics.median(self.clocks) if self.clocks else None,
            "sm_min_mhz": min(self.clocks) if self.clocks else None,
            "sm_max_mhz": self.max_clock,
            "reasons": sorted(self.reasons),
            "samples": len(self.clocks),
            "source": "nvml" if self._nvml is not None else "nvidia-smi",
        }


def dist_setup(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist

        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def barrier(world: int):
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    import torch.distributed as dist

    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def run_ours(args):
    from oracle import sdpa_oracle as O  # input generation + (rank 0, N=1) the cpu_baseline leg
    from torch_mojo_backend_b200 import _lib, raw

    rank, world, local = dist_setup(args.gpus)
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    cfg = O.CONFIGS[args.config]
    do_bwd = cfg.backward
    q, k, v, dout = (t.to(dev) for t in O.make_inputs(cfg, seed=rank))
    out = torch.empty_like(q)
    lse = torch.empty((cfg.B, cfg.Hq, cfg.S), dtype=torch.float32, device=dev)
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    code = raw.dtype_code(cfg.dtype)
    ws = torch.empty((_lib.bwd_workspace_bytes(cfg.B, cfg.Hq, cfg.Hkv, cfg.S, cfg.D, code),), dtype=torch.uint8,
                     device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    def step():
        raw.flash_fwd(q, k, v, causal=cfg.causal, scale=cfg.scale, out=out, lse=lse, status=status)
        if do_bwd:
            raw.flash_bwd(dout, q, k, v, out, lse, causal=cfg.causal, scale=cfg.scale, dq=dq, dk=dk, dv=dv,
                          workspace=ws, status=status)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier(world)
    launches0 = _lib.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    ef0, ef1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as sampler:
        barrier(world)
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        barrier(world)
        total_ms = max_over_ranks(e0.elapsed_time(e1), world)
        # forward-only and single-backward-kernel timings explain the step number
        ef0.record()
        for _ in range(args.steps):
            raw.flash_fwd(q, k, v, causal=cfg.causal, scale=cfg.scale, out=out, lse=lse, status=status)
        ef1.record()
        torch.cuda.synchronize()
        fwd_ms = ef0.elapsed_time(ef1) / args.steps
        bwd_part_ms = {}
        if do_bwd:
            for name, part in (("dkdv", 2), ("dq", 4)):
                eb0, eb1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                eb0.record()
                for _ in range(args.steps):
                    raw.flash_bwd(dout, q, k, v, out, lse, causal=cfg.causal, scale=cfg.scale, dq=dq, dk=dk, dv=dv,
                                  workspace=ws, status=status, parts=part)
                eb1.record()
                torch.cuda.synchronize()
                bwd_part_ms[name] = eb0.elapsed_time(eb1) / args.steps
    launches = (_lib.launch_count() - launches0)
    timed_launches = args.steps * (1 + (3 if do_bwd else 0))
    if int(status.item()) != 0:
        raise RuntimeError(f"kernel status word is 0x{int(status.item()) & 0xffffffff:x}")

    ms_per_step = total_ms / args.steps
    step_flops = cfg.fwd_flops() + (cfg.bwd_flops() if do_bwd else 0.0)
    value = world * step_flops / (ms_per_step * 1e-3) / 1e12

    # ---- end to end through the public operator API on the mojo device, host buffers in/out
    e2e = None if args.no_e2e else run_e2e(cfg, rank, world, local, args)

    burst, sustained, peak_src = load_peaks()
    if do_bwd:
        # The dK/dV kernel is the longest launch.  Its algorithmic work is the 4 tile GEMMs of the 5 a
        # backward needs that it covers (S^T, dP^T, dV, dK): 0.8 x the backward FLOPs (2.0 x forward).
        dom_flops, dom_ms, dom_name = 0.8 * cfg.bwd_flops(), bwd_part_ms["dkdv"], "bwd_dkdv_kernel (S^T, dP^T, dV, dK)"
    else:
        dom_flops, dom_ms, dom_name = cfg.fwd_flops(), fwd_ms, "fwd_kernel"
    achieved = dom_flops / (dom_ms * 1e-3) / 1e12
    roofline = {
        "bound": "tensor", "kernel": dom_name, "achieved": round(achieved, 2), "peak": burst, "unit": "TFLOP/s",
        "frac": round(achieved / burst, 4), "peak_source": f"of {peak_src} (cuBLAS bf16 burst)",
        "frac_of_nominal_2250": round(achieved / NOMINAL_BF16_TFLOPS, 4),
        "traffic": BWD_DKDV_DRAM_TRAFFIC_BYTES if (do_bwd and cfg.name == "C3") else None,
        "ms_per_launch": round(dom_ms, 4),
    }
    detail = {
        "fwd_ms": round(fwd_ms, 4), "fwd_tflops": round(cfg.fwd_flops() / (fwd_ms * 1e-3) / 1e12, 2),
        "fwd_frac_of_nominal_2250": round(cfg.fwd_flops() / (fwd_ms * 1e-3) / 1e12 / NOMINAL_BF16_TFLOPS, 4),
    }
    if do_bwd:
        bwd_ms = ms_per_step - fwd_ms
        detail.update({
            "bwd_ms": round(bwd_ms, 4), "bwd_tflops": round(cfg.bwd_flops() / (bwd_ms * 1e-3) / 1e12, 2),
            "bwd_frac_of_nominal_2250": round(cfg.bwd_flops() / (bwd_ms * 1e-3) / 1e12 / NOMINAL_BF16_TFLOPS, 4),
            "bwd_dkdv_kernel_ms": round(bwd_part_ms["dkdv"], 4), "bwd_dq_kernel_ms": round(bwd_part_ms["dq"], 4),
        })

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        # about ten seconds of CPU work on a bounded slice of the same workload
        tf, secs, threads, sample = O.time_cpu(cfg, backward=do_bwd, sample_heads=args.cpu_sample_heads, reps=2,
                                               target_seconds=10.0)
        cpu_baseline = {"value": round(tf, 4), "unit": "TFLOP/s", "cores": threads, "kind": "port",
                        "sample": sample}

    if rank == 0:
        line = {
            "metric": METRIC, "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": str(cfg.dtype).replace("torch.", ""),
            "data": "synthetic",
            "config": {
                "workload": f"{cfg.name}: {'causal' if cfg.causal else 'non-causal'} "
                            f"{'fwd+bwd' if do_bwd else 'fwd'} B={cfg.B} Hq={cfg.Hq} Hkv={cfg.Hkv} S={cfg.S} "
                            f"D={cfg.D} per GPU",
                "l2": "inputs larger than L2 (no flush needed)" if cfg.fwd_bytes() > 126e6
                      else "working set fits in L2 (L2-hot number)",
                "seed": "torch.Generator().manual_seed(rank); q,k,v,dO drawn in that order",
            },
            "frac_of_nominal_2250": round(value / world / NOMINAL_BF16_TFLOPS, 4),
            "detail": detail, "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
            "gpu_launches": int(launches), "gpu_launches_in_step_region": int(timed_launches),
            "clocks": sampler.summary(),
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


def run_e2e(cfg, rank, world, local, args):
    """Same step through the `mojo` device's operator API with HOST buffers: pinned host
    tensors in, out and gradients read back into pinned host tensors, all inside the timed
    region.  Two ways of driving it are timed:

    * ``single_call``: one F.scaled_dot_product_attention call and one ``backward`` over the
      whole batch, every copy and kernel on one stream (copies and compute in sequence);
    * the headline: the batch walked one batch entry at a time through
      ``aten::_scaled_dot_product_flash_attention`` and ``..._backward`` (the two operators the
      device registers), with uploads, kernels and downloads on three streams, so that PCIe in
      both directions and the kernels overlap.  Same inputs, same bytes moved, same results.
    """
    import torch_mojo_backend_b200 as tmb
    from oracle import sdpa_oracle as O

    tmb.register_mojo_devices()
    torch.mojo.set_device(local)
    cpu_inputs = O.make_inputs(cfg, seed=rank)
    host = []
    for t in cpu_inputs:
        p = tmb.pinned_empty(t.shape, t.dtype)
        p.copy_(t)
        host.append(p)
    hq, hk, hv, hdo = host
    steps = max(1, min(args.steps, 5))
    gqa = cfg.Hq != cfg.Hkv
    h2d = sum(t.numel() * t.element_size() for t in ((hq, hk, hv, hdo) if cfg.backward else (hq, hk, hv)))
    # results land in pre-pinned host buffers: out, and dq/dk/dv when the config has a backward
    res_out = tmb.pinned_empty(hq.shape, hq.dtype)
    res_grads = [tmb.pinned_empty(t.shape, t.dtype) for t in (hq, hk, hv)] if cfg.backward else []
    d2h = sum(t.numel() * t.element_size() for t in [res_out] + res_grads)
    dev = torch.device("mojo", local)

    def step():
        q = hq.to(dev, non_blocking=True)
        k = hk.to(dev, non_blocking=True)
        v = hv.to(dev, non_blocking=True)
        if cfg.backward:
            for t in (q, k, v):
                t.requires_grad_()
            do = hdo.to(dev, non_blocking=True)
        out = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=cfg.causal, scale=cfg.scale,
                                                               enable_gqa=gqa)
        res_out.copy_(out.detach(), non_blocking=True)
        if cfg.backward:
            out.backward(do)
            for dst, t in zip(res_grads, (q, k, v)):
                dst.copy_(t.grad, non_blocking=True)
        return res_out

    # ---- pipelined over the batch entries: three streams, events between them
    main = torch.cuda.current_stream(local)
    s_in, s_run, s_out = (torch.cuda.Stream(device=local) for _ in range(3))
    flash_fwd = torch.ops.aten._scaled_dot_product_flash_attention
    flash_bwd = torch.ops.aten._scaled_dot_product_flash_attention_backward

    # pieces: contiguous blocks of the host buffers, about 40 MB of upload each (smaller ones
    # cost more in host-side dispatch than the overlap wins) - ranges of batch entries, or, when
    # a single batch entry is larger than that, its kv heads in two groups (never cutting a GQA
    # group)
    rep_q = cfg.Hq // cfg.Hkv
    wanted = max(1, min(2 * cfg.B, h2d // (40 << 20)))
    if wanted <= cfg.B:
        bounds = [round(n * cfg.B / wanted) for n in range(wanted + 1)]
        pieces = [(slice(a, b), (slice(None), slice(None))) for a, b in zip(bounds, bounds[1:]) if b > a]
    else:
        split = 2 if cfg.Hkv % 2 == 0 else 1
        pieces = [(slice(i, i + 1), (slice(g * cfg.Hkv // split * rep_q, (g + 1) * cfg.Hkv // split * rep_q),
                                     slice(g * cfg.Hkv // split, (g + 1) * cfg.Hkv // split)))
                  for i in range(cfg.B) for g in range(split)]

    def step_pipelined(keep):
        """`keep` collects every device tensor of the step: the three streams use one another's
        allocations, so nothing may go back to the allocator before the final synchronisation."""
        for s in (s_in, s_run, s_out):
            s.wait_stream(main)
        for i, (qs, ks) in pieces:
            with torch.cuda.stream(s_in):
                dq_in = [hq[i, qs].to(dev, non_blocking=True), hk[i, ks].to(dev, non_blocking=True),
                         hv[i, ks].to(dev, non_blocking=True)]
                if cfg.backward:
                    dq_in.append(hdo[i, qs].to(dev, non_blocking=True))
                uploaded = torch.cuda.Event()
                uploaded.record(s_in)
            with torch.cuda.stream(s_run):
                s_run.wait_event(uploaded)
                fwd = flash_fwd(dq_in[0], dq_in[1], dq_in[2], 0.0, cfg.causal, False, scale=cfg.scale)
                out, lse = fwd[0], fwd[1]
                grads = ()
                if cfg.backward:
                    grads = flash_bwd(dq_in[3], dq_in[0], dq_in[1], dq_in[2], out, lse, None, None, fwd[4], fwd[5],
                                      0.0, cfg.causal, fwd[6], fwd[7], scale=cfg.scale)
                computed = torch.cuda.Event()
                computed.record(s_run)
            with torch.cuda.stream(s_out):
                s_out.wait_event(computed)
                res_out[i, qs].copy_(out, non_blocking=True)
                for dst, g, hs in zip(res_grads, grads, (qs, ks, ks)):
                    dst[i, hs].copy_(g, non_blocking=True)
            keep.extend(dq_in)
            keep.extend((out, lse) + tuple(grads))
        for s in (s_in, s_run, s_out):
            main.wait_stream(s)

    def time_steps(fn):
        barrier(world)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier(world)
        return max_over_ranks(e0.elapsed_time(e1), world) / steps

    flops = cfg.fwd_flops() + (cfg.bwd_flops() if cfg.backward else 0.0)
    for _ in range(2):
        step()
    ms_single = time_steps(step)
    # the pipelined walk must reproduce the single call bit for bit before it is timed
    torch.cuda.synchronize()
    ref = [res_out.clone()] + [g.clone() for g in res_grads]
    for t in [res_out] + res_grads:
        t.zero_()
    keep = []
    step_pipelined(keep)
    torch.cuda.synchronize()
    same = all(torch.equal(a, b) for a, b in zip(ref, [res_out] + res_grads))
    step_pipelined(keep)
    torch.cuda.synchronize()
    keep.clear()

    def pipelined_and_release():
        # the host reads the results after every step anyway; once the step has drained, its
        # device tensors go back to the allocator, so every step reuses the same blocks
        step_pipelined(keep)
        main.synchronize()
        keep.clear()

    ms_pipe = time_steps(pipelined_and_release)
    tf = lambda ms: round(world * flops / (ms * 1e-3) / 1e12, 2)
    pipelined = {"value": tf(ms_pipe), "ms_per_step": round(ms_pipe, 3), "pieces": len(pieces),
                 "matches_single_call_bitwise": bool(same),
                 "api": "aten::_scaled_dot_product_flash_attention + _backward on mojo tensors, the batch in "
                        f"{len(pieces)} contiguous pieces; uploads, kernels and downloads on three streams"}
    single = {"value": tf(ms_single), "ms_per_step": round(ms_single, 3),
              "api": "F.scaled_dot_product_attention + backward over the whole batch, one stream"}
    # both are the public operator API with pinned host buffers in and out; the headline is the
    # faster way of driving it for this workload (small steps do not repay the pipelining)
    best_ms, mode = (ms_pipe, "pipelined") if ms_pipe <= ms_single else (ms_single, "single_call")
    return {"value": tf(best_ms), "unit": "TFLOP/s", "ms_per_step": round(best_ms, 3), "steps": steps,
            "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "mode": mode,
            "pipelined": pipelined, "single_call": single}


def run_reference(args):
    """The reference arm: the reference's own path cannot be built here (it needs the Mojo
    toolchain), so — as its tests do — torch's CPU SDPA stands in, timed on all host cores on a
    bounded slice of the same workload.  Only rank 0 works."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import sdpa_oracle as O

    cfg = O.CONFIGS[args.config]
    threads = os.cpu_count() or 1
    vals, secs_all, sample = [], [], ""
    for i in range(args.warmup + args.steps):
        tf, secs, threads, sample = O.time_cpu(cfg, backward=cfg.backward, sample_heads=args.cpu_sample_heads, reps=1,
                                               threads=threads)
        if i >= args.warmup:
            vals.append(tf)
            secs_all.append(secs)
    value = statistics.median(vals)
    line = {
        "impl": "reference", "metric": METRIC, "value": round(value, 4), "unit": "TFLOP/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(1e3 * statistics.median(secs_all), 2), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": str(cfg.dtype).replace("torch.", ""), "data": "synthetic",
        "config": {"workload": f"{cfg.name} (CPU slice: {sample})"},
        "cpu_baseline": {"value": round(value, 4), "unit": "TFLOP/s", "cores": threads, "kind": "port",
                         "sample": sample},
        "e2e": {"value": round(value, 4), "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "reference's Mojo FA4 build is not installable offline and rejects sm_100; torch CPU SDPA "
                "(the oracle the reference's own tests use) is timed instead",
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--config", default="C3", choices=["C1", "C2", "C3", "C4", "C5"])
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--cpu-sample-heads", type=int, default=0,
                    help="KV-head groups of one batch entry in the CPU sample (0: sized to about 2 TFLOP a repetition)")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiling runs)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
