"""Benchmark of the flash-attention hot path: TFLOP/s of one forward(+backward) step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--config C3] [--scaling auto|weak|strong]
                    [--impl ours|reference]

A "step" is one forward and (where the configuration has one) one backward pass of the
attention operator over one batch of seeded synthetic tensors.  The path shards over
(batch, kv-head group) units with no collective.  With N > 1 (launched under
``torch.distributed.run``, one rank per GPU):

* ``weak`` scaling (the default for C1-C3): every rank owns an independent batch of the full
  per-GPU size, drawn from seed = rank; ``value`` is the aggregate over all ranks.
* ``strong`` scaling (the default for C4 and C5, the two configurations defined as a split of
  one problem): the full problem is drawn once from seed 0 and rank r takes its contiguous slice
  of the (batch, kv-head group) units - C4: 32 heads -> 4 per GPU at N = 8; C5: 64 batch entries
  -> 64/N per GPU.  After the timed region the shards' results are gathered on rank 0 with NCCL
  ``all_gather`` and compared, bit for bit, with rank 0's own run of the whole problem on one
  GPU (``validation`` in the JSON line).

FLOPs follow the reference's convention: forward ``4*B*Hq*S*S*D`` halved when causal, backward
2.5x forward (benchmarks/test_attention.py:46,163).

Rank 0 prints ONE JSON line.  ``value`` is timed with CUDA events on tensors already resident
in HBM; ``e2e`` runs the same step on HOST tensors through the package's public API
(``HostAttentionPipeline`` over the `mojo`-device operators; ``e2e.single_call``: one
``F.scaled_dot_product_attention`` + ``backward`` over the whole batch), host<->device copies
inside the timed region; ``roofline`` times the dominant kernel alone; ``cpu_baseline`` is the
CPU oracle timed on the host cores on a bounded slice of the same workload.
``detail`` times the forward, the backward and its kernels on their own and, on one GPU, the
split-KV decode call on a 32k-token cache with its HBM roofline (outside the timed region).
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

NOMINAL_BF16_TFLOPS = 2250.0
SEED_NOTE_WEAK = "torch.Generator().manual_seed(rank); q,k,v,dO drawn in that order"
FALLBACK_BF16_TFLOPS = 1590.0
# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from one
# ncu capture of that kernel on that workload (bytes per launch)
DRAM_TRAFFIC_BYTES = {("C3", "bwd_dkdv_kernel"): 395.7e6, ("C4", "fwd_kernel"): None}


def metric_name(cfg) -> str:
    dt = str(cfg.dtype).replace("torch.", "").replace("bfloat16", "bf16").replace("float16", "fp16").replace("float32", "fp32")
    return f"flash-attn {'fwd+bwd' if cfg.backward else 'fwd'} TFLOP/s ({dt}, {'causal' if cfg.causal else 'non-causal'})"


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
            self._stop.wait(0.004 if self._nvml is not None else 0.1)

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


def dist_setup():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist

        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        # each rank keeps to its own slice of the host cores (its copies and dispatch then do not
        # migrate across the other ranks' cores)
        try:
            cores = sorted(os.sched_getaffinity(0))
            per = max(1, len(cores) // world)
            os.sched_setaffinity(0, set(cores[local * per:(local + 1) * per]) or set(cores))
        except (AttributeError, OSError):
            pass
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


def shard_slices(cfg, rank: int, world: int):
    """(batch slice, query-head slice, kv-head slice) of rank `rank`: the contiguous slice of the
    flattened (batch, kv head) index it owns; the batch is split first, then kv heads with the
    query heads that read them (a GQA group is never split)."""
    group = cfg.Hq // cfg.Hkv
    if cfg.B % world == 0:
        per = cfg.B // world
        return slice(rank * per, (rank + 1) * per), slice(None), slice(None)
    if world % cfg.B == 0 and cfg.Hkv % (world // cfg.B) == 0:
        ranks_per_entry = world // cfg.B
        b, part = divmod(rank, ranks_per_entry)
        hk = cfg.Hkv // ranks_per_entry
        return slice(b, b + 1), slice(part * hk * group, (part + 1) * hk * group), slice(part * hk, (part + 1) * hk)
    raise ValueError(f"{cfg.name} does not split over {world} ranks")


def attention_step(raw, q, k, v, dout, cfg, bufs, status):
    raw.flash_fwd(q, k, v, causal=cfg.causal, scale=cfg.scale, out=bufs["out"], lse=bufs["lse"], status=status)
    if cfg.backward:
        raw.flash_bwd(dout, q, k, v, bufs["out"], bufs["lse"], causal=cfg.causal, scale=cfg.scale, dq=bufs["dq"],
                      dk=bufs["dk"], dv=bufs["dv"], workspace=bufs["ws"], status=status)


def make_bufs(_lib, raw, q, k, v, cfg):
    B, Hq, S, D = q.shape
    code = raw.dtype_code(q.dtype)
    bufs = {"out": torch.empty_like(q), "lse": torch.empty((B, Hq, S), dtype=torch.float32, device=q.device)}
    if cfg.backward:
        bufs.update(dq=torch.empty_like(q), dk=torch.empty_like(k), dv=torch.empty_like(v),
                    ws=torch.empty((_lib.bwd_workspace_bytes(B, Hq, k.shape[1], S, D, code),), dtype=torch.uint8,
                                   device=q.device))
    return bufs


def validate_shards(cfg, world, rank, slices, cpu_full, bufs, _lib, raw, dev):
    """all_gather every rank's out / lse (and dq / dk / dv) to rank 0 and compare, bit for bit,
    with rank 0's own run of the WHOLE problem on one GPU."""
    import torch.distributed as dist

    names = ["out", "lse"] + (["dq", "dk", "dv"] if cfg.backward else [])
    gathered = {}
    for name in names:
        mine = bufs[name].contiguous()
        parts = [torch.empty_like(mine) for _ in range(world)]
        dist.all_gather(parts, mine)
        gathered[name] = parts
    if rank != 0:
        return None
    q, k, v, dout = (t.to(dev) for t in cpu_full)
    full = make_bufs(_lib, raw, q, k, v, cfg)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    attention_step(raw, q, k, v, dout, cfg, full, status)
    torch.cuda.synchronize()
    report = {"gathered_with": "nccl all_gather", "ranks": world, "tensors": {}, "status_word": int(status.item())}
    ok = int(status.item()) == 0
    for name in names:
        same = True
        for r, part in enumerate(gathered[name]):
            bs, qs, ks = shard_slices(cfg, r, world)
            hs = ks if name in ("dk", "dv") else qs
            ref = full[name][bs, hs]
            same = same and torch.equal(part, ref.contiguous())
        # a checksum of the reassembled tensor, as evidence that something was compared
        total = sum(float(p.float().abs().sum().item()) for p in gathered[name])
        report["tensors"][name] = {"bitwise_equal_to_single_gpu": bool(same), "abs_sum": total}
        ok = ok and same
    report["validated"] = bool(ok)
    return report


def run_ours(args):
    from oracle import sdpa_oracle as O  # input generation + (rank 0, N=1) the cpu_baseline leg
    from torch_mojo_backend_b200 import _lib, raw

    rank, world, local = dist_setup()
    dev = torch.device("cuda", local)
    torch.cuda.set_device(dev)
    cfg_full = O.CONFIGS[args.config]
    scaling = args.scaling
    if scaling == "auto":
        scaling = "strong" if (world > 1 and args.config in ("C4", "C5")) else "weak"
    if world == 1:
        scaling = "weak" if args.scaling == "auto" else scaling
    do_bwd = cfg_full.backward
    if scaling == "strong" and world > 1:
        cpu_full = O.make_inputs(cfg_full, seed=0)
        slices = shard_slices(cfg_full, rank, world)
        bs, qs, ks = slices
        q, k, v, dout = (cpu_full[0][bs, qs].contiguous().to(dev), cpu_full[1][bs, ks].contiguous().to(dev),
                         cpu_full[2][bs, ks].contiguous().to(dev), cpu_full[3][bs, qs].contiguous().to(dev))
        cfg = O.shard(cfg_full, rank, world)
        seed_note = "torch.Generator().manual_seed(0) for the whole problem, sliced per rank"
    else:
        cpu_full, slices = None, None
        cfg = cfg_full
        q, k, v, dout = (t.to(dev) for t in O.make_inputs(cfg, seed=rank))
        seed_note = SEED_NOTE_WEAK
    bufs = make_bufs(_lib, raw, q, k, v, cfg)
    status = torch.zeros(1, dtype=torch.int32, device=dev)

    def step():
        attention_step(raw, q, k, v, dout, cfg, bufs, status)

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    barrier(world)
    launches0 = _lib.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with ClockSampler(local) as sampler:
        barrier(world)
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        barrier(world)
        total_ms = max_over_ranks(e0.elapsed_time(e1), world)
    launches_step_region = _lib.launch_count() - launches0
    # forward-only and single-backward-kernel timings explain the step number.  They run after the
    # clock sampler has stopped: a 0.5 ms kernel launched one at a time from Python is sensitive to
    # the sampler thread taking the interpreter lock between launches.
    def time_launches(fn, reps):
        # a short idle first: the timed step region above ran from an idle GPU, and a loop that starts
        # while the board's power average is still high is clocked down under the power cap
        torch.cuda.synchronize()
        time.sleep(0.3)
        for _ in range(3):
            fn()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        for _ in range(reps):
            fn()
        b.record()
        torch.cuda.synchronize()
        return a.elapsed_time(b) / reps

    reps = max(args.steps, 10)
    fwd_ms = time_launches(lambda: raw.flash_fwd(q, k, v, causal=cfg.causal, scale=cfg.scale, out=bufs["out"],
                                                 lse=bufs["lse"], status=status), reps)
    bwd_part_ms = {}
    if do_bwd:
        for name, part in (("all", 7), ("dkdv", 2), ("dq", 4)):
            bwd_part_ms[name] = time_launches(
                lambda: raw.flash_bwd(dout, q, k, v, bufs["out"], bufs["lse"], causal=cfg.causal, scale=cfg.scale,
                                      dq=bufs["dq"], dk=bufs["dk"], dv=bufs["dv"], workspace=bufs["ws"], status=status,
                                      parts=part), reps)
    launches = (_lib.launch_count() - launches0)
    timed_launches = args.steps * (1 + (3 if do_bwd else 0))
    if int(status.item()) != 0:
        raise RuntimeError(f"kernel status word is 0x{int(status.item()) & 0xffffffff:x}")

    ms_per_step = total_ms / args.steps
    flops_of = lambda c: c.fwd_flops() + (c.bwd_flops() if do_bwd else 0.0)
    # weak: every rank did a full per-GPU problem; strong: together the ranks did the one full problem
    job_flops = world * flops_of(cfg) if scaling == "weak" else flops_of(cfg_full)
    value = job_flops / (ms_per_step * 1e-3) / 1e12

    validation = None
    if scaling == "strong" and world > 1:
        validation = validate_shards(cfg_full, world, rank, slices, cpu_full, bufs, _lib, raw, dev)

    # ---- end to end on HOST tensors through the package's public API
    e2e = None if args.no_e2e else run_e2e(cfg, q, k, v, dout, rank, world, local, args)

    burst, sustained, peak_src = load_peaks()
    if do_bwd:
        # The dK/dV kernel is the longest launch.  Its algorithmic work is the 4 tile GEMMs of the 5 a
        # backward needs that it covers (S^T, dP^T, dV, dK): 0.8 x the backward FLOPs (2.0 x forward).
        dom_flops, dom_ms, dom_key = 0.8 * cfg.bwd_flops(), bwd_part_ms["dkdv"], "bwd_dkdv_kernel"
        dom_name = "bwd_dkdv_kernel (S^T, dP^T, dV, dK)"
    else:
        dom_flops, dom_ms, dom_key, dom_name = cfg.fwd_flops(), fwd_ms, "fwd_kernel", "fwd_kernel"
    achieved = dom_flops / (dom_ms * 1e-3) / 1e12
    roofline = {
        "bound": "tensor", "kernel": dom_name, "achieved": round(achieved, 2), "peak": burst, "unit": "TFLOP/s",
        "frac": round(achieved / burst, 4), "peak_source": f"of {peak_src} (cuBLAS bf16 burst)",
        "frac_of_nominal_2250": round(achieved / NOMINAL_BF16_TFLOPS, 4),
        "traffic": DRAM_TRAFFIC_BYTES.get((cfg.name, dom_key)) if world == 1 else None,
        "ms_per_launch": round(dom_ms, 4),
    }
    detail = {
        "fwd_ms": round(fwd_ms, 4), "fwd_tflops": round(cfg.fwd_flops() / (fwd_ms * 1e-3) / 1e12, 2),
        "fwd_frac_of_nominal_2250": round(cfg.fwd_flops() / (fwd_ms * 1e-3) / 1e12 / NOMINAL_BF16_TFLOPS, 4),
    }
    if do_bwd:
        # the backward timed on its own like the forward (preprocess + both kernels, as one call issues them);
        # forward-only + backward-only need not add up to the step exactly: the step alternates the two
        bwd_ms = bwd_part_ms["all"]
        detail.update({
            "bwd_ms": round(bwd_ms, 4), "bwd_tflops": round(cfg.bwd_flops() / (bwd_ms * 1e-3) / 1e12, 2),
            "bwd_frac_of_nominal_2250": round(cfg.bwd_flops() / (bwd_ms * 1e-3) / 1e12 / NOMINAL_BF16_TFLOPS, 4),
            "bwd_dkdv_kernel_ms": round(bwd_part_ms["dkdv"], 4), "bwd_dq_kernel_ms": round(bwd_part_ms["dq"], 4),
        })

    if rank == 0 and world == 1 and not args.no_e2e:
        # The other forward the library serves, outside the timed region: one new token per sequence
        # against a 32k-token cache through the split-KV call.  HBM-bound: K and V are read once.
        from torch_mojo_backend_b200 import decode_bench
        hbm_gbs, hbm_src = decode_bench.hbm_peak()
        d = decode_bench.run_shape((8, 32, 8, 1, 32768, 128), 20, torch.bfloat16, 2, hbm_gbs, hbm_src)
        detail["splitkv_decode"] = {
            "workload": "B=8 Hq=32 Hkv=8 Sq=1 Sk=32768 D=128 bf16, causal bottom-right, K+V larger than L2",
            "ms": d["ms"], "kv_gbs": d["gbs"], "roofline": {"bound": "hbm", "achieved": d["gbs"], "peak": hbm_gbs,
                                                          "unit": "GB/s", "frac": d["frac"],
                                                          "peak_source": f"of {hbm_src} (copy bandwidth)"},
            "prefill_kernel_ms": d["prefill_ms"],
        }

    cpu_baseline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        # about ten seconds of CPU work on a bounded slice of the same workload
        tf, secs, threads, sample = O.time_cpu(cfg, backward=do_bwd, sample_heads=args.cpu_sample_heads, reps=2,
                                               target_seconds=10.0)
        cpu_baseline = {"value": round(tf, 4), "unit": "TFLOP/s", "cores": threads, "kind": "port",
                        "sample": sample}

    if rank == 0:
        per_gpu = (f"B={cfg.B} Hq={cfg.Hq} Hkv={cfg.Hkv} S={cfg.S} D={cfg.D} per GPU")
        whole = (f" of the whole B={cfg_full.B} Hq={cfg_full.Hq} Hkv={cfg_full.Hkv}" if scaling == "strong" and world > 1
                 else "")
        line = {
            "metric": metric_name(cfg_full), "value": round(value, 2), "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": round(ms_per_step, 4), "higher_is_better": True,
            "scaling": scaling, "vs_baseline": None, "dtype": str(cfg.dtype).replace("torch.", ""),
            "data": "synthetic",
            "config": {
                "workload": f"{cfg.name}: {'causal' if cfg.causal else 'non-causal'} "
                            f"{'fwd+bwd' if do_bwd else 'fwd'} {per_gpu}{whole}",
                "l2": "inputs larger than L2 (no flush needed)" if cfg.fwd_bytes() > 126e6
                      else "working set fits in L2 (L2-hot number)",
                "seed": seed_note,
            },
            "frac_of_nominal_2250": round(value / world / NOMINAL_BF16_TFLOPS, 4),
            "detail": detail, "roofline": roofline, "cpu_baseline": cpu_baseline, "e2e": e2e,
            "validation": validation,
            "gpu_launches": int(launches_step_region), "gpu_launches_expected_in_step_region": int(timed_launches),
            "gpu_launches_incl_detail_timings": int(launches),
            "clocks": sampler.summary(),
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        import torch.distributed as dist

        dist.destroy_process_group()


def run_e2e(cfg, q_dev, k_dev, v_dev, dout_dev, rank, world, local, args):
    """The same step on HOST tensors: pinned host q, k, v, dO in, out and the gradients back in
    pinned host tensors, every copy inside the timed region.  Two ways of driving it are timed:

    * ``single_call``: one F.scaled_dot_product_attention call and one ``backward`` over the
      whole batch on `mojo` tensors, every copy and kernel on one stream;
    * ``pipelined``: ``torch_mojo_backend_b200.HostAttentionPipeline`` - the batch cut into
      pieces of whole (batch entry, kv-head group) units that go through the two registered
      flash operators with uploads, kernels and downloads on three streams, the host waiting for
      each step's results before it enqueues the next step.  Same inputs, same bytes moved,
      bitwise the same results (checked here before timing).
    * ``overlapped``: the same pipeline with two steps in flight: the host enqueues step i + 1,
      then waits for step i's results (``PendingPass.wait``; two sets of result buffers), so the
      uploads of a step run under the downloads of the step before and neither PCIe direction idles
      while a step fills or drains.  Every step's inputs are still uploaded and its results still
      land in host memory and are waited for inside the timed region.

    ``value`` is the best of the pipelined ways when the step is large enough to repay the
    pipelining (more than one piece), else the single call.
    """
    import torch_mojo_backend_b200 as tmb

    tmb.register_mojo_devices()
    torch.mojo.set_device(local)
    host = []
    for t in (q_dev, k_dev, v_dev, dout_dev):
        p = tmb.pinned_empty(t.shape, t.dtype)
        p.copy_(t.cpu())
        host.append(p)
    hq, hk, hv, hdo = host
    steps = max(1, min(args.steps, 10))
    gqa = cfg.Hq != cfg.Hkv
    h2d = sum(t.numel() * t.element_size() for t in ((hq, hk, hv, hdo) if cfg.backward else (hq, hk, hv)))
    # results land in pre-pinned host buffers: out, and dq/dk/dv when the config has a backward
    res_out = tmb.pinned_empty(hq.shape, hq.dtype)
    res_grads = tuple(tmb.pinned_empty(t.shape, t.dtype) for t in (hq, hk, hv)) if cfg.backward else None
    d2h = sum(t.numel() * t.element_size() for t in (res_out,) + (res_grads or ()))
    dev = torch.device("mojo", local)

    def single_call():
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

    pipe = tmb.HostAttentionPipeline(local)
    n_pieces = len(pipe.pieces(hq, hk, cfg.backward))

    def pipelined():
        pipe.run(hq, hk, hv, hdo if cfg.backward else None, is_causal=cfg.causal, scale=cfg.scale, out=res_out,
                 grads=res_grads)
        # the host reads the results after every step anyway; once the step has drained, its
        # device tensors go back to the allocator, so every step reuses the same blocks
        pipe.synchronize()

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
        single_call()
    ms_single = time_steps(single_call)
    torch.cuda.synchronize()
    ref = [res_out.clone()] + [g.clone() for g in (res_grads or ())]
    for t in (res_out,) + (res_grads or ()):
        t.zero_()
    pipelined()
    same = all(torch.equal(a, b) for a, b in zip(ref, (res_out,) + (res_grads or ())))
    pipelined()
    ms_pipe = time_steps(pipelined)

    # two steps in flight: a second set of result buffers, and the host always one step behind
    res2_out = tmb.pinned_empty(hq.shape, hq.dtype)
    res2_grads = tuple(tmb.pinned_empty(t.shape, t.dtype) for t in (hq, hk, hv)) if cfg.backward else None
    sets = ((res_out, res_grads), (res2_out, res2_grads))

    # with steps overlapping, a step needs no fine pieces of its own to fill and drain quickly: larger
    # pieces mean fewer copies and less dispatch (measured on C3: 8.5 ms a step with 40 MB pieces, 8.2 with 96 MB)
    pipe_over = tmb.HostAttentionPipeline(local, piece_bytes=96 << 20)
    n_pieces_over = len(pipe_over.pieces(hq, hk, cfg.backward))

    def overlapped_steps(n):
        waiting = None
        for i in range(n):
            o, g = sets[i % 2]
            p = pipe_over.enqueue(hq, hk, hv, hdo if cfg.backward else None, is_causal=cfg.causal, scale=cfg.scale, out=o,
                             grads=g)
            if waiting is not None:
                waiting.wait()      # the host has step i - 1's results before it goes on to step i + 1
            waiting = p
        waiting.wait()
        pipe_over.synchronize()

    for t in (res_out, res2_out) + (res_grads or ()) + (res2_grads or ()):
        t.zero_()
    overlapped_steps(2)
    same_over = all(torch.equal(a, b) for a, b in zip(ref, (res_out,) + (res_grads or ()))) and \
        all(torch.equal(a, b) for a, b in zip(ref, (res2_out,) + (res2_grads or ())))
    barrier(world)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    overlapped_steps(steps)     # ends with the current stream ordered behind the pipeline's streams
    e1.record()
    barrier(world)
    ms_over = max_over_ranks(e0.elapsed_time(e1), world) / steps
    tf = lambda ms: round(world * flops / (ms * 1e-3) / 1e12, 2)
    gbs = lambda nbytes, ms: round(nbytes / (ms * 1e-3) / 1e9, 2)
    entry = lambda ms, api, extra: dict({"value": tf(ms), "ms_per_step": round(ms, 3), "api": api,
                                         "h2d_gbs_per_gpu": gbs(h2d, ms), "d2h_gbs_per_gpu": gbs(d2h, ms)}, **extra)
    single = entry(ms_single, "F.scaled_dot_product_attention + backward on mojo tensors, whole batch, one stream", {})
    piped = entry(ms_pipe, "torch_mojo_backend_b200.HostAttentionPipeline: the batch in pieces; uploads, kernels and "
                           "downloads on three streams", {"pieces": n_pieces, "matches_single_call_bitwise": bool(same)})
    over = entry(ms_over, "HostAttentionPipeline.enqueue / PendingPass.wait: as pipelined, two steps in flight, the host "
                          "one step behind", {"pieces": n_pieces_over, "matches_single_call_bitwise": bool(same_over)})
    use_pipe = n_pieces > 1 and same
    best_ms, mode = (ms_pipe, "pipelined") if use_pipe else (ms_single, "single_call")
    if use_pipe and same_over and ms_over < ms_pipe:
        best_ms, mode = ms_over, "overlapped" 
    try:
        cores = sorted(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        cores = []
    return {"value": tf(best_ms), "unit": "TFLOP/s", "ms_per_step": round(best_ms, 3), "steps": steps,
            "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h), "mode": mode,
            "h2d_gbs_per_gpu": gbs(h2d, best_ms), "d2h_gbs_per_gpu": gbs(d2h, best_ms),
            "bound": "host link: the step moves h2d + d2h bytes over PCIe around a few ms of kernels; with several "
                     "ranks on one host the copies of all ranks share the host's memory and PCIe fabric",
            "host_cores_of_this_rank": len(cores), "ranks_on_host": world,
            "overlapped": over, "pipelined": piped, "single_call": single}


def run_reference(args):
    """The reference arm: the reference's own path cannot be built here (it needs the Mojo
    toolchain), so - as its tests do - torch's CPU SDPA stands in, timed on all host cores on a
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
        "impl": "reference", "metric": metric_name(cfg), "value": round(value, 4), "unit": "TFLOP/s",
        "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(1e3 * statistics.median(secs_all), 2), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": str(cfg.dtype).replace("torch.", ""), "data": "synthetic",
        # the same `config` as the GPU arm prints for this workload (the CPU sample is in cpu_baseline.sample)
        "config": {"workload": f"{cfg.name}: {'causal' if cfg.causal else 'non-causal'} "
                               f"{'fwd+bwd' if cfg.backward else 'fwd'} B={cfg.B} Hq={cfg.Hq} Hkv={cfg.Hkv} S={cfg.S} "
                               f"D={cfg.D} per GPU",
                   "l2": "inputs larger than L2 (no flush needed)" if cfg.fwd_bytes() > 126e6
                         else "working set fits in L2 (L2-hot number)",
                   "seed": SEED_NOTE_WEAK},
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
    ap.add_argument("--scaling", default="auto", choices=["auto", "weak", "strong"],
                    help="N > 1: weak = a full per-GPU problem on every rank; strong = one problem split over the "
                         "ranks, gathered and validated (auto: strong for C4 and C5)")
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
