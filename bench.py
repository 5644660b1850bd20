"""Benchmark of the gated-delta-rule path: GDN forward + backward tokens/s on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg1] [--impl ours|reference]

One "step" is one forward + backward of ``chunk_gated_delta_rule`` over one synthetic batch.  At every N each rank
runs the whole workload (the path has no cross-(sequence, head) coupling: ranks shard independent batches, no
collective on the data path), so scaling is weak and ``value`` is ``N x tokens / max-over-ranks time``.

Printed JSON line (rank 0):
  value         tokens/s with the inputs resident in HBM, device-timed (CUDA events), K steps, max over ranks
  e2e           the same metric through the public entry point with HOST (pinned) buffers: every step copies its
                inputs host->device and its outputs and gradients device->host inside the timed region
  roofline      the dominant kernel: achieved = its algorithmic HBM bytes (or FLOPs) per launch / its mean device
                time, measured live with CUDA events around each launch in a separate profiled pass of the same steps
  path_roofline the whole step against max(FLOPs / tensor peak, compulsory bytes / HBM peak)
  cpu_baseline  the CPU oracle (a port of the reference's torch path) timed on this host's cores on a bounded sample
  clocks        SM clocks and throttle reasons sampled with nvidia-smi during the timed region

``--impl reference`` times the CPU oracle alone (the reference's own kernels need CUDA >= 13.4 and cannot be built
with this toolkit; its torch emulation path is what the oracle restates), on rank 0 only.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "gdn_fwd_bwd_tokens_per_sec"  # on a KDA workload the same metric of the per-channel-decay variant
UNIT = "tokens/s"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def peaks() -> tuple[dict, str]:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.is_file():
        try:
            data = json.loads(path.read_text())
            return {k: float(data[k]) for k in FALLBACK_PEAKS if k in data} | {}, "measured"
        except (ValueError, KeyError):
            pass
    return dict(FALLBACK_PEAKS), "fallback"


# --------------------------------------------------------------------------------------------------------------------
# clocks
# --------------------------------------------------------------------------------------------------------------------
class ClockSampler:
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int) -> None:
        self.index = index
        self.file = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.proc = None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=self.file, stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        if self.proc is not None:
            self.proc.terminate()
            try:
                self.proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()

    def summary(self) -> dict:
        self.file.flush()
        rows = [line.split(",") for line in Path(self.file.name).read_text().splitlines() if line.count(",") >= 8]
        os.unlink(self.file.name)
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        sm = [float(r[1]) for r in rows if r[1].strip().replace(".", "").isdigit()]
        smax = [float(r[2]) for r in rows if r[2].strip().replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any("Active" == r[5 + i].strip() for r in rows)]
        busy = [c for c in sm if c > 0.5 * max(sm)] if sm else []
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(smax) if smax else None,
                "reasons": reasons, "samples": len(rows)}


# --------------------------------------------------------------------------------------------------------------------
# the CPU arm (oracle port): the only place bench.py touches oracle/
# --------------------------------------------------------------------------------------------------------------------
def cpu_tokens_per_sec(workload_name: str, sample_tokens: int, steps: int, warmup: int) -> dict:
    from oracle import gdn_oracle as oracle

    from miles_ext_kernels_b200.workloads import make_workload

    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    work = make_workload(workload_name, tokens=sample_tokens)
    B, T = work.q.shape[:2]
    flat = lambda t: t.reshape(B * T, *t.shape[2:]).float()  # noqa: E731
    seq_lens = tuple(b - a for a, b in zip(work.cu_seqlens[:-1], work.cu_seqlens[1:])) if work.cu_seqlens else (T,) * B
    args = [flat(t) for t in (work.q, work.k, work.v, work.g, work.beta)]

    def step():
        if work.config.op == "kda":
            from oracle import kda_oracle

            kda_oracle.chunked_forward_backward(*args, seq_lens, flat(work.do))
        else:
            oracle.chunked_forward_backward(*args, seq_lens, flat(work.do), h0=work.h0, dht=work.dht,
                                            output_final_state=work.config.final_state)

    for _ in range(warmup):
        step()
    start = time.perf_counter()
    for _ in range(steps):
        step()
    seconds = time.perf_counter() - start
    return {
        "value": B * T * steps / seconds, "unit": UNIT, "cores": cores, "kind": "port",
        "sample": f"{workload_name} cut to {B * T} tokens (B={B}, T={T}), all heads, fp32 torch on the host, "
                  f"{steps} step(s) after {warmup} warm-up",
        "seconds_per_step": seconds / steps, "tokens": B * T,
    }


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    sample = 4096 if args.steps + args.warmup <= 8 else 1024
    cpu = cpu_tokens_per_sec(args.workload, sample, args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": cpu["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * cpu["seconds_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": args.workload, "sample": cpu["sample"]},
        "cpu_baseline": {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cpu["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------------------------------------------------
# our arm
# --------------------------------------------------------------------------------------------------------------------
KERNEL_BYTES = {
    # algorithmic bytes per token of each kernel's own reads + writes at (H, HV), d = 128; per-chunk tensors are
    # counted per token (A, Aqk: 64 x 64 bf16 per 64 tokens = 128 B per token and head; h / dh tapes: 128 x 128 bf16
    # per 64 tokens = 512 B per token and head)
    "gdn_gate_cumsum": lambda H, HV: 8 * HV,
    "gdn_l2norm": lambda H, HV: 2 * 256 * H + 4 * H,
    "gdn_wy_fwd": lambda H, HV: 2 * 256 * H + 256 * HV + 8 * HV + (2 * 128 + 2 * 256) * HV,
    "gdn_fwd_h": lambda H, HV: 256 * H + (2 * 256 + 4) * HV + (512 + 256) * HV,
    "gdn_fwd_o": lambda H, HV: 256 * H + (128 + 256 + 512 + 4) * HV + 256 * HV,
    # the scan with the output fused in: fwd_h's traffic + q, Aqk in and o out (h is not read back)
    "gdn_fwd_ho": lambda H, HV: 2 * 256 * H + (2 * 256 + 4 + 128) * HV + (512 + 2 * 256) * HV,
    "gdn_bwd_dh": lambda H, HV: 2 * 256 * H + (256 + 256 + 128 + 4) * HV + (512 + 256) * HV,
    "gdn_bwd_tail": lambda H, HV: 2 * 256 * H + (256 + 8 + 2 * 128 + 2 * 512 + 3 * 256) * HV + 2 * 256 * H
    + (256 + 8) * HV,
}
KERNEL_BYTES.update({
    # KDA (H = HV): g, G and dg are [., 128] fp32 per head
    "kda_prep": lambda H, HV: (2 * 256 + 512 + 512 + 3 * 256 + 8) * HV,
    "kda_intra": lambda H, HV: (4 * 256 + 512 + 4 + 2 * 128 + 2 * 256) * HV,
    "kda_fwd_h": lambda H, HV: (3 * 256 + 8 + 512 + 256) * HV,
    "kda_fwd_o": lambda H, HV: (256 + 128 + 256 + 512 + 256) * HV,
    "kda_bwd_dh": lambda H, HV: (4 * 256 + 128 + 8 + 512 + 256) * HV,
    "kda_bwd_tail": lambda H, HV: (4 * 256 + 512 + 4 + 128 + 2 * 512 + 3 * 256 + 2 * 2 * 256 + 3 * 2 * 512 + 16
                                   + 2 * 512 + 256 + 512 + 4) * HV,
    "qk_grad_finish": lambda H, HV: (512 + 256) * HV,
})
# dram__bytes_read.sum + dram__bytes_write.sum of one launch in the committed ncu capture of an 8,192-token cut of cfg1
# (H=16, HV=32; profiles/gdn_kernels_8192_tokens_full_set.md).  Every tensor is per token or per chunk, so traffic
# grows in proportion to the tokens: `roofline.traffic` scales these to the launch that was timed.
NCU_TRAFFIC_BYTES_AT_8192_TOKENS = {
    "gdn_wy_fwd": 136.9e6 + 149.2e6,
    "gdn_fwd_ho": 237.5e6 + 225.8e6,
    "gdn_bwd_dh": 237.4e6 + 154.6e6,
    "gdn_bwd_tail": 807.5e6 + 122.8e6,
}
KERNEL_FLOPS = {  # per (chunk, value head): dense contractions as 2 m n k
    "gdn_wy_fwd": 2 * 128 * 64 * 128 + 2 * 64**3 / 3 + 2 * 2 * 64 * 128 * 64,
    "gdn_fwd_h": 2 * 64 * 128 * 128 + 2 * 128 * 128 * 64,
    "gdn_fwd_o": 2 * 64 * 128 * 128 + 2 * 64 * 128 * 64,
    "gdn_fwd_ho": 2 * 2 * 64 * 128 * 128 + 2 * 128 * 128 * 64 + 2 * 64 * 128 * 64,
    "gdn_bwd_dh": 2 * 64 * 128 * 128 + 2 * 64 * 128 * 64 + 2 * 2 * 128 * 128 * 64,
    # 4 products [64 x 128, K = 128], 3 of [64 x 64, K = 128], 6 of [64 x 128, K = 64], 2 of [64 x 64, K = 64]
    "gdn_bwd_tail": 4 * 2 * 64 * 128 * 128 + 3 * 2 * 64 * 64 * 128 + 6 * 2 * 64 * 128 * 64 + 2 * 2 * 64**3,
}


def run_ours(args) -> None:
    import torch.distributed as dist

    import miles_ext_kernels_b200 as package
    from miles_ext_kernels_b200.cake import gdn, kda
    from miles_ext_kernels_b200.cake._impl.gdn import native
    from miles_ext_kernels_b200.workloads import bytes_per_token, flops_per_token, make_workload

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); the kernels have no CPU fallback")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)
    package.configure(cake_gdn_variant="det")
    gdn.chunk_gated_delta_rule, kda.chunk_kda  # noqa: B018  import the implementations before timing

    work = make_workload(args.workload, tokens=args.tokens)
    cfg = work.config
    tokens = work.num_tokens
    H, HV = work.q.shape[2], work.v.shape[2]
    host = {n: getattr(work, n) for n in ("q", "k", "v", "g", "beta", "do", "h0", "dht") if getattr(work, n) is not None}
    resident = {n: t.to(device) for n, t in host.items()}
    cu_dev = None if work.cu_seqlens is None else torch.tensor(work.cu_seqlens, dtype=torch.int32, device=device)

    def step(t: dict, cu=None):
        cu_cpu, cu_gpu = (work.cu_seqlens, cu_dev) if cu is None else cu
        q, k, v = (t[n].detach().requires_grad_(True) for n in ("q", "k", "v"))
        g, beta = t["g"].detach().requires_grad_(True), t["beta"].detach().requires_grad_(True)
        h0 = t["h0"].detach().requires_grad_(True) if "h0" in t else None
        if cfg.op == "kda":
            o, final = kda.chunk_kda(q, k, v, g, beta, cu_gpu, cu_seqlens_cpu=cu_cpu), None
        else:
            o, final = gdn.chunk_gated_delta_rule(q, k, v, g=g, beta=beta, initial_state=h0,
                                                  output_final_state=cfg.final_state, cu_seqlens=cu_gpu,
                                                  cu_seqlens_cpu=cu_cpu, use_qk_l2norm_in_kernel=False)
        if final is not None and "dht" in t:
            torch.autograd.backward([o, final], [t["do"], t["dht"]])
        else:
            o.backward(t["do"])
        outs = [o, q.grad, k.grad, v.grad, g.grad, beta.grad] + ([h0.grad] if h0 is not None else []) + (
            [final] if final is not None else [])
        return outs

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps: int) -> float:
        """Device milliseconds of `steps` calls of fn, max over ranks."""
        barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            fn()
        end.record()
        barrier()
        ms = torch.tensor([start.elapsed_time(end)], device=device)
        if world > 1:
            dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        return float(ms.item())

    # clocks are sampled from the warm-up on (a 10-step timed region is shorter than nvidia-smi's sampling period);
    # only samples taken under load enter the median
    with ClockSampler(local) as sampler:
        for _ in range(max(args.warmup, 3)):
            step(resident)
        log = native.LaunchLog(timed=False)
        native.set_launch_log(log)
        ms = timed(lambda: step(resident), args.steps)
        native.set_launch_log(None)
        if ms < 400.0:  # keep the GPU busy with the same step until the sampler has seen it under load
            busy_until = time.perf_counter() + 0.5
            while time.perf_counter() < busy_until:
                step(resident)
            torch.cuda.synchronize()
    clocks = sampler.summary()
    launches = log.count

    # end to end: pinned host buffers in, outputs and gradients out to pinned host buffers, every step, through the
    # package's host-memory pipeline (parts of the call on three streams: copy in, compute, copy out)
    from miles_ext_kernels_b200 import host_io

    if work.cu_seqlens is None:
        parts = host_io.batch_parts(work.q.shape[0])
    else:
        parts = host_io.packed_parts(work.cu_seqlens, 8)
    part_cu = {id(p): (p.cu_seqlens, torch.tensor(p.cu_seqlens, dtype=torch.int32, device=device))
               for p in parts if p.cu_seqlens is not None}
    pipeline = host_io.HostPipeline(device, parts, per_token=("q", "k", "v", "g", "beta", "do"))
    total = (work.q.shape[0], work.q.shape[1], len(work.cu_seqlens) - 1 if work.cu_seqlens else work.q.shape[0])

    def e2e_step():
        return pipeline.run(host, lambda part, t: step(t, part_cu.get(id(part))), range(6), total)

    e2e_step()
    ms_e2e = timed(e2e_step, args.steps)
    h2d = sum(t.numel() * t.element_size() for t in host.values())
    d2h = sum(x.numel() * x.element_size() for x in e2e_step())
    torch.cuda.synchronize()

    # the form the training framework calls (GDN only): q, k, v as views of one packed row [q heads | k heads |
    # v heads] (what a fused projection writes), raw q / k with the L2 norm inside the op; the op reads the views in
    # place and the gradient comes back as one packed row
    miles_form = None
    if cfg.op == "gdn":
        lead = resident["q"].shape[:2]
        mixed = torch.cat([resident["q"].reshape(*lead, -1), resident["k"].reshape(*lead, -1),
                           resident["v"].reshape(*lead, -1)], dim=-1).contiguous()

        def miles_step():
            row = mixed.detach().requires_grad_(True)
            q, k, v = gdn.packed_qkv_views(row, H, HV)
            g, beta = resident["g"].detach().requires_grad_(True), resident["beta"].detach().requires_grad_(True)
            h0 = resident["h0"] if "h0" in resident else None
            o, _ = gdn.chunk_gated_delta_rule(q, k, v, g=g, beta=beta, initial_state=h0, cu_seqlens=cu_dev,
                                              cu_seqlens_cpu=work.cu_seqlens, use_qk_l2norm_in_kernel=True)
            o.backward(resident["do"])
            return row.grad

        for _ in range(3):
            miles_step()
        ms_miles = timed(miles_step, args.steps)
        miles_form = {"ms_per_step": ms_miles / args.steps, "value": world * tokens / (ms_miles * 1e-3 / args.steps),
                      "unit": UNIT, "what": "q, k, v as packed_qkv_views of one [q | k | v] row, read in place; L2 norm "
                      "of q / k in the op; the gradient is one packed row"}
        del mixed

    # per-kernel device times: a separate pass of the same steps with events around every launch
    prof = native.LaunchLog(timed=True)
    native.set_launch_log(prof)
    for _ in range(args.steps):
        step(resident)
    torch.cuda.synchronize()
    native.set_launch_log(None)
    per_kernel = {name: (sum(v) / len(v), len(v), sum(v)) for name, v in prof.milliseconds().items()}
    top = max(per_kernel, key=lambda n: per_kernel[n][2])
    peak, peak_kind = peaks()
    mean_ms = per_kernel[top][0]
    gbs = KERNEL_BYTES.get(top, lambda H, HV: 0.0)(H, HV) * tokens / (mean_ms * 1e-3) / 1e9
    tiles = (tokens / 64) * HV
    tfs = KERNEL_FLOPS.get(top, 0.0) * tiles / (mean_ms * 1e-3) / 1e12
    frac_hbm, frac_tc = gbs / peak["hbm_gbs"], tfs / peak["bf16_tflops"]
    if frac_tc > frac_hbm:
        roofline = {"bound": "tensor", "achieved": tfs, "peak": peak["bf16_tflops"], "unit": "TFLOP/s", "frac": frac_tc}
    else:
        roofline = {"bound": "hbm", "achieved": gbs, "peak": peak["hbm_gbs"], "unit": "GB/s", "frac": frac_hbm}
    traffic = None
    if (H, HV) == (16, 32) and top in NCU_TRAFFIC_BYTES_AT_8192_TOKENS:
        traffic = NCU_TRAFFIC_BYTES_AT_8192_TOKENS[top] * tokens / 8192
    roofline.update(kernel=top, ms_per_launch=mean_ms, traffic=traffic, traffic_unit="bytes per launch",
                    traffic_source="ncu capture at 8,192 tokens, scaled by tokens", peak_source=f"of {peak_kind}",
                    share_of_step=per_kernel[top][2] / sum(v[2] for v in per_kernel.values()))

    step_s = ms * 1e-3 / args.steps
    t_roof = max(flops_per_token(HV) * tokens / (peak["bf16_tflops_sustained"] * 1e12),
                 bytes_per_token(H, HV, op=cfg.op) * tokens / (peak["hbm_gbs"] * 1e9))
    value = world * tokens / step_s
    line = {
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3),
        "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic",
        "config": {"workload": f"{cfg.name}: {cfg.description}", "tokens_per_gpu": tokens, "num_qk_heads": H,
                   "num_v_heads": HV, "head_dim": 128, "chunk": 64, "state": "fp32",
                   "l2_hygiene": "inputs (q+k+v+dO = 768 MiB at cfg1) are larger than the 126 MB L2",
                   "sharding": "each rank runs the whole workload; no collective on the data path"},
        "e2e": {"value": world * tokens / (ms_e2e * 1e-3 / args.steps), "unit": UNIT, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e / args.steps, "parts": len(parts)},
        "gpu_launches": launches,
        "roofline": roofline,
        "path_roofline": {"t_roof_ms": 1e3 * t_roof, "frac": t_roof / step_s, "flops_per_token": flops_per_token(HV),
                          "bytes_per_token": bytes_per_token(H, HV, op=cfg.op), "peak_source": f"of {peak_kind}"},
        "miles_form": miles_form,
        "kernels_ms": {n: {"mean": v[0], "launches": v[1], "total": v[2]} for n, v in per_kernel.items()},
        "clocks": clocks,
    }
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_tokens_per_sec(args.workload, 8192, 1, 1)
        line["cpu_baseline"] = {k: cpu[k] for k in ("value", "unit", "cores", "kind", "sample")}
    if rank == 0:
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def run_adjacent(args) -> None:
    """The two row-wise ops either side of the path in a layer, at cfg1's shape on one GPU: ``--workload conv1d`` (the
    packed causal conv1d + SiLU over the ``[q | k | v]`` row, 8,192 channels) and ``--workload gated_rmsnorm`` (the
    SiLU-gated RMSNorm over the output's rows of 128).  Both are HBM-bound; the line's roofline entry is the backward
    kernel's."""
    import miles_ext_kernels_b200 as package
    from miles_ext_kernels_b200.cake.conv1d import causal_conv1d
    from miles_ext_kernels_b200.cake.gated_rmsnorm import rmsnorm_silu_gate

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); the kernels have no CPU fallback")
    device = torch.device("cuda", 0)
    package.configure()
    tokens = args.tokens or 32768
    gen = torch.Generator(device=device).manual_seed(11)
    if args.workload == "conv1d":
        channels = 8192
        x = torch.randn(1, tokens, channels, device=device, generator=gen).bfloat16()
        w = (0.5 * torch.randn(channels, 4, device=device, generator=gen)).requires_grad_(True)
        dy = torch.randn(1, tokens, channels, device=device, generator=gen).bfloat16()
        cu = torch.arange(0, tokens + 1, tokens // 4, dtype=torch.int32, device=device)
        elements = tokens * channels
        fwd_bytes, bwd_bytes = 4 * elements, 6 * elements  # bf16: x -> y; x, dy -> dx
        what = f"packed causal conv1d + SiLU: {tokens} tokens x {channels} channels, 4 documents, fp32 taps"
        z = None

        def forward(leaf):
            return causal_conv1d(leaf, w, cu)
    else:
        rows = tokens * 32
        x = torch.randn(rows, 128, device=device, generator=gen).bfloat16()
        z = torch.randn(rows, 128, device=device, generator=gen).bfloat16().requires_grad_(True)
        w = torch.randn(128, device=device, generator=gen).bfloat16().requires_grad_(True)
        dy = torch.randn(rows, 128, device=device, generator=gen).bfloat16()
        elements = rows * 128
        fwd_bytes, bwd_bytes = 6 * elements, 10 * elements  # bf16: x, z -> y; x, z, dy -> dx, dz
        what = f"SiLU-gated RMSNorm: {rows} rows of 128 ({tokens} tokens x 32 value heads)"

        def forward(leaf):
            return rmsnorm_silu_gate(leaf, z, w, 1e-6)

    def timed(fn):
        for _ in range(max(3, args.warmup)):
            fn()
        torch.cuda.synchronize()
        begin, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        begin.record()
        for _ in range(args.steps):
            fn()
        end.record()
        torch.cuda.synchronize()
        return begin.elapsed_time(end) / args.steps

    def both():
        leaf = x.detach().requires_grad_(True)
        for parameter in (w, z):
            if parameter is not None:
                parameter.grad = None  # no accumulation kernels inside the timed region
        forward(leaf).backward(dy)

    peak, peak_kind = peaks()
    with ClockSampler(0) as sampler:
        with torch.no_grad():
            ms_fwd = timed(lambda: forward(x))
        ms_both = timed(both)
    clocks = sampler.summary()
    ms_bwd = ms_both - ms_fwd
    achieved = bwd_bytes / (ms_bwd * 1e-3) / 1e9
    print(json.dumps({
        "metric": f"{args.workload}_fwd_bwd_tokens_per_sec", "value": tokens / (ms_both * 1e-3), "unit": UNIT, "n_gpus": 1,
        "steps": args.steps, "warmup": max(3, args.warmup), "ms_per_step": ms_both, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": what, "l2_hygiene": "inputs are larger than the 126 MB L2"},
        "ms_forward": ms_fwd, "ms_backward": ms_bwd,
        "forward_gbs": fwd_bytes / (ms_fwd * 1e-3) / 1e9,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / peak["hbm_gbs"], "kernel": f"{args.workload} backward (with its autograd glue)",
                     "traffic": None, "peak_source": f"of {peak_kind}"},
        "clocks": clocks,
    }))


def main() -> None:
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--workload", default="cfg1")
    parser.add_argument("--tokens", type=int, default=None, help="cut the workload to this many tokens (profiling)")
    parser.add_argument("--impl", choices=("ours", "reference"), default="ours")
    parser.add_argument("--no-cpu-baseline", action="store_true")
    args = parser.parse_args()
    if args.workload in ("conv1d", "gated_rmsnorm"):
        run_adjacent(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
