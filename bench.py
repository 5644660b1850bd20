"""Benchmark of the gated-delta-rule path: GDN forward + backward tokens/s on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg1] [--impl ours|reference]

One "step" is one forward + backward of ``chunk_gated_delta_rule`` over one synthetic batch.  At every N each rank
runs the whole workload (the path has no cross-(sequence, head) coupling: ranks shard independent batches, no
collective on the data path), so scaling is weak and ``value`` is ``N x tokens / max-over-ranks time``.

The one configuration with a real exchange between ranks -- one long sequence split context-parallel -- is timed and
checked on the same line when N >= 2:
  cp            one sequence of N x 32,768 tokens (H = HV = 32) in contiguous slices through
                ``kcp_chunk_gated_delta_rule``: ms per step (max over ranks), whole-job tokens/s, efficiency = the
                slice alone / the N-rank step, the exchange's own device time and the bytes each rank receives
  cp_parity     o and every gradient of a short case (N x 2,048 tokens) gathered to rank 0, against the undivided call
  kda_sharded   the per-channel-decay variant with one 4,096-token sequence per rank (no exchange)

Printed JSON line (rank 0):
  value         tokens/s with the inputs resident in HBM, device-timed (CUDA events), K steps, max over ranks
  e2e           the same metric through the public entry point with HOST (pinned) buffers: every step copies its
                inputs host->device and its outputs and gradients device->host inside the timed region
  roofline      the dominant kernel: achieved = its algorithmic HBM bytes (or FLOPs) per launch / its mean device
                time, measured live with CUDA events around each launch in a separate profiled pass of the same steps
  path_roofline the whole step against max(FLOPs / tensor peak, compulsory bytes / HBM peak)
  cpu_baseline  the reference's own CPU path (its torch emulation through its public entry point, from
                ``oracle/_ref``; the oracle port where that cannot run) timed on this host's cores on a bounded sample
  clocks        SM clocks and throttle reasons sampled with nvidia-smi during the timed region

``--impl reference`` times that CPU path alone, on rank 0 only (the reference's own kernels need CUDA >= 13.4 and
cannot be built with this toolkit).  Both CPU legs use the same sample of the workload, named in ``config``.
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
# the CPU arm: the only place bench.py touches oracle/
# --------------------------------------------------------------------------------------------------------------------
CPU_SAMPLE_TOKENS = 2048  # of the workload, for both CPU legs (the reference's CPU path does ~0.4-1 k tokens/s)


def cpu_tokens_per_sec(workload_name: str, steps: int, warmup: int) -> dict:
    """Forward + backward on the host's cores over the first ``CPU_SAMPLE_TOKENS`` tokens of the workload: through the
    reference's own CPU path (``oracle/_ref``: packed call, no initial / final state, as its context-parallel
    contract has it) when it is there and can run the workload, else through the oracle port."""
    from oracle import gdn_oracle as oracle
    from oracle import reference_arm

    from miles_ext_kernels_b200.workloads import make_workload

    cores = len(os.sched_getaffinity(0))
    torch.set_num_threads(cores)
    work = make_workload(workload_name, tokens=CPU_SAMPLE_TOKENS)
    B, T = work.q.shape[:2]
    flat = lambda t: t.reshape(B * T, *t.shape[2:])  # noqa: E731
    seq_lens = tuple(b - a for a, b in zip(work.cu_seqlens[:-1], work.cu_seqlens[1:])) if work.cu_seqlens else (T,) * B
    use_reference = reference_arm.available() and work.config.op == "gdn" and work.h0 is None
    if use_reference:
        cu = (0, *(sum(seq_lens[: i + 1]) for i in range(len(seq_lens))))
        args = [flat(t) for t in (work.q, work.k, work.v, work.g, work.beta, work.do)]

        def step():
            reference_arm.forward_backward(*args, cu)
    else:
        args = [flat(t).float() for t in (work.q, work.k, work.v, work.g, work.beta)]

        def step():
            if work.config.op == "kda":
                from oracle import kda_oracle

                kda_oracle.chunked_forward_backward(*args, seq_lens, flat(work.do).float())
            else:
                oracle.chunked_forward_backward(*args, seq_lens, flat(work.do).float(), h0=work.h0, dht=work.dht,
                                                output_final_state=work.config.final_state)

    for _ in range(warmup):
        step()
    start = time.perf_counter()
    for _ in range(steps):
        step()
    seconds = time.perf_counter() - start
    how = ("the reference's own torch emulation through its public entry point (oracle/_ref), packed, no final state"
           if use_reference else "the oracle port, fp32 torch")
    return {
        "value": B * T * steps / seconds, "unit": UNIT, "cores": cores, "kind": "reference" if use_reference else "port",
        "sample": f"{workload_name} cut to {B * T} tokens (B={B}, T={T}), all heads, {how}, on the host, "
                  f"{steps} step(s) after {warmup} warm-up",
        "seconds_per_step": seconds / steps, "tokens": B * T,
    }


def _workload_title(name: str) -> str:
    from miles_ext_kernels_b200.workloads import CONFIGS

    cfg = CONFIGS.get(name)
    return name if cfg is None else f"{cfg.name}: {cfg.description}"


def run_reference(args) -> None:
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cpu = cpu_tokens_per_sec(args.workload, args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": METRIC, "value": cpu["value"], "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * cpu["seconds_per_step"],
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        # the same workload string as the GPU arm's line; what was timed of it is the bounded sample named beside it
        "config": {"workload": _workload_title(args.workload), "sample": cpu["sample"], "cpu_processes": 1,
                   "cpu_sample_tokens": CPU_SAMPLE_TOKENS},
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
# Measured DRAM traffic per token (dram__bytes_read.sum + dram__bytes_write.sum of one launch under ncu, divided by
# the launch's tokens), keyed by the head counts of the capture and the kernel.  Every tensor of the path is per
# token or per chunk, so traffic grows in proportion to the tokens: `roofline.traffic` scales these to the launch that
# was timed; a head configuration that was never captured reports null.
NCU_TRAFFIC_BYTES_PER_TOKEN = {
    (16, 32): {  # an 8,192-token cut of cfg1
        "gdn_wy_fwd": (137.0e6 + 150.7e6) / 8192,
        "gdn_fwd_ho": (236.2e6 + 225.8e6) / 8192,
        "gdn_bwd_dh": (236.0e6 + 154.8e6) / 8192,
        "gdn_bwd_tail": (807.5e6 + 122.1e6) / 8192,
    },
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


class Clock:
    """Device time of a run of steps, max over ranks, with a barrier and a synchronisation on both sides."""

    def __init__(self, device, world: int) -> None:
        self.device, self.world = device, world

    def barrier(self) -> None:
        if self.world > 1:
            import torch.distributed as dist

            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(self, value: float) -> float:
        t = torch.tensor([value], dtype=torch.float64, device=self.device)
        if self.world > 1:
            import torch.distributed as dist

            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def timed(self, fn, steps: int) -> float:
        """Device milliseconds of `steps` calls of fn, max over ranks."""
        self.barrier()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            fn()
        end.record()
        self.barrier()
        return self.max_over_ranks(start.elapsed_time(end))


def _leaves(x: dict, names=("q", "k", "v", "g", "beta")):
    return [x[n].detach().requires_grad_(True) for n in names]


def context_parallel(clock: Clock, device, rank: int, world: int, steps: int) -> dict:
    """One sequence of ``world x 32,768`` tokens, H = HV = 32, in contiguous slices, one per rank: forward + backward
    through ``kcp_chunk_gated_delta_rule`` with each of the two boundary-state exchanges, against the same slice run
    alone (no context, no exchange) on every rank."""
    import miles_ext_kernels_b200 as package
    from miles_ext_kernels_b200.cake import gdn
    from miles_ext_kernels_b200.cake._impl.gdn import kcp
    from miles_ext_kernels_b200.workloads import make_workload

    work = make_workload("cfg4", seed=4 + 1000 * rank)  # this rank's slice: the same distributions, its own values
    T, H, HV = work.q.shape[1], work.q.shape[2], work.v.shape[2]
    x = {n: getattr(work, n).to(device) for n in ("q", "k", "v", "g", "beta", "do")}
    cu_local = (0, T)
    cu_dev = torch.tensor(cu_local, dtype=torch.int32, device=device)
    context = gdn.build_kcp_context((0, world * T), device=device)

    def alone():
        q, k, v, g, beta = _leaves(x)
        o, _ = gdn.chunk_gated_delta_rule(q, k, v, g=g, beta=beta, cu_seqlens=cu_dev, cu_seqlens_cpu=cu_local)
        o.backward(x["do"])

    def together():
        q, k, v, g, beta = _leaves(x)
        gdn.kcp_chunk_gated_delta_rule(q, k, v, g, beta, context).backward(x["do"])

    for _ in range(3):
        alone()
    ms_alone = clock.timed(alone, steps) / steps
    out = {"workload": f"cfg4: one sequence of {world * T} tokens, H=HV={HV}, d=128, {world} contiguous slices of {T}",
           "slice_alone_ms": ms_alone, "modes": {}}
    for mode in ("parallel", "sequential"):
        package.configure(cake_gdn_variant="det", cake_gdn_kcp_exchange=mode)
        for _ in range(3):
            together()
        ms = clock.timed(together, steps) / steps
        log = kcp.ExchangeLog()
        kcp.set_exchange_log(log)
        for _ in range(steps):
            together()
        torch.cuda.synchronize()
        kcp.set_exchange_log(None)
        spent = log.milliseconds()
        out["modes"][mode] = {
            "ms_per_step": ms, "value": world * T / (ms * 1e-3), "unit": UNIT, "efficiency": ms_alone / ms,
            "exchange_ms_forward": clock.max_over_ranks(spent.get("forward", 0.0) / steps),
            "exchange_ms_backward": clock.max_over_ranks(spent.get("backward", 0.0) / steps),
            "bytes_received_per_rank_per_step": clock.max_over_ranks(log.bytes_received / steps),
        }
    package.configure(cake_gdn_variant="det")
    best = min(out["modes"], key=lambda m: out["modes"][m]["ms_per_step"])
    out.update(exchange=best, **out["modes"][best])
    out["what"] = ("exchange_ms_*: pre-scan of the rank's fragment + all-gather of the (B, M) summaries + fold (parallel), "
                   "or the wait for the neighbour's state + its transfer (sequential); device time, max over ranks")
    return out


def context_parallel_parity(device, rank: int, world: int) -> dict:
    """A short sequence (``world x 2,048`` tokens, H = HV = 32) split over the ranks: o and every gradient gathered to
    rank 0 and compared with the undivided call on rank 0.  Budgets: relative RMS error <= 6e-3 and largest error <=
    2e-2 of the largest reference magnitude, per tensor.  Weak gates (g = -0.5 U(0, 1)) carry state across every
    cut; the benchmark's strong gates are checked too.  A control run in which nothing crosses the cuts (every slice
    as a sequence of its own) goes through the same comparison and has to be rejected under the weak gates."""
    import torch.distributed as dist

    import miles_ext_kernels_b200 as package
    from miles_ext_kernels_b200.cake import gdn

    T, H, HV = 2048, 32, 32
    S = world * T
    names = ("q", "k", "v", "g", "beta", "do")
    cases, ok = {}, True
    for gate in ("weak", "strong"):
        gen = torch.Generator(device=device).manual_seed(40 if gate == "weak" else 41)
        full = {}
        if rank == 0:
            unit = lambda t: t / torch.sqrt((t * t).sum(-1, keepdim=True) + 1e-6)  # noqa: E731
            full["q"] = unit(torch.randn(1, S, H, 128, device=device, generator=gen)).bfloat16()
            full["k"] = unit(torch.randn(1, S, H, 128, device=device, generator=gen)).bfloat16()
            full["v"] = torch.randn(1, S, HV, 128, device=device, generator=gen).bfloat16()
            full["beta"] = torch.sigmoid(torch.randn(1, S, HV, device=device, generator=gen)).bfloat16()
            u = torch.rand(1, S, HV, device=device, generator=gen)
            if gate == "weak":
                full["g"] = -0.5 * u
            else:
                a = torch.randn(1, S, HV, device=device, generator=gen)
                full["g"] = -torch.nn.functional.softplus(a) * torch.exp(u * math.log(16.0))
            full["do"] = torch.randn(1, S, HV, 128, device=device, generator=gen).bfloat16()
        else:
            for n in names:
                heads = H if n in ("q", "k") else HV
                shape = (1, S, heads, 128) if n in ("q", "k", "v", "do") else (1, S, heads)
                full[n] = torch.empty(shape, dtype=torch.float32 if n == "g" else torch.bfloat16, device=device)
        for n in names:
            dist.broadcast(full[n], src=0)
        mine = {n: full[n][:, rank * T:(rank + 1) * T].contiguous() for n in names}
        want = None
        if rank == 0:
            leaves = _leaves(full)
            cu = (0, S)
            o, _ = gdn.chunk_gated_delta_rule(*leaves[:3], g=leaves[3], beta=leaves[4], cu_seqlens_cpu=cu,
                                              cu_seqlens=torch.tensor(cu, dtype=torch.int32, device=device))
            o.backward(full["do"])
            want = [o.detach()] + [t.grad for t in leaves]
            magnitudes = [float(t.float().abs().max()) for t in want]
        context = gdn.build_kcp_context((0, S), device=device)
        cu_mine = (0, T)
        cu_mine_dev = torch.tensor(cu_mine, dtype=torch.int32, device=device)

        def run(mode):
            """This rank's slice: under the context with the exchange `mode`, or (mode None) as a sequence of its own
            with nothing crossing the cuts -- the control that the comparison below must reject."""
            leaves = _leaves(mine)
            if mode is None:
                o, _ = gdn.chunk_gated_delta_rule(*leaves[:3], g=leaves[3], beta=leaves[4], cu_seqlens=cu_mine_dev,
                                                  cu_seqlens_cpu=cu_mine)
            else:
                package.configure(cake_gdn_variant="det", cake_gdn_kcp_exchange=mode)
                o = gdn.kcp_chunk_gated_delta_rule(*leaves, context)
            o.backward(mine["do"])
            return [o.detach()] + [t.grad for t in leaves]

        for mode in ("parallel", "sequential", None):
            worst_rms = worst_abs = 0.0
            finite, same_bits = True, True
            for i, local in enumerate(run(mode)):
                whole = torch.empty((world * local.shape[1], *local.shape[2:]), dtype=local.dtype, device=device)
                dist.all_gather_into_tensor(whole, local[0].contiguous())
                if rank == 0:
                    ref, got = want[i][0].double(), whole.double()
                    err = got - ref
                    finite = finite and bool(torch.isfinite(got).all()) and bool(torch.isfinite(ref).all())
                    same_bits = same_bits and bool(torch.equal(got, ref))
                    rms = float(err.square().mean().sqrt() / ref.square().mean().sqrt().clamp_min(1e-30))
                    top = float(err.abs().max() / ref.abs().max().clamp_min(1e-30))
                    # a NaN must not hide behind max(): it fails the comparison below through `finite`
                    worst_rms = rms if rms > worst_rms or rms != rms else worst_rms
                    worst_abs = top if top > worst_abs or top != top else worst_abs
            passed = finite and worst_rms <= 6e-3 and worst_abs <= 2e-2
            record = {"rel_rms": worst_rms, "max_abs_rel": worst_abs, "finite": finite, "same_bits": same_bits}
            if mode is None:
                # nothing crossed the cuts: with gates that carry state the comparison must say so, or it proves nothing
                record["rejected"] = not passed
                if gate == "weak":
                    ok = ok and not passed
                cases[f"{gate}/control: no exchange"] = record
            else:
                record["ok"] = passed
                ok = ok and passed
                cases[f"{gate}/{mode}"] = record
        del full, mine, want
    package.configure(cake_gdn_variant="det")
    return {"ok": ok, "tokens": S, "num_heads": HV, "tensors": "o, dq, dk, dv, dg, dbeta", "worst_over_tensors": cases,
            "largest_reference_magnitudes": magnitudes if rank == 0 else None,
            "budget": {"rel_rms": 6e-3, "max_abs_rel": 2e-2}}


def kda_one_sequence_per_rank(clock: Clock, device, rank: int, world: int, steps: int) -> dict:
    """The per-channel-decay variant sharded by batch: one 4,096-token sequence (H = 32) per rank, no exchange."""
    from miles_ext_kernels_b200.cake import kda
    from miles_ext_kernels_b200.workloads import bytes_per_token, flops_per_token, make_workload

    work = make_workload("cfg3", seed=3 + 1000 * rank)
    x = {n: getattr(work, n).to(device) for n in ("q", "k", "v", "g", "beta", "do")}
    cu_dev = torch.tensor(work.cu_seqlens, dtype=torch.int32, device=device)
    tokens, H = work.num_tokens, work.q.shape[2]

    def step():
        q, k, v, g, beta = _leaves(x)
        kda.chunk_kda(q, k, v, g, beta, cu_dev, cu_seqlens_cpu=work.cu_seqlens).backward(x["do"])

    for _ in range(3):
        step()
    ms = clock.timed(step, steps) / steps
    peak, peak_kind = peaks()
    t_roof = max(flops_per_token(H) * tokens / (peak["bf16_tflops_sustained"] * 1e12),
                 bytes_per_token(H, H, op="kda") * tokens / (peak["hbm_gbs"] * 1e9))
    return {"workload": f"cfg3: KDA, one sequence of {tokens} tokens per GPU, H={H}, d=128", "ms_per_step": ms,
            "value": world * tokens / (ms * 1e-3), "unit": UNIT,
            "path_roofline_frac": t_roof / (ms * 1e-3), "peak_source": f"of {peak_kind}"}


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

    clock = Clock(device, world)
    timed = clock.timed

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

    landing = e2e_step()
    ms_e2e = timed(e2e_step, args.steps)
    h2d = sum(t.numel() * t.element_size() for t in host.values())
    d2h = sum(x.numel() * x.element_size() for x in landing)
    torch.cuda.synchronize()

    # the copy floor of this box at this N: the step's bytes in and out on two streams at once, no kernel in between
    # (every rank at the same time; the ranks share the host's memory and its PCIe root ports)
    side = torch.cuda.Stream(device)
    sources = [torch.empty(x.shape, dtype=x.dtype, device=device) for x in landing]

    def copies_only():
        main = torch.cuda.current_stream(device)
        side.wait_stream(main)
        for n, t in host.items():
            resident[n].copy_(t, non_blocking=True)
        with torch.cuda.stream(side):
            for src, dst in zip(sources, landing):
                dst.copy_(src, non_blocking=True)
        main.wait_stream(side)

    copies_only()
    ms_floor = timed(copies_only, args.steps)
    del sources

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
    if top in NCU_TRAFFIC_BYTES_PER_TOKEN.get((H, HV), {}):
        traffic = NCU_TRAFFIC_BYTES_PER_TOKEN[(H, HV)][top] * tokens
    roofline.update(kernel=top, ms_per_launch=mean_ms, traffic=traffic, traffic_unit="bytes per launch",
                    traffic_source="ncu capture of a smaller cut, scaled by tokens", peak_source=f"of {peak_kind}",
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
                   "sharding": "each rank runs the whole workload; no collective on the data path (the context-parallel "
                               "configuration, which has one, is the `cp` block of this line when N >= 2)",
                   "cpu_sample_tokens": CPU_SAMPLE_TOKENS},
        "e2e": {"value": world * tokens / (ms_e2e * 1e-3 / args.steps), "unit": UNIT, "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": ms_e2e / args.steps, "parts": len(parts),
                "copy_floor_ms": ms_floor / args.steps,
                "copy_floor_gbs_per_rank": {"h2d": h2d / (ms_floor * 1e-3 / args.steps) / 1e9,
                                            "d2h": d2h / (ms_floor * 1e-3 / args.steps) / 1e9},
                "copy_floor_what": "the step's bytes in and out on two streams at once with no kernel between them, "
                                   "every rank at the same time (max over ranks): what this host's PCIe and memory "
                                   "allow at this N"},
        "gpu_launches": launches,
        "roofline": roofline,
        "path_roofline": {"t_roof_ms": 1e3 * t_roof, "frac": t_roof / step_s, "flops_per_token": flops_per_token(HV),
                          "bytes_per_token": bytes_per_token(H, HV, op=cfg.op), "peak_source": f"of {peak_kind}"},
        "miles_form": miles_form,
        "kernels_ms": {n: {"mean": v[0], "launches": v[1], "total": v[2]} for n, v in per_kernel.items()},
        "clocks": clocks,
    }
    # free this workload before the others
    del resident, host, work, pipeline, landing
    torch.cuda.empty_cache()
    if not args.no_extra:
        line["kda_sharded"] = kda_one_sequence_per_rank(clock, device, rank, world, args.steps)
        if world > 1:
            line["cp"] = context_parallel(clock, device, rank, world, args.steps)
            torch.cuda.empty_cache()
            line["cp_parity"] = context_parallel_parity(device, rank, world)
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_tokens_per_sec(args.workload, 1, 1)
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
    parser.add_argument("--no-extra", action="store_true", help="skip the kda_sharded / cp / cp_parity blocks")
    args = parser.parse_args()
    if args.workload in ("conv1d", "gated_rmsnorm"):
        run_adjacent(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
