#!/usr/bin/env python
"""Benchmark of the attention forward hot path.  Prints ONE JSON line.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Workloads (``--workload``):
  c2 (default)  MHA forward, non-causal, fp16, B=2 H=8 D=128 at N=8192 — the largest point of the
                N = 512..8192 sweep the headline metric is quoted on; the other four N are timed
                once each and reported under ``sweep``.  With --gpus N every rank runs its own
                B=2 shard of a batch of 2*N (sharded by batch x head, no communication): weak scaling.
                The same run also times, device-side only, the two configurations whose scaling
                target is a STRONG one — c3 and c5 below — on the same N GPUs and reports them under
                ``strong_scaling``; at one GPU it adds the INT8-QK configuration (``int8qk_c4``).
  c3            GQA causal bf16 B=4 Hq=32 Hkv=8 N=4096 D=128, the (batch x KV-head) groups split
                across the ranks, no communication: strong scaling.
  c4            SageAttention-style INT8-QK forward, B=2 H=16 N=8192 D=64: the step is the pre-pass
                (K mean-smoothing + int8 quantisation of Q and K) plus the attention kernel; the
                attention kernel alone is reported under ``attention_only``.
  c5            causal MHA fp16 B=1 H=32 N=131072 D=128 in ring / context-parallel mode: zig-zag
                sequence split, K/V pairs travel over NCCL send/recv while the resident Q blocks
                attend to the visiting pair, the rows' running state carried inside the attention
                kernel from step to step: strong scaling.  (--seq-len overrides N for quick checks.)

A step is one forward pass over one batch.  ``value`` is TFLOPS (4*B*H*N^2*D flops, halved for
causal) with inputs resident in HBM, timed with CUDA events on the launch stream; L2 is flushed
between steps (a 256 MiB write, outside the timed intervals).  ``e2e`` is the same metric through
the public Python operator with pinned HOST buffers: host->device copies of q, k, v and the
device->host copy of the output are inside the timed region.

``--impl reference`` times the reference's CPU PyTorch attention path (restated in
oracle/attention_oracle.py) on the host cores, on a bounded sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "mini-attention_b200"))

import torch  # noqa: E402

WORKLOADS = {
    "c2": dict(B=2, Hq=8, Hkv=8, N=8192, D=128, dtype="fp16", causal=False,
               name="MHA fwd non-causal fp16 B=2 H=8 N=8192 D=128 (top of the N=512..8192 sweep)"),
    "c3": dict(B=4, Hq=32, Hkv=8, N=4096, D=128, dtype="bf16", causal=True,
               name="GQA fwd causal bf16 B=4 Hq=32 Hkv=8 N=4096 D=128, (batch x KV-head) groups sharded"),
    "c4": dict(B=2, Hq=16, Hkv=16, N=8192, D=64, dtype="fp16", causal=False, int8qk=True,
               name="INT8-QK fwd non-causal B=2 H=16 N=8192 D=64 (fp16 in, K offset N(0,2) per channel, "
                    "int8 Q/K per 128-token block, fp16 PV); pre-pass inside the step"),
    "c5": dict(B=1, Hq=32, Hkv=32, N=131072, D=128, dtype="fp16", causal=True,
               name="long-context causal MHA fwd fp16 B=1 H=32 N=131072 D=128, zig-zag ring over the GPUs"),
}
SWEEP_N = (512, 1024, 2048, 4096)
METRIC = "attention fwd TFLOPS (fp16, D=128, N=512-8192) and % of B200 dense peak"
# Measured DRAM traffic per launch of the dominant kernel (workload key -> entry), taken from the ncu
# captures summarised under profiles/ and kept in a small file beside those summaries.
NCU_TRAFFIC_FILE = ROOT / "profiles" / "ncu_traffic.json"


def flops(B, H, N, D, causal):
    f = 4.0 * B * H * N * N * D
    return f / 2 if causal else f


def ncu_traffic(key):
    try:
        return float(json.loads(NCU_TRAFFIC_FILE.read_text())[key]["dram_bytes_per_launch"])
    except Exception:
        return None


def measured_peak(sustained: bool = False):
    """Tensor-core denominator: the measured cuBLAS bf16 rate of this pool's B200s, as a burst (a
    kernel timed alone between L2 flushes) or sustained under the power cap (a step of seconds of
    back-to-back launches, as the long-context ring workload is)."""
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            d = json.loads(p.read_text())
            if sustained:
                return float(d["bf16_tflops_sustained"]), "measured sustained (MEASURED_PEAKS.json bf16_tflops_sustained)"
            return float(d["bf16_tflops"]), "measured burst (MEASURED_PEAKS.json bf16_tflops)"
        except Exception:
            pass
    if sustained:
        return 1400.0, "fallback (1.4 PFLOP/s sustained, earlier measurement on this pool)"
    return 1590.0, "fallback (1.59 PFLOP/s, earlier measurement on this pool)"


def workload_config(w, world):
    """The ``config`` object of the JSON line: the workload only, identical for both arms."""
    return {"workload": w["name"], "batch": w["B"], "heads_q": w["Hq"], "heads_kv": w["Hkv"], "seq_len": w["N"],
            "head_dim": w["D"], "causal": w["causal"], "input_dtype": w["dtype"], "parallelism": f"shard{world}",
            "l2": "GPU arm: flushed between steps (256 MiB write outside the timed intervals); CPU arm: not applicable"}


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100", "-i", str(index)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in out.splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# ------------------------------------------------------------------------- CPU arm
def cpu_attention_sample(w, budget_s: float):
    """Time the reference's CPU PyTorch attention on (batch, head) slices of the workload until
    about `budget_s` seconds are spent.  Returns (TFLOPS, cores, description)."""
    import torch.nn.functional as F
    from oracle.attention_oracle import attention_reference, make_inputs
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    dt = torch.float16 if w["dtype"] == "fp16" else torch.bfloat16
    G = w["Hq"] // w["Hkv"]
    # one KV-head group (G query heads sharing one KV head) of one batch element per unit;
    # very long sequences are sampled at N=16384 (the N x N score matrix must fit in host memory)
    n_cpu = min(w["N"], 16384)
    q, k, v = make_inputs(1, G, 1, n_cpu, n_cpu, w["D"], dt, seed=0)
    unit_flops = flops(1, G, n_cpu, w["D"], w["causal"])
    total_units = w["B"] * w["Hkv"]

    def sdpa():  # the reference test's call (tests/test_correctness.py:35-43), GQA by expand
        return F.scaled_dot_product_attention(q, k.expand(-1, G, -1, -1), v.expand(-1, G, -1, -1),
                                              is_causal=w["causal"])

    def explicit():  # reference() of the Triton file: fp32 matmul / softmax / matmul
        return attention_reference(q, k, v, causal=w["causal"])

    best = None
    for name, fn in (("F.scaled_dot_product_attention", sdpa), ("fp32 matmul-softmax-matmul", explicit)):
        t0 = time.perf_counter()
        fn()
        first = time.perf_counter() - t0
        reps = max(1, min(total_units, int((budget_s / 2) / max(first, 1e-3))))
        t0 = time.perf_counter()
        for _ in range(reps):
            fn()
        dt_s = (time.perf_counter() - t0) / reps
        tf = unit_flops / dt_s / 1e12
        if best is None or tf > best[0]:
            best = (tf, name, reps)
    tf, name, reps = best
    desc = (f"{name} on CPU, {reps} of {total_units} (batch x KV-head) units of the workload "
            f"(each {G} query head(s) x N={n_cpu}" + (f", sampled below the workload's N={w['N']}" if n_cpu != w["N"] else "")
            + f"), {cores} threads")
    return tf, cores, desc


def cpu_baseline_median(w, samples: int, budget_s: float):
    """Median of `samples` independent samples (a single short sample varies by tens of per cent)."""
    runs = [cpu_attention_sample(w, budget_s) for _ in range(samples)]
    runs.sort(key=lambda r: r[0])
    tf, cores, desc = runs[len(runs) // 2]
    return tf, cores, desc + f"; median of {samples} samples ({', '.join(f'{r[0]:.2f}' for r in runs)} TFLOPS)"


def run_reference_arm(args, w, rank):
    """The reference's own CPU path on this box's host cores.  A step is one bounded sample of the
    workload; `value` is the median over the steps and `ms_per_step` the time one whole step of the
    workload would take at that rate."""
    if rank != 0:
        return
    for _ in range(args.warmup):
        cpu_attention_sample(w, 1.0)
    steps = max(args.steps, 3)
    runs = [cpu_attention_sample(w, max(2.0, 60.0 / steps)) for _ in range(steps)]
    runs.sort(key=lambda r: r[0])
    value, cores, desc = runs[len(runs) // 2]
    desc += f"; median of {steps} samples"
    total = flops(w["B"], w["Hq"], w["N"], w["D"], w["causal"]) * max(args.gpus, 1) if args.workload == "c2" \
        else flops(w["B"], w["Hq"], w["N"], w["D"], w["causal"])
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "TFLOPS", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total / value / 1e9,
        "higher_is_better": True, "scaling": "weak" if args.workload in ("c2", "c4") else "strong", "vs_baseline": None,
        "dtype": w["dtype"], "data": "synthetic", "config": workload_config(w, max(args.gpus, 1)),
        "cpu_baseline": {"value": value, "unit": "TFLOPS", "cores": cores, "kind": "port", "sample": desc},
        "e2e": {"value": value, "unit": "TFLOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def reference_gpu_kernel_leg(B, H, N_list, D, dev, flush, stream):
    """Optional baseline: the reference's own mma.sync kernel (newest tree) rebuilt for sm_100 by
    oracle/build_ref_kernel.py, timed on this GPU with the same protocol in two of its configurations:
    K7 (the end of its K1..K7 progression) and BL4 (Br=128, Bc=128, 8 warps, the largest tile of its
    Blackwell list, _bench_sm120.py:90-103).  Its output is compared with the product kernel's on the
    same inputs once per N.  Returns {} when the built extension is not present."""
    try:
        from oracle.build_ref_kernel import load_built
        ext = load_built()
    except Exception as e:  # missing file, ABI mismatch ...
        return {"unavailable": repr(e)}
    if ext is None:
        return {}
    import miniattn
    from miniattn.kernel_configs import DType, FlashForwardKernelConfig, get_kernel_progression_configs
    cfgs = {"K7": get_kernel_progression_configs()[6],
            "BL4": FlashForwardKernelConfig(DType.FP16, 128, 128, 128, 8, True, True, True, 2, 2, 2, True, True)}
    out = {"kernel": "reference flash_forward_kernel (mma.sync) rebuilt for sm_100; configs K7 and BL4"}
    for n in N_list:
        q = torch.randn(B, n, H, D, device=dev, dtype=torch.float16)  # the reference's (B,N,H,D) layout
        k, v = torch.randn_like(q), torch.randn_like(q)
        ours = miniattn.flash_attn_fwd(q, k, v, layout="bnhd")
        entry = {}
        for tag, cfg in cfgs.items():
            o = torch.empty_like(q)
            try:
                for _ in range(3):
                    ext.forward(cfg, q, k, v, o, False)
                torch.cuda.synchronize(dev)
            except Exception as e:
                entry[tag] = {"unavailable": repr(e)[:200]}
                continue
            tot = 0.0
            for _ in range(10):
                flush.zero_()
                torch.cuda.synchronize(dev)
                # benchmark=True: the extension brackets its own launch with CUDA events
                # (flash_attention.cu:111-131); its Python-side call overhead stays outside
                _, ms = ext.forward(cfg, q, k, v, o, True)
                tot += ms
            entry[tag] = {"ms": tot / 10, "tflops": flops(B, H, n, D, False) / (tot / 10) / 1e9,
                          "max_abs_diff_vs_product_kernel": (o.float() - ours.float()).abs().max().item()}
        out[str(n)] = entry
    return out


# ------------------------------------------------------------------------- GPU arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="c2", choices=sorted(WORKLOADS))
    ap.add_argument("--kernel", default="auto")
    ap.add_argument("--seq-len", type=int, default=0, help="override the workload's sequence length")
    ap.add_argument("--no-balance", action="store_true",
                    help="plain launch (one CTA per work item) instead of the balanced one, for A/B timings")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sweep", action="store_true",
                    help="skip the one-shot timings of the smaller N and the extra legs (profiling runs)")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer end-to-end leg (profiling runs)")
    args = ap.parse_args()
    w = dict(WORKLOADS[args.workload])
    if args.seq_len:
        w["N"] = args.seq_len
        w["name"] += f" [N overridden to {args.seq_len}]"
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))

    if args.impl == "reference":
        run_reference_arm(args, w, rank)
        return

    args.warmup = max(args.warmup, 3)
    import miniattn
    import torch.distributed as dist
    from miniattn import parallel as par
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the attention path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream(dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    ring_group = [None]

    def get_ring_group():  # K/V pairs travel on a high-priority NCCL stream (made once, on first use)
        if world > 1 and ring_group[0] is None:
            ring_group[0] = par.ring_process_group()
        return ring_group[0]

    last_median = [0.0]

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            flush.zero_()
            fn()
        barrier()
        evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        for a, b_ in evs:
            flush.zero_()
            a.record(stream)
            fn()
            b_.record(stream)
        barrier()
        per_step = [a.elapsed_time(b_) for a, b_ in evs]
        ms = sum(per_step)
        last_median[0] = statistics.median(per_step)  # this rank's median step, reported beside the mean
        if world > 1:
            t = torch.tensor([ms], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms / steps

    def shard_of(key, wl):
        """Per-rank shape, scaling kind, whole-job flops and per-rank flops of a workload."""
        B, Hq, Hkv, N, D, causal = wl["B"], wl["Hq"], wl["Hkv"], wl["N"], wl["D"], wl["causal"]
        if key == "c3":
            # strong scaling: split the B*Hkv groups (whole groups stay on one GPU); per-rank tensors
            # are (1, G*groups, N, D) / (1, groups, N, D)
            groups = B * Hkv
            assert groups % world == 0, "group count must divide by the number of GPUs"
            per = groups // world
            G = Hq // Hkv
            return dict(B=1, Hq=per * G, Hkv=per, N=N), "strong", flops(B, Hq, N, D, causal), \
                flops(1, per * G, N, D, causal)
        if key == "c5":
            assert N % (2 * world * 128) == 0, "sequence must split into 2*world blocks of whole tiles"
            tot = flops(B, Hq, N, D, causal)   # this rank holds its two zig-zag blocks
            return dict(B=B, Hq=Hq, Hkv=Hkv, N=N // world), "strong", tot, tot / world
        tot = flops(B, Hq, N, D, causal)
        return dict(B=B, Hq=Hq, Hkv=Hkv, N=N), "weak", tot * world, tot

    def ring_parity_check(grp):
        """The same ring (same transport, same kernels) on a sequence short enough for one launch:
        every rank's rows against the single-launch kernel over the whole sequence, untimed."""
        n_chk = 4096 * world
        gen = torch.Generator(device=dev).manual_seed(99)   # same tensors on every rank
        full = [torch.randn(1, 8, n_chk, 128, device=dev, dtype=torch.float16, generator=gen) for _ in range(3)]
        single = miniattn.flash_attn_fwd(*full, causal=True)
        mine = [par.zigzag_split(t_, world)[rank].contiguous() for t_ in full]
        out = par.ring_forward(*mine, causal=True, rank=rank, world=world, group=grp, verify_origin=world > 1)
        err = (out.float() - par.zigzag_split(single, world)[rank].float()).abs().max()
        if world > 1:
            dist.all_reduce(err, op=dist.ReduceOp.MAX)
        return {"what": f"ring over {world} rank(s) vs one launch, causal fp16 B=1 H=8 N={n_chk} D=128, origin tags verified",
                "max_abs_diff": float(err.item()), "tolerance": 2e-3, "ok": bool(err.item() <= 2e-3)}

    def device_leg(key, steps, warmup):
        """Device-timed run of another workload on the same ranks (inputs made on the device)."""
        wl = WORKLOADS[key]
        dtl = torch.float16 if wl["dtype"] == "fp16" else torch.bfloat16
        sh, kind, tot, per_rank = shard_of(key, wl)
        gen = torch.Generator(device=dev).manual_seed(4321 + rank)
        ql = torch.randn(sh["B"], sh["Hq"], sh["N"], wl["D"], device=dev, dtype=dtl, generator=gen)
        kl = torch.randn(sh["B"], sh["Hkv"], sh["N"], wl["D"], device=dev, dtype=dtl, generator=gen)
        vl = torch.randn(sh["B"], sh["Hkv"], sh["N"], wl["D"], device=dev, dtype=dtl, generator=gen)
        res = {"workload": wl["name"], "scaling": kind, "n_gpus": world, "per_gpu": sh, "steps": steps, "warmup": warmup}
        if wl.get("int8qk"):
            kl += 2.0 * torch.randn(1, 1, 1, wl["D"], device=dev, dtype=dtl, generator=gen)
            bufs_l = miniattn.Int8QK(sh["B"], sh["Hq"], sh["Hkv"], sh["N"], sh["N"], wl["D"], dev)
            ol = torch.empty_like(ql)
            ms = timed(lambda: miniattn.flash_attn_fwd_int8qk(ql, kl, vl, out=ol, buffers=bufs_l), steps, warmup)
            ms_a = timed(lambda: miniattn.flash_attn_fwd_int8qk(ql, kl, vl, out=ol, buffers=bufs_l, quantize=False),
                         steps, warmup)
            ms_f = timed(lambda: miniattn.flash_attn_fwd(ql, kl, vl, out=ol), steps, warmup)
            res.update({"attention_only_ms": ms_a, "fp16_kernel_same_shape_ms": ms_f,
                        "launches_per_step": 3})
        elif key == "c5":
            grp = get_ring_group()
            ms = timed(lambda: par.ring_forward(ql, kl, vl, causal=True, rank=rank, world=world, group=grp), steps, warmup)
            res["launches_per_step"] = sum(len(par.ring_step_tasks(rank, world, s_, True)) for s_ in range(world))
            res["parity_check"] = ring_parity_check(grp)
        else:
            ol = torch.empty_like(ql)
            ms = timed(lambda: miniattn.flash_attn_fwd(ql, kl, vl, causal=wl["causal"], out=ol), steps, warmup)
            res["launches_per_step"] = 1
        peak_l, src_l = measured_peak(sustained=(key == "c5"))
        res.update({"ms_per_step": ms, "tflops": tot / ms / 1e9, "per_gpu_tflops": per_rank / ms / 1e9,
                    "frac_of_measured_peak_per_gpu": per_rank / ms / 1e9 / peak_l, "peak_source": src_l,
                    "timing": "sum of per-step CUDA-event intervals, max over ranks; L2 flushed between steps"})
        return res

    dt = torch.float16 if w["dtype"] == "fp16" else torch.bfloat16
    B, Hq, Hkv, N, D, causal = w["B"], w["Hq"], w["Hkv"], w["N"], w["D"], w["causal"]
    ring = args.workload == "c5"
    shard, scaling, total_flops, step_flops = shard_of(args.workload, w)
    sB, sHq, sHkv, sN = shard["B"], shard["Hq"], shard["Hkv"], shard["N"]

    g = torch.Generator().manual_seed(1234 + rank)
    hq = torch.randn(sB, sHq, sN, D, generator=g).to(dt).pin_memory()
    hk = torch.randn(sB, sHkv, sN, D, generator=g).to(dt).pin_memory()
    hv = torch.randn(sB, sHkv, sN, D, generator=g).to(dt).pin_memory()
    ho = torch.empty_like(hq).pin_memory()
    q, k, v = hq.to(dev), hk.to(dev), hv.to(dev)
    o = torch.empty_like(q)
    launches_per_step = 1
    int8 = bool(w.get("int8qk"))
    if int8:
        hk.copy_((hk.float() + 2.0 * torch.randn(1, 1, 1, D, generator=g)).to(dt))  # per-channel K offset
        k.copy_(hk)
        bufs = miniattn.Int8QK(sB, sHq, sHkv, sN, sN, D, dev)
        launches_per_step = 3  # Q quantiser + K column sums, K quantiser, attention

        def attend():
            miniattn.flash_attn_fwd_int8qk(q, k, v, causal=causal, out=o, buffers=bufs)
    elif ring:
        launches_per_step = sum(len(par.ring_step_tasks(rank, world, s_, causal)) for s_ in range(world))
        ring_out = [o]
        grp_main = get_ring_group()

        def attend():
            ring_out[0] = par.ring_forward(q, k, v, causal=causal, rank=rank, world=world, group=grp_main)
    else:
        def attend():
            miniattn.flash_attn_fwd(q, k, v, causal=causal, out=o, kernel=args.kernel,
                                    balance=not args.no_balance)

    if ring or int8:
        def step_e2e():
            q.copy_(hq, non_blocking=True)
            k.copy_(hk, non_blocking=True)
            v.copy_(hv, non_blocking=True)
            attend()
            ho.copy_(ring_out[0] if ring else o, non_blocking=True)
    else:
        def step_e2e():  # the public host-buffer operator: copies overlapped with compute per chunk
            miniattn.flash_attn_fwd_host(hq, hk, hv, ho, causal=causal, device=dev, kernel=args.kernel)

    sampler = ClockSampler(local_rank) if rank == 0 else None
    if sampler is not None:
        time.sleep(0.6)  # let nvidia-smi start sampling before the timed region
    ms_dev = timed(attend, args.steps, args.warmup)
    ms_dev_median = last_median[0]
    clocks = sampler.stop() if sampler else None
    ms_e2e = ms_dev if args.no_e2e else timed(step_e2e, max(3, args.steps // 2), 3)
    status = miniattn.device_status(dev)

    extra = {}
    if int8:
        def attn_only():
            miniattn.flash_attn_fwd_int8qk(q, k, v, causal=causal, out=o, buffers=bufs, quantize=False)

        def prepass_only():
            miniattn.flash_attn_fwd_int8qk(q, k, v, causal=causal, out=o, buffers=bufs, attend=False)
        ms_a = timed(attn_only, args.steps, 3)
        ms_p = timed(prepass_only, args.steps, 3)
        pre_bytes = (sHq + 2 * sHkv) * sB * sN * D * 2 + (sHq + sHkv) * sB * sN * D
        extra["attention_only"] = {"ms": ms_a, "tflops": step_flops / ms_a / 1e9}
        extra["prepass_only"] = {"ms": ms_p, "algorithmic_bytes": pre_bytes, "hbm_gbs": pre_bytes / ms_p / 1e6}
        ms_f = timed(lambda: miniattn.flash_attn_fwd(q, k, v, causal=causal, out=o), args.steps, 3)
        extra["fp16_kernel_same_shape"] = {"ms": ms_f, "tflops": step_flops / ms_f / 1e9}
        # Half of the flops (Q K^T) may run at the int8 rate, half (P V) at the 16-bit rate:
        # t >= F/2/P_int8 + F/2/P_16.  No int8 peak is measured on this pool; twice the measured
        # 16-bit peak stands in for it (the ratio of the nominal dense figures, 4.5 / 2.25 PFLOP/s).
        peak16, _ = measured_peak()
        t_bound_ms = (step_flops / 2 / (2 * peak16 * 1e12) + step_flops / 2 / (peak16 * 1e12)) * 1e3
        extra["int8_blended_bound"] = {"ms": t_bound_ms, "frac_attention_only": t_bound_ms / ms_a,
                                       "int8_peak_assumed_tflops": 2 * peak16}
        # At D = 64 the exponentials bound the kernel before the tensor pipe does: one exp2 per
        # score, 16 per clock per SM (the special-function unit), at the maximum SM clock.
        props = torch.cuda.get_device_properties(dev)
        mhz = (clocks or {}).get("sm_max_mhz") or 1965.0
        t_exp_ms = (sB * sHq * sN * sN * (0.5 if causal else 1.0)) / (16.0 * props.multi_processor_count * mhz * 1e6) * 1e3
        extra["exp2_bound"] = {"ms": t_exp_ms, "frac_attention_only": t_exp_ms / ms_a}
    sweep = {}
    legs = args.workload == "c2" and not args.no_sweep and not args.seq_len
    if legs and rank == 0:
        for n in SWEEP_N:
            qs = torch.randn(B, Hq, n, D, device=dev, dtype=dt)
            ks, vs = torch.randn_like(qs), torch.randn_like(qs)
            os_ = torch.empty_like(qs)
            fn = lambda: miniattn.flash_attn_fwd(qs, ks, vs, out=os_, kernel=args.kernel,  # noqa: E731
                                                 balance=not args.no_balance)
            for _ in range(3):
                fn()
            torch.cuda.synchronize(dev)
            tot = 0.0
            for _ in range(10):
                flush.zero_()
                a, b_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(stream); fn(); b_.record(stream)
                b_.synchronize()
                tot += a.elapsed_time(b_)
            sweep[str(n)] = {"ms": tot / 10, "tflops": flops(B, Hq, n, D, False) / (tot / 10) / 1e9}
    if legs and rank == 0 and world == 1:
        ref_leg = reference_gpu_kernel_leg(B, Hq, SWEEP_N + (N,), D, dev, flush, stream)
        if ref_leg:
            extra["reference_kernel_on_this_gpu"] = ref_leg
    if legs:
        # The two configurations whose scaling target is a strong one, on the same ranks.  Every rank
        # takes part (the ring exchanges K/V pairs); the headline tensors are released first.
        del q, k, v, o
        torch.cuda.empty_cache()
        barrier()
        strong = {"c3": device_leg("c3", min(args.steps, 50), 3)}
        if world == 1:   # before the ring leg, whose seconds at the power cap leave the clocks low for a while
            extra["int8qk_c4"] = device_leg("c4", min(args.steps, 30), 3)
        strong["c5"] = device_leg("c5", 5, 3)
        torch.cuda.empty_cache()
        extra["strong_scaling"] = strong
        status |= miniattn.device_status(dev)
    if world > 1:
        dist.barrier()

    if rank == 0:
        peak, peak_src = measured_peak(sustained=ring)  # the ring step runs ~0.15 s of launches back to back
        value = total_flops / ms_dev / 1e9
        achieved = step_flops / ms_dev / 1e9
        cfg = workload_config(w, world)
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOPS", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_dev, "ms_per_step_median_rank0": ms_dev_median,
            "higher_is_better": True, "scaling": scaling,
            "vs_baseline": None, "dtype": ("int8 QK^T (s32 acc) + " + w["dtype"] + " PV" if w.get("int8qk") else w["dtype"]),
            "data": "synthetic",
            "config": cfg,
            "method": {"per_gpu": shard,
                       "parallelism": (f"zig-zag ring over {world} GPU(s): NCCL send/recv of K/V pairs, running state "
                                       "carried inside the attention kernel" if ring
                                       else f"batch x head shards over {world} GPU(s), no communication"),
                       "launch": "plain" if args.no_balance else "balanced (key ranges cut to fill the last round of CTAs)",
                       "timing": "sum of per-step CUDA-event intervals on the launch stream, max over ranks"},
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peak, "unit": "TFLOP/s",
                         "frac": achieved / peak, "traffic": ncu_traffic(args.workload),
                         "peak_source": peak_src, "frac_of_nominal_2250": achieved / 2250.0,
                         "algorithmic_flops_per_step": step_flops,
                         "algorithmic_hbm_bytes_per_step": (2 * sHq + 2 * sHkv) * sB * sN * D * 2,
                         "hbm_gbs": (2 * sHq + 2 * sHkv) * sB * sN * D * 2 / ms_dev / 1e6},
            "e2e": None if args.no_e2e else {
                "value": total_flops / ms_e2e / 1e9, "unit": "TFLOPS", "ms_per_step": ms_e2e,
                "h2d_bytes_per_step": hq.numel() * 2 + hk.numel() * 2 + hv.numel() * 2,
                "d2h_bytes_per_step": ho.numel() * 2},
            "gpu_launches": args.steps * launches_per_step,
            "clocks": clocks,
            "device_status": status,
            "kernel": args.kernel,
        }
        if sweep:
            line["sweep"] = sweep
        line.update(extra)
        if world == 1 and not args.no_cpu_baseline:
            tf, cores, desc = cpu_baseline_median(w, 3, 7.0)
            line["cpu_baseline"] = {"value": tf, "unit": "TFLOPS", "cores": cores, "kind": "port", "sample": desc}
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
