#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cfg3|cfg5]

One step = causal bf16 attention forward + backward over one batch of synthetic input.
Default workload `cfg5` (benchmark configuration 5): Q,K,V,dO [B=1,H=64,S=32768,D=128], Q/K/V ~
0.5*N(0,1), dO ~ N(0,1).  With N > 1 (launched under torchrun, one process per GPU) the 64
heads are sharded over the ranks in contiguous ranges -- strong scaling, no collective on the
data path -- and the step all-gathers O over NCCL on a side stream, overlapped with the
backward.  At N = 1 the line also carries `cfg3` (benchmark configuration 3, [4,32,4096,128]: the shape
the forward target is stated on) and `decode` (config 4).  `--workload cfg3` makes config 3 the
main workload (weak scaling: every rank owns its own 128 slices).  FLOPs are counted as the task defines them: 2 per MAC,
forward = 2 GEMMs, backward = 5 GEMMs (2.5x forward), causal = half of dense.

Prints ONE JSON line (rank 0).  `value` is device-timed with inputs resident in HBM;
`e2e` goes through the host-buffer C-ABI calls (pinned host memory, uploads and downloads
inside the timed region).  `--impl reference` times the CPU oracle (a NumPy port of the
reference's composed ops; the reference's own Python cannot travel to the GPU box) on
bounded samples of the same workload.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (B, H, S, D) per rank
    "cfg3": dict(B=4, H=32, S=4096, D=128, desc="bf16 causal fwd+bwd, Q/K/V [4,32,4096,128] per GPU"),
    "cfg5": dict(B=1, H=64, S=32768, D=128, desc="bf16 causal fwd+bwd, Q/K/V [1,64,32768,128], heads sharded over the GPUs"),
    "cfg2": dict(B=8, H=16, S=1024, D=64, desc="bf16 causal fwd+bwd, Q/K/V [8,16,1024,64] per GPU"),
}
# DRAM traffic per launch (dram__bytes_read.sum + dram__bytes_write.sum) measured with ncu; keyed by
# workload, because the same kernel moves different bytes per launch on each.  "per_slice" entries were
# captured on a few slices of the workload's slice shape and scale with the slice count (the kernels walk
# the slices one after the other, so a slice's traffic does not depend on how many follow).
NCU_TRAFFIC_BYTES = {
    "cfg3": {"attn_fwd_sm100": 591.5e6, "attn_bwd_sm100_dkv": 851.6e6, "attn_bwd_sm100_dq": 728.4e6,
             "attn_bwd_fused_sm100": 1507.7e6},
    "cfg2": {"attn_fwd_sm100": 52.3e6, "attn_bwd_fused_sm100": 132.1e6},
    "cfg5_per_slice": {"attn_fwd_sm100": 26.08e6, "attn_bwd_sm100_dkv": 35.10e6, "attn_bwd_sm100_dq": 34.66e6},
    # config 4 = 8 x the captured batch-8 launch (the full launch holds 8.6 GB, too large a capture)
    "decode": {"attn_decode": 8.637e9, "attn_decode_gq_sm100": 8.622e9},
}


def fwd_flops(B, H, S, L, D, causal=True):
    return 4.0 * B * H * S * L * D * (0.5 if causal else 1.0)


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return dict(bf16=float(d["bf16_tflops"]), bf16_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])),
                    hbm=float(d["hbm_gbs"]), source="measured")
    return dict(bf16=1590.0, bf16_sustained=1400.0, hbm=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu = gpu_index
        self.lines = []
        self.proc = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.gpu), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1])); mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------ CPU arm
def cpu_sample_seconds(S, D, seed, n_threads=None):
    """One (batch, head) slice of the workload, causal fwd+bwd, through the CPU oracle."""
    from oracle import attention_oracle as orc
    q, k, v, do = orc.make_inputs(seed, 1, 1, S, S, D, sigma=0.5)
    t0 = time.perf_counter()
    orc.attention_backward(q, k, v, do, causal=True)
    return time.perf_counter() - t0


def cpu_threads():
    try:
        from threadpoolctl import threadpool_info
        n = [p.get("num_threads", 1) for p in threadpool_info() if p.get("user_api") == "blas"]
        if n:
            return int(max(n))
    except Exception:
        pass
    return os.cpu_count() or 1


def use_all_host_threads():
    """torchrun exports OMP_NUM_THREADS=1 to its ranks; the CPU arm is one process and takes every core."""
    try:
        from threadpoolctl import threadpool_limits
        threadpool_limits(limits=len(os.sched_getaffinity(0)), user_api="blas")
    except Exception:
        pass


def run_reference_arm(args, w, rank):
    if rank != 0:
        return
    use_all_host_threads()
    S, D = w["S"], w["D"]
    S_cpu = min(S, 4096)       # a 32768^2 fp32 score matrix does not fit a bounded step; sample query/key prefix
    for _ in range(max(args.warmup, 0)):
        cpu_sample_seconds(S_cpu, D, 1)
    ts = [cpu_sample_seconds(S_cpu, D, 100 + i) for i in range(args.steps)]
    fl = 3.5 * fwd_flops(1, 1, S_cpu, S_cpu, D, True)
    sec = float(np.mean(ts))
    val = fl / sec / 1e12
    what = "one (batch,head) slice" if S_cpu == S else f"the S=L={S_cpu} prefix of one (batch,head) slice"
    sample = f"{what} per step, causal fwd+bwd, D={D}, fp32 NumPy, all BLAS threads"
    line = {
        "impl": "reference", "metric": "attention fwd+bwd TFLOP/s", "value": val, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec * 1e3,
        "higher_is_better": True, "scaling": "strong" if args.workload == "cfg5" else "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic", "config": {"workload": w["desc"], "sampled": sample},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": cpu_threads(), "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------ GPU arm
ALG_FWD_UNITS = {  # algorithmic FLOPs per launch, in units of the forward's count
    "attn_fwd_sm100": 1.0,        # QK^T, PV
    "attn_bwd_sm100_dkv": 2.0,    # S recompute, dP, dV, dK  (4 of the 5 backward GEMMs)
    "attn_bwd_sm100_dq": 0.5,     # dQ (its S and dP recompute is overhead of the two-pass design)
    "attn_bwd_fused_sm100": 2.5,  # single pass: all 5 backward GEMMs, nothing recomputed
}


def verify_slice(tt, name, tensors, S, D, n_local):
    """Re-checks a timed result against the CPU oracle after the timed region: one sampled local slice,
    whole for S <= 4096, the first and last 128-row query blocks (O, lse, dQ, and dK/dV of the last key
    block, which only those rows feed) for longer slices.  Returns the `verified` block of the line."""
    from oracle import attention_oracle as orc
    q, k, v, do, out, lse, dq, dk, dv = tensors
    f = lambda t, i: t.reshape(n_local, *t.shape[2:])[i].float().cpu().numpy()
    idx = n_local - 1
    errs, ok = {}, True

    def upd(key, got, ref, tol):
        nonlocal ok
        e = orc.max_abs_err(got, ref)
        errs[key] = max(errs.get(key, 0.0), e)
        ok = ok and (e <= tol)

    if S <= 4096:
        o_r, l_r, dq_r, dk_r, dv_r = orc.attention_backward_chunked(f(q, idx), f(k, idx), f(v, idx), f(do, idx), True)
        upd("o", f(out, idx), o_r, 2e-2); upd("lse", f(lse, idx), l_r, 2e-2)
        upd("dq", f(dq, idx), dq_r, orc.bf16_grad_tol(dq_r))
        upd("dk", f(dk, idx), dk_r, orc.bf16_grad_tol(dk_r)); upd("dv", f(dv, idx), dv_r, orc.bf16_grad_tol(dv_r))
        what = f"local slice {idx} in full against the oracle"
    else:
        kn, vn = f(k, idx), f(v, idx)
        for row0 in (0, S - 128):
            sl = slice(row0, row0 + 128)
            o_r, l_r, dq_r, dk_p, dv_p, _ = orc.attention_backward_rows(f(q, idx)[sl], f(do, idx)[sl], kn, vn, row0, S, True)
            upd("o", f(out, idx)[sl], o_r, 2e-2); upd("lse", f(lse, idx)[sl], l_r, 2e-2)
            upd("dq", f(dq, idx)[sl], dq_r, orc.bf16_grad_tol(dq_r))
            if row0 == S - 128:
                upd("dk", f(dk, idx)[sl], dk_p[row0:], orc.bf16_grad_tol(dk_p[row0:]))
                upd("dv", f(dv, idx)[sl], dv_p[row0:], orc.bf16_grad_tol(dv_p[row0:]))
        what = f"local slice {idx}: first and last 128 query rows (O, lse, dQ) and last 128 keys (dK, dV) against the oracle"
    return {"ok": bool(ok), "max_abs_err": errs, "what": what}


def gpu_numa_affinity(gpu_index):
    """Binds this process to the CPU cores next to its GPU (NVML's affinity mask), so that the pinned
    host buffers it allocates afterwards land in that socket's memory.  Returns the core count or None."""
    try:
        import pynvml
        pynvml.nvmlInit()
        h = pynvml.nvmlDeviceGetHandleByIndex(gpu_index)
        n_words = (os.cpu_count() + 63) // 64
        mask = pynvml.nvmlDeviceGetCpuAffinity(h, n_words)
        cores = [64 * w + b for w, word in enumerate(mask) for b in range(64) if (word >> b) & 1]
        allowed = sorted(set(cores) & set(os.sched_getaffinity(0)))
        if allowed:
            os.sched_setaffinity(0, allowed)
            return len(allowed)
    except Exception:
        pass
    return None


def run_workload(tt, name, steps, warmup, world, rank, dev, peaks, e2e_steps, sample_clocks, sharded=None, verify=True):
    """Times `steps` forward+backward steps of workload `name`; returns the fields of the JSON line.
    `sharded` (a ShardedAttention) is the library's multi-GPU path: forward + all-gather of O on the
    library's side stream, backward overlapping it."""
    import ctypes
    import torch
    import torch.distributed as dist
    capi = tt.capi
    w = WORKLOADS[name]
    B, H, S, D = w["B"], w["H"], w["S"], w["D"]
    strong = name == "cfg5"
    if strong:
        _, cnt = capi.shard_range(B * H, world, rank)
        Bl, Hl = 1, cnt
    else:
        Bl, Hl = B, H
    n_local = Bl * Hl
    g = torch.Generator(device=dev).manual_seed(1234 + rank)
    mk = lambda sig: (torch.randn((Bl, Hl, S, D), generator=g, device=dev) * sig).to(torch.bfloat16)
    q, k, v, do = mk(0.5), mk(0.5), mk(0.5), mk(1.0)
    out = torch.empty_like(q)
    lse = torch.empty((Bl, Hl, S), dtype=torch.float32, device=dev)
    desc = capi.make_desc(Bl, Hl, S, S, D, capi.TT_BF16, True, None)
    ws = torch.empty(max(int(capi.lib.tt_attn_bwd_workspace_bytes(ctypes.byref(desc))), 256), dtype=torch.uint8, device=dev)
    grads = {}
    use_mgpu = sharded is not None and world > 1 and strong
    out_full = torch.empty((world * n_local, S, D), dtype=torch.bfloat16, device=dev) if use_mgpu else None

    def step():
        if use_mgpu:
            sharded.forward(q, k, v, B, H, causal=True, out=out, lse=lse, out_full=out_full)
            grads["g"] = sharded.backward(q, k, v, out, lse, do, B, H, causal=True, workspace=ws)
            sharded.wait()
        else:
            tt.attention_forward(q, k, v, causal=True, out=out, lse=lse)
            grads["g"] = tt.attention_backward(q, k, v, out, lse, do, causal=True, workspace=ws)

    def barrier():
        if world > 1:
            dist.barrier()

    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    tt.check_device_status()
    barrier()
    sampler = ClockSampler(dev.index)
    if sample_clocks:
        sampler.start()
        time.sleep(0.25)
    capi.profile_reset()
    capi.profile_enable(True)
    launches0 = capi.launch_count()
    torch.cuda.synchronize()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    barrier()
    ms_total = e0.elapsed_time(e1)
    launches = capi.launch_count() - launches0
    capi.profile_enable(False)
    prof = capi.profile_read()
    clocks = sampler.stop() if sample_clocks else None
    tt.check_device_status()
    if world > 1:
        t = torch.tensor([ms_total], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_step = ms_total / steps
    ms_step_local = ms_step
    f_fwd = fwd_flops(Bl, Hl, S, S, D, True)                       # this rank's forward count per step
    f_step_all = 3.5 * fwd_flops(B, H, S, S, D, True) if strong else 3.5 * f_fwd * world
    value = f_step_all / (ms_step * 1e-3) / 1e12

    # the timed outputs against the oracle (rank 0 reports; every rank's result is its own shard's)
    verified = None
    if verify:
        try:
            verified = verify_slice(tt, name, (q, k, v, do, out, lse) + tuple(grads["g"][:3]), S, D, n_local)
            if use_mgpu:
                torch.cuda.synchronize()
                b0 = rank * n_local
                verified["gathered_out_matches_shard"] = bool(torch.equal(out_full[b0:b0 + n_local], out.reshape(n_local, S, D)))
                verified["ok"] = verified["ok"] and verified["gathered_out_matches_shard"]
        except Exception as e:  # noqa: BLE001
            verified = {"ok": False, "error": str(e)}

    # per-kernel rooflines from the events recorded inside the timed region
    kernels = {}
    total_ms = max(sum(x[0] for x in prof.values()), 1e-9)
    if name == "cfg3":
        traffic = dict(NCU_TRAFFIC_BYTES["cfg3"]); traffic_note = None
    elif name == "cfg5":
        traffic = {k_: v_ * n_local for k_, v_ in NCU_TRAFFIC_BYTES["cfg5_per_slice"].items()}
        traffic_note = ("ncu capture of two S=32768 slices, scaled by the slice count of the launch (inputs cross DRAM "
                        "once; the outputs of the two-slice capture stayed in L2, add 8.4-16.8 MB per slice for them)")
    elif name == "cfg2":
        traffic = dict(NCU_TRAFFIC_BYTES["cfg2"]); traffic_note = None
    else:
        traffic, traffic_note = {}, None
    for kname, (ms, n) in prof.items():
        per = ms / n
        ent = {"launches": n, "ms_per_launch": per, "share": ms / total_ms}
        if kname in ALG_FWD_UNITS:
            ach = ALG_FWD_UNITS[kname] * f_fwd / (per * 1e-3) / 1e12
            ent.update({"bound": "tensor", "achieved": ach, "peak": peaks["bf16"], "unit": "TFLOP/s",
                        "frac": ach / peaks["bf16"], "traffic": traffic.get(kname)})
        kernels[kname] = ent
    dom = max((n for n in kernels if n in ALG_FWD_UNITS), key=lambda n: kernels[n]["share"], default=None)
    roofline = None
    if dom:
        roofline = {k_: kernels[dom][k_] for k_ in ("bound", "achieved", "peak", "unit", "frac", "traffic")}
        roofline["kernel"] = dom
        roofline["peak_source"] = f"bf16_tflops (burst) of {peaks['source']} MEASURED_PEAKS.json"
        if name == "cfg5":
            # this step keeps the GPU at its power cap for the whole timed region (see "clocks"): the
            # fraction of the sustained cuBLAS figure is given beside the (conservative) burst one
            roofline["peak_sustained"] = peaks["bf16_sustained"]
            roofline["frac_of_sustained"] = roofline["achieved"] / peaks["bf16_sustained"]
        if traffic_note and roofline["traffic"]:
            roofline["traffic_note"] = traffic_note
    fwd_tf = kernels.get("attn_fwd_sm100", {}).get("achieved")

    # end to end through the host-buffer C ABI (pinned host memory)
    e2e = None
    if e2e_steps > 0:
        hq, hk, hv, hdo = (x.cpu().pin_memory() for x in (q, k, v, do))
        ho, hl = torch.empty_like(hq).pin_memory(), torch.empty((Bl, Hl, S), dtype=torch.float32).pin_memory()
        hdq, hdk, hdv = (torch.empty_like(hq).pin_memory() for _ in range(3))
        nb = hq.numel() * 2
        nl = hl.numel() * 4

        def e2e_step():
            tt.attention_step_host(hq, hk, hv, hdo, causal=True, out=ho, lse=hl, dq=hdq, dk=hdk, dv=hdv)

        def timed(fn, n):
            barrier()
            t0 = time.perf_counter()
            for _ in range(n):
                fn()
            torch.cuda.synchronize()
            sec = (time.perf_counter() - t0) / n
            if world > 1:
                t = torch.tensor([sec], dtype=torch.float64, device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                sec = float(t.item())
            return sec

        # copy-only leg: exactly the step's bytes, uploads and downloads at the same time on two streams,
        # every rank at once -- what the host<->device links give this step with nothing to compute
        s_up, s_dn = torch.cuda.Stream(device=dev), torch.cuda.Stream(device=dev)
        d_in = [torch.empty_like(q) for _ in range(4)]
        d_lse = torch.empty_like(lse)

        def copy_step():
            with torch.cuda.stream(s_up):
                for dst, src in zip(d_in, (hq, hk, hv, hdo)):
                    dst.copy_(src, non_blocking=True)
            with torch.cuda.stream(s_dn):
                for dst, src in zip((ho, hdq, hdk, hdv), d_in):
                    dst.copy_(src, non_blocking=True)
                hl.copy_(d_lse, non_blocking=True)

        for _ in range(2):
            copy_step()
        torch.cuda.synchronize()
        copy_sec = timed(copy_step, max(3, e2e_steps))
        del d_in, d_lse
        for _ in range(2):
            e2e_step()
        sec = timed(e2e_step, e2e_steps)
        bound_ms = max(copy_sec * 1e3, ms_step_local)
        e2e = {"value": f_step_all / sec / 1e12, "unit": "TFLOP/s", "ms_per_step": sec * 1e3,
               "h2d_bytes_per_step": int(4 * nb), "d2h_bytes_per_step": int(4 * nb + nl),
               "steps": e2e_steps, "warmup": 2,
               "copy_ms": copy_sec * 1e3,
               "copy_gbs_each_way": {"h2d": 4 * nb / copy_sec / 1e9, "d2h": (4 * nb + nl) / copy_sec / 1e9,
                                     "all_ranks": world * (8 * nb + nl) / copy_sec / 1e9},
               "device_ms": ms_step_local,
               "frac_of_copy_bound": bound_ms / (sec * 1e3),
               "api": "tt_attn_fwd_bwd_host: pinned host buffers; slice chunks pipelined over upload, compute and download streams"}
        try:
            ev = verify_slice(tt, name, (hq, hk, hv, hdo, ho, hl, hdq, hdk, hdv), S, D, n_local)
            e2e["verified"] = ev
        except Exception as e:  # noqa: BLE001
            e2e["verified"] = {"ok": False, "error": str(e)}
        del hq, hk, hv, hdo, ho, hl, hdq, hdk, hdv
        tt.capi.lib.tt_pool_trim()
    return dict(value=value, ms_per_step=ms_step, scaling="strong" if strong else "weak", kernels=kernels,
                roofline=roofline, fwd_tflops=fwd_tf, e2e=e2e, clocks=clocks, gpu_launches=int(launches),
                n_local=n_local, desc=w["desc"], S=S, D=D, verified=verified,
                pct_of_bf16_peak={"fwd": (fwd_tf / peaks["bf16"] * 100) if fwd_tf else None,
                                  "fwd_bwd": value / world / peaks["bf16"] * 100})


def run_decode(tt, dev, peaks, batch):
    """benchmark configuration 4 (HBM-bound): reported beside the step metric, not part of it."""
    import torch
    capi = tt.capi
    try:
        dB, dH, dL, dD = batch, 32, 8192, 128
        dq_ = torch.randn((dB, dH, 1, dD), device=dev).to(torch.bfloat16)
        dk_ = torch.randn((dB, dH, dL, dD), device=dev).to(torch.bfloat16)
        dv_ = torch.randn((dB, dH, dL, dD), device=dev).to(torch.bfloat16)
        dout_ = torch.empty_like(dq_)
        dws = torch.empty(max(tt.decode_workspace_bytes(dB, dH, dL, dD), 256), dtype=torch.uint8, device=dev)
        for _ in range(3):
            tt.attention_decode(dq_, dk_, dv_, out=dout_, workspace=dws, need_lse=False)
        torch.cuda.synchronize()
        capi.profile_reset(); capi.profile_enable(True)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(20):
            tt.attention_decode(dq_, dk_, dv_, out=dout_, workspace=dws, need_lse=False)
        b.record(); torch.cuda.synchronize()
        capi.profile_enable(False)
        dprof = capi.profile_read()
        ms = a.elapsed_time(b) / 20
        by = 2.0 * dB * dH * dL * dD * 2 + 2.0 * dB * dH * dD * 2
        # head dim 128 runs on the keys-on-rows tensor-core kernel; the split-KV kernel serves the other shapes
        kname = "attn_decode_gq_sm100" if dprof.get("attn_decode_gq_sm100", (0.0, 0))[1] > 0 else "attn_decode"
        kms = dprof[kname][0] / dprof[kname][1]
        # the timed output against the oracle: the last slice (for batch 64 its last element has index
        # 2^31 - 1 and its bytes sit behind 2^32) and one in the middle
        from oracle import attention_oracle as orc
        errs = []
        for b, h in ((dB - 1, dH - 1), (dB // 2, 7)):
            cpu = lambda t: t[b:b + 1, h:h + 1].float().cpu().numpy()
            o_r, _ = orc.attention_forward(cpu(dq_), cpu(dk_), cpu(dv_), False)
            errs.append(orc.max_abs_err(cpu(dout_), o_r))
        verified = {"ok": bool(max(errs) <= 2e-2), "max_abs_err": max(errs),
                    "what": f"slices ({dB - 1},{dH - 1}) and ({dB // 2},7) against the oracle"}
        del dk_, dv_
        return {"workload": f"bf16 decode Q [{dB},32,1,128], K/V [{dB},32,8192,128]", "ms": ms, "gbs": by / ms / 1e6,
                "verified": verified,
                "grouped": run_decode_grouped(tt, dev, peaks, dB),
                "roofline": {"bound": "hbm", "achieved": by / kms / 1e6, "peak": peaks["hbm"], "unit": "GB/s",
                             "frac": by / kms / 1e6 / peaks["hbm"],
                             "traffic": NCU_TRAFFIC_BYTES["decode"].get(kname) if dB == 64 else None,
                             "traffic_note": "ncu capture of the batch-8 launch x 8 (the full launch is too large to capture)",
                             "kernel": kname, "peak_source": f"hbm_gbs of {peaks['source']} MEASURED_PEAKS.json"}}
    except Exception as e:  # noqa: BLE001
        return {"error": str(e)}


def run_decode_grouped(tt, dev, peaks, dB, hkv=8, page=64):
    """The serving form of the decode configuration: 32 query heads over 8 key/value heads (groups
    of 4), cache dense and as a shuffled pool of 64-row pages.  Both run on the keys-on-rows
    tensor-core decode kernel (the paged one gathers its tiles page by page); GB/s counts the K and
    V bytes, which cross HBM once per group."""
    import torch
    try:
        dH, dL, dD = 32, 8192, 128
        q = torch.randn((dB, dH, 1, dD), device=dev).to(torch.bfloat16)
        k = torch.randn((dB, hkv, dL, dD), device=dev).to(torch.bfloat16)
        v = torch.randn((dB, hkv, dL, dD), device=dev).to(torch.bfloat16)
        out = torch.empty_like(q)
        ws = torch.empty(max(tt.decode_workspace_bytes(dB, dH, dL, dD, Hkv=hkv), 256), dtype=torch.uint8, device=dev)
        mp = dL // page
        perm = torch.randperm(dB * mp, device=dev).to(torch.int32).reshape(dB, mp)
        to_pages = lambda t: t.reshape(dB, hkv, mp, page, dD).permute(0, 2, 1, 3, 4).reshape(dB * mp, hkv, page, dD)
        kpool, vpool = torch.empty_like(to_pages(k)), torch.empty_like(to_pages(v))
        kpool[perm.flatten().long()] = to_pages(k)
        vpool[perm.flatten().long()] = to_pages(v)
        lens = torch.full((dB,), dL, dtype=torch.int32, device=dev)
        calls = {"dense": lambda: tt.attention_decode(q, k, v, out=out, workspace=ws, need_lse=False),
                 "paged": lambda: tt.attention_decode_paged(q, kpool, vpool, block_table=perm, seq_lens=lens, out=out,
                                                            workspace=ws, need_lse=False)}
        by = 2.0 * dB * hkv * dL * dD * 2
        res = {"workload": f"Q [{dB},32,1,128], K/V [{dB},{hkv},8192,128], pages of {page} rows"}
        for name, fn in calls.items():
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(20):
                fn()
            b.record(); torch.cuda.synchronize()
            ms = a.elapsed_time(b) / 20
            res[name] = {"ms": ms, "bound": "hbm", "achieved": by / ms / 1e6, "peak": peaks["hbm"], "unit": "GB/s",
                         "frac": by / ms / 1e6 / peaks["hbm"]}
        return res
    except Exception as e:  # noqa: BLE001
        return {"error": str(e)}


def run_varlen(tt, dev, peaks):
    """A packed variable-length batch: 16 sequences of seeded lengths between 300 and 4096 tokens, 32 heads,
    D = 128, causal, token-major [total, H, D].  FLOPs as for the dense workloads, summed over the sequences
    (forward 4*H*S_b^2*D / 2, backward 2.5 x)."""
    import torch
    try:
        H, D = 32, 128
        rng = np.random.default_rng(16)
        lens = [int(x) for x in rng.integers(300, 4097, size=16)]
        total = sum(lens)
        g = torch.Generator(device=dev).manual_seed(16)
        mk = lambda sig: (torch.randn((total, H, D), generator=g, device=dev) * sig).to(torch.bfloat16)
        q, k, v, do = mk(0.5), mk(0.5), mk(0.5), mk(1.0)
        cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device=dev)
        mx = max(lens)
        out, lse = tt.attention_forward_varlen(q, k, v, cu, cu, mx, mx, causal=True)
        fl_f = sum(4.0 * H * n * n * D * 0.5 for n in lens)
        legs = {"fwd": (lambda: tt.attention_forward_varlen(q, k, v, cu, cu, mx, mx, causal=True, out=out, lse=lse), fl_f),
                "bwd": (lambda: tt.attention_backward_varlen(q, k, v, cu, cu, mx, mx, out, lse, do, causal=True), 2.5 * fl_f)}
        res = {"workload": f"bf16 causal, 16 packed sequences of {min(lens)}..{mx} tokens ({total} in all), H={H}, D={D}"}
        for name, (fn, fl) in legs.items():
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(10):
                fn()
            b.record(); torch.cuda.synchronize()
            ms = a.elapsed_time(b) / 10
            res[name] = {"ms": ms, "bound": "tensor", "achieved": fl / ms / 1e9, "peak": peaks["bf16"], "unit": "TFLOP/s",
                         "frac": fl / ms / 1e9 / peaks["bf16"]}
        # one sequence re-checked against the oracle (the last one)
        from oracle import attention_oracle as orc
        lo, hi = int(cu[-2]), int(cu[-1])
        f = lambda t: t[lo:hi, 0].float().cpu().numpy()
        dq, dk, dv = tt.attention_backward_varlen(q, k, v, cu, cu, mx, mx, out, lse, do, causal=True)
        o_r, l_r, dq_r, dk_r, dv_r = orc.attention_backward_chunked(f(q), f(k), f(v), f(do), True)
        errs = {"o": orc.max_abs_err(f(out), o_r), "dq": orc.max_abs_err(f(dq), dq_r), "dk": orc.max_abs_err(f(dk), dk_r),
                "dv": orc.max_abs_err(f(dv), dv_r)}
        ok = errs["o"] <= 2e-2 and all(errs[n] <= orc.bf16_grad_tol(r) for n, r in (("dq", dq_r), ("dk", dk_r), ("dv", dv_r)))
        res["verified"] = {"ok": bool(ok), "max_abs_err": errs, "what": "last sequence, head 0, in full against the oracle"}
        return res
    except Exception as e:  # noqa: BLE001
        return {"error": str(e)}


def run_softmax(tt, dev, peaks, rows=262144):
    """Row softmax forward and backward on a score-matrix sized input (HBM-bound): fp32
    [262144, 1024] = 1 GiB per tensor, far above L2.  Algorithmic bytes: forward reads x and
    writes y (8 B per element), backward reads y, dy and writes dx (12 B per element)."""
    import torch
    capi = tt.capi
    try:
        cols = 1024
        x = torch.randn((rows, cols), device=dev)
        y, dy, dx = torch.empty_like(x), torch.randn((rows, cols), device=dev), torch.empty_like(x)
        for _ in range(3):
            tt.softmax_forward(x, out=y); tt.softmax_backward(y, dy, dx=dx)
        torch.cuda.synchronize()
        capi.profile_reset(); capi.profile_enable(True)
        for _ in range(10):
            tt.softmax_forward(x, out=y); tt.softmax_backward(y, dy, dx=dx)
        torch.cuda.synchronize()
        capi.profile_enable(False)
        prof = capi.profile_read()
        out = {"workload": f"fp32 rows [{rows},{cols}]"}
        for key, nbytes in (("softmax_rows_fwd", 8.0 * rows * cols), ("softmax_rows_bwd", 12.0 * rows * cols)):
            ms = prof[key][0] / prof[key][1]
            out[key] = {"ms": ms, "bound": "hbm", "achieved": nbytes / ms / 1e6, "peak": peaks["hbm"], "unit": "GB/s",
                        "frac": nbytes / ms / 1e6 / peaks["hbm"]}
        return out
    except Exception as e:  # noqa: BLE001
        return {"error": str(e)}


def run_fc(tt, dev, peaks, M=16384):
    """The projection either side of attention at config 3's size: x [B*S = 16384, H*D = 4096] bf16
    times w [4096, 4096] (+ bias), forward and the two backward products, each 2*M*K*N flops on the
    tcgen05 GEMM kernel.  Operands (134 MB + 34 MB + 134 MB) exceed L2."""
    import torch
    capi = tt.capi
    try:
        K, N = 4096, 4096
        x = torch.randn((M, K), device=dev).to(torch.bfloat16)
        w = (torch.randn((K, N), device=dev) / 64).to(torch.bfloat16)
        b = torch.randn((N,), device=dev).to(torch.bfloat16)
        dy = torch.randn((M, N), device=dev).to(torch.bfloat16)
        y = torch.empty((M, N), device=dev, dtype=torch.bfloat16)
        legs = {"fwd": lambda: tt.fc_forward(x, w, b, out=y),
                "dx": lambda: tt.fc_backward(x, w, dy, need_dw=False, need_db=False),
                "dw": lambda: tt.fc_backward(x, w, dy, need_dx=False, need_db=False)}
        out = {"workload": f"bf16 x [{M},{K}] . w [{K},{N}] + bias"}
        fl = 2.0 * M * K * N
        for name, fn in legs.items():
            for _ in range(3):
                fn()
            torch.cuda.synchronize()
            capi.profile_reset(); capi.profile_enable(True)
            for _ in range(10):
                fn()
            torch.cuda.synchronize()
            capi.profile_enable(False)
            ms_total, n = capi.profile_read()["fc_gemm_sm100"]
            ms = ms_total / n
            out[name] = {"ms": ms, "bound": "tensor", "achieved": fl / ms / 1e9, "peak": peaks["bf16"],
                         "unit": "TFLOP/s", "frac": fl / ms / 1e9 / peaks["bf16"]}
        return out
    except Exception as e:  # noqa: BLE001
        return {"error": str(e)}


def run_fp32(tt, dev, peaks):
    """The reference's own dtype: fp32 causal forward+backward on the SIMT kernels (true fp32 FMAs;
    the 1e-5 tolerance rules out the tensor-core formats), Q/K/V [2,8,2048,64].  Reported beside
    the bf16 step so that the cost of staying in fp32 is visible; not part of the step metric."""
    import torch
    try:
        B, H, S, D = 2, 8, 2048, 64
        q, k, v, do = (torch.randn((B, H, S, D), device=dev) * 0.5 for _ in range(4))
        o, lse = tt.attention_forward(q, k, v, causal=True)
        fl_f = 4.0 * B * H * S * S * D / 2
        res = {"workload": f"fp32 causal fwd+bwd, Q/K/V [{B},{H},{S},{D}]"}
        legs = {"fwd": (lambda: tt.attention_forward(q, k, v, causal=True), fl_f),
                "bwd": (lambda: tt.attention_backward(q, k, v, o, lse, do, causal=True), 2.5 * fl_f)}
        for name, (fn, fl) in legs.items():
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(5):
                fn()
            b.record(); torch.cuda.synchronize()
            ms = a.elapsed_time(b) / 5
            res[name] = {"ms": ms, "tflops": fl / ms / 1e9}
        return res
    except Exception as e:  # noqa: BLE001
        return {"error": str(e)}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cfg5", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--only", choices=["softmax", "fc", "decode"], help="run just this side leg and print its block "
                    "(used for profiler captures of that kernel; not the benchmark line)")
    ap.add_argument("--fc-rows", type=int, default=16384, help="rows of x in the fully connected leg")
    ap.add_argument("--softmax-rows", type=int, default=262144, help="rows of the row-softmax leg")
    ap.add_argument("--no-fc", action="store_true", help="skip the fully connected layer leg at N=1")
    ap.add_argument("--no-softmax", action="store_true", help="skip the row-softmax leg at N=1")
    ap.add_argument("--no-fp32", action="store_true", help="skip the fp32 (SIMT kernels) side measurement at N=1")
    ap.add_argument("--no-varlen", action="store_true", help="skip the packed variable-length side measurement at N=1")
    ap.add_argument("--no-cfg3", action="store_true", help="skip the S=4096 side measurement at N=1")
    ap.add_argument("--no-cfg2", action="store_true", help="skip the S=1024, D=64 side measurement at N=1")
    ap.add_argument("--heads", type=int, default=0, help="override the head count of the main workload (small profiler "
                    "captures of the same slice shape; the line is then not the benchmark line)")
    ap.add_argument("--e2e-steps", type=int, default=5)
    ap.add_argument("--no-verify", action="store_true", help="skip the oracle re-check of the timed outputs")
    ap.add_argument("--decode-batch", type=int, default=64, help="batch of the decode leg (64 = benchmark configuration 4)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.heads > 0:
        WORKLOADS[args.workload] = dict(WORKLOADS[args.workload], H=args.heads,
                                        desc=WORKLOADS[args.workload]["desc"] + f" (heads overridden: {args.heads})")
    w = WORKLOADS[args.workload]
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))

    if args.impl == "reference":
        run_reference_arm(args, w, rank)
        return

    import torch
    import torch.distributed as dist
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the attention kernels have no CPU implementation")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
    tt = importlib.import_module("pku-aiprogramming_b200")
    peaks = load_peaks()

    if args.only:
        if rank == 0:
            res = (run_fc(tt, dev, peaks, args.fc_rows) if args.only == "fc" else
                   run_decode(tt, dev, peaks, args.decode_batch) if args.only == "decode" else
                   run_softmax(tt, dev, peaks, args.softmax_rows))
            print(json.dumps({"leg": args.only, "result": res}), flush=True)
        return

    # pinned host buffers of the end-to-end leg should sit in the memory next to this rank's GPU
    numa_cores = gpu_numa_affinity(local_rank) if args.e2e_steps > 0 else None
    sharded = None
    if world > 1:
        sharder = importlib.import_module("pku-aiprogramming_b200.sharder")
        sharded = sharder.ShardedAttention.from_process_group(device=dev)

    def side_block(wname, n_steps, n_warm):
        r = run_workload(tt, wname, n_steps, n_warm, 1, 0, dev, peaks, 0, sample_clocks=False, verify=not args.no_verify)
        return {"workload": r["desc"], "fwd_bwd_tflops": r["value"], "ms_per_step": r["ms_per_step"],
                "fwd_tflops": r["fwd_tflops"], "pct_of_bf16_peak": r["pct_of_bf16_peak"], "kernels": r["kernels"],
                "verified": r["verified"]}

    side = side2 = None
    if rank == 0 and world == 1 and args.workload != "cfg2" and not args.no_cfg2:
        side2 = side_block("cfg2", 50, 10)
    if rank == 0 and world == 1 and args.workload != "cfg3" and not args.no_cfg3:
        # the S=4096/D=128 shape the forward target (>= 60 % of bf16 peak) is stated on.  It runs BEFORE
        # the main workload: that one drives the GPU into its power cap for seconds, and a 50 ms
        # measurement taken right behind it inherits the lowered clock (its peak, the burst figure of
        # MEASURED_PEAKS.json, was taken on an idle GPU)
        side = side_block("cfg3", 20, 5)
    main_res = run_workload(tt, args.workload, args.steps, args.warmup, world, rank, dev, peaks, args.e2e_steps,
                            sample_clocks=(rank == 0), sharded=sharded, verify=not args.no_verify)
    if world > 1:
        import torch
        okt = torch.tensor([1 if (main_res["verified"] or {}).get("ok", True) else 0], device=dev)
        dist.all_reduce(okt, op=dist.ReduceOp.MIN)
        if main_res["verified"] is not None:
            main_res["verified"]["ok_on_every_rank"] = bool(okt.item())
    decode = run_decode(tt, dev, peaks, args.decode_batch) if (rank == 0 and not args.no_decode) else None

    fc = run_fc(tt, dev, peaks, args.fc_rows) if (rank == 0 and world == 1 and not args.no_fc) else None
    softmax = run_softmax(tt, dev, peaks, args.softmax_rows) if (rank == 0 and world == 1 and not args.no_softmax) else None
    fp32 = run_fp32(tt, dev, peaks) if (rank == 0 and world == 1 and not args.no_fp32) else None
    varlen = run_varlen(tt, dev, peaks) if (rank == 0 and world == 1 and not args.no_varlen) else None

    # CPU baseline: the oracle on a bounded sample of the same workload (rank 0, N = 1)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        S, D = main_res["S"], main_res["D"]
        S_cpu = min(S, 4096)
        t1 = cpu_sample_seconds(S_cpu, D, 7)
        n = int(min(16, max(2, round(12.0 / max(t1, 1e-3)))))
        ts = [cpu_sample_seconds(S_cpu, D, 8 + i) for i in range(n)]
        fl = 3.5 * fwd_flops(1, 1, S_cpu, S_cpu, D, True)
        what = "whole (batch,head) slices" if S_cpu == S else f"the S=L={S_cpu} prefix of (batch,head) slices"
        cpu = {"value": fl / float(np.mean(ts)) / 1e12, "unit": "TFLOP/s", "cores": cpu_threads(), "kind": "port",
               "sample": f"{n} samples of {what}, causal fwd+bwd, D={D}, fp32 NumPy oracle, "
                         f"{float(np.mean(ts)):.2f} s per sample"}

    if rank == 0:
        line = {
            "metric": "attention fwd+bwd TFLOP/s", "value": main_res["value"], "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": main_res["ms_per_step"], "higher_is_better": True,
            "scaling": main_res["scaling"], "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": main_res["desc"], "causal": True,
                       "flop_count": "2/MAC, fwd 2 GEMMs, bwd 5 GEMMs, causal = half",
                       "l2": "inputs per step (>= 0.5 GB) exceed the 126 MB L2",
                       "collective": ("tt_mgpu_attn_fwd: ncclAllGather of O issued by the library on its own side "
                                      "stream, overlapped with the backward (tt_mgpu_attn_bwd), joined by tt_mgpu_wait")
                                     if (world > 1 and main_res["scaling"] == "strong") else "none",
                       "parallelism": f"{world} x contiguous (batch,head) shards"},
            "fwd_tflops": main_res["fwd_tflops"], "pct_of_bf16_peak": main_res["pct_of_bf16_peak"],
            "roofline": main_res["roofline"], "kernels": main_res["kernels"], "verified": main_res["verified"],
            "cfg3": side, "cfg2": side2, "decode": decode,
            "softmax_rows": softmax, "fc": fc, "fp32": fp32, "varlen": varlen,
            "cpu_baseline": cpu, "e2e": main_res["e2e"], "clocks": main_res["clocks"],
            "gpu_launches": main_res["gpu_launches"], "host_numa_cores": numa_cores,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()                      # every rank is between steps, nothing of ours is in flight
        sharded.close()
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
