#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

One "step" is one pass of the hot path over one synthetic batch:
  * headline workload (N=1): GQA causal prefill in bf16 -- B=4, Hq=32, Hkv=8, S=2048,
    head_dim 128, RoPE theta 1e4 applied to Q and K, K/V appended into an empty cache of
    capacity 4096 -- one call of vb200_prefill_fwd.  metric = attention TFLOP/s,
    FLOPs = 4*B*Hq*D*S*(S+1)/2 (QK^T and PV over the causal triangle only).
  * also reported in the same line: batched GQA decode (B=32, Hq=32, Hkv=8, D=128, ragged
    contexts U[1024,8192], 256 consecutive steps) as KV-read GB/s, and -- at N>1 -- the
    sequence-sharded long-context decode (131072 keys split over the GPUs, one all-gather);
    "model": the 24-layer Llama-style decoder around the path (8 prompts x 512 ids, prefill +
    128 greedy tokens through the host layer's Generator) as tokens/s with the attention time share.
  * N>1: prefill and batched decode partition by (batch x kv_head) with no collective, so
    every rank runs the same per-GPU workload on its own units (weak scaling).

Timing: CUDA events on the launching stream; each timed step has its own event pair and
L2 is flushed (256 MiB write) between steps; max over ranks.  A clock/throttle record is
sampled with nvidia-smi during the timed region.

--impl reference times the reference's own CPU attention (oracle/_ref when it was built,
else the plain-C port) on a bounded sample of the same workload, on all host cores.
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

# headline workload (the configuration the metric is quoted on)
C2 = dict(B=4, Hq=32, Hkv=8, S=2048, D=128, cap=4096, theta=10000.0)
C3 = dict(B=32, Hq=32, Hkv=8, D=128, lo=1024, hi=8192, steps=256)
C4 = dict(B=1, Hq=64, Hkv=8, D=128, L=131072)
C5 = dict(vocab=32000, dim=2048, layers=24, Hq=16, Hkv=4, ffn=5632, B=8, P=512, new=128)


def prefill_flops(c):
    return 4.0 * c["B"] * c["Hq"] * c["D"] * c["S"] * (c["S"] + 1) / 2.0


def load_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm=float(d["hbm_gbs"]), tf=float(d["bf16_tflops"]), tf_sustained=float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), source="measured")
    return dict(hbm=6650.0, tf=1590.0, tf_sustained=1400.0, source="fallback")


def load_traffic():
    """DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernels,
    copied from the ncu captures summarised in profiles/prefill_sm100_c2.md and
    profiles/decode_gqa_mma_c3.md (captured on exactly these workloads, so no scaling applies)."""
    return {"prefill_sm100_bytes_per_launch": 138.3e6, "decode_splitkv_bytes_per_launch": 705.5e6}


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.idx, self.proc, self.lines = gpu_index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.idx}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        self.thread.join(timeout=2)
        mhz, mx, reasons = [], None, set()
        for ts, line in self.lines:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 9 or not (t0 - 0.05 <= ts <= t1 + 0.15):
                continue
            try:
                mhz.append(float(f[1])); mx = float(f[2])
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        mhz.sort()
        return {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": len(mhz)}


# ----------------------------------------------------------------------------------------------
# CPU arm: the reference's own CPU attention on a bounded sample, all host threads
# ----------------------------------------------------------------------------------------------
def cpu_prefill_sample(target_seconds=12.0, threads=None, S=None, total_slices=None, what="the headline prefill"):
    """Time flash_attention_cpu_dispatch (src/ops/flash_attention.cpp:218-364) on (batch, head)
    slices of the headline workload (S=2048, D=128, causal; RoPE applied to the slice first with
    the reference's functions), independent slices on `threads` host threads.  Returns TFLOP/s."""
    import numpy as np
    from oracle.binding import Oracle, Ref, ref_available
    kind = "reference" if ref_available() else "port"
    eng = Ref() if kind == "reference" else Oracle()
    threads = threads or max(1, min(os.cpu_count() or 1, 64))
    S, D = S or C2["S"], C2["D"]
    total_slices = total_slices or C2["B"] * C2["Hq"]
    scale = float(1.0 / np.sqrt(D))

    def make_slice(seed):
        rng = np.random.default_rng(seed)
        return tuple((0.5 * rng.standard_normal((1, 1, S, D))).astype(np.float32) for _ in range(3))

    def one_slice(qkv):
        q, k, v = qkv
        qr = eng.apply_rope(q, 0, C2["theta"])
        kr = eng.apply_rope(k, 0, C2["theta"])
        eng.flash_attention(qr, kr, v, scale, True)

    t0 = time.time(); one_slice(make_slice(1)); t_one = time.time() - t0          # calibrate (single thread)
    per_thread = max(1, int(target_seconds / max(t_one, 1e-3)))
    per_thread = min(per_thread, 64)
    done = [0] * threads
    data = [make_slice(1 + i) for i in range(threads)]            # one distinct (batch, head) slice per thread

    def work(i):
        for _ in range(per_thread):
            one_slice(data[i])
            done[i] += 1

    ths = [threading.Thread(target=work, args=(i,)) for i in range(threads)]
    t0 = time.time()
    for t in ths: t.start()
    for t in ths: t.join()
    dt = time.time() - t0
    slices = sum(done)
    flops = slices * 4.0 * D * S * (S + 1) / 2.0
    # the reference's attention code is single-threaded: one core's rate is its own figure, `value` the all-threads one
    one_core = (4.0 * D * S * (S + 1) / 2.0) / max(t_one, 1e-9) / 1e12
    return dict(value=flops / dt / 1e12, unit="TFLOP/s", cores=threads, kind=kind, value_one_core=one_core,
                sample=f"{slices} slice passes = {threads} distinct seeded (batch, head) slices of {what} (one per host thread; the workload has "
                       f"{total_slices}) x {per_thread} repeats each (S={S}, D={D}, fp32, RoPE + causal flash), {dt:.1f} s; "
                       f"single-thread slice {t_one * 1e3:.0f} ms"), dt


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cb, dt = cpu_prefill_sample(target_seconds=10.0)
    steps = max(1, args.steps)
    line = {
        "impl": "reference", "metric": "prefill attn TFLOP/s & decode KV-read GB/s vs B200 roofline",
        "value": cb["value"], "unit": "TFLOP/s", "n_gpus": args.gpus, "steps": steps, "warmup": args.warmup,
        "ms_per_step": dt * 1e3 / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": "GQA causal prefill B=4 Hq=32 Hkv=8 S=2048 D=128, RoPE theta 1e4 (reference CPU code, bounded sample)"},
        "cpu_baseline": cb,
        "e2e": {"value": cb["value"], "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(line)


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
class Ctx:
    """Per-process state of the GPU arm: device, ranks, helpers."""

    def __init__(self):
        import torch
        import torch.distributed as dist
        from vesper_b200 import capi
        self.torch, self.dist, self.capi = torch, dist, capi
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.rank = int(os.environ.get("RANK", "0"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if not torch.cuda.is_available():
            raise RuntimeError("bench.py needs a CUDA device; there is no CPU fallback (use --impl reference for the CPU arm)")
        torch.cuda.set_device(self.local)
        self.dev = torch.device("cuda", self.local)
        self.L = capi.load()
        if self.world > 1:
            dist.init_process_group("nccl", device_id=self.dev)
        self.peaks = load_peaks()
        self.traffic = load_traffic()
        self.flush_buf = torch.empty(256 << 20, dtype=torch.uint8, device=self.dev)

    def flush_l2(self):
        self.flush_buf.fill_(1)

    def sync_all(self):
        self.torch.cuda.synchronize()
        if self.world > 1:
            self.dist.barrier()
            self.torch.cuda.synchronize()

    def max_over_ranks(self, x):
        if self.world == 1:
            return x
        t = self.torch.tensor([x], dtype=self.torch.float64, device=self.dev)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def event(self):
        return self.torch.cuda.Event(enable_timing=True)


def bind_to_gpu_numa_node(torch, local):
    """Pin this process (and so the pages its pinned buffers are first touched on, and its copy threads) to the CPUs of
    the NUMA node the GPU hangs off, read from sysfs.  Returns what was done, for the JSON line."""
    info = {"numa_node": None, "cpus": None}
    try:
        try:
            props = torch.cuda.get_device_properties(local)
            bdf = f"{props.pci_domain_id:04x}:{props.pci_bus_id:02x}:{props.pci_device_id:02x}.0"
        except AttributeError:
            out = subprocess.run(["nvidia-smi", f"--id={local}", "--query-gpu=pci.bus_id", "--format=csv,noheader"],
                                 capture_output=True, text=True, timeout=20).stdout.strip().lower()
            bdf = out[-12:]                                      # "00000000:1b:00.0" -> "0000:1b:00.0"
        node = int(open(f"/sys/bus/pci/devices/{bdf}/numa_node").read().strip())
        info["numa_node"] = node
        if node < 0:
            return info
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
            info["cpus"] = len(cpus)
    except (OSError, ValueError, subprocess.SubprocessError):
        pass
    return info


def bench_prefill(cx, K, W, quick=False):
    """Headline: C2 prefill.  Returns the fields of the JSON line that come from it."""
    import ctypes as C
    import numpy as np
    torch, capi, L, dev = cx.torch, cx.capi, cx.L, cx.dev
    c = C2
    B, Hq, Hkv, S, D = c["B"], c["Hq"], c["Hkv"], c["S"], c["D"]
    placement = bind_to_gpu_numa_node(torch, cx.local)          # before the pinned host buffers are allocated
    g = torch.Generator(device="cpu").manual_seed(1 + cx.rank)
    hq = (0.5 * torch.randn(B, Hq, S, D, generator=g)).to(torch.bfloat16).pin_memory()
    hk = (0.5 * torch.randn(B, Hkv, S, D, generator=g)).to(torch.bfloat16).pin_memory()
    hv = (0.5 * torch.randn(B, Hkv, S, D, generator=g)).to(torch.bfloat16).pin_memory()
    ho = torch.empty(B, Hq, S, D, dtype=torch.bfloat16).pin_memory()
    hl = torch.empty(B, Hq, S, dtype=torch.float32).pin_memory()
    q, k, v = hq.to(dev), hk.to(dev), hv.to(dev)
    o = torch.empty_like(q)
    lse = torch.empty(B, Hq, S, dtype=torch.float32, device=dev)
    kc = torch.zeros(B, Hkv, c["cap"], D, dtype=torch.bfloat16, device=dev)
    vc = torch.zeros_like(kc)
    scale = float(1.0 / np.sqrt(D))
    a = capi.prefill_args(q, k, v, o, lse, scale=scale, causal=True, theta=c["theta"], k_cache=kc, v_cache=vc)
    ws = torch.empty(max(256, L.vb200_prefill_workspace_bytes(C.byref(a))), dtype=torch.uint8, device=dev)
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()

    def step():
        capi.check(L.vb200_prefill_fwd(C.byref(a)))

    for _ in range(W):
        step()
    cx.sync_all()
    sampler = ClockSampler(cx.local)
    sampler.start()
    time.sleep(0.3)
    L.vb200_reset_launch_count()
    evs = [(cx.event(), cx.event()) for _ in range(K)]
    cx.sync_all()
    t0 = time.time()
    for i in range(K):
        cx.flush_l2()
        evs[i][0].record()
        step()
        evs[i][1].record()
    cx.sync_all()
    t1 = time.time()
    launches = int(L.vb200_launch_count())
    total_ms = cx.max_over_ranks(sum(s.elapsed_time(e) for s, e in evs))
    ms_per_step = total_ms / K
    # the dominant kernel's own duration: a separate pass, because the event brackets inside the
    # library make consecutive calls wait for each other
    capi.profile_enable(True)
    for _ in range(min(K, 10)):
        cx.flush_l2()
        step()
    torch.cuda.synchronize()
    kern_ms, kern_n = capi.profile_read()
    capi.profile_enable(False)
    # the timed region lasts only milliseconds: keep the same step running a little longer so
    # the 100 ms clock sampler sees this load (skipped in profiling runs)
    if not quick:
        t_busy = time.time()
        while time.time() - t_busy < 0.6:
            step()
        torch.cuda.synchronize()
        t1 = time.time()
    clocks = sampler.stop(t0, t1)
    flops = prefill_flops(c)
    kern_avg_ms = kern_ms / max(1, kern_n)
    achieved = flops / (kern_avg_ms * 1e-3) / 1e12

    # end to end through the C ABI with host buffers: H2D of q,k,v and D2H of O,LSE every step.
    # (a) serial on one stream; (b) the batch cut into its B sequences and pipelined over three streams
    # (copy in / compute / copy out), which is what a caller with host-resident tensors would do: PCIe is
    # full duplex, so the step then costs about max(bytes in, bytes out) / link rate instead of their sum.
    def e2e_step():
        q.copy_(hq, non_blocking=True); k.copy_(hk, non_blocking=True); v.copy_(hv, non_blocking=True)
        step()
        ho.copy_(o, non_blocking=True); hl.copy_(lse, non_blocking=True)

    fence = [True]            # the pipelined form orders its copy-in stream after the main stream once per batch of steps

    def timed_e2e(fn):
        for _ in range(2):
            fn()
        cx.sync_all()
        e0, e1 = cx.event(), cx.event()
        Ke = min(K, 10)
        e0.record()
        fence[0] = True
        for _ in range(Ke):
            fn()
        e1.record()
        cx.sync_all()
        return cx.max_over_ranks(e0.elapsed_time(e1)) / Ke

    e2e_serial_ms = timed_e2e(e2e_step)

    s_in, s_cmp, s_out = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()
    main = torch.cuda.current_stream()
    # One sequence per slice.  A slice's q, k, v sit back to back in ONE pinned host buffer and one device buffer (what a
    # caller that owns its host tensors would arrange), O and LSE likewise: one copy in and one copy out per slice
    # instead of five (each copy call costs ~10 us of engine turnaround, 20 of them per step were 0.1-0.2 ms).
    nq, nk, nl = Hq * S * D * 2, Hkv * S * D * 2, Hq * S * 4                   # bytes of q / k (= v) / lse of one sequence
    slices = []
    for i in range(B):
        h_in = torch.empty(nq + 2 * nk, dtype=torch.uint8).pin_memory()
        h_in[:nq].view(torch.bfloat16).copy_(hq[i].reshape(-1))
        h_in[nq:nq + nk].view(torch.bfloat16).copy_(hk[i].reshape(-1))
        h_in[nq + nk:].view(torch.bfloat16).copy_(hv[i].reshape(-1))
        d_in = torch.empty(nq + 2 * nk, dtype=torch.uint8, device=dev)
        d_out = torch.empty(nq + nl, dtype=torch.uint8, device=dev)
        h_out = torch.empty(nq + nl, dtype=torch.uint8).pin_memory()
        qi = d_in[:nq].view(torch.bfloat16).view(1, Hq, S, D)
        ki = d_in[nq:nq + nk].view(torch.bfloat16).view(1, Hkv, S, D)
        vi = d_in[nq + nk:].view(torch.bfloat16).view(1, Hkv, S, D)
        oi = d_out[:nq].view(torch.bfloat16).view(1, Hq, S, D)
        li = d_out[nq:].view(torch.float32).view(1, Hq, S)
        ai = capi.prefill_args(qi, ki, vi, oi, li, scale=scale, causal=True, theta=c["theta"], k_cache=kc[i:i + 1], v_cache=vc[i:i + 1],
                               stream=s_cmp)
        wsi = torch.empty(max(256, L.vb200_prefill_workspace_bytes(C.byref(ai))), dtype=torch.uint8, device=dev)
        ai.workspace, ai.workspace_bytes = wsi.data_ptr(), wsi.numel()
        slices.append(dict(args=ai, ws=wsi, h_in=h_in, d_in=d_in, d_out=d_out, h_out=h_out, o=oi,
                           ev_in=torch.cuda.Event(), ev_cmp=torch.cuda.Event(), ev_out=torch.cuda.Event()))
    first = [True]

    def e2e_pipelined():
        # Consecutive steps overlap as well: step i+1's copies in run while step i's last results leave (each slice's
        # device buffers are guarded by the events below), so in steady state a step costs the larger of its bytes in
        # and bytes out at the full-duplex link rate.  Only the first step of a batch waits for the main stream (the
        # timing event recorded there).
        if fence[0]:
            start = torch.cuda.Event()
            start.record(main)
            s_in.wait_event(start)
            fence[0] = False
        for sl in slices:
            with torch.cuda.stream(s_in):
                if not first[0]:
                    s_in.wait_event(sl["ev_cmp"])                # the previous step's kernel has read this slice
                sl["d_in"].copy_(sl["h_in"], non_blocking=True)
                sl["ev_in"].record(s_in)
            with torch.cuda.stream(s_cmp):
                s_cmp.wait_event(sl["ev_in"])
                if not first[0]:
                    s_cmp.wait_event(sl["ev_out"])               # the previous step's result of this slice has left
                capi.check(L.vb200_prefill_fwd(C.byref(sl["args"])))
                sl["ev_cmp"].record(s_cmp)
            with torch.cuda.stream(s_out):
                s_out.wait_event(sl["ev_cmp"])
                sl["h_out"].copy_(sl["d_out"], non_blocking=True)
                sl["ev_out"].record(s_out)
        first[0] = False
        main.wait_event(slices[-1]["ev_out"])

    e2e_ms = timed_e2e(e2e_pipelined)
    torch.cuda.synchronize()
    e2e_ok = bool(torch.equal(slices[-1]["h_out"][:nq].view(torch.bfloat16), slices[-1]["o"].reshape(-1).cpu())) and \
        bool(torch.equal(slices[-1]["o"].reshape(-1).cpu(), o[B - 1].reshape(-1).cpu()))
    capi.check_kernel_status(cx.local)
    pk = cx.peaks
    return {
        "value": cx.world * flops / (ms_per_step * 1e-3) / 1e12, "ms_per_step": ms_per_step, "gpu_launches": launches,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": pk["tf"], "unit": "TFLOP/s", "frac": achieved / pk["tf"],
                     "peak_source": pk["source"] + " (burst cuBLAS bf16)", "frac_of_sustained": achieved / pk["tf_sustained"],
                     "frac_of_nominal_2250": achieved / 2250.0, "kernel": L.vb200_last_prefill_kernel().decode(), "kernel_ms": kern_avg_ms,
                     "traffic": cx.traffic.get("prefill_sm100_bytes_per_launch")},
        "e2e": {"value": cx.world * flops / (e2e_ms * 1e-3) / 1e12, "unit": "TFLOP/s", "value_per_gpu": flops / (e2e_ms * 1e-3) / 1e12,
                "host_placement": placement,
                "h2d_bytes_per_step": (hq.numel() + hk.numel() + hv.numel()) * 2, "d2h_bytes_per_step": ho.numel() * 2 + hl.numel() * 4,
                "ms_per_step": e2e_ms, "how": f"the batch as {len(slices)} sequence slices (q, k, v of a slice in one pinned buffer, O and LSE in another: one copy each way per slice) pipelined over copy-in / compute / copy-out streams, consecutive steps overlapping (every step's copies inside the timed region)",
                "ms_per_step_serial_single_stream": e2e_serial_ms, "result_copied_back_matches_device": e2e_ok},
        "clocks": clocks,
    }


def bench_decode(cx, nsteps, W):
    """C3: batched ragged GQA decode, `nsteps` consecutive steps each appending one token."""
    import ctypes as C
    import numpy as np
    torch, capi, L, dev = cx.torch, cx.capi, cx.L, cx.dev
    d = C3
    B, Hq, Hkv, D = d["B"], d["Hq"], d["Hkv"], d["D"]
    rs = np.random.RandomState(2)
    lens0 = rs.randint(d["lo"], d["hi"] + 1, size=B).astype(np.int32)
    nprof = min(32, nsteps)
    cap = d["hi"] + nsteps + nprof + W + 8
    gd = torch.Generator(device=dev).manual_seed(3 + cx.rank)
    kc = torch.randn(B, Hkv, cap, D, generator=gd, device=dev, dtype=torch.bfloat16)
    vc = torch.randn(B, Hkv, cap, D, generator=gd, device=dev, dtype=torch.bfloat16)
    q1 = torch.randn(B, Hq, 1, D, generator=gd, device=dev, dtype=torch.bfloat16)
    k1 = torch.randn(B, Hkv, 1, D, generator=gd, device=dev, dtype=torch.bfloat16)
    v1 = torch.randn(B, Hkv, 1, D, generator=gd, device=dev, dtype=torch.bfloat16)
    o1 = torch.empty_like(q1)
    seq = torch.from_numpy(lens0).to(dev)
    scale = float(1.0 / np.sqrt(D))
    da = capi.decode_args(q1, o1, kc, vc, scale=scale, k_new=k1, v_new=v1, theta=10000.0, seq_lens=seq,
                          advance_lens=True, max_len=int(lens0.max()) + nsteps + nprof + W + 1)
    dws = torch.empty(L.vb200_decode_workspace_bytes(C.byref(da)), dtype=torch.uint8, device=dev)
    da.workspace, da.workspace_bytes = dws.data_ptr(), dws.numel()

    def step():
        capi.check(L.vb200_decode_fwd(C.byref(da)))

    for _ in range(W):
        step()
    cx.sync_all()
    lens_start = lens0.astype(np.int64) + W
    L.vb200_reset_launch_count()
    d0, d1 = cx.event(), cx.event()
    d0.record()
    for _ in range(nsteps):
        step()
    d1.record()
    cx.sync_all()
    launches = int(L.vb200_launch_count())
    dec_ms = cx.max_over_ranks(d0.elapsed_time(d1))
    # K and V rows read once per KV head, including the token appended in the step
    step_bytes = lambda t: float(np.sum(2 * Hkv * (lens_start + t + 1) * D * 2))
    dec_bytes = sum(step_bytes(t) for t in range(nsteps))
    capi.profile_enable(True)          # kernel-only pass over the next nprof steps
    for _ in range(nprof):
        step()
    torch.cuda.synchronize()
    kern_ms, _ = capi.profile_read()
    capi.profile_enable(False)
    prof_bytes = sum(step_bytes(t) for t in range(nsteps, nsteps + nprof))
    kgbs = prof_bytes / (kern_ms * 1e-3) / 1e9 if kern_ms > 0 else None
    capi.check_kernel_status(cx.local)
    assert seq.cpu().numpy().tolist() == (lens0 + W + nsteps + nprof).tolist()
    pk = cx.peaks
    return {
        "metric": "decode KV-read GB/s", "value": cx.world * dec_bytes / (dec_ms * 1e-3) / 1e9, "unit": "GB/s",
        "ms_per_step": dec_ms / nsteps, "steps": nsteps,
        "config": {"workload": f"batched GQA decode B={B} Hq={Hq} Hkv={Hkv} D={D} bf16 cache, ragged contexts U[{d['lo']},{d['hi']}] (seed 2), "
                               f"{nsteps} consecutive steps each appending one token (RoPE + append fused); inputs larger than L2 "
                               f"({dec_bytes / nsteps / 1e6:.0f} MB of K/V per step)"},
        "gpu_launches": launches,
        "roofline": {"bound": "hbm", "achieved": kgbs, "peak": pk["hbm"], "unit": "GB/s", "frac": (kgbs / pk["hbm"]) if kgbs else None,
                     "peak_source": pk["source"], "frac_of_nominal_8TBs": (kgbs / 8000.0) if kgbs else None,
                     "kernel": "decode_gqa_mma_kernel", "kernel_ms": kern_ms / max(1, nprof),
                     "step_achieved": dec_bytes / (dec_ms * 1e-3) / 1e9, "step_frac": dec_bytes / (dec_ms * 1e-3) / 1e9 / pk["hbm"],
                     "step_frac_of_nominal_8TBs": dec_bytes / (dec_ms * 1e-3) / 1e9 / 8000.0,
                     "traffic": cx.traffic.get("decode_splitkv_bytes_per_launch")},
    }


def bench_sharded(cx, nsteps=50):
    """C4: long-context decode with the KV sequence sharded over the ranks.  At N>1 the partial records are
    exchanged and merged by the fused peer-memory kernel (vb200_exchange_combine); the all-gather + combine
    path is timed beside it."""
    import numpy as np
    from vesper_b200.sharded import PeerExchange, ShardedDecodeStep, cuda_step, shard_range
    torch, capi, dev, world = cx.torch, cx.capi, cx.dev, cx.world
    s4 = C4
    Bq, Hq, Hkv, D, L4 = s4["B"], s4["Hq"], s4["Hkv"], s4["D"], s4["L"]
    begin, end = shard_range(L4, world, cx.rank)
    g4 = torch.Generator(device=dev).manual_seed(5)
    ks = torch.randn(Bq, Hkv, end - begin, D, generator=g4, device=dev, dtype=torch.bfloat16)
    vs = torch.randn(Bq, Hkv, end - begin, D, generator=g4, device=dev, dtype=torch.bfloat16)
    q4 = torch.randn(Bq, Hq, 1, D, generator=torch.Generator(device=dev).manual_seed(6), device=dev, dtype=torch.bfloat16)
    part = torch.empty(Bq * Hq, D + 2, dtype=torch.float32, device=dev)
    gath = torch.empty(world, Bq * Hq, D + 2, dtype=torch.float32, device=dev)
    out4 = torch.empty(Bq * Hq, D, dtype=torch.bfloat16, device=dev)
    qpos = torch.full((Bq,), L4, dtype=torch.int32, device=dev)
    step4 = ShardedDecodeStep(world, cx.rank, L4)
    ws4 = torch.empty(64 << 20, dtype=torch.uint8, device=dev)
    scale = float(1.0 / np.sqrt(D))
    dist = cx.dist if world > 1 else None
    exchange, exchange_error = None, None
    if world > 1:
        try:
            exchange = PeerExchange(cx.dist, world, cx.rank, Bq * Hq, D, dev)
        except Exception as e:                      # peer memory could not be mapped: the all-gather path still runs
            exchange_error = f"{type(e).__name__}: {e}"[:200]

    def step_gather():
        cuda_step(step4, q4, ks, vs, scale=scale, theta=10000.0, partial_buf=part, out=out4, gathered=gath, workspace=ws4, dist=dist, qpos=qpos)

    def step_fused():
        cuda_step(step4, q4, ks, vs, scale=scale, theta=10000.0, partial_buf=part, out=out4, workspace=ws4, exchange=exchange, qpos=qpos)

    def step_local_only():
        # this rank's shard alone (split kernel + combine into a partial record, nothing exchanged): what is left of a
        # step's time is the exchange's share
        capi.decode(q4, None, ks, vs, scale=scale, theta=10000.0, uniform_len=end - begin, max_len=end - begin, pos_offset=begin,
                    q_positions=qpos, partial_out=part, workspace=ws4)

    one_launch_ok = exchange is not None and exchange.supports_one_launch(Bq, Hq, Hkv)

    def step_one_launch():
        cuda_step(step4, q4, ks, vs, scale=scale, theta=10000.0, partial_buf=part, out=out4, workspace=ws4, exchange=exchange, qpos=qpos, one_launch=True)

    def timed(fn, n):
        for _ in range(5):
            fn()
        cx.sync_all()
        s0, s1 = cx.event(), cx.event()
        s0.record()
        for _ in range(n):
            fn()
        s1.record()
        cx.sync_all()
        return cx.max_over_ranks(s0.elapsed_time(s1)) / n

    ms_gather = timed(step_gather, nsteps)
    ms_local = None
    if world > 1:
        try:
            cx.sync_all()
            graph_local = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph_local):
                for _ in range(nsteps):
                    step_local_only()
            for _ in range(2):
                graph_local.replay()
            cx.sync_all()
            s0, s1 = cx.event(), cx.event()
            s0.record()
            graph_local.replay()
            s1.record()
            cx.sync_all()
            ms_local = cx.max_over_ranks(s0.elapsed_time(s1)) / nsteps
        except Exception as e:
            exchange_error = f"graph (local only): {type(e).__name__}: {e}"[:200]
    ms_fused = ms_graph = ms_one = ms_one_graph = None
    graph_one = None
    if one_launch_ok:
        ms_one = timed(step_one_launch, nsteps)
        try:
            cx.sync_all()
            graph_one = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph_one):
                for _ in range(nsteps):
                    step_one_launch()
            for _ in range(2):
                graph_one.replay()
            cx.sync_all()
            s0, s1 = cx.event(), cx.event()
            s0.record()
            graph_one.replay()
            s1.record()
            cx.sync_all()
            ms_one_graph = cx.max_over_ranks(s0.elapsed_time(s1)) / nsteps
        except Exception as e:
            exchange_error = f"graph (one launch): {type(e).__name__}: {e}"[:200]
    if exchange is not None:
        ms_fused = timed(step_fused, nsteps)
        # the same steps replayed from one CUDA graph (the library is capture-safe and the exchange numbers its
        # calls on the device): removes the host's launch cost, which is comparable to a step at 8 GPUs
        try:
            cx.sync_all()
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(nsteps):
                    step_fused()
            for _ in range(2):
                graph.replay()
            cx.sync_all()
            s0, s1 = cx.event(), cx.event()
            s0.record()
            graph.replay()
            s1.record()
            cx.sync_all()
            ms_graph = cx.max_over_ranks(s0.elapsed_time(s1)) / nsteps
        except Exception as e:
            exchange_error = f"graph: {type(e).__name__}: {e}"[:200]
    # correctness of what was timed (a 1-GPU test box cannot run the N > 1 parity tests): the chosen path's result
    # against the all-gather path's, bit for bit, and against the CPU oracle's attention over the whole 131072-key
    # context for 4 sampled query heads (their KV heads' shards are collected on rank 0 for that)
    paths_bit_identical, max_abs_err, err_heads, one_launch_max_diff = None, None, [0, 21, 42, 63], None
    step_gather()
    cx.sync_all()
    out_gather = out4.clone()
    if exchange is not None:
        out4.zero_()
        step_fused()
        cx.sync_all()
        same = bool(torch.equal(out4, out_gather))
        if ms_graph is not None:
            out4.zero_()
            graph.replay()
            cx.sync_all()
            same = same and bool(torch.equal(out4, out_gather))
        if one_launch_ok:
            # the one-launch step merges its splits in another order: equal up to one rounding of the bf16 output
            out4.zero_()
            step_one_launch()
            cx.sync_all()
            one_launch_max_diff = float((out4.float() - out_gather.float()).abs().max().item())
            if ms_one_graph is not None:
                out4.zero_()
                graph_one.replay()
                cx.sync_all()
                one_launch_max_diff = max(one_launch_max_diff, float((out4.float() - out_gather.float()).abs().max().item()))
        flag = torch.tensor([1 if same else 0], dtype=torch.int32, device=dev)
        cx.dist.all_reduce(flag, op=cx.dist.ReduceOp.MIN)
        paths_bit_identical = bool(flag.item())
    try:
        n_rep = Hq // Hkv
        kv_sel = [h // n_rep for h in err_heads]
        k_loc, v_loc = ks[:, kv_sel].contiguous(), vs[:, kv_sel].contiguous()
        if world > 1:
            k_all = [torch.empty_like(k_loc) for _ in range(world)]
            v_all = [torch.empty_like(v_loc) for _ in range(world)]
            cx.dist.all_gather(k_all, k_loc)
            cx.dist.all_gather(v_all, v_loc)
            k_full, v_full = torch.cat(k_all, dim=2), torch.cat(v_all, dim=2)
        else:
            k_full, v_full = k_loc, v_loc
        if cx.rank == 0:
            from oracle.binding import Oracle          # the checker, outside every timed region
            orc = Oracle()
            q_rot = orc.apply_rope(q4[:, err_heads].float().cpu().numpy(), L4, 10000.0)
            want, _ = orc.decode_ragged(q_rot[:, :, 0], k_full.float().cpu().numpy(), v_full.float().cpu().numpy(), [L4])
            got = out_gather.view(Bq, Hq, D)[:, err_heads].float().cpu().numpy()
            max_abs_err = float(np.abs(got - want).max())
    except Exception as e:
        exchange_error = (exchange_error or "") + f" oracle check: {type(e).__name__}: {e}"[:200]
    candidates = [("all-gather + combine", ms_gather)] + ([("fused peer-memory exchange", ms_fused)] if ms_fused else []) + \
                 ([("fused peer-memory exchange, CUDA-graph replay", ms_graph)] if ms_graph else []) + \
                 ([("decode + split merge + exchange in one launch", ms_one)] if ms_one else []) + \
                 ([("decode + split merge + exchange in one launch, CUDA-graph replay", ms_one_graph)] if ms_one_graph else [])
    path, ms = min(candidates, key=lambda c: c[1])
    nbytes = 2.0 * Hkv * L4 * D * 2
    capi.check_kernel_status(cx.local)
    per_gpu = nbytes / world / (ms * 1e-3) / 1e9
    return {
        "metric": "long-context decode KV-read GB/s (aggregate)", "value": nbytes / (ms * 1e-3) / 1e9, "unit": "GB/s",
        "ms_per_step": ms, "scaling": "strong", "path": path,
        "ms_per_step_all_gather_path": ms_gather, "ms_per_step_fused_exchange": ms_fused, "ms_per_step_fused_exchange_graph": ms_graph,
        "ms_per_step_one_launch": ms_one, "ms_per_step_one_launch_graph": ms_one_graph, "one_launch_max_diff_vs_all_gather_path": one_launch_max_diff,
        "ms_per_step_local_shard_only_graph": ms_local,
        "exchange_share_of_step": (1.0 - ms_local / ms) if (ms_local and ms > 0) else None,
        "exchange_error": exchange_error,
        "paths_bit_identical": paths_bit_identical, "max_abs_err": max_abs_err,
        "max_abs_err_what": f"query heads {err_heads} over the whole context against the CPU oracle (gate 1e-2, bf16)",
        "config": {"workload": f"split-KV decode B=1 Hq={Hq} Hkv={Hkv} D={D} bf16, context {L4} sharded over {world} GPU(s); "
                               f"partial (O/l, m, l) records of {Hq * (D + 2) * 4} B per rank exchanged, then LSE merge"},
        "roofline": {"bound": "hbm", "achieved": per_gpu, "peak": cx.peaks["hbm"], "unit": "GB/s per GPU",
                     "frac": per_gpu / cx.peaks["hbm"], "peak_source": cx.peaks["source"]},
    }


def bench_model(cx, reps=3, layers=None, new=None):
    """C5: random-init Llama-style decoder (24 layers, d_model 2048, 16 query / 4 KV heads of 128, SwiGLU 5632,
    RMSNorm, RoPE 1e4, vocab 32000, bf16 weights ~ N(0, 0.02)); 8 prompts of 512 uniform-random ids, prefill then
    128 greedy tokens through generation::Generator of the host layer (device-resident loop, CUDA-graph replay).
    Every rank runs the whole workload (units = sequences, no collective): weak scaling."""
    import time

    import numpy as np
    from vesper_b200.model import TransformerLM, param_shapes
    capi = cx.capi
    c = dict(C5)
    if layers:
        c["layers"] = layers         # profiling runs only: a shallower stack launches the same kernels
    if new:
        c["new"] = new
    shapes = param_shapes(c["vocab"], c["dim"], c["layers"], c["Hq"], c["Hkv"], c["ffn"])
    m = TransformerLM(c["vocab"], c["dim"], c["layers"], c["Hq"], c["Hkv"], c["ffn"], c["P"] + c["new"], norm_eps=1e-6, rope_base=10000.0)
    rng = np.random.default_rng(7)
    n_params = 0
    for name in sorted(shapes):
        shape = shapes[name]
        w = np.ones(shape, np.float32) if len(shape) == 1 else (0.02 * rng.standard_normal(shape, dtype=np.float32))
        m.set_param(name, w)
        n_params += w.size
    prompt = np.random.default_rng(8).integers(0, c["vocab"], size=(c["B"], c["P"])).astype(np.int32)
    m.generate_greedy(prompt, min(8, c["new"]))                    # warm-up: kernels configured, buffers allocated
    cx.sync_all()
    pre_ms, dec_ms, wall_ms, steps = [], [], [], 0
    for _ in range(reps):
        cx.flush_l2()
        cx.sync_all()
        capi.load().vb200_reset_launch_count()
        t0 = time.perf_counter()
        toks, t = m.generate_greedy(prompt, c["new"])
        wall_ms.append((time.perf_counter() - t0) * 1e3)
        launches = int(capi.load().vb200_launch_count())
        pre_ms.append(t["prefill_ms"]); dec_ms.append(t["decode_ms"]); steps = t["decode_steps"]
    # attention share: the same generation, eager, with the attention kernels bracketed by events
    capi.profile_enable(True)
    _, tp = m.generate_greedy(prompt, c["new"], use_graph=False)
    attn_ms, attn_launches = capi.profile_read()
    capi.profile_enable(False)
    capi.check_kernel_status(cx.local)
    pre = cx.max_over_ranks(float(np.median(pre_ms)))
    dec = cx.max_over_ranks(float(np.median(dec_ms)))
    wall = cx.max_over_ranks(float(np.median(wall_ms)))
    cpu_attn = None
    if cx.rank == 0 and cx.world == 1 and not layers:
        # the reference's CPU attention for ONE layer of the prompt pass (128 (batch, head) slices of S = 512), all host threads
        cb, _ = cpu_prefill_sample(target_seconds=2.0, S=c["P"], total_slices=c["B"] * c["Hq"], what="one layer of the model's prompt pass")
        layer_flops = 4.0 * c["B"] * c["Hq"] * 128 * c["P"] * (c["P"] + 1) / 2.0
        cpu_attn = dict(cb, ms_per_layer_prompt_attention=layer_flops / (cb["value"] * 1e12) * 1e3)
    new_tokens = c["B"] * c["new"] * cx.world
    weight_bytes = 2.0 * (n_params - c["vocab"] * c["dim"])          # bf16; the embedding table is gathered, not streamed
    m.close()
    return {
        "metric": "generated tokens/s (prefill + greedy decode)", "value": new_tokens / ((pre + dec) * 1e-3), "unit": "tokens/s",
        "prefill_ms": pre, "decode_ms": dec, "decode_steps": steps, "ms_per_decode_step": dec / max(1, steps),
        "prefill_tokens_per_s": c["B"] * c["P"] * cx.world / (pre * 1e-3),
        "attention_time_share": attn_ms / (tp["prefill_ms"] + tp["decode_ms"]),
        "attention_kernel_ms": attn_ms, "attention_kernel_launches": int(attn_launches),
        "graph_replay": True, "launches_recorded_outside_graph": launches, "scaling": "weak",
        "cpu_baseline_attention": cpu_attn,
        "e2e": {"value": new_tokens / (wall * 1e-3), "unit": "tokens/s", "ms": wall,
                "h2d_bytes_per_step": int(prompt.nbytes), "d2h_bytes_per_step": int(toks.nbytes)},
        "roofline": {"bound": "hbm", "what": "decode step: bf16 weights streamed once per step",
                     "achieved": weight_bytes / (dec / max(1, steps) * 1e-3) / 1e9, "peak": cx.peaks["hbm"], "unit": "GB/s",
                     "frac": weight_bytes / (dec / max(1, steps) * 1e-3) / 1e9 / cx.peaks["hbm"], "peak_source": cx.peaks["source"]},
        "config": {"workload": f"Llama-style decoder {c['layers']} layers d_model {c['dim']} Hq={c['Hq']} Hkv={c['Hkv']} D=128 SwiGLU {c['ffn']} "
                               f"vocab {c['vocab']} bf16 weights N(0,0.02); {c['B']} prompts x {c['P']} random ids, prefill + {c['new']} greedy tokens; "
                               "per GPU (sequences are the units, no collective)", "parameters": int(n_params)},
    }


def run_ours(args):
    cx = Ctx()
    K, W = max(1, args.steps), max(3, args.warmup)
    only = args.only
    pre = bench_prefill(cx, K, W, quick=args.no_cpu_baseline) if only in ("all", "prefill") else None
    dec = bench_decode(cx, args.decode_steps, W) if only in ("all", "decode") else None
    shd = bench_sharded(cx) if only in ("all", "sharded") else None
    mdl = bench_model(cx, layers=args.model_layers, new=args.model_new) if only in ("all", "model") else None
    cpu_baseline = None
    if cx.rank == 0 and cx.world == 1 and not args.no_cpu_baseline and only == "all":
        cpu_baseline, _ = cpu_prefill_sample(target_seconds=12.0)
    if cx.rank == 0:
        line = {
            "metric": "prefill attn TFLOP/s & decode KV-read GB/s vs B200 roofline",
            "value": pre["value"] if pre else None, "unit": "TFLOP/s", "n_gpus": cx.world, "steps": K, "warmup": W,
            "ms_per_step": pre["ms_per_step"] if pre else None, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"GQA causal prefill B={C2['B']} Hq={C2['Hq']} Hkv={C2['Hkv']} S={C2['S']} D={C2['D']} bf16 (fp32 accumulate), "
                                   f"RoPE theta 1e4 on Q and K, K/V appended into an empty cache of capacity {C2['cap']}; per GPU, units "
                                   "(batch x kv_head) partitioned over ranks with no collective",
                       "l2": "256 MiB flush write between timed steps", "flops": "4*B*Hq*D*S*(S+1)/2"},
            "roofline": pre["roofline"] if pre else None,
            "e2e": pre["e2e"] if pre else None,
            "gpu_launches": pre["gpu_launches"] if pre else (dec["gpu_launches"] if dec else 0),
            "clocks": pre["clocks"] if pre else None,
            "decode": dec,
            "decode_sharded": shd,
            "model": mdl,
        }
        if cpu_baseline is not None:
            line["cpu_baseline"] = cpu_baseline
        emit(line)
    if cx.world > 1:
        cx.dist.destroy_process_group()


_REAL_STDOUT = None


def emit(line: dict):
    """Print the one JSON line on the real stdout."""
    out = _REAL_STDOUT or sys.stdout
    out.write(json.dumps(line) + "\n")
    out.flush()


def main():
    # libraries (NCCL's version banner, for one) write to fd 1: keep stdout for the JSON line alone
    global _REAL_STDOUT
    _REAL_STDOUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the timed CPU sample (profiling runs)")
    ap.add_argument("--decode-steps", type=int, default=C3["steps"], help="consecutive decode steps (default: the workload's 256)")
    ap.add_argument("--model-layers", type=int, default=0, help="profiling runs: depth of the model section's decoder (default: the workload's 24)")
    ap.add_argument("--model-new", type=int, default=0, help="profiling runs: tokens to generate in the model section (default: 128)")
    ap.add_argument("--only", default="all", choices=["all", "prefill", "decode", "sharded", "model"], help="run one section (profiling runs)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
