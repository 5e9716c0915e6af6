#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--others c2,c1,c3,c4,kv] [--impl b200|reference]

One "step" is one pass of the hot path over one batch of synthetic input (one layer-step). The headline workload
at every N is the long-context decode of the Llama-3-70B attention shape (batch 1, Hq=64, Hkv=8, D=128, one
million cached tokens, F16 K/V in the engine's HeadMajor layout, seed 4), with the KV sequence sharded over the N
GPUs of the node: rank r holds tokens [r*T/N, (r+1)*T/N), runs the split-KV decode over its slice, and the (o, lse)
partials of all ranks are merged - in the same launch, through NVLink peer stores - into the F32 [64,128] output.
Total work is fixed as N grows ("scaling": "strong"). Rank 0 prints ONE JSON line:

  value     algorithmic HBM bytes of the whole step / device time per step (max over ranks), TB/s aggregate
  e2e       the same metric through the C ABI with HOST buffers: per step q and the rank's K/V slice are copied from
            pinned host memory, the step runs, the output is copied back and read
  roofline  decode_f16_kernel on the local slice against the measured HBM copy bandwidth of this pool
  cpu_baseline  the reference's AVX2 CPU attention (restated in oracle/) on the host cores, same inputs (N=1 only)
  parity    the merged output against the CPU oracle (one KV head over all 2^20 tokens) and against an independent
            merge of NCCL-gathered partials, both computed outside the timed region

At N=1 the other benchmark configurations ride along under "other_configs" (batched decode, single short decode,
KIVI Q4 decode with H2O scores, BF16 causal prefill, KV executors), each with its own CPU baseline and parity figure.
`--impl reference` times the reference's own CPU implementation of the headline step on the host cores.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "decode_attn_hbm_throughput"
UNIT = "TB/s"
OUT_ATOL, OUT_RTOL = 2e-3, 1e-2


def host_cores() -> int:
    """Cores this process may run on. The CPU arms size their thread pool from this, not from the OpenMP default,
    which a launcher may have set to 1 through OMP_NUM_THREADS."""
    return max(1, len(os.sched_getaffinity(0)))


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def ncu_traffic_ratio():
    """DRAM bytes moved per algorithmic byte by decode_f16_kernel, from the ncu capture summarised under profiles/
    (a small tracked JSON beside the summary, refreshed with it). None when the file is absent."""
    p = os.path.join(ROOT, "profiles", "decode_f16_traffic.json")
    try:
        with open(p) as f:
            d = json.load(f)
        return float(d["dram_bytes"]) / float(d["algorithmic_bytes"]), d.get("source", p)
    except Exception:
        return None, None


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    BITS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int, period: float = 0.005):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples = []
        self.max_mhz = None
        self._stop_evt = threading.Event()
        self.window = [None, None]
        self.ok = False
        try:
            import pynvml

            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
            self.ok = True
        except Exception:
            self.ok = False

    def run(self):
        if not self.ok:
            return
        while not self._stop_evt.is_set():
            try:
                mhz = int(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM))
                bits = int(self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
                self.samples.append((time.perf_counter(), mhz, bits))
            except Exception:
                pass
            time.sleep(self.period)

    def stop(self):
        self._stop_evt.set()

    def summary(self):
        if not self.ok or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": [], "samples": 0}
        t0, t1 = self.window
        inside = [s for s in self.samples if t0 is not None and t0 <= s[0] <= t1] or self.samples
        mhz = sorted(s[1] for s in inside)
        reasons = set()
        for s in inside:
            for bit, name in self.BITS.items():
                if s[2] & bit:
                    reasons.add(name)
        return {"sm_mhz": mhz[len(mhz) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(reasons),
                "samples": len(inside)}


# ───────────────────────────── headline workload: 1M-token decode, sharded by sequence ─────────────────────────────

TOKENS_OVERRIDE = None   # --tokens: a shorter cache of the same shape, for profiler captures of a small case


def c5_shape():
    from argus_engine_b200 import workloads as wl

    return (TOKENS_OVERRIDE or wl.C5_T), wl.C5_HQ, wl.C5_HKV, wl.C5_D


def c5_bytes(tokens=None) -> int:
    """Algorithmic bytes of the step: every K and V row read once, q read, out written."""
    T, hq, hkv, d = c5_shape()
    tokens = T if tokens is None else tokens
    return tokens * hkv * d * 2 * 2 + 2 * hq * d * 4


def c5_config(world):
    T, hq, hkv, d = c5_shape()
    return {"workload": "long-context GQA decode attention, Llama-3-70B attention shape, KV sequence sharded over the GPUs",
            "batch": 1, "heads_q": hq, "heads_kv": hkv, "head_dim": d, "kv_tokens_total": T, "kv_tokens_per_gpu": T // world,
            "kv_dtype": "f16", "kv_layout": "HeadMajor [Hkv,T/N,D]", "seed": 4,
            "inputs": "PCG64 standard_normal, one stream per (tensor, KV head, 65536-token block)",
            "l2": f"each GPU streams {T // world * hkv * d * 4 / 1e6:.0f} MB of K/V per step, more than the 126 MB L2: no flush needed"}


def cpu_c5_step(q, k, v, tokens, threads):
    """The reference's CPU decode (AVX2 arm, one task per query head) over the first `tokens` cached positions."""
    from oracle import oracle as orc

    T, hq, hkv, d = c5_shape()
    out, _ = orc.attention_gen(q, k.view(np.uint16), v.view(np.uint16), hq, hkv, d, tokens, True, avx2=True, n_threads=threads)
    return out


def run_reference(args):
    """--impl reference: the reference's own CPU implementation of the headline step on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from argus_engine_b200 import workloads as wl

    T, hq, hkv, d = c5_shape()
    cores = host_cores()
    q = wl.config5_q()
    k, v = wl.config5_slice(0, T, threads=cores)
    # bounded sample: time a prefix of the cached tokens per step when whole steps would not fit into ~2 minutes
    probe = 1 << 16
    cpu_c5_step(q, k, v, probe, cores)
    t = time.perf_counter()
    cpu_c5_step(q, k, v, probe, cores)
    per_tok = (time.perf_counter() - t) / probe
    total_steps = args.steps + args.warmup
    tokens = T
    if per_tok * T * total_steps > 120.0:
        tokens = max(probe, int(120.0 / (per_tok * total_steps)) // 4096 * 4096)
    for _ in range(args.warmup):
        cpu_c5_step(q, k, v, tokens, cores)
    t = time.perf_counter()
    for _ in range(args.steps):
        cpu_c5_step(q, k, v, tokens, cores)
    dt = (time.perf_counter() - t) / max(1, args.steps)
    value = c5_bytes(tokens) / dt / 1e12
    sample = (f"the whole step ({T} tokens, {c5_bytes() / 1e6:.0f} MB algorithmic)" if tokens == T else
              f"the first {tokens} of {T} cached tokens per step ({c5_bytes(tokens) / 1e6:.0f} MB algorithmic); ms_per_step is "
              "scaled to the whole step")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3 * T / tokens, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic", "config": c5_config(max(1, args.gpus)),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def _time_events(fn, iters, warmup=3):
    """Median and mean device time (ms) of fn() over `iters` calls, CUDA events on the current stream."""
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(iters)]
    for a, b in evs:
        a.record()
        fn()
        b.record()
    torch.cuda.synchronize()
    ts = sorted(a.elapsed_time(b) for a, b in evs)
    return ts[len(ts) // 2], sum(ts) / len(ts)


def _time_graph(fn, calls=10, reps=7, warmup=3):
    """Device time (ms) per fn() call from CUDA-graph replays of `calls` back-to-back calls (median over `reps` replays):
    what a serving loop that captures its step sees - no launch gaps from the Python caller inside the timed region."""
    import torch

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    with torch.cuda.stream(stream):
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=stream):
            for _ in range(calls):
                fn()
        g.replay()
        stream.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ts = []
        for _ in range(reps):
            a.record(stream)
            g.replay()
            b.record(stream)
            stream.synchronize()
            ts.append(a.elapsed_time(b) / calls)
    return sorted(ts)[len(ts) // 2]


def _cpu_time(fn, min_s=3.0, max_reps=50):
    """Mean wall time of fn() on the host: one warm-up call, then repeats for about `min_s` seconds."""
    fn()
    reps, t0 = 0, time.perf_counter()
    while reps < 2 or (time.perf_counter() - t0 < min_s and reps < max_reps):
        fn()
        reps += 1
    return (time.perf_counter() - t0) / reps, reps


def _parity(got, want, atol=OUT_ATOL, rtol=OUT_RTOL):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    return {"max_abs": float(np.max(np.abs(got - want))) if got.size else 0.0,
            "within_tolerance": bool(np.all(np.abs(got - want) <= atol + rtol * np.abs(want))),
            "atol": atol, "rtol": rtol}


def headline_c5(be, dist, world, rank, args, peaks, sampler):
    """Times K steps of the sharded decode and checks the result. Returns the pieces of the JSON line."""
    import torch

    from argus_engine_b200 import DecodeExtras
    from argus_engine_b200 import workloads as wl
    from argus_engine_b200.sharded import make_gpu_decoder, shard_range

    T, hq, hkv, d = c5_shape()
    lo, hi = shard_range(T, world, rank)
    n_local = hi - lo
    k_host, v_host = wl.config5_slice(lo, hi)
    q_host = wl.config5_q()
    k, v, q = torch.from_numpy(k_host).cuda(), torch.from_numpy(v_host).cuda(), torch.from_numpy(q_host).cuda()
    out = torch.zeros(hq, d, device="cuda")

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def allmax(x):
        if dist is None:
            return x
        t = torch.tensor([x], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    exchange = "none (one GPU)"
    dec = None
    if world > 1:
        fused = os.environ.get("ARGUS_B200_SHARDED_EXCHANGE", "fused") != "nccl"
        try:
            dec = make_gpu_decoder(be, k, v, n_local, hq, hkv, d, fused=fused)
        except Exception as e:   # symmetric memory unavailable: NCCL all-gather + merge kernel
            sys.stderr.write(f"[bench] peer buffers unavailable ({e}); using the NCCL gather\n")
            fused = False
            dec = make_gpu_decoder(be, k, v, n_local, hq, hkv, d)
        exchange = ("flagged 128-byte lines pushed to the peers, collected and merged in the decode kernel's epilogue "
                    "(one launch per step)" if fused else "decode kernel, NCCL all-gather, merge kernel")
        step = lambda: dec.step(q, out)   # noqa: E731
    else:
        step = lambda: be.attention_gen(q, k, v, out, hq, hkv, d, n_local)   # noqa: E731

    barrier()
    n0 = be.launch_count
    step()
    launches_per_step = be.launch_count - n0
    for _ in range(max(3, args.warmup) - 1):
        step()
    barrier()
    # one step captured in a CUDA graph: a replay costs the host a few microseconds, so that at 8 GPUs (about 80 us of
    # device time per step) the ranks are not waiting for each other's Python
    graph = None
    try:
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            step()
        graph = g
    except Exception as e:
        torch.cuda.synchronize()
        sys.stderr.write(f"[bench] graph capture of the step failed ({e}); launching eagerly\n")
    run = graph.replay if graph is not None else step
    for _ in range(3):
        run()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.window[0] = time.perf_counter()
    e0.record()
    for _ in range(args.steps):
        run()
    e1.record()
    barrier()
    sampler.window[1] = time.perf_counter()
    ms_local = e0.elapsed_time(e1) / max(1, args.steps)
    ms = allmax(ms_local)
    ms_min = -allmax(-ms_local)

    # ── checks, outside the timed region ──
    status = int(allmax(float(be.check_status())))
    plen = hq * d + hq
    part = torch.zeros(plen, device="cuda")
    be.attention_gen(q, k, v, part[:hq * d].view(hq, d), hq, hkv, d, n_local, extras=DecodeExtras(lse=part[hq * d:]))
    parts = torch.zeros(world, plen, device="cuda")
    if dist is not None:
        dist.all_gather_into_tensor(parts.view(-1), part)
    else:
        parts[0].copy_(part)
    pn = parts.cpu().numpy().astype(np.float64)
    o_r, lse_r = pn[:, :hq * d].reshape(world, hq, d), pn[:, hq * d:]
    w = np.exp(lse_r - lse_r.max(0, keepdims=True))
    merged64 = (w[:, :, None] * o_r).sum(0) / w.sum(0)[:, None]
    got = out.cpu().numpy()
    vs_gather = float(np.max(np.abs(got - merged64)))
    par_oracle = None
    if rank == 0:
        from oracle import oracle as orc

        kvh, g = 3, hq // hkv
        k3, v3 = wl.config5_slice(0, T, heads=[kvh])
        want, _ = orc.attention_gen(q_host[kvh * g:(kvh + 1) * g], k3.view(np.uint16), v3.view(np.uint16), g, 1, d, T,
                                    avx2=True, n_threads=host_cores())
        par_oracle = _parity(got[kvh * g:(kvh + 1) * g], want)
        par_oracle["checked"] = f"query heads {kvh * g}..{(kvh + 1) * g - 1} (KV head {kvh}) over all {T} tokens, AVX2 arm of the oracle"
        del k3, v3

    # ── end to end through the C ABI with host buffers ──
    hq_pin = torch.from_numpy(q_host).pin_memory()
    hk_pin, hv_pin = torch.from_numpy(k_host).pin_memory(), torch.from_numpy(v_host).pin_memory()
    out_pin = torch.zeros(hq, d).pin_memory()
    h2d = q.numel() * 4 + (k.numel() + v.numel()) * 2
    d2h = out.numel() * 4
    n_e2e = max(2, min(args.steps, 5))

    def e2e_step():
        q.copy_(hq_pin, non_blocking=True)
        k.copy_(hk_pin, non_blocking=True)
        v.copy_(hv_pin, non_blocking=True)
        step()
        out_pin.copy_(out, non_blocking=True)
        torch.cuda.synchronize()
        return float(out_pin[0, 0])

    e2e_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(n_e2e):
        e2e_step()
    e2e_s = allmax((time.perf_counter() - t0) / n_e2e)
    del hk_pin, hv_pin

    # The same with the KV cache where the engine keeps it, in device memory: a decode step moves q and the new token's
    # K/V row from the host, the rank that owns the end of the sequence writes the row into its cache, the step runs,
    # the output is copied back and read.
    # q, the new row and the output stay in pinned host memory and the kernels read / write them in place over PCIe
    # (40 KB in, 32 KB out), so the step is launches and one stream synchronisation, no copy operations.
    knew = torch.from_numpy(k_host[:, -1, :].astype(np.float32)[None].copy()).pin_memory() if n_local else None
    vnew = torch.from_numpy(v_host[:, -1, :].astype(np.float32)[None].copy()).pin_memory() if n_local else None
    owner = rank == world - 1 and n_local > 0

    def resident_ops():
        if world == 1:
            be.decode_step(hq_pin, knew[0], vnew[0], k, v, out_pin, hq, hkv, d, n_local - 1)
            return
        if owner:
            be.kv_scatter(knew, vnew, k, v, n_local - 1)
        dec.step(hq_pin, out_pin)

    def resident_step():
        resident_ops()
        torch.cuda.synchronize()
        return float(out_pin[0, 0])

    n_res = max(20, min(args.steps, 200))
    resident_step()
    barrier()
    t0 = time.perf_counter()
    for _ in range(n_res):
        resident_step()
    res_s = allmax((time.perf_counter() - t0) / n_res)
    graph_s = -1.0
    try:
        gstream = torch.cuda.Stream()
        with torch.cuda.stream(gstream):
            g2 = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g2, stream=gstream):
                resident_ops()
            for _ in range(3):
                g2.replay()
                gstream.synchronize()
            barrier()
            t0 = time.perf_counter()
            for _ in range(n_res):
                g2.replay()
                gstream.synchronize()
                _ = float(out_pin[0, 0])
            graph_s = (time.perf_counter() - t0) / n_res
    except Exception as e:
        torch.cuda.synchronize()
        sys.stderr.write(f"[bench] graph capture of the resident step failed: {e}\n")
    graph_s = allmax(graph_s)
    nbytes = c5_bytes()
    resident = {"value": nbytes / res_s / 1e12, "unit": UNIT, "ms_per_step": res_s * 1e3, "steps": n_res,
                "h2d_bytes_per_step": int(q.numel() * 4 + 2 * hkv * d * 4), "d2h_bytes_per_step": d2h,
                "graph_replay": None if graph_s <= 0 else {"value": nbytes / graph_s / 1e12, "ms_per_step": graph_s * 1e3},
                "note": "KV cache resident in HBM as in the engine; q, the new token's K/V row and the output live in pinned host "
                        "memory and are read / written by the kernels in place; per step: the row is written into the cache by "
                        "the rank that owns the end of the sequence (at N=1 inside the decode launch: argus_b200_decode_step), "
                        "the sharded step runs, the host synchronises and reads the output"}
    status2 = int(allmax(float(be.check_status())))
    ratio, ratio_src = ncu_traffic_ratio()
    local_bytes = c5_bytes(n_local)
    achieved = local_bytes / (ms * 1e-3) / 1e9
    res = {
        "value": nbytes / (ms * 1e-3) / 1e12, "ms": ms, "ms_fastest_rank": ms_min,
        "launches": int(launches_per_step * args.steps), "launches_per_step": int(launches_per_step),
        "launch": "CUDA graph replay of the step" if graph is not None else "eager",
        "exchange": exchange, "gather_bytes_per_rank": plen * 4,
        "roofline": {"bound": "hbm", "kernel": "decode_f16_kernel<128,4,3> on this GPU's slice (with the exchange in its epilogue at N>1)",
                     "achieved": achieved, "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                     "peak_source": peaks["source"], "algorithmic_bytes_per_launch": local_bytes,
                     "traffic": None if ratio is None else ratio * local_bytes,
                     "traffic_source": None if ratio is None else
                     f"dram__bytes_read.sum + dram__bytes_write.sum per algorithmic byte of one ncu capture of a smaller slice, "
                     f"scaled by the tokens of this launch ({ratio_src})"},
        "e2e": {"value": nbytes / e2e_s / 1e12, "unit": UNIT, "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                "ms_per_step": e2e_s * 1e3, "steps": n_e2e,
                "note": "conservative: every rank copies its whole K/V slice from pinned host memory every step (PCIe-bound by "
                        "construction; in the engine the cache is device-resident, see e2e_kv_resident)"},
        "e2e_kv_resident": resident,
        "parity": {"vs_oracle": par_oracle, "max_abs_vs_gathered_float64_merge": vs_gather,
                   "exchange_status": max(status, status2)},
    }
    del k, v
    torch.cuda.empty_cache()
    return res, (q_host, k_host, v_host)


# ───────────────────────────── the other configurations (one GPU) ─────────────────────────────

def decode_bytes(case) -> int:
    """Algorithmic bytes of one decode step: K+V rows read once, q read, out written."""
    kv = sum(case.lens) * case.hkv * case.d * 2 * 2
    return kv + 2 * len(case.lens) * case.hq * case.d * 4


def cpu_decode_step(case, seq_ids, threads):
    """The reference's CPU decode (AVX2 arm, one task per query head, sequences looped serially as the engine would)."""
    from oracle import oracle as orc

    outs = []
    for i in seq_ids:
        o, _ = orc.attention_gen(case.q[i], case.k[i].view(np.uint16), case.v[i].view(np.uint16), case.hq, case.hkv,
                                 case.d, case.lens[i], True, avx2=True, n_threads=threads)
        outs.append(o)
    return outs


def batched_decode_block(be, peaks, args):
    """Batched GQA decode of the Llama-3-8B layer shape: B=16, Hq=32, Hkv=8, D=128, lengths U[1024,8192] (seed 1)."""
    import torch

    from argus_engine_b200 import workloads as wl

    case = wl.config2()
    B, hq, hkv, d = len(case.lens), case.hq, case.hkv, case.d
    step_bytes = decode_bytes(case)
    cores = host_cores()
    q = torch.from_numpy(case.q).cuda()
    kv_sets = []
    for _ in range(2):   # two KV copies alternate so that no step finds its K/V in L2 (310 MB each)
        kv_sets.append(([torch.from_numpy(a).cuda() for a in case.k], [torch.from_numpy(a).cuda() for a in case.v]))
    out = torch.zeros(B, hq, d, device="cuda")
    flip = [0]

    def step():
        ks, vs = kv_sets[flip[0] & 1]
        flip[0] += 1
        be.attention_gen_batched(q, ks, vs, case.lens, out, hq, hkv, d)

    steps = max(20, min(args.steps, 500))
    for _ in range(5):
        step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        step()
    e1.record()
    torch.cuda.synchronize()
    ms_eager = e0.elapsed_time(e1) / steps     # calls issued one by one from Python (16 descriptors built per call)
    ms = _time_graph(step, calls=10)           # the same calls replayed from a CUDA graph, as the headline is timed
    got = out.cpu().numpy()
    want = cpu_decode_step(case, range(B), cores)
    par = _parity(got, np.stack(want))
    par["checked"] = "all 16 sequences against the AVX2 arm of the oracle"

    hq_pin = torch.from_numpy(case.q).pin_memory()
    hk_pin = [torch.from_numpy(a).pin_memory() for a in case.k]
    hv_pin = [torch.from_numpy(a).pin_memory() for a in case.v]
    out_pin = torch.zeros(B, hq, d).pin_memory()
    dq = torch.empty_like(q)
    dk, dv = kv_sets[0]
    h2d = q.numel() * 4 + sum(a.numel() * 2 for a in hk_pin) * 2
    d2h = out.numel() * 4

    def e2e_step():
        dq.copy_(hq_pin, non_blocking=True)
        for i in range(B):
            dk[i].copy_(hk_pin[i], non_blocking=True)
            dv[i].copy_(hv_pin[i], non_blocking=True)
        be.attention_gen_batched(dq, dk, dv, case.lens, out, hq, hkv, d)
        out_pin.copy_(out, non_blocking=True)
        torch.cuda.synchronize()
        return float(out_pin[0, 0, 0])

    e2e_step()
    n_e2e = 10
    t0 = time.perf_counter()
    for _ in range(n_e2e):
        e2e_step()
    e2e_s = (time.perf_counter() - t0) / n_e2e

    knew = torch.stack([torch.from_numpy(case.k[i][:, case.lens[i] - 1, :].astype(np.float32)) for i in range(B)]).pin_memory()
    vnew = torch.stack([torch.from_numpy(case.v[i][:, case.lens[i] - 1, :].astype(np.float32)) for i in range(B)]).pin_memory()
    write_pos = [int(t) - 1 for t in case.lens]

    def resident_ops():   # q, the new rows and the output stay in pinned host memory; the kernel reads / writes them in place
        be.decode_step_batched(hq_pin, knew, vnew, dk, dv, write_pos, out_pin, hq, hkv, d)

    n_res = 100
    resident_ops()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(n_res):
        resident_ops()
        torch.cuda.synchronize()
        _ = float(out_pin[0, 0, 0])
    res_s = (time.perf_counter() - t0) / n_res
    graph_s = None
    try:
        gstream = torch.cuda.Stream()
        with torch.cuda.stream(gstream):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=gstream):
                resident_ops()
            for _ in range(3):
                g.replay()
                gstream.synchronize()
            t0 = time.perf_counter()
            for _ in range(n_res):
                g.replay()
                gstream.synchronize()
                _ = float(out_pin[0, 0, 0])
            graph_s = (time.perf_counter() - t0) / n_res
    except Exception as e:
        torch.cuda.synchronize()
        sys.stderr.write(f"[bench] graph capture of the batched resident step failed: {e}\n")
    dt, reps = _cpu_time(lambda: cpu_decode_step(case, range(B), cores), 5.0)
    achieved = step_bytes / (ms * 1e-3) / 1e9
    ratio, ratio_src = ncu_traffic_ratio()
    res = {
        "workload": "batched GQA decode attention, Llama-3-8B layer shape (B=16, Hq=32, Hkv=8, D=128, KV lengths U[1024,8192] seed 1)",
        "value": step_bytes / (ms * 1e-3) / 1e12, "unit": UNIT, "us_per_layer_step": ms * 1e3, "steps": steps,
        "us_per_layer_step_eager": ms_eager * 1e3,
        "timing": "CUDA-graph replay of 10 calls on alternating KV copies, median of 7 replays; eager = the same calls issued "
                  "one by one from Python between two CUDA events",
        "kv_tokens_total": int(sum(case.lens)), "l2": "310 MB of K/V per step exceed the 126 MB L2; two KV copies alternate",
        "roofline": {"bound": "hbm", "kernel": "decode_f16_kernel<128,4,3>", "achieved": achieved, "peak": peaks["hbm_gbs"],
                     "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"], "peak_source": peaks["source"],
                     "algorithmic_bytes_per_launch": step_bytes, "traffic": None if ratio is None else ratio * step_bytes,
                     "traffic_source": ratio_src},
        "cpu_baseline": {"value": step_bytes / dt / 1e12, "unit": UNIT, "cores": cores, "kind": "port", "ms_per_step": dt * 1e3,
                         "sample": f"the whole step (16 sequences, {step_bytes / 1e6:.1f} MB algorithmic), mean of {reps} runs"},
        "e2e": {"value": step_bytes / e2e_s / 1e12, "unit": UNIT, "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
                "ms_per_step": e2e_s * 1e3, "steps": n_e2e,
                "note": "conservative: the whole KV cache of the step is copied from pinned host memory every step"},
        "e2e_kv_resident": {"value": step_bytes / res_s / 1e12, "unit": UNIT, "ms_per_step": res_s * 1e3, "steps": n_res,
                            "h2d_bytes_per_step": int(q.numel() * 4 + 2 * knew.numel() * 4), "d2h_bytes_per_step": int(d2h),
                            "graph_replay": None if graph_s is None else {"value": step_bytes / graph_s / 1e12,
                                                                          "ms_per_step": graph_s * 1e3},
                            "note": "KV cache resident in HBM; q, the 16 new K/V rows and the output live in pinned host memory; per "
                                    "step ONE launch writes the rows and attends (argus_b200_decode_step_batched, reading and "
                                    "writing the host buffers in place), then the host synchronises and reads the output"},
        "parity": par,
    }
    del kv_sets, hk_pin, hv_pin
    torch.cuda.empty_cache()
    return res


def other_configs(be, peaks, which, args):
    """The remaining benchmark configurations on one GPU (shorter runs; same timing hygiene), each with the reference's
    CPU path timed beside it on a stated sample and a parity figure against the oracle."""
    import torch

    from argus_engine_b200 import DecodeExtras
    from argus_engine_b200 import workloads as wl
    from oracle import oracle as orc

    cores = host_cores()
    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()  # noqa: E731
    res = {}
    if "c2" in which:
        res["batched_decode_f16_B16"] = batched_decode_block(be, peaks, args)
    if "c1" in which:
        # One short sequence (B=1, Hq=32, Hkv=8, D=64, T=2048, seed 0): launch-latency dominated, so the figure is
        # microseconds per layer-step. 40 KV copies (168 MB > L2) replayed from one CUDA graph, and the same 40 calls
        # issued one by one, so that both the device time and the time with host launch gaps are on record.
        case = wl.config1()
        q = dev(case.q)
        out = torch.zeros(1, 32, 64, device="cuda")
        ks = [dev(case.k[0]) for _ in range(40)]
        vs = [dev(case.v[0]) for _ in range(40)]

        def forty():
            for i in range(40):
                be.attention_gen(q[0], ks[i], vs[i], out[0], 32, 8, 64, 2048)

        eager_med, _ = _time_events(forty, 10)
        st = torch.cuda.Stream()
        with torch.cuda.stream(st):
            forty()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st):
                forty()
            med, _ = _time_events(g.replay, 20)
        nbytes = decode_bytes(case)
        want = cpu_decode_step(case, [0], cores)[0]
        dt, reps = _cpu_time(lambda: cpu_decode_step(case, [0], cores), 2.0, 2000)
        res["decode_f16_B1_T2048_D64"] = {
            "us_per_layer_step": med * 1e3 / 40, "us_per_layer_step_eager": eager_med * 1e3 / 40,
            "achieved_gbs": nbytes / (med / 40) / 1e6, "algorithmic_bytes": nbytes,
            "timing": "CUDA-graph replay of 40 calls on 40 KV copies; eager = the same 40 calls issued from Python",
            "cpu_baseline": {"value": dt * 1e6, "unit": "us/layer-step", "cores": cores, "kind": "port",
                             "sample": f"the whole step, mean of {reps} runs"},
            "parity": _parity(out[0].cpu().numpy(), want)}
        del ks, vs
    if "c3" in which:
        # KIVI Q4 decode with the H2O vector: B=8, Hq=32, Hkv=8, D=128, T=32768 (32640 packed + 128 residual), seed 2.
        # Inputs go through the device-resident container: ring writes + the bit-exact device flush.
        from argus_engine_b200.kivi_cache import KiviDeviceCache

        src = wl.config3_source()
        B, T = len(src.k), src.k[0].shape[0]
        seqs, qts, rts = [], [], []
        for i in range(B):
            cache = KiviDeviceCache(be, 8, 128, T, 128, 4)
            cache.update(dev(src.k[i]), dev(src.v[i]))
            seqs.append(cache.seq(res_f16=True))
            qts.append(cache.q_tokens)
            rts.append(cache.res_pos)
        q = dev(src.q)
        q_host = src.q
        del src
        out = torch.zeros(B, 32, 128, device="cuda")
        ex = DecodeExtras(head_scores=torch.zeros(B, 8, T, device="cuda"), score_stride=T)
        fn = lambda: be.kivi_attention_batched(q, seqs, out, 32, 8, 128, 128, 4, 1 / np.sqrt(128), res_f16=True,  # noqa: E731
                                               extras=ex)
        med_eager, _ = _time_events(fn, 20)
        med = _time_graph(fn)
        fn_plain = lambda: be.kivi_attention_batched(q, seqs, out, 32, 8, 128, 128, 4, 1 / np.sqrt(128), res_f16=True)  # noqa: E731
        med_plain = _time_graph(fn_plain)
        fn()
        torch.cuda.synchronize()
        nbytes = wl.kivi_step_bytes(qts, rts, 32, 8, 128, 4, 2, True)
        # CPU: what the reference does for a Q4 window cache on this backend - dequantise the whole cache into an F32
        # view, then the AVX2 decode with score export and the GQA score accumulation; one sequence, scaled to eight.
        i = B - 1
        qk, qv, rk, rv, qt, rt = seqs[i]
        hqk, hqv = qk.cpu().numpy(), qv.cpu().numpy()
        hrk, hrv = rk.float().cpu().numpy(), rv.float().cpu().numpy()

        def cpu_seq():
            vk, vv = orc.kivi_assemble_view(hqk, hqv, hrk, hrv, 8, 128, 128, 4, qt, rt)
            o, p = orc.attention_gen(q_host[i], vk, vv, 32, 8, 128, T, head_major=False, want_scores=True, avx2=True,
                                     n_threads=cores)
            sh = np.zeros(8 * T, dtype=np.float32)
            orc.score_accumulate_layer(p, T, 32, 8, T, np.zeros(T, dtype=np.float32), sh)
            return o, sh

        want_o, want_sh = cpu_seq()
        dt, reps = _cpu_time(cpu_seq, 4.0, 20)
        par = _parity(out[i].cpu().numpy(), want_o)
        par["head_scores"] = _parity(ex.head_scores[i].cpu().numpy(), want_sh.reshape(8, T), 1e-7, 1e-2)
        par["checked"] = "the last of the 8 sequences: output and the fused [Hkv,T] group-mean vector"
        res["kivi_q4_decode_h2o_B8_T32768"] = {
            "us_per_layer_step": med * 1e3, "achieved_gbs": nbytes / med / 1e6,
            "frac_of_hbm_peak": nbytes / med / 1e6 / peaks["hbm_gbs"], "algorithmic_bytes": nbytes,
            "us_per_layer_step_without_scores": med_plain * 1e3, "us_per_layer_step_eager": med_eager * 1e3,
            "timing": "CUDA-graph replay of 10 calls (decode + score finalize kernels each), median of 7 replays; eager = one "
                      "call at a time from Python between CUDA events",
            "l2": "338 MB of packed KV per step exceed the 126 MB L2",
            "cpu_baseline": {"value": dt * B * 1e3, "unit": "ms/layer-step", "cores": cores, "kind": "port",
                             "sample": f"1 of {B} sequences (dequantise to an F32 view, AVX2 decode with scores, GQA accumulation), "
                                       f"mean of {reps} runs, scaled by {B}"},
            "parity": par}
        del seqs
    if "c4" in which:
        # Causal GQA prefill: B=4, S=4096, Hq=32, Hkv=8, D=128, BF16, seed 3, drawn on the host by the seeded generator
        B, S = 4, 4096
        case = wl.config4(B, S)
        q = dev(case.q).to(torch.bfloat16)
        k = dev(case.k).to(torch.bfloat16)
        v = dev(case.v).to(torch.bfloat16)
        out = torch.empty_like(q)
        fn = lambda: be.flash_attention_prefill(q, k, v, out, 32, 8, S, S, 128, S, B, True)  # noqa: E731
        med, _ = _time_events(fn, 20)
        fl = wl.prefill_flops(B, S, S, 32, 128)
        # CPU: the scalar tiled prefill on a subset of the 128 (batch, head) pairs, one pair per core, scaled linearly
        n_pairs = min(cores, 16)
        pairs = (5 * 32 // 4, 5 * 32 // 4 + n_pairs)   # pairs 40..: batch 1, heads 8.. (any pair costs the same)
        t0 = time.perf_counter()
        want = orc.flash_prefill(case.q, case.k, case.v, 32, 8, S, S, 128, S, bh_range=pairs, n_threads=cores)
        dt = time.perf_counter() - t0
        got = out.float().cpu().numpy().reshape(B * S, 32, 128)
        wantr = wl._round_bf16(want).reshape(B * S, 32, 128)
        sel_g, sel_w = [], []
        for bh in range(*pairs):
            b, h = divmod(bh, 32)
            sel_g.append(got[b * S:(b + 1) * S, h])
            sel_w.append(wantr[b * S:(b + 1) * S, h])
        par = _parity(np.stack(sel_g), np.stack(sel_w))
        par["checked"] = f"(batch, head) pairs {pairs[0]}..{pairs[1] - 1} of 128, all 4096 rows, oracle output rounded to BF16"
        res["prefill_bf16_B4_S4096"] = {
            "ms": med, "tflops": fl / med / 1e9, "frac_of_bf16_peak": fl / med / 1e9 / peaks["bf16_tflops"],
            "frac_of_bf16_sustained": fl / med / 1e9 / peaks["bf16_tflops_sustained"], "flops": fl,
            "p_operand": "F16 P against an F16 copy of each V tile made in shared memory (holds 2e-3)",
            "cpu_baseline": {"value": dt * (B * 32) / n_pairs * 1e3, "unit": "ms", "cores": cores, "kind": "port",
                             "sample": f"{n_pairs} of {B * 32} (batch, head) pairs, one per core, scaled linearly ({dt:.1f} s measured)"},
            "parity": par}
        del q, k, v, out, case
    if "kv" in which:
        res["kv_executors"] = kv_executor_block(be, peaks)
    return res


def kv_executor_block(be, peaks):
    """The callers either side of attention on a device-resident F16 cache [Hkv=8, 256K tokens, D=128] (1 GiB of K+V)."""
    import torch

    from argus_engine_b200 import workloads as wl

    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()  # noqa: E731
    hkv, d, cap = 8, 128, 1 << 18
    gen = torch.Generator(device="cuda").manual_seed(5)
    k = torch.randn(hkv, cap, d, device="cuda", generator=gen).to(torch.float16)
    v = torch.randn(hkv, cap, d, device="cuda", generator=gen).to(torch.float16)
    cpu = torch.Generator().manual_seed(5)
    heavy = (torch.randperm(cap - 4 - 4096, generator=cpu)[: cap // 2].sort().values + 4)
    keep = torch.cat([torch.arange(4), heavy, torch.arange(cap - 4096, cap)]).to(torch.int32).cuda()
    med, _ = _time_events(lambda: be.kv_compact(k, v, keep, 0), 5)   # later repeats move the same row count
    moved = int(keep.numel()) * hkv * d * 2 * 2                      # K and V rows that change place (upper bound)
    kvres = {"compact_keep_positions": {"ms": med, "rows_kept": int(keep.numel()), "of": cap,
                                        "algorithmic_gbs": 2 * moved / med / 1e6,
                                        "frac_of_hbm_peak": 2 * moved / med / 1e6 / peaks["hbm_gbs"],
                                        "note": "H2O-like keep list: 4 sink + 50 % heavy hitters + 4096 recent; bytes = rows read + written once"}}
    S = 4096
    ks = torch.randn(S, hkv, d, device="cuda", generator=gen)
    vs = torch.randn(S, hkv, d, device="cuda", generator=gen)
    med, _ = _time_events(lambda: be.kv_scatter(ks, vs, k, v, 1000), 20)
    kvres["kv_scatter_prefill_4096_rows"] = {"us": med * 1e3, "gbs": S * hkv * d * (4 + 2) * 2 / med / 1e6}
    M = 32768
    perm = torch.randperm(cap, generator=cpu)
    into, frm = perm[:M].to(torch.int32).cuda(), perm[M:2 * M].to(torch.int32).cuda()
    iw, fw = torch.full((M,), 0.6, device="cuda"), torch.full((M,), 0.4, device="cuda")
    fs = torch.arange(M + 1, dtype=torch.int32, device="cuda")
    med, _ = _time_events(lambda: be.kv_weighted_merge(k, v, into, iw, fs, frm, fw), 10)
    kvres["weighted_merge_32768_pairs"] = {"us": med * 1e3, "gbs": M * hkv * d * 2 * 2 * 3 / med / 1e6}
    S = 4096
    qf = torch.randn(S, 32, d, device="cuda", generator=gen)
    sum_out = torch.zeros(32, S, device="cuda")
    med, _ = _time_events(lambda: be.prefill_attention_scores(qf, k, v, S, 0, 32, sum_out=sum_out), 20)
    kvres["prefill_attention_scores_S4096_window32"] = {"us": med * 1e3}
    ne, nr = 4096, 8192
    ev, rt = perm[:ne].to(torch.int32).cuda(), perm[ne:ne + nr].sort().values.to(torch.int32).cuda()
    med, _ = _time_events(lambda: be.d2o_nearest(k, ev, rt), 5)
    kvres["d2o_nearest_4096x8192"] = {"ms": med, "pair_dots_per_s": ne * nr / med * 1e3,
                                      "note": "1024-channel sequential-order F32 dot products (bit-exact index selection)"}
    del k, v
    # paged layout option: the batched decode's tokens in a shuffled pool of 256-token pages, same kernel with a page lookup
    case = wl.config2()
    ptok = 256
    npg = [(t + ptok - 1) // ptok for t in case.lens]
    order = torch.randperm(sum(npg), generator=cpu)
    pools = []
    for _ in range(2):   # two pools alternate so that a step does not find the other step's pages in L2
        pools.append((torch.zeros(sum(npg), 8, ptok, 128, device="cuda", dtype=torch.float16),
                      torch.zeros(sum(npg), 8, ptok, 128, device="cuda", dtype=torch.float16)))
    tables, nxt = [], 0
    for i, t in enumerate(case.lens):
        ids = order[nxt:nxt + npg[i]]
        nxt += npg[i]
        kd_, vd_ = dev(case.k[i]), dev(case.v[i])
        for j, pg in enumerate(ids.tolist()):
            lo, hi = j * ptok, min((j + 1) * ptok, t)
            for kp, vp in pools:
                kp[pg, :, :hi - lo] = kd_[:, lo:hi]
                vp[pg, :, :hi - lo] = vd_[:, lo:hi]
        tables.append(ids.to(torch.int32).cuda())
    qd = dev(case.q)
    outp = torch.zeros(len(case.lens), 32, 128, device="cuda")
    flip = [0]

    def paged_step():
        kp, vp = pools[flip[0] & 1]
        flip[0] += 1
        be.attention_gen_paged(qd, kp, vp, tables, case.lens, outp, 32)

    med, _ = _time_events(paged_step, 50)
    nbytes = decode_bytes(case)
    kvres["paged_decode_B16_256_token_pages"] = {"us_per_layer_step": med * 1e3, "achieved_gbs": nbytes / med / 1e6,
                                                 "frac_of_hbm_peak": nbytes / med / 1e6 / peaks["hbm_gbs"]}
    return kvres


def run_b200(args):
    import torch

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    torch.cuda.set_device(local)
    from argus_engine_b200 import B200Backend

    be = B200Backend(local)
    peaks = measured_peaks()
    sampler = ClockSampler(local)
    sampler.start()
    head, host_inputs = headline_c5(be, dist, world, rank, args, peaks, sampler)
    sampler.stop()

    cpu = None
    if rank == 0 and world == 1:
        q_host, k_host, v_host = host_inputs
        T = c5_shape()[0]
        cores = host_cores()
        dt, reps = _cpu_time(lambda: cpu_c5_step(q_host, k_host, v_host, T, cores), 10.0, 40)
        cpu = {"value": c5_bytes() / dt / 1e12, "unit": UNIT, "cores": cores, "kind": "port", "ms_per_step": dt * 1e3,
               "sample": f"the whole step ({T} tokens, {c5_bytes() / 1e6:.0f} MB algorithmic), mean of {reps} runs"}
    del host_inputs

    extra = {}
    if world == 1 and args.others:
        extra = other_configs(be, peaks, args.others.split(","), args)

    if rank == 0:
        line = {
            "metric": METRIC, "value": head["value"], "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": head["ms"], "us_per_layer_step": head["ms"] * 1e3,
            "ms_per_step_fastest_rank": head["ms_fastest_rank"],
            "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": c5_config(world), "exchange": head["exchange"], "gather_bytes_per_rank": head["gather_bytes_per_rank"],
            "launch": head["launch"], "roofline": head["roofline"], "cpu_baseline": cpu, "e2e": head["e2e"],
            "e2e_kv_resident": head["e2e_kv_resident"], "gpu_launches": head["launches"],
            "gpu_launches_per_step": head["launches_per_step"], "clocks": sampler.summary(), "parity": head["parity"],
            "other_configs": extra,
        }
        print(json.dumps(line), flush=True)
    be.close()
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--others", default="c2,c1,c3,c4,kv", help="comma list of further configurations to time at N=1 ('' = none)")
    ap.add_argument("--tokens", type=int, default=0, help="cached tokens of the headline workload (default 2^20); a smaller "
                    "multiple of 65536 gives the small case a profiler capture wants")
    args = ap.parse_args()
    if args.tokens:
        global TOKENS_OVERRIDE
        TOKENS_OVERRIDE = int(args.tokens)
    if args.impl == "reference":
        if args.steps == 200:
            args.steps = 10
            args.warmup = min(args.warmup, 2)
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
