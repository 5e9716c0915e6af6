#!/usr/bin/env python
"""Benchmark of the attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--others c1,c3,c4] [--no-sharded] [--impl b200|reference]

One "step" is one pass of the hot path over one batch of synthetic input (one layer-step). The default
workload is the batched GQA decode of the Llama-3-8B layer shape (B=16, Hq=32, Hkv=8, D=128, per-sequence
KV lengths U[1024,8192] from seed 1, F16 K/V in the engine's HeadMajor layout). Rank 0 prints ONE JSON line:

  value     algorithmic HBM bytes per step / device time per step, inputs resident in HBM (TB/s)
  e2e       the same metric through the C ABI with HOST buffers: per step the inputs are copied from pinned
            host memory, the kernel runs, the output is copied back and read
  roofline  the dominant kernel against the measured HBM copy bandwidth of this pool
  cpu_baseline  the reference's AVX2 CPU attention (restated in oracle/) on the host cores, same inputs

With --gpus N > 1 (under torch.distributed.run) every rank runs an independent replica of the workload
(batched decode has no exchange step), timed as the max over ranks; the sequence-sharded 1M-token decode,
which does have one gather, is reported beside it under "sharded".
`--impl reference` times the reference's own CPU implementation of the same step on the host cores.
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


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops": float(d["bf16_tflops"]),
                "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d["bf16_tflops"])), "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    BITS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int, period: float = 0.02):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.reasons = [], set()
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


# ───────────────────────────── workloads ─────────────────────────────

def c2_case():
    from argus_engine_b200 import workloads as wl

    return wl.config2()


def decode_bytes(case) -> int:
    """Algorithmic bytes of one decode step: K+V rows read once, q read, out written."""
    kv = sum(case.lens) * case.hkv * case.d * 2 * 2
    return kv + 2 * len(case.lens) * case.hq * case.d * 4


def cpu_decode_step(case, seq_ids, threads=0):
    """The reference's CPU decode (AVX2 arm, one task per query head, sequences looped serially)."""
    from oracle import oracle as orc

    out = None
    for i in seq_ids:
        out, _ = orc.attention_gen(case.q[i], case.k[i].view(np.uint16), case.v[i].view(np.uint16), case.hq, case.hkv,
                                   case.d, case.lens[i], True, avx2=True, n_threads=threads)
    return out


def run_reference(args):
    """--impl reference: the reference's own CPU implementation of the step on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as orc

    case = c2_case()
    n = len(case.lens)
    cores = orc.num_threads()
    t = time.perf_counter()
    cpu_decode_step(case, range(n))
    one = time.perf_counter() - t
    total_steps = args.steps + args.warmup
    # bounded sample: keep the whole run within ~2 minutes by timing a prefix of the batch per step
    n_sample = n
    if one * total_steps > 120.0:
        n_sample = max(1, int(n * 120.0 / (one * total_steps)))
    ids = list(range(n_sample))
    sample_bytes = sum(case.lens[i] for i in ids) * case.hkv * case.d * 4 + 2 * n_sample * case.hq * case.d * 4
    for _ in range(args.warmup):
        cpu_decode_step(case, ids)
    t = time.perf_counter()
    for _ in range(args.steps):
        cpu_decode_step(case, ids)
    dt = (time.perf_counter() - t) / max(1, args.steps)
    value = sample_bytes / dt / 1e12
    sample = f"{n_sample} of {n} sequences of the batch per step ({sample_bytes / 1e6:.1f} MB algorithmic)"
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt * 1e3 * n / n_sample, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": workload_config("c2", case),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(name, case):
    return {"workload": f"{name}: batched GQA decode attention, Llama-3-8B layer shape", "batch": len(case.lens),
            "heads_q": case.hq, "heads_kv": case.hkv, "head_dim": case.d, "kv_lens": "U[1024,8192] seed 1",
            "kv_tokens_total": int(sum(case.lens)), "kv_dtype": "f16", "kv_layout": "HeadMajor [Hkv,cap,D]",
            "l2": "inputs (310 MB) exceed the 126 MB L2; two KV copies are alternated between steps"}


NCU_TRAFFIC_BYTES = 313.8e6   # per launch of decode_f16_kernel on configs[1], from the committed ncu summary


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


def other_configs(be, peaks, which):
    """The remaining benchmark configurations on one GPU (shorter runs; same timing hygiene). Returned as a
    dict that rides along in the JSON line; the headline stays the batched F16 decode."""
    import torch

    from argus_engine_b200 import DecodeExtras
    from argus_engine_b200 import workloads as wl

    dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()  # noqa: E731
    res = {}
    if "c1" in which:
        # configs[0]: launch-latency dominated, so the figure is microseconds per layer-step. 40 KV copies
        # (168 MB > L2) replayed from one CUDA graph, i.e. device time without host launch gaps.
        case = wl.config1()
        q = dev(case.q)
        out = torch.zeros(1, 32, 64, device="cuda")
        ks = [dev(case.k[0]) for _ in range(40)]
        vs = [dev(case.v[0]) for _ in range(40)]
        st = torch.cuda.Stream()
        with torch.cuda.stream(st):
            for i in range(3):
                be.attention_gen(q[0], ks[i], vs[i], out[0], 32, 8, 64, 2048)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st):
                for i in range(40):
                    be.attention_gen(q[0], ks[i], vs[i], out[0], 32, 8, 64, 2048)
            med, _ = _time_events(g.replay, 20)
        nbytes = decode_bytes(case)
        res["c1_decode_f16_T2048"] = {"us_per_layer_step": med * 1e3 / 40, "achieved_gbs": nbytes / (med / 40) / 1e6,
                                      "algorithmic_bytes": nbytes, "timing": "CUDA-graph replay of 40 calls on 40 KV copies"}
        del ks, vs
    if "c3" in which:
        # inputs go through the device-resident container: ring writes + the bit-exact device flush
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
        del src
        out = torch.zeros(B, 32, 128, device="cuda")
        ex = DecodeExtras(head_scores=torch.zeros(B, 8, T, device="cuda"), score_stride=T)
        fn = lambda: be.kivi_attention_batched(q, seqs, out, 32, 8, 128, 128, 4, 1 / np.sqrt(128), res_f16=True,  # noqa: E731
                                               extras=ex)
        med, _ = _time_events(fn, 20)
        nbytes = wl.kivi_step_bytes(qts, rts, 32, 8, 128, 4, 2, True)
        res["c3_kivi_q4_h2o"] = {"us_per_layer_step": med * 1e3, "achieved_gbs": nbytes / med / 1e6,
                                 "frac_of_hbm_peak": nbytes / med / 1e6 / peaks["hbm_gbs"], "algorithmic_bytes": nbytes,
                                 "l2": "338 MB of packed KV per step exceed the 126 MB L2"}
        del seqs
    if "c4" in which:
        B, S = 4, 4096
        gen = torch.Generator(device="cuda").manual_seed(3)
        q = torch.randn(B, S, 32, 128, device="cuda", generator=gen).to(torch.bfloat16)
        k = torch.randn(B, 8, S, 128, device="cuda", generator=gen).to(torch.bfloat16)
        v = torch.randn(B, 8, S, 128, device="cuda", generator=gen).to(torch.bfloat16)
        out = torch.empty_like(q)
        fn = lambda: be.flash_attention_prefill(q, k, v, out, 32, 8, S, S, 128, S, B, True)  # noqa: E731
        med, _ = _time_events(fn, 20)
        fl = wl.prefill_flops(B, S, S, 32, 128)
        res["c4_prefill_bf16"] = {"ms": med, "tflops": fl / med / 1e9, "frac_of_bf16_peak": fl / med / 1e9 / peaks["bf16_tflops"],
                                  "frac_of_bf16_sustained": fl / med / 1e9 / peaks["bf16_tflops_sustained"],
                                  "flops": fl, "p_operand": "F16 P against an F16 copy of each V tile made in shared memory (holds 2e-3)"}
    if "kv" in which:
        # the callers either side of attention on a device-resident F16 cache [Hkv=8, 256K tokens, D=128] (1 GiB of K+V)
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
        # paged layout option: configs[1]'s tokens in a shuffled pool of 256-token pages, same kernel with a page lookup
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
        kvres["paged_decode_c2_256_token_pages"] = {"us_per_layer_step": med * 1e3, "achieved_gbs": nbytes / med / 1e6,
                                                    "frac_of_hbm_peak": nbytes / med / 1e6 / peaks["hbm_gbs"]}
        res["kv_executors"] = kvres
    return res


def sharded_c5(be, dist, world, rank, peaks, iters=20):
    """configs[4]: 1M-token decode sharded by KV sequence over `world` GPUs. Per step: split-KV kernel over the
    local T/N slice -> one all-gather of (o, lse) -> merge. Device time, max over ranks."""
    import torch

    from argus_engine_b200.sharded import make_gpu_decoder, shard_range

    T, hq, hkv, d = 1 << 20, 64, 8, 128
    lo, hi = shard_range(T, world, rank)
    gen = torch.Generator(device="cuda").manual_seed(4 + rank)
    k = torch.randn(hkv, hi - lo, d, device="cuda", generator=gen, dtype=torch.float32).to(torch.float16)
    v = torch.randn(hkv, hi - lo, d, device="cuda", generator=gen, dtype=torch.float32).to(torch.float16)
    q = torch.randn(hq, d, device="cuda", generator=torch.Generator(device="cuda").manual_seed(4))
    fused = world > 1 and os.environ.get("ARGUS_B200_SHARDED_NCCL") is None
    try:
        dec = make_gpu_decoder(be, k, v, hi - lo, hq, hkv, d, fused=fused)
    except Exception:   # symmetric memory unavailable: NCCL all-gather + merge kernel
        fused = False
        dec = make_gpu_decoder(be, k, v, hi - lo, hq, hkv, d)
    out = torch.zeros(hq, d, device="cuda")
    for _ in range(3):
        dec.step(q, out)
    graph = dec.capture(q, out)
    run = graph.replay if graph is not None else (lambda: dec.step(q, out))
    for _ in range(3):
        run()
    if dist is not None:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        run()
    e1.record()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    if dist is not None:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    nbytes = T * hkv * d * 2 * 2 + 2 * hq * d * 4
    del k, v
    return {"workload": "c5: 1M-token decode, Hq=64 Hkv=8 D=128, KV sharded by sequence", "n_gpus": world,
            "us_per_layer_step": ms * 1e3, "value_tbs": nbytes / (ms * 1e-3) / 1e12,
            "frac_of_aggregate_hbm_peak": nbytes / (ms * 1e-3) / 1e9 / (peaks["hbm_gbs"] * world),
            "gather_bytes_per_rank": (hq * d + hq) * 4, "scaling": "strong", "l2": "shard >= 537 MB > L2",
            "exchange": "fused peer-store exchange + merge kernel" if fused else "NCCL all-gather + merge kernel",
            "launch": "CUDA graph replay of the step" if graph is not None else "eager"}


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
    case = c2_case()
    B, hq, hkv, d = len(case.lens), case.hq, case.hkv, case.d
    step_bytes = decode_bytes(case)

    # device-resident inputs: two KV copies, alternated so that no step finds its K/V in L2
    q = torch.from_numpy(case.q).cuda()
    kv_sets = []
    for _ in range(2):
        kv_sets.append(([torch.from_numpy(a).cuda() for a in case.k], [torch.from_numpy(a).cuda() for a in case.v]))
    out = torch.zeros(B, hq, d, device="cuda")

    def step(i):
        ks, vs = kv_sets[i & 1]
        be.attention_gen_batched(q, ks, vs, case.lens, out, hq, hkv, d)

    sampler = ClockSampler(local)
    sampler.start()

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    for i in range(max(3, args.warmup)):
        step(i)
    barrier()
    launches0 = be.launch_count
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.window[0] = time.perf_counter()
    e0.record()
    for i in range(args.steps):
        step(i)
    e1.record()
    barrier()
    sampler.window[1] = time.perf_counter()
    launches = be.launch_count - launches0
    ms = e0.elapsed_time(e1) / max(1, args.steps)
    if dist is not None:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    value = world * step_bytes / (ms * 1e-3) / 1e12

    # parity of the timed configuration against the oracle on one sequence (cheap, outside the timed region)
    parity = None
    if rank == 0:
        from oracle import oracle as orc

        i = int(np.argmin(case.lens))
        want, _ = orc.attention_gen(case.q[i], case.k[i].view(np.uint16), case.v[i].view(np.uint16), hq, hkv, d,
                                    case.lens[i])
        parity = float(np.max(np.abs(out[i].cpu().numpy() - want)))

    # end-to-end through the C ABI with host buffers
    hq_pin = torch.from_numpy(case.q).pin_memory()
    hk_pin = [torch.from_numpy(a).pin_memory() for a in case.k]
    hv_pin = [torch.from_numpy(a).pin_memory() for a in case.v]
    out_pin = torch.zeros(B, hq, d).pin_memory()
    dq = torch.empty_like(q)
    dk, dv = kv_sets[0]
    h2d = q.numel() * 4 + sum(a.numel() * 2 for a in hk_pin) * 2
    d2h = out.numel() * 4
    n_e2e = max(3, min(args.steps, 20))

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
    barrier()
    t0 = time.perf_counter()
    for _ in range(n_e2e):
        e2e_step()
    e2e_s = (time.perf_counter() - t0) / n_e2e
    if dist is not None:
        t = torch.tensor([e2e_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e_val = world * step_bytes / e2e_s / 1e12

    # The same with the KV cache where the engine keeps it, in device memory: a decode step then moves q and the new
    # token's K/V row from the host, writes the rows into the caches (argus_b200_kv_scatter_batched, one launch), runs
    # the attention call and reads the output back.
    knew = torch.stack([torch.from_numpy(case.k[i][:, case.lens[i] - 1, :].astype(np.float32)) for i in range(B)]).pin_memory()
    vnew = torch.stack([torch.from_numpy(case.v[i][:, case.lens[i] - 1, :].astype(np.float32)) for i in range(B)]).pin_memory()
    dknew, dvnew = torch.empty(B, hkv, d, device="cuda"), torch.empty(B, hkv, d, device="cuda")

    write_pos = [int(t) - 1 for t in case.lens]

    def resident_step():
        dq.copy_(hq_pin, non_blocking=True)
        dknew.copy_(knew, non_blocking=True)
        dvnew.copy_(vnew, non_blocking=True)
        be.kv_scatter_batched(dknew, dvnew, dk, dv, write_pos)
        be.attention_gen_batched(dq, dk, dv, case.lens, out, hq, hkv, d)
        out_pin.copy_(out, non_blocking=True)
        torch.cuda.synchronize()
        return float(out_pin[0, 0, 0])

    resident_step()
    barrier()
    n_res = max(20, min(args.steps, 200))
    t0 = time.perf_counter()
    for _ in range(n_res):
        resident_step()
    res_s = (time.perf_counter() - t0) / n_res
    # the same step captured once in a CUDA graph (copies from the pinned buffers, both launches, copy back): what a
    # serving loop in the engine's own language would issue without Python between the calls
    graph_s = None
    try:
        gstream = torch.cuda.Stream()
        with torch.cuda.stream(gstream):
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=gstream):
                dq.copy_(hq_pin, non_blocking=True)
                dknew.copy_(knew, non_blocking=True)
                dvnew.copy_(vnew, non_blocking=True)
                be.kv_scatter_batched(dknew, dvnew, dk, dv, write_pos)
                be.attention_gen_batched(dq, dk, dv, case.lens, out, hq, hkv, d)
                out_pin.copy_(out, non_blocking=True)
            for _ in range(3):
                g.replay()
                gstream.synchronize()
            t0 = time.perf_counter()
            for _ in range(n_res):
                g.replay()
                gstream.synchronize()
                _ = float(out_pin[0, 0, 0])
            graph_s = (time.perf_counter() - t0) / n_res
    except Exception as e:   # capture refused: keep the eager figure
        graph_s = None
        sys.stderr.write(f"[bench] graph capture of the resident step failed: {e}\n")
    if dist is not None:
        t = torch.tensor([res_s, graph_s if graph_s is not None else -1.0], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        res_s = float(t[0].item())
        graph_s = float(t[1].item()) if graph_s is not None else None
    e2e_resident = {"value": world * step_bytes / res_s / 1e12, "unit": UNIT, "ms_per_step": res_s * 1e3, "steps": n_res,
                    "h2d_bytes_per_step": int(q.numel() * 4 + 2 * knew.numel() * 4), "d2h_bytes_per_step": d2h,
                    "graph_replay": None if graph_s is None else {"value": world * step_bytes / graph_s / 1e12,
                                                                  "ms_per_step": graph_s * 1e3},
                    "note": "KV cache resident in HBM as in the engine; per step: q + new K/V rows H2D, one launch writing the 16 "
                            "rows, the attention call, output D2H, host sync; the output equals that of the timed step; "
                            "graph_replay = the same step replayed from one CUDA graph"}
    sampler.stop()

    cpu = None
    if rank == 0 and world == 1:
        from oracle import oracle as orc

        cores = orc.num_threads()
        cpu_decode_step(case, range(B))
        reps, t0 = 0, time.perf_counter()
        while reps < 3 or (time.perf_counter() - t0 < 10.0 and reps < 50):
            cpu_decode_step(case, range(B))
            reps += 1
        dt = (time.perf_counter() - t0) / reps
        cpu = {"value": step_bytes / dt / 1e12, "unit": UNIT, "cores": cores, "kind": "port",
               "sample": f"the whole step (16 sequences, {step_bytes / 1e6:.1f} MB algorithmic), mean of {reps} runs",
               "ms_per_step": dt * 1e3}

    del kv_sets, hk_pin, hv_pin
    torch.cuda.empty_cache()
    extra = {}
    if world == 1 and args.others:
        extra = other_configs(be, peaks, args.others.split(","))
    shard = sharded_c5(be, dist, world, rank, peaks) if args.sharded else None

    if rank == 0:
        achieved = step_bytes / (ms * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(3, args.warmup), "ms_per_step": ms, "us_per_layer_step": ms * 1e3,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
            "config": workload_config("c2", case),
            "roofline": {"bound": "hbm", "kernel": "decode_f16_kernel<128,4,3>", "achieved": achieved,
                         "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": achieved / peaks["hbm_gbs"],
                         "peak_source": peaks["source"], "traffic": NCU_TRAFFIC_BYTES,
                         "traffic_source": "dram__bytes_read.sum + dram__bytes_write.sum of one ncu capture of this "
                                           "workload (profiles/decode_f16_c2_batched_decode.md)",
                         "algorithmic_bytes_per_launch": step_bytes},
            "cpu_baseline": cpu,
            "e2e": {"value": e2e_val, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_s * 1e3, "steps": n_e2e,
                    "note": "conservative: the whole KV cache of the step is copied from pinned host memory every step"},
            "e2e_kv_resident": e2e_resident,
            "gpu_launches": int(launches),
            "clocks": sampler.summary(),
            "parity_max_abs_vs_oracle": parity,
            "other_configs": extra,
            "sharded": shard,
        }
        print(json.dumps(line), flush=True)
    be.close()
    if dist is not None:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=2000)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--others", default="c1,c3,c4,kv", help="comma list of further configs to time at N=1 ('' = none)")
    ap.add_argument("--no-sharded", dest="sharded", action="store_false", help="skip the sharded 1M-token decode")
    args = ap.parse_args()
    if args.impl == "reference":
        if args.steps == 2000:
            args.steps = 20
            args.warmup = min(args.warmup, 3)
        run_reference(args)
    else:
        run_b200(args)


if __name__ == "__main__":
    main()
