#!/usr/bin/env python
"""Benchmark of the VecAttention prefill hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload c4|c3|c2|c5|mini]
                    [--scaling strong|weak] [--impl graft|reference]

A step is one call of ``VecAttention_prefill`` (pool -> select -> vector-sparse attention) over
one layer's q/k/v of the named synthetic workload (default: the 118.8 K-token video-DiT shape, the
largest configuration that fits one GPU).  ``value`` is effective TFLOP/s: the FLOPs of the
selected (query tile, key) pairs only, 4 * rows * head_dim per pair, summed over all ranks,
divided by the slowest rank's device time.  One JSON line is printed by rank 0.

Under ``torchrun`` (N > 1) every rank drives one GPU.  ``--scaling strong`` (default): the heads of
the one layer are sharded across the ranks, whole KV groups per rank, no communication on the
path; ``--scaling weak``: every rank runs the whole single-GPU workload on its own draw of the data.

``--impl reference`` times the CPU restatement of the reference's PyTorch path (the oracle) with
all host threads on a bounded sample of the same workload; rank 0 only.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
# dram__bytes_read.sum + dram__bytes_write.sum per launch of the attention kernel, from the ncu
# capture summarised under profiles/ (workload -> bytes); None until a capture exists
# workload -> bytes; c4 was captured at full size (one-pass metrics): profiles/launch_list_c4.md
NCU_TRAFFIC_BYTES = {"c2h8": 303.4e6, "c4": 6.30e9 + 0.725e9}  # profiles/sparse_attn64_kernel_c2h8.md
NCU_SELECT_TRAFFIC_BYTES = {"c4": (729.9e6 + 12.9e6) + (810.9e6 + 658.3e6) + (670.5e6 + 1.71e9)}  # pool + mask + expand
# the capture is of 8 heads; DRAM traffic of this kernel grows in proportion to the heads processed
NCU_TRAFFIC_PER_HEAD_32K = 303.4e6 / 8
D = 128
CONFIG_HEADS = {"c2": 32, "c3": 40, "c4": 24, "c5": 28, "c2h8": 8}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            p = json.load(f)
        p["_source"] = "measured"
        return p
    p = dict(FALLBACK_PEAKS)
    p["_source"] = "fallback"
    return p


class ClockSampler:
    """SM clock and throttle reasons of one GPU, read through NVML every few milliseconds by a
    background thread while the warm-up and the timed region run (reading only; nothing is set)."""
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap"}

    def __init__(self, index: int, period_s: float = 0.003):
        self.index, self.period = index, period_s
        self.samples, self.bits, self.max_mhz = [], 0, None
        self.thread, self.stop, self.nvml, self.handle = None, threading.Event(), None, None

    def __enter__(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            try:  # the CUDA device's own identity, so that CUDA_VISIBLE_DEVICES renumbering cannot mislead
                uuid = str(torch.cuda.get_device_properties(self.index).uuid)
                uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:  # noqa: BLE001
                vis = os.environ.get("CUDA_VISIBLE_DEVICES", "")
                ids = [v for v in vis.split(",") if v.strip().isdigit()]
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(int(ids[self.index]) if self.index < len(ids) else self.index)
            self.nvml = pynvml
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
            self.thread = threading.Thread(target=self._run, daemon=True)
            self.thread.start()
        except Exception:  # noqa: BLE001 - no NVML: the summary says so
            self.nvml = None
        return self

    def _run(self):
        n = self.nvml
        reasons = getattr(n, "nvmlDeviceGetCurrentClocksEventReasons", None) or n.nvmlDeviceGetCurrentClocksThrottleReasons
        while not self.stop.is_set():
            try:
                self.samples.append(float(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM)))
                self.bits |= int(reasons(self.handle))
            except Exception:  # noqa: BLE001
                pass
            self.stop.wait(self.period)

    def __exit__(self, *exc):
        self.stop.set()
        if self.thread is not None:
            self.thread.join(timeout=2)

    def summary(self):
        out = {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": []}
        if self.samples:
            out["sm_mhz"] = statistics.median(self.samples)
            out["sm_min_mhz"] = min(self.samples)
            out["samples"] = len(self.samples)
        out["reasons"] = sorted(name for bit, name in self.REASONS.items() if self.bits & bit)
        if self.nvml is None:
            out["note"] = "NVML not available"
        return out


def effective_flops(counts: torch.Tensor, wl, blocks_per_tile=None) -> float:
    """4 * rows * D FLOPs per (query tile, key) pair; a ragged last tile counts its real rows."""
    pq = wl.q_pooling_size
    rows = torch.full((wl.nq,), pq, dtype=torch.float64, device=counts.device)
    rows[-1] = wl.seq_len - (wl.nq - 1) * pq
    keys = counts.to(torch.float64)
    if blocks_per_tile is not None:
        keys = keys + blocks_per_tile.to(torch.float64) * 64
    return float((keys * rows.view(1, 1, -1)).sum()) * 4.0 * D


def time_cuda(fn, warmup: int, iters: int) -> float:
    """Mean milliseconds per call on the current stream (CUDA events, synchronised both sides)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(iters):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def time_cuda_spread(fn, warmup: int = 10, reps: int = 20, flush: bool = False) -> dict:
    """Median and 20th / 80th percentile of single-call times (CUDA events around every call), the protocol of the
    reference's layer benchmark (spattn/benchmarks/bench_attn_layer.py:311-325: 10 warm-up calls, 20 timed).  With
    ``flush`` a buffer larger than L2 is overwritten before every timed call, outside the timed span."""
    for _ in range(warmup):
        fn()
    scrub = torch.empty(256 << 20, dtype=torch.uint8, device="cuda") if flush else None
    times = []
    for _ in range(reps):
        if scrub is not None:
            scrub.fill_(1)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
    times.sort()
    pick = lambda q: times[min(len(times) - 1, int(q * len(times)))]
    return {"median": statistics.median(times), "p20": pick(0.2), "p80": pick(0.8)}


def cpu_sample(name: str, threshold: float, tiles: int, sample_seed: int = 0):
    """Inputs of the bounded CPU sample: one head, the first ``tiles`` query tiles, all keys."""
    from vecattention_b200.synth import make_workload
    from vecattention_b200.synth import CONFIGS
    rep = CONFIGS[name]["heads"] // CONFIGS[name]["kv_heads"]
    wl = make_workload(name, device="cpu", heads=range(0, rep), sample_seed=sample_seed)
    wl.q = wl.q[:, :1]  # one query head (of the first KV group)
    rows = min(wl.seq_len, tiles * wl.q_pooling_size)
    return wl, wl.q[:, :, :rows].contiguous()


def run_cpu_sample(wl, q_rows, threshold: float, keep: bool = False):
    """One pass of the oracle over the sample; returns (seconds, effective FLOPs) and, with ``keep``, also the
    output and the per-tile selection counts."""
    from oracle import vecattn_oracle as O
    t0 = time.perf_counter()
    if wl.causal:
        out, sel = O.vecattention_prefill(q_rows, wl.k[:, :1, : q_rows.shape[2]], wl.v[:, :1, : q_rows.shape[2]],
                                          threshold, wl.q_pooling_size, wl.k_local_size, wl.group_k_block, True,
                                          wl.chunk_size, return_selection=True)
    else:
        out, sel = O.vecattention_prefill(q_rows, wl.k[:, :1], wl.v[:, :1], threshold, wl.q_pooling_size,
                                          wl.k_local_size, wl.group_k_block, False, wl.chunk_size,
                                          return_selection=True)
    dt = time.perf_counter() - t0
    pq = wl.q_pooling_size
    flops = 0.0
    t = 0
    for cc, _ in sel:
        for c in cc.flatten().tolist():
            rows = min(pq, q_rows.shape[2] - t * pq)
            flops += 4.0 * D * rows * c
            t += 1
    if keep:
        return dt, flops, out, torch.cat([cc for cc, _ in sel], dim=2)
    return dt, flops


def reference_arm(args):
    """The reference's CPU/PyTorch path (oracle restatement) on the host cores."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    thr = args.threshold if args.threshold else 0.5
    wl, q_rows = cpu_sample(args.workload, thr, args.cpu_tiles)
    if not args.threshold:
        from oracle import vecattn_oracle as O
        thr = _calibrate_cpu(wl, q_rows, O)
    for _ in range(max(1, min(args.warmup, 1))):
        run_cpu_sample(wl, q_rows, thr)
    secs, flops = [], 0.0
    for _ in range(args.steps):
        dt, flops = run_cpu_sample(wl, q_rows, thr)
        secs.append(dt)
    t = sum(secs) / len(secs)
    value = flops / t / 1e12
    sample = f"1 head x {q_rows.shape[2] // wl.q_pooling_size} query tiles x all {wl.seq_len} keys of {wl.name} per step"
    line = {
        "impl": "reference", "metric": "vecattention_prefill_effective_tflops", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": t * 1e3,
        "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": wl.name, "threshold": thr, "sample": sample},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def _calibrate_cpu(wl, q_rows, O) -> float:
    avg = O.pool_q(q_rows, wl.q_pooling_size)
    nq = avg.shape[2]
    pq = wl.q_pooling_size
    elig = sum(max(0, min(wl.seq_len, g * pq) - pq) for g in range(nq)) if wl.causal else nq * wl.seq_len
    lo, hi = 1e-9, 1.0
    kk = wl.k[:, :1]
    for _ in range(12):
        mid = math.sqrt(lo * hi)
        cnt, _ = O.select_columns(avg, kk, 0, -math.log(mid + 1e-9), wl.causal, pq, wl.k_local_size,
                                  wl.causal, wl.group_k_block)
        if float(cnt.sum()) / max(elig, 1) > wl.keep:
            lo = mid
        else:
            hi = mid
    return math.sqrt(lo * hi)


def _calibrated_threshold(va, wl, args):
    """MinP threshold that reaches the workload's keep ratio on this data (untimed)."""
    from vecattention_b200.synth import calibrate_threshold
    if args.threshold:
        return args.threshold
    pq, bk, g = wl.q_pooling_size, wl.k_local_size, wl.group_k_block
    avg_all = va.average_vector(wl.q, pq)
    rep = wl.heads // wl.kv_heads

    def counts_at(th, hslice):
        kv = slice(hslice.start // rep, max(1, hslice.stop // rep))
        cnt, _ = va.fuse_qk_softmax_minp_wo_causal(avg_all[:, hslice].contiguous(), wl.k[:, kv], 0,
                                                   -math.log(th + 1e-9), wl.causal, pq, bk, wo_initial=wl.causal,
                                                   group_k_block=g, trim=False, capacity=4)
        return cnt
    return calibrate_threshold(wl, counts_at)


def _stage_times(va, api, wl, thr, counts, bcnt, bidx, out):
    """Per-kernel times through the same entry points the operator uses, the way the operator runs them: one
    launch per stage for the whole sequence when its index lists fit the single-pass budget, else chunk by chunk."""
    pq, bk, g, chunk = wl.q_pooling_size, wl.k_local_size, wl.group_k_block, wl.chunk_size
    avg = va.average_vector(wl.q, pq)
    t_pool = time_cuda(lambda: va.average_vector(wl.q, pq), 3, 10)
    idx_all = wl.batch * wl.heads * wl.nq * ((wl.seq_len + 3) // 4 * 4) * 4
    free, _ = torch.cuda.mem_get_info()
    step_rows = wl.seq_len if idx_all <= min(32 << 30, int(free * 0.4)) else chunk
    sel_ms = att_ms = 0.0
    overlap = spread = None
    gap = -math.log(thr + 1e-9)
    for i in range(0, wl.seq_len, step_rows):
        t0, t1 = i // pq, min(wl.nq, -(-(i + step_rows) // pq))
        avg_c = avg[:, :, t0:t1].contiguous()
        sel = lambda: va.fuse_qk_softmax_minp_wo_causal(avg_c, wl.k, t0, gap, wl.causal, pq, bk, wo_initial=wl.causal,
                                                        group_k_block=g, trim=False)
        cc, ci = sel()
        sel_ms += time_cuda(sel, 2, 5)
        sk_eff = min(wl.seq_len, i + step_rows) if wl.causal else wl.seq_len
        qc, oc = wl.q[:, :, i:i + step_rows], out[:, :, i:i + step_rows]
        bc, bi = bcnt[:, :, t0:t1].contiguous(), bidx[:, :, t0:t1].contiguous()
        att = lambda: api._sparse_attn_bhsd(qc, wl.k[:, :, :sk_eff], wl.v[:, :, :sk_eff], pq, bc, bi, cc, ci,
                                            wl.causal, q_offset=i, out=oc)
        att_ms += time_cuda(att, 2, 5)
        if i == 0:
            overlap = _adjacent_tile_overlap(cc, ci, wl.seq_len)
        if step_rows >= wl.seq_len:  # one pass: the same two calls under the reference benchmark's protocol
            spread = {"warmup": 10, "reps": 20, "select_ms": time_cuda_spread(sel), "attn_ms": time_cuda_spread(att),
                      "select_ms_l2_flushed": time_cuda_spread(sel, flush=True)}
        del cc, ci
    out_d = {"pool_ms": t_pool, "select_ms": sel_ms, "attn_ms": att_ms, "adjacent_tile_union_over_mean": overlap}
    if spread is not None:
        out_d["spread"] = spread
    return out_d


def _adjacent_tile_overlap(cc, ci, sk, pairs=64):
    """How far the selected-column lists of neighbouring query tiles coincide: |A union B| / mean(|A|, |B|) over a
    sample of adjacent tile pairs of the first head (1 = identical lists, 2 = disjoint).  It bounds what sharing
    one gathered key set between two tiles could save."""
    nq = cc.shape[2]
    if nq < 2:
        return None
    tiles = torch.linspace(0, nq - 2, min(pairs, nq - 1)).long().unique().tolist()
    union = mean = 0.0
    for t in tiles:
        m = torch.zeros(2, sk + 1, dtype=torch.bool, device=ci.device)
        for j in range(2):
            n = int(cc[0, 0, t + j])
            m[j, ci[0, 0, t + j, :n].long()] = True
        union += float((m[0] | m[1]).sum())
        mean += float(m.sum()) / 2
    return union / max(mean, 1.0)


def _rooflines(wl, peaks, stage, flops, counts):
    esz = 2
    kept_total = float(counts.sum())
    sel_bytes = (wl.q.numel() + wl.k.numel()) * esz + 4 * kept_total + 4 * counts.numel()
    achieved_tf = flops / (stage["attn_ms"] * 1e-3) / 1e12
    full = wl.heads == CONFIG_HEADS.get(wl.name)
    traffic = (NCU_TRAFFIC_PER_HEAD_32K * wl.heads if wl.name in ("c2", "c2h8") else
               NCU_TRAFFIC_BYTES.get(wl.name) if full else None)
    roofline = {"kernel": "sparse_attn64_kernel" if wl.q_pooling_size == 64 else "sparse_attn128_kernel", "bound": "tensor",
                "achieved": achieved_tf, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
                "frac": achieved_tf / peaks["bf16_tflops"], "traffic": traffic,
                "traffic_note": ("ncu capture of 8 heads x 32 K tokens, scaled by heads" if wl.name in ("c2", "c2h8") else
                                 "one-pass ncu capture of this workload at full size (profiles/launch_list_c4.md): 1.5x the "
                                 "algorithmic 4.6 GB, K/V of two 61 MB heads do not both stay in the 126 MB L2" if traffic else
                                 "not captured for this workload or head count"),
                "peak_source": peaks["_source"] + " burst"}
    if peaks.get("bf16_tflops_sustained"):
        # the kernel runs for tens of milliseconds back to back under the power cap (see `clocks`): the denominator a
        # seconds-long GEMM loop reaches is given beside the burst figure; `frac` stays the fraction of the burst peak
        roofline["peak_sustained"] = peaks["bf16_tflops_sustained"]
        roofline["frac_of_sustained"] = achieved_tf / peaks["bf16_tflops_sustained"]
    sel_gbs = sel_bytes / ((stage["pool_ms"] + stage["select_ms"]) * 1e-3) / 1e9
    est_flops = 2.0 * wl.nq * wl.seq_len * D * wl.heads * wl.batch * (0.5 if wl.causal else 1.0)
    roofline_select = {"kernel": "pool_q_kernel+select_mask_kernel+select_expand_kernel", "bound": "hbm", "achieved": sel_gbs,
                       "peak": peaks["hbm_gbs"], "unit": "GB/s", "frac": sel_gbs / peaks["hbm_gbs"],
                       "algorithmic_bytes": sel_bytes, "peak_source": peaks["_source"],
                       "traffic": NCU_SELECT_TRAFFIC_BYTES.get(wl.name) if full else None,
                       "estimate_tflops": est_flops / (stage["select_ms"] * 1e-3) / 1e12,
                       "estimate_frac_of_tensor_peak": est_flops / (stage["select_ms"] * 1e-3) / 1e12 / peaks["bf16_tflops"]}
    return roofline, roofline_select


def _dense_baseline(wl):
    """Dense attention on the same GPU, for context: the best of the library kernels that run here, on four
    heads, scaled to all heads.  Returns (ms, which)."""
    hd = min(wl.heads, 4)
    rep = wl.heads // wl.kv_heads
    qd = wl.q[:, :hd]
    kd = wl.k[:, : max(1, hd // rep)].repeat_interleave(min(rep, hd), dim=1)[:, :hd]
    vd = wl.v[:, : max(1, hd // rep)].repeat_interleave(min(rep, hd), dim=1)[:, :hd]
    best, which, tried = None, None, {}
    cands = {"torch_sdpa": lambda: torch.nn.functional.scaled_dot_product_attention(qd, kd, vd, is_causal=wl.causal)}
    try:
        from flash_attn import flash_attn_func
        qf, kf, vf = (x.transpose(1, 2).contiguous() for x in (qd, kd, vd))
        cands["flash_attn"] = lambda: flash_attn_func(qf, kf, vf, causal=wl.causal)
    except Exception:  # noqa: BLE001
        pass
    try:
        import flashinfer
        q1, k1, v1 = (x[0].transpose(0, 1).contiguous() for x in (qd, kd, vd))
        cands["flashinfer"] = lambda: flashinfer.single_prefill_with_kv_cache(q1, k1, v1, causal=wl.causal)
    except Exception:  # noqa: BLE001
        pass
    for name, f in cands.items():
        try:
            ms = time_cuda(f, 1, 3) * wl.heads / hd
            tried[name] = ms
            if best is None or ms < best:
                best, which = ms, name
        except Exception as e:  # noqa: BLE001 - a library kernel that does not run on this GPU is skipped
            tried[name] = f"unavailable: {type(e).__name__}"
            torch.cuda.synchronize()
    return best, which, tried


def _reference_triton_select_ms(wl, thr):
    """The reference's own Triton selection (installed under baseline/_ref) on the same inputs, chunk by chunk
    as its operator calls it: the in-family GPU kernel the selection stage is measured against.  None if the
    reference is not installed or does not run."""
    ref_dir = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(ref_dir, "spattn")) or wl.heads != wl.kv_heads:
        return None, "reference not installed under baseline/_ref" if wl.heads == wl.kv_heads else "reference has no GQA"
    try:
        import types
        if ref_dir not in sys.path:
            sys.path.insert(0, ref_dir)
        stub = types.ModuleType("vllm_flash_attn")
        stub.sparse_attn_func = None
        sys.modules.setdefault("vllm_flash_attn", stub)
        from spattn.src.kernels.vecattention_kernels import fuse_qk_softmax_minp_wo_causal as ref_select
        from spattn.src.utils import average_vector as ref_pool
        pq, bk, g, chunk = wl.q_pooling_size, wl.k_local_size, wl.group_k_block, wl.chunk_size
        gap = -math.log(thr + 1e-9)

        def run():
            for i in range(0, wl.seq_len, chunk):
                avg = ref_pool(wl.q[:, :, i:i + chunk], pq, use_triton=True)
                ref_select(avg, wl.k, i // pq, gap, wl.causal, pq, bk, wo_initial=wl.causal, group_k_block=g)
        return time_cuda(run, 1, 2), "average_vector(use_triton=True) + fuse_qk_softmax_minp_wo_causal per chunk"
    except Exception as e:  # noqa: BLE001
        torch.cuda.synchronize()
        return None, f"reference Triton selection did not run: {type(e).__name__}: {e}"[:200]


def _pre_attention_leg(wl, peaks):
    """RMSNorm + rotary embedding of Q and K in one pass, on tensors of this workload's shape in (B,S,H*D) storage:
    an HBM-bound kernel (every element read once, written once)."""
    from vecattention_b200.preattn import qk_norm_rope
    dev = wl.q.device
    g = torch.Generator(device=dev).manual_seed(11)
    q = torch.randn(wl.batch, wl.seq_len, wl.heads * D, generator=g, device=dev, dtype=torch.float32).to(wl.dtype)
    k = torch.randn(wl.batch, wl.seq_len, wl.kv_heads * D, generator=g, device=dev, dtype=torch.float32).to(wl.dtype)
    wq = torch.ones(wl.heads * D, dtype=wl.dtype, device=dev)
    wk = torch.ones(wl.kv_heads * D, dtype=wl.dtype, device=dev)
    ang = torch.rand(wl.seq_len, D // 2, generator=g, device=dev) * 6.283
    cos, sin = torch.cos(ang).contiguous(), torch.sin(ang).contiguous()
    qo, ko = torch.empty_like(q), torch.empty_like(k)
    f = lambda: qk_norm_rope(q, k, wq, wk, 1e-6, cos, sin, heads=wl.heads, kv_heads=wl.kv_heads)
    ms = time_cuda(f, 2, 5)
    nbytes = 2 * (q.numel() + k.numel()) * 2 + 2 * cos.numel() * 4
    del qo, ko
    res = {"kernel": "qk_norm_rope_rows_kernel", "ms": ms, "achieved": nbytes / (ms * 1e-3) / 1e9, "unit": "GB/s",
           "peak": peaks["hbm_gbs"], "frac": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm_gbs"], "algorithmic_bytes": nbytes}
    # the per-head form on (B,H,L,128) tensors of the same size (per-element tables, text tokens last)
    from vecattention_b200.preattn import qk_head_norm_rope
    qh = q.view(wl.batch, wl.seq_len, wl.heads, D).transpose(1, 2).contiguous()
    kh = k.view(wl.batch, wl.seq_len, wl.kv_heads, D).transpose(1, 2).contiguous()
    del q, k
    txt = 256
    ang2 = torch.rand(wl.seq_len - txt, D, generator=g, device=dev) * 6.283
    cos2, sin2 = torch.cos(ang2).contiguous(), torch.sin(ang2).contiguous()
    wh = torch.ones(D, dtype=wl.dtype, device=dev)
    f2 = lambda: qk_head_norm_rope(qh, kh, wh, wh, 1e-6, cos2, sin2, txt)
    ms2 = time_cuda(f2, 2, 5)
    nbytes2 = 2 * (qh.numel() + kh.numel()) * 2 + 2 * cos2.numel() * 4
    res["per_head_form"] = {"kernel": "qk_head_norm_rope_kernel", "ms": ms2, "achieved": nbytes2 / (ms2 * 1e-3) / 1e9,
                            "unit": "GB/s", "frac": nbytes2 / (ms2 * 1e-3) / 1e9 / peaks["hbm_gbs"],
                            "algorithmic_bytes": nbytes2}
    return res


def _measure(va, api, wl, thr, args, barrier, status, out):
    """Warm-up, then exactly ``args.steps`` timed steps bracketed by barrier + synchronize.  Returns ms for all steps."""
    pq, bk, g, chunk = wl.q_pooling_size, wl.k_local_size, wl.group_k_block, wl.chunk_size

    def step():
        va.VecAttention_prefill(wl.q, wl.k, wl.v, thr, pq, bk, g, wl.causal, chunk, out=out, status=status)
    for _ in range(args.warmup):
        step()
    barrier()
    if args.profile_window:
        torch.cuda.profiler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(args.steps):
        step()
    e1.record()
    barrier()
    if args.profile_window:
        torch.cuda.profiler.stop()
    return e0.elapsed_time(e1)


def _launches_per_step(wl):
    idx_all_bytes = wl.batch * wl.heads * wl.nq * ((wl.seq_len + 3) // 4 * 4) * 4
    free, _ = torch.cuda.mem_get_info()
    n_chunks = 1 if idx_all_bytes <= min(32 << 30, int(free * 0.4)) else math.ceil(wl.seq_len / wl.chunk_size)
    return n_chunks * 5  # pool + selection (two kernels) + block tables + attention per pass


def _parity_on_cpu_sample(va, cwl, q_rows, thr, ref_out, ref_counts, dev):
    """The CUDA operator on the tensors of the CPU sample against the oracle's result for them."""
    causal = cwl.causal
    k = cwl.k[:, :1, : q_rows.shape[2]] if causal else cwl.k[:, :1]
    v = cwl.v[:, :1, : q_rows.shape[2]] if causal else cwl.v[:, :1]
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    out, counts = va.VecAttention_prefill(q_rows.to(dev), k.to(dev), v.to(dev), thr, cwl.q_pooling_size, cwl.k_local_size,
                                          cwl.group_k_block, causal, cwl.chunk_size, return_selection=True, status=status)
    err = (out.float().cpu() - ref_out.float()).abs()
    return {"count_diffs": int((counts.cpu() - ref_counts).abs().sum()), "selected_pairs": int(ref_counts.sum()),
            "max_abs": float(err.max()), "mean_abs": float(err.mean()), "status_word": int(status.item()),
            "checker": "CPU oracle on the cpu_baseline sample (selection pinned to the reference; attention parity unpinned)"}


def graft_arm(args):
    import torch.distributed as dist
    import vecattention_b200 as va
    from vecattention_b200 import api
    from vecattention_b200.sharding import local_slices
    from vecattention_b200.synth import CONFIGS, make_workload

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device (there is no CPU path for the product arm)")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    cfg = CONFIGS[args.workload]
    strong = args.scaling == "strong"
    if strong and world > cfg["kv_heads"]:
        raise SystemExit(f"{args.workload} has {cfg['kv_heads']} KV groups: it cannot be sharded over {world} GPUs")
    if args.shard:  # one rank's share of the heads on a single GPU, without a process group (for kernel work)
        r, n = (int(x) for x in args.shard.split("/"))
        hs, _ = local_slices(cfg["heads"], cfg["kv_heads"], r, n)
        wl = make_workload(args.workload, device=dev, heads=range(hs.start, hs.stop), keep=args.keep or None)
    elif strong and world > 1:
        hs, _ = local_slices(cfg["heads"], cfg["kv_heads"], rank, world)
        wl = make_workload(args.workload, device=dev, heads=range(hs.start, hs.stop), keep=args.keep or None)
    else:
        wl = make_workload(args.workload, device=dev, sample_seed=rank, keep=args.keep or None)
    pq, bk, g, chunk = wl.q_pooling_size, wl.k_local_size, wl.group_k_block, wl.chunk_size
    thr = _calibrated_threshold(va, wl, args)
    if world > 1 and strong and not args.threshold:  # one threshold for the layer: rank 0's calibration
        t = torch.tensor([thr], dtype=torch.float64, device=dev)
        dist.broadcast(t, 0)
        thr = float(t[0])
    out = torch.empty_like(wl.q)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    _, counts = va.VecAttention_prefill(wl.q, wl.k, wl.v, thr, pq, bk, g, wl.causal, chunk, return_selection=True)
    bcnt, bidx = api.block_tables(wl.batch, wl.heads, wl.seq_len, pq, wl.causal, dev)
    flops = effective_flops(counts, wl, bcnt if wl.causal else None)
    kept_pairs = float(counts.sum())
    launches = args.steps * _launches_per_step(wl)

    # ---- timed region: exactly K steps, device time, max over ranks ----
    with ClockSampler(local_rank) as clk:
        ms_total = _measure(va, api, wl, thr, args, barrier, status, out)
    clocks = clk.summary()

    # ---- end to end through the public API with host buffers, on every rank at once: q, k, v start in pinned
    # host memory and the output ends there, every step; the host entry point pipelines head slices (copy in /
    # compute / copy out) over three streams.  Device time, max over ranks. ----
    e2e_ms = e2e_err = 0.0
    h2d = d2h = 0
    if not args.profile_window:
        esz_ = wl.q.element_size()
        qh, kh, vh = (x.cpu().pin_memory() for x in (wl.q, wl.k, wl.v))
        oh = torch.empty_like(qh).pin_memory()
        staging = {}

        def e2e_step():
            va.VecAttention_prefill_host(qh, kh, vh, thr, pq, bk, g, wl.causal, chunk, out=oh, staging=staging)
        n_e2e = max(3, min(args.steps, 5))
        for _ in range(2):
            e2e_step()
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for _ in range(n_e2e):
            e2e_step()
        f1.record()
        barrier()
        e2e_ms = f0.elapsed_time(f1) / n_e2e
        e2e_err = float((oh.to(out.device).float() - out.float()).abs().max())
        h2d = (qh.numel() + kh.numel() + vh.numel()) * esz_
        d2h = oh.numel() * esz_
        del staging, qh, kh, vh, oh

    # ---- combine the ranks, then leave the process group: everything below is rank 0's own work and must not
    # keep the other ranks spinning in a collective ----
    local = torch.tensor([ms_total, e2e_ms, e2e_err, float(status.item()), flops, float(h2d), float(d2h), kept_pairs,
                          float(wl.eligible_pairs_per_head() * wl.heads * wl.batch)], dtype=torch.float64, device=dev)
    if world > 1:
        mx, sm = local.clone(), local.clone()
        dist.all_reduce(mx, op=dist.ReduceOp.MAX)
        dist.all_reduce(sm, op=dist.ReduceOp.SUM)
        per_rank = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(per_rank, local)
        barrier()
        dist.destroy_process_group()
    else:
        mx = sm = local
        per_rank = [local]
    if int(mx[3]) != 0:
        raise RuntimeError(f"a kernel reported status {int(mx[3])} (1 = index overflow, 2 = internal wait timeout) during the timed region")
    if rank != 0:
        return
    ms_step = float(mx[0]) / args.steps
    flops_all = float(sm[4])
    value = flops_all / (ms_step * 1e-3) / 1e12
    kept = float(sm[7]) / float(sm[8])
    heads_total = cfg["heads"] if strong else wl.heads
    config = {"workload": wl.name, "batch": wl.batch, "heads": heads_total, "kv_heads": cfg["kv_heads"] if strong else wl.kv_heads,
              "heads_per_gpu": wl.heads, "seq_len": wl.seq_len, "head_dim": D, "causal": wl.causal, "q_pooling_size": pq,
              "k_local_size": bk, "group_k_block": g, "chunk_size": chunk, "threshold": thr, "keep_ratio": kept,
              "effective_flops_per_step": flops_all,
              "l2": "inputs larger than L2 (q+k+v = %.0f MB per GPU), no flush" % ((wl.q.numel() + 2 * wl.k.numel()) * 2 / 1e6),
              "parallelism": ("heads sharded, no collective on the path" if strong else "replicated workload per GPU")}
    line = {"metric": "vecattention_prefill_effective_tflops", "value": value, "unit": "TFLOP/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True,
            "scaling": args.scaling, "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": config,
            "ms_per_layer": ms_step, "gpu_launches": launches, "clocks": clocks, "status_word": 0,
            "rank_ms_per_step": [float(r[0]) / args.steps for r in per_rank]}
    if args.profile_window:
        line["note"] = "profile window run: per-kernel, end-to-end and CPU legs skipped"
        print(json.dumps(line), flush=True)
        return
    line["e2e"] = {"value": flops_all / (float(mx[1]) * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": float(mx[1]),
                   "h2d_bytes_per_step": int(sm[5]), "d2h_bytes_per_step": int(sm[6]),
                   "max_abs_diff_vs_device_call": float(mx[2]),
                   "note": "VecAttention_prefill_host on every rank at once: pinned host q/k/v in, pinned host output out, "
                           "head slices pipelined over three streams; device time, max over ranks"}

    # ---- rank 0 only from here on ----
    peaks = load_peaks()
    stage = _stage_times(va, api, wl, thr, counts, bcnt, bidx, out)
    roofline, roofline_select = _rooflines(wl, peaks, stage, flops, counts)
    dense_ms, dense_which, dense_tried = _dense_baseline(wl)
    ref_sel_ms, ref_sel_note = _reference_triton_select_ms(wl, thr)
    line["pre_attention"] = _pre_attention_leg(wl, peaks)
    line.update({"stage_ms": stage, "roofline": roofline, "roofline_select": roofline_select,
                 "dense_attention_ms": dense_ms,
                 "dense_attention": {"ms_this_gpus_heads": dense_ms, "kernel": dense_which, "tried_ms": dense_tried,
                                     "note": "four heads timed, scaled to this GPU's heads"},
                 "reference_triton_select_ms": ref_sel_ms,
                 "reference_triton_select": {"ms": ref_sel_ms, "note": ref_sel_note,
                                             "ours_ms": stage["pool_ms"] + stage["select_ms"]}})

    # ---- CPU baseline: the oracle on a bounded sample, host cores of this box; its result also checks the GPU ----
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    cwl, q_rows = cpu_sample(args.workload, thr, args.cpu_tiles)
    _, _, ref_out, ref_counts = run_cpu_sample(cwl, q_rows, thr, keep=True)
    line["parity"] = _parity_on_cpu_sample(va, cwl, q_rows, thr, ref_out, ref_counts, dev)
    reps, secs, cflops = 0, 0.0, 0.0
    while secs < 10.0 and reps < 1000:
        dt, cflops = run_cpu_sample(cwl, q_rows, thr)
        secs += dt
        reps += 1
    line["cpu_baseline"] = {"value": cflops * reps / secs / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                            "sample": f"1 head x {q_rows.shape[2] // pq} query tiles x all {cwl.seq_len} keys of "
                                      f"{cwl.name}, {reps} passes, {secs:.1f} s"}
    del cwl, q_rows, ref_out

    # ---- the other configurations in brief (one GPU only): the same measurement with fewer steps ----
    if world == 1 and args.others:
        others = {}
        del wl, out, counts, bcnt, bidx
        torch.cuda.empty_cache()
        # (configuration 3 also at half and twice its keep ratio)
        todo = [(w, None) for w in ("c2", "c3", "c4", "c5", "d128") if w != args.workload] + [("c3", 0.05), ("c3", 0.20)]
        for name, okeep in todo:
            owl = make_workload(name, device=dev, keep=okeep)
            othr = _calibrated_threshold(va, owl, args)
            oout = torch.empty_like(owl.q)
            _, ocnt = va.VecAttention_prefill(owl.q, owl.k, owl.v, othr, owl.q_pooling_size, owl.k_local_size,
                                              owl.group_k_block, owl.causal, owl.chunk_size, return_selection=True)
            obc, obi = api.block_tables(owl.batch, owl.heads, owl.seq_len, owl.q_pooling_size, owl.causal, dev)
            oflops = effective_flops(ocnt, owl, obc if owl.causal else None)
            oargs = argparse.Namespace(**{**vars(args), "steps": 3, "warmup": 3})
            oms = _measure(va, api, owl, othr, oargs, barrier, status, oout) / 3
            ostage = _stage_times(va, api, owl, othr, ocnt, obc, obi, oout)
            orf, ors = _rooflines(owl, peaks, ostage, oflops, ocnt)
            others[name if okeep is None else f"{name}_keep{int(round(okeep * 100)):02d}"] = {"ms_per_layer": oms, "effective_tflops": oflops / (oms * 1e-3) / 1e12, "threshold": othr,
                            "keep_ratio": float(ocnt.sum()) / (owl.eligible_pairs_per_head() * owl.heads * owl.batch),
                            "stage_ms": ostage, "roofline_frac": orf["frac"], "roofline_select_frac": ors["frac"]}
            del owl, oout, ocnt, obc, obi
            torch.cuda.empty_cache()
        if int(status.item()) != 0:
            raise RuntimeError(f"a kernel reported status {int(status.item())}")
        line["other_workloads"] = others
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="graft", choices=["graft", "reference"])
    ap.add_argument("--workload", default="c4", choices=["c2", "c3", "c4", "c5", "d128", "c2h8", "mini"])
    ap.add_argument("--scaling", default="strong", choices=["weak", "strong"])
    ap.add_argument("--threshold", type=float, default=0.0, help="skip calibration and use this MinP threshold")
    ap.add_argument("--keep", type=float, default=0.0, help="calibrate the threshold to this keep ratio instead of the workload's")
    ap.add_argument("--cpu-tiles", type=int, default=512, help="query tiles in the bounded CPU sample")
    ap.add_argument("--no-others", dest="others", action="store_false",
                    help="skip the brief measurement of the other configurations (one-GPU runs only)")
    ap.add_argument("--shard", default="", help="r/n: run rank r's head shard of an n-way sharded layer on one GPU")
    ap.add_argument("--profile-window", action="store_true",
                    help="bracket the timed region with cudaProfilerStart/Stop (for `ncu --profile-from-start off`) "
                         "and skip the per-kernel, end-to-end and CPU legs")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "graft" else args.warmup
    if args.impl == "reference":
        reference_arm(args)
    else:
        graft_arm(args)


if __name__ == "__main__":
    main()
