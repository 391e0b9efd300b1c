"""Benchmark of the chunk-causal attention hot path (prologue -> [Ulysses in] -> attention -> [Ulysses out]).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg3|cfg1|cfg2|cfg4] [--exchange fused|nccl]
                    [--impl ours|reference] [--no-e2e] [--no-cpu-baseline] [--no-other-configs] [--no-gpu-dispatch-baseline]

One process per GPU (under torchrun for N > 1; RANK / LOCAL_RANK / WORLD_SIZE / MASTER_* from the environment).
Rank 0 prints ONE JSON line.  A "step" is one pass of the hot path over one batch of seeded synthetic inputs of
the named configuration: per-head LayerNorm + 3D RoPE of Q and K, (for N > 1: head<->sequence exchange in),
block-causal attention, (exchange out).  `value` = useful (unmasked) attention FLOPs of the whole job / step time.

Every rank generates the FULL input tensors from the workload's one seed and keeps its own sequence slice, so the
N-GPU job computes the same problem as the 1-GPU job; after the timed region rank 0 checks sampled rows of its output
against the CPU oracle and the line carries the result as "parity" (the process exits non-zero if it fails).
"""
import argparse
import json
import math
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "magi-1_b200")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import numpy as np
import torch

WORKLOADS = {
    # 24B-style 720p layer: 48/8 heads, 45x80 patches x 6 frames per chunk, 4 chunks, block-causal (cfg 3)
    "cfg3": dict(name="24B-720p: Hq48/Hkv8 d128, 4 chunks x 21600 tok (T24 H45 W80), block-causal, bf16",
                 hq=48, hkv=8, H=45, W=80, frames_per_chunk=6, n_chunks=4, seed=3,
                 # dram__bytes_read+write of attn_fwd_kernel per launch: ncu capture of the cfg1 launch (592.5 MB)
                 # scaled by the bytes the launch processes (x 2477.3 / 613.4)
                 traffic_bytes=2392.9e6),
    # 4.5B-style layer: 24/8 heads, 30x52 patches x 6 frames per chunk, 4 chunks (cfg 1)
    "cfg1": dict(name="4.5B-style: Hq24/Hkv8 d128, 4 chunks x 9360 tok (T24 H30 W52), block-causal, bf16",
                 hq=24, hkv=8, H=30, W=52, frames_per_chunk=6, n_chunks=4, seed=1, traffic_bytes=592.5e6),
    # KV-cache decode step (cfg 2): batch 2 (CFG), 4 denoising chunks each, chunk i sees its own cached prefix of i chunks + itself
    "cfg2": dict(name="4.5B-style decode: b2 x 4 denoising chunks x 9360 tok, own paged bf16 prefix (0..3 chunks) + self",
                 hq=24, hkv=8, H=30, W=52, frames_per_chunk=6, n_chunks=4, seed=2, decode=True, batch=2, n_prefix=3),
    # FP8 e4m3 of cfg 3 (cfg 4): chunks 0..2 read from an fp8 page cache, chunk 3 fresh; two-term Q/P
    "cfg4": dict(name="24B-720p FP8 e4m3: Hq48/Hkv8 d128, 4 q chunks x 21600 tok, K/V of chunks 0-2 from fp8 pages, chunk 3 fresh",
                 hq=48, hkv=8, H=45, W=80, frames_per_chunk=6, n_chunks=4, seed=3, fp8=True),
}

CPU_SAMPLE_ROWS = 4096   # q rows per chunk range in the CPU baseline sample (about 10 s of host work at cfg3)
PARITY_ROWS = 64         # sampled q rows of rank 0's output checked against the oracle after the timed region
BF16_MAX_ABS, BF16_MIN_COS, FP8_MIN_COS = 2e-2, 0.9999, 0.999


def useful_flops(hq, chunk_tokens, n_chunks):
    pairs = sum((i + 1) for i in range(n_chunks)) * chunk_tokens * chunk_tokens
    return 4.0 * 128 * hq * pairs


def measure_fp8_peak(dev):
    """Dense e4m3 GEMM 8192^3 through torch._scaled_mm (cuBLASLt), best of 10, CUDA events: the FP8 denominator that
    the driver-written peaks file does not carry."""
    try:
        n = 8192
        a = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn)
        b = torch.randn(n, n, device=dev).to(torch.float8_e4m3fn).t()
        one = torch.ones((), device=dev)
        best = 1e9
        for i in range(13):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            torch._scaled_mm(a, b, scale_a=one, scale_b=one, out_dtype=torch.bfloat16)
            e1.record()
            torch.cuda.synchronize()
            if i >= 3:
                best = min(best, e0.elapsed_time(e1))
        return 2.0 * n ** 3 / (best * 1e-3) / 1e12
    except Exception:  # pragma: no cover
        return None


def load_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return dict(bf16_burst=p["bf16_tflops"], bf16_sustained=p["bf16_tflops_sustained"], hbm=p["hbm_gbs"], src="measured")
    except Exception:
        return dict(bf16_burst=1590.0, bf16_sustained=1400.0, hbm=6650.0, src="fallback")


def nvml_handle(nv, index):
    """NVML handle of CUDA device `index` of this process: matched by PCI address, since NVML numbers the physical GPUs
    while CUDA numbers the visible ones."""
    try:
        pr = torch.cuda.get_device_properties(index)
        return nv.nvmlDeviceGetHandleByPciBusId(f"{pr.pci_domain_id:08x}:{pr.pci_bus_id:02x}:{pr.pci_device_id:02x}.0")
    except Exception:
        return nv.nvmlDeviceGetHandleByIndex(index)


def bind_to_gpu_cpus(index):
    """Run this rank on the CPUs NVML reports as local to its GPU (read-only query), so that the pinned host buffers of
    the end-to-end leg are first touched - and therefore placed - on the GPU's own NUMA node.  Silently a no-op where the
    query or the affinity call is not available or the mask would be empty."""
    try:
        import pynvml as nv
        nv.nvmlInit()
        h = nvml_handle(nv, index)
        words = nv.nvmlDeviceGetCpuAffinity(h, (os.cpu_count() + 63) // 64 + 16)
        cpus = {64 * i + b for i, wd in enumerate(words) for b in range(64) if (wd >> b) & 1}
        cpus &= os.sched_getaffinity(0)
        if cpus:
            os.sched_setaffinity(0, cpus)
    except Exception:
        pass


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.stop_flag, self.max_mhz = index, [], set(), False, None

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nvml_handle(nv, self.index)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)
            names = {nv.nvmlClocksThrottleReasonSwPowerCap: "sw_power_cap", nv.nvmlClocksThrottleReasonHwSlowdown: "hw_slowdown",
                     nv.nvmlClocksThrottleReasonHwThermalSlowdown: "hw_thermal_slowdown",
                     nv.nvmlClocksThrottleReasonSwThermalSlowdown: "sw_thermal_slowdown"}
            while not self.stop_flag:
                self.samples.append(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksThrottleReasons(h)
                for bit, nm in names.items():
                    if r & bit:
                        self.reasons.add(nm)
                time.sleep(0.05)
        except Exception as e:  # NVML unavailable: report that instead of inventing numbers
            self.reasons.add(f"nvml_unavailable:{type(e).__name__}")

    def summary(self):
        return {"sm_mhz": float(np.median(self.samples)) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons)}


# ------------------------------------------------------------------------------------------------ reference arm
def cpu_attention_sample(w, q_rows_per_range, threads):
    """The reference's attention math in eager fp32 PyTorch on the host (oracle port), on a bounded sample:
    one KV-head group, `q_rows_per_range` query rows of each of the chunk ranges against their full key ranges."""
    from oracle import chunk_attn_oracle as O
    torch.set_num_threads(threads)
    C = w["H"] * w["W"] * w["frames_per_chunk"]
    n, G = w["n_chunks"], w["hq"] // w["hkv"]
    g = torch.Generator().manual_seed(w["seed"])
    k = torch.randn(n * C, 1, 128, generator=g)
    v = torch.randn(n * C, 1, 128, generator=g)
    q = torch.randn(n * q_rows_per_range, G, 128, generator=g)
    qr = [[i * q_rows_per_range, (i + 1) * q_rows_per_range] for i in range(n)]
    segs = [[[0, (i + 1) * C]] for i in range(n)]
    flops = 4.0 * 128 * G * q_rows_per_range * sum((i + 1) * C for i in range(n))
    t0 = time.perf_counter()
    O.range_attention(q, k, v, qr, segs)
    dt = time.perf_counter() - t0
    return flops, dt


def run_reference(args, w, rank, world):
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    rows = CPU_SAMPLE_ROWS // 4
    for _ in range(args.warmup):
        cpu_attention_sample(w, 32, threads)
    tot_f, tot_t = 0.0, 0.0
    for _ in range(args.steps):
        f, t = cpu_attention_sample(w, rows, threads)
        tot_f += f
        tot_t += t
    val = tot_f / tot_t / 1e12
    C = w["H"] * w["W"] * w["frames_per_chunk"]
    sample = f"1 of {w['hkv']} KV-head groups, {rows} q rows of each of the {w['n_chunks']} chunk ranges vs their full key ranges, fp32 eager torch"
    line = {"impl": "reference", "metric": "chunk_causal_attn_useful_tflops", "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": tot_t / args.steps * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": w["name"], "chunk_tokens": C,
                       "useful_tflop_per_step": useful_flops(w["hq"], C, w["n_chunks"]) * w.get("batch", 1) / 1e12,
                       "parallelism": "host cpu", "step": "bounded sample of the attention math (see cpu_baseline.sample)"},
            "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample},
            "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------ parity probes
def _probe_rows(lo, hi, C, seed):
    """Sampled token ids in [lo, hi): both ends, the edges of 128-row tiles / 256-row work items / chunks, random rows."""
    cand = [lo, lo + 1, lo + 127, lo + 128, lo + 255, lo + 256, hi - 97, hi - 96, hi - 2, hi - 1]
    for c in range(lo // C, (hi - 1) // C + 1):
        cand += [c * C - 1, c * C, c * C + 128, (c + 1) * C - 96, (c + 1) * C - 1]
    gen = torch.Generator().manual_seed(seed)
    rnd = (torch.randint(0, hi - lo, (PARITY_ROWS,), generator=gen) + lo).tolist()
    rows = sorted({r for r in cand if lo <= r < hi})
    for r in rnd:
        if len(rows) >= PARITY_ROWS:
            break
        if r not in rows:
            rows.append(r)
    return torch.tensor(sorted(rows), dtype=torch.long)


def _oracle_rows(q_rows, rows, k, v, q_ranges, k_segments):
    """Oracle output of the sampled rows: q_rows[i] is token rows[i]; rows are sorted, so each range's samples are
    consecutive.  k_segments[i] = list of (start, end) key intervals of range i."""
    from oracle import chunk_attn_oracle as O
    sub_q, sub_k, pos = [], [], 0
    for (qs, qe), seg in zip(np.asarray(q_ranges).reshape(-1, 2), k_segments):
        m = int(((rows >= int(qs)) & (rows < int(qe))).sum())
        if m:
            sub_q.append([pos, pos + m])
            sub_k.append(seg)
            pos += m
    assert pos == len(rows)
    out, _ = O.range_attention(q_rows.float(), k.float(), v.float(), sub_q, sub_k)
    return out


def _parity_verdict(got, ref, fp8):
    from oracle import chunk_attn_oracle as O
    got, ref = got.float().cpu(), ref.float().cpu()
    max_abs = float((got - ref).abs().max())
    cos = O.cosine(got, ref)
    finite = bool(torch.isfinite(got).all())
    ok = finite and (cos >= FP8_MIN_COS if fp8 else (max_abs <= BF16_MAX_ABS and cos >= BF16_MIN_COS))
    return {"rows": int(got.shape[0]), "heads": int(got.shape[1]), "max_abs": max_abs, "cosine": cos, "ok": bool(ok),
            "against": "CPU fp32 oracle (prologue + attention) on the same seeded inputs",
            "tolerance": f"cosine >= {FP8_MIN_COS}" if fp8 else f"max_abs <= {BF16_MAX_ABS}, cosine >= {BF16_MIN_COS}"}


# ------------------------------------------------------------------------------------------------ our arm
def run_ours(args, wname, rank, world, local_rank, steps, warmup, want_e2e, want_cpu, dist):
    """Times one workload; returns the result dictionary on rank 0 (None elsewhere)."""
    import magi_b200 as mb
    from magi_b200 import host, ops
    w = WORKLOADS[wname]
    dev = torch.device("cuda", local_rank)
    cp = world
    Hq, Hkv = w["hq"], w["hkv"]
    C = w["H"] * w["W"] * w["frames_per_chunk"]
    n = w["n_chunks"]
    S = n * C
    flops = useful_flops(Hq, C, n)
    peaks = load_peaks()
    fp8, decode = bool(w.get("fp8")), bool(w.get("decode"))
    if decode and cp > 1:
        raise SystemExit(f"workload {wname} is a single-GPU benchmark line")

    gq, bq, gk, bk = host.synthetic_norm_params(w["seed"])
    sin_f, cos_f = host.split_sin_cos(host.rotary_table(n * w["frames_per_chunk"], w["H"], w["W"]))
    splits = host.cp_split_sizes(S, cp)
    off = sum(splits[:rank])
    s_loc = splits[rank]
    probe = None

    if not decode:
        # ---- the FULL projections from the one seed on every rank, then this rank's sequence slice
        g = torch.Generator(device=dev).manual_seed(w["seed"])
        rows = _probe_rows(0, splits[0], C, w["seed"] + 100) if rank == 0 else None

        def full(heads, keep_rows=False, keep_all=False):
            t = torch.randn(S, heads, 128, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
            extra = None
            if rank == 0 and keep_rows:
                extra = t[rows.to(dev)].cpu()
            if rank == 0 and keep_all:
                extra = t.cpu()
            return t[off:off + s_loc].clone(), extra
        xq, xq_rows = full(Hq, keep_rows=True)
        xk, xk_all = full(Hkv, keep_all=True)
        xv, xv_all = full(Hkv, keep_all=True)
        if rank == 0:
            probe = dict(rows=rows, xq_rows=xq_rows, xk=xk_all, xv=xv_all)
        torch.cuda.empty_cache()
        sin, cos = sin_f[off:off + s_loc].contiguous().to(dev), cos_f[off:off + s_loc].contiguous().to(dev)
        gq, bq, gk, bk = [t.to(dev) for t in (gq, bq, gk, bk)]
        qr = torch.as_tensor(host.q_ranges_for_chunks(n, C), device=dev)
        kr = torch.as_tensor(host.default_k_ranges(n, C), device=dev)

    fused = cp > 1 and args.exchange == "fused"
    ua = None
    if cp > 1:
        from magi_b200.ulysses import FusedUlyssesAttention, UlyssesAttention
        ua = FusedUlyssesAttention(dist.group.WORLD, Hq, Hkv, splits, n_out_buffers=2) if fused else \
            UlyssesAttention(cp_group=dist.group.WORLD, n_q_heads=Hq, n_kv_heads=Hkv, split_sizes=splits)
    attn_ev, prologue_ev = [], []
    state = {}   # what the parity probe needs from the set-up

    def timed_attn(record, fn):
        if record:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        r = fn()
        if record:
            e1.record()
            attn_ev.append((e0, e1))
        return r

    if decode:
        # ---- cfg 2: b x n denoising chunks; the clean prefix chunks live in the paged cache (filled outside the timed region)
        B, NP = w["batch"], w["n_prefix"]
        flops = B * flops
        g2 = torch.Generator(device=dev).manual_seed(w["seed"])
        xq = torch.randn(B * S, Hq, 128, generator=g2, device=dev, dtype=torch.float32).to(torch.bfloat16)
        xk = torch.randn(B * S, Hkv, 128, generator=g2, device=dev, dtype=torch.float32).to(torch.bfloat16)
        xv = torch.randn(B * S, Hkv, 128, generator=g2, device=dev, dtype=torch.float32).to(torch.bfloat16)
        cache = mb.ChunkPagedKVCache(n_layers=1, max_chunks=B * NP, chunk_tokens=C, n_kv_heads=Hkv, device=local_rank)
        pages = []
        for pc in range(B * NP):
            kvp = torch.randn(C, Hkv, 256, generator=g2, device=dev, dtype=torch.float32).to(torch.bfloat16)
            cache.append_kv(0, pc, kvp)
            pages.append(kvp.cpu())
        gq, bq, gk, bk = [t.to(dev) for t in (gq, bq, gk, bk)]
        sin_b, cos_b = sin_f.repeat(B, 1).to(dev), cos_f.repeat(B, 1).to(dev)
        qr_np = host.q_ranges_for_chunks(n, C, batch=B)
        qr = torch.as_tensor(qr_np, device=dev)
        kr_np, ko_np = host.own_prefix_k_segments(n, C, NP, batch=B)
        kr, ko = torch.as_tensor(kr_np, device=dev), torch.as_tensor(ko_np, device=dev)
        q_buf, k_buf, out_buf = torch.empty_like(xq), torch.empty_like(xk), torch.empty_like(xq)
        s_loc = B * S
        state.update(pages=pages, qr_np=qr_np, kr_np=kr_np, ko_np=ko_np, sin_b=sin_b, cos_b=cos_b)

        def step(record=False):
            mb.qk_norm_rope(xq, gq, bq, cos_b, sin_b, out=q_buf)
            mb.qk_norm_rope(xk, gk, bk, cos_b, sin_b, out=k_buf)
            timed_attn(record, lambda: mb.chunk_attn(q_buf, k_buf, xv, qr, kr, C, (NP + 1) * C, k_range_offsets=ko, out=out_buf,
                                                     return_lse=False, cache=cache, layer=0, prefix_chunk_ids=list(range(B * NP))))
            return out_buf
    elif fp8:
        # ---- cfg 4: K/V of chunks 0..n-2 sit in an fp8 page cache (head-sharded for N > 1, filled outside the timed
        # region from the prologued K and V of those chunks), the last chunk is fresh; Q and P run as two e4m3 terms
        hkv_loc = Hkv // cp
        hs = slice(rank * hkv_loc, (rank + 1) * hkv_loc)
        cache = mb.ChunkPagedKVCache(n_layers=1, max_chunks=n - 1, chunk_tokens=C, n_kv_heads=hkv_loc, dtype="fp8", device=local_rank)
        g_all = torch.Generator(device=dev).manual_seed(w["seed"])
        torch.randn(S, Hq, 128, generator=g_all, device=dev, dtype=torch.float32)          # skip xq's part of the stream
        xk_f = torch.randn(S, Hkv, 128, generator=g_all, device=dev, dtype=torch.float32).to(torch.bfloat16)
        xv_f = torch.randn(S, Hkv, 128, generator=g_all, device=dev, dtype=torch.float32).to(torch.bfloat16)
        k_all = mb.qk_norm_rope(xk_f, gk, bk, cos_f.to(dev), sin_f.to(dev))
        for pc in range(n - 1):
            cache.append(0, pc, k_all[pc * C:(pc + 1) * C, hs], xv_f[pc * C:(pc + 1) * C, hs])
        del k_all, xk_f, xv_f
        torch.cuda.empty_cache()
        prefix_ids = list(range(n - 1))
        if cp == 1:
            xk_cur, xv_cur = xk[(n - 1) * C:], xv[(n - 1) * C:]
            cos_cur, sin_cur = cos[(n - 1) * C:].contiguous(), sin[(n - 1) * C:].contiguous()
            q_buf = torch.empty(S, Hq, 128, dtype=torch.bfloat16, device=dev)
            k_buf = torch.empty(C, Hkv, 128, dtype=torch.bfloat16, device=dev)
            out_buf = torch.empty(S, Hq, 128, dtype=torch.bfloat16, device=dev)

            def step(record=False):
                mb.qk_norm_rope(xq, gq, bq, cos, sin, out=q_buf)
                mb.qk_norm_rope(xk_cur, gk, bk, cos_cur, sin_cur, out=k_buf)
                q8, qs, q8lo = mb.quantize_e4m3(q_buf, C, residual=True)
                k8, ks = mb.quantize_e4m3(k_buf, C)
                v8, vs = mb.quantize_e4m3(xv_cur, C)
                timed_attn(record, lambda: mb.chunk_attn(q8, k8, v8, qr, kr, C, S, out=out_buf, return_lse=False, cache=cache, layer=0,
                                                         prefix_chunk_ids=prefix_ids, q_scale=qs, k_scale=ks, v_scale=vs,
                                                         scale_chunk_tokens=C, q_lo=q8lo))
                return out_buf
        else:
            if not fused:
                raise SystemExit("cfg4 at N > 1 runs over the fused exchange")

            def step(record=False):
                return ua.forward(xq, xk, xv, gq, bq, gk, bk, cos, sin, qr, kr, C, S, attn_events=attn_ev if record else None,
                                  cache=cache, layer=0, prefix_chunk_ids=prefix_ids, kv_current_offset=(n - 1) * C,
                                  fp8_chunk_tokens=C)
    else:
        q_buf = torch.empty(s_loc, Hq, 128, dtype=torch.bfloat16, device=dev)
        k_buf = torch.empty(s_loc, Hkv, 128, dtype=torch.bfloat16, device=dev)
        out_buf = torch.empty(s_loc, Hq, 128, dtype=torch.bfloat16, device=dev)

        def step(record=False):
            if cp == 1:
                if record:
                    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    e0.record()
                mb.qk_norm_rope(xq, gq, bq, cos, sin, out=q_buf)
                if record:
                    e1.record()
                    prologue_ev.append((e0, e1))
                mb.qk_norm_rope(xk, gk, bk, cos, sin, out=k_buf)
                timed_attn(record, lambda: mb.chunk_attn(q_buf, k_buf, xv, qr, kr, C, S, out=out_buf, return_lse=False))
                return out_buf
            return ua.forward(xq, xk, xv, gq, bq, gk, bk, cos, sin, qr, kr, C, S, attn_events=attn_ev if record else None)

    def barrier():
        if cp > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(warmup):
        step()
    barrier()
    assert mb.Context.get(local_rank).status() == 0, "device status word reports a failure during warm-up"
    sampler = ClockSampler(local_rank)
    sampler.start()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    launches0 = ops.KERNEL_LAUNCHES[0]
    t0.record()
    for _ in range(steps):
        result = step(record=True)
    t1.record()
    barrier()
    launches = ops.KERNEL_LAUNCHES[0] - launches0
    sampler.stop_flag = True
    ms = t0.elapsed_time(t1)
    attn_ms = sum(a.elapsed_time(b) for a, b in attn_ev) / max(1, len(attn_ev))
    if cp > 1:
        tt = torch.tensor([ms, attn_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, attn_ms = tt.tolist()
    ms_per_step = ms / steps
    sampler.join(timeout=1.0)
    assert mb.Context.get(local_rank).status() == 0, "device status word reports a failure during the timed region"

    # ---- parity of what was just timed: sampled rows of rank 0's output against the CPU oracle
    parity = None
    cos_vs_bf16 = None
    if fp8:
        # the bf16 kernel on the same inputs, all chunks fresh: the FP8 acceptance bar is its cosine against this output
        out8 = result[:s_loc].clone()
        if cp == 1:
            k_all = mb.qk_norm_rope(xk, gk, bk, cos, sin)
            out16, _ = mb.chunk_attn(q_buf, k_all, xv, qr, kr, C, S, return_lse=False)
        else:
            out16 = ua.forward(xq, xk, xv, gq, bq, gk, bk, cos, sin, qr, kr, C, S)[:s_loc]
        a, b = out8.double().flatten(), out16.double().flatten()
        dots = torch.stack([a @ b, a @ a, b @ b])
        if cp > 1:
            dist.all_reduce(dots)
        cos_vs_bf16 = float(dots[0] / (dots[1] * dots[2]).sqrt())
        del out16, a, b
    if rank == 0:
        from oracle import chunk_attn_oracle as O
        if decode:
            B, NP = w["batch"], w["n_prefix"]
            rows = _probe_rows(0, B * S, C, w["seed"] + 100)
            kv_all = torch.cat(state["pages"]).float()
            q_ref = O.qk_prologue(xq[rows.to(dev)].cpu(), gq.cpu(), bq.cpu(), state["cos_b"][rows.to(dev)].cpu(), state["sin_b"][rows.to(dev)].cpu())
            k_ref = O.qk_prologue(xk.cpu(), gk.cpu(), bk.cpu(), state["cos_b"].cpu(), state["sin_b"].cpu())
            k_virt = torch.cat([kv_all[..., :128], k_ref.float()])
            v_virt = torch.cat([kv_all[..., 128:], xv.float().cpu()])
            segs = [[list(r) for r in state["kr_np"][state["ko_np"][i]:state["ko_np"][i + 1]]] for i in range(len(state["ko_np"]) - 1)]
            ref = _oracle_rows(q_ref, rows, k_virt, v_virt, state["qr_np"], segs)
            parity = _parity_verdict(result[rows.to(dev)], ref, False)
        else:
            rows = probe["rows"]
            kmax = (int(rows.max()) // C + 1) * C
            gq_c, bq_c, gk_c, bk_c = [t.cpu() for t in (gq, bq, gk, bk)]
            q_ref = O.qk_prologue(probe["xq_rows"], gq_c, bq_c, cos_f[rows], sin_f[rows])
            k_ref = O.qk_prologue(probe["xk"][:kmax], gk_c, bk_c, cos_f[:kmax], sin_f[:kmax])
            ref = _oracle_rows(q_ref, rows, k_ref, probe["xv"][:kmax], host.q_ranges_for_chunks(n, C),
                               [[list(r)] for r in host.default_k_ranges(n, C)])
            parity = _parity_verdict(result[(rows - off).to(dev)], ref, fp8)
            if cos_vs_bf16 is not None:
                parity["cosine_vs_bf16_kernel_whole_output"] = cos_vs_bf16
                parity["ok"] = bool(parity["ok"] and cos_vs_bf16 >= FP8_MIN_COS)
    probe = None

    # ---- end to end through the public API with host buffers (H2D of the step's inputs, D2H of its output)
    e2e = None
    if want_e2e:
        hq_, hk_, hv_ = xq.cpu().pin_memory(), xk.cpu().pin_memory(), xv.cpu().pin_memory()
        ho = torch.empty(s_loc, Hq, 128, dtype=torch.bfloat16).pin_memory()

        # The user-level pipeline: step i+1's inputs are copied host->device on a copy stream while step i computes, and
        # step i's output goes device->host on a third stream (double-buffered device inputs and outputs: on one GPU two
        # output tensors, under the fused exchange the two result buffers FusedUlyssesAttention rotates through).  Every
        # step still moves all of its inputs and its whole output across PCIe inside the timed region.
        pipelined = not fp8 and not decode
        main_s = torch.cuda.current_stream()
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        in_bufs = [(xq, xk, xv)] + ([(torch.empty_like(xq), torch.empty_like(xk), torch.empty_like(xv))] if pipelined else [])
        n_out = 2 if pipelined and (cp == 1 or fused) else 1
        out_bufs = [out_buf, torch.empty_like(out_buf)] if cp == 1 and n_out == 2 else [None] * n_out
        ev_in = [torch.cuda.Event() for _ in in_bufs]
        ev_free = [torch.cuda.Event() for _ in in_bufs]
        ev_out = [torch.cuda.Event() for _ in range(n_out)]
        copy_ev = []   # (h2d start, h2d end, d2h start, d2h end) per timed step
        counter = [0]

        def e2e_step(record=False):
            nonlocal xq, xk, xv, out_buf
            i = counter[0]
            counter[0] += 1
            if not pipelined:
                xq.copy_(hq_, non_blocking=True)
                xk.copy_(hk_, non_blocking=True)
                xv.copy_(hv_, non_blocking=True)
                ho.copy_(step()[:s_loc], non_blocking=True)
                return
            bi, bo = i % len(in_bufs), i % n_out
            evs = [torch.cuda.Event(enable_timing=True) for _ in range(4)] if record else None
            with torch.cuda.stream(s_in):
                if i >= len(in_bufs):
                    s_in.wait_event(ev_free[bi])       # the step that last read these buffers has finished
                if record:
                    evs[0].record(s_in)
                for dst, src in zip(in_bufs[bi], (hq_, hk_, hv_)):
                    dst.copy_(src, non_blocking=True)
                if record:
                    evs[1].record(s_in)
                ev_in[bi].record(s_in)
            main_s.wait_event(ev_in[bi])
            if i >= n_out:
                # the device->host copy out of the result buffer this step will overwrite is done; under the fused exchange
                # this wait also keeps the other ranks out of that buffer: they store into it only after this step's first
                # barrier, which this rank joins after the wait
                main_s.wait_event(ev_out[bo])
            xq, xk, xv = in_bufs[bi]
            if cp == 1:
                out_buf = out_bufs[bo]
            o = step()
            ev_free[bi].record(main_s)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_free[bi])
                if record:
                    evs[2].record(s_out)
                ho.copy_(o[:s_loc], non_blocking=True)
                if record:
                    evs[3].record(s_out)
                ev_out[bo].record(s_out)
            if record:
                copy_ev.append(evs)

        def e2e_drain():
            main_s.wait_stream(s_in)
            main_s.wait_stream(s_out)

        for _ in range(2):
            e2e_step()
        e2e_drain()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k_e2e = max(4, steps)
        a.record()
        for _ in range(k_e2e):
            e2e_step(record=True)
        e2e_drain()
        b.record()
        barrier()
        e_ms = a.elapsed_time(b)
        if cp > 1:
            tt = torch.tensor([e_ms], device=dev, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            e_ms = tt.item()
        h2d = (hq_.numel() + hk_.numel() + hv_.numel()) * 2
        d2h = ho.numel() * 2
        e2e = {"value": flops / (e_ms / k_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e_ms / k_e2e,
               "h2d_bytes_per_step": h2d * cp, "d2h_bytes_per_step": d2h * cp,
               "pipeline": "copies overlapped with the neighbouring steps on side streams, double-buffered inputs and results"
               if pipelined else "sequential"}
        if copy_ev:
            h_ms = sum(e[0].elapsed_time(e[1]) for e in copy_ev) / len(copy_ev)
            d_ms = sum(e[2].elapsed_time(e[3]) for e in copy_ev) / len(copy_ev)
            e2e["rank0_h2d_gbs"] = h2d / (h_ms * 1e-3) / 1e9
            e2e["rank0_d2h_gbs"] = d2h / (d_ms * 1e-3) / 1e9
            e2e["rank0_h2d_ms"], e2e["rank0_d2h_ms"] = h_ms, d_ms

    res = None
    if rank == 0:
        cpu_b = None
        if cp == 1 and want_cpu:
            threads = os.cpu_count() or 1
            cpu_attention_sample(w, 16, threads)
            f, t = cpu_attention_sample(w, CPU_SAMPLE_ROWS, threads)
            # BASELINE config 0 (the CPU-runnable case: 3 chunks x 128 tokens, 8/2 heads, fp32) timed in full
            from oracle import chunk_attn_oracle as O
            q0, k0, v0 = O.make_qkv(0, 384, 8, 2, scale=1.0 / math.sqrt(128))
            qr0, kr0 = O.consecutive_q_ranges(3, 128), O.default_k_ranges(3, 128)
            O.range_attention(q0, k0, v0, qr0, [[list(r)] for r in kr0])
            t_c0 = time.perf_counter()
            for _ in range(20):
                O.range_attention(q0, k0, v0, qr0, [[list(r)] for r in kr0])
            cfg0_ms = (time.perf_counter() - t_c0) / 20 * 1e3
            cpu_b = {"value": f / t / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port", "seconds": t, "cfg0_full_ms": cfg0_ms,
                     "sample": f"1 of {Hkv} KV-head groups, {CPU_SAMPLE_ROWS} q rows of each of the {n} chunk ranges vs their full key ranges, fp32 eager torch"}
        per_gpu_flops = flops / cp
        achieved = per_gpu_flops / (attn_ms * 1e-3) / 1e12
        res = dict(w=w, C=C, flops=flops, cp=cp, fused=fused, ms_per_step=ms_per_step, attn_ms=attn_ms, achieved=achieved,
                   per_gpu_flops=per_gpu_flops, clocks=sampler.summary(), launches=launches, parity=parity, cpu_b=cpu_b,
                   e2e=e2e, peaks=peaks, fp8=fp8, decode=decode)
        if prologue_ev:
            pms = sum(a.elapsed_time(b) for a, b in prologue_ev) / len(prologue_ev)
            pbytes = 2 * xq.numel() * 2 + 2 * cos.numel() * 4  # bf16 read + bf16 write of Q, cos+sin once
            res["prologue_q"] = {"kernel": "prologue8_kernel", "bound": "hbm", "ms": pms, "algorithmic_bytes": pbytes,
                                 "achieved_gbs": pbytes / (pms * 1e-3) / 1e9, "peak_gbs": peaks["hbm"],
                                 "frac": pbytes / (pms * 1e-3) / 1e9 / peaks["hbm"]}
        if fp8:
            res["fp8_peak"] = measure_fp8_peak(dev)
    if ua is not None and fused:
        ua.close()
    return res


def bench_modulate(dev, rows, hidden, n_gates, peaks):
    """The layer's gated post-norm residual (bias_modulate_add, dit_module.py:288-307) on the attention projection's
    fp32 output at the workload's token count: HBM-bound, x (fp32) and the residual (bf16) read once, bf16 written once."""
    import types
    import magi_b200 as mb
    g = torch.Generator(device=dev).manual_seed(9)
    x = torch.randn(rows, hidden, generator=g, device=dev, dtype=torch.float32)
    res = torch.randn(rows, hidden, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    gate = torch.tanh(torch.randn(n_gates, 2 * hidden, generator=g, device=dev)).to(torch.bfloat16)[:, :hidden]
    cmap = torch.arange(rows, device=dev) * n_gates // rows
    norm = types.SimpleNamespace(weight=0.1 * torch.randn(hidden, generator=g, device=dev), bias=torch.zeros(hidden, device=dev),
                                 eps=1e-6, zero_centered_gamma=True)
    out = torch.empty(rows, hidden, dtype=torch.bfloat16, device=dev)
    for _ in range(3):
        mb.bias_modulate_add(x, res, cmap, gate, norm, out=out)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(5):
        mb.bias_modulate_add(x, res, cmap, gate, norm, out=out)
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / 5
    nbytes = rows * hidden * (4 + 2 + 2)
    # spot check against the same arithmetic in torch on a few rows
    idx = torch.tensor([0, rows // 2, rows - 1], device=dev)
    y = x[idx] * gate[cmap[idx]].float()
    ref = torch.nn.functional.layer_norm(y, (hidden,), norm.weight + 1, norm.bias, 1e-6) + res[idx].float()
    err = float((out[idx].float() - ref).abs().max())
    return {"kernel": "modulate_kernel", "bound": "hbm", "rows": rows, "hidden": hidden, "ms": ms, "algorithmic_bytes": nbytes,
            "achieved_gbs": nbytes / (ms * 1e-3) / 1e9, "peak_gbs": peaks["hbm"], "frac": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm"],
            "max_abs_vs_torch_fp32_on_3_rows": err, "l2": "4.2 GB per launch, far beyond the 126 MB L2"}


def bench_div_clamp(dev, rows, hidden, peaks):
    """The FP8 linears' activation quantiser (div_clamp_to, dit_module.py:364-384) on the layer input at the workload's
    token count: HBM-bound, bf16 read once, e4m3 written once."""
    import magi_b200 as mb
    g = torch.Generator(device=dev).manual_seed(10)
    x = (torch.randn(rows, hidden, generator=g, device=dev) * 3).to(torch.bfloat16)
    scale = torch.rand(hidden, generator=g, device=dev) * 0.05 + 0.01
    out = torch.empty(rows, hidden, dtype=torch.float8_e4m3fn, device=dev)
    for _ in range(3):
        mb.div_clamp_to(x, scale, out=out)
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(5):
        mb.div_clamp_to(x, scale, out=out)
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / 5
    nbytes = rows * hidden * 3
    idx = torch.tensor([0, rows // 2, rows - 1], device=dev)
    ref = torch.clamp(x[idx].float() / scale, -448, 448).bfloat16().to(torch.float8_e4m3fn)
    same = bool(torch.equal(out[idx].view(torch.uint8), ref.view(torch.uint8)))
    return {"kernel": "div_clamp_e4m3_kernel", "bound": "hbm", "rows": rows, "hidden": hidden, "ms": ms, "algorithmic_bytes": nbytes,
            "achieved_gbs": nbytes / (ms * 1e-3) / 1e9, "peak_gbs": peaks["hbm"], "frac": nbytes / (ms * 1e-3) / 1e9 / peaks["hbm"],
            "bytes_equal_torch_on_3_rows": same}


def bench_qkv_projection(dev, index, rows, hidden, hq, hkv, peaks, seconds=1.5, iters=None):
    """get_qkv from the linear on (dit_module.py:953-1003) at the workload's token count: one launch of the projection
    GEMM (three weights) with the prologue in its epilogue, against the same work as the reference dispatches it - library
    GEMMs whose bf16 results go to HBM, then the prologue kernel on Q and K.  Tensor-bound; timed back to back for
    `seconds` (the regime of MEASURED_PEAKS.json's sustained figure) with the SM clock sampled."""
    import magi_b200 as mb
    from magi_b200 import host
    g = torch.Generator(device=dev).manual_seed(12)
    x = torch.randn(rows, hidden, generator=g, device=dev).to(torch.bfloat16)
    ws = [(torch.randn(h * 128, hidden, generator=g, device=dev) * hidden ** -0.5).to(torch.bfloat16) for h in (hq, hkv, hkv)]
    gq, bq, gk, bk = [t.to(dev) for t in host.synthetic_norm_params(12)]
    cos = torch.rand(rows, 48, generator=g, device=dev)
    sin = torch.rand(rows, 48, generator=g, device=dev)
    outs = [torch.empty(rows, h, 128, dtype=torch.bfloat16, device=dev) for h in (hq, hkv, hkv)]
    ys = [torch.empty(rows, h * 128, dtype=torch.bfloat16, device=dev) for h in (hq, hkv, hkv)]
    flops = 2.0 * rows * hidden * (hq + 2 * hkv) * 128

    def fused():
        mb.linear_qkv_norm_rope(x, [dict(weight=ws[0], gamma=gq, beta=bq, out=outs[0]), dict(weight=ws[1], gamma=gk, beta=bk, out=outs[1]),
                                    dict(weight=ws[2], norm_mode="none", out=outs[2])], cos, sin)

    def unfused():
        for i in range(3):
            torch.matmul(x, ws[i].t(), out=ys[i])
        mb.qk_norm_rope(ys[0].view(rows, hq, 128), gq, bq, cos, sin, out=outs[0])
        mb.qk_norm_rope(ys[1].view(rows, hkv, 128), gk, bk, cos, sin, out=outs[1])

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        n_it = iters or max(5, int(seconds * 1e3 / a.elapsed_time(b)))
        sampler = ClockSampler(index)
        sampler.start()
        a.record()
        for _ in range(n_it):
            fn()
        b.record()
        torch.cuda.synchronize()
        sampler.stop_flag = True
        sampler.join()
        return a.elapsed_time(b) / n_it, sampler.summary()

    # the same three projections as the middle layers run them (PerTensorQuantizedFp8Linear, dit_module.py:409-410):
    # activation quantiser, then e4m3 GEMMs; fused = quantiser + this kernel with e4m3 operands, library = quantiser +
    # torch._scaled_mm (cuBLASLt) + prologue kernel
    in_scale = torch.full((hidden,), 0.02, device=dev)
    w8 = [(w_ * 300).to(torch.float8_e4m3fn) for w_ in ws]
    sa, sb = in_scale[:1].clone(), torch.tensor([1 / 300.0], device=dev)
    x8 = torch.empty(rows, hidden, dtype=torch.float8_e4m3fn, device=dev)

    def fused8():
        mb.div_clamp_to(x, in_scale, out=x8)
        mb.linear_qkv_norm_rope(x8, [dict(weight=w8[0], gamma=gq, beta=bq, out=outs[0], w_scale=sb),
                                     dict(weight=w8[1], gamma=gk, beta=bk, out=outs[1], w_scale=sb),
                                     dict(weight=w8[2], norm_mode="none", out=outs[2], w_scale=sb)], cos, sin, x_scale=sa)

    def unfused8():
        mb.div_clamp_to(x, in_scale, out=x8)
        for i in range(3):
            ys[i].copy_(torch._scaled_mm(x8, w8[i].t(), scale_a=sa.reshape(()), scale_b=sb.reshape(()), out_dtype=torch.bfloat16))
        mb.qk_norm_rope(ys[0].view(rows, hq, 128), gq, bq, cos, sin, out=outs[0])
        mb.qk_norm_rope(ys[1].view(rows, hkv, 128), gk, bk, cos, sin, out=outs[1])

    seconds_full, seconds = seconds, seconds / 3
    ms_u8, _ = timed(unfused8)
    ref8 = outs[0][:4].float().clone()
    ms_f8, clk_f8 = timed(fused8)
    err8 = float((outs[0][:4].float() - ref8).abs().max())
    seconds = seconds_full
    ms_u, clk_u = timed(unfused)
    ref_rows = torch.tensor([0, rows // 2, rows - 1], device=dev)
    ref = [outs[0][ref_rows].float().clone(), outs[1][ref_rows].float().clone(), ys[2].view(rows, hkv, 128)[ref_rows].float().clone()]
    ms_f, clk_f = timed(fused)
    err = float(torch.stack([(o[ref_rows].float() - r).abs().max() for o, r in zip(outs, ref)]).max())
    tf = flops / (ms_f * 1e-3) / 1e12
    return {"kernel": "linear_prologue_kernel", "bound": "tensor", "rows": rows, "in_features": hidden, "heads": [hq, hkv, hkv],
            "ms": ms_f, "flops": flops, "achieved_tflops": tf, "peak_tflops": peaks["bf16_sustained"], "frac": tf / peaks["bf16_sustained"],
            "peak": "sustained bf16 (back-to-back launches, %s)" % (f"{iters} steps" if iters else f"{seconds} s"), "clocks": clk_f,
            "library_gemm_then_prologue_ms": ms_u, "library_gemm_then_prologue_clocks": clk_u,
            "max_abs_vs_library_gemm_then_prologue_on_3_rows": err, "launches": 1,
            "e4m3_operands": {"what": "activation quantiser + the three projections with e4m3 x and W (the middle layers' FP8 linears)",
                              "ms": ms_f8, "achieved_tflops": flops / (ms_f8 * 1e-3) / 1e12, "clocks": clk_f8,
                              "quantiser_library_fp8_gemm_then_prologue_ms": ms_u8, "max_abs_vs_that_on_4_rows": err8, "launches": 2}}


def flash_child(wname):
    """Child process of the default 1-GPU run: the reference's fallback dispatch on this GPU - a loop of flash_attn_func
    over the ranges (inference/model/dit/dit_module.py:1049-1065) with the flash-attn build of the image - on the same
    seeded, prologued inputs.  Comparison only, never a dispatch target; it runs in its own process so that flash-attn's
    library never enters the process whose numbers are reported."""
    import flash_attn
    import magi_b200 as mb
    from magi_b200 import host
    w = WORKLOADS[wname]
    dev = torch.device("cuda", 0)
    C, n, Hq, Hkv = w["H"] * w["W"] * w["frames_per_chunk"], w["n_chunks"], w["hq"], w["hkv"]
    S = n * C
    g = torch.Generator(device=dev).manual_seed(w["seed"])
    xq = torch.randn(S, Hq, 128, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    xk = torch.randn(S, Hkv, 128, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    xv = torch.randn(S, Hkv, 128, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    gq, bq, gk, bk = host.synthetic_norm_params(w["seed"])
    sin, cos = host.split_sin_cos(host.rotary_table(n * w["frames_per_chunk"], w["H"], w["W"]))
    q = mb.qk_norm_rope(xq, gq, bq, cos.to(dev), sin.to(dev))
    k = mb.qk_norm_rope(xk, gk, bk, cos.to(dev), sin.to(dev))
    qr, kr = host.q_ranges_for_chunks(n, C), host.default_k_ranges(n, C)

    def loop():
        return [flash_attn.flash_attn_func(q=q[None, a:b], k=k[None, c:d], v=xv[None, c:d]) for (a, b), (c, d) in zip(qr, kr)]
    loop()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(3):
        outs = loop()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / 3
    ours, _ = mb.chunk_attn(q, k, xv, qr, kr, C, S, return_lse=False)
    theirs = torch.cat([o[0] for o in outs])
    torch.cuda.synchronize()
    x, y = ours.double().flatten(), theirs.double().flatten()
    print(json.dumps({"ms": ms, "value": useful_flops(Hq, C, n) / (ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                      "cosine_vs_this_library": float((x @ y) / (x.norm() * y.norm())),
                      "max_abs_vs_this_library": float((ours.float() - theirs.float()).abs().max()),
                      "what": f"loop of flash_attn_func per range, flash-attn {flash_attn.__version__} (the reference pins 2.4.2), "
                              f"attention only, same prologued inputs, child process"}), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="cfg3", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-other-configs", action="store_true",
                    help="1 GPU: do not time the other BASELINE configurations (cfg1, cfg2, cfg4) after the main workload")
    ap.add_argument("--no-gpu-dispatch-baseline", action="store_true",
                    help="1 GPU: do not time the reference's flash_attn_func fallback loop in a child process")
    ap.add_argument("--exchange", default="fused", choices=["fused", "nccl"],
                    help="N > 1: Ulysses exchange fused into the kernels over peer memory, or NCCL all-to-all + copies")
    ap.add_argument("--modulate-only", type=int, default=0, metavar="ROWS",
                    help="time only the gated post-norm residual kernel on ROWS rows of the workload's hidden size and print its block")
    ap.add_argument("--projection-only", action="store_true",
                    help="time only the Q/K/V projection with the prologue in its epilogue at the workload's shape (--steps launches of each "
                         "form, back to back) and print its block")
    ap.add_argument("--flash-child", default=None, help=argparse.SUPPRESS)
    args = ap.parse_args()
    if args.flash_child:
        flash_child(args.flash_child)
        return
    w = WORKLOADS[args.workload]
    if args.modulate_only:
        torch.cuda.set_device(0)
        print(json.dumps(bench_modulate(torch.device("cuda", 0), args.modulate_only, w["hq"] * 128, w["n_chunks"], load_peaks())), flush=True)
        return
    if args.projection_only:
        torch.cuda.set_device(0)
        C_ = w["H"] * w["W"] * w["frames_per_chunk"]
        print(json.dumps(bench_qkv_projection(torch.device("cuda", 0), 0, w["n_chunks"] * C_, w["hq"] * 128, w["hq"], w["hkv"], load_peaks(), iters=args.steps)), flush=True)
        return
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, w, rank, world)
        return
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    if args.warmup < 3:
        args.warmup = 3
    torch.cuda.set_device(local_rank)
    bind_to_gpu_cpus(local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    r = run_ours(args, args.workload, rank, world, local_rank, args.steps, args.warmup, not args.no_e2e,
                 not args.no_cpu_baseline, dist)
    failed = False
    if rank == 0:
        peaks, cp, fused, C = r["peaks"], r["cp"], r["fused"], r["C"]
        achieved = r["achieved"]
        line = {
            "metric": "chunk_causal_attn_useful_tflops", "value": r["flops"] / (r["ms_per_step"] * 1e-3) / 1e12, "unit": "TFLOP/s",
            "n_gpus": cp, "steps": args.steps, "warmup": args.warmup, "ms_per_step": r["ms_per_step"], "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3" if r["fp8"] else "bf16", "data": "synthetic",
            "config": {"workload": w["name"], "chunk_tokens": C, "useful_tflop_per_step": r["flops"] / 1e12,
                       "parallelism": (f"ulysses-cp{cp}, exchange " + ("fused into kernels over peer memory" if fused else "NCCL all-to-all")) if cp > 1 else "single-gpu",
                       "l2": "inputs (>= 0.6 GB per step) exceed the 126 MB L2; no explicit flush",
                       "inputs": "every rank draws the full tensors from the one seed and keeps its sequence slice",
                       "step": "qk layernorm+rope prologue, attention" + (", head<->sequence exchange in/out" if cp > 1 else "")},
            "attn_ms": r["attn_ms"],
            "pct_of_bf16_burst_peak": 100 * achieved / peaks["bf16_burst"],
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_sustained"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["bf16_sustained"], "peak_kind": f"{peaks['src']} sustained cuBLAS bf16",
                         "frac_of_burst": achieved / peaks["bf16_burst"],
                         "traffic": (w["traffic_bytes"] / cp) if w.get("traffic_bytes") else None,
                         "kernel": "attn_fwd_fp8_kernel" if r["fp8"] else "attn_fwd_kernel",
                         "per_gpu_tflop_per_launch": r["per_gpu_flops"] / 1e12},
            "clocks": r["clocks"],
            "gpu_launches": r["launches"],
            "parity": r["parity"],
        }
        if "prologue_q" in r:
            line["prologue_q"] = r["prologue_q"]
        if r["fp8"]:
            line["roofline"]["fp8_peak_measured_tflops"] = r["fp8_peak"]
            line["roofline"]["frac_of_fp8_peak"] = achieved / r["fp8_peak"] if r["fp8_peak"] else None
        if r["cpu_b"]:
            line["cpu_baseline"] = r["cpu_b"]
        if r["e2e"]:
            line["e2e"] = r["e2e"]
        failed = not (r["parity"] and r["parity"]["ok"])
    r = None
    torch.cuda.empty_cache()
    if world == 1 and rank == 0 and not args.no_other_configs:
        C_ = w["H"] * w["W"] * w["frames_per_chunk"]
        line["post_attention_modulate"] = bench_modulate(torch.device("cuda", local_rank), w["n_chunks"] * C_, w["hq"] * 128,
                                                         w["n_chunks"], load_peaks())
        torch.cuda.empty_cache()
        line["fp8_linear_quantiser"] = bench_div_clamp(torch.device("cuda", local_rank), w["n_chunks"] * C_, w["hq"] * 128, load_peaks())
        torch.cuda.empty_cache()
        line["qkv_projection_prologue"] = bench_qkv_projection(torch.device("cuda", local_rank), local_rank, w["n_chunks"] * C_, w["hq"] * 128,
                                                               w["hq"], w["hkv"], load_peaks())
        torch.cuda.empty_cache()

    # ---- 1-GPU default run only: the other BASELINE configurations, a few steps each, and the reference's fallback
    # dispatch on this GPU (child process) - so that every configuration has a number on record beside the headline one
    if world == 1 and args.workload == "cfg3":
        if not args.no_other_configs:
            others = {}
            for name in ("cfg1", "cfg2", "cfg4"):
                o = run_ours(args, name, 0, 1, local_rank, 5, 3, False, False, None)
                d = {"workload": o["w"]["name"], "ms_per_step": o["ms_per_step"], "attn_ms": o["attn_ms"],
                     "tflops": o["flops"] / (o["ms_per_step"] * 1e-3) / 1e12, "attn_tflops": o["achieved"],
                     "frac_of_bf16_sustained": o["achieved"] / o["peaks"]["bf16_sustained"], "steps": 5, "warmup": 3,
                     "sm_mhz": o["clocks"]["sm_mhz"], "parity": o["parity"]}
                if name == "cfg2":
                    d["cache"] = "bf16 pages, 6 prefix chunks read in place"
                if name == "cfg4":
                    d["cache"] = "fp8 e4m3 pages for chunks 0-2"
                    d["fp8_peak_measured_tflops"] = o["fp8_peak"]
                    d["frac_of_fp8_peak"] = o["achieved"] / o["fp8_peak"] if o["fp8_peak"] else None
                    d["cosine_vs_bf16"] = o["parity"].get("cosine_vs_bf16_kernel_whole_output") if o["parity"] else None
                if "prologue_q" in o:
                    d["prologue_q_frac_of_hbm_peak"] = o["prologue_q"]["frac"]
                failed = failed or not (o["parity"] and o["parity"]["ok"])
                others[name] = d
                o = None
                torch.cuda.empty_cache()
            line["other_configs"] = others
        if not args.no_gpu_dispatch_baseline:
            try:
                cp_ = subprocess.run([sys.executable, os.path.abspath(__file__), "--flash-child", "cfg3"], capture_output=True,
                                     text=True, timeout=420)
                last = [ln for ln in cp_.stdout.splitlines() if ln.startswith("{")]
                line["gpu_reference_dispatch"] = json.loads(last[-1]) if last else {"unavailable": (cp_.stderr or "no output")[-200:]}
            except Exception as e:  # noqa: BLE001 - comparison leg only
                line["gpu_reference_dispatch"] = {"unavailable": str(e)[:200]}
    if rank == 0:
        print(json.dumps(line), flush=True)
    if world > 1:
        flag = torch.tensor([1.0 if failed else 0.0], device=torch.device("cuda", local_rank))
        dist.all_reduce(flag)
        failed = flag.item() > 0
        dist.barrier()
        dist.destroy_process_group()
    if failed:
        raise SystemExit("parity check failed: see the \"parity\" block of the JSON line")


if __name__ == "__main__":
    main()
