"""Benchmark of the chunk-causal attention hot path (prologue -> [Ulysses in] -> attention -> [Ulysses out]).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload cfg3|cfg1|cfg2|cfg4] [--exchange fused|nccl]
                    [--impl ours|reference] [--no-e2e] [--no-cpu-baseline] [--gpu-dispatch-baseline]

One process per GPU (under torchrun for N > 1; RANK / LOCAL_RANK / WORLD_SIZE / MASTER_* from the environment).
Rank 0 prints ONE JSON line.  A "step" is one pass of the hot path over one batch of seeded synthetic inputs of
the named configuration: per-head LayerNorm + 3D RoPE of Q and K, (for N > 1: head<->sequence all-to-all in),
block-causal attention, (all-to-all out).  `value` = useful (unmasked) attention FLOPs of the whole job / step time.
"""
import argparse
import json
import math
import os
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


CPU_SAMPLE_ROWS = 4096  # q rows per chunk range in the CPU baseline sample (about 10 s of host work at cfg3)


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
    except Exception as e:  # pragma: no cover
        return None


def load_peaks():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            p = json.load(f)
        return dict(bf16_burst=p["bf16_tflops"], bf16_sustained=p["bf16_tflops_sustained"], hbm=p["hbm_gbs"], src="measured")
    except Exception:
        return dict(bf16_burst=1590.0, bf16_sustained=1400.0, hbm=6650.0, src="fallback")


class ClockSampler(threading.Thread):
    """Samples SM clock and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index):
        super().__init__(daemon=True)
        self.index, self.samples, self.reasons, self.stop_flag, self.max_mhz = index, [], set(), False, None

    def run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            h = nv.nvmlDeviceGetHandleByIndex(self.index)
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


# ------------------------------------------------------------------------------------------------ our arm
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--workload", default="cfg3", choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--gpu-dispatch-baseline", action="store_true",
                    help="also time the reference's flash_attn_func fallback loop on this GPU (comparison only; loads flash-attn)")
    ap.add_argument("--exchange", default="fused", choices=["fused", "nccl"],
                    help="N > 1: Ulysses exchange fused into the kernels over peer memory, or NCCL all-to-all + copies")
    args = ap.parse_args()
    w = WORKLOADS[args.workload]
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

    import magi_b200 as mb
    from magi_b200 import host
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    cp = world
    if cp > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=dev)
    Hq, Hkv = w["hq"], w["hkv"]
    C = w["H"] * w["W"] * w["frames_per_chunk"]
    n = w["n_chunks"]
    S = n * C
    flops = useful_flops(Hq, C, n)
    peaks = load_peaks()

    # ---- synthetic inputs (seeded); every rank generates its own sequence slice of the pre-norm projections
    splits = host.cp_split_sizes(S, cp)
    off = sum(splits[:rank])
    s_loc = splits[rank]
    g = torch.Generator(device=dev).manual_seed(w["seed"] * 1000 + rank)
    xq = torch.randn(s_loc, Hq, 128, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    xk = torch.randn(s_loc, Hkv, 128, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    xv = torch.randn(s_loc, Hkv, 128, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16)
    gq, bq, gk, bk = [t.to(dev) for t in host.synthetic_norm_params(w["seed"])]
    sin, cos = host.split_sin_cos(host.rotary_table(n * w["frames_per_chunk"], w["H"], w["W"]))
    sin, cos = sin[off:off + s_loc].contiguous().to(dev), cos[off:off + s_loc].contiguous().to(dev)
    qr = torch.as_tensor(host.q_ranges_for_chunks(n, C), device=dev)
    kr = torch.as_tensor(host.default_k_ranges(n, C), device=dev)

    if w.get("decode") and cp > 1:
        raise SystemExit(f"workload {args.workload} is a single-GPU benchmark line")
    fused = cp > 1 and args.exchange == "fused" and not w.get("fp8")
    if cp > 1:
        from magi_b200.ulysses import FusedUlyssesAttention, UlyssesAttention
        ua = FusedUlyssesAttention(dist.group.WORLD, Hq, Hkv, splits) if fused else \
            UlyssesAttention(cp_group=dist.group.WORLD, n_q_heads=Hq, n_kv_heads=Hkv, split_sizes=splits)
    attn_ev, prologue_ev = [], []
    n_launch = [0]

    def timed_attn(record, fn):
        if record:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        r = fn()
        if record:
            e1.record()
            attn_ev.append((e0, e1))
        return r

    if w.get("decode"):
        # ---- cfg 2: b x n denoising chunks; the clean prefix chunks live in the paged cache (filled outside the timed region)
        B, NP = w["batch"], w["n_prefix"]
        flops = B * flops
        g2 = torch.Generator(device=dev).manual_seed(w["seed"] * 1000 + 7)
        xq = torch.randn(B * S, Hq, 128, generator=g2, device=dev, dtype=torch.float32).to(torch.bfloat16)
        xk = torch.randn(B * S, Hkv, 128, generator=g2, device=dev, dtype=torch.float32).to(torch.bfloat16)
        xv = torch.randn(B * S, Hkv, 128, generator=g2, device=dev, dtype=torch.float32).to(torch.bfloat16)
        cache = mb.ChunkPagedKVCache(n_layers=1, max_chunks=B * NP, chunk_tokens=C, n_kv_heads=Hkv, device=local_rank)
        for pc in range(B * NP):
            kvp = torch.randn(C, Hkv, 256, generator=g2, device=dev, dtype=torch.float32).to(torch.bfloat16)
            cache.append_kv(0, pc, kvp)
        sin_b, cos_b = sin.repeat(B, 1), cos.repeat(B, 1)
        qr = torch.as_tensor(host.q_ranges_for_chunks(n, C, batch=B), device=dev)
        kr_np, ko_np = host.own_prefix_k_segments(n, C, NP, batch=B)
        kr, ko = torch.as_tensor(kr_np, device=dev), torch.as_tensor(ko_np, device=dev)
        q_buf, k_buf, out_buf = torch.empty_like(xq), torch.empty_like(xk), torch.empty_like(xq)
        s_loc = B * S

        def step(record=False):
            mb.qk_norm_rope(xq, gq, bq, cos_b, sin_b, out=q_buf)
            mb.qk_norm_rope(xk, gk, bk, cos_b, sin_b, out=k_buf)
            timed_attn(record, lambda: mb.chunk_attn(q_buf, k_buf, xv, qr, kr, C, (NP + 1) * C, k_range_offsets=ko, out=out_buf,
                                                     return_lse=False, cache=cache, layer=0, prefix_chunk_ids=list(range(B * NP))))
            n_launch[0] = 4
            return out_buf
    elif w.get("fp8") and cp == 1:
        # ---- cfg 4: fp8; K/V of chunks 0..n-2 sit in an fp8 page cache, the last chunk is fresh
        cache = mb.ChunkPagedKVCache(n_layers=1, max_chunks=n - 1, chunk_tokens=C, n_kv_heads=Hkv, dtype="fp8", device=local_rank)
        k_all = mb.qk_norm_rope(xk, gk, bk, cos, sin)
        for pc in range(n - 1):
            cache.append(0, pc, k_all[pc * C:(pc + 1) * C], xv[pc * C:(pc + 1) * C])
        del k_all
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
                                                     prefix_chunk_ids=list(range(n - 1)), q_scale=qs, k_scale=ks, v_scale=vs,
                                                     scale_chunk_tokens=C, q_lo=q8lo))
            n_launch[0] = 7
            return out_buf
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
                n_launch[0] = 4
                return out_buf
            n_launch[0] = 11 if w.get("fp8") else (5 if fused else 7)
            if fused:
                return ua.forward(xq, xk, xv, gq, bq, gk, bk, cos, sin, qr, kr, C, S, attn_events=attn_ev if record else None)
            # FP8 under context parallelism: all chunks are fresh (the head-sharded Q/K/V are quantised after the exchange)
            return ua.forward(xq, xk, xv, gq, bq, gk, bk, cos, sin, qr, kr, C, S, attn_events=attn_ev if record else None,
                              fp8_chunk_tokens=C if w.get("fp8") else 0)

    def barrier():
        if cp > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        step()
    barrier()
    assert mb.Context.get(local_rank).status() == 0, "device status word reports a failure during warm-up"
    sampler = ClockSampler(local_rank)
    sampler.start()
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    t0.record()
    for _ in range(args.steps):
        step(record=True)
    t1.record()
    barrier()
    sampler.stop_flag = True
    ms = t0.elapsed_time(t1)
    attn_ms = sum(a.elapsed_time(b) for a, b in attn_ev) / max(1, len(attn_ev))
    if cp > 1:
        tt = torch.tensor([ms, attn_ms], device=dev, dtype=torch.float64)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms, attn_ms = tt.tolist()
    ms_per_step = ms / args.steps
    sampler.join(timeout=1.0)

    # ---- end to end through the public API with host buffers (H2D of the step's inputs, D2H of its output)
    e2e = None
    if not args.no_e2e:
        hq_, hk_, hv_ = xq.cpu().pin_memory(), xk.cpu().pin_memory(), xv.cpu().pin_memory()
        ho = torch.empty(out_buf.shape[0] if cp == 1 else s_loc, Hq, 128, dtype=torch.bfloat16).pin_memory()

        # The user-level pipeline: step i+1's inputs are copied host->device on a copy stream while step i computes, and
        # step i's output goes device->host on a third stream (double-buffered device inputs; double-buffered output on
        # one GPU).  Every step still moves all of its inputs and its whole output across PCIe inside the timed region.
        pipelined = not w.get("fp8") and not w.get("decode")
        main_s = torch.cuda.current_stream()
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        in_bufs = [(xq, xk, xv)] + ([(torch.empty_like(xq), torch.empty_like(xk), torch.empty_like(xv))] if pipelined else [])
        out_bufs = [out_buf] + ([torch.empty_like(out_buf)] if pipelined and cp == 1 else []) if cp == 1 else [None]
        ev_in = [torch.cuda.Event() for _ in in_bufs]
        ev_free = [torch.cuda.Event() for _ in in_bufs]
        ev_out = [torch.cuda.Event() for _ in out_bufs]
        counter = [0]

        def e2e_step():
            nonlocal xq, xk, xv, out_buf
            i = counter[0]
            counter[0] += 1
            if not pipelined:
                xq.copy_(hq_, non_blocking=True)
                xk.copy_(hk_, non_blocking=True)
                xv.copy_(hv_, non_blocking=True)
                ho.copy_(step(), non_blocking=True)
                return
            bi, bo = i % len(in_bufs), i % len(out_bufs)
            with torch.cuda.stream(s_in):
                if i >= len(in_bufs):
                    s_in.wait_event(ev_free[bi])       # the step that last read these buffers has finished
                for dst, src in zip(in_bufs[bi], (hq_, hk_, hv_)):
                    dst.copy_(src, non_blocking=True)
                ev_in[bi].record(s_in)
            main_s.wait_event(ev_in[bi])
            if i >= len(out_bufs):
                main_s.wait_event(ev_out[bo])          # the previous device->host copy out of this output buffer is done
            xq, xk, xv = in_bufs[bi]
            if cp == 1:
                out_buf = out_bufs[bo]
            o = step()
            ev_free[bi].record(main_s)
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_free[bi])
                ho.copy_(o, non_blocking=True)
                ev_out[bo].record(s_out)

        def e2e_drain():
            main_s.wait_stream(s_in)
            main_s.wait_stream(s_out)

        for _ in range(2):
            e2e_step()
        e2e_drain()
        barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        k_e2e = max(4, args.steps)
        a.record()
        for _ in range(k_e2e):
            e2e_step()
        e2e_drain()
        b.record()
        barrier()
        e_ms = a.elapsed_time(b)
        if cp > 1:
            tt = torch.tensor([e_ms], device=dev, dtype=torch.float64)
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            e_ms = tt.item()
        h2d = (hq_.numel() + hk_.numel() + hv_.numel()) * 2
        e2e = {"value": flops / (e_ms / k_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": e_ms / k_e2e,
               "h2d_bytes_per_step": h2d * cp, "d2h_bytes_per_step": ho.numel() * 2 * cp,
               "pipeline": "copies overlapped with the neighbouring steps on side streams" if pipelined else "sequential"}

    # ---- secondary baseline, on request and for comparison only: the reference's fallback dispatch on this GPU, a loop
    # of flash_attn_func over the ranges (inference/model/dit/dit_module.py:1049-1065) with the flash-attn build of the
    # image, on the same prologued Q/K and V, after all of this build's own timing is done.  Never a dispatch target of
    # the library; flash-attn is not even imported unless the flag is given.
    gpu_dispatch = None
    if cp == 1 and args.gpu_dispatch_baseline and not w.get("fp8") and not w.get("decode"):
        try:
            import flash_attn
            qr_h, kr_h = qr.cpu().numpy(), kr.cpu().numpy()

            def dispatch_loop():
                return [flash_attn.flash_attn_func(q=q_buf[None, a:b], k=k_buf[None, c:d], v=xv[None, c:d])
                        for (a, b), (c, d) in zip(qr_h, kr_h)]
            dispatch_loop()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(3):
                dispatch_loop()
            b.record()
            torch.cuda.synchronize()
            d_ms = a.elapsed_time(b) / 3
            gpu_dispatch = {"ms": d_ms, "value": flops / (d_ms * 1e-3) / 1e12, "unit": "TFLOP/s",
                            "what": f"loop of flash_attn_func per range, flash-attn {flash_attn.__version__} (reference pins 2.4.2), attention only"}
        except Exception as e:  # noqa: BLE001 - comparison leg only
            gpu_dispatch = {"unavailable": str(e)[:160]}

    if rank == 0:
        cpu_b = None
        if cp == 1 and not args.no_cpu_baseline:
            threads = os.cpu_count() or 1
            cpu_attention_sample(w, 16, threads)
            f, t = cpu_attention_sample(w, CPU_SAMPLE_ROWS, threads)
            cpu_b = {"value": f / t / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": "port", "seconds": t,
                     "sample": f"1 of {Hkv} KV-head groups, {CPU_SAMPLE_ROWS} q rows of each of the {n} chunk ranges vs their full key ranges, fp32 eager torch"}
        per_gpu_flops = flops / cp
        achieved = per_gpu_flops / (attn_ms * 1e-3) / 1e12
        line = {
            "metric": "chunk_causal_attn_useful_tflops", "value": flops / (ms_per_step * 1e-3) / 1e12, "unit": "TFLOP/s",
            "n_gpus": cp, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "fp8_e4m3" if w.get("fp8") else "bf16", "data": "synthetic",
            "config": {"workload": w["name"], "chunk_tokens": C, "useful_tflop_per_step": flops / 1e12,
                       "parallelism": (f"ulysses-cp{cp}, exchange " + ("fused into kernels over peer memory" if fused else "NCCL all-to-all")) if cp > 1 else "single-gpu",
                       "l2": "inputs (>= 0.6 GB per step) exceed the 126 MB L2; no explicit flush",
                       "step": "qk layernorm+rope prologue, attention" + (", all-to-all in/out" if cp > 1 else "")},
            "attn_ms": attn_ms,
            "pct_of_bf16_burst_peak": 100 * achieved / peaks["bf16_burst"],
            "roofline": {"bound": "tensor", "achieved": achieved, "peak": peaks["bf16_sustained"], "unit": "TFLOP/s",
                         "frac": achieved / peaks["bf16_sustained"], "peak_kind": f"{peaks['src']} sustained cuBLAS bf16",
                         "frac_of_burst": achieved / peaks["bf16_burst"],
                         "traffic": (w["traffic_bytes"] / cp) if w.get("traffic_bytes") else None,
                         "kernel": "attn_fwd_kernel", "per_gpu_tflop_per_launch": per_gpu_flops / 1e12},
            "clocks": sampler.summary(),
            "gpu_launches": args.steps * n_launch[0],
        }
        if prologue_ev:
            pms = sum(a.elapsed_time(b) for a, b in prologue_ev) / len(prologue_ev)
            pbytes = 2 * xq.numel() * 2 + 2 * cos.numel() * 4  # bf16 read + bf16 write of Q, cos+sin once
            line["prologue_q"] = {"kernel": "prologue16_kernel", "bound": "hbm", "ms": pms, "algorithmic_bytes": pbytes,
                                  "achieved_gbs": pbytes / (pms * 1e-3) / 1e9, "peak_gbs": peaks["hbm"],
                                  "frac": pbytes / (pms * 1e-3) / 1e9 / peaks["hbm"]}
        if w.get("fp8"):
            fp8_peak = measure_fp8_peak(dev)
            line["roofline"]["fp8_peak_measured_tflops"] = fp8_peak
            line["roofline"]["frac_of_fp8_peak"] = achieved / fp8_peak if fp8_peak else None
        if cpu_b:
            line["cpu_baseline"] = cpu_b
        if e2e:
            line["e2e"] = e2e
        if gpu_dispatch:
            line["gpu_reference_dispatch"] = gpu_dispatch
        print(json.dumps(line), flush=True)
    if cp > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
