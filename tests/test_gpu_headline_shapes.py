"""Parity at the two configurations the headline numbers are quoted on: the 24B-style 720p layer (48 q heads, 8 kv heads,
4 chunks of 21600 tokens, block-causal; bf16) and its FP8 e4m3 variant with chunks 0-2 read from fp8 cache pages.

The oracle cannot run the whole 86400-token problem, so the bf16 output is checked on sampled rows (first / last row of
every chunk, the edges of the 128-row tiles and of the 256-row work items, the 96-token tail, random rows) and through
size-independent properties (block-causality bitwise, V == 1 gives exactly 1, bitwise run-to-run determinism); the FP8
output is compared with the bf16 output of the same seeded inputs over the whole tensor (cosine >= 0.999, the
acceptance bar of the FP8 variant) and on sampled rows against the oracle."""
import numpy as np
import pytest
import torch

from oracle import chunk_attn_oracle as O
from gpu_util import as_segments, assert_close, oracle_on_rows

pytestmark = pytest.mark.gpu

HQ, HKV, H, W, FRAMES, N_CHUNKS = 48, 8, 45, 80, 6, 4
C = H * W * FRAMES          # 21600 = 84 * 256 + 96 = 168 * 128 + 96
S = C * N_CHUNKS            # 86400
FP8_MIN_COS = 0.999


@pytest.fixture(scope="module")
def mb():
    import magi_b200
    return magi_b200


@pytest.fixture(scope="module")
def problem(mb):
    """Seeded N(0,1) projections -> the library's prologue (per-head LayerNorm(gamma+1, beta) + 3D RoPE) -> q, k; v as is;
    the bf16 attention output of the whole problem."""
    from magi_b200 import host
    assert C == 21600 and S == 86400
    g = torch.Generator(device="cuda").manual_seed(3)
    xq = torch.randn(S, HQ, 128, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    xk = torch.randn(S, HKV, 128, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    v = torch.randn(S, HKV, 128, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    gq, bq, gk, bk = host.synthetic_norm_params(3)
    sin, cos = host.split_sin_cos(host.rotary_table(N_CHUNKS * FRAMES, H, W))
    q = mb.qk_norm_rope(xq, gq, bq, cos.cuda(), sin.cuda())
    k = mb.qk_norm_rope(xk, gk, bk, cos.cuda(), sin.cuda())
    # the prologue at this shape, on sampled tokens, against the oracle (<= 1 bf16 ulp of values up to ~8)
    tok = torch.tensor([0, 1, 3599, 3600, C - 1, C, 2 * C + 77, S - 1])
    q_ref = O.qk_prologue(xq[tok.cuda()].cpu(), gq, bq, cos[tok], sin[tok])
    assert (q[tok.cuda()].cpu().float() - q_ref.float()).abs().max().item() <= 2 ** -4
    del xq, xk
    qr, kr = O.consecutive_q_ranges(N_CHUNKS, C), O.default_k_ranges(N_CHUNKS, C)
    out, lse = mb.chunk_attn(q, k, v, qr, kr, C, S)
    torch.cuda.synchronize()
    assert mb.Context.get().status() == 0
    return dict(q=q, k=k, v=v, qr=qr, kr=kr, out=out, lse=lse)


def _sample_rows(seed, n_random):
    edges = [0, 1, 127, 128, 255, 256, 257, C - 97, C - 96, C - 95, C - 1, C, C + 128, 2 * C - 1, 2 * C, 2 * C + 255,
             3 * C - 96, 3 * C, 3 * C + 21503, 3 * C + 21504, S - 97, S - 96, S - 2, S - 1]
    gen = torch.Generator().manual_seed(seed)
    return torch.cat([torch.tensor(edges), torch.randint(0, S, (n_random,), generator=gen)]).unique()


def test_cfg3_shape_sampled_rows_against_the_oracle(mb, problem):
    p = problem
    assert torch.isfinite(p["out"].float()).all()
    rows = _sample_rows(5, 24)
    keep, ref, ref_lse = oracle_on_rows(p["q"][rows.cuda()].float().cpu(), p["k"].float().cpu(), p["v"].float().cpu(),
                                        *_sub_problem(p["qr"], p["kr"], rows))
    assert_close(p["out"][rows.cuda()], ref, what="cfg3 sampled rows")
    assert torch.allclose(p["lse"][rows.cuda()].cpu(), ref_lse, atol=3e-3, rtol=1e-3)


def _sub_problem(qr, kr, rows):
    """Ranges of the gathered rows: row i of the sample sits at position i; one sub-range per chunk that has samples."""
    sub_q, sub_k, pos = [], [], 0
    for (qs, qe), kseg in zip(np.asarray(qr), as_segments(kr)):
        m = int(((rows >= qs) & (rows < qe)).sum())
        if m:
            sub_q.append([pos, pos + m])
            sub_k.append(kseg)
            pos += m
    return np.asarray(sub_q), sub_k, torch.arange(pos)


def test_cfg3_shape_properties(mb, problem):
    p = problem
    q, k, v, qr, kr, out = p["q"], p["k"], p["v"], p["qr"], p["kr"], p["out"]
    # bitwise run-to-run determinism
    again, _ = mb.chunk_attn(q, k, v, qr, kr, C, S, return_lse=False)
    torch.cuda.synchronize()
    assert torch.equal(again, out)
    del again
    # block-causality: changing K/V of chunk 3 must not change the outputs of chunks 0..2 (bitwise)
    k2, v2 = k.clone(), v.clone()
    k2[3 * C:] = 0
    v2[3 * C:] = 1
    out2, _ = mb.chunk_attn(q, k2, v2, qr, kr, C, S, return_lse=False)
    torch.cuda.synchronize()
    assert torch.equal(out[:3 * C], out2[:3 * C])
    assert not torch.equal(out[3 * C:], out2[3 * C:])
    del out2, k2
    # softmax rows are convex combinations: with V == 1 everywhere the output is 1
    v2.fill_(1)
    out3, _ = mb.chunk_attn(q, k, v2, qr, kr, C, S, return_lse=False)
    torch.cuda.synchronize()
    assert mb.Context.get().status() == 0
    assert (out3.float() - 1).abs().max().item() <= 2 ** -7


def test_cfg4_fp8_pages_against_the_bf16_output_of_the_same_inputs(mb, problem):
    p = problem
    q, k, v, qr, kr = p["q"], p["k"], p["v"], p["qr"], p["kr"]
    n = N_CHUNKS
    cache = mb.ChunkPagedKVCache(n_layers=1, max_chunks=n - 1, chunk_tokens=C, n_kv_heads=HKV, dtype="fp8")
    for pc in range(n - 1):
        cache.append(0, pc, k[pc * C:(pc + 1) * C], v[pc * C:(pc + 1) * C])
    q8, qs, q8lo = mb.quantize_e4m3(q, C, residual=True)
    k8, ks = mb.quantize_e4m3(k[(n - 1) * C:], C)
    v8, vs = mb.quantize_e4m3(v[(n - 1) * C:], C)
    assert qs.shape == (n * ((C + 127) // 128), HQ)
    out8, _ = mb.chunk_attn(q8, k8, v8, qr, kr, C, S, return_lse=False, cache=cache, layer=0,
                            prefix_chunk_ids=list(range(n - 1)), q_scale=qs, k_scale=ks, v_scale=vs,
                            scale_chunk_tokens=C, q_lo=q8lo)
    torch.cuda.synchronize()
    assert mb.Context.get().status() == 0
    assert torch.isfinite(out8.float()).all()
    # whole output against the bf16 kernel's, per chunk (fp64 accumulation on the device) and overall
    dots = []
    for c in range(n):
        a, b = out8[c * C:(c + 1) * C].double().flatten(), p["out"][c * C:(c + 1) * C].double().flatten()
        dots.append((float(a @ b), float(a @ a), float(b @ b)))
    per_chunk = [ab / (aa * bb) ** 0.5 for ab, aa, bb in dots]
    overall = sum(d[0] for d in dots) / (sum(d[1] for d in dots) * sum(d[2] for d in dots)) ** 0.5
    print(f"cfg4 fp8 vs cfg3 bf16 cosine: overall {overall:.5f}, per chunk {[round(c, 5) for c in per_chunk]}")
    assert overall >= FP8_MIN_COS and min(per_chunk) >= FP8_MIN_COS
    # sampled rows against the fp32 oracle on the unquantised inputs
    rows = _sample_rows(6, 8)
    keep, ref, _ = oracle_on_rows(q[rows.cuda()].float().cpu(), k.float().cpu(), v.float().cpu(), *_sub_problem(qr, kr, rows))
    cos = O.cosine(out8[rows.cuda()].cpu(), ref)
    assert cos >= FP8_MIN_COS, cos
    cache.close()
