"""Parity of the sm_100a attention forward (through the C ABI) against the CPU oracle."""
import math
import os

import numpy as np
import pytest
import torch

from oracle import chunk_attn_oracle as O
from gpu_util import as_segments, assert_close, oracle_on_rows

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mb():
    import magi_b200
    return magi_b200


def _dev(*ts):
    return [t.to(torch.bfloat16).cuda() for t in ts]


def _run(mb, q, k, v, qr, kr, max_q, offsets=None, impl="tcgen05", scale=None):
    qd, kd, vd = _dev(q, k, v)
    out, lse = mb.chunk_attn(qd, kd, vd, qr, kr, max_q, 0, softmax_scale=scale, k_range_offsets=offsets, impl=impl)
    torch.cuda.synchronize()
    assert mb.Context.get().status() == 0
    return out, lse, (qd.float().cpu(), kd.float().cpu(), vd.float().cpu())


def test_cfg0_matches_oracle_and_golden(mb, golden_dir):
    q, k, v = O.make_qkv(0, 384, 8, 2, scale=1 / math.sqrt(128))
    qr, kr = O.consecutive_q_ranges(3, 128), O.default_k_ranges(3, 128)
    out, lse, (qb, kb, vb) = _run(mb, q, k, v, qr, kr, 128)
    ref, ref_lse = O.range_attention(qb, kb, vb, qr, as_segments(kr))
    assert_close(out, ref, what="cfg0 vs oracle")
    assert torch.allclose(lse.cpu(), ref_lse, atol=2e-3, rtol=1e-3)
    gold = torch.from_numpy(np.load(os.path.join(golden_dir, "attn_cfg0.npz"))["out"])
    assert_close(out, gold, what="cfg0 vs SDPA fixture (fp32 inputs)")


@pytest.mark.parametrize("impl", ["tcgen05", "simt"])
@pytest.mark.parametrize("hq,hkv", [(1, 1), (3, 1), (8, 2), (6, 6), (24, 8)])
def test_ragged_rectangles(mb, impl, hq, hkv):
    g = torch.Generator().manual_seed(hq * 10 + hkv)
    Tq, Tk = 1000, 1500
    q = torch.randn(Tq, hq, 128, generator=g)
    k = torch.randn(Tk, hkv, 128, generator=g)
    v = torch.randn(Tk, hkv, 128, generator=g)
    # lengths that are not multiples of 128/256, a gap in q (rows 700..749), windows with k-start > 0, Lq != Lk
    qr = np.array([[0, 1], [1, 130], [130, 517], [517, 700], [750, 1000]], dtype=np.int32)
    kr = np.array([[0, 1500], [7, 8], [100, 1399], [0, 129], [256, 1281]], dtype=np.int32)
    out, lse, (qb, kb, vb) = _run(mb, q, k, v, qr, kr, 387, impl=impl)
    ref, ref_lse = O.range_attention(qb, kb, vb, qr, as_segments(kr))
    rows = torch.cat([torch.arange(a, b) for a, b in qr])
    assert_close(out[rows.cuda()], ref[rows], what=f"ragged {impl} {hq}/{hkv}")
    assert torch.allclose(lse.cpu()[rows], ref_lse[rows], atol=3e-3, rtol=1e-3)


def test_rows_outside_every_range_are_untouched(mb):
    q, k, v = O.make_qkv(5, 600, 4, 2)
    qd, kd, vd = _dev(q, k, v)
    out = torch.full((600, 4, 128), 7.0, dtype=torch.bfloat16, device="cuda")
    qr = np.array([[10, 300], [320, 590]], dtype=np.int32)
    kr = np.array([[0, 300], [0, 600]], dtype=np.int32)
    mb.chunk_attn(qd, kd, vd, qr, kr, 290, 600, out=out)
    torch.cuda.synchronize()
    o = out.float().cpu()
    for a, b in ((0, 10), (300, 320), (590, 600)):
        assert (o[a:b] == 7.0).all()
    ref, _ = O.range_attention(qd.float().cpu(), kd.float().cpu(), vd.float().cpu(), qr, as_segments(kr))
    assert_close(out[10:300], ref[10:300])


def test_multiple_k_intervals_per_q_range(mb):
    """Own cached prefix + own chunk for concurrently denoising chunks: non-contiguous k per q-range."""
    g = torch.Generator().manual_seed(17)
    C, n = 200, 3
    q = torch.randn(n * C, 6, 128, generator=g)
    k = torch.randn(6 * C, 2, 128, generator=g)
    v = torch.randn(6 * C, 2, 128, generator=g)
    qr = O.consecutive_q_ranges(n, C)
    kr = np.array([[3 * C, 4 * C], [0, C], [4 * C, 5 * C], [0, 2 * C], [5 * C, 6 * C]], dtype=np.int32)
    offs = np.array([0, 1, 3, 5], dtype=np.int32)
    out, lse, (qb, kb, vb) = _run(mb, q, k, v, qr, kr, C, offsets=offs)
    ref, _ = O.range_attention(qb, kb, vb, qr, as_segments(kr, offs))
    assert_close(out, ref, what="multi-interval")
    out2, _, _ = _run(mb, q, k, v, qr, kr, C, offsets=offs, impl="simt")
    assert_close(out2, ref, what="multi-interval simt")


def test_fused_kv_layout_and_custom_scale(mb):
    """K and V as the two halves of the reference's [tokens, Hkv, 256] buffer (strided views), scale given."""
    g = torch.Generator().manual_seed(23)
    T = 777
    q = torch.randn(T, 4, 128, generator=g).to(torch.bfloat16).cuda()
    kv = torch.randn(T, 2, 256, generator=g).to(torch.bfloat16).cuda()
    k, v = kv[..., :128], kv[..., 128:]
    qr = np.array([[0, 400], [400, 777]], dtype=np.int32)
    kr = np.array([[0, 400], [0, 777]], dtype=np.int32)
    out, lse = mb.chunk_attn(q, k, v, qr, kr, 400, 777, softmax_scale=0.05)
    torch.cuda.synchronize()
    ref, _ = O.range_attention(q.float().cpu(), k.float().cpu(), v.float().cpu(), qr, as_segments(kr), softmax_scale=0.05)
    assert_close(out, ref, what="fused kv")


def test_flex_attn_surface_and_batched_ranges(mb):
    """The reference's call shape with b = 2: q flattened (b sq), ranges [n*b, 2] (dit_module.py:1032-1043)."""
    g = torch.Generator().manual_seed(29)
    C, n, b = 160, 2, 2
    q = torch.randn(b * n * C, 6, 128, generator=g).to(torch.bfloat16).cuda()
    k = torch.randn(b * n * C, 2, 128, generator=g).to(torch.bfloat16).cuda()
    v = torch.randn(b * n * C, 2, 128, generator=g).to(torch.bfloat16).cuda()
    qr = torch.tensor([[i * C, (i + 1) * C] for i in range(b * n)], dtype=torch.int32, device="cuda")
    kr = torch.tensor([[e * n * C, e * n * C + (j + 1) * C] for e in range(b) for j in range(n)], dtype=torch.int32, device="cuda")
    out, lse = mb.flex_attn(q, k, v, qr, kr, max_seqlen_q=C, max_seqlen_k=n * C, softmax_scale=None,
                            deterministic=True, disable_fwd_atomic_reduction=True)
    torch.cuda.synchronize()
    ref, _ = O.range_attention(q.float().cpu(), k.float().cpu(), v.float().cpu(), qr.cpu().numpy(), as_segments(kr.cpu().numpy()))
    assert_close(out, ref, what="flex surface")


def test_run_to_run_determinism(mb):
    q, k, v = O.make_qkv(31, 900, 6, 2)
    qd, kd, vd = _dev(q, k, v)
    qr, kr = O.consecutive_q_ranges(3, 300), O.default_k_ranges(3, 300)
    a, _ = mb.chunk_attn(qd, kd, vd, qr, kr, 300, 900)
    b, _ = mb.chunk_attn(qd, kd, vd, qr, kr, 300, 900)
    torch.cuda.synchronize()
    assert torch.equal(a, b)


def test_argument_errors_are_reported_not_computed(mb):
    q = torch.zeros(256, 4, 128, dtype=torch.bfloat16, device="cuda")
    k = torch.zeros(256, 2, 128, dtype=torch.bfloat16, device="cuda")
    qr = np.array([[0, 256]], dtype=np.int32)
    with pytest.raises(mb.MagiError) as e:  # Hq not a multiple of Hkv
        mb.chunk_attn(q[:, :3], k, k, qr, qr, 256)
    assert e.value.code == mb._lib.E_BADARG
    with pytest.raises(mb.MagiError) as e:  # misaligned base pointer (offset by 4 elements = 8 bytes)
        flat = torch.zeros(256 * 4 * 128 + 8, dtype=torch.bfloat16, device="cuda")
        mb.chunk_attn(flat[4:4 + 256 * 4 * 128].view(256, 4, 128), k, k, qr, qr, 256)
    assert e.value.code == mb._lib.E_ALIGN
    # inconsistent ranges are caught by the device planner and surface through the status word; nothing is computed
    out = torch.full((256, 4, 128), 3.0, dtype=torch.bfloat16, device="cuda")
    bad = np.array([[0, 999]], dtype=np.int32)
    mb.chunk_attn(q, k, k, qr, bad, 256, out=out)
    assert mb.Context.get().status() == mb._lib.E_RANGE
    assert (out.float() == 3.0).all()
    assert mb.Context.get().status() == 0  # cleared
    ok, _ = mb.chunk_attn(q, k, k, qr, qr, 256)
    torch.cuda.synchronize()
    assert mb.Context.get().status() == 0 and torch.isfinite(ok.float()).all()


def test_large_magnitude_scores_stay_finite(mb):
    """Scores far from zero and a late-arriving maximum exercise the lazy-rescale branch."""
    g = torch.Generator().manual_seed(37)
    T = 700
    q = torch.randn(T, 2, 128, generator=g) * 4
    k = torch.randn(T, 2, 128, generator=g) * 4
    k[650:] *= 3  # the largest scores come in the last tile
    v = torch.randn(T, 2, 128, generator=g)
    qr = np.array([[0, T]], dtype=np.int32)
    out, lse, (qb, kb, vb) = _run(mb, q, k, v, qr, qr, T)
    ref, ref_lse = O.range_attention(qb, kb, vb, qr, as_segments(qr))
    assert_close(out, ref, what="large scores")
    assert torch.allclose(lse.cpu(), ref_lse, atol=5e-2, rtol=1e-3)


@pytest.mark.parametrize("n_seq", [257, 1024])
def test_varlen_batch_of_many_ranges(mb, n_seq):
    """Hundreds of short sequences in one call (cu_seqlens style): the planner works one thread per range - prefix sums
    for the segment and work-item lists, a rank sort for longest-K-first - and must agree with the per-range oracle,
    empty key ranges included."""
    rng = np.random.default_rng(n_seq)
    lq = rng.integers(1, 90, size=n_seq)
    lk = rng.integers(0, 200, size=n_seq)
    lk[rng.integers(0, n_seq, size=n_seq // 16)] = 0           # some sequences have no keys at all
    cq = np.concatenate([[0], np.cumsum(lq)])
    ck = np.concatenate([[0], np.cumsum(lk)])
    qr = np.stack([cq[:-1], cq[1:]], 1).astype(np.int32)
    kr = np.stack([ck[:-1], ck[1:]], 1).astype(np.int32)
    g = torch.Generator().manual_seed(n_seq)
    q = torch.randn(int(cq[-1]), 4, 128, generator=g)
    k = torch.randn(int(ck[-1]), 2, 128, generator=g)
    v = torch.randn(int(ck[-1]), 2, 128, generator=g)
    out, lse, (qb, kb, vb) = _run(mb, q, k, v, qr, kr, int(lq.max()))
    ref, ref_lse = O.range_attention(qb, kb, vb, qr, as_segments(kr))
    assert_close(out, ref, what=f"{n_seq} ranges")
    live = torch.cat([torch.arange(a, b) for (a, b), n in zip(qr, lk) if n > 0])
    assert torch.allclose(lse.cpu()[live], ref_lse[live], atol=3e-3, rtol=1e-3)
    dead = torch.cat([torch.arange(a, b) for (a, b), n in zip(qr, lk) if n == 0])
    assert (out.cpu()[dead].float() == 0).all() and torch.isinf(lse.cpu()[dead]).all()


@pytest.mark.parametrize("step", [0.5, 2.0, 9.0, 40.0])
def test_reference_maximum_keeps_growing_tile_after_tile(mb, step):
    """Keys whose scores climb by about `step` (in log2 units of the softmax weights) from one 128-token tile to the
    next: below the redo threshold the stale reference carries weights far above 1 for many tiles, above it every tile
    is redone and O rescaled, and the largest step moves the reference by more than fp32 can hold in one weight."""
    g = torch.Generator().manual_seed(41)
    T, n_tiles = 128 * 12, 12
    q = torch.randn(T, 2, 128, generator=g)
    k = torch.randn(T, 2, 128, generator=g)
    v = torch.randn(T, 2, 128, generator=g)
    # add a component along a fixed direction u to q and, growing with the tile index, to k: q.k gains ~ |u|^2 a_q a_k(tile)
    u = torch.randn(128, generator=g)
    u = u / u.norm()
    q = q + 8.0 * u
    scale_log2 = 1.4426950408889634 / 128 ** 0.5
    ramp = torch.arange(n_tiles).repeat_interleave(128).float() * (step / (8.0 * scale_log2))
    k = k + ramp[:, None, None] * u
    qr = np.array([[0, T]], dtype=np.int32)
    out, lse, (qb, kb, vb) = _run(mb, q, k, v, qr, qr, T)
    ref, ref_lse = O.range_attention(qb, kb, vb, qr, as_segments(qr))
    assert torch.isfinite(out.float()).all()
    assert_close(out, ref, what=f"growing maximum, step {step}")
    assert torch.allclose(lse.cpu(), ref_lse, atol=5e-2, rtol=1e-3)


def test_cfg1_shape_sampled_rows_and_properties(mb):
    """The 4.5B-style single-GPU benchmark shape: 24/8 heads, 4 chunks of 9360 tokens, block-causal."""
    C, n, Hq, Hkv = 9360, 4, 24, 8
    g = torch.Generator(device="cuda").manual_seed(1)
    S = C * n
    q = torch.randn(S, Hq, 128, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    k = torch.randn(S, Hkv, 128, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    v = torch.randn(S, Hkv, 128, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    qr, kr = O.consecutive_q_ranges(n, C), O.default_k_ranges(n, C)
    out, lse = mb.chunk_attn(q, k, v, qr, kr, C, S)
    torch.cuda.synchronize()
    assert mb.Context.get().status() == 0
    assert torch.isfinite(out.float()).all()
    # (1) sampled rows against the oracle: first/last rows of every chunk, tile edges, random rows
    gen = torch.Generator().manual_seed(2)
    rows = torch.cat([torch.tensor([0, 1, 127, 128, 255, 256, C - 1, C, C + 255, 2 * C - 1, 2 * C, 3 * C, S - 1, S - 16, S - 17]),
                      torch.randint(0, S, (33,), generator=gen)]).unique()
    keep, ref, ref_lse = oracle_on_rows(q.float().cpu(), k.float().cpu(), v.float().cpu(), qr, as_segments(kr), rows)
    assert_close(out[keep.cuda()], ref, what="cfg1 sampled rows")
    assert torch.allclose(lse[keep.cuda()].cpu(), ref_lse, atol=3e-3, rtol=1e-3)
    # (2) block-causality: changing K/V of chunk 3 must not change the outputs of chunks 0..2 (bitwise)
    k2, v2 = k.clone(), v.clone()
    k2[3 * C:] = 0
    v2[3 * C:] = 1
    out2, _ = mb.chunk_attn(q, k2, v2, qr, kr, C, S)
    torch.cuda.synchronize()
    assert torch.equal(out[:3 * C], out2[:3 * C])
    assert not torch.equal(out[3 * C:], out2[3 * C:])
    # (3) softmax rows are convex combinations: with V == 1 everywhere the output is exactly 1
    ones = torch.ones_like(v)
    out3, _ = mb.chunk_attn(q, k, ones, qr, kr, C, S)
    torch.cuda.synchronize()
    assert (out3.float() - 1).abs().max().item() <= 2 ** -7


def test_cfg2_shape_paged_decode_sampled_rows(mb):
    """The KV-cache decode benchmark shape: batch 2 x 4 denoising chunks of 9360 tokens, 24/8 heads; chunk i of batch
    element e attends to its own cached clean prefix (i chunks, read in place from bf16 pages) plus itself."""
    from magi_b200 import host
    C, n, B, NP, Hq, Hkv = 9360, 4, 2, 3, 24, 8
    g = torch.Generator(device="cuda").manual_seed(2)
    q = torch.randn(B * n * C, Hq, 128, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    k = torch.randn(B * n * C, Hkv, 128, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    v = torch.randn(B * n * C, Hkv, 128, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16)
    pages = [torch.randn(C, Hkv, 256, generator=g, device="cuda", dtype=torch.float32).to(torch.bfloat16) for _ in range(B * NP)]
    cache = mb.ChunkPagedKVCache(n_layers=1, max_chunks=B * NP, chunk_tokens=C, n_kv_heads=Hkv)
    order = [4, 0, 5, 2, 1, 3]                       # pages filled out of order: slot != chunk id
    for cid in order:
        cache.append_kv(0, cid, pages[cid])
    qr = host.q_ranges_for_chunks(n, C, batch=B)
    kr, ko = host.own_prefix_k_segments(n, C, NP, batch=B)
    out, lse = mb.chunk_attn(q, k, v, qr, kr, C, (NP + 1) * C, k_range_offsets=ko, cache=cache, layer=0,
                             prefix_chunk_ids=list(range(B * NP)))
    torch.cuda.synchronize()
    assert mb.Context.get().status() == 0
    # oracle on sampled rows over the materialised (prefix | current) key space
    kv_all = torch.cat(pages).float().cpu()
    k_virt = torch.cat([kv_all[..., :128], k.float().cpu()])
    v_virt = torch.cat([kv_all[..., 128:], v.float().cpu()])
    gen = torch.Generator().manual_seed(3)
    rows = torch.cat([torch.tensor([0, C - 1, C, 2 * C + 5, 4 * C - 1, 4 * C, 5 * C + 77, 8 * C - 1]),
                      torch.randint(0, B * n * C, (24,), generator=gen)]).unique()
    keep, ref, ref_lse = oracle_on_rows(q.float().cpu(), k_virt, v_virt, qr, as_segments(kr, ko), rows)
    assert_close(out[keep.cuda()], ref, what="cfg2 sampled rows")
    assert torch.allclose(lse[keep.cuda()].cpu(), ref_lse, atol=3e-3, rtol=1e-3)
    # chunk 0 of each batch element sees only itself: identical to a plain self-attention over that chunk
    solo, _ = mb.chunk_attn(q[:C], k[:C], v[:C], np.array([[0, C]], dtype=np.int32), np.array([[0, C]], dtype=np.int32), C, C)
    torch.cuda.synchronize()
    assert torch.equal(solo, out[:C])
    cache.close()
