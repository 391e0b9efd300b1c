"""The reference's denoising schedule driven through the layer mirror (prologue -> KV-cache gate/update -> attention)
against the oracle's flat-buffer restatement of _full_adjust_key_and_value + the per-range attention loop.
Steps follow the shipped 24B schedule (4 chunks, window 4): plain steps, the clean re-forward of a finished chunk
(fwd_extra_1st_chunk), steps that read a growing cached prefix with windowed k-ranges, and a distilled step that must
not store its last chunk."""
import numpy as np
import pytest
import torch

from oracle import chunk_attn_oracle as O
from gpu_util import as_segments, assert_close

pytestmark = pytest.mark.gpu

C, HQ, HKV = 260, 6, 2     # 260 tokens per chunk = 2 frames of 10 x 13 patches


def _step(layer, ip, ref_cache, gen, params, sin_cos_full, slice_point, n, k_chunks, update, extra=False, distill=False):
    import magi_b200 as mb
    from magi_b200.inference import ModelMetaArgs, PackedCoreAttnParams
    gq, bq, gk, bk = params
    T = n * C
    xq = torch.randn(T, HQ, 128, generator=gen).to(torch.bfloat16)
    xk = torch.randn(T, HKV, 128, generator=gen).to(torch.bfloat16)
    xv = torch.randn(T, HKV, 128, generator=gen).to(torch.bfloat16)
    # rotary rows of the frames being forwarded: absolute positions slice_point .. slice_point + n
    sin, cos = sin_cos_full
    rows = slice(slice_point * C, (slice_point + n) * C)
    rope = torch.cat([sin[rows], cos[rows]], dim=-1)
    qr = O.consecutive_q_ranges(n, C)
    kr = np.array([[a * C, b * C] for a, b in k_chunks], dtype=np.int32)
    meta = ModelMetaArgs(slice_point=slice_point, denoising_range_num=n, clip_token_nums=C,
                         core_attn_params=PackedCoreAttnParams.from_numpy(qr, kr, "cuda"),
                         fwd_extra_1st_chunk=extra, distill_nearly_clean_chunk=distill)
    ip.update_kv_cache = update
    out = layer.forward(xq.cuda(), xk.cuda(), xv.cuda(), ip, rope.cuda(), meta)
    torch.cuda.synchronize()
    assert mb.Context.get().status() == 0
    # oracle: same prologue, flat cache, cat(prefix, current), per-range attention
    q_ref = O.qk_prologue(xq, gq, bq, cos[rows], sin[rows]).float()
    k_ref = O.qk_prologue(xk, gk, bk, cos[rows], sin[rows]).float()
    kv = torch.cat([k_ref, xv.float()], dim=-1)
    k_all, v_all = ref_cache.adjust(kv, slice_point, C, update, fwd_extra_1st_chunk=extra, distill_nearly_clean_chunk=distill)
    ref, _ = O.range_attention(q_ref, k_all, v_all, qr, as_segments(kr))
    assert_close(out, ref, what=f"slice_point {slice_point}, n {n}, k {k_chunks}")


def test_denoising_schedule_with_paged_cache_matches_flat_cache_oracle():
    from magi_b200 import host
    from magi_b200.inference import ChunkCausalSelfAttention, InferenceParams
    params = host.synthetic_norm_params(61)
    layer = ChunkCausalSelfAttention(1, HQ, HKV, *params)
    ip = InferenceParams(max_batch_size=1, max_sequence_length=5 * C, n_layers=2)
    ref_cache = O.RefKVCache(5 * C, HKV)
    gen = torch.Generator().manual_seed(61)
    sin_cos = O.rope_table(10, 10, 13)          # 5 chunks x 2 frames
    run = lambda *a, **k: _step(layer, ip, ref_cache, gen, params, sin_cos, *a, **k)
    # stages 0..3: the window fills up; nothing is cached yet (the gate stays closed even with update_kv_cache set)
    run(0, 1, [(0, 1)], update=True)
    run(0, 3, [(0, 1), (0, 2), (0, 3)], update=False)
    assert ip.cache is None
    run(0, 4, [(0, 1), (0, 2), (0, 3), (0, 4)], update=True)
    assert ip.cache is None
    # stage 4, first step: chunk 0 is re-forwarded clean together with chunks 1..3 and everything is stored
    run(0, 4, [(0, 1), (0, 2), (0, 3), (0, 4)], update=True, extra=True)
    # stage 4, later steps: chunk 0 comes from the cache; the CFG pass without update leaves the cache alone
    run(1, 3, [(0, 2), (0, 3), (0, 4)], update=True)
    run(1, 3, [(0, 2), (0, 3), (0, 4)], update=False)
    # stage 5, first step: the clean chunk 1 sees only itself, windows start at chunk 1 (k-start > 0)
    run(1, 3, [(1, 2), (1, 3), (1, 4)], update=True, extra=True)
    run(2, 2, [(1, 3), (1, 4)], update=True)
    # a distilled step: the last (nearly clean) chunk must not be stored
    run(2, 3, [(1, 3), (1, 4), (2, 5)], update=True, distill=True)
    run(3, 2, [(2, 4), (2, 5)], update=True)
    # the cached pages hold exactly what the flat buffer holds
    for cid in range(4):
        k_page, v_page = ip.cache.read(1, cid)
        flat = ref_cache.buf[cid * C:(cid + 1) * C]
        assert (k_page.cpu().float() - flat[..., :128]).abs().max().item() <= 2 ** -5
        assert torch.equal(v_page.cpu().float(), flat[..., 128:])
    ip.cache.close()


def test_long_clip_streams_through_a_small_page_pool():
    """12 chunks with the shipped windows (noise2clean_kvrange [5,4,3,2], clean_chunk_kvrange 1): in the steady state
    every stage re-forwards the chunk that just became clean together with the four noisy ones, then denoises the four.
    Chunks behind the widest window are evicted, so 9 page slots per layer serve the whole clip, while the oracle keeps
    the reference's flat buffer of all 12 chunks.  k-ranges are the reference's absolute token offsets (k-start > 0)."""
    from magi_b200 import host
    from magi_b200.inference import ChunkCausalSelfAttention, InferenceParams
    n_chunks, window = 12, [5, 4, 3, 2]
    params = host.synthetic_norm_params(62)
    layer = ChunkCausalSelfAttention(0, HQ, HKV, *params)
    ip = InferenceParams(max_batch_size=1, max_sequence_length=n_chunks * C, n_layers=1, max_cached_chunks=9)
    ref_cache = O.RefKVCache(n_chunks * C, HKV)
    gen = torch.Generator().manual_seed(62)
    sin_cos = O.rope_table(2 * n_chunks, 10, 13)
    run = lambda *a, **k: _step(layer, ip, ref_cache, gen, params, sin_cos, *a, **k)

    def noisy_ranges(first, count):
        return [(max(c + 1 - window[j], 0), c + 1) for j, c in enumerate(range(first, first + count))]

    # fill-up: chunks 0..3 enter one by one (no cache traffic yet), then chunk 0 is finished
    for s in range(4):
        run(0, s + 1, [(0, j + 1) for j in range(s + 1)], update=True)
    for s in range(4, n_chunks + 4):
        clean = s - 4                                     # the chunk that became clean at the end of the last stage
        last = min(s, n_chunks - 1)                       # the newest chunk in flight
        noisy_first = clean + 1
        n_noisy = last - noisy_first + 1
        ip.evict_below(max(0, noisy_first + 1 - window[0]))
        # first step of the stage: the clean chunk is forwarded once more (sees only itself) and stored
        run(clean, 1 + n_noisy, [(clean, clean + 1)] + noisy_ranges(noisy_first, n_noisy), update=True, extra=True)
        if n_noisy:
            run(noisy_first, n_noisy, noisy_ranges(noisy_first, n_noisy), update=True)
            run(noisy_first, n_noisy, noisy_ranges(noisy_first, n_noisy), update=False)   # the CFG pass
    assert ip.first_live_chunk == n_chunks + 1 - window[0]
    assert ip.cache.max_chunks == 9
    ip.cache.close()


def test_host_tier_spill_and_prefetch_round_trip():
    """Pages spilled to pinned host memory and prefetched back on a side stream give bit-identical attention."""
    import magi_b200 as mb
    from magi_b200 import host
    from magi_b200.inference import HostPageStore
    Cc, n_layers = 200, 2
    g = torch.Generator().manual_seed(63)
    cache = mb.ChunkPagedKVCache(n_layers=n_layers, max_chunks=3, chunk_tokens=Cc, n_kv_heads=HKV)
    pages = {}
    for c in range(3):
        for layer in range(n_layers):
            k = torch.randn(Cc, HKV, 128, generator=g).to(torch.bfloat16).cuda()
            v = torch.randn(Cc, HKV, 128, generator=g).to(torch.bfloat16).cuda()
            cache.append(layer, c, k, v)
            pages[(layer, c)] = (k, v)
    q = torch.randn(Cc, HQ, 128, generator=g).to(torch.bfloat16).cuda()
    kc = torch.randn(Cc, HKV, 128, generator=g).to(torch.bfloat16).cuda()
    vc = torch.randn(Cc, HKV, 128, generator=g).to(torch.bfloat16).cuda()
    qr = np.array([[0, Cc]], dtype=np.int32)
    kr = np.array([[0, 4 * Cc]], dtype=np.int32)
    before = [mb.chunk_attn(q, kc, vc, qr, kr, Cc, 4 * Cc, cache=cache, layer=l, prefix_chunk_ids=[0, 1, 2])[0].clone()
              for l in range(n_layers)]
    tier = HostPageStore(cache)
    tier.spill(0)                                              # frees a slot in every layer
    with pytest.raises(mb.MagiError):
        mb.chunk_attn(q, kc, vc, qr, kr, Cc, 4 * Cc, cache=cache, layer=0, prefix_chunk_ids=[0, 1, 2])
    for layer in range(n_layers):                              # the freed slot takes a new chunk
        cache.append(layer, 3, kc, vc)
    cache.evict(3)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    ev = tier.prefetch(0, side)                                # back from the host while the main stream is free to compute
    torch.cuda.current_stream().wait_event(ev)
    after = [mb.chunk_attn(q, kc, vc, qr, kr, Cc, 4 * Cc, cache=cache, layer=l, prefix_chunk_ids=[0, 1, 2])[0]
             for l in range(n_layers)]
    torch.cuda.synchronize()
    for a, b in zip(before, after):
        assert torch.equal(a, b)
    for layer in range(n_layers):
        k_page, v_page = cache.read(layer, 0)
        assert torch.equal(k_page, pages[(layer, 0)][0]) and torch.equal(v_page, pages[(layer, 0)][1])
    cache.close()


def test_layer_from_hidden_states_matches_layer_from_projections():
    """forward_from_hidden (projection + prologue in one kernel) against forward on the library GEMM's outputs, through a
    cached step: the same pages, the same attention; only the GEMM's accumulation order differs."""
    import magi_b200 as mb
    from magi_b200 import host
    from magi_b200.inference import ChunkCausalSelfAttention, InferenceParams, ModelMetaArgs, PackedCoreAttnParams
    params = host.synthetic_norm_params(62)
    hidden, n = 384, 2
    g = torch.Generator().manual_seed(62)
    wq, wk, wv = [(torch.randn(h * 128, hidden, generator=g) * hidden ** -0.5).to(torch.bfloat16).cuda() for h in (HQ, HKV, HKV)]
    sin, cos = O.rope_table(6, 10, 13)
    outs = []
    for fused in (False, True):
        layer = ChunkCausalSelfAttention(0, HQ, HKV, *params)
        ip = InferenceParams(max_batch_size=1, max_sequence_length=3 * C, n_layers=1)
        gen = torch.Generator().manual_seed(63)
        res = []
        for slice_point, k_chunks, update in ((0, [(0, 1)], True), (1, [(0, 2), (0, 3)], False)):
            nn = len(k_chunks)
            x = (torch.randn(nn * C, hidden, generator=gen) * 1.5).to(torch.bfloat16).cuda()
            rows = slice(slice_point * C, (slice_point + nn) * C)
            rope = torch.cat([sin[rows], cos[rows]], dim=-1).cuda()
            kr = np.array([[a * C, b * C] for a, b in k_chunks], dtype=np.int32)
            meta = ModelMetaArgs(slice_point=slice_point, denoising_range_num=nn, clip_token_nums=C,
                                 core_attn_params=PackedCoreAttnParams.from_numpy(O.consecutive_q_ranges(nn, C), kr, "cuda"),
                                 fwd_extra_1st_chunk=(slice_point == 0))
            ip.update_kv_cache = update
            if fused:
                res.append(layer.forward_from_hidden(x, wq, wk, wv, ip, rope, meta).clone())
            else:
                res.append(layer.forward((x @ wq.t()).view(-1, HQ, 128), (x @ wk.t()).view(-1, HKV, 128),
                                         (x @ wv.t()).view(-1, HKV, 128), ip, rope, meta).clone())
            torch.cuda.synchronize()
            assert mb.Context.get().status() == 0
        ip.cache.close()
        outs.append(res)
    for a, b in zip(*outs):
        assert_close(b, a, max_abs=4e-2, min_cos=0.9999, what="layer from hidden states")
