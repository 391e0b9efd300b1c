"""Host-side metadata helpers of the package against the oracle and the reference-made fixtures."""
import os

import numpy as np
import torch

from oracle import chunk_attn_oracle as O


def test_rotary_table_matches_reference_fixture_and_oracle(golden_dir):
    from magi_b200 import host
    z = np.load(os.path.join(golden_dir, "rope.npz"))
    for name in ("a", "b", "c"):
        T_total, T_keep, H, W = (int(v) for v in z[f"{name}_shape"])
        emb = host.rotary_table(T_total, H, W, keep_last_frames=T_keep)
        sin, cos = host.split_sin_cos(emb)
        osin, ocos = O.rope_table(T_total, H, W, keep_last_frames=T_keep)
        assert torch.allclose(sin, osin, atol=1e-6, rtol=0) and torch.allclose(cos, ocos, atol=1e-6, rtol=0)
        if f"{name}_idx" in z:
            emb = emb[torch.from_numpy(z[f"{name}_idx"])]
        assert torch.allclose(emb, torch.from_numpy(z[f"{name}_emb"]), atol=1e-6, rtol=0)


def test_k_range_generators_match_the_reference_over_whole_schedules(golden_dir):
    """host.generate_*_kvrange and host.denoise_schedule against kranges.npz: the reference's own generators run over every
    forward step of the shipped 24B schedule, a longer clip, a prefix-video clip, the window-less default and batch 2."""
    from magi_b200 import host
    z = np.load(f"{golden_dir}/kranges.npz")
    for tag in ("base24b", "long16", "prefix", "default", "batch2"):
        cfg = z[f"{tag}_cfg"].tolist()
        num_steps, window_size, chunk_num, clean, prefix_chunks, batch, C = cfg[:7]
        n2c = cfg[7:]
        rows, kr, kr_len = z[f"{tag}_steps"], z[f"{tag}_kr"], z[f"{tag}_kr_len"]
        starts = np.concatenate([[0], np.cumsum(kr_len)])
        sched = list(host.denoise_schedule(num_steps, window_size, chunk_num, prefix_chunks))
        assert len(sched) == len(rows)
        for st, row in zip(sched, rows):
            step, off, cs, ce, ts, te, idx, extra, sp, n_den, kidx = row[:11].tolist()
            steps_of = [v for v in row[11:].tolist() if v >= 0]
            assert (st["step"], st["chunk_start"], st["chunk_end"], int(st["fwd_extra_1st_chunk"]), st["slice_point"],
                    st["denoising_range_num"], st["denoise_step_of_each_chunk"]) == (step, cs, ce, extra, sp, n_den, steps_of)
            got = host.generate_kvrange_for_denoising_video(sp, n_den, steps_of, n2c, clean, num_steps, C, batch)
            want = kr[starts[kidx]:starts[kidx + 1]]
            assert got.dtype == np.int32 and np.array_equal(got, want), (tag, step, got, want)
        for range_num in (1, 2, 7):
            assert np.array_equal(host.generate_kvrange_for_prefix_video(range_num, C, clean, n2c, batch), z[f"{tag}_prefix{range_num}"])
    assert np.array_equal(host.generate_kvrange_for_prefix_video(12, 21600), z["fallback8_prefix12"])
    assert np.array_equal(host.generate_kv_range_for_uncondition(5, 21600), z["uncond"])
    # the steady state of the shipped windows, as a readable instance: four chunks in flight at steps (24+i, 16+i, 8+i, i)
    w = host.generate_noise2clean_kvrange(3, 4, [5, 4, 3, 2], 1, [25, 17, 9, 1], 32, 100)
    assert w.tolist() == [[200, 400], [200, 500], [200, 600], [200, 700]]
    # the same stage's first step re-forwards the chunk that just became clean: it sees only itself (clean_chunk_kvrange 1)
    w = host.generate_noise2clean_kvrange(2, 5, [5, 4, 3, 2], 1, [32, 24, 16, 8, 0], 32, 100)
    assert w.tolist() == [[200, 300], [200, 400], [200, 500], [200, 600], [200, 700]]
    assert np.array_equal(host.q_ranges_for_chunks(4, 9360), O.consecutive_q_ranges(4, 9360))
    for sp in (0, 1, 3):
        assert np.array_equal(host.default_k_ranges(4, 9360, sp), O.default_k_ranges(4, 9360, sp))
    for s, cp in ((86400, 8), (37441, 4), (11, 2)):
        assert host.cp_split_sizes(s, cp) == O.cp_split_sizes(s, cp) and sum(host.cp_split_sizes(s, cp)) == s


def test_cp_ulysses_process_matches_the_reference_on_gloo_ranks(golden_dir):
    """host.cp_ulysses_process / scatter_to_context_parallel_region / cp_cross_attn_ranges against cp_xattn.npz: the
    reference's cp_ulysses_process and scatter run unmodified on 2 and 4 gloo ranks."""
    from magi_b200 import host
    z = np.load(f"{golden_dir}/cp_xattn.npz")
    for world in (2, 4):
        for rank in range(world):
            pre = f"cp{world}_r{rank}_"
            for tag, seed in (("a", 21), ("b", 21)):
                C, n, N, *caps = z[pre + f"{tag}_in"].tolist()
                S = C * n
                g = torch.Generator().manual_seed(seed)
                x = torch.randn(S, N, 8, generator=g)
                cmap = torch.arange(S, dtype=torch.int32) // C
                rope = torch.randn(S, 96, generator=g)
                qr, kr = host.cross_attn_ranges(C, n * N, caps)
                xs, cm, rp, splits, (ql, kl, mq) = host.cp_ulysses_process(world, rank, x, cmap, rope, qr, kr)
                assert splits == z[pre + f"{tag}_splits"].tolist()
                assert torch.equal(xs, torch.from_numpy(z[pre + f"{tag}_x"])) and torch.equal(rp, torch.from_numpy(z[pre + f"{tag}_rope"]))
                assert torch.equal(cm, torch.from_numpy(z[pre + f"{tag}_cmap"]))
                assert np.array_equal(ql, z[pre + f"{tag}_q"]) and np.array_equal(kl, z[pre + f"{tag}_k"])
                assert mq == int(z[pre + f"{tag}_maxq"][0])
            C, n, shuffle = z[pre + "s_in"].tolist()
            g = torch.Generator().manual_seed(22)
            x = torch.randn(C * n, 1, 4, generator=g)
            got = host.scatter_to_context_parallel_region(x, z[pre + "s_splits"].tolist(), rank, cp_shuffle_num=shuffle)
            assert torch.equal(got, torch.from_numpy(z[pre + "s_x"]))


def test_own_prefix_segments():
    from magi_b200 import host
    kr, offs = host.own_prefix_k_segments(n=4, chunk_tokens=10, n_prefix=3, batch=2)
    assert offs.tolist() == [0, 1, 3, 5, 7, 8, 10, 12, 14]
    assert kr[:7].tolist() == [[60, 70], [0, 10], [70, 80], [0, 20], [80, 90], [0, 30], [90, 100]]
    assert kr[7:10].tolist() == [[100, 110], [30, 40], [110, 120]]


def test_synthetic_norm_params_match_oracle():
    from magi_b200 import host
    for a, b in zip(host.synthetic_norm_params(3), O.make_norm_params(3)):
        assert torch.equal(a, b)


def test_cross_attention_range_helpers():
    from magi_b200 import host
    qr, kr = host.cross_attn_ranges(10, 3, [4, 0, 7])
    assert qr.tolist() == [[0, 10], [10, 20], [20, 30]] and kr.tolist() == [[0, 4], [4, 4], [4, 11]]
    splits = host.cp_split_sizes(30, 4)          # 8, 8, 7, 7
    ql, kl, mq = host.cp_cross_attn_ranges(qr, kr, splits, 1)     # rows 8..16: tail of chunk 0, head of chunk 1
    assert ql.tolist() == [[0, 2], [2, 8]] and kl.tolist() == [[0, 4], [4, 4]] and mq == 8
    ql, kl, mq = host.cp_cross_attn_ranges(qr, kr, splits, 3)     # rows 23..30: inside chunk 2
    assert ql.tolist() == [[0, 7]] and kl.tolist() == [[4, 11]] and mq == 7


def test_projection_operand_layout_is_the_reference_rearrange():
    """ProjInput's column map against the reference's own two lines (attn_linear_proj, dit_module.py:1336-1338):
    torch.concat(dim=2) followed by einops "sq b (n hn hd) -> sq b (hn n hd)", n=2, hn=8."""
    from einops import rearrange
    from magi_b200.inference import ProjInput
    sq, H = 5, 16
    core = torch.arange(sq * H * 128, dtype=torch.float32).view(sq, H, 128)
    cross = -core - 1
    want = rearrange(torch.concat([core.view(sq, 1, -1), cross.view(sq, 1, -1)], dim=2), "sq b (n hn hd) -> sq b (hn n hd)", n=2, hn=8)
    got = ProjInput.reference_layout(core, cross)
    assert torch.equal(got, want.view(sq, -1))
    # the kernel-side formula: head h of output `which` starts at (h // hpb) * 2 * hd + which * hd + (h % hpb) * 128
    hpb = H // 8
    hd = hpb * 128
    for which, src in ((0, core), (1, cross)):
        for h in range(H):
            col = (h // hpb) * 2 * hd + which * hd + (h % hpb) * 128
            assert torch.equal(got[:, col:col + 128], src[:, h])


def test_eviction_horizon_bookkeeping_and_k_range_rebasing():
    """InferenceParams.evict_below + the layer mirror's prefix list and k-range offset, with a stand-in for the cache."""
    from magi_b200 import inference as inf

    class FakeCache:
        chunk_tokens, n_kv_heads = 10, 2

        def __init__(self):
            self.pages, self.evicted = set(), []

        def append(self, layer, chunk_id, k, v):
            self.pages.add(chunk_id)

        def evict(self, chunk_id):
            if chunk_id not in self.pages:
                raise inf.ops.MagiError(-4, "not cached")
            self.pages.remove(chunk_id)
            self.evicted.append(chunk_id)

    ip = inf.InferenceParams(max_batch_size=1, max_sequence_length=120, n_layers=1, max_cached_chunks=6)
    ip.cache = FakeCache()
    ip.update_kv_cache = True
    layer = inf.ChunkCausalSelfAttention(0, 4, 2, None, None, None, None)
    qr = np.array([[0, 10], [10, 20]], dtype=np.int32)
    kr = np.array([[30, 60], [40, 70]], dtype=np.int32)          # absolute tokens: chunks 3..5 and 4..6
    params = inf.PackedCoreAttnParams(torch.as_tensor(qr), torch.as_tensor(kr), qr, kr, 10, 40)
    meta = inf.ModelMetaArgs(slice_point=5, denoising_range_num=2, clip_token_nums=10, core_attn_params=params)
    key = torch.zeros(20, 2, 128)
    for c in range(5):
        ip.cache.append(0, c, None, None)
    cache, prefix = layer.adjust_key_and_value_for_inference(key, key, ip, meta)
    assert prefix == [0, 1, 2, 3, 4] and ip.cache.pages == {0, 1, 2, 3, 4, 5, 6}     # current chunks stored at 5, 6
    ip.evict_below(3)
    ip.evict_below(2)                                              # going back is a no-op
    assert ip.first_live_chunk == 3 and ip.cache.evicted == [0, 1, 2]
    cache, prefix = layer.adjust_key_and_value_for_inference(key, key, ip, meta)
    assert prefix == [3, 4]
    # the k-range offset the attention call will use: (slice_point - len(prefix)) chunks
    assert (meta.slice_point - len(prefix)) * meta.clip_token_nums == 30 <= int(params.np_k_range.min())
    ip.evict_below(4)                                              # now the first window reaches an evicted chunk
    cache, prefix = layer.adjust_key_and_value_for_inference(key, key, ip, meta)
    import pytest
    with pytest.raises(ValueError):
        layer.core_attention(key, key, key, meta, cache, prefix)


def test_flex_attn_accepts_the_reference_call_site():
    """The drop-in seam: the keyword arguments with which FullyParallelAttention.core_attention calls the module
    variable `flex_attention` (inference/model/dit/dit_module.py:1032-1043) must all be parameters of magi_b200.flex_attn,
    and its positional arguments (q, k, v, q_range, k_range) must line up with flex_attn's leading parameters.  Read from
    the reference's source text when the checkout is there."""
    import ast
    import inspect
    import os
    import pytest
    path = os.path.join(os.environ.get("MAGI_REFERENCE_ROOT", "/root/reference"), "inference/model/dit/dit_module.py")
    if not os.path.exists(path):
        pytest.skip("reference checkout not present")
    import magi_b200
    calls = [n for n in ast.walk(ast.parse(open(path).read()))
             if isinstance(n, ast.Call) and isinstance(n.func, ast.Name) and n.func.id == "flex_attention"]
    assert calls, "no flex_attention call found in the reference"
    params = list(inspect.signature(magi_b200.flex_attn).parameters)
    for call in calls:
        assert len(call.args) <= 5 and params[:5] == ["q", "k", "v", "q_ranges", "k_ranges"]
        for kw in call.keywords:
            assert kw.arg in params, f"flex_attn lacks the keyword {kw.arg} the reference passes"
