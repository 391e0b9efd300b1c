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


def test_range_builders_match_oracle():
    from magi_b200 import host
    assert np.array_equal(host.q_ranges_for_chunks(4, 9360), O.consecutive_q_ranges(4, 9360))
    for sp in (0, 1, 3):
        assert np.array_equal(host.default_k_ranges(4, 9360, sp), O.default_k_ranges(4, 9360, sp))
    assert np.array_equal(host.windowed_k_ranges(6, 10, 100, [5, 4, 3, 2], 3), O.windowed_k_ranges(6, 10, 100, [5, 4, 3, 2], 3))
    # steady state of the shipped schedule: windows end at each chunk and start > 0
    w = host.windowed_k_ranges(6, 10, 100, [5, 4, 3, 2], 3)
    assert w.tolist() == [[0, 400], [100, 500], [300, 600], [500, 700]]
    for s, cp in ((86400, 8), (37441, 4), (11, 2)):
        assert host.cp_split_sizes(s, cp) == O.cp_split_sizes(s, cp) and sum(host.cp_split_sizes(s, cp)) == s


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
