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
