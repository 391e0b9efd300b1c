"""The CPU oracle against the fixtures made from the reference's own CPU-runnable code."""
import math
import os

import numpy as np
import torch

from oracle import chunk_attn_oracle as O


def _bf16(bits):
    return torch.from_numpy(bits.copy()).view(torch.bfloat16)


def test_prologue_matches_reference_layernorm_and_rotary(golden_dir):
    z = np.load(os.path.join(golden_dir, "prologue.npz"))
    x = _bf16(z["x"])
    gamma, beta = torch.from_numpy(z["gamma"]), torch.from_numpy(z["beta"])
    sin, cos = torch.from_numpy(z["sin"]), torch.from_numpy(z["cos"])
    ln = O.layer_norm_1p(x, gamma, beta, 1e-6)
    assert torch.allclose(ln, torch.from_numpy(z["ln_fp32"]), atol=2e-6, rtol=1e-6)
    out = O.apply_rope(ln, cos, sin)
    assert torch.allclose(out, torch.from_numpy(z["out_fp32"]), atol=2e-6, rtol=1e-6)
    got = O.qk_prologue(x, gamma, beta, cos, sin)
    ref = _bf16(z["out_bf16"])
    # identical up to fp32 reduction order: at most one bf16 ulp on a handful of elements
    diff = (got.float() - ref.float()).abs()
    assert diff.max() <= 2 ** -6
    assert (got.view(torch.int16) != ref.view(torch.int16)).float().mean() < 1e-3


def test_linear_prologue_matches_reference_projection_and_get_q(golden_dir):
    """The reference's bf16 torch.nn.Linear (fp32 accumulation, one rounding) against the oracle's exactly rounded matmul:
    an accumulator next to a bf16 rounding boundary may differ by one ulp before the norm, nothing else may."""
    z = np.load(os.path.join(golden_dir, "linear_prologue.npz"))
    x = _bf16(z["x"])
    sin, cos = torch.from_numpy(z["sin"]), torch.from_numpy(z["cos"])
    for name in ("q", "k"):
        got = O.linear_qk_prologue(x, _bf16(z["w" + name]), torch.from_numpy(z["gamma_" + name]), torch.from_numpy(z["beta_" + name]), cos, sin)
        ref = _bf16(z[name])
        assert got.shape == ref.shape
        assert (got.float() - ref.float()).abs().max() <= 4e-2
        assert (got.view(torch.int16) != ref.view(torch.int16)).float().mean() < 0.02
        assert O.cosine(got, ref) > 0.999999
    v = O.linear_qk_prologue(x, _bf16(z["wv"]), None, None, None, None, norm_mode="none")
    ref = _bf16(z["v"])
    assert (v.view(torch.int16) != ref.view(torch.int16)).float().mean() < 5e-3
    assert (v.float() - ref.float()).abs().max() <= 2 ** -6


def test_get_xqkv_matches_the_reference_method(golden_dir):
    """FullyParallelAttention.get_xqkv itself (run on the CPU for the fixture) against the oracle's restatement; the
    reference's bf16 Linear and the oracle's exactly rounded matmul may differ by one bf16 ulp before the norms."""
    z = np.load(os.path.join(golden_dir, "xqkv.npz"))
    q, k, v = O.get_xqkv(_bf16(z["x"]), _bf16(z["y"]), _bf16(z["wqx"]), _bf16(z["wkv"]), torch.from_numpy(z["gq"]),
                         torch.from_numpy(z["bq"]), torch.from_numpy(z["gk"]), torch.from_numpy(z["bk"]))
    for got, name in ((q, "q"), (k, "k"), (v, "v")):
        ref = _bf16(z[name])
        assert got.shape == ref.shape, name
        assert (got.float() - ref.float()).abs().max() <= (2 ** -6 if name == "v" else 4e-2), name
        assert (got.view(torch.int16) != ref.view(torch.int16)).float().mean() < 0.03, name
        assert O.cosine(got, ref) > 0.99999, name


def test_rope_table_matches_reference_builder(golden_dir):
    z = np.load(os.path.join(golden_dir, "rope.npz"))
    for name in ("a", "b", "c"):
        T_total, T_keep, H, W = (int(v) for v in z[f"{name}_shape"])
        sin, cos = O.rope_table(T_total, H, W, keep_last_frames=T_keep)
        emb = torch.cat([sin, cos], -1)
        if f"{name}_idx" in z:
            emb = emb[torch.from_numpy(z[f"{name}_idx"])]
        assert emb.shape[-1] == 96
        assert torch.allclose(emb, torch.from_numpy(z[f"{name}_emb"]), atol=1e-6, rtol=0)


def test_cfg0_attention_matches_sdpa_fixture(golden_dir):
    z = np.load(os.path.join(golden_dir, "attn_cfg0.npz"))
    q, k, v = O.make_qkv(0, 384, 8, 2, scale=1 / math.sqrt(128))
    sums = [q.double().sum().item(), k.double().sum().item(), v.double().sum().item()]
    assert np.allclose(sums, z["sums"], rtol=0, atol=1e-9), "seeded generator drifted"
    qr = O.consecutive_q_ranges(3, 128)
    kr = O.default_k_ranges(3, 128)
    out, lse = O.range_attention(q, k, v, qr, kr)
    assert torch.allclose(out, torch.from_numpy(z["out"]), atol=1e-6, rtol=1e-5)
    assert torch.isfinite(lse).all()


def test_range_attention_vs_sdpa_random_rectangles():
    g = torch.Generator().manual_seed(3)
    Tq, Tk, Hq, Hkv, D = 200, 333, 6, 2, 128
    q = torch.randn(Tq, Hq, D, generator=g)
    k = torch.randn(Tk, Hkv, D, generator=g)
    v = torch.randn(Tk, Hkv, D, generator=g)
    qr = np.array([[0, 70], [70, 71], [90, 200]])            # a gap: rows 71..89 belong to no range
    segs = [[[5, 77]], [[0, 333]], [[0, 40], [100, 229]]]    # windowed start, full, two segments
    out, lse = O.range_attention(q, k, v, qr, segs)
    mask = O.block_mask(qr, segs, Tq, Tk)
    kk = torch.repeat_interleave(k, 3, dim=1)
    vv = torch.repeat_interleave(v, 3, dim=1)
    rows = mask.any(dim=1)
    ref = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(0, 1)[None], kk.transpose(0, 1)[None], vv.transpose(0, 1)[None],
        attn_mask=mask | ~rows[:, None])[0].transpose(0, 1)
    assert torch.allclose(out[rows], ref[rows], atol=2e-5, rtol=1e-4)
    assert (out[~rows] == 0).all() and torch.isinf(lse[~rows]).all()


def test_kv_cache_semantics():
    C, Hkv = 8, 2
    cache = O.RefKVCache(4 * C, Hkv, d=4)
    g = torch.Generator().manual_seed(0)
    kv0 = torch.randn(2 * C, Hkv, 8, generator=g)
    # no gate -> cache untouched, plain split
    k, v = cache.adjust(kv0, 0, C, update=True)
    assert (cache.buf == 0).all() and torch.equal(k, kv0[..., :4])
    # first chunk forwarded clean: written at 0
    k, v = cache.adjust(kv0, 0, C, update=True, fwd_extra_1st_chunk=True)
    assert torch.equal(cache.buf[:2 * C], kv0)
    # later step: prefix of one chunk is read, current written behind it
    kv1 = torch.randn(2 * C, Hkv, 8, generator=g)
    k, v = cache.adjust(kv1, 1, C, update=True)
    assert k.shape[0] == 3 * C and torch.equal(k[:C], kv0[:C, :, :4]) and torch.equal(v[C:], kv1[..., 4:])
    assert torch.equal(cache.buf[C:3 * C], kv1)
    # distill: last chunk is not stored
    cache2 = O.RefKVCache(4 * C, Hkv, d=4)
    cache2.adjust(kv1, 1, C, update=True, distill_nearly_clean_chunk=True)
    assert torch.equal(cache2.buf[C:2 * C], kv1[:C]) and (cache2.buf[2 * C:] == 0).all()


def test_ulysses_ownership_matches_reference_glue(golden_dir):
    z = np.load(os.path.join(golden_dir, "ulysses.npz"))
    for tag, cp in (("cp2", 2), ("cp4", 4)):
        S, Hq, Hkv, D = (int(x) for x in z[f"{tag}_case"])
        g = torch.Generator().manual_seed(5)
        qfull = torch.randn(S, Hq, D, generator=g)
        kvfull = torch.randn(S, Hkv, 2 * D, generator=g)
        splits = O.cp_split_sizes(S, cp)
        offs = np.concatenate([[0], np.cumsum(splits)])
        q_loc = [qfull[offs[r]:offs[r + 1]] for r in range(cp)]
        kv_loc = [kvfull[offs[r]:offs[r + 1]] for r in range(cp)]
        qx = O.ulysses_input_exchange(q_loc, cp)
        kvx = O.ulysses_input_exchange(kv_loc, cp)
        ox = O.ulysses_output_exchange(qx, splits)
        for r in range(cp):
            assert np.array_equal(qx[r].numpy(), z[f"{tag}_r{r}_q_x"])
            assert np.array_equal(kvx[r].numpy(), z[f"{tag}_r{r}_kv_x"])
            assert np.array_equal(ox[r].reshape(splits[r], 1, -1).numpy(), z[f"{tag}_r{r}_o_fin"])
            assert np.array_equal(ox[r].numpy(), q_loc[r].numpy())  # exchange out is the inverse


def test_e4m3_block_quantiser_roundtrip():
    g = torch.Generator().manual_seed(9)
    x = torch.randn(300, 2, 128, generator=g) * 3
    x8, sc, spans = O.quantize_e4m3_block128(x, [0, 140])
    assert [tuple(s) for s in spans] == [(0, 128), (128, 140), (140, 268), (268, 300)]
    back = O.dequantize_e4m3_block128(x8, sc, spans)
    assert O.cosine(back, x) > 0.999
    assert (back - x).abs().max() <= x.abs().max() / 16 + 1e-6


def test_bias_modulate_add_matches_reference_fixture(golden_dir):
    """oracle.bias_modulate_add against modulate.npz: the reference's bias_modulate_add + FusedLayerNorm run on the CPU."""
    z = np.load(f"{golden_dir}/modulate.npz")
    bf = lambda a: torch.from_numpy(a.copy()).view(torch.bfloat16)
    for tag in ("f32", "bf16"):
        x = torch.from_numpy(z[f"{tag}_x"]) if tag == "f32" else bf(z[f"{tag}_x"])
        res, gate, want = bf(z[f"{tag}_res"]), bf(z[f"{tag}_gate"]), bf(z[f"{tag}_out"])
        h = x.shape[-1]
        got = O.bias_modulate_add(x, res, torch.from_numpy(z[f"{tag}_cmap"]), gate[..., h:], torch.from_numpy(z[f"{tag}_gamma"]),
                                  torch.from_numpy(z[f"{tag}_beta"])).to(torch.bfloat16)
        diff = (got.float() - want.float()).abs()
        assert (diff <= want.float().abs() * 2 ** -7 + 1e-6).all(), f"{tag}: more than one bf16 ulp off ({diff.max().item()})"
        assert (got.view(torch.int16) == want.view(torch.int16)).float().mean().item() > 0.99


def test_div_clamp_to_matches_reference_fixture(golden_dir):
    """oracle.div_clamp_to against div_clamp.npz (the reference's own div_clamp_to): byte for byte."""
    z = np.load(f"{golden_dir}/div_clamp.npz")
    x = torch.from_numpy(z["x"].copy()).view(torch.bfloat16)
    got_c = O.div_clamp_to(x, torch.from_numpy(z["scale_c"])).view(torch.uint8).numpy()
    got_s = O.div_clamp_to(x.reshape(4, 12, -1), torch.from_numpy(z["scale_s"])).view(torch.uint8).numpy()
    assert np.array_equal(got_c, z["out_c"]) and np.array_equal(got_s, z["out_s"])
