"""The caption cross-attention (next row after the self-attention core: dit_module.py:1005-1021, 1098-1136) through the
same kernels: per-head LayerNorm without rotary for q and k (q_layernorm_xattn / k_layernorm_xattn), then one short
kv range (<= 800 caption tokens) per query chunk - including an empty caption - with the reference's call shape."""
import numpy as np
import pytest
import torch

from oracle import chunk_attn_oracle as O
from gpu_util import as_segments, assert_close

pytestmark = pytest.mark.gpu


def test_cross_attention_shape_and_norm_without_rope():
    import magi_b200 as mb
    from magi_b200 import host
    C, n, Hq, Hkv = 1560, 4, 24, 8                       # one latent frame of 30x52 patches per chunk
    caps = [800, 37, 0, 411]                             # valid caption tokens per chunk; the third is empty
    g = torch.Generator().manual_seed(51)
    xq = torch.randn(n * C, Hq, 128, generator=g).to(torch.bfloat16)
    xk = torch.randn(sum(caps), Hkv, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(sum(caps), Hkv, 128, generator=g).to(torch.bfloat16)
    gq, bq, gk, bk = host.synthetic_norm_params(51)
    q_d = mb.qk_norm_rope(xq.cuda(), gq, bq, None, None)          # LayerNorm(gamma+1, beta) only
    k_d = mb.qk_norm_rope(xk.cuda(), gk, bk, None, None)
    torch.cuda.synchronize()
    q_ref = O.layer_norm_1p(xq, gq, bq).to(torch.bfloat16)
    k_ref = O.layer_norm_1p(xk, gk, bk).to(torch.bfloat16)
    assert (q_d.cpu().float() - q_ref.float()).abs().max().item() <= 2 ** -5
    assert (k_d.cpu().float() - k_ref.float()).abs().max().item() <= 2 ** -5
    qr, kr = host.cross_attn_ranges(C, n, caps)
    out = torch.full((n * C, Hq, 128), 9.0, dtype=torch.bfloat16, device="cuda")
    out, lse = mb.flex_attn(q_d, k_d, v.cuda(), torch.as_tensor(qr, device="cuda"), torch.as_tensor(kr, device="cuda"),
                            max_seqlen_q=C, max_seqlen_k=800)
    torch.cuda.synchronize()
    assert mb.Context.get().status() == 0
    ref, ref_lse = O.range_attention(q_d.cpu().float(), k_d.cpu().float(), v.float(), qr, as_segments(kr))
    assert_close(out, ref, what="cross-attention")
    assert (out[2 * C:3 * C].float() == 0).all()          # empty caption: zeros, lse = -inf
    assert torch.isinf(lse[2 * C:3 * C]).all()
    live = torch.cat([torch.arange(0, 2 * C), torch.arange(3 * C, 4 * C)])
    assert torch.allclose(lse.cpu()[live], ref_lse[live], atol=3e-3, rtol=1e-3)
    # context-parallel view of the same problem: every rank's local ranges reproduce its rows
    splits = host.cp_split_sizes(n * C, 4)
    offs = np.concatenate([[0], np.cumsum(splits)])
    for r in range(4):
        ql, kl, max_q = host.cp_cross_attn_ranges(qr, kr, splits, r)
        o_r, _ = mb.chunk_attn(q_d[offs[r]:offs[r + 1]], k_d, v.cuda(), ql, kl, max_q, 800)
        torch.cuda.synchronize()
        assert torch.equal(o_r, out[offs[r]:offs[r + 1]])


def test_get_xqkv_matches_the_reference_fixture(golden_dir):
    """inference.get_xqkv against FullyParallelAttention.get_xqkv run on the CPU (tests/golden/xqkv.npz)."""
    import os
    import magi_b200 as mb
    from magi_b200 import inference
    z = np.load(os.path.join(golden_dir, "xqkv.npz"))
    b16 = lambda a: torch.from_numpy(a.copy()).view(torch.bfloat16)
    q, k, v = inference.get_xqkv(b16(z["x"]).cuda(), b16(z["y"]).cuda(), b16(z["wqx"]).cuda(), b16(z["wkv"]).cuda(),
                                 torch.from_numpy(z["gq"]), torch.from_numpy(z["bq"]), torch.from_numpy(z["gk"]), torch.from_numpy(z["bk"]))
    torch.cuda.synchronize()
    assert mb.Context.get().status() == 0
    assert_close(q, b16(z["q"]), max_abs=4e-2, min_cos=0.99999, what="query_xattn vs reference")
    assert_close(k, b16(z["k"]), max_abs=4e-2, min_cos=0.99999, what="key_xattn vs reference")
    assert_close(v, b16(z["v"]), max_abs=2 ** -5, min_cos=0.99999, what="value_xattn vs reference")


def test_get_xqkv_from_hidden_and_caption_states():
    """get_xqkv (dit_module.py:1005-1021) from the projections on: qx + q_layernorm_xattn (no rotary) and the K|V-interleaved
    linear_kv_xattn + k_layernorm_xattn, each one kernel, then the caption cross-attention over them against the oracle."""
    import magi_b200 as mb
    from magi_b200 import host, inference
    g = torch.Generator().manual_seed(71)
    C, n, Hq, Hkv, hidden, cap_dim = 260, 2, 6, 2, 384, 512
    caps = [77, 130]
    x = (torch.randn(n * C, hidden, generator=g) * 1.3).to(torch.bfloat16)
    y = torch.randn(sum(caps), cap_dim, generator=g).to(torch.bfloat16)
    wqx = (torch.randn(Hq * 128, hidden, generator=g) * hidden ** -0.5).to(torch.bfloat16)
    wkv = (torch.randn(2 * Hkv * 128, cap_dim, generator=g) * cap_dim ** -0.5).to(torch.bfloat16)
    gq, bq, gk, bk = O.make_norm_params(71)
    q, k, v = inference.get_xqkv(x.cuda(), y.cuda(), wqx.cuda(), wkv.cuda(), gq, bq, gk, bk)
    torch.cuda.synchronize()
    assert mb.Context.get().status() == 0
    q_ref, k_ref, v_ref = O.get_xqkv(x, y, wqx, wkv, gq, bq, gk, bk)
    assert q.shape == q_ref.shape and k.shape == k_ref.shape == (sum(caps), Hkv, 128)
    assert_close(q, q_ref, max_abs=4e-2, min_cos=0.99999, what="query_xattn")
    assert_close(k, k_ref, max_abs=4e-2, min_cos=0.99999, what="key_xattn")
    assert_close(v, v_ref, max_abs=2 ** -5, min_cos=0.99999, what="value_xattn")
    qr, kr = host.cross_attn_ranges(C, n, caps)
    out, _ = mb.chunk_attn(q, k, v, qr, kr, C, max(caps), return_lse=False)
    torch.cuda.synchronize()
    ref, _ = O.range_attention(q.cpu().float(), k.cpu().float(), v.cpu().float(), qr, as_segments(kr))
    assert_close(out, ref, what="cross-attention over the fused projections")
