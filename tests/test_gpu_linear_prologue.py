"""Parity of the projection GEMM with the prologue in its epilogue (get_q / get_k / get_v from their first line,
dit_module.py:953-989) against the reference-generated fixture, the CPU oracle and the unfused CUDA path."""
import os

import numpy as np
import pytest
import torch

from oracle import chunk_attn_oracle as O
from gpu_util import assert_close

pytestmark = pytest.mark.gpu

# The accumulation order of a GEMM is not the reference's: an accumulator that lands next to a bf16 rounding boundary may
# round the other way (one bf16 ulp of the pre-norm value, 2^-8 relative), which the norm passes on scaled by
# (gamma + 1) / std.  Everything else follows the reference's order of operations.
MAX_ABS = 4e-2
MIN_COS = 0.99999


@pytest.fixture(scope="module")
def mb():
    import magi_b200
    return magi_b200


def _bf16(bits):
    return torch.from_numpy(bits.copy()).view(torch.bfloat16)


def test_linear_prologue_matches_reference_fixture(mb, golden_dir):
    """136 tokens (one ragged row tile), 3 Q heads (an odd head count: half of the last channel block is empty), 1 KV head."""
    z = np.load(os.path.join(golden_dir, "linear_prologue.npz"))
    x = _bf16(z["x"]).cuda()
    cos, sin = torch.from_numpy(z["cos"]), torch.from_numpy(z["sin"])
    for name in ("q", "k"):
        out = mb.linear_qk_norm_rope(x, _bf16(z["w" + name]).cuda(), torch.from_numpy(z["gamma_" + name]),
                                     torch.from_numpy(z["beta_" + name]), cos, sin)
        torch.cuda.synchronize()
        assert mb.Context.get().status() == 0
        ref = _bf16(z[name])
        assert_close(out, ref, max_abs=MAX_ABS, min_cos=MIN_COS, what=name)
        assert (out.cpu().view(torch.int16) != ref.view(torch.int16)).float().mean().item() < 0.05
    v = mb.linear_qk_norm_rope(x, _bf16(z["wv"]).cuda(), None, None, None, None, norm_mode="none")
    torch.cuda.synchronize()
    ref = _bf16(z["v"])
    assert (v.cpu().view(torch.int16) != ref.view(torch.int16)).float().mean().item() < 0.01
    assert_close(v, ref, max_abs=2 ** -5, min_cos=MIN_COS, what="v")


@pytest.mark.parametrize("mode", ["layernorm_1p", "rmsnorm", "none"])
def test_both_forms_against_oracle_and_unfused_path(mb, mode, monkeypatch):
    """19000 tokens x 1024 features x 8 heads: 16 k-blocks per tile (the ring wraps), several tiles per CTA, a ragged last
    row tile (the odd CTA of the last pair has 56 rows); the one-CTA form and the CTA-pair form accumulate in the same
    order and must agree bit for bit."""
    g = torch.Generator().manual_seed(31)
    T, K, H = 19000, 1024, 8
    x = (torch.randn(T, K, generator=g) * 1.2).to(torch.bfloat16)
    w = (torch.randn(H * 128, K, generator=g) * K ** -0.5).to(torch.bfloat16)
    gam, bet, _, _ = O.make_norm_params(5)
    sin, cos = O.rope_table(8, 25, 95)
    assert sin.shape[0] == T
    xd, wd = x.cuda(), w.cuda()
    outs = []
    for form in ("solo", "pair"):
        monkeypatch.setenv("MAGI_LINEAR_FORM", form)
        outs.append(mb.linear_qk_norm_rope(xd, wd, gam, bet, cos, sin, norm_mode=mode))
        torch.cuda.synchronize()
        assert mb.Context.get().status() == 0
    monkeypatch.delenv("MAGI_LINEAR_FORM")
    assert torch.equal(outs[0], outs[1])
    rows = torch.cat([torch.arange(0, 300), torch.arange(9400, 9700), torch.arange(T - 300, T), torch.randint(0, T, (400,), generator=g)])
    ref = O.linear_qk_prologue(x[rows], w, gam, bet, cos[rows], sin[rows], norm_mode=mode)
    assert_close(outs[0][rows.cuda()], ref, max_abs=MAX_ABS, min_cos=MIN_COS, what=f"fused {mode}")
    # the unfused CUDA path: library GEMM, then the prologue kernel
    y = (xd @ wd.t()).view(T, H, 128)
    unfused = y if mode == "none" else mb.qk_norm_rope(y, gam, bet, cos, sin, norm_mode=mode)
    torch.cuda.synchronize()
    assert_close(outs[0], unfused, max_abs=MAX_ABS, min_cos=MIN_COS, what=f"fused vs unfused {mode}")


def test_destination_layouts_and_strided_operands(mb):
    """x and W as column slices of wider tensors (the fused QKV weight), the result written as the Ulysses send layout
    "(cp seq) hn hd" (context_parallel.py:396) and into a K|V fused buffer (dit_module.py:991-996)."""
    g = torch.Generator().manual_seed(32)
    T, K, H, cp = 700, 384, 4, 2
    xw = (torch.randn(T, K + 128, generator=g)).to(torch.bfloat16).cuda()
    ww = (torch.randn(3 * H * 128, K + 256, generator=g) * K ** -0.5).to(torch.bfloat16).cuda()
    x, w = xw[:, 128:], ww[H * 128:2 * H * 128, 256:]
    gam, bet, _, _ = O.make_norm_params(6)
    sin, cos = O.rope_table(2, 10, 35)
    packed = mb.linear_qk_norm_rope(x, w, gam, bet, cos, sin)
    ref = O.linear_qk_prologue(x.cpu(), w.cpu(), gam, bet, cos, sin)
    assert_close(packed, ref, max_abs=MAX_ABS, min_cos=MIN_COS, what="strided operands")
    send = torch.zeros(cp, T, H // cp, 128, dtype=torch.bfloat16, device="cuda")
    mb.linear_qk_norm_rope(x, w, gam, bet, cos, sin, out=send, heads_per_block=H // cp)
    assert torch.equal(send.permute(1, 0, 2, 3).reshape(T, H, 128), packed)
    kv = torch.zeros(T, H, 256, dtype=torch.bfloat16, device="cuda")
    mb.linear_qk_norm_rope(x, w, gam, bet, cos, sin, out=kv[:, :, :128])
    mb.linear_qk_norm_rope(x, w, None, None, None, None, norm_mode="none", out=kv[:, :, 128:])
    torch.cuda.synchronize()
    assert torch.equal(kv[:, :, :128], packed)
    assert_close(kv[:, :, 128:], O.linear_qk_prologue(x.cpu(), w.cpu(), None, None, None, None, norm_mode="none"),
                 max_abs=2 ** -5, min_cos=MIN_COS, what="v into the fused buffer")


def test_bad_arguments_are_refused_on_the_host(mb):
    x = torch.zeros(64, 192, dtype=torch.bfloat16, device="cuda")
    w = torch.zeros(128, 192, dtype=torch.bfloat16, device="cuda")
    gam, bet, _, _ = O.make_norm_params(1)
    with pytest.raises(mb.MagiError, match="multiple of 128"):
        mb.linear_qk_norm_rope(x, w, gam, bet, None, None)
    x, w = torch.zeros(64, 256, dtype=torch.bfloat16, device="cuda"), torch.zeros(128, 256, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(mb.MagiError, match="rot_pairs"):
        mb.linear_qk_norm_rope(x, w, gam, bet, torch.zeros(64, 40), torch.zeros(64, 40))
    assert mb.linear_qk_norm_rope(x[:0], w, gam, bet, None, None).shape == (0, 1, 128)


@pytest.mark.parametrize("form", ["solo", "pair"])
def test_fp8_projection_against_oracle_and_library_gemm(mb, form, monkeypatch):
    """The middle layers' PerTensorQuantizedFp8Linear members (dit_module.py:409-410, :445-456) in front of get_q: the
    byte-exact quantiser's e4m3 output and the e4m3 weight go through the same kernel with kind::f8f6f4 UMMAs; sums of
    e4m3 products are exact in fp32 far beyond this K, so only the bf16 rounding of the scaled accumulator can differ."""
    from magi_b200 import inference as inf
    g = torch.Generator().manual_seed(41)
    T, K, H = 19000, 1024, 8
    x = (torch.randn(T, K, generator=g) * 2).to(torch.bfloat16)
    w8 = (torch.randn(H * 128, K, generator=g) * 20).to(torch.float8_e4m3fn)
    in_scale, w_scale = torch.full((K,), 0.02), torch.tensor([0.003])
    gam, bet, _, _ = O.make_norm_params(7)
    sin, cos = O.rope_table(8, 25, 95)
    xd, wd = x.cuda(), w8.cuda()
    x8 = mb.div_clamp_to(xd, in_scale)
    monkeypatch.setenv("MAGI_LINEAR_FORM", form)
    out = mb.linear_qk_norm_rope(x8, wd, gam, bet, cos, sin, x_scale=in_scale[:1].cuda(), w_scale=w_scale.cuda())
    torch.cuda.synchronize()
    assert mb.Context.get().status() == 0
    rows = torch.cat([torch.arange(0, 200), torch.arange(T - 200, T), torch.randint(0, T, (300,), generator=g)])
    y_ref = O.fp8_linear(x[rows], in_scale, w8, 0.02, 0.003).to(torch.bfloat16).view(-1, H, 128)
    ref = O.qk_prologue(y_ref, gam, bet, cos[rows], sin[rows])
    assert_close(out[rows.cuda()], ref, max_abs=MAX_ABS, min_cos=MIN_COS, what=f"fp8 fused {form}")
    # the unfused CUDA path: quantiser, library FP8 GEMM, prologue kernel
    lin = inf.PerTensorQuantizedFp8Linear(wd.unsqueeze(0), w_scale, in_scale)
    unfused = mb.qk_norm_rope(lin(xd).view(T, H, 128), gam, bet, cos, sin)
    torch.cuda.synchronize()
    assert_close(out, unfused, max_abs=MAX_ABS, min_cos=MIN_COS, what=f"fp8 fused vs unfused {form}")


def test_small_shapes_and_block_pointers(mb):
    """One ragged row tile with a single head and the smallest K (two k-blocks in bf16, one in e4m3), and the per-block
    destination pointers the fused Ulysses exchange uses (here two local buffers instead of two ranks' receive buffers)."""
    g = torch.Generator().manual_seed(43)
    gam, bet, _, _ = O.make_norm_params(8)
    for T, K, H in ((5, 128, 1), (129, 128, 2), (300, 256, 4)):
        x = torch.randn(T, K, generator=g).to(torch.bfloat16)
        w = (torch.randn(H * 128, K, generator=g) * K ** -0.5).to(torch.bfloat16)
        cos, sin = torch.rand(T, 48, generator=g), torch.rand(T, 48, generator=g)
        ref = O.linear_qk_prologue(x, w, gam, bet, cos, sin)
        out = mb.linear_qk_norm_rope(x.cuda(), w.cuda(), gam, bet, cos, sin)
        assert_close(out, ref, max_abs=MAX_ABS, min_cos=MIN_COS, what=f"T {T} K {K} H {H}")
        x8, w8 = (x.float() * 4).to(torch.float8_e4m3fn), (w.float() * 64).to(torch.float8_e4m3fn)
        y = ((x8.float() @ w8.float().t()) * (0.25 / 64)).to(torch.bfloat16).view(T, H, 128)
        out8 = mb.linear_qk_norm_rope(x8.cuda(), w8.cuda(), gam, bet, cos, sin, x_scale=torch.tensor([0.25]), w_scale=torch.tensor([1 / 64.]))
        assert_close(out8, O.qk_prologue(y, gam, bet, cos, sin), max_abs=MAX_ABS, min_cos=MIN_COS, what=f"e4m3 T {T} K {K} H {H}")
        if H % 2 == 0:
            bufs = [torch.zeros(T + 3, H // 2, 128, dtype=torch.bfloat16, device="cuda") for _ in range(2)]
            mb.linear_qk_norm_rope(x.cuda(), w.cuda(), gam, bet, cos, sin, heads_per_block=H // 2,
                                   block_out=([b[3:].data_ptr() for b in bufs], bufs[0].stride(0), bufs[0].stride(1)))
            torch.cuda.synchronize()
            assert torch.equal(torch.cat([b[3:] for b in bufs], dim=1), out) and all(float(b[:3].abs().max()) == 0 for b in bufs)
    assert mb.Context.get().status() == 0


@pytest.mark.parametrize("form", ["solo", "pair"])
def test_q_k_v_in_one_launch_equals_three_launches(mb, form, monkeypatch):
    """get_qkv (dit_module.py:998-1003): three weights, two norm parameter sets and three destinations in one kernel; odd
    head counts (each projection's last channel block is half empty) and a K|V fused destination.  Per tile the
    arithmetic is that of the single-projection launches, so the bytes are the same."""
    g = torch.Generator().manual_seed(47)
    T, K, Hq, Hkv = 1500, 512, 5, 3
    x = torch.randn(T, K, generator=g).to(torch.bfloat16).cuda()
    wq, wk, wv = [(torch.randn(h * 128, K, generator=g) * K ** -0.5).to(torch.bfloat16).cuda() for h in (Hq, Hkv, Hkv)]
    gq, bq, gk, bk = O.make_norm_params(9)
    cos, sin = torch.rand(T, 48, generator=g), torch.rand(T, 48, generator=g)
    monkeypatch.setenv("MAGI_LINEAR_FORM", form)
    kv = torch.zeros(T, Hkv, 256, dtype=torch.bfloat16, device="cuda")
    q, k, v = mb.linear_qkv_norm_rope(x, [dict(weight=wq, gamma=gq, beta=bq), dict(weight=wk, gamma=gk, beta=bk, out=kv[:, :, :128]),
                                          dict(weight=wv, norm_mode="none", out=kv[:, :, 128:])], cos, sin)
    torch.cuda.synchronize()
    assert mb.Context.get().status() == 0
    assert torch.equal(q, mb.linear_qk_norm_rope(x, wq, gq, bq, cos, sin))
    assert torch.equal(kv[:, :, :128], mb.linear_qk_norm_rope(x, wk, gk, bk, cos, sin))
    assert torch.equal(kv[:, :, 128:], mb.linear_qk_norm_rope(x, wv, None, None, None, None, norm_mode="none"))
    assert_close(q, O.linear_qk_prologue(x.cpu(), wq.cpu(), gq, bq, cos, sin), max_abs=MAX_ABS, min_cos=MIN_COS, what="q of qkv")
    with pytest.raises(ValueError):
        mb.linear_qkv_norm_rope(x, [dict(weight=wq, gamma=gq, beta=bq), dict(weight=wk[:, :256].contiguous(), gamma=gk, beta=bk)], cos, sin)


def test_all_four_members_of_linear_qkv_in_one_launch(mb):
    """q, qx, k, v (CustomLayerNormLinear, dit_module.py:404): the cross-attention query qx is normed by its own LayerNorm
    and NOT rotated (get_xqkv, :1005-1008) while q and k are; one launch against four single-projection launches."""
    g = torch.Generator().manual_seed(53)
    T, K, Hq, Hkv = 900, 256, 4, 2
    x = torch.randn(T, K, generator=g).to(torch.bfloat16).cuda()
    wq, wqx, wk, wv = [(torch.randn(h * 128, K, generator=g) * K ** -0.5).to(torch.bfloat16).cuda() for h in (Hq, Hq, Hkv, Hkv)]
    gq, bq, gk, bk = O.make_norm_params(10)
    gx, bx, _, _ = O.make_norm_params(11)
    cos, sin = torch.rand(T, 48, generator=g), torch.rand(T, 48, generator=g)
    q, qx, k, v = mb.linear_qkv_norm_rope(x, [dict(weight=wq, gamma=gq, beta=bq), dict(weight=wqx, gamma=gx, beta=bx, rotate=False),
                                              dict(weight=wk, gamma=gk, beta=bk), dict(weight=wv, norm_mode="none")], cos, sin)
    torch.cuda.synchronize()
    assert mb.Context.get().status() == 0
    assert torch.equal(q, mb.linear_qk_norm_rope(x, wq, gq, bq, cos, sin))
    assert torch.equal(qx, mb.linear_qk_norm_rope(x, wqx, gx, bx, None, None))
    assert torch.equal(k, mb.linear_qk_norm_rope(x, wk, gk, bk, cos, sin))
    assert torch.equal(v, mb.linear_qk_norm_rope(x, wv, None, None, None, None, norm_mode="none"))
    y = O.linear_qk_prologue(x.cpu(), wqx.cpu(), None, None, None, None, norm_mode="none")
    assert_close(qx, O.layer_norm_1p(y, gx, bx, 1e-6), max_abs=MAX_ABS, min_cos=MIN_COS, what="qx: norm, no rotary")


def test_projection_at_the_720p_shape(mb):
    """86400 tokens x 6144 features -> 48 + 8 + 8 heads in one launch (the shape bench.py times): sampled rows against the
    oracle (tile and pair edges, the last ragged tile, random rows)."""
    g = torch.Generator(device="cuda").manual_seed(59)
    T, K, Hq, Hkv = 86400, 6144, 48, 8
    x = torch.randn(T, K, generator=g, device="cuda").to(torch.bfloat16)
    wq, wk, wv = [(torch.randn(h * 128, K, generator=g, device="cuda") * K ** -0.5).to(torch.bfloat16) for h in (Hq, Hkv, Hkv)]
    gq, bq, gk, bk = O.make_norm_params(12)
    cos, sin = torch.rand(T, 48, generator=g, device="cuda"), torch.rand(T, 48, generator=g, device="cuda")
    q, k, v = mb.linear_qkv_norm_rope(x, [dict(weight=wq, gamma=gq, beta=bq), dict(weight=wk, gamma=gk, beta=bk),
                                          dict(weight=wv, norm_mode="none")], cos, sin)
    torch.cuda.synchronize()
    assert mb.Context.get().status() == 0
    gc = torch.Generator().manual_seed(59)
    rows = torch.cat([torch.tensor([0, 127, 128, 255, 256, T - 129, T - 128, T - 1]), torch.randint(0, T, (56,), generator=gc)]).cuda()
    xs, cs, sn = x[rows].cpu(), cos[rows].cpu(), sin[rows].cpu()
    assert_close(q[rows], O.linear_qk_prologue(xs, wq.cpu(), gq, bq, cs, sn), max_abs=MAX_ABS, min_cos=MIN_COS, what="720p q")
    assert_close(k[rows], O.linear_qk_prologue(xs, wk.cpu(), gk, bk, cs, sn), max_abs=MAX_ABS, min_cos=MIN_COS, what="720p k")
    assert_close(v[rows], O.linear_qk_prologue(xs, wv.cpu(), None, None, None, None, norm_mode="none"), max_abs=2 ** -5,
                 min_cos=MIN_COS, what="720p v")
    assert torch.isfinite(q.float()).all() and torch.isfinite(k.float()).all()
