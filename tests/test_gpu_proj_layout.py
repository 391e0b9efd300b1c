"""Head-block output layout: core and cross attention store their heads straight into the operand of the output
projection, i.e. the reference's cat + rearrange "sq b (n hn hd) -> sq b (hn n hd)", n=2, hn=8 (attn_linear_proj,
inference/model/dit/dit_module.py:1332-1346) costs no extra pass.  The values must be bit-identical to the plain
[tokens, heads, 128] output of the same kernel."""
import numpy as np
import pytest
import torch

from gpu_util import assert_close, as_segments
from oracle import chunk_attn_oracle as O

pytestmark = pytest.mark.gpu


def _problem(C, n, Hq, Hkv, caps, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(n * C, Hq, 128, generator=g).to(torch.bfloat16).cuda()
    k = torch.randn(n * C, Hkv, 128, generator=g).to(torch.bfloat16).cuda()
    v = torch.randn(n * C, Hkv, 128, generator=g).to(torch.bfloat16).cuda()
    xk = torch.randn(sum(caps), Hkv, 128, generator=g).to(torch.bfloat16).cuda()
    xv = torch.randn(sum(caps), Hkv, 128, generator=g).to(torch.bfloat16).cuda()
    return q, k, v, xk, xv


@pytest.mark.parametrize("impl", ["tcgen05", "simt"])
def test_core_and_cross_attention_write_the_projection_operand(impl):
    import magi_b200 as mb
    from magi_b200 import host
    from magi_b200.inference import ProjInput
    C, n, Hq, Hkv = 300, 3, 16, 4                  # 16 heads -> hn=8 blocks of 2 heads; ragged 300-token chunks
    caps = [77, 0, 130]
    q, k, v, xk, xv = _problem(C, n, Hq, Hkv, caps, 71)
    qr, kr = host.q_ranges_for_chunks(n, C), host.default_k_ranges(n, C)
    xqr, xkr = host.cross_attn_ranges(C, n, caps)
    core, _ = mb.chunk_attn(q, k, v, qr, kr, C, n * C, impl=impl)
    cross, _ = mb.chunk_attn(q, xk, xv, xqr, xkr, C, max(caps), impl=impl)
    pi = ProjInput(n * C, Hq, "cuda")
    pi.buf.fill_(7.0)
    mb.chunk_attn(q, k, v, qr, kr, C, n * C, impl=impl, return_lse=False, **pi.dest(0))
    mb.chunk_attn(q, xk, xv, xqr, xkr, C, max(caps), impl=impl, return_lse=False, **pi.dest(1))
    torch.cuda.synchronize()
    assert mb.Context.get().status() == 0
    want = ProjInput.reference_layout(core, cross)
    assert want.shape == pi.buf.shape == (n * C, 2 * Hq * 128)
    assert torch.equal(pi.buf, want)               # every column written, every value the plain kernel's
    # and the plain outputs themselves are right
    ref, _ = O.range_attention(q.cpu().float(), k.cpu().float(), v.cpu().float(), qr, as_segments(kr))
    assert_close(core, ref, what="core attention")


def test_layer_mirror_forward_into_projection_operand():
    import magi_b200 as mb
    from magi_b200 import host
    from magi_b200.inference import (ChunkCausalSelfAttention, ModelMetaArgs, PackedCoreAttnParams, ProjInput)
    T, H, W, n, Hq, Hkv = 2, 6, 10, 2, 8, 2       # chunk = 120 tokens, hn=8 blocks of one head
    C = T * H * W
    g = torch.Generator().manual_seed(72)
    xq = torch.randn(n * C, Hq, 128, generator=g).to(torch.bfloat16).cuda()
    xk = torch.randn(n * C, Hkv, 128, generator=g).to(torch.bfloat16).cuda()
    xv = torch.randn(n * C, Hkv, 128, generator=g).to(torch.bfloat16).cuda()
    gq, bq, gk, bk = host.synthetic_norm_params(72)
    table = host.rotary_table(n * T, H, W)
    layer = ChunkCausalSelfAttention(0, Hq, Hkv, gq, bq, gk, bk)
    params = PackedCoreAttnParams.from_numpy(host.q_ranges_for_chunks(n, C), host.default_k_ranges(n, C), "cuda")
    meta = ModelMetaArgs(slice_point=0, denoising_range_num=n, clip_token_nums=C, core_attn_params=params)
    rope = table.cuda()
    plain = layer.forward(xq, xk, xv, None, rope, meta)
    pi = ProjInput(n * C, Hq, "cuda")
    got = layer.forward(xq, xk, xv, None, rope, meta, proj_in=pi)
    torch.cuda.synchronize()
    assert got is pi.buf
    # only the core half is written by this call: compare those columns with the reference layout of (plain, zeros)
    want = ProjInput.reference_layout(plain, torch.zeros_like(plain))
    cols = torch.arange(2 * Hq * 128).view(8, 2, -1)[:, 0].reshape(-1).cuda()
    assert torch.equal(pi.buf[:, cols], want[:, cols])


def test_head_block_layout_argument_errors():
    import magi_b200 as mb
    from magi_b200 import host
    q, k, v, _, _ = _problem(128, 1, 8, 2, [1], 73)
    qr, kr = host.q_ranges_for_chunks(1, 128), host.default_k_ranges(1, 128)
    with pytest.raises(ValueError):                # 3-D out with the layout switched on
        mb.chunk_attn(q, k, v, qr, kr, 128, 128, out=torch.empty_like(q), out_heads_per_block=1, out_block_stride=256)
    with pytest.raises(ValueError):                # rows too narrow for the last block
        mb.chunk_attn(q, k, v, qr, kr, 128, 128, out=torch.empty(128, 8 * 128, dtype=torch.bfloat16, device="cuda"),
                      out_heads_per_block=1, out_block_stride=256)
    with pytest.raises(mb.MagiError):              # block stride not a multiple of 8 elements: rejected by the library
        mb.chunk_attn(q, k, v, qr, kr, 128, 128, out=torch.empty(128, 4096, dtype=torch.bfloat16, device="cuda"),
                      out_heads_per_block=1, out_block_stride=260)
