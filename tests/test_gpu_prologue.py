"""Parity of the fused norm + RoPE prologue and of the chunk-paged KV cache against the oracle / fixtures."""
import os

import numpy as np
import pytest
import torch

from oracle import chunk_attn_oracle as O
from gpu_util import as_segments, assert_close

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def mb():
    import magi_b200
    return magi_b200


def _bf16(bits):
    return torch.from_numpy(bits.copy()).view(torch.bfloat16)


def test_prologue_matches_reference_fixture(mb, golden_dir):
    z = np.load(os.path.join(golden_dir, "prologue.npz"))
    x = _bf16(z["x"]).cuda()
    out = mb.qk_norm_rope(x, torch.from_numpy(z["gamma"]), torch.from_numpy(z["beta"]), torch.from_numpy(z["cos"]),
                          torch.from_numpy(z["sin"]), eps=1e-6)
    torch.cuda.synchronize()
    ref = _bf16(z["out_bf16"])
    got = out.cpu()
    # same arithmetic order as the reference; only fp32 reduction order / FMA contraction differ -> <= 1 bf16 ulp
    diff = (got.float() - ref.float()).abs()
    assert diff.max().item() <= 2 ** -6, diff.max().item()
    assert (got.view(torch.int16) != ref.view(torch.int16)).float().mean().item() < 5e-3
    assert_close(got, torch.from_numpy(z["out_fp32"]), max_abs=2e-2)


@pytest.mark.parametrize("mode", ["layernorm_1p", "rmsnorm"])
def test_prologue_modes_strides_and_ulysses_layout(mb, mode):
    g = torch.Generator().manual_seed(4)
    T, Hq, Hkv = 531, 12, 4
    # x as a slice of a fused projection output [T, (Hq + 2*Hkv) * 128]
    fused = (torch.randn(T, (Hq + 2 * Hkv) * 128, generator=g) * 2 + 0.5).to(torch.bfloat16).cuda()
    xq = fused[:, :Hq * 128].view(T, Hq, 128)
    xk = fused[:, Hq * 128:(Hq + Hkv) * 128].view(T, Hkv, 128)
    gq, bq, gk, bk = O.make_norm_params(4)
    sin, cos = O.rope_table(3, 3, 59)
    assert sin.shape[0] == T
    for x, gam, bet, H in ((xq, gq, bq, Hq), (xk, gk, bk, Hkv)):
        ref = O.qk_prologue(x.cpu(), gam, bet, cos, sin, norm_mode=mode)
        out = mb.qk_norm_rope(x, gam, bet, cos, sin, norm_mode=mode)
        torch.cuda.synchronize()
        d = (out.cpu().float() - ref.float()).abs().max().item()
        assert d <= 2 ** -5, d
        assert O.cosine(out.cpu(), ref) > 0.99999
        # Ulysses send layout: "(cp seq) hn hd"
        cp = 4
        send = torch.zeros(cp, T, H // cp, 128, dtype=torch.bfloat16, device="cuda")
        mb.qk_norm_rope(x, gam, bet, cos, sin, norm_mode=mode, out=send, heads_per_block=H // cp)
        torch.cuda.synchronize()
        want = out.view(T, cp, H // cp, 128).transpose(0, 1)
        assert torch.equal(send, want.contiguous())


def test_head_block_copy_for_v(mb):
    g = torch.Generator().manual_seed(6)
    T, H = 300, 8
    kv = torch.randn(T, H, 256, generator=g).to(torch.bfloat16).cuda()
    v = kv[..., 128:]
    send = torch.zeros(2, T, 4, 128, dtype=torch.bfloat16, device="cuda")
    mb.head_block_copy(v, send, heads_per_block=4)
    torch.cuda.synchronize()
    assert torch.equal(send, v.reshape(T, 2, 4, 128).transpose(0, 1).contiguous())


def test_kv_cache_roundtrip_evict_and_capacity(mb):
    C, Hkv = 300, 2
    cache = mb.ChunkPagedKVCache(n_layers=2, max_chunks=2, chunk_tokens=C, n_kv_heads=Hkv)
    g = torch.Generator().manual_seed(8)
    kv = [torch.randn(C, Hkv, 256, generator=g).to(torch.bfloat16).cuda() for _ in range(3)]
    cache.append_kv(0, 5, kv[0])
    cache.append_kv(1, 5, kv[1])
    cache.append_kv(0, 9, kv[2][:100])              # partial page, then the rest at an offset
    cache.append_kv(0, 9, kv[2][100:], token_offset=100)
    torch.cuda.synchronize()
    k, v = cache.read(0, 5)
    assert torch.equal(k, kv[0][..., :128]) and torch.equal(v, kv[0][..., 128:])
    k, v = cache.read(1, 5)
    assert torch.equal(k, kv[1][..., :128])
    k, v = cache.read(0, 9, n_tokens=50, token_offset=90)
    assert torch.equal(v, kv[2][90:140, :, 128:])
    with pytest.raises(mb.MagiError) as e:            # both pages taken
        cache.append_kv(0, 11, kv[0])
    assert e.value.code == mb._lib.E_NOMEM
    with pytest.raises(mb.MagiError) as e:            # chunk too long
        cache.append_kv(0, 5, torch.cat([kv[0], kv[0]]))
    assert e.value.code == mb._lib.E_RANGE
    cache.evict(5)
    cache.append_kv(0, 11, kv[1])
    torch.cuda.synchronize()
    k, v = cache.read(0, 11)
    assert torch.equal(k, kv[1][..., :128])
    with pytest.raises(mb.MagiError):
        cache.read(0, 5)
    cache.close()


@pytest.mark.parametrize("impl", ["tcgen05", "simt"])
def test_attention_reads_prefix_pages_in_place(mb, impl):
    """Reference-shaped decode step: prefix = slice_point cached chunks, k_range over (prefix | current)
    (dit_module.py:891-931) vs the oracle's flat-buffer restatement."""
    C, Hq, Hkv, n_layers = 333, 6, 2, 2
    g = torch.Generator().manual_seed(12)
    clean = [torch.randn(C, Hkv, 256, generator=g).to(torch.bfloat16) for _ in range(3)]   # chunks 0..2, clean
    cur_kv = torch.randn(2 * C, Hkv, 256, generator=g).to(torch.bfloat16)                  # chunks 3,4 denoising
    q = torch.randn(2 * C, Hq, 128, generator=g).to(torch.bfloat16)
    ref_cache = O.RefKVCache(5 * C, Hkv)
    ref_cache.buf[:3 * C] = torch.cat(clean).float()
    k_ref, v_ref = ref_cache.adjust(cur_kv.float(), slice_point=3, chunk_tokens=C, update=False)
    qr = O.consecutive_q_ranges(2, C)
    for kr in (O.default_k_ranges(2, C, slice_point=3),
               np.array([[1 * C, 4 * C], [2 * C, 5 * C]], dtype=np.int32)):               # windowed: k-start > 0
        ref, _ = O.range_attention(q.float(), k_ref, v_ref, qr, as_segments(kr))
        cache = mb.ChunkPagedKVCache(n_layers=n_layers, max_chunks=4, chunk_tokens=C, n_kv_heads=Hkv)
        # pages are filled out of order and chunk 7 is a decoy so that slot != chunk id
        cache.append_kv(1, 7, clean[0].cuda())
        for cid in (2, 0, 1):
            cache.append_kv(1, cid, clean[cid].cuda())
        cd = cur_kv.cuda()
        out, _ = mb.chunk_attn(q.cuda(), cd[..., :128], cd[..., 128:], qr, kr, C, 5 * C, cache=cache, layer=1,
                               prefix_chunk_ids=[0, 1, 2], impl=impl)
        torch.cuda.synchronize()
        assert mb.Context.get().status() == 0
        assert_close(out, ref, what=f"paged prefix {impl}")
        cache.close()


def test_attention_with_prefix_only(mb):
    """All keys come from the cache (total_k = 0)."""
    C, Hkv = 260, 2
    g = torch.Generator().manual_seed(14)
    kv = torch.randn(C, Hkv, 256, generator=g).to(torch.bfloat16)
    q = torch.randn(100, 4, 128, generator=g).to(torch.bfloat16)
    cache = mb.ChunkPagedKVCache(1, 1, C, Hkv)
    cache.append_kv(0, 0, kv.cuda())
    qr = np.array([[0, 100]], dtype=np.int32)
    kr = np.array([[0, C]], dtype=np.int32)
    out, _ = mb.chunk_attn(q.cuda(), None, None, qr, kr, 100, C, cache=cache, layer=0, prefix_chunk_ids=[0])
    torch.cuda.synchronize()
    ref, _ = O.range_attention(q.float(), kv[..., :128].float(), kv[..., 128:].float(), qr, as_segments(kr))
    assert_close(out, ref, what="prefix only")
    cache.close()
