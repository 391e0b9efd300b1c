"""FP8 e4m3 path: block quantiser bit-exact against the oracle's definition, FP8 attention and FP8 cache pages against
the bf16 kernel and the fp32 oracle (cosine >= 0.999, the acceptance bar for the FP8 variant)."""
import numpy as np
import pytest
import torch

from oracle import chunk_attn_oracle as O
from gpu_util import as_segments, assert_close

pytestmark = pytest.mark.gpu
FP8_MIN_COS = 0.999          # acceptance bar, met by the two-term mode (Q and P carried as value + residual)
FP8_SINGLE_MIN_COS = 0.998   # plain e4m3 everywhere: ~2.6 % rms noise per operand gives ~0.9986 on iid N(0,1) data


@pytest.fixture(scope="module")
def mb():
    import magi_b200
    return magi_b200


def test_quantiser_matches_oracle_definition(mb):
    g = torch.Generator().manual_seed(41)
    C, T, H = 300, 700, 3                         # chunks of 300: blocks 128,128,44 | 128,128,44 | 100
    x = (torch.randn(T, H, 128, generator=g) * 2.5).to(torch.bfloat16)
    x[130:140] = 0                                # part of a block is zero
    x[256:300, 1] = 0                             # one whole (block, head) is zero -> scale 1
    x8, sc = mb.quantize_e4m3(x.cuda(), C)
    torch.cuda.synchronize()
    ref8, ref_sc, spans = O.quantize_e4m3_block128(x.float(), [0, 300, 600], 128)
    assert sc.shape == (9, H)
    got_sc = sc.cpu()
    idx = [0, 1, 2, 3, 4, 5, 6]                   # the 7 real blocks; entries 7, 8 are padding of the short last chunk
    assert torch.equal(got_sc[idx], ref_sc)
    a, b = x8.cpu().view(torch.uint8), ref8.view(torch.uint8)
    bad = (a != b)
    assert not bad.any(), f"{int(bad.sum())} of {a.numel()} codes differ, e.g. {a[bad][:8].tolist()} vs {b[bad][:8].tolist()}"


@pytest.mark.parametrize("hq,hkv", [(4, 2), (6, 1)])
def test_fp8_attention_vs_bf16_and_oracle(mb, hq, hkv):
    g = torch.Generator().manual_seed(43 + hq)
    C, n = 520, 3                                 # chunk = 4 full blocks + one of 8 tokens
    S = C * n
    q = torch.randn(S, hq, 128, generator=g).to(torch.bfloat16).cuda()
    k = torch.randn(S, hkv, 128, generator=g).to(torch.bfloat16).cuda()
    v = (torch.randn(S, hkv, 128, generator=g) * torch.linspace(0.2, 3.0, S)[:, None, None]).to(torch.bfloat16).cuda()
    qr, kr = O.consecutive_q_ranges(n, C), O.default_k_ranges(n, C)
    q8, qs, q8lo = mb.quantize_e4m3(q, C, residual=True)
    k8, ks = mb.quantize_e4m3(k, C)
    v8, vs = mb.quantize_e4m3(v, C)
    out1, lse1 = mb.chunk_attn(q8, k8, v8, qr, kr, C, S, q_scale=qs, k_scale=ks, v_scale=vs, scale_chunk_tokens=C)
    out8, lse8 = mb.chunk_attn(q8, k8, v8, qr, kr, C, S, q_scale=qs, k_scale=ks, v_scale=vs, scale_chunk_tokens=C, q_lo=q8lo)
    out16, lse16 = mb.chunk_attn(q, k, v, qr, kr, C, S)
    torch.cuda.synchronize()
    assert mb.Context.get().status() == 0
    ref, ref_lse = O.range_attention(q.float().cpu(), k.float().cpu(), v.float().cpu(), qr, as_segments(kr))
    c1, c2 = O.cosine(out1.cpu(), out16.cpu()), O.cosine(out8.cpu(), out16.cpu())
    print(f"fp8 vs bf16 cosine: single-term {c1:.5f}, two-term {c2:.5f}")
    assert c1 >= FP8_SINGLE_MIN_COS and O.cosine(out1.cpu(), ref) >= FP8_SINGLE_MIN_COS
    assert c2 >= FP8_MIN_COS and O.cosine(out8.cpu(), ref) >= FP8_MIN_COS
    assert (out8.float().cpu() - ref).abs().max().item() < 0.15
    assert torch.allclose(lse8.cpu(), ref_lse, atol=0.1, rtol=0)
    assert torch.allclose(lse1.cpu(), ref_lse, atol=0.1, rtol=0)
    # against the oracle run on the dequantised tensors the only remaining error is P's quantisation
    deq = lambda x8_, s_: O.dequantize_e4m3_block128(x8_.cpu(), s_.cpu()[[i for i in range(s_.shape[0])]],
                                                     [(c * C + b * 128, min(c * C + (b + 1) * 128, (c + 1) * C)) for c in range(n) for b in range(5)])
    ref_dq, _ = O.range_attention(deq(q8, qs), deq(k8, ks), deq(v8, vs), qr, as_segments(kr))
    assert O.cosine(out8.cpu(), ref_dq) >= 0.9995


def test_fp8_cache_pages_roundtrip_and_attention(mb):
    C, Hq, Hkv = 300, 4, 2
    g = torch.Generator().manual_seed(47)
    clean = [torch.randn(C, Hkv, 256, generator=g).to(torch.bfloat16).cuda() for _ in range(3)]
    cur = torch.randn(C, Hkv, 256, generator=g).to(torch.bfloat16).cuda()
    q = torch.randn(C, Hq, 128, generator=g).to(torch.bfloat16).cuda()
    cache = mb.ChunkPagedKVCache(n_layers=1, max_chunks=3, chunk_tokens=C, n_kv_heads=Hkv, dtype="fp8")
    for cid in (1, 0, 2):
        cache.append_kv(0, cid, clean[cid])
    torch.cuda.synchronize()
    k_back, v_back = cache.read(0, 1)
    assert O.cosine(k_back.cpu(), clean[1][..., :128].cpu()) > 0.999
    assert (k_back.float() - clean[1][..., :128].float()).abs().max().item() <= clean[1].float().abs().max().item() / 16 + 1e-3
    with pytest.raises(mb.MagiError) as e:
        cache.append_kv(0, 0, clean[0][:10], token_offset=7)      # fp8 pages are written in 128-token blocks
    assert e.value.code == mb._lib.E_ALIGN
    # chunk 3 (current, fresh fp8) attends to the three fp8 pages and itself
    qr = np.array([[0, C]], dtype=np.int32)
    kr = np.array([[0, 4 * C]], dtype=np.int32)
    q8, qs, q8lo = mb.quantize_e4m3(q, C, residual=True)
    k8, ks = mb.quantize_e4m3(cur[..., :128], C)
    v8, vs = mb.quantize_e4m3(cur[..., 128:], C)
    out8, _ = mb.chunk_attn(q8, k8, v8, qr, kr, C, 4 * C, cache=cache, layer=0, prefix_chunk_ids=[0, 1, 2],
                            q_scale=qs, k_scale=ks, v_scale=vs, scale_chunk_tokens=C, q_lo=q8lo)
    torch.cuda.synchronize()
    assert mb.Context.get().status() == 0
    kv_all = torch.cat(clean + [cur]).float().cpu()
    ref, _ = O.range_attention(q.float().cpu(), kv_all[..., :128], kv_all[..., 128:], qr, as_segments(kr))
    assert O.cosine(out8.cpu(), ref) >= FP8_MIN_COS
    # a bf16 call must refuse an fp8 cache
    with pytest.raises(mb.MagiError):
        mb.chunk_attn(q, cur[..., :128], cur[..., 128:], qr, kr, C, 4 * C, cache=cache, layer=0, prefix_chunk_ids=[0, 1, 2])
    cache.close()
