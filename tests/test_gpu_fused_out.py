"""The fused output exchange of the attention epilogue (the "gather heads" all-to-all of
inference/infra/parallelism/context_parallel.py:404-423 and the re-layout at :596 folded into the store address) on ONE
GPU: the peer table names two local buffers standing for the result buffers of two context-parallel ranks, so the
addressing - owner of a token, row inside the owner's buffer, this rank's global head position - is checked without a
second device.  Covers the bf16 kernel, the FP8 kernel, and a q-range without keys (zeros must land in the owner's
buffer, not behind the unused `out` pointer)."""
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


def _buffers(splits, h_total):
    return [torch.full((s, h_total, 128), 7.0, dtype=torch.bfloat16, device="cuda") for s in splits]


def _gathered(bufs, head_off, hq):
    return torch.cat([b[:, head_off:head_off + hq] for b in bufs])


@pytest.mark.parametrize("fp8", [False, True])
def test_rows_land_in_the_owning_ranks_buffer(mb, fp8):
    C, n, Hq, Hkv = 300, 3, 4, 2
    S = C * n
    g = torch.Generator().manual_seed(11)
    q = torch.randn(S, Hq, 128, generator=g).to(torch.bfloat16).cuda()
    k = torch.randn(S, Hkv, 128, generator=g).to(torch.bfloat16).cuda()
    v = torch.randn(S, Hkv, 128, generator=g).to(torch.bfloat16).cuda()
    qr, kr = O.consecutive_q_ranges(n, C), O.default_k_ranges(n, C)
    splits, head_off, h_total = [391, S - 391], 4, 12        # this "rank" owns global heads 4..7 of 12
    bufs = _buffers(splits, h_total)
    peers = ([b.data_ptr() for b in bufs], [0, splits[0], S], head_off, h_total * 128, 128)
    kw = {}
    if fp8:
        q8, qs, q8lo = mb.quantize_e4m3(q, C, residual=True)
        k8, ks = mb.quantize_e4m3(k, C)
        v8, vs = mb.quantize_e4m3(v, C)
        kw = dict(q_scale=qs, k_scale=ks, v_scale=vs, scale_chunk_tokens=C, q_lo=q8lo)
        plain, _ = mb.chunk_attn(q8, k8, v8, qr, kr, C, S, return_lse=False, **kw)
        mb.chunk_attn(q8, k8, v8, qr, kr, C, S, o_peers=peers, **kw)
    else:
        plain, _ = mb.chunk_attn(q, k, v, qr, kr, C, S, return_lse=False)
        mb.chunk_attn(q, k, v, qr, kr, C, S, o_peers=peers)
    torch.cuda.synchronize()
    assert mb.Context.get().status() == 0
    got = _gathered(bufs, head_off, Hq)
    assert torch.equal(got, plain)                                   # same kernel, same arithmetic: bit-equal
    for b in bufs:                                                   # other ranks' head columns are untouched
        assert (b[:, :head_off].float() == 7).all() and (b[:, head_off + Hq:].float() == 7).all()
    ref, _ = O.range_attention(q.float().cpu(), k.float().cpu(), v.float().cpu(), qr, as_segments(kr))
    if fp8:
        assert O.cosine(got.cpu(), ref) >= 0.999
    else:
        assert_close(got, ref, what="fused output exchange, one GPU")


def test_empty_key_range_stores_zeros_at_the_peer_destination(mb):
    Hq, Hkv, T = 2, 1, 520
    g = torch.Generator().manual_seed(12)
    q = torch.randn(T, Hq, 128, generator=g).to(torch.bfloat16).cuda()
    k = torch.randn(T, Hkv, 128, generator=g).to(torch.bfloat16).cuda()
    v = torch.randn(T, Hkv, 128, generator=g).to(torch.bfloat16).cuda()
    qr = np.array([[0, 200], [200, 460], [460, 520]], dtype=np.int32)
    kr = np.array([[0, 300], [77, 77], [100, 520]], dtype=np.int32)   # the middle range has no keys
    splits = [250, T - 250]                                            # the empty range straddles both owners
    bufs = _buffers(splits, Hq)
    mb.chunk_attn(q, k, v, qr, kr, 260, T, o_peers=([b.data_ptr() for b in bufs], [0, 250, T], 0, Hq * 128, 128))
    torch.cuda.synchronize()
    assert mb.Context.get().status() == 0
    got = _gathered(bufs, 0, Hq)
    assert (got[200:460].float() == 0).all()
    ref, _ = O.range_attention(q.float().cpu(), k.float().cpu(), v.float().cpu(), qr, as_segments(kr))
    assert_close(got, ref, what="empty k range with a peer table")


def test_unsupported_combinations_are_refused_on_the_host(mb):
    """lse together with a peer table, and the diagnostic kernel with a peer table, return MAGI_E_BADARG before anything
    is launched (the output pointer may legitimately be NULL in such a call)."""
    q = torch.zeros(128, 2, 128, dtype=torch.bfloat16, device="cuda")
    buf = torch.zeros(128, 2, 128, dtype=torch.bfloat16, device="cuda")
    r = np.array([[0, 128]], dtype=np.int32)
    peers = ([buf.data_ptr()], [0, 128], 0, 256, 128)
    with pytest.raises(mb.MagiError) as e:
        mb.chunk_attn(q, q, q, r, r, 128, 128, o_peers=peers, impl="simt")
    assert e.value.code == mb._lib.E_BADARG
    with pytest.raises(mb.MagiError) as e:   # offsets that do not cover total_q
        mb.chunk_attn(q, q, q, r, r, 128, 128, o_peers=([buf.data_ptr()], [0, 64], 0, 256, 128))
    assert e.value.code == mb._lib.E_RANGE
    torch.cuda.synchronize()
    assert mb.Context.get().status() == 0 and (buf.float() == 0).all()
