"""Ulysses context-parallel attention on 2 (or 4) GPUs of one box against the single-sequence CPU oracle.
Skipped when fewer than 2 GPUs are visible.  NVLS is switched off for the child ranks."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _reference_head_order(ref, cp, hkv_loc, overlap):
    """What the reference's torch.cat over the head groups (context_parallel.py:594) does to the head order inside each
    rank's block: (kv head, group, sub-head) -> (group, kv head, sub-head)."""
    s, hq, d = ref.shape
    gsub = hq // (cp * hkv_loc * overlap)
    return ref.view(s, cp, hkv_loc, overlap, gsub, d).permute(0, 1, 3, 2, 4, 5).reshape(s, hq, d)


def _worker(rank, world, port, mode):
    for p in (ROOT, os.path.join(ROOT, "magi-1_b200"), os.path.join(ROOT, "tests")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    import magi_b200 as mb
    from magi_b200 import host
    from magi_b200.ulysses import FusedUlyssesAttention, UlyssesAttention
    from oracle import chunk_attn_oracle as O
    from gpu_util import as_segments, assert_close, oracle_on_rows

    overlap, fp8, fused = mode.get("overlap", 1), mode.get("fp8", False), mode.get("fused", False)
    proj, exchange, cached = mode.get("proj", False), mode.get("exchange", "torch"), mode.get("cache", False)
    xattn, head_order = mode.get("xattn", False), mode.get("head_order", "reference")
    C, n, Hq, Hkv = (384 if cached and fp8 else 331), 3, 8, 4     # 993 tokens: uneven split over 2 and 4 ranks
    S = C * n
    g = torch.Generator().manual_seed(77)
    xq = torch.randn(S, Hq, 128, generator=g).to(torch.bfloat16)
    xk = torch.randn(S, Hkv, 128, generator=g).to(torch.bfloat16)
    xv = torch.randn(S, Hkv, 128, generator=g).to(torch.bfloat16)
    gq, bq, gk, bk = host.synthetic_norm_params(7)
    sin, cos = host.split_sin_cos(host.rotary_table(3, 1, C))
    splits = host.cp_split_sizes(S, world)
    off = sum(splits[:rank])
    sl = slice(off, off + splits[rank])
    qr, kr = host.q_ranges_for_chunks(n, C), host.default_k_ranges(n, C)
    if mode.get("empty_range"):
        kr = kr.copy()
        kr[1] = [C, C]                    # chunk 1 has no keys: its rows are zeros, on whichever rank owns them
    dev = torch.device("cuda", rank)
    ua = FusedUlyssesAttention(dist.group.WORLD, Hq, Hkv, splits, proj_hn=8 if proj else 0, n_out_buffers=2) if fused else \
        UlyssesAttention(dist.group.WORLD, Hq, Hkv, splits, overlap_degree=overlap, exchange=exchange, head_order=head_order)
    q_ref = O.qk_prologue(xq, gq, bq, cos, sin).float()
    k_ref = O.qk_prologue(xk, gk, bk, cos, sin).float()

    kw = {}
    cache = None
    if cached:
        # chunks 0 and 1 are clean: their K/V (this rank's KV heads, all tokens) live in a head-sharded page cache
        # (dit_module.py:794-798), only chunk 2's K/V count as current
        hkv_loc = Hkv // world
        hs = slice(rank * hkv_loc, (rank + 1) * hkv_loc)
        cache = mb.ChunkPagedKVCache(n_layers=2, max_chunks=2, chunk_tokens=C, n_kv_heads=hkv_loc, dtype="fp8" if fp8 else "bf16", device=rank)
        for cid in (1, 0):
            cache.append(1, cid, k_ref[cid * C:(cid + 1) * C, hs].to(torch.bfloat16).to(dev).contiguous(),
                         xv[cid * C:(cid + 1) * C, hs].to(dev).contiguous())
        kw = dict(cache=cache, layer=1, prefix_chunk_ids=[0, 1], kv_current_offset=2 * C)
    if fp8:
        kw["fp8_chunk_tokens"] = C
    cross = None
    if xattn:
        caps = [50, 0, 120]
        yk = torch.randn(sum(caps), Hkv, 128, generator=g).to(torch.bfloat16).to(dev)
        yv = torch.randn(sum(caps), Hkv, 128, generator=g).to(torch.bfloat16).to(dev)
        xqr, xkr = host.cross_attn_ranges(C, n, caps)
        ql, kl, max_q = host.cp_cross_attn_ranges(xqr, xkr, splits, rank)
        q_loc = q_ref[sl].to(torch.bfloat16).to(dev)
        if fused:
            def cross(dest, ctx):
                assert torch.cuda.current_stream() != torch.cuda.default_stream()   # the slot runs beside the barrier
                return mb.chunk_attn(q_loc, yk, yv, ql, kl, max_q, max(caps), return_lse=False, ctx=ctx, **dest)[0]
        else:
            def cross():
                return mb.chunk_attn(q_loc, yk, yv, ql, kl, max_q, max(caps), return_lse=False)[0]
        kw["cross_attn_func"] = cross

    x_in = (xq[sl].to(dev), xk[sl].to(dev), xv[sl].to(dev))
    if mode.get("from_hidden"):
        # the projections run inside the exchange: hidden states and weights in, the oracle gets the exactly rounded
        # projections (the GEMM's accumulation order is the only difference)
        hidden = 256
        xh = (torch.randn(S, hidden, generator=g) * 1.5).to(torch.bfloat16)
        ws = [(torch.randn(h * 128, hidden, generator=g) * hidden ** -0.5).to(torch.bfloat16) for h in (Hq, Hkv, Hkv)]
        xq, xk, xv = [(xh.double() @ w_.double().t()).to(torch.bfloat16).view(S, -1, 128) for w_ in ws]
        q_ref = O.qk_prologue(xq, gq, bq, cos, sin).float()
        k_ref = O.qk_prologue(xk, gk, bk, cos, sin).float()
        x_in = (xh[sl].to(dev), None, None)
        kw["proj_weights"] = tuple(w_.to(dev) for w_ in ws)
    for _ in range(3):  # later passes reuse (and rotate) the buffers
        res = ua.forward(*x_in, gq, bq, gk, bk, cos[sl], sin[sl],
                         torch.as_tensor(qr, device=dev), torch.as_tensor(kr, device=dev), C, S, **kw)
    out, x_out = res if xattn else (res, None)
    torch.cuda.synchronize()
    assert mb.Context.get(rank).status() == 0
    # oracle on the full sequence, restricted to this rank's rows
    rows, ref, _ = oracle_on_rows(q_ref, k_ref, xv.float(), qr, as_segments(kr), torch.arange(off, off + splits[rank]))
    if mode.get("empty_range"):
        own = torch.arange(off, off + splits[rank])
        full = torch.zeros(splits[rank], Hq, 128)
        full[torch.isin(own, rows)] = ref
        ref = full
        assert (out[((own >= C) & (own < 2 * C)).to(dev)].float() == 0).all()
    else:
        assert torch.equal(rows, torch.arange(off, off + splits[rank]))
    if xattn:
        x_ref, _ = mb.chunk_attn(q_loc, yk, yv, ql, kl, max_q, max(caps), return_lse=False)
        torch.cuda.synchronize()
    if proj:
        # the result buffer is the projection operand: core heads at their "(hn n hd)" columns, and the rank-local
        # cross-attention (run in the schedule's cross-attention slot, on a side stream with a context of its own)
        # fills the other half in place
        from magi_b200.inference import ProjInput
        assert out.shape == (splits[rank], 2 * Hq * 128)
        core_cols = torch.arange(2 * Hq * 128).view(8, 2, -1)[:, 0].reshape(-1).to(dev)
        core = out[:, core_cols].reshape(splits[rank], Hq, 128)
        assert_close(core, ref, what=f"fused ulysses cp{world} rank {rank}, projection layout")
        assert torch.equal(out, ProjInput.reference_layout(core, x_ref))
    elif fp8:
        assert O.cosine(out.cpu(), ref) >= 0.999, O.cosine(out.cpu(), ref)
    else:
        if not fused and overlap > 1 and head_order == "reference":
            ref = _reference_head_order(ref, world, Hkv // world, overlap)
        assert_close(out, ref, what=f"ulysses cp{world} rank {rank} {mode}")
        if xattn:
            assert torch.equal(x_out, x_ref)
    if fused:
        out = out.clone()
        ua.close()
    elif exchange == "library":
        ua.ex.close()
    if cache is not None:
        cache.close()
    dist.barrier()
    dist.destroy_process_group()


def _spawn(world, **mode):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(world, _free_port(), mode), nprocs=world, join=True)


@pytest.mark.parametrize("world", [2, 4])
def test_fused_peer_memory_exchange_matches_oracle(world):
    """Prologue and attention epilogue store straight into the peers' buffers (CUDA IPC, no all-to-all)."""
    _spawn(world, fused=True)


def test_fused_exchange_writes_the_projection_operand_with_the_cross_attention_slot():
    """attn_linear_proj's cat + rearrange (dit_module.py:1332-1346) folded into the fused output exchange; the
    cross-attention fills its half from the schedule's slot (context_parallel.py:584-591)."""
    _spawn(2, fused=True, proj=True, xattn=True)


def test_fused_exchange_from_hidden_states():
    """Projection GEMM -> prologue -> head exchange in one kernel per projection (peer stores from the GEMM's epilogue)."""
    _spawn(2, fused=True, from_hidden=True)


def test_fused_exchange_with_a_head_sharded_paged_prefix():
    """KV cache under context parallelism: the cache holds Hkv/cp heads per rank (dit_module.py:794-798)."""
    _spawn(2, fused=True, cache=True)


def test_fused_exchange_fp8_with_fp8_pages():
    _spawn(2, fused=True, cache=True, fp8=True)


def test_fused_exchange_empty_key_range():
    """A q-range without keys under the fused output exchange: zeros reach the owning rank's buffer."""
    _spawn(2, fused=True, empty_range=True)


@pytest.mark.parametrize("world,overlap,head_order", [(2, 1, "reference"), (2, 2, "reference"), (2, 2, "original"), (4, 1, "reference")])
def test_ulysses_attention_matches_oracle(world, overlap, head_order):
    _spawn(world, overlap=overlap, head_order=head_order)


def test_ulysses_attention_with_a_head_sharded_paged_prefix():
    _spawn(2, cache=True)


def test_ulysses_attention_cross_attention_slot():
    _spawn(2, overlap=2, xattn=True)


def test_exchange_through_the_library_owned_communicator():
    """magi_ulysses_* (grouped ncclSend / ncclRecv on a communicator created from a broadcast unique id)."""
    _spawn(2, overlap=2, exchange="library")


def test_ulysses_fp8_attention_matches_oracle():
    _spawn(2, fp8=True)
