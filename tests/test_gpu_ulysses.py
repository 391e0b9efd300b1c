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


def _worker(rank, world, port, overlap, fp8=False, fused=False, proj=False, exchange="torch"):
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

    C, n, Hq, Hkv = 331, 3, 8, 4          # 993 tokens: uneven split over 2 and 4 ranks
    S = C * n
    g = torch.Generator().manual_seed(77)
    xq = torch.randn(S, Hq, 128, generator=g).to(torch.bfloat16)
    xk = torch.randn(S, Hkv, 128, generator=g).to(torch.bfloat16)
    xv = torch.randn(S, Hkv, 128, generator=g).to(torch.bfloat16)
    gq, bq, gk, bk = host.synthetic_norm_params(7)
    sin, cos = host.split_sin_cos(host.rotary_table(3, 1, 331))
    splits = host.cp_split_sizes(S, world)
    off = sum(splits[:rank])
    sl = slice(off, off + splits[rank])
    qr, kr = host.q_ranges_for_chunks(n, C), host.default_k_ranges(n, C)
    ua = FusedUlyssesAttention(dist.group.WORLD, Hq, Hkv, splits, proj_hn=8 if proj else 0) if fused else \
        UlyssesAttention(dist.group.WORLD, Hq, Hkv, splits, overlap_degree=overlap, exchange=exchange)
    dev = torch.device("cuda", rank)
    for _ in range(2):  # second pass reuses the buffers
        out = ua.forward(xq[sl].to(dev), xk[sl].to(dev), xv[sl].to(dev), gq, bq, gk, bk, cos[sl], sin[sl],
                         torch.as_tensor(qr, device=dev), torch.as_tensor(kr, device=dev), C, S,
                         **({"fp8_chunk_tokens": C} if fp8 else {}))
    torch.cuda.synchronize()
    assert mb.Context.get(rank).status() == 0
    # oracle on the full sequence, restricted to this rank's rows
    q_ref = O.qk_prologue(xq, gq, bq, cos, sin).float()
    k_ref = O.qk_prologue(xk, gk, bk, cos, sin).float()
    rows, ref, _ = oracle_on_rows(q_ref, k_ref, xv.float(), qr, as_segments(kr), torch.arange(off, off + splits[rank]))
    assert torch.equal(rows, torch.arange(off, off + splits[rank]))
    if proj:
        # the result buffer is the projection operand: core heads at their "(hn n hd)" columns, and the rank-local
        # cross-attention fills the other half in place
        from magi_b200.inference import ProjInput
        caps = [50, 0, 120]
        yk = torch.randn(sum(caps), Hkv, 128, generator=g).to(torch.bfloat16).to(dev)
        yv = torch.randn(sum(caps), Hkv, 128, generator=g).to(torch.bfloat16).to(dev)
        xqr, xkr = host.cross_attn_ranges(C, n, caps)
        ql, kl, max_q = host.cp_cross_attn_ranges(xqr, xkr, splits, rank)
        q_loc = q_ref[sl].to(torch.bfloat16).to(dev)
        cross, _ = mb.chunk_attn(q_loc, yk, yv, ql, kl, max_q, max(caps))
        mb.chunk_attn(q_loc, yk, yv, ql, kl, max_q, max(caps), return_lse=False, **ua.cross_dest())
        torch.cuda.synchronize()
        assert out.shape == (splits[rank], 2 * Hq * 128)
        core_cols = torch.arange(2 * Hq * 128).view(8, 2, -1)[:, 0].reshape(-1).to(dev)
        core = out[:, core_cols].reshape(splits[rank], Hq, 128)
        assert_close(core, ref, what=f"fused ulysses cp{world} rank {rank}, projection layout")
        assert torch.equal(out, ProjInput.reference_layout(core, cross))
    elif fp8:
        assert O.cosine(out.cpu(), ref) >= 0.999, O.cosine(out.cpu(), ref)
    else:
        assert_close(out, ref, what=f"ulysses cp{world} rank {rank}")
    if fused:
        out = out.clone()
        ua.close()
    elif exchange == "library":
        ua.ex.close()
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_fused_peer_memory_exchange_matches_oracle(world):
    """Prologue and attention epilogue store straight into the peers' buffers (CUDA IPC, no all-to-all)."""
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(world, _free_port(), 1, False, True), nprocs=world, join=True)


def test_fused_exchange_writes_the_projection_operand():
    """attn_linear_proj's cat + rearrange (dit_module.py:1332-1346) folded into the fused output exchange."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port(), 1, False, True, True), nprocs=2, join=True)


@pytest.mark.parametrize("world,overlap", [(2, 1), (2, 2), (4, 1)])
def test_ulysses_attention_matches_oracle(world, overlap):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(world, _free_port(), overlap), nprocs=world, join=True)


def test_exchange_through_the_library_owned_communicator():
    """magi_ulysses_* (grouped ncclSend / ncclRecv on a communicator created from a broadcast unique id)."""
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port(), 2, False, False, False, "library"), nprocs=2, join=True)


def test_ulysses_fp8_attention_matches_oracle():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port(), 1, True), nprocs=2, join=True)
