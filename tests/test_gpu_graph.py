"""The step (prologue + attention, cached prefix included) captured once into a CUDA graph and replayed on new data:
nothing on the path synchronises with the host - ranges and page tables are consumed on the device by the planner
kernel - so a captured step replays with no launch-time work at all."""
import numpy as np
import pytest
import torch

from gpu_util import as_segments, assert_close
from oracle import chunk_attn_oracle as O

pytestmark = pytest.mark.gpu


def test_step_replays_from_a_cuda_graph():
    import magi_b200 as mb
    from magi_b200 import host
    C, n, Hq, Hkv = 384, 3, 8, 2                       # chunk 0 comes from the paged cache, chunks 1..2 are current
    g = torch.Generator().manual_seed(101)
    gq, bq, gk, bk = [t.cuda() for t in host.synthetic_norm_params(101)]
    sin, cos = host.split_sin_cos(host.rotary_table(3, 16, 24))
    sin_d, cos_d = sin[C:].contiguous().cuda(), cos[C:].contiguous().cuda()
    cache = mb.ChunkPagedKVCache(n_layers=1, max_chunks=2, chunk_tokens=C, n_kv_heads=Hkv)
    k0 = torch.randn(C, Hkv, 128, generator=g).to(torch.bfloat16)
    v0 = torch.randn(C, Hkv, 128, generator=g).to(torch.bfloat16)
    cache.append(0, 0, k0.cuda(), v0.cuda())
    T = 2 * C
    xq = torch.empty(T, Hq, 128, dtype=torch.bfloat16, device="cuda")
    xk = torch.empty(T, Hkv, 128, dtype=torch.bfloat16, device="cuda")
    xv = torch.empty(T, Hkv, 128, dtype=torch.bfloat16, device="cuda")
    q_buf, k_buf, out = torch.empty_like(xq), torch.empty_like(xk), torch.empty_like(xq)
    qr_np = host.q_ranges_for_chunks(2, C)
    kr_np = np.array([[0, 2 * C], [0, 3 * C]], dtype=np.int32)      # (cached chunk 0 | current chunks)
    qr, kr = torch.as_tensor(qr_np, device="cuda"), torch.as_tensor(kr_np, device="cuda")

    def step():
        mb.qk_norm_rope(xq, gq, bq, cos_d, sin_d, out=q_buf)
        mb.qk_norm_rope(xk, gk, bk, cos_d, sin_d, out=k_buf)
        mb.chunk_attn(q_buf, k_buf, xv, qr, kr, C, 3 * C, out=out, return_lse=False, cache=cache, layer=0, prefix_chunk_ids=[0])

    def fill(seed):
        gg = torch.Generator().manual_seed(seed)
        a = torch.randn(T, Hq, 128, generator=gg).to(torch.bfloat16)
        b = torch.randn(T, Hkv, 128, generator=gg).to(torch.bfloat16)
        c = torch.randn(T, Hkv, 128, generator=gg).to(torch.bfloat16)
        xq.copy_(a), xk.copy_(b), xv.copy_(c)
        return a, b, c

    fill(1)
    s = torch.cuda.Stream()
    with torch.cuda.stream(s):
        step()                                          # warm-up outside the capture (context set-up, module load)
    torch.cuda.current_stream().wait_stream(s)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    for seed in (2, 3):
        a, b, c = fill(seed)
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert mb.Context.get().status() == 0
        q_ref = O.qk_prologue(a, gq.cpu(), bq.cpu(), cos[C:], sin[C:]).float()
        k_ref = O.qk_prologue(b, gk.cpu(), bk.cpu(), cos[C:], sin[C:]).float()
        k_all = torch.cat([k0.float(), k_ref])
        v_all = torch.cat([v0.float(), c.float()])
        ref, _ = O.range_attention(q_ref, k_all, v_all, qr_np, as_segments(kr_np))
        assert_close(out, ref, what=f"graph replay, seed {seed}")
    cache.close()
