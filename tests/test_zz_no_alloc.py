"""The allocation-free attention entry point against the regular one, through the C ABI.

Some hosts of this library cannot allocate on the GPU once they are running - all of HBM already belongs to their own
pools - so magi_chunk_attn_fwd_noalloc plans in a fixed array inside the library instead of a context's workspace.
The array survives from call to call, so the check is made on two different problems in a row: the second would pick up
the first one's work list or status if the entry point did not clear what has to start from zero.
Collected last on purpose (file name), and self-contained so it also passes alone in a fresh process.
"""
import numpy as np
import pytest
import torch

from gpu_util import assert_close

pytestmark = pytest.mark.gpu


def _problem(seed, tq, tk, hq, hkv, qr, kr):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(tq, hq, 128, generator=g).to(torch.bfloat16).cuda()
    k = torch.randn(tk, hkv, 128, generator=g).to(torch.bfloat16).cuda()
    v = torch.randn(tk, hkv, 128, generator=g).to(torch.bfloat16).cuda()
    qr = torch.tensor(qr, dtype=torch.int32, device="cuda")
    kr = torch.tensor(kr, dtype=torch.int32, device="cuda")
    return q, k, v, qr, kr


def test_noalloc_entry_matches_regular_entry_twice_in_a_row():
    import magi_b200 as mb
    problems = [
        # a larger plan first (5 ranges, many work items) ...
        (_problem(101, 1500, 1500, 6, 2, [[0, 300], [300, 601], [601, 900], [900, 1200], [1200, 1500]],
                  [[0, 300], [0, 601], [128, 900], [0, 1200], [0, 1500]]), 301),
        # ... then a smaller one, so stale items / segments of the first call would show
        (_problem(102, 400, 777, 4, 4, [[0, 130], [200, 400]], [[5, 777], [0, 129]]), 200),
    ]
    # One warm-up call first: the very first call on a device resolves the scratch symbol and loads the kernels, which
    # the driver may back with device memory; what must not allocate is a call of a running service.
    (wq, wk, wv, wqr, wkr), wmax = problems[1]
    mb.chunk_attn_noalloc(wq, wk, wv, wqr, wkr, wmax, torch.empty_like(wq))
    torch.cuda.synchronize()
    for (q, k, v, qr, kr), max_q in problems:
        # caller-owned outputs; pre-filled so that rows outside every range can be compared too
        out = torch.full_like(q, 5.0)
        lse = torch.full((q.shape[0], q.shape[1]), 9.0, dtype=torch.float32, device="cuda")
        status = torch.full((1,), 77, dtype=torch.int32, device="cuda")
        torch.cuda.synchronize()
        # cumulative count of allocator requests: frees by the garbage collector (tensors of earlier tests) do not move it
        before = torch.cuda.memory_stats().get("allocation.all.allocated", 0)
        # torch's counters do not see a cudaMalloc made inside the library: the driver's own free-memory figure does
        free_before = torch.cuda.mem_get_info()[0]
        mb.chunk_attn_noalloc(q, k, v, qr, kr, max_q, out, lse=lse, status=status)
        torch.cuda.synchronize()
        assert torch.cuda.memory_stats().get("allocation.all.allocated", 0) == before, \
            "the allocation-free path allocated through torch"
        assert torch.cuda.mem_get_info()[0] >= free_before, "device memory was allocated behind torch's back"
        assert int(status.item()) == 0
        ref = torch.full_like(q, 5.0)
        ref_out, ref_lse = mb.chunk_attn(q, k, v, qr, kr, max_q, 0, out=ref)
        torch.cuda.synchronize()
        assert mb.Context.get().status() == 0
        rows = torch.cat([torch.arange(a, b) for a, b in qr.cpu().tolist()]).cuda()
        assert_close(out, ref_out, what="no-alloc vs regular entry")   # the tolerance of the other GPU tests ...
        assert torch.equal(out, ref_out)                                 # ... and in fact the same kernel: bit-equal
        assert torch.allclose(lse[rows], ref_lse[rows], atol=3e-3, rtol=1e-3)


def test_noalloc_entry_rejects_oversized_problems_and_reports_bad_ranges():
    import magi_b200 as mb
    (q, k, v, qr, kr), max_q = (_problem(103, 256, 256, 2, 2, [[0, 256]], [[0, 256]]), 256)
    out = torch.full_like(q, 3.0)
    with pytest.raises(mb.MagiError) as e:   # 1 range x ceil(2^23 / 256) work items > 16384
        mb.chunk_attn_noalloc(q, k, v, qr, kr, 1 << 23, out)
    assert e.value.code == mb._lib.E_NOMEM and "exceeds the fixed scratch" in str(e.value)
    bad = torch.tensor([[0, 4096]], dtype=torch.int32, device="cuda")  # beyond total_k: caught by the device planner
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    mb.chunk_attn_noalloc(q, k, v, qr, bad, max_q, out, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == mb._lib.E_RANGE and (out.float() == 3.0).all()
    # and the next call starts clean
    mb.chunk_attn_noalloc(q, k, v, qr, kr, max_q, out, status=status)
    torch.cuda.synchronize()
    assert int(status.item()) == 0 and torch.isfinite(out.float()).all() and not (out.float() == 3.0).all()
