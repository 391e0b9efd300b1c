"""Device-side failure detection without a GPU fault: every mbarrier wait of the attention kernels is bounded and reports
MAGI_E_TIMEOUT through the status word.  The self-test entry runs that wait on a barrier that nothing completes, with a
limit of about a millisecond: the launch returns, the status is readable on the host, sticky until read, and the
context keeps working."""
import time

import pytest
import torch

from gpu_util import assert_close, as_segments
from oracle import chunk_attn_oracle as O

pytestmark = pytest.mark.gpu


def _small_problem(seed):
    from magi_b200 import host
    C, n, Hq, Hkv = 160, 2, 4, 2
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(n * C, Hq, 128, generator=g).to(torch.bfloat16)
    k = torch.randn(n * C, Hkv, 128, generator=g).to(torch.bfloat16)
    v = torch.randn(n * C, Hkv, 128, generator=g).to(torch.bfloat16)
    return q, k, v, host.q_ranges_for_chunks(n, C), host.default_k_ranges(n, C), C, n * C


def test_bounded_wait_gives_up_and_reports_timeout():
    import magi_b200 as mb
    from magi_b200 import _lib
    ctx = mb.Context.get()
    assert ctx.status() == 0
    t0 = time.time()
    ctx.selftest_bounded_wait(limit_cycles=2_000_000)        # ~1 ms of SM clock
    torch.cuda.synchronize()
    assert time.time() - t0 < 5.0                            # it came back by itself
    assert ctx.status() == _lib.E_TIMEOUT
    assert ctx.status() == 0                                 # reading clears the word
    with pytest.raises(mb.MagiError):
        ctx.selftest_bounded_wait(limit_cycles=10 ** 12)     # unbounded requests are refused


def test_status_is_sticky_and_stops_later_launches_until_read():
    import magi_b200 as mb
    from magi_b200 import _lib
    ctx = mb.Context.get()
    q, k, v, qr, kr, max_q, max_k = _small_problem(81)
    ctx.selftest_bounded_wait(limit_cycles=500_000)
    # an attention call enqueued while the word is set does no work: its CTAs see the status and return
    out = torch.full((q.shape[0], q.shape[1], 128), 5.0, dtype=torch.bfloat16, device="cuda")
    mb.chunk_attn(q.cuda(), k.cuda(), v.cuda(), qr, kr, max_q, max_k, out=out, return_lse=False)
    torch.cuda.synchronize()
    assert (out.float() == 5.0).all()
    assert ctx.status() == _lib.E_TIMEOUT
    # after the host has read (and thereby cleared) the word the same context computes again
    out2, _ = mb.chunk_attn(q.cuda(), k.cuda(), v.cuda(), qr, kr, max_q, max_k)
    torch.cuda.synchronize()
    assert ctx.status() == 0
    ref, _ = O.range_attention(q.float(), k.float(), v.float(), qr, as_segments(kr))
    assert_close(out2, ref, what="attention after a reported timeout")
