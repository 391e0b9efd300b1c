"""Ulysses exchange (the N > 1 path) on world_size-2/4 gloo CPU ranks against the fixture produced by the reference's
own all_to_all_input_split / all_to_all_output_split."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, tag, golden, fail_rank):
    import sys
    for p in (ROOT, os.path.join(ROOT, "magi-1_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    from magi_b200 import host
    from magi_b200.ulysses import UlyssesExchange, kv_head_replication
    z = np.load(golden)
    S, Hq, Hkv, D = (int(x) for x in z[f"{tag}_case"])
    splits = host.cp_split_sizes(S, world)
    off = sum(splits[:rank])
    g = torch.Generator().manual_seed(5)
    qfull = torch.randn(S, Hq, D, generator=g)
    kvfull = torch.randn(S, Hkv, 2 * D, generator=g)
    ex = UlyssesExchange(dist.group.WORLD, splits)
    s_loc = splits[rank]
    # send layout "(cp seq) hn hd" (on the GPU the prologue kernel writes it directly)
    q_loc = qfull[off:off + s_loc]
    q_send = q_loc.view(s_loc, world, Hq // world, D).transpose(0, 1).contiguous()
    rep = kv_head_replication(Hkv, world)
    kv_loc = kvfull[off:off + s_loc].repeat_interleave(rep, dim=1)
    kv_send = kv_loc.view(s_loc, world, Hkv * rep // world, 2 * D).transpose(0, 1).contiguous()
    q_x, w = ex.scatter_heads(q_send)
    w.wait()
    kv_x, w = ex.scatter_heads(kv_send, async_op=True)
    w.wait()
    assert np.array_equal(q_x.numpy(), z[f"{tag}_r{rank}_q_x"])
    assert np.array_equal(kv_x.numpy(), z[f"{tag}_r{rank}_kv_x"])
    o_x, w = ex.gather_heads(q_x)
    w.wait()
    o_fin = o_x.permute(1, 0, 2, 3).reshape(s_loc, 1, -1)   # "(cp sq) hn hd -> sq b (cp hn hd)"
    assert np.array_equal(o_fin.numpy(), z[f"{tag}_r{rank}_o_fin"])
    assert torch.equal(o_fin.view(s_loc, Hq, D), q_loc)
    # argument errors surface as exceptions on the offending rank only after a consistent check on all ranks
    with pytest.raises(ValueError):
        ex.scatter_heads(q_send[:, :-1] if s_loc > 1 else q_send[:0])
    with pytest.raises(ValueError):
        UlyssesExchange(dist.group.WORLD, splits[:-1])
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("tag,world", [("cp2", 2), ("cp4", 4)])
def test_exchange_matches_reference_glue(tag, world, golden_dir):
    mp.spawn(_worker, args=(world, _free_port(), tag, os.path.join(golden_dir, "ulysses.npz"), -1), nprocs=world, join=True)


def test_kv_head_replication_rule():
    import sys
    sys.path.insert(0, os.path.join(ROOT, "magi-1_b200"))
    from magi_b200.ulysses import kv_head_replication
    assert kv_head_replication(8, 8) == 1 and kv_head_replication(8, 2) == 1 and kv_head_replication(2, 4) == 2
    with pytest.raises(ValueError):
        kv_head_replication(8, 3)


def _dropout_worker(rank, world, port, flag_dir):
    """Rank 1 leaves between two exchanges; rank 0 learns of it when its next collective times out (host-side
    failure detection: no GPU is involved, nothing hangs for longer than the process-group timeout)."""
    import datetime
    import sys
    for p in (ROOT, os.path.join(ROOT, "magi-1_b200")):
        if p not in sys.path:
            sys.path.insert(0, p)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    from magi_b200.ulysses import UlyssesExchange
    ex = UlyssesExchange(dist.group.WORLD, [3, 3])
    send = torch.arange(2 * 3 * 2 * 4, dtype=torch.float32).view(2, 3, 2, 4) + 100 * rank
    recv, w = ex.scatter_heads(send)
    w.wait()                                        # first exchange: both ranks take part
    assert recv.shape == (6, 2, 4)
    if rank == 1:
        open(os.path.join(flag_dir, "rank1_left"), "w").close()
        os._exit(0)                                 # leaves between steps, nothing of its own in flight
    failed = False
    try:
        _, w = ex.scatter_heads(send)
        w.wait()
    except Exception:
        failed = True
    assert failed, "the exchange with a missing rank must fail with an error, not return"
    open(os.path.join(flag_dir, "rank0_detected"), "w").close()
    os._exit(0)


def test_missing_rank_is_detected_by_timeout(tmp_path):
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_dropout_worker, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
    for p in procs:
        if p.is_alive():
            p.kill()
    assert (tmp_path / "rank1_left").exists() and (tmp_path / "rank0_detected").exists()
