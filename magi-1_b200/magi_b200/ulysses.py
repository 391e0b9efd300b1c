"""Ulysses context parallelism for the attention core: heads are split across the CP ranks, every rank sees the
full sequence for its heads.  Mirrors inference/infra/parallelism/context_parallel.py:381-423 (all_to_all_input_split /
all_to_all_output_split) and UlyssesScheduler.get_attn_and_xattn_with_fused_kv_comm (:503-548, :550-597):

    K|V prologue -> a2a(K|V) || Q prologue -> a2a(Q) -> [KV cache] -> attention per head group || a2a(O of previous group)

Differences from the reference, all on the data-movement side:
  * the prologue kernels write the send layout "(cp seq) hn hd" directly (no rearrange().contiguous() pass), K and V
    into one fused [.., 256] buffer so one exchange carries both (as the reference's fused-KV path);
  * the attention kernel reads K and V as strided halves of the received buffer (no chunk().contiguous());
  * the received O blocks "(cp sq) hn hd" are put into "sq (cp hn) hd" by one strided copy kernel.
torch.distributed (NCCL over NVLink, gloo in CPU tests) is the plumbing for the exchange itself.
"""
from typing import List, Optional, Sequence

import torch
import torch.distributed as dist

HEAD_DIM = 128


class UlyssesExchange:
    """The two all-to-alls, on whatever device the tensors live on (NCCL for CUDA, gloo for CPU tensors)."""

    def __init__(self, group, split_sizes: Sequence[int]):
        self.group = group
        self.cp = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.split_sizes = [int(s) for s in split_sizes]
        if len(self.split_sizes) != self.cp:
            raise ValueError(f"split_sizes has {len(self.split_sizes)} entries for a group of {self.cp}")
        self.s_local = self.split_sizes[self.rank]
        self.s_total = sum(self.split_sizes)

    def scatter_heads(self, send: torch.Tensor, recv: Optional[torch.Tensor] = None, async_op: bool = True):
        """send [cp, s_local, hn, d] (block r goes to rank r)  ->  recv [s_total, hn, d] (all tokens, own heads).
        Returns (recv, work)."""
        if send.shape[0] != self.cp or send.shape[1] != self.s_local or not send.is_contiguous():
            raise ValueError(f"send must be contiguous [cp={self.cp}, s_local={self.s_local}, hn, d], got {tuple(send.shape)}")
        if recv is None:
            recv = torch.empty((self.s_total,) + tuple(send.shape[2:]), dtype=send.dtype, device=send.device)
        work = dist.all_to_all_single(recv, send.view((self.cp * self.s_local,) + tuple(send.shape[2:])),
                                      output_split_sizes=self.split_sizes, group=self.group, async_op=async_op)
        return recv, work

    def gather_heads(self, full: torch.Tensor, recv: Optional[torch.Tensor] = None, async_op: bool = True):
        """full [s_total, hn, d] (all tokens, own heads)  ->  recv [cp, s_local, hn, d] (own tokens, block r = heads of rank r)."""
        if full.shape[0] != self.s_total or not full.is_contiguous():
            raise ValueError(f"full must be contiguous [s_total={self.s_total}, hn, d], got {tuple(full.shape)}")
        if recv is None:
            recv = torch.empty((self.cp, self.s_local) + tuple(full.shape[1:]), dtype=full.dtype, device=full.device)
        work = dist.all_to_all_single(recv.view((self.cp * self.s_local,) + tuple(full.shape[1:])), full,
                                      input_split_sizes=self.split_sizes, group=self.group, async_op=async_op)
        return recv, work


class _Done:
    """Stand-in for a torch.distributed work handle: the C-level exchange is ordered on the current stream."""

    def wait(self):
        return True


class LibraryExchange(UlyssesExchange):
    """The same two all-to-alls through the library's own NCCL communicator (magi_ulysses_*), i.e. the path a host
    without torch.distributed would take; torch.distributed is used here only to hand the 128-byte unique id around.
    Calls are ordered on the current CUDA stream."""

    def __init__(self, group, split_sizes: Sequence[int]):
        super().__init__(group, split_sizes)
        import ctypes as C
        from . import ops
        from ._lib import check, lib
        self._C, self._lib, self._check, self._ops = C, lib, check, ops
        self.ctx = ops.Context.get(torch.cuda.current_device())
        uid = C.create_string_buffer(128)
        if self.rank == 0:
            check(lib.magi_ulysses_unique_id(self.ctx.handle, uid), self.ctx.handle)
        box = [uid.raw]
        dist.broadcast_object_list(box, src=dist.get_global_rank(group, 0), group=group)
        uid = C.create_string_buffer(box[0], 128)
        sizes = (C.c_int32 * self.cp)(*self.split_sizes)
        h = C.c_void_p()
        check(lib.magi_ulysses_create(self.ctx.handle, uid, self.rank, self.cp, sizes, C.byref(h)), self.ctx.handle)
        self.handle = h

    def scatter_heads(self, send: torch.Tensor, recv: Optional[torch.Tensor] = None, async_op: bool = True):
        if send.shape[0] != self.cp or send.shape[1] != self.s_local or not send.is_contiguous():
            raise ValueError(f"send must be contiguous [cp={self.cp}, s_local={self.s_local}, hn, d], got {tuple(send.shape)}")
        if recv is None:
            recv = torch.empty((self.s_total,) + tuple(send.shape[2:]), dtype=send.dtype, device=send.device)
        row_bytes = send[0, 0].numel() * send.element_size()
        self._check(self._lib.magi_ulysses_a2a_in(self.handle, send.data_ptr(), recv.data_ptr(), row_bytes,
                                                  self._ops._stream()), self.ctx.handle)
        return recv, _Done()

    def gather_heads(self, full: torch.Tensor, recv: Optional[torch.Tensor] = None, async_op: bool = True):
        if full.shape[0] != self.s_total or not full.is_contiguous():
            raise ValueError(f"full must be contiguous [s_total={self.s_total}, hn, d], got {tuple(full.shape)}")
        if recv is None:
            recv = torch.empty((self.cp, self.s_local) + tuple(full.shape[1:]), dtype=full.dtype, device=full.device)
        row_bytes = full[0].numel() * full.element_size()
        self._check(self._lib.magi_ulysses_a2a_out(self.handle, full.data_ptr(), recv.data_ptr(), row_bytes,
                                                   self._ops._stream()), self.ctx.handle)
        return recv, _Done()

    def close(self):
        if getattr(self, "handle", None):
            torch.cuda.synchronize()
            self._lib.magi_ulysses_destroy(self.handle)
            self.handle = None


def kv_head_replication(n_kv_heads: int, cp: int) -> int:
    """KV heads are repeated when there are more ranks than heads (context_parallel.py:393-394)."""
    if cp % n_kv_heads == 0 and cp != n_kv_heads and cp > n_kv_heads:
        return cp // n_kv_heads
    if n_kv_heads % cp != 0:
        raise ValueError(f"{n_kv_heads} KV heads cannot be split over {cp} ranks")
    return 1


class UlyssesAttention:
    """Prologue + exchange + attention + exchange for one layer on one CP rank (CUDA)."""

    def __init__(self, cp_group, n_q_heads: int, n_kv_heads: int, split_sizes: Sequence[int], overlap_degree: int = 1,
                 exchange: str = "torch", head_order: str = "reference"):
        """exchange = "torch": torch.distributed all_to_all_single; "library": the library's own NCCL communicator.

        head_order matters only with overlap_degree > 1 on a rank that holds more than one KV head.  The reference
        concatenates the outputs of the head groups (torch.cat(core_attn_outs, dim=1), context_parallel.py:594) before
        the final rearrange, so inside each rank's block of the result the heads come group-major: (group i, kv head,
        sub-head) instead of the projection's (kv head, group i, sub-head).  "reference" reproduces that order bit for
        bit (what a drop-in must do); "original" keeps every head at its own global index."""
        from . import ops
        if head_order not in ("reference", "original"):
            raise ValueError("head_order must be 'reference' or 'original'")
        self.head_order = head_order
        self.ops = ops
        self.ex = {"torch": UlyssesExchange, "library": LibraryExchange}[exchange](cp_group, split_sizes)
        cp = self.ex.cp
        if n_q_heads % cp:
            raise ValueError(f"{n_q_heads} q heads cannot be split over {cp} ranks")
        self.rep = kv_head_replication(n_kv_heads, cp)
        self.hq, self.hkv = n_q_heads, n_kv_heads * self.rep
        self.hq_loc, self.hkv_loc = self.hq // cp, self.hkv // cp
        if self.hq_loc % self.hkv_loc:
            raise ValueError("local q heads must be a multiple of local kv heads")
        g = self.hq_loc // self.hkv_loc
        if overlap_degree == -1:
            overlap_degree = g
        if overlap_degree < 1 or g % overlap_degree:
            raise ValueError(f"overlap_degree {overlap_degree} must divide the GQA group size {g}")
        self.overlap = overlap_degree
        self._bufs = {}

    def _buf(self, name, shape, device):
        t = self._bufs.get(name)
        if t is None or tuple(t.shape) != tuple(shape) or t.device != device:
            t = torch.empty(shape, dtype=torch.bfloat16, device=device)
            self._bufs[name] = t
        return t

    def forward(self, xq, xk, xv, gq, bq, gk, bk, cos, sin, q_ranges, k_ranges, max_seqlen_q, max_seqlen_k,
                eps: float = 1e-6, norm_mode: str = "layernorm_1p", cache=None, layer: int = 0,
                prefix_chunk_ids: Sequence[int] = (), k_range_offsets=None, attn_events: Optional[list] = None,
                fp8_chunk_tokens: int = 0, cross_attn_func=None, kv_current_offset: int = 0):
        """xq [s_local, Hq, 128], xk / xv [s_local, Hkv, 128]: this rank's tokens, all heads (projection outputs).
        cache / prefix_chunk_ids: a head-sharded paged prefix (the cache holds this rank's Hkv/cp heads,
        dit_module.py:794-798); kv_current_offset: the received K/V from this token on are the "current" keys, earlier
        tokens are served by the prefix pages.
        cross_attn_func: optional callable run after the last head group's attention has been enqueued, while its output
        exchange is in flight (the cross-attention slot of the reference's schedule, context_parallel.py:591); forward
        then returns (O, cross_attn_func()).
        cos / sin: this rank's rows of the rotary table.  Ranges are in full-sequence token coordinates.
        fp8_chunk_tokens > 0 runs the FP8 e4m3 attention: the head-sharded Q/K/V are block-quantised after the exchange
        (scale blocks counted from each multiple of fp8_chunk_tokens; Q and P carried as two terms), the exchange itself
        and the output stay bf16.
        Returns O [s_local, Hq, 128] for this rank's tokens, heads in global order."""
        ops, ex = self.ops, self.ex
        cp, s_loc, S = ex.cp, ex.s_local, ex.s_total
        dev = xq.device
        if self.rep > 1:
            xk = xk.repeat_interleave(self.rep, dim=1)
            xv = xv.repeat_interleave(self.rep, dim=1)
        kv_send = self._buf("kv_send", (cp, s_loc, self.hkv_loc, 2 * HEAD_DIM), dev)
        ops.qk_norm_rope(xk, gk, bk, cos, sin, eps, norm_mode, out=kv_send[..., :HEAD_DIM], heads_per_block=self.hkv_loc)
        ops.head_block_copy(xv, kv_send[..., HEAD_DIM:], heads_per_block=self.hkv_loc)
        kv_recv, w_kv = ex.scatter_heads(kv_send, self._buf("kv_recv", (S, self.hkv_loc, 2 * HEAD_DIM), dev))
        q_send = self._buf("q_send", (cp, s_loc, self.hq_loc, HEAD_DIM), dev)
        ops.qk_norm_rope(xq, gq, bq, cos, sin, eps, norm_mode, out=q_send, heads_per_block=self.hq_loc)
        q_recv, w_q = ex.scatter_heads(q_send, self._buf("q_recv", (S, self.hq_loc, HEAD_DIM), dev))
        w_kv.wait()
        k_full, v_full = kv_recv[kv_current_offset:, :, :HEAD_DIM], kv_recv[kv_current_offset:, :, HEAD_DIM:]
        fp8 = {}
        if fp8_chunk_tokens > 0:
            k_full, ks = ops.quantize_e4m3(k_full, fp8_chunk_tokens)
            v_full, vs = ops.quantize_e4m3(v_full, fp8_chunk_tokens)
            fp8 = dict(k_scale=ks, v_scale=vs, scale_chunk_tokens=fp8_chunk_tokens)
        w_q.wait()

        out = self._buf("out", (s_loc, self.hq, HEAD_DIM), dev)
        o_full = self._buf("o_full", (self.overlap, S, self.hq_loc // self.overlap, HEAD_DIM), dev)
        o_recv = self._buf("o_recv", (self.overlap, cp, s_loc, self.hq_loc // self.overlap, HEAD_DIM), dev)
        g = self.hq_loc // self.hkv_loc
        gsub = g // self.overlap
        q_grp = q_recv.view(S, self.hkv_loc, g, HEAD_DIM)
        pending = None
        for i in range(self.overlap):
            # head group i: sub-heads [i*gsub, (i+1)*gsub) of every local KV head (GQA-aware split, context_parallel.py:570-578)
            qi = q_grp[:, :, i * gsub:(i + 1) * gsub].reshape(S, self.hkv_loc * gsub, HEAD_DIM) if self.overlap > 1 else q_recv
            if fp8_chunk_tokens > 0:
                qi, qs, q_lo = ops.quantize_e4m3(qi, fp8_chunk_tokens, residual=True)
                fp8.update(q_scale=qs, q_lo=q_lo)
            if attn_events is not None:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            ops.chunk_attn(qi, k_full, v_full, q_ranges, k_ranges, max_seqlen_q, max_seqlen_k, out=o_full[i], return_lse=False,
                           k_range_offsets=k_range_offsets, cache=cache, layer=layer, prefix_chunk_ids=prefix_chunk_ids, **fp8)
            if attn_events is not None:
                e1.record()
                attn_events.append((e0, e1))
            if pending is not None:
                self._finish(pending, out, gsub)
            _, w = ex.gather_heads(o_full[i], o_recv[i])
            pending = (i, w, o_recv[i])
        xattn_out = cross_attn_func() if cross_attn_func is not None else None
        self._finish(pending, out, gsub)
        return out if cross_attn_func is None else (out, xattn_out)

    def _finish(self, pending, out, gsub):
        """Wait for the exchange of head group i and place its blocks: "(cp sq) hn hd -> sq (cp hn) hd"."""
        i, w, o_recv = pending
        w.wait()
        if self.overlap == 1:
            self.ops.head_block_copy(o_recv, out)
        else:
            # group i holds sub-heads [i*gsub, (i+1)*gsub) of each local kv head: scatter them to their global positions
            cp, s_loc = o_recv.shape[0], o_recv.shape[1]
            g = self.hq_loc // self.hkv_loc
            if self.head_order == "original":
                dst = out.view(s_loc, cp, self.hkv_loc, g, HEAD_DIM)[:, :, :, i * gsub:(i + 1) * gsub]
            else:  # the reference's cat over the groups: (group, kv head, sub-head) inside each rank's block
                dst = out.view(s_loc, cp, self.overlap, self.hkv_loc, gsub, HEAD_DIM)[:, :, i]
            src = o_recv.view(cp, s_loc, self.hkv_loc, gsub, HEAD_DIM).permute(1, 0, 2, 3, 4)
            dst.copy_(src)


class FusedUlyssesAttention:
    """Ulysses attention with both exchanges fused into their producer kernels over NVLink peer memory.

    Same contract as UlyssesAttention.forward (bf16), but no all-to-all is launched:
      * the prologue kernels store each rank's share of the heads straight into that rank's receive buffers
        (the "scatter heads" exchange, context_parallel.py:381-401, becomes the prologue's store address);
      * the attention kernel's epilogue stores every output row straight into the owning rank's result buffer at this
        rank's global head position (the "gather heads" exchange and the final "(cp sq) hn hd -> sq (cp hn) hd"
        re-layout, context_parallel.py:404-423 and :596, become the epilogue's store address).
    Buffers are cudaMalloc'ed by the library and mapped by the other ranks through CUDA IPC: plain peer stores, no
    multicast object, TMA only ever reads local memory.  Two tiny NCCL all-reduces per call act as stream-ordered
    barriers ("all receive buffers are complete", "all results are complete"); successive calls need nothing more, as
    a rank can only reach the next call's stores after every rank has passed the previous barrier.
    The returned tensor is a view of one of this object's n_out_buffers result buffers, used in rotation: it stays valid
    until n_out_buffers further calls have been made (the reference returns a fresh tensor per call,
    context_parallel.py:404-423; with two buffers a consumer of call i - a device-to-host copy, the output projection
    on another stream - may still run while call i+1 computes, provided it has finished before this rank ENTERS call
    i+2: every rank writes into the buffer only after the first barrier of that call, which this rank joins later).
    """

    def __init__(self, cp_group, n_q_heads: int, n_kv_heads: int, split_sizes: Sequence[int], proj_hn: int = 0,
                 n_out_buffers: int = 1):
        """proj_hn > 0 (8 in the reference): the result buffer is the operand of the output projection,
        [s_local, 2 * Hq * 128] in the "(hn n hd)" order of attn_linear_proj (dit_module.py:1332-1346); every rank's
        epilogue stores its heads at their final columns of the core-attention half, and cross_dest() gives the
        arguments with which the (rank-local) cross-attention call fills the other half."""
        from . import ops
        self.ops = ops
        self.group = cp_group
        self.cp = dist.get_world_size(cp_group)
        self.rank = dist.get_rank(cp_group)
        cp = self.cp
        if n_q_heads % cp or n_kv_heads % cp:
            raise ValueError(f"{n_q_heads}/{n_kv_heads} heads cannot be split over {cp} ranks (KV-head replication is only "
                             f"implemented in UlyssesAttention)")
        if cp > 16:
            raise ValueError("at most 16 ranks")
        self.hq, self.hkv = n_q_heads, n_kv_heads
        self.hq_loc, self.hkv_loc = n_q_heads // cp, n_kv_heads // cp
        self.splits = [int(s) for s in split_sizes]
        if len(self.splits) != cp:
            raise ValueError("split_sizes must have one entry per rank")
        self.offsets = [0]
        for s in self.splits:
            self.offsets.append(self.offsets[-1] + s)
        S, s_max = self.offsets[-1], max(self.splits)
        self.S, self.s_loc = S, self.splits[self.rank]
        dev = torch.cuda.current_device()
        self.buf_q = ops.PeerBuffer(S * self.hq_loc * HEAD_DIM * 2, dev)
        self.buf_kv = ops.PeerBuffer(S * self.hkv_loc * 2 * HEAD_DIM * 2, dev)
        if proj_hn and n_q_heads % proj_hn:
            raise ValueError("the head count must be a multiple of proj_hn")
        self.proj_hn = int(proj_hn)
        self.o_row = (2 if proj_hn else 1) * self.hq * HEAD_DIM   # elements per token in a result buffer
        if n_out_buffers < 1:
            raise ValueError("n_out_buffers must be at least 1")
        self.bufs_o = [ops.PeerBuffer(s_max * self.o_row * 2, dev) for _ in range(n_out_buffers)]
        handles = [None] * cp
        dist.all_gather_object(handles, (self.buf_q.handle, self.buf_kv.handle, [b.handle for b in self.bufs_o]), group=cp_group)
        self.peer_q, self.peer_kv, self.peers_o = [], [], [[] for _ in self.bufs_o]
        for r in range(cp):
            if r == self.rank:
                self.peer_q.append(self.buf_q.ptr), self.peer_kv.append(self.buf_kv.ptr)
                for i, b in enumerate(self.bufs_o):
                    self.peers_o[i].append(b.ptr)
            else:
                hq_, hkv_, ho_ = handles[r]
                self.peer_q.append(self.buf_q.open_peer(hq_))
                self.peer_kv.append(self.buf_kv.open_peer(hkv_))
                for i, b in enumerate(self.bufs_o):
                    self.peers_o[i].append(b.open_peer(ho_[i]))
        self._flag = torch.zeros(1, dtype=torch.float32, device=torch.device("cuda", dev))
        self.q_recv = self.buf_q.as_tensor((S, self.hq_loc, HEAD_DIM))
        self.kv_recv = self.buf_kv.as_tensor((S, self.hkv_loc, 2 * HEAD_DIM))
        self.outs = [b.as_tensor((s_max, self.o_row) if proj_hn else (s_max, self.hq, HEAD_DIM)) for b in self.bufs_o]
        self._calls = 0
        self._side = None      # stream and context of the cross-attention slot, created on first use
        self._side_ctx = None
        self._barrier()

    @property
    def out(self) -> torch.Tensor:
        """The result buffer of the most recent forward()."""
        return self.outs[(self._calls - 1) % len(self.outs)]

    @property
    def peer_o(self) -> List[int]:
        return self.peers_o[(self._calls - 1) % len(self.outs)]

    def _barrier(self):
        dist.all_reduce(self._flag, group=self.group)

    def forward(self, xq, xk, xv, gq, bq, gk, bk, cos, sin, q_ranges, k_ranges, max_seqlen_q, max_seqlen_k,
                eps: float = 1e-6, norm_mode: str = "layernorm_1p", cache=None, layer: int = 0,
                prefix_chunk_ids: Sequence[int] = (), k_range_offsets=None, attn_events: Optional[list] = None,
                fp8_chunk_tokens: int = 0, kv_current_offset: int = 0, cross_attn_func=None, proj_weights=None):
        """Arguments as UlyssesAttention.forward.  proj_weights = (wq, wk, wv), the bf16 torch.nn.Linear weights of
        linear_qkv.q / .k / .v (dit_module.py:406-408): xq is then this rank's hidden states [s_local, hidden] (the output
        of forward_ln), xk / xv are ignored, and the three projections run as one kernel with the prologue and the head
        exchange in its epilogue.  cache / prefix_chunk_ids: a head-sharded paged prefix (the cache holds
        this rank's Hkv/cp heads, dit_module.py:794-798); the k ranges then address (prefix pages | current tokens).
        kv_current_offset: the received K/V from this token on are the "current" keys (earlier tokens, if any, are
        served by the prefix pages instead).
        fp8_chunk_tokens > 0: the head-sharded Q/K/V are block-quantised to e4m3 after the exchange (Q as two terms) and
        the FP8 kernel runs, with an fp8 cache if there is one; exchange and output stay bf16.
        cross_attn_func(dest_kwargs, ctx): the cross-attention slot of the reference's schedule
        (context_parallel.py:584-591).  It is called once the core attention is enqueued and runs on a side stream that
        is current during the call, overlapping the result barrier; `ctx` is a Context of its own (two overlapping
        attention calls must not share a plan workspace) to pass to ops.chunk_attn, and dest_kwargs (proj_hn > 0) are
        the keyword arguments that store its heads into the other half of the projection operand.  forward then returns
        (O, cross_attn_func's result) after the side stream has been joined."""
        ops = self.ops
        self._calls += 1
        off = self.offsets[self.rank]
        kv_row = self.hkv_loc * 2 * HEAD_DIM   # elements per token in a kv receive buffer
        q_row = self.hq_loc * HEAD_DIM
        k_dst = [p + off * kv_row * 2 for p in self.peer_kv]
        v_dst = [p + (off * kv_row + HEAD_DIM) * 2 for p in self.peer_kv]
        q_dst = [p + off * q_row * 2 for p in self.peer_q]
        if proj_weights is not None:
            # projection GEMMs -> prologue -> "scatter heads" exchange in ONE kernel: the GEMM's epilogue stores each
            # rank's heads of Q, K and V straight into that rank's receive buffers
            wq, wk, wv = proj_weights
            ops.linear_qkv_norm_rope(xq, [
                dict(weight=wk, gamma=gk, beta=bk, norm_mode=norm_mode, heads_per_block=self.hkv_loc, block_out=(k_dst, kv_row, 2 * HEAD_DIM)),
                dict(weight=wv, norm_mode="none", heads_per_block=self.hkv_loc, block_out=(v_dst, kv_row, 2 * HEAD_DIM)),
                dict(weight=wq, gamma=gq, beta=bq, norm_mode=norm_mode, heads_per_block=self.hq_loc, block_out=(q_dst, q_row, HEAD_DIM))],
                cos, sin, eps)
        else:
            ops.qk_norm_rope(xk, gk, bk, cos, sin, eps, norm_mode, heads_per_block=self.hkv_loc, block_out=(k_dst, kv_row, 2 * HEAD_DIM))
            ops.head_block_copy(xv, None, heads_per_block=self.hkv_loc, block_out=(v_dst, kv_row, 2 * HEAD_DIM))
            ops.qk_norm_rope(xq, gq, bq, cos, sin, eps, norm_mode, heads_per_block=self.hq_loc, block_out=(q_dst, q_row, HEAD_DIM))
        self._barrier()  # every rank's rows have landed in every receive buffer
        if attn_events is not None:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
        q_in = self.q_recv
        k_in, v_in = self.kv_recv[kv_current_offset:, :, :HEAD_DIM], self.kv_recv[kv_current_offset:, :, HEAD_DIM:]
        fp8 = {}
        if fp8_chunk_tokens > 0:
            if kv_current_offset % fp8_chunk_tokens:
                raise ValueError("kv_current_offset must be a multiple of fp8_chunk_tokens")
            q_in, qs, q_lo = ops.quantize_e4m3(q_in, fp8_chunk_tokens, residual=True)
            k_in, ks = ops.quantize_e4m3(k_in, fp8_chunk_tokens)
            v_in, vs = ops.quantize_e4m3(v_in, fp8_chunk_tokens)
            fp8 = dict(q_scale=qs, k_scale=ks, v_scale=vs, scale_chunk_tokens=fp8_chunk_tokens, q_lo=q_lo)
        ops.chunk_attn(q_in, k_in, v_in, q_ranges, k_ranges, max_seqlen_q,
                       max_seqlen_k, return_lse=False, k_range_offsets=k_range_offsets, cache=cache, layer=layer,
                       prefix_chunk_ids=prefix_chunk_ids,
                       o_peers=(self.peer_o, self.offsets, self.rank * self.hq_loc, self.o_row, HEAD_DIM) + (
                           (self.hq // self.proj_hn, 2 * (self.hq // self.proj_hn) * HEAD_DIM) if self.proj_hn else ()),
                       **fp8)
        if attn_events is not None:
            e1.record()
            attn_events.append((e0, e1))
        xattn_out = None
        if cross_attn_func is not None:
            main = torch.cuda.current_stream()
            if self._side is None:
                self._side = torch.cuda.Stream()
                self._side_ctx = ops.Context(torch.cuda.current_device())
            self._side.wait_stream(main)   # the slot may read what the prologue / earlier work on the main stream produced
            with torch.cuda.stream(self._side):
                xattn_out = cross_attn_func(self.cross_dest() if self.proj_hn else {}, self._side_ctx)
        self._barrier()  # every rank's output rows have landed in every result buffer
        if cross_attn_func is not None:
            torch.cuda.current_stream().wait_stream(self._side)
            return self.out[:self.s_loc], xattn_out
        return self.out[:self.s_loc]

    def cross_dest(self) -> dict:
        """chunk_attn keyword arguments that store this rank's cross-attention heads into the other half of the
        projection operand (proj_hn > 0)."""
        if not self.proj_hn:
            raise ValueError("created without proj_hn")
        hd = (self.hq // self.proj_hn) * HEAD_DIM
        return dict(out=self.out[:self.s_loc, hd:], out_heads_per_block=self.hq // self.proj_hn, out_block_stride=2 * hd)

    def close(self):
        torch.cuda.synchronize()
        self._barrier()
        torch.cuda.synchronize()
        for b in [self.buf_q, self.buf_kv] + self.bufs_o:
            b.close()
        if self._side_ctx is not None:
            self._side_ctx.close()
            self._side_ctx = None
