"""PyTorch-facing shim over the C ABI: torch supplies device memory and streams, nothing else.

Names and argument meaning mirror the reference's surface for this path:
  flex_attn(...)            <-> the `flex_attention` callable of inference/model/dit/dit_module.py:1032-1043
  qk_norm_rope(...)         <-> FullyParallelAttention.get_q / get_k (:953-980) after the projection
  ChunkPagedKVCache         <-> Attention._allocate_key_and_value_memory / _full_adjust_key_and_value (:800-931)
"""
import ctypes as C
import math
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import _lib
from ._lib import AttnParams, KVCacheDesc, LinearPrologueParams, ModulateParams, PrologueParams, check, lib

HEAD_DIM = 128

# Kernels of this library launched through this module since import (one entry, mutable): every wrapper below adds the
# number of kernels its C entry point launches.  The benchmark reads the difference over its timed region.
KERNEL_LAUNCHES = [0]


class Context:
    """One per (device); owns the plan workspace.  Calls sharing a context must be stream-ordered."""

    _by_device = {}

    def __init__(self, device: int):
        h = C.c_void_p()
        check(lib.magi_ctx_create(int(device), C.byref(h)))
        self.handle = h
        self.device = int(device)

    @classmethod
    def get(cls, device=None) -> "Context":
        if device is None:
            device = torch.cuda.current_device()
        device = torch.device(device).index if not isinstance(device, int) else device
        if device is None:
            device = torch.cuda.current_device()
        if device not in cls._by_device:
            cls._by_device[device] = Context(device)
        return cls._by_device[device]

    def status(self, stream=None) -> int:
        st = C.c_int(0)
        check(lib.magi_ctx_status(self.handle, _stream(stream), C.byref(st)), self.handle)
        return st.value

    def selftest_bounded_wait(self, limit_cycles: int = 2_000_000, stream=None) -> None:
        """Run the kernels' bounded mbarrier wait on a barrier that nothing completes (it gives up after limit_cycles);
        status() must read E_TIMEOUT afterwards.  Nothing faults or hangs."""
        check(lib.magi_selftest_bounded_wait(self.handle, int(limit_cycles), _stream(stream)), self.handle)

    def close(self):
        if self.handle:
            lib.magi_ctx_destroy(self.handle)
            self.handle = None


def _stream(stream=None):
    s = stream if stream is not None else torch.cuda.current_stream()
    return C.c_void_p(s.cuda_stream)


def _thd(t: torch.Tensor, name: str, dtype=torch.bfloat16):
    if not t.is_cuda:
        raise ValueError(f"{name} must be a CUDA tensor")
    if t.dtype != dtype:
        raise ValueError(f"{name} must be {dtype}, got {t.dtype}")
    if t.dim() != 3 or t.shape[2] != HEAD_DIM or t.stride(2) != 1:
        raise ValueError(f"{name} must be [tokens, heads, {HEAD_DIM}] with a contiguous last dim, got {tuple(t.shape)}")
    return t


def _ranges_dev(r, device) -> torch.Tensor:
    if isinstance(r, torch.Tensor):
        t = r.to(device=device, dtype=torch.int32)
    else:
        t = torch.as_tensor(np.asarray(r, dtype=np.int32), device=device)
    return t.reshape(-1, 2).contiguous()


def qk_norm_rope(x: torch.Tensor, gamma: torch.Tensor, beta: Optional[torch.Tensor], cos: Optional[torch.Tensor],
                 sin: Optional[torch.Tensor], eps: float = 1e-6, norm_mode: str = "layernorm_1p",
                 out: Optional[torch.Tensor] = None, heads_per_block: int = 0, stream=None, block_out=None) -> torch.Tensor:
    """x bf16 [T,H,128] (any token/head strides) -> bf16 normed + rotated.

    block_out = (ptrs, stride_t, stride_h): one raw destination base address per head block (peer-mapped receive
    buffers of the context-parallel ranks) instead of `out`; heads_per_block is then required.

    out=None gives the packed [T,H,128].  With heads_per_block = H/cp and out = [cp, T, H/cp, 128] the result
    is the Ulysses send layout "(cp seq) hn hd" written directly.
    """
    _thd(x, "x")
    T, H, _ = x.shape
    ctx = Context.get(x.device)
    if out is None and block_out is None:
        out = torch.empty(T, H, HEAD_DIM, dtype=torch.bfloat16, device=x.device)
    p = PrologueParams()
    p.struct_size = C.sizeof(PrologueParams)
    p.norm_mode = {"layernorm_1p": _lib.NORM_LAYERNORM_1P, "rmsnorm": _lib.NORM_RMSNORM_1P}[norm_mode]
    p.x, p.x_stride_t, p.x_stride_h, p.T, p.H = x.data_ptr(), x.stride(0), x.stride(1), T, H
    gamma = gamma.to(device=x.device, dtype=torch.float32).contiguous()
    p.gamma = gamma.data_ptr()
    if beta is not None:
        beta = beta.to(device=x.device, dtype=torch.float32).contiguous()
        p.beta = beta.data_ptr()
    p.eps = eps
    if cos is not None:
        cos = cos.to(device=x.device, dtype=torch.float32).contiguous()
        sin = sin.to(device=x.device, dtype=torch.float32).contiguous()
        assert cos.shape == sin.shape and cos.shape[0] == T
        p.rot_pairs, p.cos, p.sin = cos.shape[1], cos.data_ptr(), sin.data_ptr()
    keep = _fill_out(p, out, T, H, heads_per_block, block_out)
    check(lib.magi_qk_norm_rope_fwd(ctx.handle, C.byref(p), _stream(stream)), ctx.handle)
    KERNEL_LAUNCHES[0] += 1
    return out


def linear_qkv_norm_rope(x: torch.Tensor, projections, cos: Optional[torch.Tensor], sin: Optional[torch.Tensor],
                         eps: float = 1e-6, stream=None, x_scale: Optional[torch.Tensor] = None):
    """get_qkv / get_kv / get_q / get_k / get_v from the projection on (dit_module.py:953-1003) in ONE kernel: x
    [T, in_features] (the output of forward_ln) against one to four weights (q, qx, k, v).

    projections: a list of dicts, one per projection, with the keys
      weight      [H*128, in_features] (torch.nn.Linear.weight of linear_qkv.q / .k / .v), the same dtype as x
      gamma, beta the per-head norm's parameters (gamma applied as gamma + 1); not needed with norm_mode "none"
      norm_mode   "layernorm_1p" (default), "rmsnorm" or "none" (get_v: the projection as it is, no rotary)
      rotate      False: normed but not rotated (the cross-attention query of get_xqkv, :1005-1008); default True
      plain_odd_heads  True: heads 1, 3, 5, ... are left as projected - the weight of linear_kv_xattn, whose rows are
                  (k of head 0, v of head 0, k of head 1, ...), so that the output [T, 2*Hkv, 128] is the K|V buffer
                  [T, Hkv, 256] of get_xqkv (:1010-1020)
      out, heads_per_block, block_out   destination as qk_norm_rope (default: a new packed [T, H, 128])
      w_scale     e4m3 operands only: CUDA fp32 tensor, first entry used
    x and the weights are bf16, or all float8_e4m3fn (x from div_clamp_to, weights of PerTensorQuantizedFp8Linear
    members): the fp32 accumulator is then multiplied by x_scale[0] * w_scale[0] - input_scale and weight_scale, applied
    as bmm_fp8 applies them - before the bf16 rounding.  Returns the list of outputs (None where block_out was given)."""
    fp8 = x.dtype == torch.float8_e4m3fn
    want = torch.float8_e4m3fn if fp8 else torch.bfloat16
    if x.dtype != want or not x.is_cuda or x.dim() != 2 or x.stride(1) != 1:
        raise ValueError("x must be a CUDA bf16 or float8_e4m3fn matrix with a contiguous last dim")
    if not 1 <= len(projections) <= 4:
        raise ValueError("one to four projections per call")
    T, K = x.shape
    ctx = Context.get(x.device)
    arr = (LinearPrologueParams * len(projections))()
    keep, outs = [], []
    if cos is not None:
        cos = cos.to(device=x.device, dtype=torch.float32).contiguous()
        sin = sin.to(device=x.device, dtype=torch.float32).contiguous()
        assert cos.shape == sin.shape and cos.shape[0] == T
    xs = None if x_scale is None else x_scale.to(device=x.device, dtype=torch.float32).reshape(-1)
    for p, pr in zip(arr, projections):
        w = pr["weight"]
        if w.dtype != want or not w.is_cuda or w.dim() != 2 or w.stride(1) != 1 or w.shape[1] != K or w.shape[0] % HEAD_DIM:
            raise ValueError("weight must be a CUDA [H*128, in_features] matrix of x's dtype with a contiguous last dim")
        H = w.shape[0] // HEAD_DIM
        mode = pr.get("norm_mode", "layernorm_1p")
        out, block_out = pr.get("out"), pr.get("block_out")
        if out is None and block_out is None:
            out = torch.empty(T, H, HEAD_DIM, dtype=torch.bfloat16, device=x.device)
        p.struct_size = C.sizeof(LinearPrologueParams)
        p.norm_mode = {"layernorm_1p": _lib.NORM_LAYERNORM_1P, "rmsnorm": _lib.NORM_RMSNORM_1P, "none": _lib.NORM_NONE}[mode]
        p.x, p.x_stride, p.w, p.w_stride, p.T, p.H, p.in_features = x.data_ptr(), x.stride(0), w.data_ptr(), w.stride(0), T, H, K
        p.eps = eps
        p.plain_odd_heads = 1 if pr.get("plain_odd_heads") else 0
        if mode != "none":
            gamma = pr["gamma"].to(device=x.device, dtype=torch.float32).contiguous()
            p.gamma = gamma.data_ptr()
            keep.append(gamma)
            if pr.get("beta") is not None:
                beta = pr["beta"].to(device=x.device, dtype=torch.float32).contiguous()
                p.beta = beta.data_ptr()
                keep.append(beta)
            if cos is not None and pr.get("rotate", True):
                p.rot_pairs, p.cos, p.sin = cos.shape[1], cos.data_ptr(), sin.data_ptr()
        if fp8:
            p.dtype = _lib.DTYPE_FP8_E4M3
            p.x_scale = None if xs is None else xs.data_ptr()
            if pr.get("w_scale") is not None:
                ws = pr["w_scale"].to(device=x.device, dtype=torch.float32).reshape(-1)
                p.w_scale = ws.data_ptr()
                keep.append(ws)
        if T > 0:
            keep.append(_fill_out(p, out, T, H, pr.get("heads_per_block", 0), block_out))
        outs.append(out)
    if T > 0:
        check(lib.magi_linear_qkv_norm_rope_fwd(ctx.handle, arr, len(projections), _stream(stream)), ctx.handle)
        KERNEL_LAUNCHES[0] += 1
    return outs


def linear_qk_norm_rope(x: torch.Tensor, weight: torch.Tensor, gamma: Optional[torch.Tensor], beta: Optional[torch.Tensor],
                        cos: Optional[torch.Tensor], sin: Optional[torch.Tensor], eps: float = 1e-6,
                        norm_mode: str = "layernorm_1p", out: Optional[torch.Tensor] = None, heads_per_block: int = 0,
                        stream=None, block_out=None, x_scale: Optional[torch.Tensor] = None,
                        w_scale: Optional[torch.Tensor] = None) -> torch.Tensor:
    """One projection (get_q, get_k or get_v, dit_module.py:953-989) through linear_qkv_norm_rope: x [T, in_features],
    weight [H*128, in_features] -> bf16 [T, H, 128] = prologue(bf16(x @ weight^T)); norm_mode "none" is get_v."""
    return linear_qkv_norm_rope(x, [dict(weight=weight, gamma=gamma, beta=beta, norm_mode=norm_mode, out=out,
                                         heads_per_block=heads_per_block, block_out=block_out, w_scale=w_scale)],
                                cos, sin, eps, stream, x_scale)[0]


def head_block_copy(x: torch.Tensor, out: Optional[torch.Tensor], heads_per_block: int = 0, stream=None, block_out=None
                    ) -> Optional[torch.Tensor]:
    """Strided bf16 copy -> out with the same destination addressing as qk_norm_rope.

    x is [T,H,128], or a source-blocked [B, T, H/B, 128] ("(cp sq) hn hd", what the output all-to-all delivers),
    which is read as the logical [T, H, 128] with head h = b*(H/B) + h'."""
    if x.dim() == 4:
        if x.dtype != torch.bfloat16 or not x.is_cuda or x.shape[3] != HEAD_DIM or x.stride(3) != 1:
            raise ValueError("blocked x must be a CUDA bf16 [B, T, H/B, 128] tensor with a contiguous last dim")
        B, T, hb, _ = x.shape
        H = B * hb
    else:
        _thd(x, "x")
        T, H, _ = x.shape
    ctx = Context.get(x.device)
    p = PrologueParams()
    p.struct_size = C.sizeof(PrologueParams)
    if x.dim() == 4:
        p.x, p.x_stride_block, p.x_stride_t, p.x_stride_h = x.data_ptr(), x.stride(0), x.stride(1), x.stride(2)
        p.x_heads_per_block, p.T, p.H = hb, T, H
    else:
        p.x, p.x_stride_t, p.x_stride_h, p.T, p.H = x.data_ptr(), x.stride(0), x.stride(1), T, H
    keep = _fill_out(p, out, T, H, heads_per_block, block_out)
    check(lib.magi_head_block_copy(ctx.handle, C.byref(p), _stream(stream)), ctx.handle)
    KERNEL_LAUNCHES[0] += 1
    return out


def _fill_out(p, out, T, H, heads_per_block, block_out=None):
    if block_out is not None:
        ptrs, stride_t, stride_h = block_out
        if not heads_per_block or H % heads_per_block or len(ptrs) != H // heads_per_block:
            raise ValueError("block_out needs heads_per_block dividing H and one pointer per block")
        arr = (C.c_void_p * len(ptrs))(*[int(a) for a in ptrs])
        p.out_block_ptrs = C.cast(arr, C.POINTER(C.c_void_p))
        p.out_stride_t, p.out_stride_h, p.heads_per_block = int(stride_t), int(stride_h), heads_per_block
        return arr  # the caller keeps it alive until the call returns
    if out.dtype != torch.bfloat16 or not out.is_cuda or out.stride(-1) != 1:
        raise ValueError("out must be a CUDA bf16 tensor with a contiguous last dim")
    if heads_per_block and heads_per_block < H:
        if out.dim() != 4 or out.shape[0] * heads_per_block != H or out.shape[1] < T or out.shape[2] != heads_per_block:
            raise ValueError("blocked out must be [H/heads_per_block, >=T, heads_per_block, 128]")
        p.out, p.out_stride_block, p.out_stride_t, p.out_stride_h = out.data_ptr(), out.stride(0), out.stride(1), out.stride(2)
        p.heads_per_block = heads_per_block
    else:
        if out.dim() != 3 or out.shape[0] < T or out.shape[1] != H:
            raise ValueError("out must be [>=T, H, 128]")
        p.out, p.out_stride_t, p.out_stride_h = out.data_ptr(), out.stride(0), out.stride(1)


class ChunkPagedKVCache:
    """Pages of one chunk x one layer, K and V separate, bf16 or fp8 (+ per-(head,128-token) scales)."""

    def __init__(self, n_layers: int, max_chunks: int, chunk_tokens: int, n_kv_heads: int, dtype: str = "bf16",
                 device=None):
        self.ctx = Context.get(device)
        d = KVCacheDesc()
        d.struct_size = C.sizeof(KVCacheDesc)
        d.dtype = {"bf16": _lib.DTYPE_BF16, "fp8": _lib.DTYPE_FP8_E4M3}[dtype]
        d.n_layers, d.max_chunks, d.chunk_tokens, d.n_kv_heads = n_layers, max_chunks, chunk_tokens, n_kv_heads
        h = C.c_void_p()
        check(lib.magi_kv_cache_create(self.ctx.handle, C.byref(d), C.byref(h)), self.ctx.handle)
        self.handle = h
        self.dtype = dtype
        self.n_layers, self.max_chunks, self.chunk_tokens, self.n_kv_heads = n_layers, max_chunks, chunk_tokens, n_kv_heads

    @property
    def nbytes(self) -> int:
        return lib.magi_kv_cache_bytes(self.handle)

    def append(self, layer: int, chunk_id: int, k: torch.Tensor, v: torch.Tensor, token_offset: int = 0, stream=None):
        _thd(k, "k"), _thd(v, "v")
        assert k.shape == v.shape and k.shape[1] == self.n_kv_heads
        check(lib.magi_kv_cache_append(self.handle, layer, chunk_id, k.data_ptr(), k.stride(0), k.stride(1),
                                       v.data_ptr(), v.stride(0), v.stride(1), k.shape[0], token_offset,
                                       _stream(stream)), self.ctx.handle)

    def append_kv(self, layer: int, chunk_id: int, kv: torch.Tensor, token_offset: int = 0, stream=None):
        """kv: the reference's fused layout [tokens, Hkv, 2*128] (K | V on the last dim)."""
        self.append(layer, chunk_id, kv[..., :HEAD_DIM], kv[..., HEAD_DIM:], token_offset, stream)

    def evict(self, chunk_id: int):
        check(lib.magi_kv_cache_evict(self.handle, chunk_id), self.ctx.handle)

    def read_into(self, layer: int, chunk_id: int, k_out: torch.Tensor, v_out: torch.Tensor, stream=None):
        """Copy a whole page into caller-owned contiguous bf16 [chunk_tokens, Hkv, 128] tensors: device or pinned host."""
        for t in (k_out, v_out):
            if t.dtype != torch.bfloat16 or not t.is_contiguous() or tuple(t.shape) != (self.chunk_tokens, self.n_kv_heads, HEAD_DIM) \
                    or not (t.is_cuda or t.is_pinned()):
                raise ValueError("read_into needs contiguous bf16 [chunk_tokens, Hkv, 128] tensors on the device or in pinned memory")
        check(lib.magi_kv_cache_read(self.handle, layer, chunk_id, k_out.data_ptr(), v_out.data_ptr(), self.chunk_tokens, 0,
                                     _stream(stream)), self.ctx.handle)

    def append_from_host(self, layer: int, chunk_id: int, k: torch.Tensor, v: torch.Tensor, stream=None):
        """Fill a page from pinned host tensors [chunk_tokens, Hkv, 128] (read by the copy kernel over PCIe)."""
        for t in (k, v):
            if t.dtype != torch.bfloat16 or not t.is_contiguous() or not t.is_pinned() or t.shape[1] != self.n_kv_heads:
                raise ValueError("append_from_host needs contiguous pinned bf16 [tokens, Hkv, 128] tensors")
        check(lib.magi_kv_cache_append(self.handle, layer, chunk_id, k.data_ptr(), k.stride(0), k.stride(1),
                                       v.data_ptr(), v.stride(0), v.stride(1), k.shape[0], 0, _stream(stream)), self.ctx.handle)

    def read(self, layer: int, chunk_id: int, n_tokens: Optional[int] = None, token_offset: int = 0, stream=None):
        n = self.chunk_tokens - token_offset if n_tokens is None else n_tokens
        dev = torch.device("cuda", self.ctx.device)
        k = torch.empty(n, self.n_kv_heads, HEAD_DIM, dtype=torch.bfloat16, device=dev)
        v = torch.empty_like(k)
        check(lib.magi_kv_cache_read(self.handle, layer, chunk_id, k.data_ptr(), v.data_ptr(), n, token_offset,
                                     _stream(stream)), self.ctx.handle)
        return k, v

    def close(self):
        if self.handle:
            lib.magi_kv_cache_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def chunk_attn(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor], q_ranges, k_ranges,
               max_seqlen_q: int, max_seqlen_k: int = 0, softmax_scale: Optional[float] = None,
               k_range_offsets=None, cache: Optional[ChunkPagedKVCache] = None, layer: int = 0,
               prefix_chunk_ids: Sequence[int] = (), out: Optional[torch.Tensor] = None, return_lse: bool = True,
               impl: str = "tcgen05", stream=None, q_scale: Optional[torch.Tensor] = None,
               k_scale: Optional[torch.Tensor] = None, v_scale: Optional[torch.Tensor] = None,
               scale_chunk_tokens: int = 0, q_lo: Optional[torch.Tensor] = None, o_peers=None,
               out_heads_per_block: int = 0, out_block_stride: int = 0, ctx: Optional["Context"] = None
               ) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """General entry: several k intervals per q-range (k_range_offsets) and a paged prefix.

    bf16 q/k/v, or e4m3 q/k/v (torch.float8_e4m3fn) with the fp32 block scales of quantize_e4m3 (out stays bf16).

    out_heads_per_block > 0 selects the head-block output layout: `out` is then a 2-D bf16 view [Tq, row_width]
    (stride(1) == 1) and head h lands at columns (h // hpb) * out_block_stride + (h % hpb) * 128, which is how
    ProjInput (inference.py) has core and cross attention write the operand of the output projection in place.

    ctx: the context whose plan workspace the call uses (default: the per-device shared one).  Calls that share a
    context must be stream-ordered; a call that is meant to overlap another one on a side stream (cross-attention
    beside the core attention) needs a Context of its own."""
    fp8 = q.dtype == torch.float8_e4m3fn
    in_dtype = torch.float8_e4m3fn if fp8 else torch.bfloat16
    _thd(q, "q", in_dtype)
    dev = q.device
    if ctx is None:
        ctx = Context.get(dev)
    elif ctx.device != dev.index:
        raise ValueError("ctx belongs to another device")
    Tq, Hq, _ = q.shape
    p = AttnParams()
    p.struct_size = C.sizeof(AttnParams)
    p.dtype = _lib.DTYPE_FP8_E4M3 if fp8 else _lib.DTYPE_BF16
    if fp8:
        if q_scale is None or scale_chunk_tokens <= 0:
            raise ValueError("fp8 attention needs q_scale and scale_chunk_tokens")
        p.q_scale, p.scale_chunk_tokens = q_scale.data_ptr(), int(scale_chunk_tokens)
        if k_scale is not None:
            p.k_scale, p.v_scale = k_scale.data_ptr(), v_scale.data_ptr()
        if q_lo is not None:
            if q_lo.shape != q.shape or q_lo.stride() != q.stride() or q_lo.dtype != q.dtype:
                raise ValueError("q_lo must have q's shape, strides and dtype")
            p.q_lo = q_lo.data_ptr()
    p.q, p.q_stride_t, p.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1)
    if k is not None and k.shape[0] > 0:
        _thd(k, "k", in_dtype), _thd(v, "v", in_dtype)
        assert k.shape == v.shape
        p.k, p.k_stride_t, p.k_stride_h = k.data_ptr(), k.stride(0), k.stride(1)
        p.v, p.v_stride_t, p.v_stride_h = v.data_ptr(), v.stride(0), v.stride(1)
        p.total_k, p.n_kv_heads = k.shape[0], k.shape[1]
    else:
        if cache is None:
            raise ValueError("no keys: k is empty and there is no cache")
        p.total_k, p.n_kv_heads = 0, cache.n_kv_heads
    keep_peers = None
    if o_peers is not None:
        # fused output exchange: (ptrs per rank, token offsets [cp+1], first global head of this rank, stride_t, stride_h
        # [, heads per block, block stride] for the head-block layout over the global head index)
        ptrs, offs, head_off, st_t, st_h = o_peers[:5]
        if len(o_peers) == 7:
            p.o_heads_per_block, p.o_stride_block = int(o_peers[5]), int(o_peers[6])
        a_ptrs = (C.c_void_p * len(ptrs))(*[int(a) for a in ptrs])
        a_offs = (C.c_int32 * len(offs))(*[int(o) for o in offs])
        keep_peers = (a_ptrs, a_offs)
        p.o_peer_ptrs = C.cast(a_ptrs, C.POINTER(C.c_void_p))
        p.o_peer_offsets = C.cast(a_offs, C.POINTER(C.c_int32))
        p.n_o_peers, p.o_head_offset, p.o_stride_t, p.o_stride_h = len(ptrs), int(head_off), int(st_t), int(st_h)
        return_lse = False
    else:
        if out_heads_per_block > 0:
            if out is None or out.dim() != 2 or out.dtype != torch.bfloat16 or out.stride(1) != 1 or out.shape[0] < Tq:
                raise ValueError("head-block layout needs out as a 2-D bf16 view [Tq, row_width] with unit column stride")
            n_blocks = (Hq + out_heads_per_block - 1) // out_heads_per_block
            if (n_blocks - 1) * out_block_stride + out_heads_per_block * HEAD_DIM > out.shape[1] or \
                    out_block_stride < out_heads_per_block * HEAD_DIM:
                raise ValueError("head-block layout does not fit the rows of out")
            p.out, p.o_stride_t, p.o_stride_h = out.data_ptr(), out.stride(0), HEAD_DIM
            p.o_heads_per_block, p.o_stride_block = int(out_heads_per_block), int(out_block_stride)
        else:
            if out is None:
                out = torch.empty(Tq, Hq, HEAD_DIM, dtype=torch.bfloat16, device=dev)
            p.out, p.o_stride_t, p.o_stride_h = out.data_ptr(), out.stride(0), out.stride(1)
    lse = torch.empty(Tq, Hq, dtype=torch.float32, device=dev) if return_lse else None
    p.lse = lse.data_ptr() if lse is not None else None
    p.total_q, p.n_q_heads = Tq, Hq
    qr = _ranges_dev(q_ranges, dev)
    kr = _ranges_dev(k_ranges, dev)
    p.q_ranges, p.k_ranges = qr.data_ptr(), kr.data_ptr()
    p.n_ranges, p.n_k_ranges = qr.shape[0], kr.shape[0]
    ko = None
    if k_range_offsets is not None:
        ko = torch.as_tensor(np.asarray(k_range_offsets, dtype=np.int32), device=dev) \
            if not isinstance(k_range_offsets, torch.Tensor) else k_range_offsets.to(device=dev, dtype=torch.int32).contiguous()
        p.k_range_offsets = ko.data_ptr()
    p.max_seqlen_q, p.max_seqlen_k = int(max_seqlen_q), int(max_seqlen_k)
    p.softmax_scale = float(softmax_scale) if softmax_scale else 0.0
    ids = None
    if cache is not None and len(prefix_chunk_ids) > 0:
        ids = (C.c_int32 * len(prefix_chunk_ids))(*[int(c) for c in prefix_chunk_ids])
        p.cache, p.layer, p.n_prefix_chunks, p.prefix_chunk_ids = cache.handle, layer, len(prefix_chunk_ids), ids
    fn = {"tcgen05": lib.magi_chunk_attn_fwd, "simt": lib.magi_chunk_attn_fwd_simt}[impl]
    check(fn(ctx.handle, C.byref(p), _stream(stream)), ctx.handle)
    KERNEL_LAUNCHES[0] += 2  # planner + attention kernel
    # qr/kr/ko are consumed by a kernel already enqueued on this stream; torch's caching allocator only
    # reuses their memory for later work on the same stream, so dropping them here is safe.
    return out, lse


def quantize_e4m3(x: torch.Tensor, chunk_tokens: int, stream=None, residual: bool = False):
    """bf16 [T,H,128] (strided) -> (e4m3 [T,H,128], fp32 scales [ceil(T/chunk)*ceil(chunk/128), H]).
    128-token blocks are counted from each multiple of chunk_tokens; scale = absmax / 448.
    residual=True also returns the second e4m3 term e4m3(x/scale - x8) as a third value."""
    _thd(x, "x")
    T, H, _ = x.shape
    ctx = Context.get(x.device)
    nb = (chunk_tokens + 127) // 128
    n_chunks = (T + chunk_tokens - 1) // chunk_tokens
    x8 = torch.empty(T, H, HEAD_DIM, dtype=torch.float8_e4m3fn, device=x.device)
    scales = torch.ones(max(1, n_chunks * nb), H, dtype=torch.float32, device=x.device)
    lo = torch.empty_like(x8) if residual else None
    check(lib.magi_quantize_e4m3_block128(ctx.handle, x.data_ptr(), x.stride(0), x.stride(1), T, H, int(chunk_tokens),
                                          x8.data_ptr(), lo.data_ptr() if residual else None, scales.data_ptr(),
                                          _stream(stream)), ctx.handle)
    KERNEL_LAUNCHES[0] += 1
    return (x8, scales, lo) if residual else (x8, scales)


def bias_modulate_add(x: torch.Tensor, residual: Optional[torch.Tensor], condition_map: Optional[torch.Tensor],
                      gate: torch.Tensor, post_norm=None, out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """out = post_norm(x.float() * gate[condition_map]) + residual.float(), as bf16 - the reference's bias_modulate_add
    (inference/model/dit/dit_module.py:288-307) in one kernel.

    x [s, b, h] or [rows, h], bf16 or fp32; residual like x (bf16 or fp32) or None; condition_map [s, b] / [rows] int32 or
    int64 (None: gate row 0 everywhere); gate [b, n, h] or [n_gates, h], bf16 or fp32, last dim contiguous (a chunk of
    the fused gates is fine); post_norm: an object with weight, bias, eps and zero_centered_gamma (the reference's
    FusedLayerNorm), or None for the gating alone.  For b > 1 the rows are taken batch-major, as the reference's
    x.transpose(0, 1).flatten(0, 1) does, and the result comes back in x's shape."""
    dt = {torch.bfloat16: _lib.DTYPE_BF16, torch.float32: _lib.DTYPE_F32}
    shape = x.shape
    if x.dim() == 3:
        if x.shape[1] != 1:
            raise ValueError("batch > 1: pass x, residual and condition_map already flattened batch-major to [rows, h]")
        x = x[:, 0]
        residual = residual[:, 0] if residual is not None else None
        condition_map = condition_map[:, 0] if condition_map is not None else None
    if gate.dim() == 3:
        if gate.shape[0] != 1 and not gate.is_contiguous():
            raise ValueError("gate [b, n, h] with b > 1 must be contiguous")
        gate = gate.reshape(-1, gate.shape[-1]) if gate.is_contiguous() else gate[0]
    for name, t in (("x", x), ("gate", gate)) + ((("residual", residual),) if residual is not None else ()):
        if not t.is_cuda or t.dtype not in dt or t.dim() != 2 or t.stride(1) != 1:
            raise ValueError(f"{name} must be a CUDA bf16/fp32 matrix with a contiguous last dim")
    rows, h = x.shape
    ctx = Context.get(x.device)
    if out is None:
        out = torch.empty(rows, h, dtype=torch.bfloat16, device=x.device)
    p = ModulateParams()
    p.struct_size = C.sizeof(ModulateParams)
    p.x, p.x_stride, p.x_dtype = x.data_ptr(), x.stride(0), dt[x.dtype]
    if residual is not None:
        p.residual, p.residual_stride, p.residual_dtype = residual.data_ptr(), residual.stride(0), dt[residual.dtype]
    p.gate, p.gate_stride, p.gate_dtype, p.n_gates = gate.data_ptr(), gate.stride(0), dt[gate.dtype], gate.shape[0]
    if condition_map is not None:
        if condition_map.dtype not in (torch.int32, torch.int64) or condition_map.numel() != rows:
            raise ValueError("condition_map must be int32 or int64 with one entry per row")
        condition_map = condition_map.contiguous()
        p.condition_map, p.map_is_int64 = condition_map.data_ptr(), int(condition_map.dtype == torch.int64)
    keep = None
    if post_norm is not None:
        gamma = post_norm.weight.detach().to(device=x.device, dtype=torch.float32).contiguous()
        beta = post_norm.bias.detach().to(device=x.device, dtype=torch.float32).contiguous() if getattr(post_norm, "bias", None) is not None else None
        keep = (gamma, beta)
        p.gamma, p.beta = gamma.data_ptr(), beta.data_ptr() if beta is not None else None
        p.eps, p.gamma_plus_one = float(post_norm.eps), int(bool(getattr(post_norm, "zero_centered_gamma", False)))
    p.out, p.out_stride, p.rows, p.hidden = out.data_ptr(), out.stride(0), rows, h
    check(lib.magi_bias_modulate_add(ctx.handle, C.byref(p), _stream(stream)), ctx.handle)
    KERNEL_LAUNCHES[0] += 1
    return out.view(shape) if len(shape) == 3 else out


def div_clamp_to(x: torch.Tensor, scale: torch.Tensor, out: Optional[torch.Tensor] = None, stream=None) -> torch.Tensor:
    """e4m3(bf16(clamp(x.float() / scale.float(), -448, 448))): the reference's div_clamp_to
    (inference/model/dit/dit_module.py:364-384) in one kernel, byte-identical.  x bf16 [..., cols] (contiguous last dim,
    uniform row stride), scale fp32 with cols entries (per input channel) or one entry; returns float8_e4m3fn in x's shape."""
    if not x.is_cuda or x.dtype != torch.bfloat16 or x.stride(-1) != 1:
        raise ValueError("x must be a CUDA bf16 tensor with a contiguous last dim")
    cols = x.shape[-1]
    x2 = x.reshape(-1, cols)          # a view whenever the leading dims collapse; a copy otherwise
    if x2.stride(-1) != 1:
        x2 = x2.contiguous()
    rows = x2.shape[0]
    scale = scale.detach().to(device=x.device, dtype=torch.float32).reshape(-1).contiguous()
    if scale.numel() not in (1, cols):
        raise ValueError("scale must have one entry or one per channel of the last dimension")
    ctx = Context.get(x.device)
    if out is None:
        out = torch.empty(rows, cols, dtype=torch.float8_e4m3fn, device=x.device)
    elif out.dtype != torch.float8_e4m3fn or out.numel() != rows * cols or not out.is_contiguous():
        raise ValueError("out must be a contiguous float8_e4m3fn tensor of x's size")
    check(lib.magi_div_clamp_to_e4m3(ctx.handle, x2.data_ptr(), x2.stride(0) if rows > 1 else cols, rows, cols, scale.data_ptr(),
                                     int(scale.numel() == 1), out.data_ptr(), cols, _stream(stream)), ctx.handle)
    KERNEL_LAUNCHES[0] += 1
    return out.view(x.shape)


class PeerBuffer:
    """A device buffer other ranks of the box can map (CUDA IPC; plain peer loads / stores over NVLink, no multicast)."""

    def __init__(self, nbytes: int, device=None):
        self.ctx = Context.get(device)
        ptr = C.c_void_p()
        handle = C.create_string_buffer(64)
        check(lib.magi_peer_alloc(self.ctx.handle, int(nbytes), C.byref(ptr), handle), self.ctx.handle)
        self.ptr, self.handle, self.nbytes = ptr.value, handle.raw, int(nbytes)
        self._opened = []

    def open_peer(self, handle: bytes) -> int:
        ptr = C.c_void_p()
        check(lib.magi_peer_open(self.ctx.handle, handle, C.byref(ptr)), self.ctx.handle)
        self._opened.append(ptr.value)
        return ptr.value

    def as_tensor(self, shape, dtype=torch.bfloat16) -> torch.Tensor:
        """View of the local buffer as a torch tensor (no copy; the PeerBuffer must outlive the tensor)."""
        n = int(np.prod(shape))
        itemsize = torch.empty((), dtype=dtype).element_size()
        assert n * itemsize <= self.nbytes
        iface = {"shape": (n,), "typestr": {2: "<i2", 4: "<i4", 1: "|u1"}[itemsize], "data": (self.ptr, False), "version": 3}
        holder = type("_CudaArray", (), {"__cuda_array_interface__": iface})()
        t = torch.as_tensor(holder, device=torch.device("cuda", self.ctx.device))
        return t.view(dtype).view(*shape)

    def close(self):
        for ptr in self._opened:
            lib.magi_peer_close(self.ctx.handle, ptr)
        self._opened = []
        if self.ptr:
            lib.magi_peer_free(self.ctx.handle, self.ptr)
            self.ptr = None


def flex_attn(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_ranges: torch.Tensor, k_ranges: torch.Tensor,
              max_seqlen_q: int, max_seqlen_k: int, softmax_scale: Optional[float] = None,
              deterministic: bool = False, disable_fwd_atomic_reduction: bool = True, **_unused):
    """Drop-in for the reference's `flex_attention` (MagiAttention's flex_flash_attn_func surface as called at
    inference/model/dit/dit_module.py:1032-1043): packed q [(b sq),Hq,128], k/v [(b skv),Hkv,128], int32 [n,2]
    device ranges; returns (out, lse).  The kernel is deterministic and never reduces across CTAs, so
    `deterministic` and `disable_fwd_atomic_reduction` are accepted and have nothing to switch.
    Assign it with `dit_module.flex_attention = magi_b200.flex_attn`."""
    return chunk_attn(q, k, v, q_ranges, k_ranges, max_seqlen_q, max_seqlen_k, softmax_scale)


def varlen_attn(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, softmax_scale=None):
    """cu_seqlens convenience wrapper (sequence i of q attends to sequence i of k)."""
    cq = torch.as_tensor(cu_seqlens_q, dtype=torch.int32)
    ck = torch.as_tensor(cu_seqlens_k, dtype=torch.int32)
    qr = torch.stack([cq[:-1], cq[1:]], dim=1)
    kr = torch.stack([ck[:-1], ck[1:]], dim=1)
    return chunk_attn(q, k, v, qr, kr, max_seqlen_q, max_seqlen_k, softmax_scale)


def chunk_attn_noalloc(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_ranges: torch.Tensor, k_ranges: torch.Tensor,
                       max_seqlen_q: int, out: torch.Tensor, lse: Optional[torch.Tensor] = None,
                       status: Optional[torch.Tensor] = None, softmax_scale: Optional[float] = None, stream=None) -> None:
    """Attention for hosts that may not allocate on the device (all of HBM already belongs to somebody's arena).

    Every tensor is supplied by the caller - q/k/v bf16 [tokens, heads, 128], int32 device ranges [n,2], the bf16
    `out`, optionally an fp32 `lse` [tokens, Hq] and a 1-element int32 `status` - and neither this function nor the
    library entry point behind it (magi_chunk_attn_fwd_noalloc) allocates device memory: the planner's scratch is a
    fixed array inside the library.  Calls on one device must be stream-ordered (they share that array); the first
    call per device does a little set-up and should not sit inside a stream capture."""
    _thd(q, "q"), _thd(k, "k"), _thd(v, "v"), _thd(out, "out")
    for name, r in (("q_ranges", q_ranges), ("k_ranges", k_ranges)):
        if not (isinstance(r, torch.Tensor) and r.is_cuda and r.dtype == torch.int32 and r.is_contiguous() and r.dim() == 2):
            raise ValueError(f"{name} must be a contiguous int32 CUDA tensor [n, 2] supplied by the caller")
    p = AttnParams()
    p.struct_size = C.sizeof(AttnParams)
    p.dtype = _lib.DTYPE_BF16
    p.q, p.q_stride_t, p.q_stride_h = q.data_ptr(), q.stride(0), q.stride(1)
    p.k, p.k_stride_t, p.k_stride_h = k.data_ptr(), k.stride(0), k.stride(1)
    p.v, p.v_stride_t, p.v_stride_h = v.data_ptr(), v.stride(0), v.stride(1)
    p.out, p.o_stride_t, p.o_stride_h = out.data_ptr(), out.stride(0), out.stride(1)
    p.lse = lse.data_ptr() if lse is not None else None
    p.total_q, p.total_k, p.n_q_heads, p.n_kv_heads = q.shape[0], k.shape[0], q.shape[1], k.shape[1]
    p.q_ranges, p.k_ranges = q_ranges.data_ptr(), k_ranges.data_ptr()
    p.n_ranges, p.n_k_ranges = q_ranges.shape[0], k_ranges.shape[0]
    p.max_seqlen_q = int(max_seqlen_q)
    p.softmax_scale = float(softmax_scale) if softmax_scale else 0.0
    err = C.create_string_buffer(512)
    rc = lib.magi_chunk_attn_fwd_noalloc(C.byref(p), _stream(stream), status.data_ptr() if status is not None else None,
                                         err, len(err))
    if rc != _lib.MAGI_OK:
        raise _lib.MagiError(rc, err.value.decode())
