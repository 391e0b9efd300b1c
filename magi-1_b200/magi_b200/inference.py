"""Host-side mirror of the reference's attention module surface for the single-GPU strategy
(FullyParallelAttention with cp_strategy == "none", inference/model/dit/dit_module.py:1166-1173): the metadata types
the path consumes (inference/common/dataclass.py:22-83), the KV-cache gate and update rule
(adjust_key_and_value_for_inference / _full_adjust_key_and_value, dit_module.py:891-946) on top of the chunk-paged
cache, and core_attention (:1023-1066).  Same names, same argument meaning; tensors are never concatenated or copied
into a flat per-layer buffer - clean chunks live in pages and are read in place.
"""
from dataclasses import dataclass, field
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import ops

HEAD_DIM = 128


@dataclass(frozen=True)
class PackedCoreAttnParams:
    """q_range / k_range int32 [n, 2] on the device plus their numpy mirrors (inference/common/dataclass.py:22-30)."""
    q_range: torch.Tensor
    k_range: torch.Tensor
    np_q_range: np.ndarray
    np_k_range: np.ndarray
    max_seqlen_q: int
    max_seqlen_k: int

    @classmethod
    def from_numpy(cls, q_range: np.ndarray, k_range: np.ndarray, device) -> "PackedCoreAttnParams":
        q_range = np.asarray(q_range, dtype=np.int32).reshape(-1, 2)
        k_range = np.asarray(k_range, dtype=np.int32).reshape(-1, 2)
        return cls(torch.as_tensor(q_range, device=device), torch.as_tensor(k_range, device=device), q_range, k_range,
                   int((q_range[:, 1] - q_range[:, 0]).max()), int(k_range.max() - k_range.min()))


@dataclass(frozen=True)
class ModelMetaArgs:
    """The fields of the reference's ModelMetaArgs (inference/common/dataclass.py:44-59) that this path reads."""
    slice_point: int
    denoising_range_num: int
    clip_token_nums: int
    core_attn_params: PackedCoreAttnParams
    extract_prefix_video_feature: bool = False
    fwd_extra_1st_chunk: bool = False
    distill_nearly_clean_chunk: bool = False
    cp_split_sizes: Optional[List[int]] = None


class InferenceParams:
    """max_batch_size / max_sequence_length / update_kv_cache as in the reference (inference/common/dataclass.py:62-83);
    key_value_memory_dict[layer] of the reference becomes ONE chunk-paged cache shared by all layers (created on first
    use, pages of clip_token_nums tokens)."""

    def __init__(self, max_batch_size: int, max_sequence_length: int, n_layers: int = 1, kv_dtype: str = "bf16",
                 max_cached_chunks: Optional[int] = None):
        if max_batch_size != 1:
            raise ValueError("the KV cache path runs with max_batch_size == 1 (as every shipped reference config does)")
        self.max_batch_size = max_batch_size
        self.max_sequence_length = max_sequence_length
        self.sequence_len_offset = 0
        self.update_kv_cache = False
        self.n_layers = n_layers
        self.kv_dtype = kv_dtype
        self.max_cached_chunks = max_cached_chunks
        self.first_live_chunk = 0
        self.cache: Optional[ops.ChunkPagedKVCache] = None

    def evict_below(self, chunk_id: int) -> None:
        """Drop the pages of chunks < chunk_id in every layer.  The reference keeps the whole clip in its flat buffer
        (max_sequence_length = all tokens, pipeline/video_generate.py:311-314) although the k windows
        (noise2clean_kvrange / clean_chunk_kvrange, :467-508) never reach back further than a few chunks; with pages,
        a long clip only needs max_cached_chunks = window + chunks in flight slots per layer."""
        if self.cache is not None:
            for c in range(self.first_live_chunk, chunk_id):
                try:
                    self.cache.evict(c)
                except ops.MagiError:  # a chunk that was never stored
                    pass
        self.first_live_chunk = max(self.first_live_chunk, chunk_id)

    def get_cache(self, chunk_tokens: int, n_kv_heads: int, device) -> ops.ChunkPagedKVCache:
        if self.cache is None:
            max_chunks = self.max_cached_chunks or max(1, self.max_sequence_length // chunk_tokens)
            self.cache = ops.ChunkPagedKVCache(self.n_layers, max_chunks, chunk_tokens, n_kv_heads, dtype=self.kv_dtype,
                                               device=device)
        elif self.cache.chunk_tokens != chunk_tokens or self.cache.n_kv_heads != n_kv_heads:
            raise ValueError("the cache was created for another chunk size / head count")
        return self.cache


class HostPageStore:
    """Pinned-host tier under the page pool.

    The reference's kv_offload keeps the whole per-layer cache in pinned host memory and copies the prefix to the GPU for
    every layer of every step (inference/model/dit/dit_module.py:803-811, :915).  Here pages stay in HBM while a k window
    can reach them; spill() moves the pages of one chunk (all layers) to pinned memory and frees its slots, prefetch()
    brings them back on a side stream ahead of the step that needs them.  bf16 pages only (an fp8 page would be read
    back dequantised)."""

    def __init__(self, cache: ops.ChunkPagedKVCache):
        if cache.dtype != "bf16":
            raise ValueError("the host tier holds bf16 pages")
        self.cache = cache
        self.pages = {}      # chunk id -> (k [L, C, Hkv, 128], v) in pinned memory
        self._inflight = {}  # chunk id -> (k, v, event): pinned buffers that copy kernels may still be reading

    def _reap(self) -> None:
        """Release the pinned buffers of prefetches whose copies have completed."""
        for cid in [c for c, (_, _, ev) in self._inflight.items() if ev.query()]:
            del self._inflight[cid]

    def spill(self, chunk_id: int, stream=None) -> None:
        """Stream-ordered on `stream` (default: the current stream, i.e. after the step that last used the page and
        before anything that reuses its slot)."""
        self._reap()
        c = self.cache
        shape = (c.n_layers, c.chunk_tokens, c.n_kv_heads, HEAD_DIM)
        k = torch.empty(shape, dtype=torch.bfloat16).pin_memory()
        v = torch.empty(shape, dtype=torch.bfloat16).pin_memory()
        for layer in range(c.n_layers):
            c.read_into(layer, chunk_id, k[layer], v[layer], stream)
        c.evict(chunk_id)
        self.pages[chunk_id] = (k, v)

    def prefetch(self, chunk_id: int, stream: Optional[torch.cuda.Stream] = None) -> torch.cuda.Event:
        """Bring a spilled chunk back into free slots on `stream` (a side stream overlaps it with compute); wait for the
        returned event on the compute stream before the attention call that lists the chunk."""
        self._reap()
        k, v = self.pages.pop(chunk_id)
        s = stream if stream is not None else torch.cuda.current_stream()
        for layer in range(self.cache.n_layers):
            self.cache.append_from_host(layer, chunk_id, k[layer], v[layer], s)
        ev = torch.cuda.Event()
        ev.record(s)
        # The copy kernels read the pinned buffers over PCIe on `s`; torch's pinned-memory cache knows nothing about a
        # library kernel, so the buffers are held here, per chunk, until the event has completed (several prefetches
        # in a row are the normal use).
        self._inflight[chunk_id] = (k, v, ev)
        return ev


class ProjInput:
    """The operand of the attention output projection, written in place by the two attention calls.

    The reference concatenates core_attn_out and cross_attn_out along the hidden dimension and permutes it with
    "sq b (n hn hd) -> sq b (hn n hd)", n=2, hn=8 (attn_linear_proj, inference/model/dit/dit_module.py:1332-1346): two
    extra HBM passes over [sq, 2*Hq*128].  Here `buf` [n_tokens, 2*Hq*128] already has that layout; dest(0) / dest(1)
    are the keyword arguments that make ops.chunk_attn store core / cross attention heads at their final columns."""

    def __init__(self, n_tokens: int, n_q_heads: int, device, hn: int = 8):
        if n_q_heads % hn:
            raise ValueError("the head count must be a multiple of hn")
        self.n_q_heads, self.hn = n_q_heads, hn
        self.heads_per_block = n_q_heads // hn
        self.hd = self.heads_per_block * HEAD_DIM          # width of one (n, hn) piece
        self.buf = torch.empty(n_tokens, 2 * n_q_heads * HEAD_DIM, dtype=torch.bfloat16, device=device)

    def dest(self, which: int) -> dict:
        """which = 0: core attention, 1: cross attention."""
        return dict(out=self.buf[:, which * self.hd:], out_heads_per_block=self.heads_per_block,
                    out_block_stride=2 * self.hd)

    @staticmethod
    def reference_layout(core: torch.Tensor, cross: torch.Tensor, hn: int = 8) -> torch.Tensor:
        """What the reference computes from the two [sq, Hq, 128] outputs (for tests): cat + rearrange."""
        sq = core.shape[0]
        x = torch.cat([core.reshape(sq, -1), cross.reshape(sq, -1)], dim=1)           # (n hn hd)
        return x.view(sq, 2, hn, -1).permute(0, 2, 1, 3).reshape(sq, -1).contiguous()  # (hn n hd)


def bias_modulate_add(x: torch.Tensor, residual: torch.Tensor, condition_map: torch.Tensor, gate: torch.Tensor, post_norm):
    """Same name and arguments as the reference's bias_modulate_add (inference/model/dit/dit_module.py:288-307), called
    by TransformerLayer.gating_and_mlp (:1348-1367) on the attention projection's output and again after the MLP:
    x, residual [s, b, h]; condition_map [s, b]; gate [b, denoising_range_num, h] (one half of the soft-capped adaLN
    gates); post_norm: the layer's FusedLayerNorm.  One kernel, bf16 result (the reference casts to params_dtype right
    after the call)."""
    return ops.bias_modulate_add(x, residual, condition_map, gate, post_norm)


def div_clamp_to(x: torch.Tensor, scale: torch.Tensor) -> torch.Tensor:
    """Same name and arguments as the reference's div_clamp_to (inference/model/dit/dit_module.py:364-384)."""
    return ops.div_clamp_to(x, scale)


class PerTensorQuantizedFp8Linear:
    """The reference's PerTensorQuantizedFp8Linear.forward (inference/model/dit/dit_module.py:431-461): the input is
    divided by the per-input-channel `input_scale`, clamped and cast to e4m3 (one kernel here), then multiplied with the
    e4m3 weight [out_features, in_features] by a library FP8 GEMM with fp32 accumulation and rescaled.  The reference hands
    `input_scale` (a vector of in_features entries) and `weight_scale` (one entry) to flashinfer's bmm_fp8 as its two
    per-tensor scales; bmm_fp8 applies them as scalars, and so does this class, taking the first entry of each.  The GEMM is
    cuBLASLt through torch._scaled_mm: a plain library GEMM, outside the hand-written path."""

    def __init__(self, weight: torch.Tensor, weight_scale: torch.Tensor, input_scale: torch.Tensor, dtype=torch.bfloat16):
        if weight.dim() == 3:
            weight = weight[0]
        if weight.dtype != torch.float8_e4m3fn or weight.dim() != 2:
            raise ValueError("weight must be float8_e4m3fn [out_features, in_features] (or [1, out, in])")
        self.out_features, self.in_features = weight.shape
        self.weight = weight.contiguous()
        self.weight_scale = weight_scale.detach().float().reshape(-1)
        self.input_scale = input_scale.detach().float().reshape(-1)
        self.output_dtype = dtype

    def _divisor(self) -> torch.Tensor:
        return self.input_scale

    def _gemm_scales(self):
        return self.input_scale[:1], self.weight_scale[:1]

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        x8 = ops.div_clamp_to(x, self._divisor())
        a_scale, b_scale = self._gemm_scales()
        a = x8.reshape(-1, self.in_features)
        y = torch._scaled_mm(a, self.weight.t(), scale_a=a_scale.to(a.device).reshape(()), scale_b=b_scale.to(a.device).reshape(()),
                             out_dtype=self.output_dtype)
        return y.reshape(x.shape[:-1] + (self.out_features,))

    __call__ = forward


class PerChannelQuantizedFp8Linear(PerTensorQuantizedFp8Linear):
    """The reference's PerChannelQuantizedFp8Linear.forward (dit_module.py:466-495): the divisor is the per-input-channel
    `smooth_scale` [1, in_features]; the GEMM's input scale is the one-entry `input_scale`."""

    def __init__(self, weight, weight_scale, input_scale, smooth_scale, dtype=torch.bfloat16):
        super().__init__(weight, weight_scale, input_scale, dtype)
        self.smooth_scale = smooth_scale.detach().float().reshape(-1)

    def _divisor(self) -> torch.Tensor:
        return self.smooth_scale


def get_xqkv(mixed_qqkv: torch.Tensor, key_value_states: torch.Tensor, wqx: torch.Tensor, w_kv_xattn: torch.Tensor,
             q_gamma, q_beta, k_gamma, k_beta, eps: float = 1e-6):
    """FullyParallelAttention.get_xqkv (inference/model/dit/dit_module.py:1005-1021) from the projections on, two kernels:
    mixed_qqkv [(b sq), hidden] (the output of forward_ln) through linear_qkv.qx and q_layernorm_xattn (no rotary), and the
    caption states key_value_states [y_total_token, caption_dim] through linear_kv_xattn - whose weight rows are
    (k of head 0, v of head 0, k of head 1, ...), :1015 - with k_layernorm_xattn on the k halves.  Returns
    query_xattn [(b sq), Hq, 128], key_xattn and value_xattn [y_total_token, Hkv, 128] (views of one K|V buffer)."""
    (q,) = ops.linear_qkv_norm_rope(mixed_qqkv, [dict(weight=wqx, gamma=q_gamma, beta=q_beta, rotate=False)], None, None, eps)
    (kv,) = ops.linear_qkv_norm_rope(key_value_states, [dict(weight=w_kv_xattn, gamma=k_gamma, beta=k_beta, plain_odd_heads=True)],
                                     None, None, eps)
    kv = kv.view(kv.shape[0], -1, 2 * ops.HEAD_DIM)
    return q, kv[..., :ops.HEAD_DIM], kv[..., ops.HEAD_DIM:]


class ChunkCausalSelfAttention:
    """One layer's self-attention core: prologue -> KV-cache gate -> chunk-causal attention."""

    def __init__(self, layer_number: int, n_q_heads: int, n_kv_heads: int, q_gamma, q_beta, k_gamma, k_beta,
                 eps: float = 1e-6, norm_mode: str = "layernorm_1p"):
        self.layer_number, self.hq, self.hkv = layer_number, n_q_heads, n_kv_heads
        self.q_gamma, self.q_beta, self.k_gamma, self.k_beta = q_gamma, q_beta, k_gamma, k_beta
        self.eps, self.norm_mode = eps, norm_mode

    # get_q / get_k (dit_module.py:953-980) after the projection: x [(sq b), heads, 128] bf16 views
    def get_q(self, xq, cos_emb, sin_emb):
        return ops.qk_norm_rope(xq, self.q_gamma, self.q_beta, cos_emb, sin_emb, self.eps, self.norm_mode)

    def get_k(self, xk, cos_emb, sin_emb):
        return ops.qk_norm_rope(xk, self.k_gamma, self.k_beta, cos_emb, sin_emb, self.eps, self.norm_mode)

    def adjust_key_and_value_for_inference(self, key: torch.Tensor, value: torch.Tensor,
                                           inference_params: Optional[InferenceParams], meta_args: ModelMetaArgs
                                           ) -> Tuple[Optional[ops.ChunkPagedKVCache], Sequence[int]]:
        """The reference's gate and update rule (dit_module.py:891-946), on pages.

        Touches the cache only if extract_prefix_video_feature or fwd_extra_1st_chunk or slice_point > 0.  Then the
        prefix is chunks 0 .. slice_point-1 (read in place by the kernel), and with update_kv_cache the current chunks
        are written to pages slice_point + j - all of them, or all but the last when distill_nearly_clean_chunk.
        Returns (cache or None, prefix chunk ids); key / value themselves are used as they are.  After
        InferenceParams.evict_below(c) the prefix starts at chunk c."""
        if inference_params is None:
            return None, ()
        if not (meta_args.extract_prefix_video_feature or meta_args.fwd_extra_1st_chunk or meta_args.slice_point > 0):
            return None, ()
        C = meta_args.clip_token_nums
        cache = inference_params.get_cache(C, self.hkv, key.device)
        if inference_params.update_kv_cache:
            n_tok = key.shape[0] - C if meta_args.distill_nearly_clean_chunk else key.shape[0]
            if (meta_args.slice_point * C + n_tok) > inference_params.max_sequence_length:
                raise ValueError("KV cache update beyond max_sequence_length")
            for j in range((n_tok + C - 1) // C):
                lo, hi = j * C, min((j + 1) * C, n_tok)
                cache.append(self.layer_number, meta_args.slice_point + j, key[lo:hi], value[lo:hi])
        return cache, list(range(inference_params.first_live_chunk, meta_args.slice_point))

    def core_attention(self, query, key, value, meta_args: ModelMetaArgs, cache=None, prefix_chunk_ids=(),
                       proj_in: Optional[ProjInput] = None):
        """With proj_in the heads are stored at their final columns of the projection operand (proj_in.buf)."""
        p = meta_args.core_attn_params
        dest = proj_in.dest(0) if proj_in is not None else {}
        k_range = p.k_range
        if cache is not None and meta_args.slice_point > len(prefix_chunk_ids):
            # k_range counts tokens from chunk 0 of the clip (the reference's flat buffer); the page list starts at the
            # first chunk that is still cached
            off = (meta_args.slice_point - len(prefix_chunk_ids)) * meta_args.clip_token_nums
            if int(p.np_k_range.min()) < off:
                raise ValueError("k_range reaches into chunks that were evicted")
            k_range = p.k_range - off
        out, _ = ops.chunk_attn(query, key, value, p.q_range, k_range, p.max_seqlen_q, p.max_seqlen_k, cache=cache,
                                layer=self.layer_number, prefix_chunk_ids=prefix_chunk_ids, return_lse=False, **dest)
        return proj_in.buf if proj_in is not None else out

    def forward(self, xq, xk, xv, inference_params: Optional[InferenceParams], rotary_pos_emb: torch.Tensor,
                meta_args: ModelMetaArgs, proj_in: Optional[ProjInput] = None) -> torch.Tensor:
        """xq [(sq b), Hq, 128], xk / xv [(sq b), Hkv, 128]: the q / k / v projections (bf16, any strides);
        rotary_pos_emb [(sq), 96] = cat(sin, cos) as LearnableRotaryEmbeddingCat returns it.  Returns
        core_attn_out [(sq b), Hq, 128]."""
        sin_emb, cos_emb = rotary_pos_emb.tensor_split(2, -1)
        key = self.get_k(xk, cos_emb, sin_emb)
        query = self.get_q(xq, cos_emb, sin_emb)
        cache, prefix = self.adjust_key_and_value_for_inference(key, xv, inference_params, meta_args)
        return self.core_attention(query, key, xv, meta_args, cache, prefix, proj_in)

    def forward_from_hidden(self, mixed_qqkv: torch.Tensor, wq: torch.Tensor, wk: torch.Tensor, wv: torch.Tensor,
                            inference_params: Optional[InferenceParams], rotary_pos_emb: torch.Tensor,
                            meta_args: ModelMetaArgs, proj_in: Optional[ProjInput] = None) -> torch.Tensor:
        """The same layer from one step earlier: mixed_qqkv [(sq b), hidden] bf16 is the output of linear_qkv.forward_ln,
        wq / wk / wv the bf16 torch.nn.Linear weights of linear_qkv.q / .k / .v (dit_module.py:406-408).  The three
        projections run in one kernel with the prologue in its epilogue (get_qkv, :953-1003): the projections' bf16 outputs
        never go to HBM and x is read from HBM once."""
        sin_emb, cos_emb = rotary_pos_emb.tensor_split(2, -1)
        query, key, value = ops.linear_qkv_norm_rope(mixed_qqkv, [
            dict(weight=wq, gamma=self.q_gamma, beta=self.q_beta, norm_mode=self.norm_mode),
            dict(weight=wk, gamma=self.k_gamma, beta=self.k_beta, norm_mode=self.norm_mode),
            dict(weight=wv, norm_mode="none")], cos_emb, sin_emb, self.eps)
        cache, prefix = self.adjust_key_and_value_for_inference(key, value, inference_params, meta_args)
        return self.core_attention(query, key, value, meta_args, cache, prefix, proj_in)
