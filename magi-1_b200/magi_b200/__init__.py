"""magi_b200: B200 (sm_100a) chunk-wise block-causal GQA attention core behind a C ABI.

Importing the package loads libmagi_attn.so from the source tree and fails loudly if it is absent.
"""
from . import _lib
from ._lib import MagiError, LIB_PATH
from . import host
from . import inference
from .ops import (ChunkPagedKVCache, Context, PeerBuffer, bias_modulate_add, chunk_attn, div_clamp_to, chunk_attn_noalloc, flex_attn, head_block_copy, linear_qk_norm_rope, linear_qkv_norm_rope, qk_norm_rope, quantize_e4m3, varlen_attn)

__all__ = ["ChunkPagedKVCache", "Context", "PeerBuffer", "MagiError", "LIB_PATH", "bias_modulate_add", "chunk_attn", "div_clamp_to", "chunk_attn_noalloc", "flex_attn", "head_block_copy",
           "linear_qk_norm_rope", "linear_qkv_norm_rope", "qk_norm_rope", "quantize_e4m3", "varlen_attn"]
