"""Host-side metadata of the attention path, mirroring what the reference computes in Python around the kernels:
the rotary table (LearnableRotaryEmbeddingCat.get_embed as called by VideoDiTModel, inference/model/dit/dit_model.py:163-166),
the q/k range tensors (PackedCoreAttnParams, inference/model/dit/dit_model.py:220-259 and
inference/pipeline/video_generate.py:454-508) and the context-parallel sequence split
(inference/infra/parallelism/context_parallel.py:240-242).  Pure torch/numpy on the CPU; nothing here touches the GPU.
"""
import math
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

HEAD_DIM = 128


def default_bands(head_dim: int = HEAD_DIM, temperature: float = 10000.0) -> torch.Tensor:
    """Initial value of the learnable `rope.bands` parameter: temperature^(-j/nb), nb = head_dim/8 bands."""
    nb = head_dim // 8
    return 1.0 / (temperature ** (torch.arange(nb, dtype=torch.float32) / nb))


def rotary_table(T_total: int, H: int, W: int, bands: Optional[torch.Tensor] = None, keep_last_frames: Optional[int] = None
                 ) -> torch.Tensor:
    """[T*H*W, 6*nb] fp32 = cat(sin, cos): positions t = 0..T_total-1 (absolute, cached chunks included),
    h and w centred and rescaled to the 16x16 reference grid; angle columns t-bands | h-bands | w-bands.
    Only the rows of the last `keep_last_frames` frames are returned (the frames being forwarded)."""
    bands = default_bands() if bands is None else bands.detach().float().cpu()
    r = math.sqrt(H * W / 256.0)
    axes = [torch.arange(T_total, dtype=torch.float32),
            torch.arange(H, dtype=torch.float32) - (H - 1) / 2,
            torch.arange(W, dtype=torch.float32) - (W - 1) / 2]
    refs = [T_total, H / r, W / r]
    for i, (f, rf) in enumerate(zip((T_total, H, W), refs)):
        if f != 1:
            axes[i] = axes[i] / (f - 1) * (rf - 1)
    tt, hh, ww = torch.meshgrid(*axes, indexing="ij")
    ang = torch.stack([tt, hh, ww], dim=-1).unsqueeze(-1) * bands  # [T,H,W,3,nb]
    ang = ang.reshape(T_total * H * W, -1)
    emb = torch.cat([ang.sin(), ang.cos()], dim=-1)
    if keep_last_frames is not None:
        emb = emb[-keep_last_frames * H * W:]
    return emb.contiguous()


def split_sin_cos(rotary_pos_emb: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor]:
    """sin, cos = rotary_pos_emb.tensor_split(2, -1) (FullyParallelAttention.forward, dit_module.py:1147)."""
    sin, cos = rotary_pos_emb.tensor_split(2, -1)
    return sin.contiguous(), cos.contiguous()


def q_ranges_for_chunks(n: int, chunk_tokens: int, batch: int = 1) -> np.ndarray:
    """Consecutive [i*C, (i+1)*C) for the n*batch chunks of the packed query."""
    return np.array([[i * chunk_tokens, (i + 1) * chunk_tokens] for i in range(n * batch)], dtype=np.int32)


def default_k_ranges(n: int, chunk_tokens: int, slice_point: int = 0) -> np.ndarray:
    """Chunk j sees [0, (slice_point + j + 1) * C) of (prefix | current)."""
    return np.array([[0, (slice_point + j + 1) * chunk_tokens] for j in range(n)], dtype=np.int32)


def windowed_k_ranges(chunk_start: int, chunk_end: int, chunk_tokens: int, window: Sequence[int], slice_point: int
                      ) -> np.ndarray:
    """Sliding k-window per denoising chunk (noise2clean_kvrange): chunk c with window w sees chunks (c-w, c]."""
    base = chunk_start - slice_point
    out = []
    for j, c in enumerate(range(chunk_start, chunk_end)):
        w = window[min(j, len(window) - 1)]
        lo = max(c + 1 - w, base)
        out.append([(lo - base) * chunk_tokens, (c + 1 - base) * chunk_tokens])
    return np.array(out, dtype=np.int32)


def own_prefix_k_segments(n: int, chunk_tokens: int, n_prefix: int, batch: int = 1):
    """Concurrently denoising chunks that each see their own cached clean prefix plus themselves.

    Virtual K layout: [prefix chunk 0 .. n_prefix*batch - 1 | current chunks, batch-major].  Chunk i of batch
    element e attends to prefix chunks e*n_prefix .. e*n_prefix + min(i, n_prefix) - 1 and to itself.
    Returns (k_ranges [m,2], offsets [n*batch+1]) for the multi-interval form of the attention call."""
    C = chunk_tokens
    kr, offs = [], [0]
    P = n_prefix * batch
    for e in range(batch):
        for i in range(n):
            npre = min(i, n_prefix)
            if npre > 0:
                kr.append([e * n_prefix * C, (e * n_prefix + npre) * C])
            cur = P * C + (e * n + i) * C
            kr.append([cur, cur + C])
            offs.append(len(kr))
    return np.array(kr, dtype=np.int32), np.array(offs, dtype=np.int32)


def cp_split_sizes(seq_len: int, cp: int) -> List[int]:
    """Contiguous split of the sequence over the context-parallel ranks; the first seq_len % cp ranks get one more."""
    s = [seq_len // cp] * cp
    for i in range(seq_len % cp):
        s[i] += 1
    return s


def synthetic_norm_params(seed: int, d: int = HEAD_DIM):
    """Seeded stand-ins for the q/k layernorm weights (no checkpoint is available offline):
    gamma = 0.1 N(0,1) (applied as gamma + 1), beta = 0.02 N(0,1)."""
    g = torch.Generator(device="cpu").manual_seed(seed + 1000)
    return tuple(s * torch.randn(d, generator=g) for s in (0.1, 0.02, 0.1, 0.02))


def cross_attn_ranges(chunk_tokens: int, n_chunks: int, caption_lens: Sequence[int]):
    """q/kv ranges of the caption cross-attention (PackedCrossAttnParams, inference/model/dit/dit_model.py:220-244):
    query chunk i (consecutive blocks of chunk_tokens rows) attends to caption i's valid tokens in the packed
    y_xattn_flat.  Returns (q_ranges [n,2], kv_ranges [n,2]) as int32 arrays."""
    assert len(caption_lens) == n_chunks
    cq = np.arange(n_chunks + 1, dtype=np.int64) * chunk_tokens
    ck = np.concatenate([[0], np.cumsum(np.asarray(caption_lens, dtype=np.int64))])
    return (np.stack([cq[:-1], cq[1:]], 1).astype(np.int32), np.stack([ck[:-1], ck[1:]], 1).astype(np.int32))


def cp_cross_attn_ranges(q_ranges: np.ndarray, kv_ranges: np.ndarray, cp_split_sizes: Sequence[int], cp_rank: int):
    """Cross-attention ranges of one context-parallel rank: its contiguous slice of the query sequence is intersected
    with every q segment, the surviving pieces are rebased to the rank's local rows and keep their caption's kv range.
    Mirrors cp_update_cross_attn_qkv_range (inference/infra/parallelism/context_parallel.py:134-224) for batch 1,
    cp_shuffle_num 1.  Returns (q_ranges_local, kv_ranges_local, max_seqlen_q)."""
    bounds = np.concatenate([[0], np.cumsum(np.asarray(cp_split_sizes, dtype=np.int64))])
    lo, hi = int(bounds[cp_rank]), int(bounds[cp_rank + 1])
    q_out, k_out = [], []
    for (qs, qe), kr in zip(np.asarray(q_ranges).reshape(-1, 2), np.asarray(kv_ranges).reshape(-1, 2)):
        s, e = max(lo, int(qs)), min(hi, int(qe))
        if s < e:
            q_out.append([s, e])
            k_out.append([int(kr[0]), int(kr[1])])
    q_arr = np.asarray(q_out, dtype=np.int64).reshape(-1, 2)
    if len(q_arr):
        q_arr = q_arr - q_arr[:, 0].min()
    return q_arr.astype(np.int32), np.asarray(k_out, dtype=np.int32).reshape(-1, 2), hi - lo
