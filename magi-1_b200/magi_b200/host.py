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
    """Chunk j sees [0, (slice_point + j + 1) * C) of (prefix | current): generate_default_kvrange for one batch element."""
    return generate_default_kvrange(slice_point, n, chunk_tokens)


def _batched(k_chunk_ranges: np.ndarray, range_num: int, chunk_token_nums: int, batch_size: int) -> np.ndarray:
    """Chunk-unit ranges of one batch element -> token ranges of all: element i is shifted by i * range_num chunks
    (k_batch_start, video_generate.py:461-464, :495-497)."""
    r = np.asarray(k_chunk_ranges, dtype=np.int64).reshape(-1, 2)
    return (np.concatenate([r + i * range_num for i in range(batch_size)]) * chunk_token_nums).astype(np.int32)


def generate_default_kvrange(slice_point: int, denoising_range_num: int, chunk_token_nums: int, batch_size: int = 1
                             ) -> np.ndarray:
    """No windows configured: denoising chunk j sees chunks [0, slice_point + j + 1) of (cache | current).
    SampleTransport.generate_default_kvrange (inference/pipeline/video_generate.py:454-465); batch element i counts its
    chunks from i * (slice_point + denoising_range_num)."""
    ends = slice_point + 1 + np.arange(denoising_range_num)
    return _batched(np.stack([np.zeros_like(ends), ends], 1), slice_point + denoising_range_num, chunk_token_nums, batch_size)


def generate_noise2clean_kvrange(slice_point: int, denoising_range_num: int, noise2clean_kvrange: Sequence[int],
                                 clean_chunk_kvrange: int, denoise_step_of_each_chunk: Sequence[int], num_steps: int,
                                 chunk_token_nums: int, batch_size: int = 1) -> np.ndarray:
    """The k window of every denoising chunk follows how far that chunk has been denoised: a chunk at denoise step s looks
    back noise2clean_kvrange[s // (num_steps / len(noise2clean_kvrange))] chunks (itself included), a clean chunk
    (s == num_steps, the extra first chunk) clean_chunk_kvrange chunks, -1 meaning the last window.
    SampleTransport.generate_noise2clean_kvrange (inference/pipeline/video_generate.py:467-508)."""
    if len(denoise_step_of_each_chunk) != denoising_range_num:
        raise ValueError("one denoise step per denoising chunk")
    if len(noise2clean_kvrange) == 0 or num_steps % len(noise2clean_kvrange):
        raise ValueError("num_steps must be a positive multiple of len(noise2clean_kvrange)")
    if clean_chunk_kvrange == -1:
        clean_chunk_kvrange = noise2clean_kvrange[-1]
    per_stage = num_steps // len(noise2clean_kvrange)
    look_back = np.array([clean_chunk_kvrange if s == num_steps else noise2clean_kvrange[s // per_stage]
                          for s in denoise_step_of_each_chunk], dtype=np.int64)
    ends = slice_point + 1 + np.arange(denoising_range_num)
    return _batched(np.stack([np.maximum(ends - look_back, 0), ends], 1), slice_point + denoising_range_num, chunk_token_nums,
                    batch_size)


def generate_kvrange_for_denoising_video(slice_point: int, denoising_range_num: int, denoise_step_of_each_chunk: Sequence[int],
                                         noise2clean_kvrange: Sequence[int], clean_chunk_kvrange: int, num_steps: int,
                                         chunk_token_nums: int, batch_size: int = 1) -> np.ndarray:
    """The dispatch of SampleTransport.generate_kvrange_for_denoising_video (video_generate.py:510-527): windows if the
    runtime config lists any, otherwise everything before the chunk."""
    if len(noise2clean_kvrange) == 0:
        return generate_default_kvrange(slice_point, denoising_range_num, chunk_token_nums, batch_size)
    return generate_noise2clean_kvrange(slice_point, denoising_range_num, noise2clean_kvrange, clean_chunk_kvrange,
                                        denoise_step_of_each_chunk, num_steps, chunk_token_nums, batch_size)


def generate_kvrange_for_prefix_video(range_num: int, chunk_token_nums: int, clean_chunk_kvrange: int = -1,
                                      noise2clean_kvrange: Sequence[int] = (), batch_size: int = 1) -> np.ndarray:
    """Feature extraction of a clean prefix video: chunk j (1-based end) looks back clean_chunk_kvrange chunks, or the last
    window, or 8.  SampleTransport.generate_kvrange_for_prefix_video (video_generate.py:371-387)."""
    prev = clean_chunk_kvrange if clean_chunk_kvrange != -1 else (noise2clean_kvrange[-1] if len(noise2clean_kvrange) else 8)
    ends = 1 + np.arange(range_num)
    return _batched(np.stack([np.maximum(ends - prev, 0), ends], 1), range_num, chunk_token_nums, batch_size)


def generate_kv_range_for_uncondition(n_chunks: int, chunk_token_nums: int) -> np.ndarray:
    """The unconditional pass lays the chunks out as the batch and lets each see only itself:
    VideoDiTModel.generate_kv_range_for_uncondition (inference/model/dit/dit_model.py:92-101)."""
    return q_ranges_for_chunks(n_chunks, chunk_token_nums)


def generate_sequences(chunk_num: int, window_size: int, chunk_offset: int):
    """Per denoise stage: the chunks in flight [clip_start, clip_end) and their positions [t_start, t_end) in the window
    (generate_sequences, inference/pipeline/video_generate.py:164-180)."""
    stages = range(chunk_offset, chunk_num + window_size - 1)
    clip_start = [max(chunk_offset, i - window_size + 1) for i in stages]
    clip_end = [min(chunk_num, i + 1) for i in stages]
    t_start = [max(0, i - chunk_num + 1) for i in stages]
    t_end = [min(window_size, i - chunk_offset + 1) for i in stages]
    return clip_start, clip_end, t_start, t_end


def denoise_schedule(num_steps: int, window_size: int, chunk_num: int, chunk_offset: int = 0):
    """Every forward step of a clip as the sampler derives it (SampleTransport.generate_denoise_status_and_sequences,
    get_denoise_step_of_each_chunk and the slice_point rule of forward_velocity, video_generate.py:343-358, :551-571,
    :606-628).  Yields dicts: step, chunk_start, chunk_end, fwd_extra_1st_chunk, slice_point, denoising_range_num,
    denoise_step_of_each_chunk (newest chunk last; the extra clean first chunk, when forwarded, is at num_steps)."""
    per_stage = num_steps // window_size
    cs, ce, ts, te = generate_sequences(chunk_num, window_size, chunk_offset)
    for step in range(per_stage * (chunk_num + window_size - 1 - chunk_offset)):
        stage, idx = divmod(step, per_stage)
        extra = cs[stage] > chunk_offset and idx == 0
        steps_of = [i * per_stage + idx for i in range(ts[stage], te[stage])][::-1]
        if extra:
            steps_of = [num_steps] + steps_of
        yield dict(step=step, chunk_start=cs[stage], chunk_end=ce[stage], fwd_extra_1st_chunk=extra,
                   slice_point=cs[stage] - 1 if extra else cs[stage],
                   denoising_range_num=ce[stage] - cs[stage] + (1 if extra else 0), denoise_step_of_each_chunk=steps_of)


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


def scatter_to_context_parallel_region(x: torch.Tensor, cp_split_sizes: Sequence[int], cp_rank: int, cp_shuffle_num: int = 1,
                                       cp_pad_size: int = 0) -> torch.Tensor:
    """This rank's rows of a tensor split along its first dimension (scatter_to_context_parallel_region,
    inference/infra/parallelism/context_parallel.py:29-53).  With cp_shuffle_num > 1 the sequence is first cut into that
    many equal pieces, each piece is (zero-)padded by cp_pad_size / cp_shuffle_num rows and split by
    cp_split_sizes / cp_shuffle_num, and the rank's slices of all pieces are concatenated."""
    if len(cp_split_sizes) == 1:
        return x
    sizes = [int(s) for s in cp_split_sizes]
    if cp_shuffle_num > 1:
        if cp_pad_size % cp_shuffle_num or any(s % cp_shuffle_num for s in sizes):
            raise ValueError("cp_pad_size and the split sizes must be multiples of cp_shuffle_num")
        pad = cp_pad_size // cp_shuffle_num
        sizes = [s // cp_shuffle_num for s in sizes]
        pieces = torch.chunk(x, cp_shuffle_num, dim=0)
    else:
        pad, pieces = cp_pad_size, (x,)
    lo = sum(sizes[:cp_rank])
    out = []
    for piece in pieces:
        if pad:
            piece = torch.cat([piece, piece.new_zeros((pad,) + tuple(piece.shape[1:]))])
        out.append(piece[lo:lo + sizes[cp_rank]])
    return torch.cat(out).contiguous() if len(out) > 1 else out[0].contiguous()


def cp_ulysses_process(cp_size: int, cp_rank: int, x: torch.Tensor, condition_map: torch.Tensor, rope: torch.Tensor,
                       xattn_q_ranges: np.ndarray, xattn_kv_ranges: np.ndarray):
    """What a rank keeps of the embedded sequence before the first layer under Ulysses context parallelism
    (cp_ulysses_process, inference/infra/parallelism/context_parallel.py:227-254): the contiguous, possibly uneven split
    of x [seq, N, D], condition_map [seq] and rope [seq, 96], and the cross-attention ranges rewritten for the rank's rows.
    Returns (x, condition_map, rope, cp_split_sizes, (q_ranges, kv_ranges, max_seqlen_q))."""
    seq_len = x.shape[0]
    if rope.shape[0] != seq_len or condition_map.shape[0] != seq_len:
        raise ValueError("x, condition_map and rope must have the same number of rows")
    splits = cp_split_sizes(seq_len, cp_size)
    parts = [scatter_to_context_parallel_region(t, splits, cp_rank) for t in (x, condition_map, rope)]
    return parts[0], parts[1], parts[2], splits, cp_cross_attn_ranges(xattn_q_ranges, xattn_kv_ranges, splits, cp_rank)


def cp_cross_attn_ranges(q_ranges: np.ndarray, kv_ranges: np.ndarray, cp_split_sizes: Sequence[int], cp_rank: int):
    """Cross-attention ranges of one context-parallel rank: its contiguous slice of the query sequence is intersected
    with every q segment, the surviving pieces are rebased to the rank's local rows and keep their caption's kv range.
    Mirrors cp_update_cross_attn_qkv_range (inference/infra/parallelism/context_parallel.py:134-224) for batch 1,
    cp_shuffle_num 1 - the only way the Ulysses path calls it (:250), and the only way it can be called in general: with
    more batch elements or shuffle pieces the reference's closing assertion on the unique q and k boundaries (:213-215)
    fails unless the surviving captions are adjacent, and it fails likewise for an empty caption.  (Empty captions are
    accepted here; the attention kernel gives their rows zeros.)  Returns (q_ranges_local, kv_ranges_local, max_seqlen_q)."""
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
