"""Helpers shared by the GPU parity tests (the checker side runs on the CPU oracle)."""
import numpy as np
import torch

from oracle import chunk_attn_oracle as O

# Acceptance tolerances for the bf16 kernel against the fp32 oracle on identical (bf16-rounded) inputs.
MAX_ABS = 2e-2
MIN_COS = 0.9999


def assert_close(got: torch.Tensor, ref: torch.Tensor, max_abs=MAX_ABS, min_cos=MIN_COS, what=""):
    got = got.detach().float().cpu()
    ref = ref.detach().float().cpu()
    assert got.shape == ref.shape, (got.shape, ref.shape)
    assert torch.isfinite(got).all(), f"{what}: non-finite output"
    err = (got - ref).abs().max().item()
    # an all-zero reference (q-ranges without keys) has no direction: the max-abs bound alone decides
    cos = O.cosine(got, ref) if float(ref.abs().max()) > 0 else 1.0
    assert err <= max_abs and cos >= min_cos, f"{what}: max-abs {err:.4g} (<= {max_abs}), cosine {cos:.6f} (>= {min_cos})"
    return err, cos


def as_segments(k_ranges, offsets=None):
    k_ranges = np.asarray(k_ranges).reshape(-1, 2)
    if offsets is None:
        return [[list(r)] for r in k_ranges]
    return [[list(r) for r in k_ranges[offsets[i]:offsets[i + 1]]] for i in range(len(offsets) - 1)]


def oracle_on_rows(q, k, v, q_ranges, segments, rows, softmax_scale=None):
    """Oracle output for a sample of q rows only (rows: sorted 1-D LongTensor), so full-size cases stay cheap.
    Returns (out [len(rows),Hq,D], lse)."""
    q_ranges = np.asarray(q_ranges).reshape(-1, 2)
    rows = torch.as_tensor(rows, dtype=torch.long)
    sub_ranges, sub_segs, pieces, keep = [], [], [], []
    pos = 0
    for i, (qs, qe) in enumerate(q_ranges):
        sel = rows[(rows >= qs) & (rows < qe)]
        if sel.numel() == 0:
            continue
        pieces.append(q[sel])
        keep.append(sel)
        sub_ranges.append([pos, pos + sel.numel()])
        sub_segs.append(segments[i])
        pos += sel.numel()
    qq = torch.cat(pieces)
    out, lse = O.range_attention(qq, k, v, sub_ranges, sub_segs, softmax_scale)
    return torch.cat(keep), out, lse
