"""How far two runs' logits are apart: the reference's own measure of a reduced-precision path.

tools/moe_cuda_bench.py:177-212 of the reference compares the next-token logits of two builds by whether
the best token is the same, by the share of the k best tokens they have in common, and by the mean and the
largest absolute difference.  Here the same figures for rows of logits [rows, vocab], averaged over the rows
(the largest difference is the largest over all rows); the bfloat16 path is reported against the float32 path
with them.
"""
from __future__ import annotations

import torch


def compare_logits(ref: torch.Tensor, other: torch.Tensor, overlap_k: int = 5) -> dict:
    """ref, other: float tensors [rows, vocab] (or [vocab]).  Returns top1_match, overlap_at_k (both averaged
    over rows, 0..1), mean_abs, max_abs, and for scale ref_std and ref_max_abs (spread and largest magnitude of
    the reference's logits)."""
    ref, other = ref.detach().float().reshape(-1, ref.shape[-1]), other.detach().float().reshape(-1, other.shape[-1])
    if ref.shape != other.shape:
        raise ValueError(f"compare_logits: shapes differ, {tuple(ref.shape)} and {tuple(other.shape)}")
    k = max(1, min(int(overlap_k), ref.shape[1]))
    a, b = ref.topk(k, dim=1).indices, other.topk(k, dim=1).indices
    common = (a[:, :, None] == b[:, None, :]).any(-1).float().sum(1) / k
    diff = (ref - other).abs()
    finite = torch.isfinite(ref) & torch.isfinite(other)
    diff = torch.where(finite, diff, torch.full_like(diff, float("inf")))
    return {"top1_match": float((a[:, 0] == b[:, 0]).float().mean()), "overlap_at_k": float(common.mean()),
            "mean_abs": float(diff.mean()), "max_abs": float(diff.max()), "ref_std": float(ref.std()), "ref_max_abs": float(ref.abs().max())}
