"""Batch x head sharding of an attention problem over the GPUs of one box.

Every (batch, head) pair is an independent attention problem (the reference's grid dimensions y and z,
src/fmha-pipeline/fmha_forward.cu:361, and its batch split over streams, :401-417), so ranks take
contiguous ranges of the flattened (batch, head) index and never exchange data.  Because tensors are
[batch][seq][head][d], a range is expressed as sub-calls "batch b, heads h0..h1" that address the
unsharded tensor through a pointer offset and the unsharded strides.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List


@dataclass(frozen=True)
class SubCall:
    batch_begin: int
    batch_count: int
    head_begin: int
    head_count: int


def slice_range(batch: int, heads: int, world: int, rank: int):
    """Contiguous range [lo, hi) of flattened (batch, head) indices for `rank`; sizes differ by at most 1."""
    total = batch * heads
    base, extra = divmod(total, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def sub_calls(batch: int, heads: int, world: int, rank: int) -> List[SubCall]:
    """The fewest rectangular (batch range x head range) calls that cover this rank's slice range."""
    lo, hi = slice_range(batch, heads, world, rank)
    calls: List[SubCall] = []
    i = lo
    while i < hi:
        b, h = divmod(i, heads)
        if h == 0 and hi - i >= heads:                      # whole batches
            nb = (hi - i) // heads
            calls.append(SubCall(b, nb, 0, heads))
            i += nb * heads
        else:                                               # part of one batch entry
            nh = min(heads - h, hi - i)
            calls.append(SubCall(b, 1, h, nh))
            i += nh
    return calls


def element_offset(call: SubCall, seq: int, heads: int, head_dim: int) -> int:
    """Offset (elements) of a sub-call's first element inside the packed [B][S][H][D] tensor."""
    return call.batch_begin * seq * heads * head_dim + call.head_begin * head_dim


def strides(seq: int, heads: int, head_dim: int):
    """(batch, seq, head) element strides of the unsharded tensor, to pass with every sub-call."""
    return (seq * heads * head_dim, heads * head_dim, head_dim)
