"""Precomputed document maps for packed calls: `flash_attn_fp8(q, k, v, causal=True, doc_maps=maps)`.

Mirrors the reference's DocMaps (flash_attn/cute/lp_docmaps.py:107, docs/lowprec_usage.md:196-234): a training loop that
packs documents back to back builds the maps once per microbatch -- on the CPU in the data loader's worker (numpy, no
CUDA), or from a CUDA cu_seqlens without a host read -- moves them to the GPU with the batch and passes them to every
layer. Each call then runs on the 128-aligned buffer with the precomputed tables: no index building, no host sync, and
no input copies (the quantisers read Q / K / V / dO in place through the slot tables; O, dQ, dK, dV are scattered back
through the row map). Outputs are bitwise those of the cu_seqlens form with the same padded size.

Shapes are fixed by (max_num_documents, padded_size), so every microbatch's maps look alike to the plan cache and to a
captured CUDA graph (refresh a static DocMaps in place with `copy_`).
"""
from __future__ import annotations

import numpy as np
import torch

__all__ = ["DocMaps", "default_padded_size"]

_FIELDS = ("cu", "start", "len", "row_map", "slot_src", "slot_rows")


def default_padded_size(total: int, max_num_documents: int) -> int:
    """A bound that always holds: every document may waste up to 127 rows of its last 128-row tile."""
    return ((int(total) + 127 * int(max_num_documents) + 255) // 256) * 256


class DocMaps:
    """cu (N + 1,), start / len (N,), row_map (padded_size,), slot_src / slot_rows (padded_size / 128,), all int32, plus
    the host facts total, max_seqlen. Documents beyond the real ones have length zero."""

    def __init__(self, total, max_seqlen, **tensors):
        self.total, self.max_seqlen = int(total), int(max_seqlen)
        for f in _FIELDS:
            setattr(self, f, tensors[f])

    # ------------------------------------------------------------------------------------------------ construction
    @staticmethod
    def from_cu_seqlens(cu_seqlens, max_num_documents=None, max_seqlen=None, padded_size=None, total_q=None) -> "DocMaps":
        """cu_seqlens: (n + 1,) boundaries of the packed documents, cu[0] = 0, cu[-1] = total. A CPU tensor / array builds
        the maps with numpy; a CUDA tensor builds them with device ops and no host read (then total_q and max_seqlen must
        be given: they are host facts)."""
        if isinstance(cu_seqlens, torch.Tensor) and cu_seqlens.is_cuda:
            return DocMaps._from_cuda(cu_seqlens, max_num_documents, max_seqlen, padded_size, total_q)
        cu = np.asarray(cu_seqlens.cpu() if isinstance(cu_seqlens, torch.Tensor) else cu_seqlens, dtype=np.int64)
        if cu.ndim != 1 or cu.size < 2 or cu[0] != 0 or np.any(np.diff(cu) < 0):
            raise ValueError("cu_seqlens must be a non-decreasing 1-d array that starts at 0")
        n, total = cu.size - 1, int(cu[-1])
        if total_q is not None and int(total_q) != total:
            raise ValueError(f"total_q = {total_q} but cu_seqlens ends at {total}")
        N = int(max_num_documents) if max_num_documents is not None else n
        if N < n:
            raise ValueError(f"max_num_documents = {N} is smaller than the {n} documents given")
        lens = np.zeros(N, np.int64)
        lens[:n] = np.diff(cu)
        cu_full = np.concatenate([cu, np.full(N - n, total, np.int64)])
        cap = int(padded_size) if padded_size is not None else default_padded_size(total, N)
        padded = (lens + 127) // 128 * 128
        ends = np.cumsum(padded)
        if cap % 128 or cap < int(ends[-1]):
            raise ValueError(f"padded_size = {cap} must be a multiple of 128 and hold the aligned documents ({int(ends[-1])} rows)")
        start = ends - padded
        row_map = np.full(cap, -1, np.int64)
        for d in range(n):
            row_map[start[d]:start[d] + lens[d]] = cu[d] + np.arange(lens[d])
        first = row_map[::128]
        rows = np.arange(0, cap, 128)
        doc = np.minimum(np.searchsorted(ends, rows, side="right"), N - 1)
        slot_rows = np.where(first >= 0, np.minimum(128, lens[doc] - (rows - start[doc])), 0)
        msl = int(max_seqlen) if max_seqlen is not None else int(lens.max(initial=0))
        if msl < int(lens.max(initial=0)):
            raise ValueError(f"max_seqlen = {msl} is smaller than the longest document ({int(lens.max())})")
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a, dtype=np.int32))          # noqa: E731
        return DocMaps(total, msl, cu=t(cu_full), start=t(start), len=t(lens), row_map=t(row_map), slot_src=t(first),
                       slot_rows=t(slot_rows))

    @staticmethod
    def _from_cuda(cu, max_num_documents, max_seqlen, padded_size, total_q):
        if total_q is None or max_seqlen is None:
            raise ValueError("a CUDA cu_seqlens needs total_q and max_seqlen (host facts: no device value is read)")
        from ._routes import Docs
        n = int(cu.numel()) - 1
        N = int(max_num_documents) if max_num_documents is not None else n
        if N < n:
            raise ValueError(f"max_num_documents = {N} is smaller than the {n} documents given")
        cu = cu.to(torch.int32)
        if N > n:
            cu = torch.cat([cu, cu[-1:].expand(N - n)])
        cap = int(padded_size) if padded_size is not None else default_padded_size(total_q, N)
        d = Docs(cu, cu[1:] - cu[:-1], int(total_q), False, capacity=cap)
        return DocMaps(total_q, max_seqlen, cu=cu.contiguous(), start=d.start, len=d.len, row_map=d.row_map,
                       slot_src=d.slot_src, slot_rows=d.slot_rows)

    # ------------------------------------------------------------------------------------------------ tensor-like
    @property
    def max_num_documents(self) -> int:
        return int(self.len.numel())

    @property
    def padded_size(self) -> int:
        return int(self.row_map.numel())

    @property
    def device(self):
        return self.row_map.device

    def tensors(self):
        return [getattr(self, f) for f in _FIELDS]

    def to(self, device, non_blocking: bool = False) -> "DocMaps":
        return DocMaps(self.total, self.max_seqlen,
                       **{f: getattr(self, f).to(device, non_blocking=non_blocking) for f in _FIELDS})

    def pin_memory(self) -> "DocMaps":
        return DocMaps(self.total, self.max_seqlen, **{f: getattr(self, f).pin_memory() for f in _FIELDS})

    def copy_(self, other: "DocMaps", non_blocking: bool = False) -> "DocMaps":
        """In-place refresh (same shapes): what a captured graph's static maps take before each replay."""
        if other.max_num_documents != self.max_num_documents or other.padded_size != self.padded_size:
            raise ValueError("copy_ needs maps of the same max_num_documents and padded_size")
        for f in _FIELDS:
            getattr(self, f).copy_(getattr(other, f), non_blocking=non_blocking)
        self.total, self.max_seqlen = other.total, other.max_seqlen
        return self
