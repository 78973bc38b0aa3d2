"""Host-side chunk tables (the information of fla/ops/utils/index.py:155-172, prepare_chunk_indices /
prepare_chunk_offsets, in the form the kernels read)."""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import numpy as np
import torch

CHUNK = 64
_cache: dict = {}


class Tables(tuple):
    """(chunk_meta, seq_meta, (n_chunks, n_seq)) plus ``covered``: False when token rows before the first or after
    the last sequence belong to no sequence (a padded packed buffer).  The kernels never write such rows, so the
    caller zero-fills its intermediates then."""
    covered = True


def build_tables(bounds: Sequence[Tuple[int, int]]):
    """chunk_meta [n_chunks,4] = (sequence, first row, valid rows, index inside the sequence) and
    seq_meta [n_seq,2] = (first chunk, number of chunks), as int32 numpy arrays.  Chunking restarts at
    every sequence start; an empty sequence owns zero chunks."""
    bounds = np.asarray(bounds, dtype=np.int64).reshape(-1, 2)
    lens = bounds[:, 1] - bounds[:, 0]
    if (lens < 0).any():
        raise ValueError('cu_seqlens must be non-decreasing')
    nchunks = (lens + CHUNK - 1) // CHUNK
    first = np.concatenate([[0], np.cumsum(nchunks)[:-1]]) if len(nchunks) else np.zeros(0, np.int64)
    total = int(nchunks.sum())
    seq = np.repeat(np.arange(len(lens)), nchunks)
    local = np.arange(total) - np.repeat(first, nchunks)
    row = bounds[seq, 0] + local * CHUNK
    ln = np.minimum(CHUNK, bounds[seq, 1] - row)
    chunk_meta = np.stack([seq, row, ln, local], 1).astype(np.int32).reshape(-1, 4)
    seq_meta = np.stack([first, nchunks], 1).astype(np.int32).reshape(-1, 2)
    return chunk_meta, seq_meta


def tables_for(B: int, T: int, cu_seqlens: Optional[torch.Tensor], cu_seqlens_cpu: Optional[torch.Tensor],
               device: torch.device) -> Tables:
    """Device tables for a dense [B,T] batch or a packed batch; memoised by shape / by the identity of
    ``cu_seqlens`` (the reference memoises its index tensors the same way, fla/utils/_decorators.py:33-80).
    A packed batch without ``cu_seqlens_cpu`` costs one device-to-host copy on first use."""
    if cu_seqlens is None:
        key = ('dense', B, T, str(device))
        hit = _cache.get(key)
        if hit is not None:
            return hit[0]
        bounds = [(b * T, (b + 1) * T) for b in range(B)]
    else:
        key = ('varlen', id(cu_seqlens), B * T, str(device))
        hit = _cache.get(key)
        if hit is not None and hit[1] is cu_seqlens:
            return hit[0]
        cpu = cu_seqlens_cpu if cu_seqlens_cpu is not None else cu_seqlens.cpu()
        cu = cpu.to(torch.int64).tolist()
        bounds = [(cu[i], cu[i + 1]) for i in range(len(cu) - 1)]
        if cu and (cu[0] < 0 or cu[-1] > B * T):
            raise ValueError(f'cu_seqlens [{cu[0]}, {cu[-1]}] reaches outside the {B * T} token rows')
    cm, sm = build_tables(bounds)
    out = Tables((torch.from_numpy(cm).to(device), torch.from_numpy(sm).to(device), (cm.shape[0], sm.shape[0])))
    out.covered = bool(bounds) and bounds[0][0] == 0 and bounds[-1][1] == B * T
    if len(_cache) > 64:
        _cache.clear()
    _cache[key] = (out, cu_seqlens)
    return out
