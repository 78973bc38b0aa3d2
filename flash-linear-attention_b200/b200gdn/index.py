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


# ------------------------------------------------------------------------------------------- sequence split
# The state scans walk a sequence chunk by chunk, one CTA per (sequence, value head, 64 value columns).  With few
# sequences and heads that leaves most of the GPU idle, so long sequences are cut into pieces that are scanned
# concurrently (fla/ops/common/intracard_cp.py:139-180 does this for its forward pass): a pre-scan gives every piece
# its affine map, a prefix chain turns the maps into the start state of every piece, and the regular scan then runs
# over all pieces at once.  Pieces are whole numbers of chunks, so the chunking (and every chunk-local kernel) is
# unchanged.
SM_COUNT = 148
MIN_PIECE_CHUNKS = 16        # a piece shorter than this does not pay for its pre-scan
FORCE_PIECES = None          # tests: cut every sequence into (up to) this many pieces regardless of the heuristic
_split_cache: dict = {}


class SplitPlan:
    """Virtual-sequence tables and the index tensors that tie the pieces of a sequence together."""
    __slots__ = ('tables', 'n_pieces', 'n_pre', 'chains', 'n_chains', 'pre_fwd', 'pre_bwd', 'first_piece', 'last_piece',
                 'pieces_per_seq')


def piece_counts(chunks_per_seq, HV: int, slices: int):
    """How many pieces each sequence is cut into: as many as fill the SMs once, in proportion to the sequence lengths."""
    if FORCE_PIECES is not None:
        return [max(1, min(int(FORCE_PIECES), int(c))) for c in chunks_per_seq]
    slots = SM_COUNT // max(1, slices * HV)          # sequences' worth of scan CTAs that fit the device at once
    n_real = sum(1 for c in chunks_per_seq if c > 0)
    if slots < 2 or n_real >= slots:
        return [1] * len(chunks_per_seq)
    target = max(MIN_PIECE_CHUNKS, -(-sum(chunks_per_seq) // slots))   # chunks per piece
    return [max(1, min(int(c) // MIN_PIECE_CHUNKS, int(round(c / target)))) if c > 0 else 1 for c in chunks_per_seq]


def split_plan(bounds, HV: int, slices: int, device, rows: int) -> Optional[SplitPlan]:
    """None when no sequence is worth cutting; otherwise the plan (device tensors) for these bounds."""
    bounds = [(int(s), int(e)) for s, e in bounds]
    chunks = [(e - s + CHUNK - 1) // CHUNK for s, e in bounds]
    pieces = piece_counts(chunks, HV, slices)
    if max(pieces, default=1) <= 1:
        return None
    vbounds, chains, pre_fwd, pre_bwd, first_piece, last_piece = [], [], [], [], [], []
    n_pre = 0
    for (s, e), c, P in zip(bounds, chunks, pieces):
        first = len(vbounds)
        base, rem = divmod(c, P)
        start = s
        for p in range(P):
            n = base + (1 if p < rem else 0)
            end = min(e, start + n * CHUNK) if p < P - 1 else e
            vbounds.append((start, end))
            start = end
        chains.append((first, P, n_pre))
        pre_fwd += list(range(first, first + P - 1))
        pre_bwd += list(range(first + 1, first + P))
        n_pre += P - 1
        first_piece.append(first)
        last_piece.append(first + P - 1)
    cm, sm = build_tables(vbounds)
    plan = SplitPlan()
    tables = Tables((torch.from_numpy(cm).to(device), torch.from_numpy(sm).to(device), (cm.shape[0], sm.shape[0])))
    tables.covered = bool(bounds) and bounds[0][0] == 0 and bounds[-1][1] == rows
    plan.tables, plan.n_pieces, plan.n_pre, plan.n_chains = tables, len(vbounds), n_pre, len(bounds)
    plan.chains = torch.tensor(chains, dtype=torch.int32).to(device)
    plan.pre_fwd = torch.from_numpy(sm[pre_fwd]).contiguous().to(device)
    plan.pre_bwd = torch.from_numpy(sm[pre_bwd]).contiguous().to(device)
    plan.first_piece = torch.tensor(first_piece, dtype=torch.long).to(device)
    plan.last_piece = torch.tensor(last_piece, dtype=torch.long).to(device)
    plan.pieces_per_seq = pieces
    return plan


def split_plan_for(B: int, T: int, cu_seqlens, cu_seqlens_cpu, device, HV: int, slices: int) -> Optional[SplitPlan]:
    """Memoised like tables_for (by shape, or by the identity of ``cu_seqlens``)."""
    if cu_seqlens is None:
        key = ('dense', B, T, HV, slices, FORCE_PIECES, str(device))
        hit = _split_cache.get(key)
        if hit is not None:
            return hit[0]
        bounds = [(b * T, (b + 1) * T) for b in range(B)]
    else:
        key = ('varlen', id(cu_seqlens), B * T, HV, slices, FORCE_PIECES, str(device))
        hit = _split_cache.get(key)
        if hit is not None and hit[1] is cu_seqlens:
            return hit[0]
        cpu = cu_seqlens_cpu if cu_seqlens_cpu is not None else cu_seqlens.cpu()
        cu = cpu.to(torch.int64).tolist()
        bounds = [(cu[i], cu[i + 1]) for i in range(len(cu) - 1)]
    plan = split_plan(bounds, HV, slices, device, B * T)
    if len(_split_cache) > 64:
        _split_cache.clear()
    _split_cache[key] = (plan, cu_seqlens)
    return plan
