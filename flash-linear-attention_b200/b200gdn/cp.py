"""Context parallelism for the chunked gated delta rule: one long packed batch split into equal
contiguous token shards, one per rank (the semantics of fla/ops/cp/context.py and
fla/ops/cp/chunk_delta_h.py).

The state transition of a whole shard is affine, S_end = M S_start + h_ext with
M = prod_c (2^gamma_last,c I - K~_c^T W_c).  Every rank computes (M, h_ext) of the part of its LAST local
sequence with a zero start state, the pairs are exchanged, and each rank folds the pairs of the ranks that
hold the earlier parts of its FIRST local sequence into that sequence's start state.  The backward pass
mirrors this with (M^T, dh_ext) of each rank's first local sequence flowing towards lower ranks.
All ranks therefore scan concurrently; the exchange is K*(K+V) fp32 per head and rank, independent of T.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, List, Optional

import torch
import torch.distributed as dist

from . import _lib
from .index import tables_for


@dataclass
class FLACPContext:
    """Per-rank partition metadata; same fields as fla/ops/cp/context.py:22-57."""
    group: Optional[object] = None
    cu_seqlens: Optional[torch.Tensor] = None
    cu_seqlens_cpu: Optional[torch.Tensor] = None
    is_last_rank: Optional[bool] = None
    pre_num_ranks: Optional[int] = None
    is_first_rank: Optional[bool] = None
    post_num_ranks: Optional[int] = None
    conv1d_kernel_size: Optional[int] = None
    pre_num_conv_tokens: Optional[int] = None

    def copy_for_backward(self) -> 'FLACPContext':
        return FLACPContext(
            group=self.group,
            cu_seqlens=None if self.cu_seqlens is None else self.cu_seqlens.clone(),
            cu_seqlens_cpu=None if self.cu_seqlens_cpu is None else self.cu_seqlens_cpu.clone(),
            is_last_rank=self.is_last_rank, pre_num_ranks=self.pre_num_ranks, is_first_rank=self.is_first_rank,
            post_num_ranks=self.post_num_ranks, conv1d_kernel_size=self.conv1d_kernel_size,
            pre_num_conv_tokens=self.pre_num_conv_tokens)

    @property
    def num_seqs(self) -> int:
        return 0 if self.cu_seqlens is None else len(self.cu_seqlens) - 1

    @property
    def is_cp_enabled(self) -> bool:
        return self.group is not None


def get_cp_cu_seqlens(
    cu_seqlens: torch.Tensor,
    cu_seqlens_cpu: Optional[torch.Tensor] = None,
    world_size: Optional[int] = None,
    rank: Optional[int] = None,
    group=None,
    conv1d_kernel_size: Optional[int] = None,
) -> FLACPContext:
    """Partition a packed batch over ``world_size`` ranks (fla/ops/cp/context.py:60-160).

    Rank r owns tokens [r*P, (r+1)*P), P = total/world_size (must divide).  Returns the rank's local
    ``cu_seqlens`` (int32; global boundaries clipped to the interval) and how many lower / higher ranks
    hold the earlier / later parts of its first / last local sequence.
    """
    if world_size is None:
        assert group is not None
        world_size = dist.get_world_size(group=group)
        rank = dist.get_rank(group=group)
    cpu = cu_seqlens_cpu if cu_seqlens_cpu is not None else cu_seqlens.cpu()
    cu = [int(x) for x in cpu.tolist()]
    total = cu[-1]
    if total < world_size:
        raise ValueError(
            f"`total_tokens` ({total}) must be at least `world_size` ({world_size}) for context parallelism.")
    if total % world_size != 0:
        raise ValueError(
            f"`total_tokens` ({total}) must be divisible by `world_size` ({world_size}) for context parallelism.")
    part = total // world_size
    lo, hi = part * rank, part * (rank + 1)
    # sequences that overlap [lo, hi): end > lo and start < hi
    seqs = [i for i in range(len(cu) - 1) if cu[i + 1] > lo and cu[i] < hi and cu[i + 1] > cu[i]]
    first, last = seqs[0], seqs[-1]
    local: List[int] = []
    for b in cu[first:last + 2]:
        x = min(max(b, lo), hi) - lo
        if not local or local[-1] != x:
            local.append(x)
    first_start, last_end = cu[first], cu[last + 1]
    first_rank_of_first = first_start // part
    last_rank_of_last = (last_end - 1) // part
    local_cpu = torch.tensor(local, dtype=torch.int32)
    return FLACPContext(
        group=group,
        cu_seqlens=local_cpu.to(cu_seqlens.device, non_blocking=True),
        cu_seqlens_cpu=local_cpu,
        is_last_rank=rank == last_rank_of_last,
        pre_num_ranks=rank - first_rank_of_first,
        is_first_rank=rank == first_rank_of_first,
        post_num_ranks=last_rank_of_last - rank,
        conv1d_kernel_size=conv1d_kernel_size,
        pre_num_conv_tokens=max(0, lo - first_start),
    )


def build_cp_context(cu_seqlens: torch.Tensor, group, conv1d_kernel_size: Optional[int] = None,
                     cu_seqlens_cpu: Optional[torch.Tensor] = None) -> FLACPContext:
    """fla/ops/cp/context.py:163-180."""
    return get_cp_cu_seqlens(cu_seqlens, cu_seqlens_cpu=cu_seqlens_cpu, group=group,
                             conv1d_kernel_size=conv1d_kernel_size)


# ------------------------------------------------------------------------------ exchange and fold
def exchange(local: torch.Tensor, group) -> torch.Tensor:
    """All ranks contribute their [HV,K,K+V] fp32 pair, every rank receives [W,HV,K,K+V]
    (fla/ops/cp/comm.py:19-41; ranks with nothing to send contribute zeros, like the reference)."""
    world = dist.get_world_size(group=group)
    out = torch.empty(world * local.numel(), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, local.contiguous().view(-1), group=group)
    return out.view((world,) + tuple(local.shape))


def fold_prefix(gathered: torch.Tensor, rank: int, num: int, K: int, forward: bool,
                apply: Callable[[torch.Tensor, torch.Tensor, torch.Tensor, bool], torch.Tensor]) -> Optional[torch.Tensor]:
    """Compose the affine maps of the ``num`` neighbouring ranks, one step per call of ``apply`` (the host-side
    statement of the fold; on the GPU the whole chain is one launch, ``fold_on_device``).

    forward:  x = 0; for j = rank-num .. rank-1:  x = M_j x + h_j      (start state of the first local sequence)
    backward: x = 0; for j = rank+num .. rank+1:  x = M_j^T x + dh_j   (gradient at the end of the last local
              sequence; the backward pairs already hold M^T, so no transpose is applied)
    ``gathered[j] = [HV, K, K+V]`` with M in columns [0,K) and the state part in [K,K+V).
    ``apply(M, x, b, transpose)`` returns M x + b.
    """
    if num <= 0:
        return None
    order = range(rank - num, rank) if forward else range(rank + num, rank, -1)
    x = None
    for j in order:
        M = gathered[j, :, :, :K].contiguous()
        b = gathered[j, :, :, K:].contiguous()
        x = b if x is None else apply(M, x, b, False)
    return x


def affine_apply(M: torch.Tensor, x: torch.Tensor, b: Optional[torch.Tensor], transpose: bool = False) -> torch.Tensor:
    """One fold step on the device, ``M x + b`` (``M^T x + b``) per head in fp32 (b200gdn_affine_apply)."""
    a = _lib.AffineArgs()
    a.HV, a.K, a.V = M.shape[0], M.shape[1], x.shape[2]
    a.transpose_m = int(transpose)
    out = torch.empty_like(x)
    a.M, a.x, a.b, a.out = M.data_ptr(), x.data_ptr(), _lib.ptr(b), out.data_ptr()
    _lib.call('b200gdn_affine_apply', a, torch.cuda.current_stream(M.device).cuda_stream)
    return out


def fold_on_device(gathered: torch.Tensor, rank: int, num: int, K: int, forward: bool, out: torch.Tensor) -> None:
    """The same fold in one kernel launch (b200gdn_cp_fold), written into ``out [HV,K,V]``."""
    a = _lib.FoldArgs()
    a.HV, a.K, a.V = gathered.shape[1], K, gathered.shape[3] - K
    a.first, a.count, a.step = (rank - num, num, 1) if forward else (rank + num, num, -1)
    a.gathered, a.out = gathered.data_ptr(), out.data_ptr()
    _lib.call('b200gdn_cp_fold', a, torch.cuda.current_stream(gathered.device).cuda_stream)


# Optional phase timing for benchmarks: set PHASE_TIMES = {} and every forward / backward appends CUDA-event pairs
# per phase; collect_phase_times() synchronises and returns the mean milliseconds per phase and call.
PHASE_TIMES = None


class _Phase:
    def __init__(self, name, dev):
        self.name, self.dev = name, dev

    def __enter__(self):
        if PHASE_TIMES is not None:
            self.e0 = torch.cuda.Event(enable_timing=True)
            self.e0.record(torch.cuda.current_stream(self.dev))

    def __exit__(self, *exc):
        if PHASE_TIMES is not None:
            e1 = torch.cuda.Event(enable_timing=True)
            e1.record(torch.cuda.current_stream(self.dev))
            PHASE_TIMES.setdefault(self.name, []).append((self.e0, e1))


def collect_phase_times():
    if not PHASE_TIMES:
        return None
    torch.cuda.synchronize()
    return {n: sum(a.elapsed_time(b) for a, b in ev) / len(ev) for n, ev in PHASE_TIMES.items()}


def _boundary_pair(plan, chain: int, M_pre, h_pre, first_pre: int, K: int, V: int, reverse: bool, stream: int, dev):
    """(M, h) of a whole local sequence from the pairs of its pieces, which sit at consecutive positions
    first_pre .. first_pre + pieces - 1 of the pre-scan's outputs: [HV, K, K + V] for the exchange."""
    from .chunk import prefix_chains
    HV = M_pre.shape[1]
    P = plan.pieces_per_seq[chain]

    class One:   # a one-chain table for b200gdn_cp_prefix
        n_chains = 1
        chains = torch.tensor([[0, P + 1, first_pre]], dtype=torch.int32, device=dev)
    h_tot = torch.empty(1, HV, K, V, dtype=torch.float32, device=dev)
    M_tot = torch.empty(1, HV, K, K, dtype=torch.float32, device=dev)
    prefix_chains(One, M_pre, h_pre, None, None, K, V, reverse, stream, last=h_tot)
    prefix_chains(One, M_pre, None, None, None, K, K, reverse, stream, last=M_tot, identity=True)
    return torch.cat([M_tot[0], h_tot[0]], dim=-1)


class ChunkGatedDeltaRuleCPFunction(torch.autograd.Function):
    """Forward and backward of the op on one rank's shard, with the prefix exchange in between the
    intra-chunk stage and the scan (fla/ops/gated_delta_rule/chunk.py:82-93, 183-200).

    Per direction: ONE pre-scan launch gives the (h_ext, M) pairs it needs (value slices and transition-matrix slices
    side by side in the grid, as the reference's pre-process kernel does, fla/ops/cp/chunk_delta_h.py:41-315), one
    all-gather exchanges the rank-level pairs, ONE launch folds the pairs of the neighbouring ranks, and the regular
    (fused) scan runs from the folded state.  A shard with few sequences and heads is also cut into pieces that are
    scanned concurrently (index.split_plan): the same pre-scan then covers every piece, the rank-level pair is the
    composition of the boundary sequence's pieces, and a prefix chain gives every piece its start state."""

    @staticmethod
    def forward(ctx, q, k, v, g, beta, scale, cp_context):
        from .chunk import carve, new_chunk_args, prefix_chains, _stream
        from .index import split_plan_for
        in_dtypes = (q.dtype, k.dtype, v.dtype, g.dtype, beta.dtype)
        dev = q.device
        group = cp_context.group
        rank = dist.get_rank(group=group)
        with torch.cuda.device(dev):
            qb, kb, vb = (x.to(torch.bfloat16).contiguous() for x in (q, k, v))
            gf, bf = g.float().contiguous(), beta.float().contiguous()
            B, T, H, K = qb.shape
            HV, V = vb.shape[2], vb.shape[3]
            plan = split_plan_for(B, T, cp_context.cu_seqlens, cp_context.cu_seqlens_cpu, dev, HV, V // 64)
            tables = plan.tables if plan is not None else tables_for(B, T, cp_context.cu_seqlens, cp_context.cu_seqlens_cpu, dev)
            chunk_meta, seq_meta, (n_chunks, n_seq) = tables      # n_seq counts pieces under a split plan
            rows = B * T
            bf16, f32 = torch.bfloat16, torch.float32
            zero = not tables.covered
            o = (torch.zeros if zero else torch.empty)(B, T, HV, V, dtype=bf16, device=dev)
            gamma, A, qk, w, u, v_new, h = carve(
                dev, zero, ((n_chunks, HV, 64), f32), ((rows, HV, 64), bf16), ((rows, HV, 64), bf16), ((rows, HV, K), bf16),
                ((rows, HV, V), bf16), ((rows, HV, V), bf16), ((n_chunks, HV, K, V), bf16))
            st = _stream(qb)

            a = new_chunk_args(qb, kb, vb, scale, tables)
            a.g, a.beta = gf.data_ptr(), bf.data_ptr()
            a.gamma, a.A, a.qk, a.w, a.u = gamma.data_ptr(), A.data_ptr(), qk.data_ptr(), w.data_ptr(), u.data_ptr()
            a.stage_mask = _lib.FWD_INTRA
            with _Phase('fwd_intra', dev):
                _lib.call('b200gdn_chunk_fwd', a, st)

            # pairs (M, h) from a zero start state: of every piece but the last of its sequence (split plan), and of the
            # last local sequence('s last piece) when it continues on the next rank
            send = not cp_context.is_last_rank
            with _Phase('fwd_prescan', dev):
                rows_pre = [plan.pre_fwd] if plan is not None else []
                if send:
                    rows_pre.append(seq_meta[n_seq - 1:n_seq])
                n_pre = sum(int(r.shape[0]) for r in rows_pre)
                hm = torch.zeros(HV, K, K + V, dtype=f32, device=dev)
                if n_pre > 0:
                    pre = rows_pre[0] if len(rows_pre) == 1 else torch.cat(rows_pre, 0)
                    h_pre, M_pre = carve(dev, False, ((n_pre, HV, K, V), f32), ((n_pre, HV, K, K), f32))
                    p = new_chunk_args(qb, kb, vb, scale, (chunk_meta, pre, (n_chunks, n_pre)))
                    p.gamma, p.w, p.u, p.ht, p.cp_M = gamma.data_ptr(), w.data_ptr(), u.data_ptr(), h_pre.data_ptr(), M_pre.data_ptr()
                    p.stage_mask = _lib.FWD_SCAN
                    _lib.call('b200gdn_chunk_fwd', p, st)
                    if send and plan is None:
                        hm = torch.cat([M_pre[0], h_pre[0]], dim=-1)
                    elif send:   # the last sequence's pieces are the last entries of the pre-scan
                        last = plan.n_chains - 1
                        hm = _boundary_pair(plan, last, M_pre, h_pre, n_pre - plan.pieces_per_seq[last], K, V, False, st, dev)
            with _Phase('fwd_exchange', dev):
                gathered = exchange(hm, group)
            h0 = None
            with _Phase('fwd_fold', dev):
                n_real = plan.n_chains if plan is not None else n_seq
                if cp_context.pre_num_ranks > 0:
                    h0 = torch.zeros(n_real, HV, K, V, dtype=f32, device=dev)
                    fold_on_device(gathered, rank, cp_context.pre_num_ranks, K, True, h0[0])
                if plan is not None:   # the start state of every piece
                    h0_v = torch.empty(n_seq, HV, K, V, dtype=f32, device=dev)
                    prefix_chains(plan, M_pre, h_pre, h0, h0_v, K, V, False, st)
                    h0 = h0_v

            a.h0 = _lib.ptr(h0)
            a.q = qb.data_ptr()
            a.h, a.v_new, a.o = h.data_ptr(), v_new.data_ptr(), o.data_ptr()
            a.stage_mask = _lib.FWD_SCAN | _lib.FWD_OUT
            with _Phase('fwd_scan_out', dev):
                _lib.call('b200gdn_chunk_fwd', a, st)
        ctx.save_for_backward(qb, kb, vb, bf, gamma, A, qk, w, h, v_new, chunk_meta, seq_meta)
        ctx.meta = (scale, n_chunks, n_seq, in_dtypes, zero)
        ctx.cp_context, ctx.plan = cp_context, plan
        return o.to(q.dtype)

    @staticmethod
    def backward(ctx, do):
        from .chunk import carve, new_chunk_args, prefix_chains, _stream
        qb, kb, vb, bf, gamma, A, qk, w, h, v_new, chunk_meta, seq_meta = ctx.saved_tensors
        scale, n_chunks, n_seq, in_dtypes, zero = ctx.meta
        cp_context, plan = ctx.cp_context, ctx.plan
        group = cp_context.group
        rank = dist.get_rank(group=group)
        dev = qb.device
        with torch.cuda.device(dev):
            B, T, H, K = qb.shape
            HV, V = vb.shape[2], vb.shape[3]
            rows = B * T
            dob = do.to(torch.bfloat16).contiguous()
            bf16, f32 = torch.bfloat16, torch.float32
            grouped = HV > H
            dq, dk, dv, dg, dbeta, dh, dv2, dG, dk_part, dq_acc = carve(
                dev, zero, ((B, T, H, K), bf16), ((B, T, H, K), bf16), ((B, T, HV, V), bf16), ((B, T, HV), f32), ((B, T, HV), f32),
                ((n_chunks, HV, K, V), bf16), ((rows, HV, V), bf16), ((rows, HV), f32),
                ((rows, H, K) if grouped else (0,), f32), ((rows, H, K) if grouped else (0,), f32))
            if not grouped:
                dk_part = dq_acc = None
            st = _stream(qb)
            tables = (chunk_meta, seq_meta, (n_chunks, n_seq))

            # backward pairs (dM, dh) from a zero end gradient: of the first local sequence('s first piece) when it
            # continues from the previous rank, and of every piece but the first of its sequence (split plan).  The
            # pre-scan forms dv_local on chip and stores neither dv2 nor dh.
            send = not cp_context.is_first_rank
            with _Phase('bwd_prescan', dev):
                rows_pre = [seq_meta[0:1]] if send else []
                if plan is not None:
                    rows_pre.append(plan.pre_bwd)
                n_pre = sum(int(r.shape[0]) for r in rows_pre)
                dhm = torch.zeros(HV, K, K + V, dtype=f32, device=dev)
                if n_pre > 0:
                    pre = rows_pre[0] if len(rows_pre) == 1 else torch.cat(rows_pre, 0)
                    dh_pre, dM_pre = carve(dev, False, ((n_pre, HV, K, V), f32), ((n_pre, HV, K, K), f32))
                    p = new_chunk_args(qb, kb, vb, scale, (chunk_meta, pre, (n_chunks, n_pre)))
                    p.gamma, p.w, p.qk, p.d_o = gamma.data_ptr(), w.data_ptr(), qk.data_ptr(), dob.data_ptr()
                    p.dh0, p.cp_dM = dh_pre.data_ptr(), dM_pre.data_ptr()
                    p.stage_mask = _lib.BWD_DVLOCAL | _lib.BWD_SCAN
                    _lib.call('b200gdn_chunk_bwd', p, st)
                    if send and plan is None:
                        dhm = torch.cat([dM_pre[0], dh_pre[0]], dim=-1)
                    elif send:   # the first sequence's pieces are the first entries of the pre-scan
                        dhm = _boundary_pair(plan, 0, dM_pre, dh_pre, 0, K, V, True, st, dev)
            with _Phase('bwd_exchange', dev):
                gathered = exchange(dhm, group)
            dht = None
            with _Phase('bwd_fold', dev):
                n_real = plan.n_chains if plan is not None else n_seq
                if cp_context.post_num_ranks > 0:
                    dht = torch.zeros(n_real, HV, K, V, dtype=f32, device=dev)
                    fold_on_device(gathered, rank, cp_context.post_num_ranks, K, False, dht[n_real - 1])
                if plan is not None:   # the end gradient of every piece
                    dht_v = torch.empty(n_seq, HV, K, V, dtype=f32, device=dev)
                    off = 1 if send else 0   # the plan's own pairs follow the boundary piece in the pre-scan's outputs
                    prefix_chains(plan, dM_pre[off:], dh_pre[off:], dht, dht_v, K, V, True, st)
                    dht = dht_v

            a = new_chunk_args(qb, kb, vb, scale, tables)
            a.beta, a.gamma, a.A, a.qk, a.w, a.h, a.v_new = (x.data_ptr() for x in (bf, gamma, A, qk, w, h, v_new))
            a.d_o, a.dht = dob.data_ptr(), _lib.ptr(dht)
            a.dq, a.dk, a.dv, a.dg, a.dbeta = dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dg.data_ptr(), dbeta.data_ptr()
            a.dh, a.dv2, a.dk_part, a.dG, a.dq_acc = dh.data_ptr(), dv2.data_ptr(), \
                _lib.ptr(dk_part), dG.data_ptr(), _lib.ptr(dq_acc)
            a.stage_mask = 0
            with _Phase('bwd_main', dev):
                _lib.call('b200gdn_chunk_bwd', a, st)
        qd, kd, vd, gd, bd = in_dtypes
        return dq.to(qd), dk.to(kd), dv.to(vd), dg.to(gd), dbeta.to(bd), None, None


def chunk_gated_delta_rule_cp(q, k, v, g, beta, scale, cp_context: FLACPContext) -> torch.Tensor:
    """The op on this rank's shard ``[1, T/W, ...]``; inputs are already pre-processed (l2norm, gate, beta)."""
    if q.shape[0] != 1:
        raise ValueError('context parallelism expects a packed batch with B == 1')
    return ChunkGatedDeltaRuleCPFunction.apply(q, k, v, g, beta, scale, cp_context)
