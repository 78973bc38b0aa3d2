"""chunk_gated_delta_rule with the reference's signature (fla/ops/gated_delta_rule/chunk.py:395-593),
computed by the sm_100a kernels of libb200gdn.so through a torch.autograd.Function.

PyTorch is used for device memory, the current stream and autograd bookkeeping only; every stage of
the reference's pipeline (chunk.py:33-250) runs inside the library.
"""
from __future__ import annotations

import warnings
from typing import Optional

import torch

from . import _lib
from .index import split_plan_for, tables_for

_SUPPORTED_HEAD_DIMS = ((64, 64), (128, 128))


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


_DTYPE_CODE = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


class LayerOptionsFunction(torch.autograd.Function):
    """The three options fla.layers.GatedDeltaNet turns on (fla/layers/gated_deltanet.py:309-325), computed by
    b200gdn_prep_fwd / b200gdn_prep_bwd: q, k L2-normalised to bf16 (fla/modules/l2norm.py:84-144), the gate
    ``-exp(A_log) softplus(g + dt_bias)`` (fla/ops/gated_delta_rule/gate.py:63-158, with dA_log and ddt_bias) and
    ``beta = s sigmoid(beta)`` (fla/ops/common/gate.py:18-50).  Returns what the chunk kernels consume."""

    @staticmethod
    def forward(ctx, q, k, g, beta, A_log, dt_bias, flags):
        dev = q.device
        with torch.cuda.device(dev):
            a = _lib.PrepArgs()
            a.rows, a.H, a.K = q.shape[0] * q.shape[1], q.shape[2], q.shape[3]
            a.HV = g.shape[-1]
            a.flags = flags
            qn, kn, g_out, beta_out = q, k, g, beta
            rstd_q = rstd_k = None
            if flags & _lib.PREP_L2NORM:
                if q.dtype not in _DTYPE_CODE or k.dtype != q.dtype:
                    raise _lib.B200GDNError(f'q/k dtypes {q.dtype}/{k.dtype} are not supported by the L2-norm option')
                q, k = q.contiguous(), k.contiguous()
                a.qk_dtype = _DTYPE_CODE[q.dtype]
                qn, kn = (torch.empty(q.shape, dtype=torch.bfloat16, device=dev) for _ in range(2))
                rstd_q, rstd_k = (torch.empty(q.shape[:-1], dtype=torch.float32, device=dev) for _ in range(2))
                a.q, a.k, a.qn, a.kn = q.data_ptr(), k.data_ptr(), qn.data_ptr(), kn.data_ptr()
                a.rstd_q, a.rstd_k = rstd_q.data_ptr(), rstd_k.data_ptr()
            gb_in = (g.dtype if flags & _lib.PREP_GATE else beta.dtype)
            if (flags & _lib.PREP_GATE) and (flags & _lib.PREP_BETA_SIGMOID) and g.dtype != beta.dtype:
                gb_in = torch.float32
            if gb_in not in _DTYPE_CODE:
                gb_in = torch.float32
            a.gb_dtype = _DTYPE_CODE[gb_in]
            if flags & _lib.PREP_GATE:
                g = g.to(gb_in).contiguous()
                A_log_f = A_log.detach().float().contiguous()
                bias_f = None if dt_bias is None else dt_bias.detach().float().contiguous()
                g_out = torch.empty(g.shape, dtype=torch.float32, device=dev)
                a.g, a.A_log, a.dt_bias, a.g_out = g.data_ptr(), A_log_f.data_ptr(), _lib.ptr(bias_f), g_out.data_ptr()
            else:
                A_log_f = bias_f = None
            if flags & _lib.PREP_BETA_SIGMOID:
                beta = beta.to(gb_in).contiguous()
                beta_out = torch.empty(beta.shape, dtype=torch.float32, device=dev)
                a.beta, a.beta_out = beta.data_ptr(), beta_out.data_ptr()
            _lib.call('b200gdn_prep_fwd', a, _stream(q))
        ctx.flags, ctx.gb_in = flags, gb_in
        ctx.in_dtypes = (g.dtype, beta.dtype)
        ctx.has_bias = dt_bias is not None
        ctx.param_dtypes = (None if A_log is None else A_log.dtype, None if dt_bias is None else dt_bias.dtype)
        ctx.save_for_backward(q, k, rstd_q, rstd_k, g, beta, A_log_f, bias_f)
        return qn, kn, g_out, beta_out

    @staticmethod
    def backward(ctx, dqn, dkn, dg, dbeta):
        q, k, rstd_q, rstd_k, g, beta, A_log_f, bias_f = ctx.saved_tensors
        flags = ctx.flags
        dev = q.device
        dq, dk, dg_raw, dbeta_raw, dA_log, ddt_bias = dqn, dkn, dg, dbeta, None, None
        with torch.cuda.device(dev):
            a = _lib.PrepArgs()
            a.rows, a.H, a.K = q.shape[0] * q.shape[1], q.shape[2], q.shape[3]
            a.HV = g.shape[-1]
            a.flags = 0
            keep = []
            if (flags & _lib.PREP_L2NORM) and dqn is not None and dkn is not None:
                a.flags |= _lib.PREP_L2NORM
                a.qk_dtype = _DTYPE_CODE[q.dtype]
                dqn, dkn = dqn.to(torch.bfloat16).contiguous(), dkn.to(torch.bfloat16).contiguous()
                dq, dk = torch.empty_like(q), torch.empty_like(k)
                a.q, a.k, a.rstd_q, a.rstd_k = q.data_ptr(), k.data_ptr(), rstd_q.data_ptr(), rstd_k.data_ptr()
                a.dqn, a.dkn, a.dq, a.dk = dqn.data_ptr(), dkn.data_ptr(), dq.data_ptr(), dk.data_ptr()
            a.gb_dtype = _DTYPE_CODE[ctx.gb_in]
            if (flags & _lib.PREP_GATE) and dg is not None:
                a.flags |= _lib.PREP_GATE
                dg = dg.float().contiguous()
                dg_raw = torch.empty(g.shape, dtype=ctx.gb_in, device=dev)
                n_part = (a.rows + _lib.PREP_PART_ROWS - 1) // _lib.PREP_PART_ROWS
                partials = torch.empty(n_part, 2, a.HV, dtype=torch.float32, device=dev)
                dA_log = torch.empty(a.HV, dtype=torch.float32, device=dev)
                ddt_bias = torch.empty(a.HV, dtype=torch.float32, device=dev) if ctx.has_bias else None
                a.g, a.A_log, a.dt_bias = g.data_ptr(), A_log_f.data_ptr(), _lib.ptr(bias_f)
                a.dg, a.dg_raw, a.partials = dg.data_ptr(), dg_raw.data_ptr(), partials.data_ptr()
                a.dA_log, a.ddt_bias = dA_log.data_ptr(), _lib.ptr(ddt_bias)
                keep += [partials]
            if (flags & _lib.PREP_BETA_SIGMOID) and dbeta is not None:
                a.flags |= _lib.PREP_BETA_SIGMOID | (flags & _lib.PREP_NEG_EIGVAL)
                dbeta = dbeta.float().contiguous()
                dbeta_raw = torch.empty(beta.shape, dtype=ctx.gb_in, device=dev)
                a.beta, a.dbeta, a.dbeta_raw = beta.data_ptr(), dbeta.data_ptr(), dbeta_raw.data_ptr()
            if a.flags:
                _lib.call('b200gdn_prep_bwd', a, _stream(q))
        g_dtype, beta_dtype = ctx.in_dtypes
        if dg_raw is not None and dg_raw.dtype != g_dtype:
            dg_raw = dg_raw.to(g_dtype)
        if dbeta_raw is not None and dbeta_raw.dtype != beta_dtype:
            dbeta_raw = dbeta_raw.to(beta_dtype)
        if dA_log is not None:
            dA_log = dA_log.to(ctx.param_dtypes[0])
        if ddt_bias is not None:
            ddt_bias = ddt_bias.to(ctx.param_dtypes[1])
        return dq, dk, dg_raw, dbeta_raw, dA_log, ddt_bias, None


def new_chunk_args(q, k, v, scale, tables) -> _lib.ChunkArgs:
    chunk_meta, seq_meta, (n_chunks, n_seq) = tables
    a = _lib.ChunkArgs()
    a.rows = q.shape[0] * q.shape[1]
    a.H, a.HV, a.K, a.V = q.shape[2], v.shape[2], q.shape[3], v.shape[3]
    a.n_seq, a.n_chunks = n_seq, n_chunks
    a.scale = float(scale)
    a.stage_mask = 0
    a.chunk_meta, a.seq_meta = chunk_meta.data_ptr(), seq_meta.data_ptr()
    a.q, a.k, a.v = q.data_ptr(), k.data_ptr(), v.data_ptr()
    return a


def carve(dev, zero, *specs):
    """One device allocation cut into tensors: ``specs`` are (shape, dtype) pairs, every tensor starts on a 256-byte
    boundary.  A forward + backward pass needs about twenty intermediates; one allocation per pass instead of one per
    tensor keeps the host-side cost of a step small.  ``zero`` fills the allocation with zeros (needed when the packed
    buffer has rows that belong to no sequence: the kernels never write them)."""
    offs, total = [], 0
    for shape, dtype in specs:
        n = 1
        for x in shape:
            n *= int(x)
        offs.append(total)
        total += (n * dtype.itemsize + 255) // 256 * 256
    buf = (torch.zeros if zero else torch.empty)(max(total, 256), dtype=torch.uint8, device=dev)
    out = []
    for (shape, dtype), off in zip(specs, offs):
        n = 1
        for x in shape:
            n *= int(x)
        nbytes = n * dtype.itemsize
        out.append(buf[off:off + nbytes].view(dtype).view(*shape))
    return out


class Slab:
    """One device allocation cut into pieces that are only ever handed to the kernels as addresses: ``nbytes`` per piece
    (0 = no such piece, address 0), every piece on a 256-byte boundary.  Unlike ``carve`` it builds no tensor view per
    piece (three torch calls each), which is most of what an allocation-heavy step costs on the host."""
    __slots__ = ('buf', 'offs')

    def __init__(self, dev, zero, nbytes):
        offs, total = [], 0
        for n in nbytes:
            offs.append(total if n > 0 else -1)
            total += (int(n) + 255) // 256 * 256
        self.offs = offs
        self.buf = (torch.zeros if zero else torch.empty)(max(total, 256), dtype=torch.uint8, device=dev)

    @staticmethod
    def addresses(buf, offs):
        base = buf.data_ptr()
        return [base + o if o >= 0 else 0 for o in offs]


def prefix_chains(plan, M, h, x0, out, K, V, reverse: bool, stream: int, last=None, identity: bool = False) -> None:
    """b200gdn_cp_prefix over the chains of a split plan: the start state (reverse: the end gradient) of every piece."""
    a = _lib.PrefixArgs()
    a.HV, a.K, a.V = M.shape[1], K, V
    a.n_chains, a.reverse, a.identity = plan.n_chains, int(reverse), int(identity)
    a.table, a.M, a.h, a.x0 = plan.chains.data_ptr(), M.data_ptr(), _lib.ptr(h), _lib.ptr(x0)
    a.out, a.last = _lib.ptr(out), _lib.ptr(last)
    _lib.call('b200gdn_cp_prefix', a, stream)


class ChunkGatedDeltaRuleFunction(torch.autograd.Function):
    """Autograd node around b200gdn_chunk_fwd / b200gdn_chunk_bwd
    (the role of fla/ops/gated_delta_rule/chunk.py:253-392)."""

    @staticmethod
    def forward(ctx, q, k, v, g, beta, scale, initial_state, output_final_state, cu_seqlens, cu_seqlens_cpu,
                A_log=None, dt_bias=None, options=0, out_dtype=None):
        # options: _lib.PREP_L2NORM (q, k are normalised here, and the backward kernels apply the norm's backward),
        # STATE_V_FIRST (states stored [V,K]) and the PREP_GATE / PREP_BETA_SIGMOID / PREP_NEG_EIGVAL bits; g / beta are then the raw pre-activations
        # and the kernels apply (and differentiate) the activations themselves
        in_dtypes = (q.dtype, k.dtype, v.dtype, g.dtype, beta.dtype)
        out_dtype = out_dtype or q.dtype
        dev = q.device
        with torch.cuda.device(dev):
            vb = v.to(torch.bfloat16).contiguous()
            rstd_q = rstd_k = None
            if options & _lib.PREP_L2NORM:
                # q, k L2-normalised to bf16 in one pass (fla/modules/l2norm.py:84-144); the reciprocal norms go to the
                # backward kernels, which finish dq and dk with the norm's backward themselves
                if q.dtype not in _DTYPE_CODE or k.dtype != q.dtype:
                    raise _lib.B200GDNError(f'q/k dtypes {q.dtype}/{k.dtype} are not supported by the L2-norm option')
                q, k = q.contiguous(), k.contiguous()
                pa = _lib.PrepArgs()
                pa.rows, pa.H, pa.K, pa.HV = q.shape[0] * q.shape[1], q.shape[2], q.shape[3], g.shape[-1]
                pa.flags, pa.qk_dtype = _lib.PREP_L2NORM, _DTYPE_CODE[q.dtype]
                qb, kb = torch.empty(q.shape, dtype=torch.bfloat16, device=dev), torch.empty(q.shape, dtype=torch.bfloat16, device=dev)
                rstd_q = torch.empty(q.shape[:-1], dtype=torch.float32, device=dev)
                rstd_k = torch.empty(q.shape[:-1], dtype=torch.float32, device=dev)
                pa.q, pa.k, pa.qn, pa.kn = q.data_ptr(), k.data_ptr(), qb.data_ptr(), kb.data_ptr()
                pa.rstd_q, pa.rstd_k = rstd_q.data_ptr(), rstd_k.data_ptr()
                _lib.call('b200gdn_prep_fwd', pa, _stream(q))
                options &= ~_lib.PREP_L2NORM
            else:
                qb, kb = q.to(torch.bfloat16).contiguous(), k.to(torch.bfloat16).contiguous()
            gf, bf = g.float().contiguous(), beta.float().contiguous()
            h0 = None if initial_state is None else initial_state.float().contiguous()
            B, T, H, K = qb.shape
            HV, V = vb.shape[2], vb.shape[3]
            # few sequences and heads: long sequences are cut into pieces that are scanned concurrently
            plan = split_plan_for(B, T, cu_seqlens, cu_seqlens_cpu, dev, HV, V // 64)
            # states stored [V,K]: the scans read and write that layout themselves; only the split path, which composes
            # states as [K,V] matrices, transposes at its boundary
            transpose_states = bool(options & _lib.STATE_V_FIRST) and plan is not None
            if transpose_states:
                options &= ~_lib.STATE_V_FIRST
                h0 = None if h0 is None else h0.transpose(-1, -2).contiguous()
            tables = plan.tables if plan is not None else tables_for(B, T, cu_seqlens, cu_seqlens_cpu, dev)
            n_chunks, n_seq = tables[2]          # n_seq counts pieces under a split plan
            n_real = plan.n_chains if plan is not None else n_seq
            rows = B * T
            a = new_chunk_args(qb, kb, vb, scale, tables)
            bf16, f32 = torch.bfloat16, torch.float32
            need_grad = any(ctx.needs_input_grad[:5]) or ctx.needs_input_grad[6]
            zero = not tables.covered
            o = (torch.zeros if zero else torch.empty)(B, T, HV, V, dtype=bf16, device=dev)
            st_shape = (n_seq, HV, V, K) if options & _lib.STATE_V_FIRST else (n_seq, HV, K, V)
            ht = torch.empty(st_shape, dtype=f32, device=dev) if output_final_state else None
            # h and v_new are only read by the backward pass: without one they are not even written
            # gamma, A, qk, w, v_new, h: known to the host only as addresses, kept for the backward pass as one tensor.
            # u is read by the forward scan only: an allocation of its own, returned to the pool when this pass ends
            slab = Slab(dev, zero, (n_chunks * HV * 64 * 4, rows * HV * 64 * 2, rows * HV * 64 * 2, rows * HV * K * 2,
                                    rows * HV * V * 2 if need_grad else 0, n_chunks * HV * K * V * 2 if need_grad else 0))
            p_gamma, p_A, p_qk, p_w, p_vnew, p_h = Slab.addresses(slab.buf, slab.offs)
            u_buf = (torch.zeros if zero else torch.empty)(rows * HV * V, dtype=bf16, device=dev)
            p_u = u_buf.data_ptr()
            a.g, a.beta, a.h0 = gf.data_ptr(), bf.data_ptr(), _lib.ptr(h0)
            A_log_f = A_log.detach().float().contiguous() if (options & _lib.PREP_GATE) else None
            bias_f = dt_bias.detach().float().contiguous() if (options & _lib.PREP_GATE) and dt_bias is not None else None
            a.options, a.A_log, a.dt_bias = options, _lib.ptr(A_log_f), _lib.ptr(bias_f)
            a.o, a.ht = o.data_ptr(), _lib.ptr(ht)
            a.gamma, a.A, a.qk, a.w, a.u, a.h, a.v_new = p_gamma, p_A, p_qk, p_w, p_u, p_h, p_vnew
            st = _stream(qb)
            if plan is None:
                _lib.call('b200gdn_chunk_fwd', a, st)
            else:
                a.stage_mask = _lib.FWD_INTRA
                _lib.call('b200gdn_chunk_fwd', a, st)
                # the affine map (M, h) of every piece but the last of its sequence, from a zero start state
                h_pre, M_pre, h0_v = carve(dev, False, ((plan.n_pre, HV, K, V), f32), ((plan.n_pre, HV, K, K), f32),
                                           ((n_seq, HV, K, V), f32))
                p = new_chunk_args(qb, kb, vb, scale, (tables[0], plan.pre_fwd, (n_chunks, plan.n_pre)))
                p.gamma, p.w, p.u, p.ht, p.cp_M = p_gamma, p_w, p_u, h_pre.data_ptr(), M_pre.data_ptr()
                p.stage_mask = _lib.FWD_SCAN
                _lib.call('b200gdn_chunk_fwd', p, st)
                prefix_chains(plan, M_pre, h_pre, h0, h0_v, K, V, False, st)
                a.h0 = h0_v.data_ptr()
                a.stage_mask = _lib.FWD_SCAN | _lib.FWD_OUT
                _lib.call('b200gdn_chunk_fwd', a, st)
                if ht is not None:
                    ht = ht.index_select(0, plan.last_piece)
        if need_grad:
            ctx.save_for_backward(qb, kb, vb, bf, slab.buf, tables[0], tables[1],
                                  gf if (options & _lib.PREP_GATE) else None, A_log_f, bias_f, rstd_q, rstd_k)
            ctx.slab_offs = slab.offs
        ctx.meta = (scale, n_chunks, n_seq, initial_state is not None, in_dtypes, options,
                    None if A_log is None else A_log.dtype, None if dt_bias is None else dt_bias.dtype, zero)
        ctx.plan = plan
        ctx.transpose_states = transpose_states
        if transpose_states and ht is not None:
            ht = ht.transpose(-1, -2).contiguous()
        return o.to(out_dtype), ht

    @staticmethod
    def backward(ctx, do, dht):
        qb, kb, vb, bf, saved, chunk_meta, seq_meta, gf, A_log_f, bias_f, rstd_q, rstd_k = ctx.saved_tensors
        p_gamma, p_A, p_qk, p_w, p_vnew, p_h = Slab.addresses(saved, ctx.slab_offs)
        scale, n_chunks, n_seq, has_h0, in_dtypes, options, A_dtype, bias_dtype, zero = ctx.meta
        dev = qb.device
        dA_log = ddt_bias = None
        with torch.cuda.device(dev):
            B, T, H, K = qb.shape
            HV, V = vb.shape[2], vb.shape[3]
            rows = B * T
            dob = do.to(torch.bfloat16).contiguous()
            dhtf = None if dht is None else dht.float().contiguous()
            if ctx.transpose_states and dhtf is not None:
                dhtf = dhtf.transpose(-1, -2).contiguous()
            a = new_chunk_args(qb, kb, vb, scale, (chunk_meta, seq_meta, (n_chunks, n_seq)))
            bf16, f32 = torch.bfloat16, torch.float32
            grouped = HV > H
            gate = bool(options & _lib.PREP_GATE)
            # the results are tensors of their own (they outlive the call); the workspace is one allocation known to the
            # host only as addresses
            new = torch.zeros if zero else torch.empty
            dq, dk = new(B, T, H, K, dtype=bf16, device=dev), new(B, T, H, K, dtype=bf16, device=dev)
            dv = new(B, T, HV, V, dtype=bf16, device=dev)
            dg, dbeta = new(B, T, HV, dtype=f32, device=dev), new(B, T, HV, dtype=f32, device=dev)
            st_shape = (n_seq, HV, V, K) if options & _lib.STATE_V_FIRST else (n_seq, HV, K, V)
            dh0 = torch.empty(st_shape, dtype=f32, device=dev) if has_h0 else None
            dA_log = torch.empty(HV, dtype=f32, device=dev) if gate else None
            ddt_bias = torch.empty(HV, dtype=f32, device=dev) if gate and bias_f is not None else None
            ws = Slab(dev, zero, (n_chunks * HV * K * V * 2, rows * HV * V * 2, rows * HV * 4,
                                  rows * H * K * 4 if grouped else 0, rows * H * K * 4 if grouped else 0,
                                  n_chunks * HV * 2 * 4 if gate else 0))
            p_dh, p_dv2, p_dG, p_dk_part, p_dq_acc, p_gate_partials = Slab.addresses(ws.buf, ws.offs)
            a.beta, a.gamma, a.A, a.qk, a.w, a.h, a.v_new = bf.data_ptr(), p_gamma, p_A, p_qk, p_w, p_h, p_vnew
            a.d_o, a.dht = dob.data_ptr(), _lib.ptr(dhtf)
            a.rstd_q, a.rstd_k = _lib.ptr(rstd_q), _lib.ptr(rstd_k)   # given: dq, dk come out w.r.t. the un-normalised q, k
            a.dq, a.dk, a.dv, a.dg, a.dbeta, a.dh0 = dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), dg.data_ptr(), \
                dbeta.data_ptr(), _lib.ptr(dh0)
            a.dh, a.dv2, a.dk_part, a.dG, a.dq_acc = p_dh, p_dv2, p_dk_part, p_dG, p_dq_acc
            a.options = options
            if gate:
                a.g, a.A_log, a.dt_bias = gf.data_ptr(), A_log_f.data_ptr(), _lib.ptr(bias_f)
                a.gate_partials, a.dA_log, a.ddt_bias = p_gate_partials, dA_log.data_ptr(), _lib.ptr(ddt_bias)
            st = _stream(qb)
            plan = ctx.plan
            if plan is None:
                _lib.call('b200gdn_chunk_bwd', a, st)
            else:
                # the backward affine map (dM, dh) of every piece but the first of its sequence, from a zero end gradient;
                # the pre-scan forms dv_local on chip and stores neither dv2 nor dh
                dh_pre, dM_pre, dht_v = carve(dev, False, ((plan.n_pre, HV, K, V), f32), ((plan.n_pre, HV, K, K), f32),
                                              ((n_seq, HV, K, V), f32))
                p = new_chunk_args(qb, kb, vb, scale, (chunk_meta, plan.pre_bwd, (n_chunks, plan.n_pre)))
                p.gamma, p.w, p.qk, p.d_o = p_gamma, p_w, p_qk, dob.data_ptr()
                p.dh0, p.cp_dM = dh_pre.data_ptr(), dM_pre.data_ptr()
                p.stage_mask = _lib.BWD_DVLOCAL | _lib.BWD_SCAN
                _lib.call('b200gdn_chunk_bwd', p, st)
                prefix_chains(plan, dM_pre, dh_pre, dhtf, dht_v, K, V, True, st)
                a.dht = dht_v.data_ptr()
                _lib.call('b200gdn_chunk_bwd', a, st)
                if dh0 is not None:
                    dh0 = dh0.index_select(0, plan.first_piece)
            if ctx.transpose_states and dh0 is not None:
                dh0 = dh0.transpose(-1, -2).contiguous()
        qd, kd, vd, gd, bd = in_dtypes
        if dA_log is not None:
            dA_log = dA_log.to(A_dtype)
        if ddt_bias is not None:
            ddt_bias = ddt_bias.to(bias_dtype)
        return (dq.to(qd), dk.to(kd), dv.to(vd), dg.to(gd), dbeta.to(bd), None, dh0, None, None, None,
                dA_log, ddt_bias, None, None)


def chunk_gated_delta_rule(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    beta: torch.Tensor,
    scale: Optional[float] = None,
    initial_state: Optional[torch.Tensor] = None,
    output_final_state: bool = False,
    use_qk_l2norm_in_kernel: bool = False,
    use_beta_sigmoid_in_kernel: bool = False,
    allow_neg_eigval: bool = False,
    state_v_first: bool = False,
    cu_seqlens: Optional[torch.Tensor] = None,
    cu_seqlens_cpu: Optional[torch.Tensor] = None,
    chunk_indices: Optional[torch.Tensor] = None,
    cp_context=None,
    **kwargs,
):
    r"""Chunked gated delta rule, same contract as the reference's ``chunk_gated_delta_rule``
    (fla/ops/gated_delta_rule/chunk.py:395-593).

    q, k ``[B,T,H,K]``; v ``[B,T,HV,V]`` (``HV % H == 0``: each q/k head serves ``HV/H`` value heads);
    g, beta ``[B,T,HV]``; ``initial_state [N,HV,K,V]`` (``[N,HV,V,K]`` with ``state_v_first``);
    ``cu_seqlens [N+1]`` for packed sequences (then ``B == 1``).  Returns ``(o [B,T,HV,V] in q.dtype,
    final_state fp32 or None)``.  Keyword options ``use_gate_in_kernel``, ``A_log``, ``dt_bias``,
    ``chunk_size`` (16/32/64 accepted; the result does not depend on it and 64 is always used) and the
    deprecated ``transpose_state_layout`` are honoured; ``head_first`` raises as in the reference.
    ``chunk_indices`` is accepted and ignored (the chunk tables are rebuilt from ``cu_seqlens``).

    Precision: the tensor-core kernels compute on bf16 q, k, v (fp32 accumulation, fp32 gates and states).  fp16 /
    fp32 q, k, v are accepted, ROUNDED TO BF16 on entry, and ``o`` and the gradients are cast back to the caller's
    dtypes: the result has bf16 accuracy (the reference's own fp32 test uses the bf16-level tolerance 0.005,
    tests/ops/test_gdn.py:203-278).  Callers that need fp32 arithmetic use the reference's Triton path:
    ``B200GDNBackend``'s verifier declines non-bf16 inputs so that the dispatcher falls through to it.
    A packed buffer may have padding rows before ``cu_seqlens[0]`` or after ``cu_seqlens[-1]``; their outputs and
    gradients are zero, and their q / k / v / do values must be finite.
    """
    out_dtype = q.dtype
    if 'transpose_state_layout' in kwargs:
        if state_v_first:
            raise ValueError("Cannot pass both `state_v_first` and the deprecated `transpose_state_layout`.")
        warnings.warn("`transpose_state_layout` is deprecated and renamed to `state_v_first`.",
                      DeprecationWarning, stacklevel=2)
        state_v_first = kwargs.pop('transpose_state_layout')
    if q.shape[2] != k.shape[2]:
        raise ValueError(
            f"q and k must have the same number of heads, "
            f"but got q.shape[2]={q.shape[2]} and k.shape[2]={k.shape[2]}")
    H, HV = q.shape[2], v.shape[2]
    if HV % H != 0:
        raise ValueError(
            f"For GVA, num_v_heads (HV={HV}) must be evenly divisible by "
            f"num_heads (H={H}), but got HV % H = {HV % H}")
    if 'head_first' in kwargs:
        raise DeprecationWarning("head_first has been removed. Inputs must be in `[B, T, H, ...]` format.")
    chunk_size = kwargs.pop('chunk_size', 64)
    if chunk_size not in (16, 32, 64):
        raise ValueError(f"`chunk_size` must be 16, 32, or 64 for Gated Delta Rule, got {chunk_size}.")
    if cp_context is not None:
        assert initial_state is None, "Initial state is not supported for CP"
        assert output_final_state is False, "Output final state is not supported for CP"
        assert cp_context.cu_seqlens is not None, "cu_seqlens is required for CP"
        cu_seqlens = cp_context.cu_seqlens
        if cp_context.cu_seqlens_cpu is not None:
            cu_seqlens_cpu = cp_context.cu_seqlens_cpu
    if cu_seqlens is not None:
        if q.shape[0] != 1:
            raise ValueError(
                f"The batch size is expected to be 1 rather than {q.shape[0]} when using `cu_seqlens`."
                f"Please flatten variable-length inputs before processing.")
        if initial_state is not None and initial_state.shape[0] != len(cu_seqlens) - 1:
            raise ValueError(
                f"The number of initial states is expected to be equal to the number of input sequences, "
                f"i.e., {len(cu_seqlens) - 1} rather than {initial_state.shape[0]}.")
    use_gate_in_kernel = kwargs.get('use_gate_in_kernel', False)
    A_log = kwargs.get('A_log')
    dt_bias = kwargs.get('dt_bias')
    if use_gate_in_kernel:
        assert A_log is not None, "A_log must be provided when use_gate_in_kernel=True."
    if allow_neg_eigval and not use_beta_sigmoid_in_kernel:
        raise ValueError("`allow_neg_eigval=True` requires `use_beta_sigmoid_in_kernel=True`.")
    if scale is None:
        scale = k.shape[-1] ** -0.5
    if not q.is_cuda:
        raise _lib.B200GDNError('chunk_gated_delta_rule runs on a CUDA device only (no CPU path)')
    if (q.shape[-1], v.shape[-1]) not in _SUPPORTED_HEAD_DIMS:
        raise _lib.B200GDNError(f'head dimensions K={q.shape[-1]}, V={v.shape[-1]} are not built; '
                                f'supported: {_SUPPORTED_HEAD_DIMS}')

    # The three options the layer turns on (fla/layers/gated_deltanet.py:309-325): one pass of the library before the
    # chunk kernels, one after their backward.
    flags = ((_lib.PREP_L2NORM if use_qk_l2norm_in_kernel else 0) | (_lib.PREP_GATE if use_gate_in_kernel else 0)
             | (_lib.PREP_BETA_SIGMOID if use_beta_sigmoid_in_kernel else 0) | (_lib.PREP_NEG_EIGVAL if allow_neg_eigval else 0))
    if use_gate_in_kernel and A_log.numel() != v.shape[2]:
        raise ValueError(f"A_log must have HV={v.shape[2]} elements, got {A_log.numel()}.")
    use_cp = cp_context is not None and getattr(cp_context, 'group', None) is not None
    # The gate and beta activations are fused into the first forward and the last backward kernel; the L2 norm is one
    # pass before the forward kernels and its backward is fused into the kernels that complete dq and dk.  Under
    # context parallelism all three run as passes of their own before / after the chunk kernels.
    fused = 0 if use_cp else flags & (_lib.PREP_L2NORM | _lib.PREP_GATE | _lib.PREP_BETA_SIGMOID | _lib.PREP_NEG_EIGVAL)
    pre = flags & ~fused
    if pre & (_lib.PREP_L2NORM | _lib.PREP_GATE | _lib.PREP_BETA_SIGMOID):
        q, k, g, beta = LayerOptionsFunction.apply(q, k, g, beta, A_log if pre & _lib.PREP_GATE else None,
                                                   dt_bias if pre & _lib.PREP_GATE else None, pre)
    if cp_context is not None and getattr(cp_context, 'group', None) is not None:
        from .cp import chunk_gated_delta_rule_cp
        o = chunk_gated_delta_rule_cp(q, k, v, g, beta, scale, cp_context)   # no states cross this interface
        return o.to(out_dtype), None

    # states stored [V,K] (state_v_first): read and written in that layout by the scans themselves
    o, final_state = ChunkGatedDeltaRuleFunction.apply(
        q, k, v, g, beta, scale, initial_state, output_final_state, cu_seqlens, cu_seqlens_cpu,
        A_log if fused & _lib.PREP_GATE else None, dt_bias if fused & _lib.PREP_GATE else None,
        fused | (_lib.STATE_V_FIRST if state_v_first else 0), out_dtype)
    return o, final_state


chunk_gdn = chunk_gated_delta_rule
