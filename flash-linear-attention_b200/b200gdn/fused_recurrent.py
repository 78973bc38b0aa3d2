"""fused_recurrent_gated_delta_rule with the reference's signature
(fla/ops/gated_delta_rule/fused_recurrent.py:309-475): the decode / short-prefill step, forward only."""
from __future__ import annotations

import warnings
from typing import Optional

import torch

from . import _lib

_DTYPE_CODE = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


class FusedRecurrentFunction(torch.autograd.Function):

    @staticmethod
    def forward(ctx, q, k, v, g, beta, A_log, dt_bias, scale, initial_state, output_final_state, flags, cu_seqlens,
                inplace_state, state_indices=None):
        dev = q.device
        with torch.cuda.device(dev):
            dt = q.dtype if q.dtype in _DTYPE_CODE else torch.float32
            qc, kc, vc = (x.to(dt).contiguous() for x in (q, k, v))
            B, T, H, K = qc.shape
            HV, V = vc.shape[2], vc.shape[3]
            n_seq = B if cu_seqlens is None else cu_seqlens.numel() - 1
            a = _lib.RecurrentArgs()
            a.B, a.T, a.H, a.HV, a.K, a.V, a.n_seq = B, T, H, HV, K, V, n_seq
            a.scale, a.flags, a.qkv_dtype = float(scale), flags, _DTYPE_CODE[dt]
            keep = []

            def f32(t):
                if t is None:
                    return None
                t = t.float().contiguous()
                keep.append(t)
                return t.data_ptr()
            cu32 = None
            if cu_seqlens is not None:
                cu32 = cu_seqlens.to(device=dev, dtype=torch.int32).contiguous()
            a.cu_seqlens = _lib.ptr(cu32)
            a.q, a.k, a.v = qc.data_ptr(), kc.data_ptr(), vc.data_ptr()
            a.g, a.beta, a.A_log, a.dt_bias = f32(g), f32(beta), f32(A_log), f32(dt_bias)
            h0 = None if initial_state is None else initial_state.float().contiguous()
            a.h0 = _lib.ptr(h0)
            o = torch.empty_like(vc)
            ht = None
            idx32 = None
            if state_indices is not None:
                # a pool of state slots addressed per sequence; the update happens in the pool itself
                if h0 is None or h0.data_ptr() != initial_state.data_ptr():
                    raise ValueError("`state_indices` needs `initial_state` to be the fp32 contiguous pool of state slots.")
                if state_indices.numel() != n_seq:
                    raise ValueError(f"`state_indices` must have one entry per sequence ({n_seq}), got {state_indices.numel()}.")
                idx32 = state_indices.to(device=dev, dtype=torch.int32).contiguous()
                a.state_indices = idx32.data_ptr()
                a.n_slots = initial_state.shape[0]
                ht = initial_state
                ctx.mark_dirty(initial_state)   # the pool is updated in place and returned
            elif output_final_state:
                if inplace_state and h0 is not None and h0.data_ptr() == initial_state.data_ptr():
                    ht = initial_state
                    ctx.mark_dirty(initial_state)
                else:
                    shape = (n_seq, HV, V, K) if flags & _lib.REC_STATE_V_FIRST else (n_seq, HV, K, V)
                    ht = torch.empty(shape, dtype=torch.float32, device=dev)
            a.o, a.ht = o.data_ptr(), _lib.ptr(ht)
            _lib.call('b200gdn_recurrent_fwd', a, torch.cuda.current_stream(dev).cuda_stream)
        return o.to(q.dtype), ht

    @staticmethod
    def backward(ctx, do, dht):
        raise NotImplementedError(
            "Backward pass is not implemented for the fused recurrent path (as in the reference, "
            "fla/ops/gated_delta_rule/fused_recurrent.py:299-306); use chunk_gated_delta_rule for training.")


def fused_recurrent_gated_delta_rule(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: Optional[torch.Tensor] = None,
    gk: Optional[torch.Tensor] = None,
    gv: Optional[torch.Tensor] = None,
    beta: Optional[torch.Tensor] = None,
    scale: Optional[float] = None,
    initial_state: Optional[torch.Tensor] = None,
    output_final_state: bool = False,
    use_qk_l2norm_in_kernel: bool = False,
    use_gate_in_kernel: bool = False,
    A_log: Optional[torch.Tensor] = None,
    dt_bias: Optional[torch.Tensor] = None,
    use_beta_sigmoid_in_kernel: bool = False,
    allow_neg_eigval: bool = False,
    state_v_first: bool = False,
    cu_seqlens: Optional[torch.Tensor] = None,
    **kwargs,
):
    r"""Recurrent gated delta rule, same contract as the reference's ``fused_recurrent_gated_delta_rule``.

    q, k ``[B,T,H,K]``; v ``[B,T,HV,V]``; g, beta ``[B,T,HV]``; ``initial_state [N,HV,K,V]``
    (``[N,HV,V,K]`` with ``state_v_first``).  Per-dimension decays ``gk`` / ``gv`` and per-channel beta
    ``[B,T,HV,V]`` belong to other operators of the reference and are rejected.  The extra keyword
    ``inplace_state=True`` writes the final state over ``initial_state`` (fp32, contiguous) instead of
    allocating a new tensor.  The extra keyword ``state_indices [N]`` (no counterpart in the reference) makes
    ``initial_state`` a pool of state slots ``[n_slots,HV,K,V]``: sequence ``n`` reads and updates slot
    ``state_indices[n]`` in place (distinct slots per call), and the pool is returned as the final state.  An index
    outside ``[0, n_slots)`` (a serving engine's ``-1`` padding) marks a padding sequence: its slot is left untouched
    and its output row is meaningless.
    """
    if 'transpose_state_layout' in kwargs:
        if state_v_first:
            raise ValueError("Cannot pass both `state_v_first` and the deprecated `transpose_state_layout`.")
        warnings.warn("`transpose_state_layout` is deprecated and renamed to `state_v_first`.",
                      DeprecationWarning, stacklevel=2)
        state_v_first = kwargs.pop('transpose_state_layout')
    inplace_state = bool(kwargs.pop('inplace_state', False))
    state_indices = kwargs.pop('state_indices', None)
    if gk is not None or gv is not None:
        raise NotImplementedError('per-dimension decays gk / gv are not part of the gated delta rule path')
    if cu_seqlens is not None:
        if q.shape[0] != 1:
            raise ValueError(
                f"The batch size is expected to be 1 rather than {q.shape[0]} when using `cu_seqlens`."
                f"Please flatten variable-length inputs before processing.")
        if state_indices is None and initial_state is not None and initial_state.shape[0] != len(cu_seqlens) - 1:
            raise ValueError(
                f"The number of initial states is expected to be equal to the number of input sequences, "
                f"i.e., {len(cu_seqlens) - 1} rather than {initial_state.shape[0]}.")
    if scale is None:
        scale = k.shape[-1] ** -0.5
    if beta is None:
        beta = torch.ones_like(q[..., 0]).repeat_interleave(v.shape[2] // q.shape[2], dim=-1)
    if beta.ndim != 3:
        raise NotImplementedError('per-channel beta [B,T,HV,V] is not part of the gated delta rule path')
    if use_gate_in_kernel:
        if A_log is None:
            raise ValueError("`A_log` must be provided when `use_gate_in_kernel=True`.")
        if g is None:
            raise ValueError("`g` (raw pre-activation) must be provided when `use_gate_in_kernel=True`.")
    else:
        A_log = None
        dt_bias = None
    if allow_neg_eigval and not use_beta_sigmoid_in_kernel:
        raise ValueError("`allow_neg_eigval=True` requires `use_beta_sigmoid_in_kernel=True`.")
    if not q.is_cuda:
        raise _lib.B200GDNError('fused_recurrent_gated_delta_rule runs on a CUDA device only (no CPU path)')
    flags = 0
    flags |= _lib.REC_L2NORM if use_qk_l2norm_in_kernel else 0
    flags |= _lib.REC_GATE if use_gate_in_kernel else 0
    flags |= _lib.REC_BETA_SIGMOID if use_beta_sigmoid_in_kernel else 0
    flags |= _lib.REC_NEG_EIGVAL if allow_neg_eigval else 0
    flags |= _lib.REC_STATE_V_FIRST if state_v_first else 0
    return FusedRecurrentFunction.apply(q, k, v, g, beta, A_log, dt_bias, scale, initial_state, output_final_state,
                                        flags, cu_seqlens, inplace_state, state_indices)


fused_recurrent_gdn = fused_recurrent_gated_delta_rule
