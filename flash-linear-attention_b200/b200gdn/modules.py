"""The two steps either side of the mixer in fla.layers.GatedDeltaNet, with the reference's interfaces:

* ``causal_conv1d`` / ``ShortConvolution`` — the short causal depthwise convolution (+ SiLU) applied to the q, k, v
  projections (fla/modules/conv/causal_conv1d.py:17-160, fla/modules/conv/short_conv.py:24-260), including the
  decode step on a cache and the context-parallel form whose first local sequence starts from the previous rank's
  last W-1 tokens (fla/modules/conv/cp/ops.py:15-260);
* ``rms_norm_gated`` / ``FusedRMSNormGated`` — the gated RMS norm on the mixer's output
  (fla/modules/fused_norm_gate.py:861-884, 1007-1068).

Both run as HBM-streaming kernels of libb200gdn.so (b200gdn_conv_fwd/bwd, b200gdn_norm_gate_fwd/bwd); there is no
fallback path.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist
import torch.nn as nn

from . import _lib
from .index import tables_for

_DTYPE_CODE = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def _stream(t: torch.Tensor) -> int:
    return torch.cuda.current_stream(t.device).cuda_stream


class CausalConv1dFunction(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, weight, bias, residual, initial_state, activation, output_final_state, cu_seqlens, cu_seqlens_cpu,
                inplace_state):
        if x.dtype not in _DTYPE_CODE:
            raise _lib.B200GDNError(f'causal_conv1d: dtype {x.dtype} is not supported')
        dev = x.device
        with torch.cuda.device(dev):
            B, T, D = x.shape
            W = weight.shape[-1]
            xc = x.contiguous()
            tables = tables_for(B, T, cu_seqlens, cu_seqlens_cpu, dev)
            n_tiles, n_seq = tables[2]
            wf = weight.detach().float().contiguous()
            bf = None if bias is None else bias.detach().float().contiguous()
            res = None if residual is None else residual.to(x.dtype).contiguous()
            h0 = None if initial_state is None else initial_state.to(x.dtype).contiguous()
            y = (torch.zeros_like if not tables.covered else torch.empty_like)(xc)
            final = None
            if output_final_state:
                if inplace_state and h0 is not None and h0.data_ptr() == initial_state.data_ptr():
                    final = initial_state      # the decode step updates the cache in place
                else:
                    final = torch.empty(n_seq, D, W, dtype=x.dtype, device=dev)
            a = _lib.ConvArgs()
            a.rows, a.D, a.W, a.n_seq, a.n_tiles = B * T, D, W, n_seq, n_tiles
            a.flags = _lib.CONV_SILU if activation in ('silu', 'swish') else 0
            a.dtype = _DTYPE_CODE[x.dtype]
            a.tile_meta, a.seq_meta = tables[0].data_ptr(), tables[1].data_ptr()
            a.x, a.weight, a.bias, a.residual = xc.data_ptr(), wf.data_ptr(), _lib.ptr(bf), _lib.ptr(res)
            a.initial_state, a.y, a.final_state = _lib.ptr(h0), y.data_ptr(), _lib.ptr(final)
            _lib.call('b200gdn_conv_fwd', a, _stream(xc))
        ctx.save_for_backward(xc, wf, bf, h0, tables[0], tables[1])
        ctx.meta = (a.flags, n_tiles, n_seq, weight.dtype, None if bias is None else bias.dtype, residual is not None,
                    None if residual is None else residual.dtype, None if initial_state is None else initial_state.dtype,
                    tables.covered)
        if final is not None:
            ctx.mark_non_differentiable(final) if final is not initial_state else ctx.mark_dirty(initial_state)
        return y, final

    @staticmethod
    def backward(ctx, dy, dfinal):
        xc, wf, bf, h0, tile_meta, seq_meta = ctx.saved_tensors
        flags, n_tiles, n_seq, w_dtype, b_dtype, has_res, res_dtype, h0_dtype, covered = ctx.meta
        dev = xc.device
        with torch.cuda.device(dev):
            B, T, D = xc.shape
            W = wf.shape[-1]
            dyc = dy.to(xc.dtype).contiguous()
            dx = (torch.zeros_like if not covered else torch.empty_like)(xc)
            dw = torch.empty(D, W, dtype=torch.float32, device=dev)
            db = torch.empty(D, dtype=torch.float32, device=dev) if bf is not None else None
            dh0 = torch.empty(n_seq, D, W, dtype=xc.dtype, device=dev) if h0 is not None else None
            partials = torch.empty(2 * n_tiles, D, W + 1, dtype=torch.float32, device=dev)
            a = _lib.ConvArgs()
            a.rows, a.D, a.W, a.n_seq, a.n_tiles = B * T, D, W, n_seq, n_tiles
            a.flags, a.dtype = flags, _DTYPE_CODE[xc.dtype]
            a.tile_meta, a.seq_meta = tile_meta.data_ptr(), seq_meta.data_ptr()
            a.x, a.weight, a.bias, a.initial_state = xc.data_ptr(), wf.data_ptr(), _lib.ptr(bf), _lib.ptr(h0)
            a.dy, a.dx, a.dweight, a.dbias = dyc.data_ptr(), dx.data_ptr(), dw.data_ptr(), _lib.ptr(db)
            a.dinitial_state, a.partials = _lib.ptr(dh0), partials.data_ptr()
            _lib.call('b200gdn_conv_bwd', a, _stream(xc))
        return (dx, dw.to(w_dtype), None if db is None else db.to(b_dtype), dy.to(res_dtype) if has_res else None,
                None if dh0 is None else dh0.to(h0_dtype), None, None, None, None, None)


class _HaloExchange(torch.autograd.Function):
    """The last W-1 token rows of every rank go to the next rank (forward); the gradient of what a rank received goes
    back to the previous rank (backward).  One small all-gather per direction, as the reference's
    conv_cp_send_recv_fwd / _bwd (fla/ops/cp/comm.py:64-137)."""

    @staticmethod
    def forward(ctx, tails, group):
        world, rank = dist.get_world_size(group=group), dist.get_rank(group=group)
        out = torch.empty((world,) + tuple(tails.shape), dtype=tails.dtype, device=tails.device)
        dist.all_gather_into_tensor(out.view(-1), tails.contiguous().view(-1), group=group)
        ctx.group, ctx.world, ctx.rank = group, world, rank
        return out[rank - 1].clone() if rank > 0 else torch.zeros_like(tails)

    @staticmethod
    def backward(ctx, dheads):
        out = torch.empty((ctx.world,) + tuple(dheads.shape), dtype=dheads.dtype, device=dheads.device)
        src = dheads.contiguous() if ctx.rank > 0 else torch.zeros_like(dheads)
        dist.all_gather_into_tensor(out.view(-1), src.view(-1), group=ctx.group)
        return (out[ctx.rank + 1].clone() if ctx.rank + 1 < ctx.world else torch.zeros_like(dheads)), None


def causal_conv1d_cp(x, weight, bias=None, activation=None, cp_context=None, **kwargs):
    """Context-parallel causal convolution (fla/modules/conv/cp/ops.py:218-260): the rank's first local sequence starts
    from the previous rank's last W-1 tokens when it continues a sequence from there.  The exchange is differentiable,
    so the gradient of those borrowed tokens flows back to the rank that owns them."""
    if cp_context is None:
        raise ValueError("cp_context must be provided for causal_conv1d_cp")
    assert cp_context.conv1d_kernel_size is not None, "conv1d_kernel_size must be provided for causal_conv1d_cp"
    assert cp_context.cu_seqlens is not None, "cu_seqlens must be provided for causal_conv1d_cp"
    assert x.dim() == 3 and x.shape[0] == 1, f"CP requires [1, T, D], got {tuple(x.shape)}"
    W, D = weight.shape[-1], weight.shape[0]
    heads = _HaloExchange.apply(x[0, -(W - 1):], cp_context.group)          # [W-1, D]: the previous rank's tail
    n_seq = len(cp_context.cu_seqlens) - 1
    valid = 0 if cp_context.is_first_rank else min(W - 1, int(cp_context.pre_num_conv_tokens))
    first = torch.zeros(D, W, dtype=x.dtype, device=x.device)
    if valid > 0:
        first = torch.cat([first[:, :W - valid], heads[-valid:].transpose(0, 1)], dim=1)
    initial_state = torch.cat([first[None], torch.zeros(n_seq - 1, D, W, dtype=x.dtype, device=x.device)], dim=0)
    # every rank's graph keeps the exchange (a zero-valued dependence where nothing was borrowed), so that all ranks
    # enter the collective of its backward pass
    initial_state = initial_state + (heads * 0).sum()
    y, _ = CausalConv1dFunction.apply(x, weight, bias, None, initial_state, activation, False, cp_context.cu_seqlens,
                                      cp_context.cu_seqlens_cpu, False)
    return y


def causal_conv1d(
    x: torch.Tensor,
    weight: Optional[torch.Tensor] = None,
    bias: Optional[torch.Tensor] = None,
    residual: Optional[torch.Tensor] = None,
    initial_state: Optional[torch.Tensor] = None,
    output_final_state: Optional[bool] = False,
    activation: Optional[str] = None,
    backend: Optional[str] = 'triton',
    cu_seqlens: Optional[torch.Tensor] = None,
    cu_seqlens_cpu: Optional[torch.Tensor] = None,
    chunk_indices: Optional[torch.Tensor] = None,
    cp_context=None,
    **kwargs,
) -> Tuple[torch.Tensor, Optional[torch.Tensor]]:
    """Causal depthwise convolution with the reference's signature (fla/modules/conv/causal_conv1d.py:17-160).

    x ``[B,T,D]`` (``B == 1`` with ``cu_seqlens``), weight ``[D,W]`` (W in 2..4), bias ``[D]``, residual ``[B,T,D]``,
    initial_state ``[N,D,W]`` (its last W-1 entries are the inputs before each sequence).  Returns ``(y, final_state)``;
    ``final_state [N,D,W]`` holds the last W inputs.  ``backend`` and ``chunk_indices`` are accepted and ignored.
    The extra keyword ``inplace_state=True`` writes the final state over ``initial_state``.
    """
    if activation not in (None, 'silu', 'swish'):
        raise ValueError(f"Activation `{activation}` not supported yet.")
    if not x.is_cuda:
        raise _lib.B200GDNError('causal_conv1d runs on a CUDA device only (no CPU path)')
    if cp_context is not None:
        assert initial_state is None, "Initial state is not supported for CP"
        assert output_final_state is False, "Output final state is not supported for CP"
        assert residual is None, "Residual is not supported for CP"
        return causal_conv1d_cp(x, weight, bias, activation, cp_context), None
    if cu_seqlens is not None and x.shape[0] != 1:
        raise ValueError(f"The batch size is expected to be 1 rather than {x.shape[0]} when using `cu_seqlens`.")
    y, final = CausalConv1dFunction.apply(x, weight, bias, residual, initial_state, activation, bool(output_final_state),
                                          cu_seqlens, cu_seqlens_cpu, bool(kwargs.get('inplace_state', False)))
    return y, final


class ShortConvolution(nn.Conv1d):
    """Depthwise causal convolution layer with the parameters and the forward contract of the reference's
    ``ShortConvolution`` (fla/modules/conv/short_conv.py:24-260): weight ``[D,1,W]``, optional bias, SiLU by default;
    ``forward(x, residual, mask, cache, output_final_state, cu_seqlens)`` returns ``(y, cache)``.  With one token per
    sequence and a cache the cache is updated in place (the decode step)."""

    def __init__(self, hidden_size: int, kernel_size: int, bias: bool = False, activation: Optional[str] = 'silu',
                 backend: Optional[str] = 'b200', device=None, dtype=None, **kwargs):
        super().__init__(in_channels=hidden_size, out_channels=hidden_size, kernel_size=kernel_size, groups=hidden_size,
                         bias=bias, padding=kernel_size - 1, device=device, dtype=dtype)
        self.hidden_size = hidden_size
        if activation is not None:
            assert activation in ['silu', 'swish'], f"Activation `{activation}` not supported yet."
        self.activation = activation
        self.backend = backend

    def forward(self, x, residual=None, mask=None, cache=None, output_final_state=False, cu_seqlens=None,
                chunk_indices=None, **kwargs):
        B, T = x.shape[0], x.shape[1]
        N = B if cu_seqlens is None else len(cu_seqlens) - 1
        if mask is not None:
            if cu_seqlens is not None:
                raise ValueError("`mask` and `cu_seqlens` cannot be provided at the same time")
            x = x.mul_(mask.unsqueeze(-1))
        weight = self.weight.squeeze(1)
        if B * T == N:   # decoding: one token per sequence, the cache (created when absent) is updated in place
            if cache is None:
                cache = x.new_zeros(N, self.hidden_size, self.kernel_size[0])
            y, cache = causal_conv1d(x, weight, self.bias, residual, cache, True, self.activation, cu_seqlens=cu_seqlens,
                                     inplace_state=True)
            return y, (cache if output_final_state else None)
        return causal_conv1d(x, weight, self.bias, residual, cache, output_final_state, self.activation,
                             cu_seqlens=cu_seqlens, **kwargs)

    @property
    def state_size(self) -> int:
        return self.hidden_size * self.kernel_size[0]


class RMSNormGatedFunction(torch.autograd.Function):

    @staticmethod
    def forward(ctx, x, g, weight, bias, activation, eps):
        if x.dtype not in _DTYPE_CODE:
            raise _lib.B200GDNError(f'rms_norm_gated: dtype {x.dtype} is not supported')
        dev = x.device
        with torch.cuda.device(dev):
            D = x.shape[-1]
            xc, gc = x.contiguous(), g.to(x.dtype).contiguous()
            rows = xc.numel() // D
            wf = None if weight is None else weight.detach().float().contiguous()
            bf = None if bias is None else bias.detach().float().contiguous()
            y = torch.empty_like(xc)
            rstd = torch.empty(rows, dtype=torch.float32, device=dev)
            a = _lib.NormGateArgs()
            a.D, a.rows, a.eps = D, rows, float(eps)
            a.flags = _lib.NORM_GATE_SIGMOID if activation == 'sigmoid' else 0
            a.dtype = _DTYPE_CODE[x.dtype]
            a.x, a.g, a.weight, a.bias, a.y, a.rstd = xc.data_ptr(), gc.data_ptr(), _lib.ptr(wf), _lib.ptr(bf), y.data_ptr(), \
                rstd.data_ptr()
            _lib.call('b200gdn_norm_gate_fwd', a, _stream(xc))
        ctx.save_for_backward(xc, gc, wf, bf, rstd)
        ctx.meta = (a.flags, float(eps), g.dtype, None if weight is None else weight.dtype, None if bias is None else bias.dtype)
        return y

    @staticmethod
    def backward(ctx, dy):
        xc, gc, wf, bf, rstd = ctx.saved_tensors
        flags, eps, g_dtype, w_dtype, b_dtype = ctx.meta
        dev = xc.device
        with torch.cuda.device(dev):
            D = xc.shape[-1]
            rows = xc.numel() // D
            dyc = dy.to(xc.dtype).contiguous()
            dx, dg = torch.empty_like(xc), torch.empty_like(gc)
            n_ctas = _lib.load().b200gdn_norm_gate_ctas(rows)
            partials = torch.empty(n_ctas, 2, D, dtype=torch.float32, device=dev)
            dw = torch.empty(D, dtype=torch.float32, device=dev) if wf is not None else None
            db = torch.empty(D, dtype=torch.float32, device=dev) if bf is not None else None
            a = _lib.NormGateArgs()
            a.D, a.rows, a.eps, a.flags, a.dtype = D, rows, eps, flags, _DTYPE_CODE[xc.dtype]
            a.x, a.g, a.weight, a.bias, a.rstd = xc.data_ptr(), gc.data_ptr(), _lib.ptr(wf), _lib.ptr(bf), rstd.data_ptr()
            a.dy, a.dx, a.dg, a.dweight, a.dbias, a.partials = dyc.data_ptr(), dx.data_ptr(), dg.data_ptr(), _lib.ptr(dw), \
                _lib.ptr(db), partials.data_ptr()
            _lib.call('b200gdn_norm_gate_bwd', a, _stream(xc))
        return (dx, dg.to(g_dtype), None if dw is None else dw.to(w_dtype), None if db is None else db.to(b_dtype), None, None)


def rms_norm_gated(x, g, weight, bias=None, activation: str = 'swish', residual=None, prenorm: bool = False,
                   residual_in_fp32: bool = False, eps: float = 1e-6):
    """``(x rstd weight + bias) act(g)`` over the last dimension, the reference's ``rms_norm_gated``
    (fla/modules/fused_norm_gate.py:861-884); ``act`` is swish / silu (default) or sigmoid.  The residual / prenorm
    form is not part of the Gated DeltaNet layer and is declined."""
    if activation not in ('swish', 'silu', 'sigmoid'):
        raise ValueError(f"Unsupported activation: {activation}")
    if residual is not None or prenorm:
        raise NotImplementedError('rms_norm_gated: the residual / prenorm form is not built (the layer does not use it)')
    if not x.is_cuda:
        raise _lib.B200GDNError('rms_norm_gated runs on a CUDA device only (no CPU path)')
    return RMSNormGatedFunction.apply(x, g, weight, bias, activation, eps)


class FusedRMSNormGated(nn.Module):
    """Same parameters and forward contract as the reference's ``FusedRMSNormGated``
    (fla/modules/fused_norm_gate.py:1007-1068)."""

    def __init__(self, hidden_size: int, elementwise_affine: bool = True, eps: float = 1e-5, activation: str = 'swish',
                 device=None, dtype=None):
        super().__init__()
        self.hidden_size, self.elementwise_affine, self.eps, self.activation = hidden_size, elementwise_affine, eps, activation
        if activation not in ('swish', 'silu', 'sigmoid'):
            raise ValueError(f"Unsupported activation: {activation}")
        if elementwise_affine:
            self.weight = nn.Parameter(torch.ones(hidden_size, device=device, dtype=dtype))
        else:
            self.register_parameter('weight', None)
        self.register_parameter('bias', None)

    def forward(self, x, g, residual=None, prenorm=False, residual_in_fp32=False):
        return rms_norm_gated(x, g, self.weight, self.bias, self.activation, residual=residual, eps=self.eps,
                              prenorm=prenorm, residual_in_fp32=residual_in_fp32)
