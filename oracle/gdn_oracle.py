"""CPU oracle for the chunked gated delta rule (GDN token mixer).

TEST INFRASTRUCTURE ONLY.  Nothing in the product package imports this module;
it is the checker used by the tests, by the smoke check and by the benchmark's
CPU-baseline leg.  It is a restatement, in plain torch on the CPU, of the
algorithm of fla-org/flash-linear-attention (version 0.5.2):

* ``naive_recurrent``            follows fla/ops/gated_delta_rule/naive.py:13-64
  (token-by-token recurrence; extended here to grouped value heads and packed
  variable-length input exactly as the reference tests do it, i.e. q/k heads
  repeated over their value-head group, tests/ops/test_gdn.py:108-200, 712-803).
* ``recurrent_step_options``     follows the in-kernel options of
  fla/ops/gated_delta_rule/fused_recurrent.py:114-174 (l2norm, gate, sigmoid).
* the ``stage_*`` functions      follow the reference's stage decomposition
  (fla/ops/gated_delta_rule/chunk.py:33-250) with the per-stage math of
  fla/ops/utils/cumsum.py:33-68, gated_delta_rule/chunk_fwd.py:40-328,
  gated_delta_rule/wy_fast.py:43-251, common/chunk_delta_h.py:58-683 and
  common/chunk_o.py:56-342, written on 64-row zero-padded tiles of a
  flattened ``[rows, heads, dim]`` layout (the layout the CUDA kernels use).
* ``err_ratio`` / ``assert_close`` follow fla/utils/_testing.py:18-41.

Parity pin: tests/golden/make_golden.py imports the reference itself and stores
its outputs (naive recurrence, naive chunk form, and autograd gradients) as
fixtures; tests/test_oracle.py checks every function here against them.

All gates are handled like the reference does: gamma = chunk-local cumsum(g) *
log2(e), and every exponential is exp2 of a gamma difference.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

BT = 64
RCP_LN2 = 1.4426950216  # fla/ops/utils/constant.py:10


# --------------------------------------------------------------------------- metric
def err_ratio(ref: torch.Tensor, out: torch.Tensor) -> float:
    """RMSE(ref - out) / RMSE(ref)  (fla/utils/_testing.py:22-25)."""
    ref = ref.detach().double().flatten()
    out = out.detach().double().flatten()
    err = (ref - out).square().mean().sqrt().item()
    base = ref.square().mean().sqrt().item()
    return err / (base + 1e-8)


def assert_close(name: str, ref: torch.Tensor, out: torch.Tensor, ratio: float, atol: float = 1e-6) -> float:
    """Pass when max-abs <= atol, else require err_ratio < ratio (fla/utils/_testing.py:28-41)."""
    ref = ref.detach()
    out = out.detach()
    assert ref.shape == out.shape, f"{name}: shape {tuple(ref.shape)} vs {tuple(out.shape)}"
    abs_err = (ref.double() - out.double()).abs().max().item() if ref.numel() else 0.0
    if abs_err <= atol:
        return 0.0
    assert not torch.isnan(ref).any(), f"{name}: NaN in reference"
    assert not torch.isnan(out).any(), f"{name}: NaN in output"
    r = err_ratio(ref, out)
    assert r < ratio, f"{name}: max-abs {abs_err:.6g} err-ratio {r:.6g} >= {ratio}"
    return r


# --------------------------------------------------------------------------- helpers
def seq_bounds(B: int, T: int, cu_seqlens: Optional[Sequence[int]]) -> List[Tuple[int, int]]:
    """[(bos, eos)] in flattened-row coordinates; dense input is B sequences of T rows."""
    if cu_seqlens is None:
        return [(b * T, (b + 1) * T) for b in range(B)]
    cu = [int(x) for x in cu_seqlens]
    return [(cu[i], cu[i + 1]) for i in range(len(cu) - 1)]


def chunk_table(bounds: Sequence[Tuple[int, int]]) -> List[Tuple[int, int, int]]:
    """[(sequence id, first row, valid rows)] for every 64-row chunk; chunking restarts at
    each sequence start (fla/ops/utils/index.py:155-172)."""
    out = []
    for n, (bos, eos) in enumerate(bounds):
        s = bos
        while s < eos:
            out.append((n, s, min(BT, eos - s)))
            s += BT
    return out


def _tile(x: torch.Tensor, start: int, length: int) -> torch.Tensor:
    """Rows [start, start+length) of x, zero-padded to 64 rows."""
    t = x[start:start + length]
    if length < BT:
        pad = torch.zeros((BT - length,) + tuple(t.shape[1:]), dtype=t.dtype)
        t = torch.cat([t, pad], 0)
    return t


def _rd(x: torch.Tensor, emulate: bool) -> torch.Tensor:
    """Optional bf16 rounding point (the reference stores A, w, u, v_new, h, dh in bf16)."""
    return x.to(torch.bfloat16).to(x.dtype) if emulate else x


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """x * rsqrt(sum(x^2) + eps)  (fla/modules/l2norm.py:84-109)."""
    return x * torch.rsqrt(x.square().sum(-1, keepdim=True) + eps)


def gdn_gate(g: torch.Tensor, A_log: torch.Tensor, dt_bias: Optional[torch.Tensor]) -> torch.Tensor:
    """-exp(A_log) * softplus(g + dt_bias)  (fla/ops/gated_delta_rule/gate.py:21-46)."""
    g = g.float() if g.dtype not in (torch.float32, torch.float64) else g
    if dt_bias is not None:
        g = g + dt_bias.to(g.dtype)
    return -A_log.to(g.dtype).exp() * F.softplus(g)


# --------------------------------------------------------------------------- ground truth
def naive_recurrent(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, beta: torch.Tensor,
    scale: Optional[float] = None, initial_state: Optional[torch.Tensor] = None,
    output_final_state: bool = False, cu_seqlens: Optional[Sequence[int]] = None,
    dtype: torch.dtype = torch.float32,
):
    """Token-by-token gated delta rule (fla/ops/gated_delta_rule/naive.py:13-64).

    q, k ``[B,T,H,K]``; v ``[B,T,HV,V]``; g, beta ``[B,T,HV]``; initial_state ``[N,HV,K,V]``.
    Per token:  S *= exp(g);  r = beta * (v - S^T k);  S += k r^T;  o = S^T (scale * q).
    Differentiable, so torch autograd over it is the gradient oracle.
    """
    B, T, H, K = q.shape
    HV, V = v.shape[2], v.shape[3]
    G = HV // H
    if scale is None:
        scale = K ** -0.5
    qf = q.to(dtype).repeat_interleave(G, dim=2).reshape(B * T, HV, K)
    kf = k.to(dtype).repeat_interleave(G, dim=2).reshape(B * T, HV, K)
    vf = v.to(dtype).reshape(B * T, HV, V)
    gf = g.to(dtype).reshape(B * T, HV)
    bf = beta.to(dtype).reshape(B * T, HV)
    bounds = seq_bounds(B, T, cu_seqlens)
    outs = []
    finals = []
    for n, (bos, eos) in enumerate(bounds):
        S = torch.zeros(HV, K, V, dtype=dtype) if initial_state is None else initial_state[n].to(dtype)
        for t in range(bos, eos):
            S = S * gf[t].exp()[:, None, None]
            r = (vf[t] - torch.einsum('hkv,hk->hv', S, kf[t])) * bf[t][:, None]
            S = S + kf[t][:, :, None] * r[:, None, :]
            outs.append(torch.einsum('hkv,hk->hv', S, qf[t] * scale))
        finals.append(S)
    o = torch.stack(outs, 0).reshape(B, T, HV, V) if outs else torch.zeros(B, T, HV, V, dtype=dtype)
    ht = torch.stack(finals, 0) if output_final_state else None
    return o, ht


def naive_with_grads(q, k, v, g, beta, scale, h0, do, dht, cu_seqlens=None, dtype=torch.float64):
    """Outputs and all input gradients of loss = <o,do> + <ht,dht> by autograd over the
    recurrence (how tests/ops/test_gdn.py:108-200 builds its gradient reference)."""
    leaves = [x.detach().to(dtype).clone().requires_grad_(True) for x in (q, k, v, g, beta)]
    h0_ = None if h0 is None else h0.detach().to(dtype).clone().requires_grad_(True)
    o, ht = naive_recurrent(*leaves, scale=scale, initial_state=h0_, output_final_state=True,
                            cu_seqlens=cu_seqlens, dtype=dtype)
    loss = (o * do.to(dtype)).sum()
    if dht is not None:
        loss = loss + (ht * dht.to(dtype)).sum()
    loss.backward()
    grads = dict(dq=leaves[0].grad, dk=leaves[1].grad, dv=leaves[2].grad, dg=leaves[3].grad,
                 dbeta=leaves[4].grad, dh0=None if h0_ is None else h0_.grad)
    return o.detach(), ht.detach(), grads


def recurrent_step_options(
    q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
    use_qk_l2norm_in_kernel=False, use_gate_in_kernel=False, A_log=None, dt_bias=None,
    use_beta_sigmoid_in_kernel=False, allow_neg_eigval=False, state_v_first=False,
    cu_seqlens=None, dtype=torch.float32,
):
    """The decode-path recurrence with the in-kernel options of
    fla/ops/gated_delta_rule/fused_recurrent.py:114-174 applied first."""
    q, k = q.to(dtype), k.to(dtype)
    if use_qk_l2norm_in_kernel:
        q, k = l2norm(q), l2norm(k)
    g = g.to(dtype)
    if use_gate_in_kernel:
        g = gdn_gate(g, A_log, dt_bias)
    beta = beta.to(dtype)
    if use_beta_sigmoid_in_kernel:
        beta = torch.sigmoid(beta) * (2.0 if allow_neg_eigval else 1.0)
    h0 = initial_state
    if h0 is not None and state_v_first:
        h0 = h0.transpose(-1, -2)
    o, ht = naive_recurrent(q, k, v, g, beta, scale, h0, output_final_state, cu_seqlens, dtype)
    if ht is not None and state_v_first:
        ht = ht.transpose(-1, -2).contiguous()
    return o, ht


# --------------------------------------------------------------------------- forward stages
def stage_intra(k, v, g, beta, bounds, emulate_bf16=False):
    """Chunk-local cumsum, A = (I + strict_tril(beta_i <k_i,k_j> 2^(gam_i-gam_j)))^-1,
    U = A (beta*V), W = A (beta*2^gam*K).

    fla/ops/utils/cumsum.py:33-68, gated_delta_rule/chunk_fwd.py:40-328, wy_fast.py:43-106.
    k ``[R,H,K]``, v ``[R,HV,V]``, g/beta ``[R,HV]`` -> gamma ``[R,HV]``, A ``[R,HV,64]``,
    w ``[R,HV,K]``, u ``[R,HV,V]``.
    """
    R, H, K = k.shape
    HV, V = v.shape[1], v.shape[2]
    G = HV // H
    dt = k.dtype
    gam = torch.zeros(R, HV, dtype=dt)
    A_out = torch.zeros(R, HV, BT, dtype=dt)
    w = torch.zeros(R, HV, K, dtype=dt)
    u = torch.zeros(R, HV, V, dtype=dt)
    eye = torch.eye(BT, dtype=dt)
    strict = torch.tril(torch.ones(BT, BT, dtype=torch.bool), -1)
    for (_, s, L) in chunk_table(bounds):
        kc = _tile(k, s, L).repeat_interleave(G, dim=1).transpose(0, 1)   # [HV,64,K]
        vc = _tile(v, s, L).transpose(0, 1)                                # [HV,64,V]
        gc = _tile(g, s, L).transpose(0, 1)                                # [HV,64]
        bc = _tile(beta, s, L).transpose(0, 1)
        gm = gc.cumsum(-1) * RCP_LN2
        D = torch.exp2((gm[:, :, None] - gm[:, None, :]).masked_fill(~strict, 0.0))
        Lm = (bc[:, :, None] * (kc @ kc.transpose(1, 2)) * D).masked_fill(~strict, 0.0)
        A = torch.linalg.solve_triangular(eye + Lm, eye.expand(HV, BT, BT), upper=False)
        A = _rd(A, emulate_bf16)
        wc = A @ _rd(kc * (bc * torch.exp2(gm))[:, :, None], emulate_bf16)
        uc = A @ _rd(vc * bc[:, :, None], emulate_bf16)
        gam[s:s + L] = gm.transpose(0, 1)[:L]
        A_out[s:s + L] = A.transpose(0, 1)[:L]
        w[s:s + L] = _rd(wc, emulate_bf16).transpose(0, 1)[:L]
        u[s:s + L] = _rd(uc, emulate_bf16).transpose(0, 1)[:L]
    return gam, A_out, w, u


def stage_scan_fwd(k, w, u, gam, h0, bounds, emulate_bf16=False):
    """Serial state scan (fla/ops/common/chunk_delta_h.py:58-348): per chunk store the state at
    chunk START, v_new = u - w S, S <- 2^gam_last S + (k 2^(gam_last-gam))^T v_new.

    -> h ``[NT,HV,K,V]``, v_new ``[R,HV,V]``, ht ``[N,HV,K,V]``.
    """
    R, H, K = k.shape
    HV, V = u.shape[1], u.shape[2]
    G = HV // H
    dt = k.dtype
    table = chunk_table(bounds)
    h = torch.zeros(len(table), HV, K, V, dtype=dt)
    v_new = torch.zeros(R, HV, V, dtype=dt)
    ht = torch.zeros(len(bounds), HV, K, V, dtype=dt)
    S = None
    prev = -1
    for c, (n, s, L) in enumerate(table):
        if n != prev:
            if prev >= 0:
                ht[prev] = S
            S = torch.zeros(HV, K, V, dtype=dt) if h0 is None else h0[n].to(dt).clone()
            prev = n
        kc = _tile(k, s, L).repeat_interleave(G, dim=1).transpose(0, 1)
        wc = _tile(w, s, L).transpose(0, 1)
        uc = _tile(u, s, L).transpose(0, 1)
        gm = _tile(gam, s, L).transpose(0, 1).clone()
        gl = gm[:, L - 1]
        gm[:, L:] = gl[:, None]                       # padded rows carry the last valid gamma
        Sb = _rd(S, emulate_bf16)
        h[c] = Sb
        vn = uc - wc @ Sb
        v_new[s:s + L] = _rd(vn, emulate_bf16).transpose(0, 1)[:L]
        vt = _rd(vn * torch.exp2(gl[:, None] - gm)[:, :, None], emulate_bf16)
        S = S * torch.exp2(gl)[:, None, None] + kc.transpose(1, 2) @ vt
    if prev >= 0:
        ht[prev] = S
    return h, v_new, ht


def stage_out(q, k, v_new, h, gam, scale, bounds, emulate_bf16=False):
    """o = scale [ (q h) 2^gam + tril(q k^T 2^(gam_i-gam_j)) v_new ]  (fla/ops/common/chunk_o.py:56-153)."""
    R, H, K = q.shape
    HV, V = v_new.shape[1], v_new.shape[2]
    G = HV // H
    dt = q.dtype
    o = torch.zeros(R, HV, V, dtype=dt)
    lower = torch.tril(torch.ones(BT, BT, dtype=torch.bool))
    for c, (_, s, L) in enumerate(chunk_table(bounds)):
        qc = _tile(q, s, L).repeat_interleave(G, dim=1).transpose(0, 1)
        kc = _tile(k, s, L).repeat_interleave(G, dim=1).transpose(0, 1)
        vn = _tile(v_new, s, L).transpose(0, 1)
        gm = _tile(gam, s, L).transpose(0, 1).clone()
        gm[:, L:] = gm[:, L - 1:L]
        D = torch.exp2((gm[:, :, None] - gm[:, None, :]).masked_fill(~lower, 0.0))
        P = _rd(((qc @ kc.transpose(1, 2)) * D).masked_fill(~lower, 0.0), emulate_bf16)
        oc = (qc @ h[c]) * torch.exp2(gm)[:, :, None] + P @ vn
        o[s:s + L] = (oc * scale).transpose(0, 1)[:L]
    return o


def stage_qk(q, k, gam, HV, bounds):
    """The chunk-local attention tile of the output and of dv_local, without the scale:
    qk[i, j] = <q_i, k_j> 2^(gam_i - gam_j) for j <= i, else 0  (fla/ops/common/chunk_o.py:115-127, 505-520);
    one row of 64 entries per (token, value head)."""
    R, H, K = q.shape
    G = HV // H
    out = torch.zeros(R, HV, BT, dtype=q.dtype)
    lower = torch.tril(torch.ones(BT, BT, dtype=torch.bool))
    for (_, s, L) in chunk_table(bounds):
        qc = _tile(q, s, L).repeat_interleave(G, dim=1).transpose(0, 1)
        kc = _tile(k, s, L).repeat_interleave(G, dim=1).transpose(0, 1)
        gm = _tile(gam, s, L).transpose(0, 1).clone()
        gm[:, L:] = gm[:, L - 1:L]
        D = torch.exp2((gm[:, :, None] - gm[:, None, :]).masked_fill(~lower, 0.0))
        P = ((qc @ kc.transpose(1, 2)) * D).masked_fill(~lower, 0.0)
        out[s:s + L] = P.transpose(0, 1)[:L]
    return out


def chunk_fwd(q, k, v, g, beta, scale, h0, bounds, emulate_bf16=False):
    """All forward stages chained (fla/ops/gated_delta_rule/chunk.py:33-123)."""
    gam, A, w, u = stage_intra(k, v, g, beta, bounds, emulate_bf16)
    h, v_new, ht = stage_scan_fwd(k, w, u, gam, h0, bounds, emulate_bf16)
    o = stage_out(q, k, v_new, h, gam, scale, bounds, emulate_bf16)
    return dict(gamma=gam, A=A, w=w, u=u, h=h, v_new=v_new, ht=ht, o=o, qk=stage_qk(q, k, gam, HV=v.shape[1], bounds=bounds))


# --------------------------------------------------------------------------- backward stages
def stage_dv_local(q, k, gam, do, scale, bounds, emulate_bf16=False):
    """dv_local[j] = sum_{i>=j} scale <k_j,q_i> 2^(gam_i-gam_j) do_i  (fla/ops/common/chunk_o.py:465-540)."""
    R, H, K = q.shape
    HV, V = do.shape[1], do.shape[2]
    G = HV // H
    dt = q.dtype
    dv = torch.zeros(R, HV, V, dtype=dt)
    lower = torch.tril(torch.ones(BT, BT, dtype=torch.bool))
    for (_, s, L) in chunk_table(bounds):
        qc = _tile(q, s, L).repeat_interleave(G, dim=1).transpose(0, 1)
        kc = _tile(k, s, L).repeat_interleave(G, dim=1).transpose(0, 1)
        dc = _tile(do, s, L).transpose(0, 1)
        gm = _tile(gam, s, L).transpose(0, 1).clone()
        gm[:, L:] = gm[:, L - 1:L]
        D = torch.exp2((gm[:, :, None] - gm[:, None, :]).masked_fill(~lower, 0.0))
        P = _rd(((qc @ kc.transpose(1, 2)) * D).masked_fill(~lower, 0.0) * scale, emulate_bf16)
        dv[s:s + L] = (P.transpose(1, 2) @ dc).transpose(0, 1)[:L]
    return dv


def stage_scan_bwd(q, k, w, gam, do, dv_local, dht, scale, bounds, emulate_bf16=False):
    """Reverse scan (fla/ops/common/chunk_delta_h.py:369-683): per chunk store dS at chunk END,
    dv2 = (k dS) 2^(gam_last-gam) + dv_local,
    dS <- 2^gam_last dS + scale (q 2^gam)^T do - w^T dv2.

    -> dh ``[NT,HV,K,V]``, dh0 ``[N,HV,K,V]``, dv2 ``[R,HV,V]``.
    """
    R, H, K = q.shape
    HV, V = do.shape[1], do.shape[2]
    G = HV // H
    dt = q.dtype
    table = chunk_table(bounds)
    dh = torch.zeros(len(table), HV, K, V, dtype=dt)
    dh0 = torch.zeros(len(bounds), HV, K, V, dtype=dt)
    dv2 = torch.zeros(R, HV, V, dtype=dt)
    dS = None
    prev = -1
    for c in range(len(table) - 1, -1, -1):
        n, s, L = table[c]
        if n != prev:
            if prev >= 0:
                dh0[prev] = dS
            dS = torch.zeros(HV, K, V, dtype=dt) if dht is None else dht[n].to(dt).clone()
            prev = n
        qc = _tile(q, s, L).repeat_interleave(G, dim=1).transpose(0, 1)
        kc = _tile(k, s, L).repeat_interleave(G, dim=1).transpose(0, 1)
        wc = _tile(w, s, L).transpose(0, 1)
        dc = _tile(do, s, L).transpose(0, 1)
        dl = _tile(dv_local, s, L).transpose(0, 1)
        gm = _tile(gam, s, L).transpose(0, 1).clone()
        gl = gm[:, L - 1]
        gm[:, L:] = gl[:, None]
        dSb = _rd(dS, emulate_bf16)
        dh[c] = dSb
        d2 = (kc @ dSb) * torch.exp2(gl[:, None] - gm)[:, :, None] + dl
        d2 = _rd(d2, emulate_bf16)
        dv2[s:s + L] = d2.transpose(0, 1)[:L]
        qg = _rd(dc * (torch.exp2(gm) * scale)[:, :, None], emulate_bf16)
        dS = dS * torch.exp2(gl)[:, None, None] + qc.transpose(1, 2) @ qg - wc.transpose(1, 2) @ d2
    if prev >= 0:
        dh0[prev] = dS
    return dh, dh0, dv2


def stage_dqkwg(q, k, v_new, gam, h, dv2, do, dh, scale, bounds, emulate_bf16=False):
    """dq, dk (summed over each value-head group), dw = -dv2 h^T and the gate gradient with
    respect to the chunk-local cumsum (natural log), fla/ops/common/chunk_o.py:172-342:

        dP   = tril(do v_new^T 2^(gam_i-gam_j)) scale
        dq   = scale (do h^T) 2^gam + dP k
        dk   = dP^T q + (v_new dh^T) 2^(gam_last-gam)
        dG_i = <dq_i,q_i> - <dk_i,k_i>, plus at the last row
               2^gam_last <h,dh> + sum_i <(v_new dh^T)_i 2^(gam_last-gam_i), k_i>.
    -> dq ``[R,H,K]``, dk_part ``[R,H,K]``, dw ``[R,HV,K]``, dG_part ``[R,HV]`` (64-row semantics:
    the last-row term of a ragged chunk is returned in ``dG_tail[c]`` so the caller can fold it in).
    """
    R, H, K = q.shape
    HV, V = do.shape[1], do.shape[2]
    G = HV // H
    dt = q.dtype
    table = chunk_table(bounds)
    dq = torch.zeros(R, H, K, dtype=dt)
    dk = torch.zeros(R, H, K, dtype=dt)
    dw = torch.zeros(R, HV, K, dtype=dt)
    dG = torch.zeros(R, HV, dtype=dt)
    dG_tail = torch.zeros(len(table), HV, dtype=dt)
    lower = torch.tril(torch.ones(BT, BT, dtype=torch.bool))
    for c, (_, s, L) in enumerate(table):
        qc = _tile(q, s, L).repeat_interleave(G, dim=1).transpose(0, 1)
        kc = _tile(k, s, L).repeat_interleave(G, dim=1).transpose(0, 1)
        vn = _tile(v_new, s, L).transpose(0, 1)
        dc = _tile(do, s, L).transpose(0, 1)
        d2 = _tile(dv2, s, L).transpose(0, 1)
        gm = _tile(gam, s, L).transpose(0, 1).clone()
        gl = gm[:, L - 1]
        gm[:, L:] = gl[:, None]
        D = torch.exp2((gm[:, :, None] - gm[:, None, :]).masked_fill(~lower, 0.0))
        dP = _rd(((dc @ vn.transpose(1, 2)) * D).masked_fill(~lower, 0.0) * scale, emulate_bf16)
        dq_c = (dc @ h[c].transpose(1, 2)) * (torch.exp2(gm) * scale)[:, :, None] + dP @ kc
        dk_state = (vn @ dh[c].transpose(1, 2)) * torch.exp2(gl[:, None] - gm)[:, :, None]
        dk_c = dP.transpose(1, 2) @ qc + dk_state
        dw_c = -(d2 @ h[c].transpose(1, 2))
        dG_c = (dq_c * qc).sum(-1) - (dk_c * kc).sum(-1)                    # [HV,64]
        tail = torch.exp2(gl) * (h[c] * dh[c]).sum((-1, -2)) + (dk_state * kc).sum((-1, -2))
        dG_c[:, BT - 1] += tail                                            # row 63 (padded rows share gamma_last)
        dG_tail[c] = tail
        dq[s:s + L] = dq_c.reshape(H, G, BT, K).sum(1).transpose(0, 1)[:L]
        dk[s:s + L] = dk_c.reshape(H, G, BT, K).sum(1).transpose(0, 1)[:L]
        dw[s:s + L] = _rd(dw_c, emulate_bf16).transpose(0, 1)[:L]
        # rows beyond L hold only the tail term; fold them onto the last valid row so that the
        # stored [R,HV] array carries the complete 64-row information
        dG_valid = dG_c[:, :L].clone()
        dG_valid[:, L - 1] += dG_c[:, L:].sum(-1)
        dG[s:s + L] = dG_valid.transpose(0, 1)
    return dq, dk, dw, dG


def stage_wy_bwd(k, v, beta, gam, A, dw, du, dk_part, dG_part, bounds, emulate_bf16=False):
    """Backward of stage_intra (fla/ops/gated_delta_rule/wy_fast.py:123-251), then the reverse
    chunk-local cumsum that turns dG into dg (fla/ops/gated_delta_rule/chunk.py:244-246):

        dKbg = A^T dw,  dVb = A^T du,  dA = strict_tril(dw (k beta 2^gam)^T + du (v beta)^T)
        M    = -strict_tril(A^T dA A^T) 2^(gam_i-gam_j)
        dk   = dk_part + dKbg beta 2^gam + (M k) beta + (M beta_row)^T k      (group-summed)
        dv   = dVb beta
        dbeta= rowsum(dKbg k 2^gam) + rowsum(dVb v) + rowsum((M k) k)
        dG   = dG_part + rowsum(dKbg k) beta 2^gam + beta rowsum((M k) k) - rowsum(((M beta_row)^T k) k)
        dg   = reverse cumsum of dG inside the chunk.
    """
    R, H, K = k.shape
    HV, V = v.shape[1], v.shape[2]
    G = HV // H
    dt = k.dtype
    dk = dk_part.clone()
    dv = torch.zeros(R, HV, V, dtype=dt)
    db = torch.zeros(R, HV, dtype=dt)
    dg = torch.zeros(R, HV, dtype=dt)
    strict = torch.tril(torch.ones(BT, BT, dtype=torch.bool), -1)
    for (_, s, L) in chunk_table(bounds):
        kc = _tile(k, s, L).repeat_interleave(G, dim=1).transpose(0, 1)
        vc = _tile(v, s, L).transpose(0, 1)
        bc = _tile(beta, s, L).transpose(0, 1)
        gm = _tile(gam, s, L).transpose(0, 1).clone()
        gm[:, L:] = gm[:, L - 1:L]
        Ac = _tile(A, s, L).transpose(0, 1).clone()                         # [HV,64,64]
        idx = torch.arange(L, BT)
        Ac[:, idx, idx] = 1.0                                               # padded rows are identity rows
        dwc = _tile(dw, s, L).transpose(0, 1)
        duc = _tile(du, s, L).transpose(0, 1)
        eg = torch.exp2(gm)
        At = Ac.transpose(1, 2)
        dKbg = At @ dwc
        dVb = At @ duc
        dA = (dwc @ kc.transpose(1, 2)) * (bc * eg)[:, None, :] + (duc @ vc.transpose(1, 2)) * bc[:, None, :]
        dA = _rd(dA.masked_fill(~strict, 0.0), emulate_bf16)
        X = At @ _rd(dA @ At, emulate_bf16)
        D = torch.exp2((gm[:, :, None] - gm[:, None, :]).masked_fill(~strict, 0.0))
        M = _rd((-X * D).masked_fill(~strict, 0.0), emulate_bf16)
        MK = M @ kc
        M2K = _rd(M * bc[:, :, None], emulate_bf16).transpose(1, 2) @ kc
        dk_c = dKbg * (bc * eg)[:, :, None] + MK * bc[:, :, None] + M2K
        dv_c = dVb * bc[:, :, None]
        r_kbg = (dKbg * kc).sum(-1)
        r_mk = (MK * kc).sum(-1)
        db_c = r_kbg * eg + (dVb * vc).sum(-1) + r_mk
        dG_c = r_kbg * bc * eg + bc * r_mk - (M2K * kc).sum(-1)
        dG_c[:, :L] += _tile(dG_part, s, L).transpose(0, 1)[:, :L]
        dg_c = dG_c.flip(-1).cumsum(-1).flip(-1)
        dk[s:s + L] += dk_c.reshape(H, G, BT, K).sum(1).transpose(0, 1)[:L]
        dv[s:s + L] = dv_c.transpose(0, 1)[:L]
        db[s:s + L] = db_c.transpose(0, 1)[:L]
        dg[s:s + L] = dg_c.transpose(0, 1)[:L]
    return dk, dv, db, dg


def chunk_bwd(q, k, v, g, beta, scale, h0, do, dht, bounds, fwd=None, emulate_bf16=False):
    """All backward stages chained (fla/ops/gated_delta_rule/chunk.py:126-250)."""
    if fwd is None:
        fwd = chunk_fwd(q, k, v, g, beta, scale, h0, bounds, emulate_bf16)
    gam = fwd['gamma']
    dv_local = stage_dv_local(q, k, gam, do, scale, bounds, emulate_bf16)
    dh, dh0, dv2 = stage_scan_bwd(q, k, fwd['w'], gam, do, dv_local, dht, scale, bounds, emulate_bf16)
    dq, dk_part, dw, dG = stage_dqkwg(q, k, fwd['v_new'], gam, fwd['h'], dv2, do, dh, scale, bounds, emulate_bf16)
    dk, dv, db, dg = stage_wy_bwd(k, v, beta, gam, fwd['A'], dw, dv2, dk_part, dG, bounds, emulate_bf16)
    return dict(dv_local=dv_local, dh=dh, dh0=dh0, dv2=dv2, dq=dq, dk_part=dk_part, dw=dw, dG=dG,
                dk=dk, dv=dv, dbeta=db, dg=dg)


# --------------------------------------------------------------------------- seeded inputs
def make_inputs(B, T, H, HV, K, V, seed=0, dtype=torch.float32, cu_seqlens=None, with_h0=True, h0_std=0.1):
    """The synthetic input distributions of the benchmark configurations: q, k ~ N(0,1)
    L2-normalised over K, v ~ N(0,1), g = logsigmoid(N(0,1)), beta = sigmoid(N(0,1)),
    h0 ~ N(0, h0_std^2); generated in fp32 on the CPU from ``seed`` then cast."""
    gen = torch.Generator().manual_seed(seed)
    q = F.normalize(torch.randn(B, T, H, K, generator=gen), p=2, dim=-1).to(dtype)
    k = F.normalize(torch.randn(B, T, H, K, generator=gen), p=2, dim=-1).to(dtype)
    v = torch.randn(B, T, HV, V, generator=gen).to(dtype)
    g = F.logsigmoid(torch.randn(B, T, HV, generator=gen))
    beta = torch.sigmoid(torch.randn(B, T, HV, generator=gen))
    N = B if cu_seqlens is None else len(cu_seqlens) - 1
    h0 = (torch.randn(N, HV, K, V, generator=gen) * h0_std) if with_h0 else None
    do = torch.randn(B, T, HV, V, generator=gen).to(dtype)
    dht = torch.randn(N, HV, K, V, generator=gen) * h0_std
    return dict(q=q, k=k, v=v, g=g, beta=beta, h0=h0, do=do, dht=dht)


def random_cu_seqlens(n_seq: int, total: int, lo: int, hi: int, seed: int = 0) -> List[int]:
    """n_seq lengths drawn uniformly from [lo, hi] and adjusted to sum to ``total``."""
    gen = torch.Generator().manual_seed(seed)
    lens = torch.randint(lo, hi + 1, (n_seq,), generator=gen).double()
    lens = (lens * (total / lens.sum())).floor().long().clamp(min=1)
    i = 0
    while int(lens.sum()) != total:
        d = 1 if int(lens.sum()) < total else -1
        if lens[i % n_seq] + d >= 1:
            lens[i % n_seq] += d
        i += 1
    cu = [0]
    for x in lens.tolist():
        cu.append(cu[-1] + int(x))
    return cu


# --------------------------------------------------------------------------- the steps either side of the mixer
def causal_conv1d_ref(x, weight, bias=None, residual=None, initial_state=None, activation=None, cu_seqlens=None,
                      output_final_state=False):
    """Short causal depthwise convolution per sequence (the reference's torch statement of it,
    tests/modules/test_conv.py:31-73, generalised to packed sequences and the ``[N,D,W]`` cache of
    fla/modules/conv/causal_conv1d.py:17-160): ``y[t,d] = act(bias[d] + sum_w weight[d,w] x[t-(W-1)+w, d])`` with the
    inputs before a sequence taken from the last W-1 cache entries (zero without a cache); ``final_state[n,d,:]`` =
    the last W inputs.  x ``[B,T,D]``; differentiable (torch autograd is the gradient oracle)."""
    B, T, D = x.shape
    W = weight.shape[-1]
    xs = x.reshape(B * T, D)
    bounds = seq_bounds(B, T, cu_seqlens)
    ys, finals, pos = [], [], 0
    for n, (s, e) in enumerate(bounds):
        if s > pos:                                                               # rows that belong to no sequence
            ys.append(torch.zeros(s - pos, D, dtype=x.dtype))
        seq = xs[s:e].transpose(0, 1)[None]                                       # [1,D,L]
        cache = torch.zeros(1, D, W, dtype=x.dtype) if initial_state is None else initial_state[n:n + 1].to(x.dtype)
        full = torch.cat([cache, seq], dim=-1)                                    # W cache entries, then the sequence
        out = F.conv1d(full, weight.to(x.dtype)[:, None, :], None if bias is None else bias.to(x.dtype), groups=D)
        out = out[..., 1:]                                                        # output of token t sits at index t + 1
        if activation in ('silu', 'swish'):
            out = F.silu(out)
        ys.append(out[0].transpose(0, 1))
        finals.append(full[..., -W:])
        pos = e
    if pos < B * T:
        ys.append(torch.zeros(B * T - pos, D, dtype=x.dtype))
    y = torch.cat(ys, 0).reshape(B, T, D)
    if residual is not None:
        y = y + residual
    return (y, torch.cat(finals, 0)) if output_final_state else (y, None)


def rms_norm_gated_ref(x, g, weight=None, bias=None, activation='swish', eps=1e-6):
    """``(x rstd weight + bias) act(g)`` over the last dimension, rstd = 1/sqrt(mean(x^2) + eps), act = g sigmoid(g)
    (swish / silu) or sigmoid(g)  (fla/modules/fused_norm_gate.py:36-124, RMS form without residual)."""
    rstd = torch.rsqrt(x.square().mean(-1, keepdim=True) + eps)
    y = x * rstd
    if weight is not None:
        y = y * weight
    if bias is not None:
        y = y + bias
    return y * (torch.sigmoid(g) if activation == 'sigmoid' else g * torch.sigmoid(g))
