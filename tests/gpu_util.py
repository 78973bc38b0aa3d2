"""Helpers for the GPU parity tests: run the C-ABI passes on seeded inputs and return every
intermediate so each stage can be compared with the oracle's stage of the same name."""
import torch

from b200gdn import _lib
from b200gdn.chunk import new_chunk_args
from b200gdn.index import build_tables
from oracle import gdn_oracle as O


def flat(x):
    return x.reshape(x.shape[0] * x.shape[1], *x.shape[2:])


def make_case(B, T, H, HV, K, V, cu=None, seed=0, with_h0=True):
    d = O.make_inputs(B, T, H, HV, K, V, seed=seed, cu_seqlens=cu, with_h0=with_h0)
    # the kernels see bf16 q/k/v/do; the oracle gets the same rounded values in fp32
    for n in ('q', 'k', 'v', 'do'):
        d[n] = d[n].to(torch.bfloat16)
    d['bounds'] = O.seq_bounds(B, T, cu)
    d['scale'] = K ** -0.5
    d['dims'] = (B, T, H, HV, K, V)
    return d


def oracle_chain(d, dtype=torch.float32, emulate_bf16=False):
    q, k, v, g, beta, do = (flat(d[n]).to(dtype) for n in ('q', 'k', 'v', 'g', 'beta', 'do'))
    h0 = None if d['h0'] is None else d['h0'].to(dtype)
    fwd = O.chunk_fwd(q, k, v, g, beta, d['scale'], h0, d['bounds'], emulate_bf16)
    bwd = O.chunk_bwd(q, k, v, g, beta, d['scale'], h0, do, d['dht'].to(dtype), d['bounds'], fwd=fwd,
                      emulate_bf16=emulate_bf16)
    return fwd, bwd


def gamma_to_chunks(gamma_rows, bounds):
    """[rows,HV] -> the kernels' per-chunk layout [n_chunks,HV,64] (tail repeats the last valid value)."""
    out = []
    for (_, s, L) in O.chunk_table(bounds):
        g = gamma_rows[s:s + L]
        if L < 64:
            g = torch.cat([g, g[-1:].expand(64 - L, -1)], 0)
        out.append(g.transpose(0, 1))
    return torch.stack(out, 0).contiguous()


def gamma_from_chunks(gamma_chunks, bounds, rows):
    out = torch.zeros(rows, gamma_chunks.shape[1], dtype=gamma_chunks.dtype)
    for c, (_, s, L) in enumerate(O.chunk_table(bounds)):
        out[s:s + L] = gamma_chunks[c].transpose(0, 1)[:L]
    return out


def run_abi(d, dev='cuda', fwd_mask=0, bwd_mask=0, overrides=None, do_bwd=True):
    """Forward (and backward) through b200gdn_chunk_fwd / b200gdn_chunk_bwd.  ``overrides`` replaces
    saved tensors (by name) before the backward pass, e.g. with the oracle's, to isolate one stage."""
    B, T, H, HV, K, V = d['dims']
    rows = B * T
    cm, sm = build_tables(d['bounds'])
    chunk_meta, seq_meta = torch.from_numpy(cm).to(dev), torch.from_numpy(sm).to(dev)
    n_chunks, n_seq = cm.shape[0], sm.shape[0]
    q, k, v, do = (d[n].to(dev).contiguous() for n in ('q', 'k', 'v', 'do'))
    g, beta = d['g'].float().to(dev).contiguous(), d['beta'].float().to(dev).contiguous()
    h0 = None if d['h0'] is None else d['h0'].float().to(dev).contiguous()
    dht = d['dht'].float().to(dev).contiguous()
    bf = dict(dtype=torch.bfloat16, device=dev)
    f32 = dict(dtype=torch.float32, device=dev)
    nan = float('nan')
    t = dict(
        o=torch.full((rows, HV, V), nan, **bf), ht=torch.full((n_seq, HV, K, V), nan, **f32),
        gamma=torch.full((n_chunks, HV, 64), nan, **f32), A=torch.full((rows, HV, 64), nan, **bf),
        qk=torch.full((rows, HV, 64), nan, **bf),
        w=torch.full((rows, HV, K), nan, **bf), u=torch.full((rows, HV, V), nan, **bf),
        h=torch.full((n_chunks, HV, K, V), nan, **bf), v_new=torch.full((rows, HV, V), nan, **bf),
        dq=torch.full((rows, H, K), nan, **bf), dk=torch.full((rows, H, K), nan, **bf),
        dv=torch.full((rows, HV, V), nan, **bf), dg=torch.full((rows, HV), nan, **f32),
        dbeta=torch.full((rows, HV), nan, **f32), dh0=torch.full((n_seq, HV, K, V), nan, **f32),
        dh=torch.full((n_chunks, HV, K, V), nan, **bf), dv2=torch.full((rows, HV, V), nan, **bf),
        dk_part=torch.full((rows, H, K), nan, **f32) if HV > H else None,
        dG=torch.full((rows, HV), nan, **f32), dq_acc=torch.full((rows, H, K), nan, **f32) if HV > H else None,
    )
    a = new_chunk_args(q, k, v, d['scale'], (chunk_meta, seq_meta, (n_chunks, n_seq)))
    a.g, a.beta, a.h0 = g.data_ptr(), beta.data_ptr(), _lib.ptr(h0)
    a.d_o, a.dht = do.data_ptr(), dht.data_ptr()
    if overrides:
        for name, val in overrides.items():
            if name == 'gamma':
                val = gamma_to_chunks(val, d['bounds'])
            t[name] = val.to(dev).to(t[name].dtype).contiguous()
    for name, val in t.items():
        setattr(a, name, _lib.ptr(val))
    st = torch.cuda.current_stream().cuda_stream
    a.stage_mask = fwd_mask
    if fwd_mask >= 0:
        _lib.call('b200gdn_chunk_fwd', a, st)
    if do_bwd:
        a.stage_mask = bwd_mask
        _lib.call('b200gdn_chunk_bwd', a, st)
    torch.cuda.synchronize()
    out = {n_: x.float().cpu() for n_, x in t.items() if x is not None}
    out['gamma'] = gamma_from_chunks(out['gamma'], d['bounds'], rows)
    return out
