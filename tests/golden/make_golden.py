"""Generate the golden fixtures in this folder from the reference implementation itself.

Run where a checkout of fla-org/flash-linear-attention is available (CPU is enough):

    python tests/golden/make_golden.py --reference /path/to/flash-linear-attention

It imports the reference's own torch functions
(fla/ops/gated_delta_rule/naive.py: naive_recurrent_gated_delta_rule, naive_chunk_gated_delta_rule;
fla/ops/gated_delta_rule/gate.py: naive_gdn_gate; fla/ops/cp/context.py: get_cp_cu_seqlens),
runs them on seeded inputs (oracle.gdn_oracle.make_inputs, regenerated identically by the tests)
and stores outputs and autograd gradients as .npz.  Grouped value heads and packed sequences are
fed to the reference the way its own tests do (q/k repeated per group, one call per sequence:
tests/ops/test_gdn.py:108-200, 712-803).  The fixtures are what pins the oracle.
"""
import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.abspath(os.path.join(HERE, '..', '..')))

CASES = {
    # name: (B, T, H, HV, K, V, cu_seqlens, seed, with_grads)
    'config1_naive_cpu': (1, 1024, 4, 4, 64, 64, None, 0, False),
    'small_dense': (2, 128, 2, 2, 64, 64, None, 1, True),
    'gva_dense': (1, 192, 2, 4, 64, 64, None, 2, True),
    'varlen_ragged': (1, 300, 2, 4, 64, 64, [0, 37, 101, 165, 300], 3, True),
    'd128_dense': (1, 128, 1, 1, 128, 128, None, 4, True),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--reference', required=True, help='checkout of fla-org/flash-linear-attention (0.5.2) to import')
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    from fla.ops.cp.context import get_cp_cu_seqlens
    from fla.ops.gated_delta_rule.gate import naive_gdn_gate
    from fla.ops.gated_delta_rule.naive import naive_chunk_gated_delta_rule, naive_recurrent_gated_delta_rule

    from oracle.gdn_oracle import make_inputs, seq_bounds

    for name, (B, T, H, HV, K, V, cu, seed, with_grads) in CASES.items():
        d = make_inputs(B, T, H, HV, K, V, seed=seed, cu_seqlens=cu)
        G = HV // H
        scale = K ** -0.5
        dt = torch.float32   # the reference computes in fp32 internally (naive.py:40)
        leaves = {n: d[n].detach().to(dt).clone().requires_grad_(with_grads) for n in ('q', 'k', 'v', 'g', 'beta', 'h0')}
        bounds = seq_bounds(B, T, cu)
        os_, hts, ocs = [], [], []
        for n, (bos, eos) in enumerate(bounds):
            def rows(x):
                return x.reshape(1, B * T, *x.shape[2:])[:, bos:eos]
            qn = rows(leaves['q']).repeat_interleave(G, dim=2)
            kn = rows(leaves['k']).repeat_interleave(G, dim=2)
            h0n = leaves['h0'][n:n + 1] if cu is not None else leaves['h0']
            if cu is None and n > 0:
                break
            if cu is None:
                qn = leaves['q'].repeat_interleave(G, dim=2)
                kn = leaves['k'].repeat_interleave(G, dim=2)
                vn, gn, bn = leaves['v'], leaves['g'], leaves['beta']
            else:
                vn, gn, bn = rows(leaves['v']), rows(leaves['g']), rows(leaves['beta'])
            o, ht = naive_recurrent_gated_delta_rule(qn, kn, vn, bn, gn, scale=scale, initial_state=h0n,
                                                     output_final_state=True)
            oc, _ = naive_chunk_gated_delta_rule(qn.detach().float(), kn.detach().float(), vn.detach().float(),
                                                 gn.detach().float(), bn.detach().float(), scale=scale,
                                                 initial_state=h0n.detach().float(), output_final_state=True)
            os_.append(o)
            hts.append(ht)
            ocs.append(oc)
        o = torch.cat(os_, 1).reshape(B, T, HV, V) if cu is not None else os_[0]
        oc = torch.cat(ocs, 1).reshape(B, T, HV, V) if cu is not None else ocs[0]
        ht = torch.cat(hts, 0)
        out = dict(o=o.detach().float().numpy(), ht=ht.detach().float().numpy(),
                   o_chunk=oc.detach().float().numpy())
        if with_grads:
            loss = (o * d['do'].to(o.dtype)).sum() + (ht * d['dht'].to(ht.dtype)).sum()
            loss.backward()
            for n in ('q', 'k', 'v', 'g', 'beta', 'h0'):
                out['d' + n] = leaves[n].grad.float().numpy()
        if name == 'config1_naive_cpu':
            out['o'] = out['o'][:, ::8]          # every 8th token keeps the file small
            out['o_chunk'] = out['o_chunk'][:, ::8]
        np.savez_compressed(os.path.join(HERE, name + '.npz'), **out)
        print(name, {k: v.shape for k, v in out.items()})

    # gate and context-partition fixtures
    gen = torch.Generator().manual_seed(7)
    graw = torch.randn(3, 50, 6, generator=gen)
    A_log = torch.randn(6, generator=gen)
    dt_bias = torch.randn(6, generator=gen)
    np.savez_compressed(os.path.join(HERE, 'gate.npz'), g=graw.numpy(), A_log=A_log.numpy(), dt_bias=dt_bias.numpy(),
                        out=naive_gdn_gate(graw, A_log, dt_bias).numpy(),
                        out_nobias=naive_gdn_gate(graw, A_log, None).numpy())
    cp = {}
    cp_cases = [([0, 5, 12], 3), ([0, 4096], 4), ([0, 100, 200, 1000, 1024], 4), ([0, 7, 8, 9, 64], 8),
                ([0, 3000, 3001, 8192], 8)]
    for ci, (cu, W) in enumerate(cp_cases):
        for r in range(W):
            c = get_cp_cu_seqlens(torch.tensor(cu, dtype=torch.long), world_size=W, rank=r)
            cp[f'{ci}_{r}'] = np.array(c.cu_seqlens_cpu.tolist() + [-1, c.pre_num_ranks, c.post_num_ranks,
                                       int(c.is_first_rank), int(c.is_last_rank), c.pre_num_conv_tokens])
        cp[f'case{ci}'] = np.array(cu + [-1, W])
    np.savez_compressed(os.path.join(HERE, 'cp_context.npz'), **cp)
    print('gate, cp_context written')


if __name__ == '__main__':
    main()
