"""Golden outputs of the reference's own Triton chunk path (what the north star measures correctness against).

    python tests/golden/make_triton_golden.py --reference /path/to/flash-linear-attention

Needs a CUDA GPU and a checkout of fla-org/flash-linear-attention (0.5.2) with Triton: runs
``fla.ops.gated_delta_rule.chunk_gated_delta_rule`` (backend dispatch disabled, i.e. the stock Triton kernels)
forward + backward on seeded inputs (``oracle.make_inputs``; q/k/v/do rounded to bf16) and stores o, the final
state and all gradients as fp32 arrays in ``tests/golden/triton_<case>.npz``.  Inputs are not stored: the tests
regenerate them from the same seeds.  The committed files were produced on a B200 with Triton 3.6.
"""
import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

TRITON_CASES = {
    # name: (B, T, H, HV, K, V, cu_seqlens, seed)
    'triton_d128_dense': (2, 256, 2, 2, 128, 128, None, 21),
    'triton_d128_varlen_gva': (1, 300, 2, 4, 128, 128, [0, 37, 101, 165, 300], 22),
    'triton_d64_dense': (1, 192, 2, 2, 64, 64, None, 23),
}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--reference', required=True, help='checkout of fla-org/flash-linear-attention (0.5.2) to import')
    ap.add_argument('--out', default=HERE)
    args = ap.parse_args()
    os.environ['FLA_DISABLE_BACKEND_DISPATCH'] = '1'
    sys.path.insert(0, args.reference)
    from fla.ops.gated_delta_rule import chunk_gated_delta_rule

    from oracle.gdn_oracle import make_inputs
    dev = 'cuda'
    for name, (B, T, H, HV, K, V, cu, seed) in TRITON_CASES.items():
        d = make_inputs(B, T, H, HV, K, V, seed=seed, cu_seqlens=cu)
        leaves = {n: d[n].to(torch.bfloat16).to(dev).requires_grad_(True) for n in ('q', 'k', 'v')}
        leaves.update({n: d[n].float().to(dev).requires_grad_(True) for n in ('g', 'beta', 'h0')})
        cu_t = None if cu is None else torch.tensor(cu, dtype=torch.long, device=dev)
        o, ht = chunk_gated_delta_rule(leaves['q'], leaves['k'], leaves['v'], leaves['g'], leaves['beta'], scale=K ** -0.5,
                                       initial_state=leaves['h0'], output_final_state=True, cu_seqlens=cu_t)
        loss = (o.float() * d['do'].to(torch.bfloat16).float().to(dev)).sum() + (ht * d['dht'].to(dev)).sum()
        loss.backward()
        out = dict(o=o.detach().float().cpu().numpy(), ht=ht.detach().float().cpu().numpy())
        for n in ('q', 'k', 'v', 'g', 'beta', 'h0'):
            out['d' + n] = leaves[n].grad.float().cpu().numpy()
        np.savez_compressed(os.path.join(args.out, name + '.npz'), **out)
        print(name, {k: v.shape for k, v in out.items()})


if __name__ == '__main__':
    main()
