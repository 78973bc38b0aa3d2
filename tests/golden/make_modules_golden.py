"""Fixtures for the convolution in front of the mixer, produced by the reference's own torch statement of it
(causal_conv1d_ref_torch, tests/modules/test_conv.py:31-73 of the reference checkout) on seeded inputs, with autograd
gradients.  Run where the reference checkout is importable:

    PYTHONPATH=/path/to/reference:/path/to/reference/tests/modules python tests/golden/make_modules_golden.py
"""
import os

import numpy as np
import torch

CONV_CASES = {
    # name: (B, T, D, W, activation, bias, cache)
    'conv_w4_silu': (2, 75, 32, 4, 'silu', True, True),
    'conv_w3_plain': (1, 130, 16, 3, None, False, False),
    'conv_w2_short': (3, 1, 24, 2, 'silu', True, True),
}


def main():
    from test_conv import causal_conv1d_ref_torch
    here = os.path.dirname(os.path.abspath(__file__))
    for name, (B, T, D, W, act, has_bias, has_cache) in CONV_CASES.items():
        gen = torch.Generator().manual_seed(1234)
        x = torch.randn(B, T, D, generator=gen, dtype=torch.float64, requires_grad=True)
        w = (torch.randn(D, W, generator=gen, dtype=torch.float64) * 0.5).requires_grad_(True)
        b = torch.randn(D, generator=gen, dtype=torch.float64).requires_grad_(True) if has_bias else None
        cache = torch.randn(B, D, W - 1, generator=gen, dtype=torch.float64).requires_grad_(True) if has_cache else None
        dy = torch.randn(B, T, D, generator=gen, dtype=torch.float64)
        out = causal_conv1d_ref_torch(x.transpose(1, 2), w, b, initial_state=cache, output_final_state=True, activation=act)
        y, final = out[0].transpose(1, 2), out[1]
        (y * dy).sum().backward()
        rec = dict(x=x, w=w, dy=dy, y=y, final=final, dx=x.grad, dw=w.grad)
        if has_bias:
            rec.update(b=b, db=b.grad)
        if has_cache:
            rec.update(cache=cache, dcache=cache.grad)
        np.savez_compressed(os.path.join(here, name + '.npz'), **{k: v.detach().numpy() for k, v in rec.items()})
        print(name, 'written')


if __name__ == '__main__':
    main()
