"""GPU parity of the two steps either side of the mixer (short causal convolution, gated RMS norm) against their
oracles and the reference fixtures; tolerances as in the reference's tests (tests/modules/test_conv.py: 1e-3 err-ratio
in fp32, 5e-3 in half precision; tests/modules/test_layernorm_gated.py: 1e-3)."""
import os

import numpy as np
import pytest
import torch

from oracle import gdn_oracle as O
from tests.golden.make_modules_golden import CONV_CASES

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), 'golden')


@pytest.mark.parametrize('name', list(CONV_CASES))
def test_conv_against_reference_fixture(name):
    from b200gdn.modules import causal_conv1d
    B, T, D, W, act, has_bias, has_cache = CONV_CASES[name]
    gold = {k: torch.from_numpy(v).float() for k, v in np.load(os.path.join(GOLD, name + '.npz')).items()}
    dev = 'cuda'
    x = gold['x'].to(dev).requires_grad_(True)
    w = gold['w'].to(dev).requires_grad_(True)
    b = gold['b'].to(dev).requires_grad_(True) if has_bias else None
    cache = None
    if has_cache:
        c = gold['cache'].to(dev).requires_grad_(True)
        cache = torch.cat([torch.zeros(B, D, 1, device=dev), c], dim=-1)
    y, final = causal_conv1d(x, w, b, initial_state=cache, output_final_state=True, activation=act)
    (y * gold['dy'].to(dev)).sum().backward()
    O.assert_close('y', gold['y'], y.detach().cpu(), 1e-4)
    assert torch.allclose(final[..., 1:].cpu(), gold['final'], atol=1e-6)
    O.assert_close('dx', gold['dx'], x.grad.cpu(), 1e-4)
    O.assert_close('dw', gold['dw'], w.grad.cpu(), 1e-4)
    if has_bias:
        O.assert_close('db', gold['db'], b.grad.cpu(), 1e-4)
    if has_cache:
        O.assert_close('dcache', gold['dcache'], c.grad.cpu(), 1e-4)


@pytest.mark.parametrize('dtype,tol', [(torch.float32, 1e-4), (torch.bfloat16, 5e-3), (torch.float16, 2e-3)])
@pytest.mark.parametrize('W', [2, 3, 4])
def test_conv_packed_sequences_with_cache_and_residual(dtype, tol, W):
    """Packed ragged sequences (one shorter than the kernel, one spanning several 64-token tiles), cache, bias, residual."""
    from b200gdn.modules import causal_conv1d
    dev = 'cuda'
    cu = [0, 2, 3, 140, 204, 333]
    T, D, N = 333, 2048 + 64, 5
    gen = torch.Generator().manual_seed(11)
    x = torch.randn(1, T, D, generator=gen).to(dtype)
    w = (torch.randn(D, W, generator=gen) * 0.5)
    b = torch.randn(D, generator=gen)
    res = torch.randn(1, T, D, generator=gen).to(dtype)
    cache = torch.randn(N, D, W, generator=gen).to(dtype)
    dy = torch.randn(1, T, D, generator=gen).to(dtype)
    leaves = [t.float().double().requires_grad_(True) for t in (x, w, b, res, cache)]
    ry, rfinal = O.causal_conv1d_ref(*leaves[:4], leaves[4], 'silu', cu, True)
    (ry * dy.double()).sum().backward()
    g = [t.to(dev).requires_grad_(True) for t in (x, w, b, res, cache)]
    y, final = causal_conv1d(g[0], g[1], g[2], residual=g[3], initial_state=g[4], output_final_state=True, activation='silu',
                             cu_seqlens=torch.tensor(cu, device=dev))
    y.backward(dy.to(dev))
    assert y.dtype == dtype and final.dtype == dtype and final.shape == (N, D, W)
    O.assert_close('y', ry.float(), y.float().cpu(), tol)
    O.assert_close('final', rfinal.float(), final.float().cpu(), tol)
    for nme, a, r in zip(('dx', 'dw', 'db', 'dres', 'dcache'), g, leaves):
        got, want = a.grad.float().cpu(), r.grad.float()
        if nme == 'dcache':   # the oldest cache entry never enters the convolution
            assert torch.count_nonzero(got[..., 0]) == 0
        O.assert_close(nme, want, got, tol * (4 if nme in ('dw', 'db') and dtype != torch.float32 else 1))


def test_short_convolution_module_prefill_then_decode():
    """The layer object: a prefill with final state, then single-token steps that update the cache in place, against one
    pass over the whole sequence (tests/modules/test_conv.py:365-437, 560-640 of the reference test this contract)."""
    from b200gdn.modules import ShortConvolution
    dev = 'cuda'
    B, T, D, W = 3, 70, 256, 4
    torch.manual_seed(0)
    conv = ShortConvolution(D, W, bias=True, activation='silu', device=dev, dtype=torch.float32)
    x = torch.randn(B, T + 3, D, device=dev)
    full, _ = conv(x)
    y0, cache = conv(x[:, :T], output_final_state=True)
    assert torch.allclose(y0, full[:, :T], atol=1e-5)
    ptr = cache.data_ptr()
    for t in range(T, T + 3):
        yt, cache = conv(x[:, t:t + 1], cache=cache, output_final_state=True)
        assert cache.data_ptr() == ptr
        assert torch.allclose(yt[:, 0], full[:, t], atol=1e-5)
    want = O.causal_conv1d_ref(x.cpu().double(), conv.weight.squeeze(1).cpu().double(), conv.bias.cpu().double(), None, None, 'silu')[0]
    O.assert_close('module vs oracle', want.float(), full.cpu(), 1e-4)
    with pytest.raises(ValueError):
        conv(x, mask=torch.ones(B, T + 3, device=dev), cu_seqlens=torch.tensor([0, 1], device=dev))


@pytest.mark.parametrize('dtype,tol', [(torch.float32, 1e-4), (torch.bfloat16, 5e-3), (torch.float16, 2e-3)])
@pytest.mark.parametrize('D,act,affine', [(128, 'swish', True), (64, 'sigmoid', False), (256, 'silu', True), (512, 'swish', True)])
def test_rms_norm_gated(dtype, tol, D, act, affine):
    from b200gdn.modules import FusedRMSNormGated
    dev = 'cuda'
    B, T, H = 2, 300, 3
    gen = torch.Generator().manual_seed(7)
    x = torch.randn(B, T, H, D, generator=gen).to(dtype)
    g = torch.randn(B, T, H, D, generator=gen).to(dtype)
    dy = torch.randn(B, T, H, D, generator=gen).to(dtype)
    w = torch.randn(D, generator=gen) if affine else None
    norm = FusedRMSNormGated(D, elementwise_affine=affine, eps=1e-5, activation=act, device=dev)
    if affine:
        norm.weight.data.copy_(w)
    xr, gr = x.double().requires_grad_(True), g.double().requires_grad_(True)
    wr = w.double().requires_grad_(True) if affine else None
    ry = O.rms_norm_gated_ref(xr, gr, wr, None, act, 1e-5)
    (ry * dy.double()).sum().backward()
    xg, gg = x.to(dev).requires_grad_(True), g.to(dev).requires_grad_(True)
    y = norm(xg, gg)
    y.backward(dy.to(dev))
    assert y.dtype == dtype and y.shape == x.shape
    O.assert_close('y', ry.float(), y.float().cpu(), tol)
    O.assert_close('dx', xr.grad.float(), xg.grad.float().cpu(), tol)
    O.assert_close('dg', gr.grad.float(), gg.grad.float().cpu(), tol)
    if affine:
        O.assert_close('dw', wr.grad.float(), norm.weight.grad.float().cpu(), tol * 2)


def test_module_errors():
    from b200gdn import B200GDNError
    from b200gdn.modules import causal_conv1d, rms_norm_gated
    x = torch.zeros(1, 8, 16, device='cuda')
    with pytest.raises(ValueError, match='not supported'):
        causal_conv1d(x, torch.zeros(16, 4, device='cuda'), activation='gelu')
    with pytest.raises(B200GDNError, match='kernel size'):
        causal_conv1d(x, torch.zeros(16, 5, device='cuda'))
    with pytest.raises(NotImplementedError):
        rms_norm_gated(x, x, None, residual=x)
    with pytest.raises(B200GDNError, match='are built'):
        rms_norm_gated(torch.zeros(4, 96, device='cuda'), torch.zeros(4, 96, device='cuda'), None)
