"""The CPU oracle against the golden fixtures generated from the reference itself
(tests/golden/make_golden.py) and against its own ground truth."""
import os

import numpy as np
import pytest
import torch

from oracle import gdn_oracle as O
from tests.golden.make_golden import CASES

GOLD = os.path.join(os.path.dirname(__file__), 'golden')


def _load(name):
    return {k: torch.from_numpy(v) for k, v in np.load(os.path.join(GOLD, name + '.npz')).items()}


def _flat(x):
    return x.reshape(x.shape[0] * x.shape[1], *x.shape[2:])


@pytest.mark.parametrize('name', list(CASES))
def test_naive_matches_reference_fixture(name):
    B, T, H, HV, K, V, cu, seed, with_grads = CASES[name]
    gold = _load(name)
    d = O.make_inputs(B, T, H, HV, K, V, seed=seed, cu_seqlens=cu)
    o, ht = O.naive_recurrent(d['q'], d['k'], d['v'], d['g'], d['beta'], K ** -0.5, d['h0'], True, cu)
    if name == 'config1_naive_cpu':
        o = o[:, ::8]
    # <= 1e-5 against the reference's naive recurrence in fp32
    assert O.err_ratio(gold['o'], o) < 1e-5
    assert O.err_ratio(gold['ht'], ht) < 1e-5
    # the reference's own chunked torch form agrees with its recurrence to the same level
    assert O.err_ratio(gold['o'], gold['o_chunk']) < 1e-5


@pytest.mark.parametrize('name', [n for n in CASES if CASES[n][-1]])
@pytest.mark.parametrize('dtype', [torch.float32, torch.float64])
def test_stage_chain_matches_reference_fixture(name, dtype):
    """Forward and explicit backward stage math (the math the CUDA kernels transcribe)
    against the reference's outputs and autograd gradients."""
    B, T, H, HV, K, V, cu, seed, _ = CASES[name]
    gold = _load(name)
    d = O.make_inputs(B, T, H, HV, K, V, seed=seed, cu_seqlens=cu)
    bounds = O.seq_bounds(B, T, cu)
    q, k, v, g, beta, do = (_flat(d[n]).to(dtype) for n in ('q', 'k', 'v', 'g', 'beta', 'do'))
    h0, dht = d['h0'].to(dtype), d['dht'].to(dtype)
    scale = K ** -0.5
    fwd = O.chunk_fwd(q, k, v, g, beta, scale, h0, bounds)
    bwd = O.chunk_bwd(q, k, v, g, beta, scale, h0, do, dht, bounds, fwd=fwd)
    tol = 2e-5 if dtype == torch.float32 else 1e-5
    assert O.err_ratio(_flat(gold['o']), fwd['o']) < tol
    assert O.err_ratio(gold['ht'], fwd['ht']) < tol
    for gname, oname in (('dq', 'dq'), ('dk', 'dk'), ('dv', 'dv'), ('dbeta', 'dbeta'), ('dg', 'dg')):
        assert O.err_ratio(_flat(gold[gname]), bwd[oname]) < 5 * tol, gname
    assert O.err_ratio(gold['dh0'], bwd['dh0']) < 5 * tol


def test_stage_chain_bf16_emulation_within_reference_tolerance():
    """With the reference's bf16 rounding points emulated the chain stays inside the tolerances the
    reference's own tests use (tests/ops/test_gdn.py:108-200: 0.005 / 0.008 / 0.02)."""
    B, T, H, HV, K, V = 1, 256, 2, 2, 64, 64
    d = O.make_inputs(B, T, H, HV, K, V, seed=11)
    bounds = O.seq_bounds(B, T, None)
    rb = lambda x: x.to(torch.bfloat16).float()
    q, k, v, do = (_flat(rb(d[n])) for n in ('q', 'k', 'v', 'do'))
    g, beta = _flat(d['g']), _flat(d['beta'])
    scale = K ** -0.5
    o, ht, gr = O.naive_with_grads(rb(d['q']), rb(d['k']), rb(d['v']), d['g'], d['beta'], scale, d['h0'],
                                   rb(d['do']), d['dht'])
    fwd = O.chunk_fwd(q, k, v, g, beta, scale, d['h0'], bounds, emulate_bf16=True)
    bwd = O.chunk_bwd(q, k, v, g, beta, scale, d['h0'], do, d['dht'], bounds, fwd=fwd, emulate_bf16=True)
    assert O.err_ratio(_flat(o), fwd['o']) < 0.005
    assert O.err_ratio(ht, fwd['ht']) < 0.005
    for n in ('dq', 'dk', 'dv'):
        assert O.err_ratio(_flat(gr[n]), bwd[n]) < 0.008, n
    for n in ('dg', 'dbeta'):
        assert O.err_ratio(_flat(gr[n]), bwd[n]) < 0.02, n
    assert O.err_ratio(gr['dh0'], bwd['dh0']) < 0.008


def test_gate_fixture():
    gold = _load('gate')
    assert torch.allclose(O.gdn_gate(gold['g'], gold['A_log'], gold['dt_bias']), gold['out'], atol=1e-6, rtol=1e-6)
    assert torch.allclose(O.gdn_gate(gold['g'], gold['A_log'], None), gold['out_nobias'], atol=1e-6, rtol=1e-6)


def test_recurrent_options_equal_preprocessing():
    """In-kernel options == the same op on pre-processed inputs (tests/ops/test_gdn.py:451-709)."""
    gen = torch.Generator().manual_seed(5)
    B, T, H, HV, K, V = 2, 5, 2, 4, 16, 8
    q = torch.randn(B, T, H, K, generator=gen)
    k = torch.randn(B, T, H, K, generator=gen)
    v = torch.randn(B, T, HV, V, generator=gen)
    graw = torch.randn(B, T, HV, generator=gen)
    braw = torch.randn(B, T, HV, generator=gen)
    A_log = torch.randn(HV, generator=gen) * 0.1
    dt_bias = torch.randn(HV, generator=gen) * 0.1
    h0 = torch.randn(B, HV, V, K, generator=gen)
    o1, s1 = O.recurrent_step_options(q, k, v, graw, braw, None, h0, True, True, True, A_log, dt_bias, True, True, True)
    o2, s2 = O.naive_recurrent(O.l2norm(q), O.l2norm(k), v, O.gdn_gate(graw, A_log, dt_bias),
                               2 * torch.sigmoid(braw), None, h0.transpose(-1, -2), True)
    assert torch.allclose(o1, o2, atol=1e-6)
    assert torch.allclose(s1, s2.transpose(-1, -2), atol=1e-6)


def test_metric():
    a = torch.tensor([1.0, 2.0, 3.0])
    assert O.err_ratio(a, a) == 0.0
    assert abs(O.err_ratio(a, a * 1.01) - 0.01) < 1e-6
    O.assert_close('x', a, a + 1e-7, 1e-9)
    with pytest.raises(AssertionError):
        O.assert_close('x', a, a * 1.1, 0.01)


@pytest.mark.parametrize('name', ['triton_d128_dense', 'triton_d128_varlen_gva', 'triton_d64_dense'])
def test_oracle_against_reference_triton_path(name):
    """The oracle (exact fp32 math on the bf16-rounded inputs) against the outputs and gradients of the reference's
    own Triton chunk path recorded on a B200 (tests/golden/make_triton_golden.py), within the tolerances the
    reference's tests use for that path (tests/ops/test_gdn.py:203-278)."""
    from tests.golden.make_triton_golden import TRITON_CASES
    B, T, H, HV, K, V, cu, seed = TRITON_CASES[name]
    gold = _load(name)
    d = O.make_inputs(B, T, H, HV, K, V, seed=seed, cu_seqlens=cu)
    rb = lambda x: x.to(torch.bfloat16).float()
    o, ht, gr = O.naive_with_grads(rb(d['q']), rb(d['k']), rb(d['v']), d['g'], d['beta'], K ** -0.5, d['h0'],
                                   rb(d['do']), d['dht'], cu_seqlens=cu)
    assert O.err_ratio(o, gold['o']) < 0.005
    assert O.err_ratio(ht, gold['ht']) < 0.005
    for n in ('dq', 'dk', 'dv', 'dh0'):
        assert O.err_ratio(gr[n], gold[n]) < 0.008, n
    for n in ('dg', 'dbeta'):
        assert O.err_ratio(gr[n], gold[n]) < 0.02, n


@pytest.mark.parametrize('name', ['conv_w4_silu', 'conv_w3_plain', 'conv_w2_short'])
def test_conv_oracle_matches_reference_fixture(name):
    """The convolution oracle against the reference's own torch statement (fixtures by tests/golden/make_modules_golden.py):
    outputs, final state and all gradients."""
    from tests.golden.make_modules_golden import CONV_CASES
    B, T, D, W, act, has_bias, has_cache = CONV_CASES[name]
    gold = {k: torch.from_numpy(v) for k, v in np.load(os.path.join(GOLD, name + '.npz')).items()}
    x = gold['x'].clone().requires_grad_(True)
    w = gold['w'].clone().requires_grad_(True)
    b = gold['b'].clone().requires_grad_(True) if has_bias else None
    cache = None
    if has_cache:   # the reference's test cache holds W-1 entries; the operator's cache has W (the oldest is unused)
        c = gold['cache'].clone().requires_grad_(True)
        cache = torch.cat([torch.zeros(B, D, 1, dtype=c.dtype), c], dim=-1)
    y, final = O.causal_conv1d_ref(x, w, b, None, cache, act, None, True)
    (y * gold['dy']).sum().backward()
    assert torch.allclose(y, gold['y'], atol=1e-10)
    assert torch.allclose(final[..., 1:], gold['final'], atol=1e-12)
    assert torch.allclose(x.grad, gold['dx'], atol=1e-10) and torch.allclose(w.grad, gold['dw'], atol=1e-9)
    if has_bias:
        assert torch.allclose(b.grad, gold['db'], atol=1e-9)
    if has_cache:
        assert torch.allclose(c.grad, gold['dcache'], atol=1e-10)


def test_rms_norm_gated_oracle_against_plain_torch():
    """The gated-norm oracle against torch's own rms_norm and activations, as the reference's test builds its
    expectation (tests/modules/test_layernorm_gated.py:82-116)."""
    gen = torch.Generator().manual_seed(3)
    x, g = torch.randn(5, 7, 128, generator=gen, dtype=torch.float64), torch.randn(5, 7, 128, generator=gen, dtype=torch.float64)
    w = torch.randn(128, generator=gen, dtype=torch.float64)
    for act, fn in (('swish', torch.nn.functional.silu), ('sigmoid', torch.sigmoid)):
        want = torch.nn.functional.rms_norm(x, (128,), w, eps=1e-5) * fn(g)
        assert torch.allclose(O.rms_norm_gated_ref(x, g, w, None, act, 1e-5), want, atol=1e-12)
