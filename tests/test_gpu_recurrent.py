"""GPU parity of the decode path against the oracle recurrence (reference tolerance 0.002,
tests/ops/test_gdn.py:48-105; fp32 inputs are held to 1e-5)."""
import pytest
import torch

from oracle import gdn_oracle as O

pytestmark = pytest.mark.gpu


def _inputs(B, T, H, HV, K, V, seed, dtype):
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn(B, T, H, K, generator=gen).to(dtype)
    k = torch.randn(B, T, H, K, generator=gen).to(dtype)
    v = torch.randn(B, T, HV, V, generator=gen).to(dtype)
    graw = torch.randn(B, T, HV, generator=gen)
    braw = torch.randn(B, T, HV, generator=gen)
    A_log = torch.randn(HV, generator=gen) * 0.3
    dt_bias = torch.randn(HV, generator=gen) * 0.3
    return q, k, v, graw, braw, A_log, dt_bias, gen


@pytest.mark.parametrize('K,V', [(128, 128), (64, 64), (32, 64), (256, 128)])
@pytest.mark.parametrize('v_first', [False, True])
@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16])
def test_recurrent_options(K, V, v_first, dtype):
    from b200gdn import fused_recurrent_gated_delta_rule
    B, T, H, HV = 2, 9, 2, 4
    q, k, v, graw, braw, A_log, dt_bias, gen = _inputs(B, T, H, HV, K, V, 1, dtype)
    h0 = torch.randn(B, HV, *((V, K) if v_first else (K, V)), generator=gen) * 0.5
    ref_o, ref_ht = O.recurrent_step_options(
        q.float(), k.float(), v.float(), graw, braw, None, h0, True, True, True, A_log, dt_bias, True, True, v_first)
    dev = 'cuda'
    o, ht = fused_recurrent_gated_delta_rule(
        q.to(dev), k.to(dev), v.to(dev), graw.to(dev), beta=braw.to(dev), initial_state=h0.to(dev),
        output_final_state=True, use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, A_log=A_log.to(dev),
        dt_bias=dt_bias.to(dev), use_beta_sigmoid_in_kernel=True, allow_neg_eigval=True, state_v_first=v_first)
    assert o.dtype == dtype and ht.dtype == torch.float32
    tol = 1e-5 if dtype == torch.float32 else 0.004
    O.assert_close('o', ref_o, o.float().cpu(), tol)
    O.assert_close('ht', ref_ht, ht.cpu(), 1e-5)


def test_recurrent_plain_varlen_and_inplace():
    from b200gdn import fused_recurrent_gated_delta_rule
    H, HV, K, V = 2, 2, 128, 128
    cu = [0, 3, 4, 20, 31]
    T = cu[-1]
    d = O.make_inputs(1, T, H, HV, K, V, seed=2, cu_seqlens=cu, h0_std=0.5)
    ref_o, ref_ht = O.naive_recurrent(d['q'], d['k'], d['v'], d['g'], d['beta'], None, d['h0'], True, cu)
    dev = 'cuda'
    state = d['h0'].to(dev).clone()
    o, ht = fused_recurrent_gated_delta_rule(
        d['q'].to(dev), d['k'].to(dev), d['v'].to(dev), d['g'].to(dev), beta=d['beta'].to(dev), initial_state=state,
        output_final_state=True, cu_seqlens=torch.tensor(cu, device=dev), inplace_state=True)
    assert ht.data_ptr() == state.data_ptr()
    O.assert_close('o', ref_o, o.cpu(), 1e-5)
    O.assert_close('ht', ref_ht, ht.cpu(), 1e-5)
    # no initial state, no final state, beta defaults to ones
    o2, none = fused_recurrent_gated_delta_rule(d['q'].to(dev), d['k'].to(dev), d['v'].to(dev), d['g'].to(dev))
    ref_o2, _ = O.naive_recurrent(d['q'], d['k'], d['v'], d['g'], torch.ones_like(d['beta']), None, None, False)
    assert none is None
    O.assert_close('o2', ref_o2, o2.cpu(), 1e-5)


def test_recurrent_matches_config1_fixture():
    """BASELINE config 1 (B1 T1024 H4 K=V=64 fp32) against the reference's own output."""
    import os
    import numpy as np
    from b200gdn import fused_recurrent_gated_delta_rule
    gold = np.load(os.path.join(os.path.dirname(__file__), 'golden', 'config1_naive_cpu.npz'))
    d = O.make_inputs(1, 1024, 4, 4, 64, 64, seed=0)
    dev = 'cuda'
    o, ht = fused_recurrent_gated_delta_rule(d['q'].to(dev), d['k'].to(dev), d['v'].to(dev), d['g'].to(dev),
                                             beta=d['beta'].to(dev), initial_state=d['h0'].to(dev),
                                             output_final_state=True)
    O.assert_close('o', torch.from_numpy(gold['o']), o.cpu()[:, ::8], 1e-5)
    O.assert_close('ht', torch.from_numpy(gold['ht']), ht.cpu(), 1e-5)


def test_recurrent_errors():
    from b200gdn import fused_recurrent_gated_delta_rule
    dev = 'cuda'
    q = torch.zeros(1, 4, 2, 64, device=dev)
    g = torch.zeros(1, 4, 2, device=dev)
    with pytest.raises(NotImplementedError):
        fused_recurrent_gated_delta_rule(q, q, q, g, gk=q)
    with pytest.raises(ValueError, match='A_log'):
        fused_recurrent_gated_delta_rule(q, q, q, g, use_gate_in_kernel=True)
    o, _ = fused_recurrent_gated_delta_rule(q.requires_grad_(True), q, q, g)
    with pytest.raises(NotImplementedError):
        o.sum().backward()


@pytest.mark.parametrize('B', [1, 16, 256])
def test_decode_sweep_single_token_steps(B):
    """Decode sweep of the long-context configuration: single-token steps at batch 1..256 with a
    [B,16,128,128] fp32 state, three consecutive steps with the state carried in place; checked against
    the delta-rule update written out in plain fp32 torch on the same device."""
    from b200gdn import fused_recurrent_gated_delta_rule
    dev = 'cuda'
    H, K, V = 16, 128, 128
    gen = torch.Generator(device=dev).manual_seed(B)
    state = torch.randn(B, H, K, V, device=dev, generator=gen) * 0.1
    ref = state.clone()
    scale = K ** -0.5
    for step in range(3):
        q = torch.nn.functional.normalize(torch.randn(B, 1, H, K, device=dev, generator=gen), dim=-1)
        k = torch.nn.functional.normalize(torch.randn(B, 1, H, K, device=dev, generator=gen), dim=-1)
        v = torch.randn(B, 1, H, V, device=dev, generator=gen)
        g = torch.nn.functional.logsigmoid(torch.randn(B, 1, H, device=dev, generator=gen))
        beta = torch.sigmoid(torch.randn(B, 1, H, device=dev, generator=gen))
        o, ht = fused_recurrent_gated_delta_rule(q, k, v, g, beta=beta, initial_state=state, output_final_state=True,
                                                 inplace_state=True)
        assert ht.data_ptr() == state.data_ptr()
        # S <- S e^g ; u = beta (v - S^T k) ; S <- S + k u^T ; o = scale S^T q      (fla/ops/gated_delta_rule/naive.py:41-60)
        ref = ref * g[:, 0, :, None, None].exp()
        u = (v[:, 0] - torch.einsum('bhkv,bhk->bhv', ref, k[:, 0])) * beta[:, 0, :, None]
        ref = ref + torch.einsum('bhk,bhv->bhkv', k[:, 0], u)
        o_ref = torch.einsum('bhkv,bhk->bhv', ref, q[:, 0]) * scale
        O.assert_close(f'o step {step}', o_ref.cpu(), o[:, 0].cpu(), 1e-5)
        O.assert_close(f'state step {step}', ref.cpu(), state.cpu(), 1e-5)


def test_decode_step_in_cuda_graph():
    """The decode step only enqueues work on the caller's stream, so a serving loop can capture it in a CUDA graph
    (static input buffers, state updated in place) and replay it; replays must reproduce the eager steps."""
    from b200gdn import fused_recurrent_gated_delta_rule
    dev = 'cuda'
    B, H, K, V = 8, 16, 128, 128
    gen = torch.Generator(device=dev).manual_seed(5)
    mk = lambda *s: torch.randn(*s, device=dev, generator=gen)
    steps = [dict(q=torch.nn.functional.normalize(mk(B, 1, H, K), dim=-1), k=torch.nn.functional.normalize(mk(B, 1, H, K), dim=-1),
                  v=mk(B, 1, H, V), g=torch.nn.functional.logsigmoid(mk(B, 1, H)), beta=torch.sigmoid(mk(B, 1, H)))
             for _ in range(4)]
    state0 = mk(B, H, K, V) * 0.1
    # eager
    s_e = state0.clone()
    outs_e = []
    for st in steps:
        o, _ = fused_recurrent_gated_delta_rule(st['q'], st['k'], st['v'], st['g'], beta=st['beta'], initial_state=s_e,
                                                output_final_state=True, inplace_state=True)
        outs_e.append(o.clone())
    # captured once, replayed per step
    buf = {n: torch.empty_like(x) for n, x in steps[0].items()}
    s_g = state0.clone()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):   # warm-up outside the capture (library load, first launch)
        for n in buf:
            buf[n].copy_(steps[0][n])
        fused_recurrent_gated_delta_rule(buf['q'], buf['k'], buf['v'], buf['g'], beta=buf['beta'], initial_state=s_g.clone(),
                                         output_final_state=True, inplace_state=True)
    torch.cuda.current_stream().wait_stream(side)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        o_g, _ = fused_recurrent_gated_delta_rule(buf['q'], buf['k'], buf['v'], buf['g'], beta=buf['beta'], initial_state=s_g,
                                                  output_final_state=True, inplace_state=True)
    s_g.copy_(state0)
    for i, st in enumerate(steps):
        for n in buf:
            buf[n].copy_(st[n])
        graph.replay()
        assert torch.equal(o_g, outs_e[i]), f'step {i}'
    assert torch.equal(s_g, s_e)


@pytest.mark.parametrize('K', [128, 64])
@pytest.mark.parametrize('T', [1, 3])
@pytest.mark.parametrize('dtype', [torch.float32, torch.bfloat16, torch.float16])
def test_large_batch_kernels_with_options(K, T, dtype):
    """Enough (sequence, head) pairs for the large-batch kernels: T = 1 takes the streaming kernel (bulk-copy ring,
    persistent CTAs), T = 3 the whole-state kernel; both with every in-kernel option on, grouped value heads, and the
    state out of place, against the oracle recurrence."""
    from b200gdn import fused_recurrent_gated_delta_rule
    B, H, HV, V = 40, 4, 8, 128     # 320 (sequence, head) pairs
    q, k, v, graw, braw, A_log, dt_bias, gen = _inputs(B, T, H, HV, K, V, 3, dtype)
    h0 = torch.randn(B, HV, K, V, generator=gen) * 0.5
    ref_o, ref_ht = O.recurrent_step_options(
        q.float(), k.float(), v.float(), graw, braw, None, h0, True, True, True, A_log, dt_bias, True, True, False)
    dev = 'cuda'
    o, ht = fused_recurrent_gated_delta_rule(
        q.to(dev), k.to(dev), v.to(dev), graw.to(dev), beta=braw.to(dev), initial_state=h0.to(dev),
        output_final_state=True, use_qk_l2norm_in_kernel=True, use_gate_in_kernel=True, A_log=A_log.to(dev),
        dt_bias=dt_bias.to(dev), use_beta_sigmoid_in_kernel=True, allow_neg_eigval=True)
    assert o.dtype == dtype and ht.dtype == torch.float32
    tol = 1e-5 if dtype == torch.float32 else 0.004
    O.assert_close('o', ref_o, o.float().cpu(), tol)
    O.assert_close('ht', ref_ht, ht.cpu(), 1e-5)
    import b200gdn
    b200gdn.device_status()


@pytest.mark.parametrize('B,T', [(40, 1), (40, 2), (6, 1)])
def test_state_pool_addressed_by_indices(B, T):
    """`state_indices`: the state lives in a pool of slots (a serving engine's cache); each sequence reads and
    updates its slot in place.  Must equal gather -> plain call -> scatter, bit for bit, and leave other slots alone.
    (B = 40 exercises the streaming and the whole-state kernels, B = 6 the sliced kernel.)"""
    from b200gdn import fused_recurrent_gated_delta_rule
    dev = 'cuda'
    H, HV, K, V, P = 4, 8, 128, 128, 64
    gen = torch.Generator(device=dev).manual_seed(B * 10 + T)
    mk = lambda *s: torch.randn(*s, device=dev, generator=gen)
    q, k = torch.nn.functional.normalize(mk(B, T, H, K), dim=-1), torch.nn.functional.normalize(mk(B, T, H, K), dim=-1)
    v, g, beta = mk(B, T, HV, V), torch.nn.functional.logsigmoid(mk(B, T, HV)), torch.sigmoid(mk(B, T, HV))
    pool = mk(P, HV, K, V) * 0.3
    idx = torch.randperm(P, device=dev, generator=gen)[:B]
    o_ref, ht_ref = fused_recurrent_gated_delta_rule(q, k, v, g, beta=beta, initial_state=pool[idx].contiguous(),
                                                     output_final_state=True)
    want = pool.clone()
    want[idx] = ht_ref
    o, out_pool = fused_recurrent_gated_delta_rule(q, k, v, g, beta=beta, initial_state=pool, state_indices=idx)
    assert out_pool.data_ptr() == pool.data_ptr()
    assert torch.equal(o, o_ref)
    assert torch.equal(pool, want)
