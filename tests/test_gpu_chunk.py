"""GPU parity of the chunk path: every stage through the C ABI against the oracle's stage, then the
public API against the naive recurrence with the reference's own tolerances
(tests/ops/test_gdn.py:108-200: o/ht 0.005, dq/dk/dv/dh0 0.008, dbeta/dg 0.02)."""
import ctypes
import os

import numpy as np
import pytest
import torch

from oracle import gdn_oracle as O
from tests.golden.make_golden import CASES
from tests.gpu_util import flat, make_case, oracle_chain, run_abi

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), 'golden')

STAGE_CASES = {
    'd64_dense': dict(B=2, T=128, H=2, HV=2, K=64, V=64),
    'd128_dense': dict(B=2, T=256, H=2, HV=2, K=128, V=128),
    'd128_gva': dict(B=1, T=192, H=2, HV=4, K=128, V=128),
    'd128_ragged': dict(B=1, T=333, H=1, HV=2, K=128, V=128, cu=[0, 1, 16, 80, 143, 270, 333]),
    'd64_ragged_gva': dict(B=1, T=300, H=2, HV=4, K=64, V=64, cu=[0, 37, 101, 165, 300]),
    'd128_nh0': dict(B=1, T=100, H=2, HV=2, K=128, V=128, with_h0=False),
    'd128_group4': dict(B=2, T=130, H=1, HV=4, K=128, V=128),
}

# err-ratio bounds per tensor (bf16 storage: eps = 2^-8 = 0.0039 per rounding)
FWD_TOL = dict(gamma=1e-5, A=0.005, qk=0.005, w=0.005, u=0.005, h=0.005, v_new=0.005, ht=0.005, o=0.005)
BWD_TOL = dict(dh=0.008, dh0=0.008, dv2=0.008, dq=0.008, dk=0.008, dv=0.008, dbeta=0.02, dg=0.02)


@pytest.mark.parametrize('name', list(STAGE_CASES))
def test_stages_against_oracle(name):
    d = make_case(seed=3, **STAGE_CASES[name])
    fwd, bwd = oracle_chain(d)
    out = run_abi(d)
    for n, tol in FWD_TOL.items():
        O.assert_close(f'{name}:{n}', fwd[n], out[n], tol)
    if d['h0'] is None:
        BWD = {k: v for k, v in BWD_TOL.items() if k != 'dh0'}
    else:
        BWD = BWD_TOL
    for n, tol in BWD.items():
        O.assert_close(f'{name}:{n}', bwd[n], out[n], tol)


@pytest.mark.parametrize('name', ['d128_dense', 'd64_ragged_gva'])
def test_backward_stages_isolated(name):
    """Each backward kernel alone, fed with the oracle's inputs for that stage."""
    from b200gdn import _lib
    d = make_case(seed=5, **STAGE_CASES[name])
    fwd, bwd = oracle_chain(d)
    saved = {n: fwd[n] for n in ('gamma', 'A', 'qk', 'w', 'h', 'v_new')}
    o1 = run_abi(d, fwd_mask=-1, bwd_mask=_lib.BWD_DVLOCAL, overrides=dict(saved))
    O.assert_close('dv_local', bwd['dv_local'], o1['dv2'], 0.005)
    o2 = run_abi(d, fwd_mask=-1, bwd_mask=_lib.BWD_SCAN, overrides=dict(saved, dv2=bwd['dv_local']))
    for n in ('dh', 'dh0', 'dv2'):
        O.assert_close(n, bwd[n], o2[n], 0.005)
    # the same two stages in one kernel (dv_local formed inside the reverse scan from the forward pass's qk tile)
    o2f = run_abi(d, fwd_mask=-1, bwd_mask=_lib.BWD_DVLOCAL | _lib.BWD_SCAN, overrides=dict(saved))
    for n in ('dh', 'dh0', 'dv2'):
        O.assert_close(n + ' (fused scan)', bwd[n], o2f[n], 0.005)
    o3 = run_abi(d, fwd_mask=-1, bwd_mask=_lib.BWD_DQKWG, overrides=dict(saved, dv2=bwd['dv2'], dh=bwd['dh']))
    # after this stage the dk buffer holds the chunk-local part of dk (bf16), to which the WY stage adds in place
    for n, m in (('dq', 'dq'), ('dk', 'dk_part'), ('dG', 'dG')):
        O.assert_close(n, bwd[m], o3[n], 0.005)
    o4 = run_abi(d, fwd_mask=-1, bwd_mask=_lib.BWD_WY,
                 overrides=dict(saved, dv2=bwd['dv2'], dk=bwd['dk_part'], dG=bwd['dG']))
    for n in ('dk', 'dv', 'dbeta', 'dg'):
        O.assert_close(n, bwd[n], o4[n], 0.005)


@pytest.mark.parametrize('name', [n for n in CASES if CASES[n][-1]])
def test_public_api_against_reference_fixture(name):
    """chunk_gated_delta_rule + autograd against the reference's own outputs and gradients."""
    from b200gdn import chunk_gated_delta_rule
    B, T, H, HV, K, V, cu, seed, _ = CASES[name]
    gold = {k: torch.from_numpy(v) for k, v in np.load(os.path.join(GOLD, name + '.npz')).items()}
    d = O.make_inputs(B, T, H, HV, K, V, seed=seed, cu_seqlens=cu)
    dev = 'cuda'
    q, k, v = (d[n].to(dev).to(torch.bfloat16).requires_grad_(True) for n in ('q', 'k', 'v'))
    g, beta, h0 = (d[n].to(dev).requires_grad_(True) for n in ('g', 'beta', 'h0'))
    cu_t = None if cu is None else torch.tensor(cu, dtype=torch.long, device=dev)
    o, ht = chunk_gated_delta_rule(q, k, v, g, beta, initial_state=h0, output_final_state=True, cu_seqlens=cu_t)
    ((o.float() * d['do'].to(dev)).sum() + (ht * d['dht'].to(dev)).sum()).backward()
    assert o.dtype == torch.bfloat16 and ht.dtype == torch.float32
    O.assert_close('o', gold['o'], o.float().cpu(), 0.005)
    O.assert_close('ht', gold['ht'], ht.cpu(), 0.005)
    O.assert_close('dq', gold['dq'], q.grad.float().cpu(), 0.008)
    O.assert_close('dk', gold['dk'], k.grad.float().cpu(), 0.008)
    O.assert_close('dv', gold['dv'], v.grad.float().cpu(), 0.008)
    O.assert_close('dh0', gold['dh0'], h0.grad.cpu(), 0.008)
    O.assert_close('dbeta', gold['dbeta'], beta.grad.cpu(), 0.02)
    O.assert_close('dg', gold['dg'], g.grad.cpu(), 0.02)


@pytest.mark.parametrize('HV', [4, 2])
def test_options_equal_preprocessing(HV):
    """In-kernel options == the op on pre-processed inputs (tests/ops/test_gdn.py:281-448, 881-1190); grouped value
    heads (HV = 4 over H = 2) and one value head per q/k head: the L2 norm's backward is applied where dq and dk are
    completed, which the two cases do in different code paths."""
    from b200gdn import chunk_gated_delta_rule
    dev = 'cuda'
    B, T, H, K, V = 2, 150, 2, 128, 128
    gen = torch.Generator().manual_seed(9)
    q = torch.randn(B, T, H, K, generator=gen).to(dev).to(torch.bfloat16)
    k = torch.randn(B, T, H, K, generator=gen).to(dev).to(torch.bfloat16)
    v = torch.randn(B, T, HV, V, generator=gen).to(dev).to(torch.bfloat16)
    graw = torch.randn(B, T, HV, generator=gen).to(dev)
    braw = torch.randn(B, T, HV, generator=gen).to(dev)
    A_log = (torch.randn(HV, generator=gen) * 0.3).to(dev)
    dt_bias = (torch.randn(HV, generator=gen) * 0.3).to(dev)
    h0 = (torch.randn(B, HV, V, K, generator=gen) * 0.1).to(dev)

    def run(in_kernel):
        leaves = [x.clone().requires_grad_(True) for x in (q, k, v, graw, braw, A_log, dt_bias, h0)]
        q_, k_, v_, g_, b_, A_, dt_, h0_ = leaves
        if in_kernel:
            o, ht = chunk_gated_delta_rule(q_, k_, v_, g_, b_, initial_state=h0_, output_final_state=True,
                                           use_qk_l2norm_in_kernel=True, use_beta_sigmoid_in_kernel=True,
                                           allow_neg_eigval=True, state_v_first=True, use_gate_in_kernel=True,
                                           A_log=A_, dt_bias=dt_, chunk_size=32)
        else:
            qn = O.l2norm(q_.float()).to(torch.bfloat16)
            kn = O.l2norm(k_.float()).to(torch.bfloat16)
            o, ht = chunk_gated_delta_rule(qn, kn, v_, O.gdn_gate(g_, A_, dt_), 2 * torch.sigmoid(b_),
                                           initial_state=h0_.transpose(-1, -2), output_final_state=True)
            ht = ht.transpose(-1, -2)
        (o.float().square().sum() + ht.square().sum()).backward()
        return [o.float(), ht] + [x.grad.float() for x in leaves]
    a, b = run(True), run(False)
    # the two sides round the normalised q / k to bf16 from fp32 values that differ in the last bit here and there
    # (1/sqrt in the kernel as in the reference's l2norm kernel, rsqrt in torch): a flipped bf16 ulp is 4e-3 relative.
    for i, (x, y) in enumerate(zip(a, b)):
        if i not in (2, 3):
            O.assert_close(f'option-equivalence[{i}]', y.cpu(), x.cpu(), 1e-3)
    # dq / dk (results 2, 3).  The kernels apply the norm's backward (dy - y <dy,y>) rstd from the fp32 dy with y the
    # bf16-normalised tensor; the route above does it in torch from the bf16-rounded dy with y in fp32.  With this loss
    # the final-state gradient makes dk of the last rows almost parallel to k (component along k 40 times the rest), the
    # projection cancels it, and what is left is dominated by bf16 rounding on either route: both are held to the fp64
    # recurrence with the options inside the graph, and the kernels' route must be at least as close to it as torch's
    # (or within the tolerance the reference holds this option to, tests/ops/test_gdn.py:225-280)
    G = HV // H
    q64, k64 = q.cpu().double().requires_grad_(True), k.cpu().double().requires_grad_(True)
    o64, ht64 = O.naive_recurrent(O.l2norm(q64).repeat_interleave(G, 2), O.l2norm(k64).repeat_interleave(G, 2), v.cpu().double(),
                                  O.gdn_gate(graw.cpu().double(), A_log.cpu().double(), dt_bias.cpu().double()),
                                  2 * torch.sigmoid(braw.cpu().double()), scale=K ** -0.5,
                                  initial_state=h0.cpu().double().transpose(-1, -2), output_final_state=True, dtype=torch.float64)
    (o64.square().sum() + ht64.square().sum()).backward()
    for i, ref in ((2, q64.grad), (3, k64.grad)):
        e_kernel, e_torch = O.err_ratio(ref.float(), a[i].cpu()), O.err_ratio(ref.float(), b[i].cpu())
        assert e_kernel <= max(0.005, 1.1 * e_torch), f'option-equivalence[{i}]: {e_kernel} vs oracle, torch route {e_torch}'


@pytest.mark.parametrize('HV,dht_scale', [(2, 0.1), (2, 30.0), (4, 30.0)])
def test_l2norm_option_against_the_oracle(HV, dht_scale):
    """use_qk_l2norm_in_kernel: dq and dk (the norm's backward is applied where the kernels complete them) against the
    fp64 recurrence with the norm inside the graph, with one value head per q/k head and with grouped heads, and with a
    final-state gradient large enough to dominate the last rows (where dk is nearly parallel to k and the projection
    cancels most of it).  The north star's tolerance for dq / dk; the route through pre-normalised inputs is held to
    the same, as a yardstick."""
    from b200gdn import chunk_gated_delta_rule
    dev = 'cuda'
    B, T, H, K, V = 2, 150, 2, 128, 128
    gen = torch.Generator().manual_seed(9)
    q = torch.randn(B, T, H, K, generator=gen).to(torch.bfloat16)
    k = torch.randn(B, T, H, K, generator=gen).to(torch.bfloat16)
    v = torch.randn(B, T, HV, V, generator=gen).to(torch.bfloat16)
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, HV, generator=gen))
    b = torch.sigmoid(torch.randn(B, T, HV, generator=gen))
    do = torch.randn(B, T, HV, V, generator=gen).to(torch.bfloat16)
    dht = torch.randn(B, HV, K, V, generator=gen) * dht_scale

    def run(in_kernel):
        q_, k_ = (x.to(dev).clone().requires_grad_(True) for x in (q, k))
        if in_kernel:
            o, ht = chunk_gated_delta_rule(q_, k_, v.to(dev), g.to(dev), b.to(dev), output_final_state=True,
                                           use_qk_l2norm_in_kernel=True)
        else:
            o, ht = chunk_gated_delta_rule(O.l2norm(q_.float()).to(torch.bfloat16), O.l2norm(k_.float()).to(torch.bfloat16),
                                           v.to(dev), g.to(dev), b.to(dev), output_final_state=True)
        torch.autograd.backward([o, ht], [do.to(dev), dht.to(dev)])
        return q_.grad.float().cpu(), k_.grad.float().cpu()
    fused, pre = run(True), run(False)
    q64, k64 = q.double().requires_grad_(True), k.double().requires_grad_(True)
    G = HV // H
    o, ht = O.naive_recurrent(O.l2norm(q64).repeat_interleave(G, 2), O.l2norm(k64).repeat_interleave(G, 2), v.double(),
                              g.double(), b.double(), scale=K ** -0.5, initial_state=None, output_final_state=True,
                              dtype=torch.float64)
    ((o * do.double()).sum() + (ht * dht.double()).sum()).backward()
    for name, ref, got, yard in (('dq', q64.grad, fused[0], pre[0]), ('dk', k64.grad, fused[1], pre[1])):
        O.assert_close(f'{name} fused norm backward vs oracle', ref.float(), got, 0.008)
        O.assert_close(f'{name} pre-normalised route vs oracle', ref.float(), yard, 0.008)
        O.assert_close(f'{name} last rows, fused vs oracle', ref[:, -3:].float(), got[:, -3:], 0.008)


def test_api_errors():
    from b200gdn import chunk_gated_delta_rule
    dev = 'cuda'
    q = torch.zeros(2, 64, 2, 128, device=dev, dtype=torch.bfloat16)
    v = torch.zeros(2, 64, 3, 128, device=dev, dtype=torch.bfloat16)
    g = torch.zeros(2, 64, 3, device=dev)
    with pytest.raises(ValueError, match='evenly divisible'):
        chunk_gated_delta_rule(q, q, v, g, g)
    v = torch.zeros(2, 64, 2, 128, device=dev, dtype=torch.bfloat16)
    g = torch.zeros(2, 64, 2, device=dev)
    with pytest.raises(ValueError, match='batch size is expected to be 1'):
        chunk_gated_delta_rule(q, q, v, g, g, cu_seqlens=torch.tensor([0, 64, 128], device=dev))
    with pytest.raises(DeprecationWarning):
        chunk_gated_delta_rule(q, q, v, g, g, head_first=True)
    with pytest.raises(ValueError, match='chunk_size'):
        chunk_gated_delta_rule(q, q, v, g, g, chunk_size=128)
    with pytest.raises(ValueError, match='allow_neg_eigval'):
        chunk_gated_delta_rule(q, q, v, g, g, allow_neg_eigval=True)


def test_determinism_and_no_uninitialised_reads():
    """Two runs are bit-identical (no atomics anywhere), and outputs never contain the NaN the buffers
    were poisoned with (the reference's NaN-poison fixture, tests/conftest.py:135-148)."""
    d = make_case(seed=7, **STAGE_CASES['d128_ragged'])
    a = run_abi(d)
    b = run_abi(d)
    for n in ('o', 'ht', 'dq', 'dk', 'dv', 'dg', 'dbeta', 'dh0'):
        assert not torch.isnan(a[n]).any(), n
        assert torch.equal(a[n], b[n]), n
    # none of the bounded device waits (mbarriers of TMA copies and tensor-core commits) expired
    import b200gdn
    b200gdn.device_status()


def test_full_size_properties():
    """Headline shape (B4 T4096 H16 K=V=128): the oracle is too slow here, so check properties:
    chunk path == token-by-token kernel (an independent implementation), and linearity in v."""
    from b200gdn import chunk_gated_delta_rule, fused_recurrent_gated_delta_rule
    dev = 'cuda'
    B, T, H, K = 4, 4096, 16, 128
    gen = torch.Generator(device=dev).manual_seed(0)
    q = torch.nn.functional.normalize(torch.randn(B, T, H, K, device=dev, generator=gen), dim=-1).to(torch.bfloat16)
    k = torch.nn.functional.normalize(torch.randn(B, T, H, K, device=dev, generator=gen), dim=-1).to(torch.bfloat16)
    v1 = torch.randn(B, T, H, K, device=dev, generator=gen).to(torch.bfloat16)
    v2 = torch.randn(B, T, H, K, device=dev, generator=gen).to(torch.bfloat16)
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, H, device=dev, generator=gen))
    beta = torch.sigmoid(torch.randn(B, T, H, device=dev, generator=gen))
    h0 = torch.randn(B, H, K, K, device=dev, generator=gen) * 0.1
    o_c, ht_c = chunk_gated_delta_rule(q, k, v1, g, beta, initial_state=h0, output_final_state=True)
    o_r, ht_r = fused_recurrent_gated_delta_rule(q, k, v1, g, beta=beta, initial_state=h0, output_final_state=True)
    O.assert_close('o chunk vs recurrent', o_r.float().cpu(), o_c.float().cpu(), 0.005)
    O.assert_close('ht chunk vs recurrent', ht_r.cpu(), ht_c.cpu(), 0.005)
    o1, _ = chunk_gated_delta_rule(q, k, v1, g, beta)
    o2, _ = chunk_gated_delta_rule(q, k, v2, g, beta)
    o12, _ = chunk_gated_delta_rule(q, k, (v1.float() + v2.float()).to(torch.bfloat16), g, beta)
    O.assert_close('linearity in v', (o1.float() + o2.float()).cpu(), o12.float().cpu(), 0.01)


def _inputs(B, T, H, HV, K, V, seed, dev='cuda'):
    gen = torch.Generator(device=dev).manual_seed(seed)
    q = torch.nn.functional.normalize(torch.randn(B, T, H, K, device=dev, generator=gen), dim=-1).to(torch.bfloat16)
    k = torch.nn.functional.normalize(torch.randn(B, T, H, K, device=dev, generator=gen), dim=-1).to(torch.bfloat16)
    v = torch.randn(B, T, HV, V, device=dev, generator=gen).to(torch.bfloat16)
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, HV, device=dev, generator=gen))
    beta = torch.sigmoid(torch.randn(B, T, HV, device=dev, generator=gen))
    do = torch.randn(B, T, HV, V, device=dev, generator=gen).to(torch.bfloat16)
    return q, k, v, g, beta, do


def _fwd_bwd(q, k, v, g, beta, do, **kw):
    from b200gdn import chunk_gated_delta_rule
    leaves = [x.detach().clone().requires_grad_(True) for x in (q, k, v, g, beta)]
    o, ht = chunk_gated_delta_rule(*leaves, output_final_state=True, **kw)
    o.backward(do)
    return [o, ht] + [x.grad for x in leaves]


def test_full_size_varlen_gva_equals_per_sequence_runs():
    """Packed GVA configuration at full size (16 q/k heads, 32 value heads, K=V=128, 16 sequences with lengths
    in [256, 8192] summing to 65536 tokens): the packed run must reproduce, sequence by sequence, the runs of
    each sequence on its own (outputs, final states and all gradients), and the chunk forward must agree with the
    token-by-token kernel."""
    from b200gdn import fused_recurrent_gated_delta_rule
    rng = np.random.default_rng(0)
    n, total = 16, 65536
    lens = rng.integers(256, 8193, size=n).astype(np.int64)
    lens = np.maximum(256, (lens * (total / lens.sum())).astype(np.int64))
    lens[-1] += total - lens.sum()
    assert lens.min() >= 256 and lens.sum() == total
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device='cuda')
    q, k, v, g, beta, do = _inputs(1, total, 16, 32, 128, 128, seed=3)
    packed = _fwd_bwd(q, k, v, g, beta, do, cu_seqlens=cu)
    o_r, ht_r = fused_recurrent_gated_delta_rule(q, k, v, g, beta=beta, output_final_state=True, cu_seqlens=cu)
    O.assert_close('o chunk vs recurrent', o_r.float().cpu(), packed[0].float().cpu(), 0.005)
    O.assert_close('ht chunk vs recurrent', ht_r.cpu(), packed[1].cpu(), 0.005)
    names = ('o', 'ht', 'dq', 'dk', 'dv', 'dg', 'dbeta')
    for i in (0, 7, 15):   # first, a middle and the last sequence (the others take the same code path)
        s, e = int(cu[i]), int(cu[i + 1])
        alone = _fwd_bwd(q[:, s:e], k[:, s:e], v[:, s:e], g[:, s:e], beta[:, s:e], do[:, s:e])
        for nme, a, p in zip(names, alone, packed):
            ref = p[i:i + 1] if nme == 'ht' else p[:, s:e]
            assert torch.equal(a, ref), f'sequence {i}: {nme} differs between the packed and the single run'


def test_full_size_head_and_batch_shards_are_independent():
    """Training shape B8 T8192 H32 K=V=128: a head shard and a batch shard computed on their own are bit-identical
    to the corresponding slices of the full computation (what lets heads / batch be split over GPUs with no
    communication), and the forward agrees with the token-by-token kernel on a slice."""
    from b200gdn import fused_recurrent_gated_delta_rule
    q, k, v, g, beta, do = _inputs(8, 8192, 32, 32, 128, 128, seed=4)
    full = _fwd_bwd(q, k, v, g, beta, do)
    hs = slice(8, 16)
    part = _fwd_bwd(q[:, :, hs], k[:, :, hs], v[:, :, hs], g[:, :, hs], beta[:, :, hs], do[:, :, hs])
    for nme, a, f in zip(('o', 'ht', 'dq', 'dk', 'dv', 'dg', 'dbeta'), part, full):
        ref = f[:, hs] if nme == 'ht' else f[:, :, hs]
        assert torch.equal(a, ref), f'head shard: {nme}'
    part = _fwd_bwd(q[2:4], k[2:4], v[2:4], g[2:4], beta[2:4], do[2:4])
    for nme, a, f in zip(('o', 'ht', 'dq', 'dk', 'dv', 'dg', 'dbeta'), part, full):
        assert torch.equal(a, f[2:4]), f'batch shard: {nme}'
    o_r, ht_r = fused_recurrent_gated_delta_rule(q[:1, :, :4], k[:1, :, :4], v[:1, :, :4], g[:1, :, :4], beta=beta[:1, :, :4],
                                                 output_final_state=True)
    O.assert_close('o chunk vs recurrent', o_r.float().cpu(), full[0][:1, :, :4].float().cpu(), 0.005)
    O.assert_close('ht chunk vs recurrent', ht_r.cpu(), full[1][:1, :4].cpu(), 0.005)


@pytest.mark.parametrize('qk_dtype,gb_dtype', [(torch.float32, torch.float32), (torch.bfloat16, torch.bfloat16),
                                               (torch.float16, torch.float32)])
def test_layer_option_kernels_against_torch(qk_dtype, gb_dtype):
    """The pre/post pass of the library (L2 norm, gate, beta sigmoid; forward and backward) against the same
    formulas in plain fp32 torch with autograd (fla/modules/l2norm.py:84-144, fla/ops/gated_delta_rule/gate.py:21-46,
    fla/ops/common/gate.py:18-50).  Tolerances: fp32 results 1e-5; results stored in bf16 / fp16 2e-3."""
    from b200gdn import _lib
    from b200gdn.chunk import LayerOptionsFunction
    dev = 'cuda'
    B, T, H, HV, K = 2, 300, 3, 6, 128
    gen = torch.Generator(device=dev).manual_seed(11)
    q = (torch.randn(B, T, H, K, device=dev, generator=gen) * 2).to(qk_dtype)
    k = (torch.randn(B, T, H, K, device=dev, generator=gen) * 0.5).to(qk_dtype)
    g = (torch.randn(B, T, HV, device=dev, generator=gen) * 3).to(gb_dtype)     # both softplus branches
    g[0, 0, 0] = 25.0
    beta = torch.randn(B, T, HV, device=dev, generator=gen).to(gb_dtype)
    A_log = torch.randn(HV, device=dev, generator=gen) * 0.3
    dt_bias = torch.randn(HV, device=dev, generator=gen) * 0.3
    grads = [torch.randn(B, T, H, K, device=dev, generator=gen).to(torch.bfloat16) for _ in range(2)]
    grads += [torch.randn(B, T, HV, device=dev, generator=gen) for _ in range(2)]
    flags = _lib.PREP_L2NORM | _lib.PREP_GATE | _lib.PREP_BETA_SIGMOID | _lib.PREP_NEG_EIGVAL

    leaves = [x.clone().requires_grad_(True) for x in (q, k, g, beta, A_log, dt_bias)]
    outs = LayerOptionsFunction.apply(*leaves, flags)
    torch.autograd.backward(outs, grads)

    ref = [x.clone().float().requires_grad_(True) for x in (q, k, g, beta, A_log, dt_bias)]
    rq, rk, rg, rb, rA, rdt = ref
    r_outs = [rq * torch.rsqrt(rq.square().sum(-1, keepdim=True) + 1e-6),
              rk * torch.rsqrt(rk.square().sum(-1, keepdim=True) + 1e-6),
              -rA.exp() * torch.nn.functional.softplus(rg + rdt), 2 * torch.sigmoid(rb)]
    torch.autograd.backward(r_outs, [x.float() for x in grads])

    assert outs[0].dtype == torch.bfloat16 and outs[2].dtype == torch.float32 and outs[3].dtype == torch.float32
    O.assert_close('qn', r_outs[0].cpu(), outs[0].float().cpu(), 2e-3)
    O.assert_close('kn', r_outs[1].cpu(), outs[1].float().cpu(), 2e-3)
    O.assert_close('g', r_outs[2].cpu(), outs[2].cpu(), 1e-5)
    O.assert_close('beta', r_outs[3].cpu(), outs[3].cpu(), 1e-5)
    lo_qk = 1e-5 if qk_dtype == torch.float32 else 2e-3
    lo_gb = 1e-5 if gb_dtype == torch.float32 else 3e-3
    for name, a, b, tol in (('dq', leaves[0], ref[0], lo_qk), ('dk', leaves[1], ref[1], lo_qk), ('dg', leaves[2], ref[2], lo_gb),
                            ('dbeta', leaves[3], ref[3], lo_gb), ('dA_log', leaves[4], ref[4], 1e-5),
                            ('ddt_bias', leaves[5], ref[5], 1e-5)):
        assert a.grad.dtype == a.dtype, name
        O.assert_close(name, b.grad.cpu(), a.grad.float().cpu(), tol)


def test_chunk_forward_in_cuda_graph():
    """A prefill step (forward only, static buffers) captured in a CUDA graph replays to the eager result: the library
    only enqueues kernels on the caller's stream, and the tensor maps it builds on the host are kernel parameters."""
    from b200gdn import chunk_gated_delta_rule
    q, k, v, g, beta, _ = _inputs(2, 512, 4, 4, 128, 128, seed=6)
    with torch.no_grad():
        o_e, ht_e = chunk_gated_delta_rule(q, k, v, g, beta, output_final_state=True)   # also warms the chunk tables
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            chunk_gated_delta_rule(q, k, v, g, beta, output_final_state=True)
        torch.cuda.current_stream().wait_stream(side)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            o_g, ht_g = chunk_gated_delta_rule(q, k, v, g, beta, output_final_state=True)
        v2 = torch.randn_like(v.float()).to(torch.bfloat16)
        o_e2, ht_e2 = chunk_gated_delta_rule(q, k, v2, g, beta, output_final_state=True)
        graph.replay()
        assert torch.equal(o_g, o_e) and torch.equal(ht_g, ht_e)
        v.copy_(v2)
        graph.replay()
        assert torch.equal(o_g, o_e2) and torch.equal(ht_g, ht_e2)


@pytest.mark.parametrize('name', ['triton_d128_dense', 'triton_d128_varlen_gva', 'triton_d64_dense'])
def test_public_api_against_reference_triton_path(name):
    """Outputs and gradients of the reference's own Triton chunk path on a B200 (tests/golden/make_triton_golden.py)
    on identical seeded inputs; tolerances of the reference's tests (tests/ops/test_gdn.py:203-278: o, ht 0.005;
    dq, dk, dv, dh0 0.008; dbeta, dg 0.02)."""
    from b200gdn import chunk_gated_delta_rule
    from tests.golden.make_triton_golden import TRITON_CASES
    B, T, H, HV, K, V, cu, seed = TRITON_CASES[name]
    gold = np.load(os.path.join(os.path.dirname(__file__), 'golden', name + '.npz'))
    d = O.make_inputs(B, T, H, HV, K, V, seed=seed, cu_seqlens=cu)
    dev = 'cuda'
    leaves = {n: d[n].to(torch.bfloat16).to(dev).requires_grad_(True) for n in ('q', 'k', 'v')}
    leaves.update({n: d[n].float().to(dev).requires_grad_(True) for n in ('g', 'beta', 'h0')})
    cu_t = None if cu is None else torch.tensor(cu, dtype=torch.long, device=dev)
    o, ht = chunk_gated_delta_rule(leaves['q'], leaves['k'], leaves['v'], leaves['g'], leaves['beta'], scale=K ** -0.5,
                                   initial_state=leaves['h0'], output_final_state=True, cu_seqlens=cu_t)
    ((o.float() * d['do'].to(torch.bfloat16).float().to(dev)).sum() + (ht * d['dht'].to(dev)).sum()).backward()
    O.assert_close('o', torch.from_numpy(gold['o']), o.float().cpu(), 0.005)
    O.assert_close('ht', torch.from_numpy(gold['ht']), ht.cpu(), 0.005)
    for n, tol in (('q', 0.008), ('k', 0.008), ('v', 0.008), ('h0', 0.008), ('beta', 0.02), ('g', 0.02)):
        O.assert_close('d' + n, torch.from_numpy(gold['d' + n]), leaves[n].grad.float().cpu(), tol)


def test_wait_expiry_is_reported_and_context_survives():
    """Failure detection without a GPU fault: a kernel whose wait can never complete gives up after its (short)
    limit, the host reads B200GDN_ERR_TIMEOUT, the flag clears, and the context keeps working."""
    import b200gdn
    from b200gdn import _lib
    lib = _lib.load()
    b200gdn.device_status()                                     # clean before
    st = torch.cuda.current_stream().cuda_stream
    assert lib.b200gdn_selftest_wait_expiry(ctypes.c_void_p(st)) == 0
    with pytest.raises(b200gdn.B200GDNError, match='selftest'):
        b200gdn.device_status()
    b200gdn.device_status()                                     # flag was cleared by the read
    d = make_case(seed=1, **STAGE_CASES['d128_dense'])          # and real work still runs and is right
    fwd, _ = oracle_chain(d)
    out = run_abi(d, do_bwd=False)
    O.assert_close('o after expiry', fwd['o'], out['o'], 0.005)


@pytest.mark.parametrize('gscale', [0.02, 12.0])
def test_extreme_gates(gscale):
    """Nearly no decay (g ~ -0.01) and very strong decay (g down to -100 per token: 2^gamma underflows inside a
    chunk): every factor the kernels form is 2^(non-positive), so nothing overflows and results stay finite and
    within tolerance of the fp64 oracle chain."""
    d = make_case(seed=13, **STAGE_CASES['d128_ragged'])
    d['g'] = d['g'] * gscale
    fwd, bwd = oracle_chain(d, dtype=torch.float64)
    out = run_abi(d)
    for n in ('o', 'ht', 'dq', 'dk', 'dv', 'dg', 'dbeta', 'dh0'):
        assert torch.isfinite(out[n]).all(), n
    for n, tol in FWD_TOL.items():
        if n != 'gamma':
            O.assert_close(f'{n}', fwd[n].float(), out[n], tol)
    for n, tol in BWD_TOL.items():
        O.assert_close(f'{n}', bwd[n].float(), out[n], tol)


def test_fused_gate_and_beta_equal_the_separate_passes():
    """The gate / beta activations fused into the first forward and the last backward kernel against the same
    activations run as separate passes (LayerOptionsFunction) around the plain op: identical outputs, gradients
    equal to fp32 rounding (the two evaluate sigmoid in a different order)."""
    from b200gdn import _lib, chunk_gated_delta_rule
    from b200gdn.chunk import LayerOptionsFunction
    dev = 'cuda'
    B, T, H, HV, K, V = 2, 200, 2, 4, 128, 128
    q, k, v, _, _, do = _inputs(B, T, H, HV, K, V, seed=21)
    gen = torch.Generator(device=dev).manual_seed(22)
    graw = torch.randn(B, T, HV, device=dev, generator=gen) * 2
    braw = torch.randn(B, T, HV, device=dev, generator=gen)
    A_log = torch.randn(HV, device=dev, generator=gen) * 0.3
    dt_bias = torch.randn(HV, device=dev, generator=gen) * 0.3

    def run(fused):
        leaves = [x.clone().requires_grad_(True) for x in (q, k, v, graw, braw, A_log, dt_bias)]
        q_, k_, v_, g_, b_, A_, dt_ = leaves
        if fused:
            o, _ = chunk_gated_delta_rule(q_, k_, v_, g_, b_, use_gate_in_kernel=True, A_log=A_, dt_bias=dt_,
                                          use_beta_sigmoid_in_kernel=True, allow_neg_eigval=True)
        else:
            flags = _lib.PREP_GATE | _lib.PREP_BETA_SIGMOID | _lib.PREP_NEG_EIGVAL
            _, _, g2, b2 = LayerOptionsFunction.apply(q_, k_, g_, b_, A_, dt_, flags)
            o, _ = chunk_gated_delta_rule(q_, k_, v_, g2, b2)
        o.backward(do)
        return [o] + [x.grad for x in leaves]
    a, b = run(True), run(False)
    assert torch.equal(a[0], b[0])
    for i in (1, 2, 3):
        assert torch.equal(a[i], b[i]), i            # dq, dk, dv do not pass through the activations
    for i, name in ((4, 'dg'), (5, 'dbeta'), (6, 'dA_log'), (7, 'ddt_bias')):
        O.assert_close(name, b[i].float().cpu(), a[i].float().cpu(), 1e-5)


def _record(name, ratios):
    """Keep the measured err-ratios of the full-size checks in the folder B200GDN_TEST_ARTIFACTS names (when it is
    set and exists); the assertions themselves do not depend on it."""
    import json
    out = os.environ.get('B200GDN_TEST_ARTIFACTS', '')
    if out and os.path.isdir(out):
        with open(os.path.join(out, f'parity_{name}.json'), 'w') as f:
            json.dump({k: float(v) for k, v in ratios.items()}, f, indent=1)


# err-ratio bounds of the reference's own tests (tests/ops/test_gdn.py:108-200)
REF_TOL = dict(o=0.005, ht=0.005, dq=0.008, dk=0.008, dv=0.008, dh0=0.008, dg=0.02, dbeta=0.02)


def test_full_size_backward_against_oracle_one_head():
    """Headline shape B4 T4096 H16 K=V=128, forward AND backward (with an initial state and a gradient on the final
    state): heads and batch rows are independent, so one (batch row, head) slice of the full-size run is compared
    with the fp64 token-by-token oracle and its autograd gradients over the full 4096 tokens."""
    from b200gdn import chunk_gated_delta_rule
    dev = 'cuda'
    B, T, H, K = 4, 4096, 16, 128
    gen = torch.Generator().manual_seed(0)
    nrm = torch.nn.functional.normalize
    q = nrm(torch.randn(B, T, H, K, generator=gen), dim=-1).to(torch.bfloat16)
    k = nrm(torch.randn(B, T, H, K, generator=gen), dim=-1).to(torch.bfloat16)
    v = torch.randn(B, T, H, K, generator=gen).to(torch.bfloat16)
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, H, generator=gen))
    beta = torch.sigmoid(torch.randn(B, T, H, generator=gen))
    h0 = torch.randn(B, H, K, K, generator=gen) * 0.1
    do = torch.randn(B, T, H, K, generator=gen).to(torch.bfloat16)
    dht = torch.randn(B, H, K, K, generator=gen) * 0.1
    leaves = [x.to(dev).requires_grad_(True) for x in (q, k, v, g, beta, h0)]
    o, ht = chunk_gated_delta_rule(*leaves[:5], initial_state=leaves[5], output_final_state=True)
    torch.autograd.backward([o, ht], [do.to(dev), dht.to(dev)])
    b, h = 2, 5
    sl = lambda x: x[b:b + 1, :, h:h + 1].float()
    ro, rht, rg = O.naive_with_grads(sl(q), sl(k), sl(v), sl(g), sl(beta), K ** -0.5, h0[b:b + 1, h:h + 1],
                                     sl(do), dht[b:b + 1, h:h + 1])
    got = dict(o=o[b:b + 1, :, h:h + 1].float().cpu(), ht=ht[b:b + 1, h:h + 1].cpu())
    for n, leaf in zip(('dq', 'dk', 'dv', 'dg', 'dbeta'), leaves[:5]):
        got[n] = leaf.grad[b:b + 1, :, h:h + 1].float().cpu()
    got['dh0'] = leaves[5].grad[b:b + 1, h:h + 1].cpu()
    want = dict(o=ro, ht=rht, **rg)
    ratios = {n: O.err_ratio(want[n].float(), got[n]) for n in REF_TOL}
    _record('headline_one_head', ratios)
    for n, tol in REF_TOL.items():
        O.assert_close(f'headline (b={b}, h={h}) {n}', want[n].float(), got[n], tol)


def test_full_size_varlen_gva_backward_against_oracle_one_sequence():
    """Packed GVA configuration at full size (16 q/k heads, 32 value heads, 16 sequences, 65536 tokens): one
    sequence and one value head of the packed forward + backward against the fp64 oracle over that whole sequence
    (outputs, final state, all gradients incl. dh0).  dq / dk of a q/k head sum over its group of value heads, so
    they are compared on a run whose other value head of the group receives a zero output gradient."""
    from b200gdn import chunk_gated_delta_rule
    dev = 'cuda'
    cu = O.random_cu_seqlens(16, 65536, 256, 8192, seed=0)
    H, HV, K, V, total = 16, 32, 128, 128, 65536
    gen = torch.Generator().manual_seed(1)
    nrm = torch.nn.functional.normalize
    q = nrm(torch.randn(1, total, H, K, generator=gen), dim=-1).to(torch.bfloat16)
    k = nrm(torch.randn(1, total, H, K, generator=gen), dim=-1).to(torch.bfloat16)
    v = torch.randn(1, total, HV, V, generator=gen).to(torch.bfloat16)
    g = torch.nn.functional.logsigmoid(torch.randn(1, total, HV, generator=gen))
    beta = torch.sigmoid(torch.randn(1, total, HV, generator=gen))
    h0 = torch.randn(16, HV, K, V, generator=gen) * 0.1
    do = torch.randn(1, total, HV, V, generator=gen).to(torch.bfloat16)
    dht = torch.randn(16, HV, K, V, generator=gen) * 0.1
    # the shortest sequence that still spans several chunks keeps the oracle's run time in seconds
    lens = [cu[i + 1] - cu[i] for i in range(16)]
    n = min(range(16), key=lambda i: lens[i])
    s, e = cu[n], cu[n + 1]
    hv = 11
    hq = hv // (HV // H)
    other = hq * (HV // H) + (1 - hv % (HV // H))
    do = do.clone()
    do[:, s:e, other] = 0          # the group's other value head contributes nothing to dq / dk of this sequence
    dht = dht.clone()
    dht[n, other] = 0
    leaves = [x.to(dev).requires_grad_(True) for x in (q, k, v, g, beta, h0)]
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)
    o, ht = chunk_gated_delta_rule(*leaves[:5], initial_state=leaves[5], output_final_state=True, cu_seqlens=cu_t)
    torch.autograd.backward([o, ht], [do.to(dev), dht.to(dev)])
    ro, rht, rg = O.naive_with_grads(q[:, s:e, hq:hq + 1].float(), k[:, s:e, hq:hq + 1].float(), v[:, s:e, hv:hv + 1].float(),
                                     g[:, s:e, hv:hv + 1], beta[:, s:e, hv:hv + 1], K ** -0.5, h0[n:n + 1, hv:hv + 1],
                                     do[:, s:e, hv:hv + 1].float(), dht[n:n + 1, hv:hv + 1])
    got = dict(o=o[:, s:e, hv:hv + 1].float().cpu(), ht=ht[n:n + 1, hv:hv + 1].cpu(),
               dq=leaves[0].grad[:, s:e, hq:hq + 1].float().cpu(), dk=leaves[1].grad[:, s:e, hq:hq + 1].float().cpu(),
               dv=leaves[2].grad[:, s:e, hv:hv + 1].float().cpu(), dg=leaves[3].grad[:, s:e, hv:hv + 1].cpu(),
               dbeta=leaves[4].grad[:, s:e, hv:hv + 1].cpu(), dh0=leaves[5].grad[n:n + 1, hv:hv + 1].cpu())
    want = dict(o=ro, ht=rht, **rg)
    ratios = {nme: O.err_ratio(want[nme].float(), got[nme]) for nme in REF_TOL}
    ratios['sequence_length'] = e - s
    _record('varlen_gva_one_sequence', ratios)
    for nme, tol in REF_TOL.items():
        O.assert_close(f'packed GVA (sequence {n}, value head {hv}) {nme}', want[nme].float(), got[nme], tol)


def test_padding_rows_outside_cu_seqlens():
    """A packed buffer with rows before cu_seqlens[0] and after cu_seqlens[-1] (a serving buffer padded to a fixed
    size): the valid rows must equal the run on the unpadded buffer bit for bit, and nothing may turn NaN, although
    the kernels load whole 64-row tiles that reach into the padding."""
    lead, trail = 70, 45
    cu = [0, 37, 101, 165, 300]
    q, k, v, g, beta, do = _inputs(1, 300, 2, 4, 128, 128, seed=11)
    cu_t = torch.tensor(cu, dtype=torch.int32, device='cuda')
    ref = _fwd_bwd(q, k, v, g, beta, do, cu_seqlens=cu_t)

    def pad(x):
        shape = list(x.shape)
        a, b = shape.copy(), shape.copy()
        a[1], b[1] = lead, trail
        # finite but large padding values: they must never reach a valid row
        return torch.cat([torch.full(a, 3.0, dtype=x.dtype, device=x.device), x,
                          torch.full(b, -2.0, dtype=x.dtype, device=x.device)], 1)
    cu_p = torch.tensor([c + lead for c in cu], dtype=torch.int32, device='cuda')
    out = _fwd_bwd(pad(q), pad(k), pad(v), pad(g), pad(beta), pad(do), cu_seqlens=cu_p)
    for nme, a, p in zip(('o', 'ht', 'dq', 'dk', 'dv', 'dg', 'dbeta'), ref, out):
        assert not torch.isnan(p).any(), nme
        got = p if nme == 'ht' else p[:, lead:lead + 300]
        assert torch.equal(a, got), f'{nme} of the valid rows changed with padding around them'


def test_trailing_empty_sequence():
    """cu_seqlens ending in an empty sequence (and one in the middle): it owns no chunk, its final state is its
    initial state and its dh0 is the gradient of the final state."""
    from b200gdn import chunk_gated_delta_rule
    dev = 'cuda'
    cu = [0, 100, 100, 230, 230]
    d = O.make_inputs(1, 230, 2, 2, 128, 128, seed=13, cu_seqlens=cu)
    leaves = [d[n].to(dev).to(torch.bfloat16).requires_grad_(True) for n in ('q', 'k', 'v')]
    leaves += [d[n].to(dev).requires_grad_(True) for n in ('g', 'beta', 'h0')]
    o, ht = chunk_gated_delta_rule(*leaves[:5], initial_state=leaves[5], output_final_state=True,
                                   cu_seqlens=torch.tensor(cu, device=dev))
    torch.autograd.backward([o, ht], [d['do'].to(dev).to(torch.bfloat16), d['dht'].to(dev)])
    ro, rht, rg = O.naive_with_grads(*(d[n].to(torch.bfloat16).float() for n in ('q', 'k', 'v')), d['g'], d['beta'],
                                     128 ** -0.5, d['h0'], d['do'].to(torch.bfloat16).float(), d['dht'], cu_seqlens=cu)
    O.assert_close('o', ro.float(), o.float().cpu(), 0.005)
    O.assert_close('ht', rht.float(), ht.cpu(), 0.005)
    assert torch.equal(ht[1].cpu(), d['h0'][1]) and torch.equal(ht[3].cpu(), d['h0'][3])
    O.assert_close('dh0', rg['dh0'].float(), leaves[5].grad.cpu(), 0.008)
    assert torch.equal(leaves[5].grad[3].cpu(), d['dht'][3])
    import b200gdn
    b200gdn.device_status()


def test_fp32_and_fp16_inputs_are_rounded_to_bf16_and_keep_their_dtype():
    """q, k, v in fp32 / fp16: the result is the bf16 computation on the rounded inputs (documented), returned in
    the caller's dtype, gradients in each input's dtype."""
    from b200gdn import chunk_gated_delta_rule
    dev = 'cuda'
    d = O.make_inputs(2, 130, 2, 2, 128, 128, seed=17)
    for dt in (torch.float32, torch.float16):
        x = [d[n].to(dev).to(dt).requires_grad_(True) for n in ('q', 'k', 'v')]
        gb = [d[n].to(dev).requires_grad_(True) for n in ('g', 'beta')]
        o, _ = chunk_gated_delta_rule(*x, *gb, use_qk_l2norm_in_kernel=(dt == torch.float32))
        o.float().square().sum().backward()
        assert o.dtype == dt and all(t.grad.dtype == dt for t in x)
        y = [t.detach().to(torch.bfloat16).requires_grad_(True) for t in x]
        gb2 = [t.detach().clone().requires_grad_(True) for t in gb]
        o2, _ = chunk_gated_delta_rule(*y, *gb2, use_qk_l2norm_in_kernel=(dt == torch.float32))
        assert o2.dtype == torch.bfloat16
        # fp16: both runs see identical bf16 operands (only the cast of o to fp16 differs, small values land in fp16's
        # subnormal range); fp32 + norm pass: the normalised q / k are rounded to bf16 from slightly different values
        O.assert_close(f'o {dt} inputs vs bf16 inputs', o2.float().cpu(), o.float().cpu(), 1e-3 if dt == torch.float16 else 0.005)


@pytest.mark.parametrize('name', ['d128_ragged', 'd64_ragged_gva', 'd128_dense'])
def test_forward_stage_by_stage_equals_the_fused_scan(name):
    """The forward pass run one stage per call (scan kernel, then the stand-alone output kernel) against the default
    call, where the scan forms the output itself: both against the oracle, and h / v_new / ht bit-identical."""
    from b200gdn import _lib
    d = make_case(seed=23, **STAGE_CASES[name])
    fwd, _ = oracle_chain(d)
    fused = run_abi(d, do_bwd=False)
    a = run_abi(d, fwd_mask=_lib.FWD_INTRA, do_bwd=False)
    saved = {n: a[n] for n in ('gamma', 'A', 'qk', 'w', 'u')}
    b = run_abi(d, fwd_mask=_lib.FWD_SCAN, do_bwd=False, overrides=dict(saved))
    for n in ('h', 'v_new', 'ht'):
        assert torch.equal(b[n], fused[n]), n
    c = run_abi(d, fwd_mask=_lib.FWD_OUT, do_bwd=False, overrides=dict(saved, h=b['h'], v_new=b['v_new']))
    O.assert_close('o staged', fwd['o'], c['o'], 0.005)
    O.assert_close('o fused', fwd['o'], fused['o'], 0.005)
    O.assert_close('o fused vs staged', c['o'], fused['o'], 0.004)


@pytest.mark.parametrize('pieces', [2, 3, 5])
def test_sequence_split_equals_the_unsplit_scan(pieces):
    """Long sequences cut into pieces that are scanned concurrently (pre-scan of each piece's affine map, prefix chain,
    then the regular scan over all pieces): outputs, final state and every gradient against the oracle and against the
    unsplit run, on ragged packed sequences with grouped value heads, an initial state and a final-state gradient."""
    from b200gdn import chunk_gated_delta_rule, index
    dev = 'cuda'
    cu = [0, 37, 700, 700, 1500, 1563]
    d = O.make_inputs(1, 1563, 2, 4, 128, 128, seed=29, cu_seqlens=cu)
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)

    def run():
        leaves = [d[n].to(dev).to(torch.bfloat16).requires_grad_(True) for n in ('q', 'k', 'v')]
        leaves += [d[n].to(dev).requires_grad_(True) for n in ('g', 'beta', 'h0')]
        o, ht = chunk_gated_delta_rule(*leaves[:5], initial_state=leaves[5], output_final_state=True, cu_seqlens=cu_t)
        torch.autograd.backward([o, ht], [d['do'].to(dev).to(torch.bfloat16), d['dht'].to(dev)])
        return [o.float().cpu(), ht.cpu()] + [x.grad.float().cpu() for x in leaves]
    plain = run()
    index.FORCE_PIECES = pieces
    try:
        index._split_cache.clear()
        plan = index.split_plan_for(1, 1563, cu_t, None, torch.device(dev), 4, 2)
        assert plan is not None and max(plan.pieces_per_seq) == pieces
        split = run()
    finally:
        index.FORCE_PIECES = None
        index._split_cache.clear()
    ro, rht, rg = O.naive_with_grads(*(d[n].to(torch.bfloat16).float() for n in ('q', 'k', 'v')), d['g'], d['beta'], 128 ** -0.5,
                                     d['h0'], d['do'].to(torch.bfloat16).float(), d['dht'], cu_seqlens=cu)
    want = [ro, rht, rg['dq'], rg['dk'], rg['dv'], rg['dg'], rg['dbeta'], rg['dh0']]
    names = ('o', 'ht', 'dq', 'dk', 'dv', 'dg', 'dbeta', 'dh0')
    for n, w_, s_, p_ in zip(names, want, split, plain):
        O.assert_close(f'{n} split vs oracle', w_.float(), s_, REF_TOL[n])
        O.assert_close(f'{n} split vs unsplit', p_, s_, 0.004)


@pytest.mark.parametrize('pieces', [None, 3])
def test_state_v_first_layout(pieces):
    """states stored [N,HV,V,K] (the reference's state_v_first, tests/ops/test_gdn.py:385-461): the scans read h0 / dht
    and write ht / dh0 in that layout themselves; the split path transposes at its boundary.  Bit-identical to the run
    on transposed states."""
    from b200gdn import chunk_gated_delta_rule, index
    dev = 'cuda'
    cu = [0, 37, 700, 700, 1500, 1563]
    d = O.make_inputs(1, 1563, 2, 4, 128, 128, seed=33, cu_seqlens=cu)
    cu_t = torch.tensor(cu, dtype=torch.int32, device=dev)

    def run(v_first):
        leaves = [d[n].to(dev).to(torch.bfloat16).requires_grad_(True) for n in ('q', 'k', 'v')]
        leaves += [d[n].to(dev).requires_grad_(True) for n in ('g', 'beta')]
        h0 = d['h0'].to(dev)
        h0 = (h0.transpose(-1, -2).contiguous() if v_first else h0).requires_grad_(True)
        dht = d['dht'].to(dev)
        o, ht = chunk_gated_delta_rule(*leaves, initial_state=h0, output_final_state=True, cu_seqlens=cu_t,
                                       state_v_first=v_first)
        torch.autograd.backward([o, ht], [d['do'].to(dev).to(torch.bfloat16), dht.transpose(-1, -2).contiguous() if v_first else dht])
        outs = [o, ht.transpose(-1, -2) if v_first else ht] + [x.grad for x in leaves]
        return [x.float().cpu() for x in outs + [h0.grad.transpose(-1, -2) if v_first else h0.grad]]
    index.FORCE_PIECES = pieces
    try:
        index._split_cache.clear()
        a, b = run(False), run(True)
    finally:
        index.FORCE_PIECES = None
        index._split_cache.clear()
    for i, (x, y) in enumerate(zip(a, b)):
        assert torch.equal(x, y), f'state_v_first differs in result {i}'


def test_sequence_split_heuristic_on_one_long_sequence():
    """One sequence of 32768 tokens with 4 heads: the planner cuts it (the scans would otherwise occupy 8 of 148 SMs), and
    the result agrees with the token-by-token kernel."""
    from b200gdn import chunk_gated_delta_rule, fused_recurrent_gated_delta_rule, index
    q, k, v, g, beta, do = _inputs(1, 32768, 4, 4, 128, 128, seed=31)
    plan = index.split_plan_for(1, 32768, None, None, q.device, 4, 2)
    assert plan is not None and plan.n_pieces > 1
    o, ht = chunk_gated_delta_rule(q, k, v, g, beta, output_final_state=True)
    o_r, ht_r = fused_recurrent_gated_delta_rule(q, k, v, g, beta=beta, output_final_state=True)
    O.assert_close('o chunk (split) vs recurrent', o_r.float().cpu(), o.float().cpu(), 0.005)
    O.assert_close('ht chunk (split) vs recurrent', ht_r.cpu(), ht.cpu(), 0.005)
