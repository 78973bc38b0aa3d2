"""Host logic: chunk tables, context-parallel partition (against the reference's own integer outputs),
back-end verifier, prefix fold, and a world_size-2 gloo run of the exchange + fold plumbing."""
import os

import numpy as np
import pytest
import torch

from b200gdn.backend import B200GDNBackend
from b200gdn.cp import fold_prefix, get_cp_cu_seqlens
from b200gdn.index import build_tables
from oracle.gdn_oracle import chunk_table

GOLD = os.path.join(os.path.dirname(__file__), 'golden')


@pytest.mark.parametrize('bounds', [
    [(0, 64)], [(0, 1)], [(0, 65), (65, 65), (65, 300)], [(0, 37), (37, 101), (101, 165), (165, 300)],
    [(i * 4096, (i + 1) * 4096) for i in range(4)],
])
def test_chunk_tables(bounds):
    cm, sm = build_tables(bounds)
    want = chunk_table(bounds)
    assert [(int(r[0]), int(r[1]), int(r[2])) for r in cm] == want
    assert int(sm[:, 1].sum()) == len(want)
    for n, (first, cnt) in enumerate(sm):
        assert all(int(cm[first + i, 0]) == n and int(cm[first + i, 3]) == i for i in range(cnt))
    assert cm.dtype == np.int32 and sm.dtype == np.int32


def test_chunk_tables_reject_decreasing():
    with pytest.raises(ValueError):
        build_tables([(0, 10), (10, 5)])


def test_cp_partition_matches_reference_fixture():
    gold = np.load(os.path.join(GOLD, 'cp_context.npz'))
    ci = 0
    while f'case{ci}' in gold:
        arr = gold[f'case{ci}'].tolist()
        cu, W = arr[:-2], arr[-1]
        for r in range(W):
            ref = gold[f'{ci}_{r}'].tolist()
            cut = ref.index(-1)
            ctx = get_cp_cu_seqlens(torch.tensor(cu, dtype=torch.long), world_size=W, rank=r)
            assert ctx.cu_seqlens_cpu.tolist() == ref[:cut]
            assert [ctx.pre_num_ranks, ctx.post_num_ranks, int(ctx.is_first_rank), int(ctx.is_last_rank),
                    ctx.pre_num_conv_tokens] == ref[cut + 1:]
            assert ctx.cu_seqlens_cpu.dtype == torch.int32
        ci += 1
    assert ci == 5


def test_cp_partition_reference_known_answers():
    """The reference's own expectations (tests/context_parallel/test_cp_context.py:13-55)."""
    with pytest.raises(ValueError, match=r'`total_tokens` \(10\) must be divisible by `world_size` \(3\)'):
        get_cp_cu_seqlens(torch.tensor([0, 10]), world_size=3, rank=0)
    with pytest.raises(ValueError, match=r'`total_tokens` \(2\) must be at least `world_size` \(3\)'):
        get_cp_cu_seqlens(torch.tensor([0, 2]), world_size=3, rank=0)
    c = get_cp_cu_seqlens(torch.tensor([0, 5, 12]), world_size=3, rank=1)
    assert c.cu_seqlens_cpu.tolist() == [0, 1, 4]
    assert (c.pre_num_conv_tokens, c.pre_num_ranks, c.post_num_ranks) == (4, 1, 1)
    assert not c.is_first_rank and not c.is_last_rank


def _torch_apply(M, x, b, transpose):
    return (M.transpose(-1, -2) if transpose else M) @ x + b


def test_fold_prefix_composes_affine_maps():
    gen = torch.Generator().manual_seed(0)
    W, HV, K, V = 4, 2, 8, 6
    gathered = torch.randn(W, HV, K, K + V, generator=gen)
    assert fold_prefix(gathered, 2, 0, K, True, _torch_apply) is None
    x = fold_prefix(gathered, 3, 3, K, True, _torch_apply)
    want = torch.zeros(HV, K, V)
    for j in range(3):
        want = gathered[j, :, :, :K] @ want + gathered[j, :, :, K:]
    assert torch.allclose(x, want, atol=1e-5)
    y = fold_prefix(gathered, 0, 2, K, False, _torch_apply)
    want = torch.zeros(HV, K, V)
    for j in (2, 1):
        want = gathered[j, :, :, :K] @ want + gathered[j, :, :, K:]
    assert torch.allclose(y, want, atol=1e-5)


def test_backend_verifier():
    be = B200GDNBackend()
    q = torch.zeros(1, 64, 2, 128, dtype=torch.bfloat16)
    g = torch.zeros(1, 64, 2)
    ok, why = be.verify('chunk_gated_delta_rule', q, q, q, g, g)
    assert not ok and 'CUDA' in why
    assert B200GDNBackend.backend_type == 'b200_gdn' and B200GDNBackend.priority < 3
    os.environ['FLA_B200_GDN'] = '0'
    try:
        assert not B200GDNBackend.is_enabled()
    finally:
        del os.environ['FLA_B200_GDN']
    assert B200GDNBackend.is_enabled()


def _gloo_worker(rank, world, port, q):
    import torch.distributed as dist
    from b200gdn.cp import exchange, fold_prefix, get_cp_cu_seqlens
    dist.init_process_group('gloo', init_method=f'tcp://127.0.0.1:{port}', rank=rank, world_size=world)
    try:
        HV, K, V = 2, 4, 3
        gen = torch.Generator().manual_seed(100 + rank)
        local = torch.randn(HV, K, K + V, generator=gen)
        gathered = exchange(local, None)
        ctx = get_cp_cu_seqlens(torch.tensor([0, 64]), world_size=world, rank=rank)
        x = fold_prefix(gathered, rank, ctx.pre_num_ranks, K, True, _torch_apply)
        q.put((rank, gathered, ctx.pre_num_ranks, ctx.post_num_ranks, x))
    except Exception as e:  # surface the failure instead of letting the parent wait for its timeout
        q.put((rank, repr(e), 0, 0, None))
    finally:
        dist.destroy_process_group()


def test_exchange_and_fold_two_ranks_gloo():
    import torch.multiprocessing as mp
    ctx = mp.get_context('spawn')
    q = ctx.Queue()
    port = 29500 + os.getpid() % 400
    procs = [ctx.Process(target=_gloo_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    res = sorted([q.get(timeout=120) for _ in procs], key=lambda t: t[0])
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(not isinstance(r[1], str) for r in res), res
    (_, g0, pre0, post0, x0), (_, g1, pre1, post1, x1) = res
    assert torch.equal(g0, g1) and g0.shape[0] == 2
    assert (pre0, post0, pre1, post1) == (0, 1, 1, 0)
    assert x0 is None
    assert torch.allclose(x1, g0[0, :, :, 4:])      # one predecessor: its h_ext


def test_backend_verifier_serves_bf16_only():
    """fp16 / fp32 q, k, v are declined so that the dispatcher falls through to the reference's own path, which
    keeps their precision (the kernels here compute on bf16 operands)."""
    be = B200GDNBackend()

    class FakeCuda(torch.Tensor):
        is_cuda = True
    g = torch.zeros(1, 64, 2)
    for dt, want in ((torch.bfloat16, True), (torch.float16, False), (torch.float32, False)):
        q = torch.zeros(1, 64, 2, 128, dtype=dt).as_subclass(FakeCuda)
        ok, why = be.chunk_gated_delta_rule_verifier(q, q, q, g, g)
        assert ok is want, (dt, why)
        if not want:
            assert 'bf16' in why
    q = torch.zeros(1, 64, 2, 96, dtype=torch.bfloat16).as_subclass(FakeCuda)
    ok, why = be.chunk_gated_delta_rule_verifier(q, q, q, g, g)
    assert not ok and 'not built' in why


REF_INSTALL = os.path.join(os.path.dirname(__file__), '..', 'baseline', '_ref')

_INSTALL_PROBE = r'''
import sys
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[2])
import fla
import fla.layers.gated_deltanet as layer_mod
import fla.ops.gated_delta_rule as op_mod
from fla.ops.gated_delta_rule.backends import gdr_registry
import b200gdn
from b200gdn.backend import B200GDNBackend
stock_layer, stock_op = layer_mod.fused_recurrent_gated_delta_rule, op_mod.fused_recurrent_gated_delta_rule
gdr_registry._ensure_initialized() if hasattr(gdr_registry, '_ensure_initialized') else None
before = set(gdr_registry._backends)
assert b200gdn.install() is True
assert 'b200_gdn' in gdr_registry._backends and isinstance(gdr_registry._backends['b200_gdn'], B200GDNBackend)
assert layer_mod.fused_recurrent_gated_delta_rule is b200gdn.fused_recurrent_gated_delta_rule
assert op_mod.fused_recurrent_gated_delta_rule is b200gdn.fused_recurrent_gated_delta_rule
# without a B200 the backend reports itself unavailable, so the registry must not select it here
import torch
if not torch.cuda.is_available():
    assert not B200GDNBackend.is_available()
b200gdn.install()   # idempotent: the saved stock functions survive a second call
b200gdn.uninstall()
assert set(gdr_registry._backends) == before
assert layer_mod.fused_recurrent_gated_delta_rule is stock_layer
assert op_mod.fused_recurrent_gated_delta_rule is stock_op
b200gdn.uninstall()  # and a second uninstall is harmless
print('install-ok', fla.__version__)
'''


@pytest.mark.skipif(not os.path.isdir(os.path.join(REF_INSTALL, 'fla')), reason='no reference install under baseline/_ref')
def test_install_and_uninstall_against_the_reference_registry():
    """install() registers the backend in the reference's own registry object and rebinds the decode function in
    the two modules that import it by name; uninstall() restores all three (fla/ops/backends/__init__.py:96-157,
    fla/ops/gated_delta_rule/backends/__init__.py:14-17)."""
    import subprocess
    import sys
    pkg = os.path.join(os.path.dirname(__file__), '..', 'flash-linear-attention_b200')
    out = subprocess.run([sys.executable, '-c', _INSTALL_PROBE, os.path.abspath(pkg), os.path.abspath(REF_INSTALL)],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout + out.stderr
    assert 'install-ok 0.5.2' in out.stdout


def test_slab_hands_out_aligned_addresses_and_null_for_absent_pieces():
    """The step's workspace is one allocation known to the host only as addresses: every piece on a 256-byte boundary,
    pieces of zero bytes get the null address, pieces do not overlap, and the addresses can be rebuilt from the saved
    tensor and offsets (what the backward pass does)."""
    import torch
    from b200gdn.chunk import Slab
    sizes = (1000, 0, 256, 77, 0, 4096)
    slab = Slab(torch.device('cpu'), True, sizes)
    addr = Slab.addresses(slab.buf, slab.offs)
    base = slab.buf.data_ptr()
    assert [a == 0 for a in addr] == [n == 0 for n in sizes]
    live = [(a - base, n) for a, n in zip(addr, sizes) if n]
    assert all(off % 256 == 0 for off, _ in live)
    for (o0, n0), (o1, _) in zip(live, live[1:]):
        assert o0 + n0 <= o1
    assert live[-1][0] + live[-1][1] <= slab.buf.numel()
    assert Slab.addresses(slab.buf, list(slab.offs)) == addr
    assert int(slab.buf.sum()) == 0                      # zero=True fills the allocation
    assert Slab(torch.device('cpu'), False, (0, 0)).buf.numel() >= 256   # never an empty allocation
