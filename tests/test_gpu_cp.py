"""Context parallelism on real GPUs (NCCL): every rank runs its shard with a cp_context; outputs and
gradients must equal the single-GPU run on the whole packed batch.  Scenarios follow the reference's
tests/context_parallel/test_cp_gdn.py:314-457 (a sequence cut by the shard boundary, boundary-aligned
sequences, many short sequences, grouped value heads, one long sequence over all ranks)."""
import os

import pytest
import torch

pytestmark = pytest.mark.gpu

SCENARIOS = {
    # name: (world, total tokens, cu_seqlens, H, HV)
    'cp2_single': (2, 1024, [0, 1024], 2, 2),
    'cp2_cut': (2, 1024, [0, 700, 1024], 2, 2),
    'cp2_aligned': (2, 1024, [0, 512, 1024], 2, 2),
    'cp2_many_short_gva': (2, 1024, [0, 100, 250, 400, 530, 777, 1024], 2, 4),
    'cp4_complex': (4, 2048, [0, 300, 1500, 1600, 2048], 2, 2),
    'cp4_single': (4, 2048, [0, 2048], 1, 2),
    'cp8_single': (8, 8192, [0, 8192], 1, 1),
    # the same with every local sequence also cut into pieces that are scanned concurrently (sixth field: pieces)
    'cp2_cut_split3': (2, 4096, [0, 2700, 4096], 2, 2, 3),
    'cp2_many_short_gva_split2': (2, 4096, [0, 400, 1000, 1600, 2130, 3100, 4096], 2, 4, 2),
    'cp4_complex_split2': (4, 8192, [0, 1200, 6000, 6400, 8192], 2, 2, 2),
    # the long-context configuration at full size: one sequence of 524288 tokens, 16 heads (inputs made on the device)
    'cp2_long': (2, 524288, [0, 524288], 16, 16),
    'cp4_long': (4, 524288, [0, 524288], 16, 16),
    'cp8_long': (8, 524288, [0, 524288], 16, 16),
}


def _worker(rank, world, port, name, q):
    import torch.distributed as dist
    from b200gdn import build_cp_context, chunk_gated_delta_rule
    from oracle import gdn_oracle as O
    _, T, cu, H, HV = SCENARIOS[name][:5]
    K = V = 128
    if len(SCENARIOS[name]) > 5:
        from b200gdn import index
        index.FORCE_PIECES = SCENARIOS[name][5]
    torch.cuda.set_device(rank)
    dev = torch.device('cuda', rank)
    dist.init_process_group('nccl', init_method=f'tcp://127.0.0.1:{port}', rank=rank, world_size=world, device_id=dev)
    try:
        if T <= 65536:
            d = O.make_inputs(1, T, H, HV, K, V, seed=17, cu_seqlens=cu, with_h0=False)
            full = {n: d[n].to(dev) for n in ('q', 'k', 'v', 'g', 'beta', 'do')}
            for n in ('q', 'k', 'v', 'do'):
                full[n] = full[n].to(torch.bfloat16)
        else:   # same distributions, generated on the device (identical on every rank: same seed, same generator)
            gen = torch.Generator(device=dev).manual_seed(17)
            nrm = torch.nn.functional.normalize
            full = {
                'q': nrm(torch.randn(1, T, H, K, device=dev, generator=gen), dim=-1).to(torch.bfloat16),
                'k': nrm(torch.randn(1, T, H, K, device=dev, generator=gen), dim=-1).to(torch.bfloat16),
                'v': torch.randn(1, T, HV, V, device=dev, generator=gen).to(torch.bfloat16),
                'g': torch.nn.functional.logsigmoid(torch.randn(1, T, HV, device=dev, generator=gen)),
                'beta': torch.sigmoid(torch.randn(1, T, HV, device=dev, generator=gen)),
                'do': torch.randn(1, T, HV, V, device=dev, generator=gen).to(torch.bfloat16),
            }
        cu_t = torch.tensor(cu, dtype=torch.long, device=dev)
        # single-GPU run of the same operator on the whole batch (never cut into pieces in the forced scenarios)
        if len(SCENARIOS[name]) > 5:
            index.FORCE_PIECES = 1
        ref_leaves = [full[n].clone().requires_grad_(True) for n in ('q', 'k', 'v', 'g', 'beta')]
        o_ref, _ = chunk_gated_delta_rule(*ref_leaves, cu_seqlens=cu_t)
        o_ref.backward(full['do'])
        # this rank's shard
        if len(SCENARIOS[name]) > 5:
            index.FORCE_PIECES = SCENARIOS[name][5]
            index._split_cache.clear()
        P = T // world
        sl = slice(rank * P, (rank + 1) * P)
        ctx = build_cp_context(cu_t, group=dist.group.WORLD, cu_seqlens_cpu=torch.tensor(cu, dtype=torch.long))
        leaves = [full[n][:, sl].clone().requires_grad_(True) for n in ('q', 'k', 'v', 'g', 'beta')]
        o, ht = chunk_gated_delta_rule(*leaves, cp_context=ctx)
        assert ht is None
        o.backward(full['do'][:, sl])
        torch.cuda.synchronize()
        def ratio(a, b):   # the oracle's error ratio, evaluated on the device (the long case is 1 G elements)
            a, b = a.detach().float(), b.detach().float()
            return float((a - b).square().mean().sqrt() / (a.square().mean().sqrt() + 1e-8))
        errs = {'o': ratio(o_ref[:, sl], o)}
        for nme, a, b in zip(('dq', 'dk', 'dv', 'dg', 'dbeta'), ref_leaves, leaves):
            errs[nme] = ratio(a.grad[:, sl], b.grad)
        import b200gdn
        b200gdn.device_status()   # no bounded device wait expired on this rank
        if errs['o'] > 0.005:     # where along the shard the outputs differ (32 blocks), for the failure message
            n = P // 32
            errs['o_blocks'] = [round(ratio(o_ref[:, sl][:, i * n:(i + 1) * n], o[:, i * n:(i + 1) * n]), 4) for i in range(32)]
        q.put((rank, errs))
    except Exception as e:
        import traceback
        q.put((rank, 'ERROR ' + repr(e) + traceback.format_exc()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('name', list(SCENARIOS))
def test_context_parallel_matches_single_gpu(name):
    world = SCENARIOS[name][0]
    if torch.cuda.device_count() < world:
        pytest.skip(f'needs {world} GPUs')
    import torch.multiprocessing as mp
    ctx = mp.get_context('spawn')
    q = ctx.Queue()
    port = 29600 + (os.getpid() + hash(name)) % 300
    procs = [ctx.Process(target=_worker, args=(r, world, port, name, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=600) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, errs in res:
        assert not isinstance(errs, str), f'rank {rank}: {errs}'
        # same tolerance as the reference's CP test (assert_close ratio 3e-3 .. 5e-3 against its own single-GPU run)
        for n, e in errs.items():
            if n == 'o_blocks':
                continue
            assert e < 0.005, f'{name} rank {rank} {n}: {e} {errs}'


def test_fold_kernels_match_the_host_fold():
    """The single-launch prefix fold and the one-step affine kernel against the host statement of the fold in fp64
    (forward and backward direction, every possible number of neighbouring ranks)."""
    from b200gdn.cp import affine_apply, fold_on_device, fold_prefix
    W, HV, K, V = 8, 3, 128, 128
    gen = torch.Generator().manual_seed(5)
    gathered = torch.randn(W, HV, K, K + V, generator=gen)
    gathered[..., :K] *= K ** -0.5   # keep the chained products O(1)
    dev_g = gathered.cuda()

    def host(M, x, b, transpose):
        return (M.double().transpose(-1, -2) if transpose else M.double()) @ x.double() + b.double()
    for rank, num, fwd in [(7, 7, True), (3, 1, True), (5, 2, True), (0, 7, False), (4, 3, False), (6, 1, False)]:
        want = fold_prefix(gathered, rank, num, K, fwd, host).float()
        out = torch.empty(HV, K, V, device='cuda')
        fold_on_device(dev_g, rank, num, K, fwd, out)
        assert torch.allclose(out.cpu(), want, rtol=1e-4, atol=1e-4), (rank, num, fwd, float((out.cpu() - want).abs().max()))
        got = fold_prefix(dev_g, rank, num, K, fwd, affine_apply)
        assert torch.allclose(got.cpu(), want, rtol=1e-4, atol=1e-4)
    M, x, b = dev_g[0, :, :, :K].contiguous(), dev_g[1, :, :, K:].contiguous(), dev_g[2, :, :, K:].contiguous()
    assert torch.allclose(affine_apply(M, x, b, True).cpu(), host(M.cpu(), x.cpu(), b.cpu(), True).float(), rtol=1e-4, atol=1e-4)


def _conv_worker(rank, world, port, q):
    import torch.distributed as dist
    from b200gdn import build_cp_context
    from b200gdn.modules import causal_conv1d
    torch.cuda.set_device(rank)
    dev = torch.device('cuda', rank)
    dist.init_process_group('nccl', init_method=f'tcp://127.0.0.1:{port}', rank=rank, world_size=world, device_id=dev)
    try:
        T, D, W = 512, 192, 4
        cu = [0, 100, 255, 258, 512]   # sequences cut by the shard boundary, and one that starts 2 tokens before it
        gen = torch.Generator().manual_seed(23)
        x = torch.randn(1, T, D, generator=gen).to(dev)
        w = (torch.randn(D, W, generator=gen) * 0.5).to(dev)
        b = torch.randn(D, generator=gen).to(dev)
        dy = torch.randn(1, T, D, generator=gen).to(dev)
        cu_t = torch.tensor(cu, dtype=torch.long, device=dev)
        ref = [t.clone().requires_grad_(True) for t in (x, w, b)]
        y_ref, _ = causal_conv1d(*ref, activation='silu', cu_seqlens=cu_t)
        y_ref.backward(dy)
        P = T // world
        sl = slice(rank * P, (rank + 1) * P)
        ctx = build_cp_context(cu_t, group=dist.group.WORLD, conv1d_kernel_size=W, cu_seqlens_cpu=torch.tensor(cu, dtype=torch.long))
        loc = [x[:, sl].clone().requires_grad_(True), w.clone().requires_grad_(True), b.clone().requires_grad_(True)]
        y, _ = causal_conv1d(*loc, activation='silu', cp_context=ctx)
        y.backward(dy[:, sl])
        dw, db = loc[1].grad.clone(), loc[2].grad.clone()
        dist.all_reduce(dw)
        dist.all_reduce(db)
        errs = dict(y=float((y - y_ref[:, sl]).abs().max()), dx=float((loc[0].grad - ref[0].grad[:, sl]).abs().max()),
                    dw=float((dw - ref[1].grad).abs().max() / ref[1].grad.abs().max()),
                    db=float((db - ref[2].grad).abs().max() / ref[2].grad.abs().max()))
        q.put((rank, errs))
    except Exception as e:
        import traceback
        q.put((rank, 'ERROR ' + repr(e) + traceback.format_exc()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize('world', [2, 4])
def test_context_parallel_convolution_matches_single_gpu(world):
    """The convolution in front of the mixer under context parallelism: every rank's first sequence starts from the
    previous rank's last W-1 tokens, whose gradient flows back to that rank (tests/context_parallel of the reference
    checks its conv the same way against a single-GPU run)."""
    if torch.cuda.device_count() < world:
        pytest.skip(f'needs {world} GPUs')
    import torch.multiprocessing as mp
    ctx = mp.get_context('spawn')
    q = ctx.Queue()
    port = 29900 + os.getpid() % 90 + world
    procs = [ctx.Process(target=_conv_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = [q.get(timeout=600) for _ in procs]
    for p in procs:
        p.join(timeout=60)
    for rank, errs in res:
        assert not isinstance(errs, str), f'rank {rank}: {errs}'
        assert errs['y'] < 1e-5 and errs['dx'] < 1e-5 and errs['dw'] < 1e-5 and errs['db'] < 1e-5, (rank, errs)
