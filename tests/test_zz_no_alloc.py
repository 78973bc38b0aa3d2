"""b200gdn_chunk_fwd_static, the forward entry point for hosts that cannot allocate device memory
(a server whose memory pool already owns the whole GPU, a plug-in in a foreign CUDA context): its
intermediates live in an array built into the library instead of caller-supplied buffers.

Called through the C ABI and compared with b200gdn_chunk_fwd on the same inputs, twice in a row with
different problems, because the built-in array is shared between calls and keeps the previous call's
contents.  This file sorts last so that a run stopping at the first failure has run every other test.
"""
import ctypes as C

import pytest
import torch

from oracle import gdn_oracle as O
from tests.gpu_util import make_case

STATIC_BYTES = 64 << 20


def _lib_and_fn():
    from b200gdn import _lib
    lib = _lib.load()
    fn = lib.b200gdn_chunk_fwd_static
    fn.restype = C.c_int
    fn.argtypes = [C.c_void_p, C.c_void_p]
    return _lib, lib, fn


def _args_for(d, dev):
    from b200gdn import _lib
    from b200gdn.chunk import new_chunk_args
    from b200gdn.index import build_tables
    B, T, H, HV, K, V = d['dims']
    cm, sm = build_tables(d['bounds'])
    keep = dict(chunk_meta=torch.from_numpy(cm).to(dev), seq_meta=torch.from_numpy(sm).to(dev))
    for n in ('q', 'k', 'v'):
        keep[n] = d[n].to(dev).contiguous()
    for n in ('g', 'beta', 'h0'):
        keep[n] = d[n].float().to(dev).contiguous()
    a = new_chunk_args(keep['q'], keep['k'], keep['v'], d['scale'],
                       (keep['chunk_meta'], keep['seq_meta'], (cm.shape[0], sm.shape[0])))
    a.g, a.beta, a.h0 = keep['g'].data_ptr(), keep['beta'].data_ptr(), keep['h0'].data_ptr()
    a.struct_bytes = C.sizeof(a)
    return a, keep, (B * T, HV, K, V, cm.shape[0], sm.shape[0])


@pytest.mark.gpu
def test_static_scratch_forward_matches_regular_forward_twice():
    _lib, lib, fn = _lib_and_fn()
    dev = torch.device('cuda')
    stream = torch.cuda.current_stream().cuda_stream
    cases = [dict(B=1, T=333, H=1, HV=2, K=128, V=128, cu=[0, 1, 16, 80, 143, 270, 333], seed=21),
             dict(B=2, T=256, H=2, HV=4, K=64, V=64, seed=22)]
    for kw in cases:   # two calls in a row on different problems: stale contents must not matter
        d = make_case(**kw)
        a, keep, (rows, HV, K, V, n_chunks, n_seq) = _args_for(d, dev)
        bf = dict(dtype=torch.bfloat16, device=dev)
        f32 = dict(dtype=torch.float32, device=dev)
        # regular entry point with caller-allocated intermediates
        o_ref = torch.empty(rows, HV, V, **bf)
        ht_ref = torch.empty(n_seq, HV, K, V, **f32)
        scratch = dict(gamma=torch.empty(n_chunks, HV, 64, **f32), A=torch.empty(rows, HV, 64, **bf), qk=torch.empty(rows, HV, 64, **bf),
                       w=torch.empty(rows, HV, K, **bf), u=torch.empty(rows, HV, V, **bf),
                       h=torch.empty(n_chunks, HV, K, V, **bf), v_new=torch.empty(rows, HV, V, **bf))
        a.o, a.ht = o_ref.data_ptr(), ht_ref.data_ptr()
        for n, x in scratch.items():
            setattr(a, n, x.data_ptr())
        assert lib.b200gdn_chunk_fwd(C.byref(a), C.c_void_p(stream)) == 0, lib.b200gdn_last_error()
        # static entry point: inputs and outputs only
        o = torch.full((rows, HV, V), float('nan'), **bf)
        ht = torch.full((n_seq, HV, K, V), float('nan'), **f32)
        a.o, a.ht = o.data_ptr(), ht.data_ptr()
        for n in scratch:
            setattr(a, n, None)
        before = torch.cuda.memory_allocated()
        assert fn(C.byref(a), C.c_void_p(stream)) == 0, lib.b200gdn_last_error()
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == before
        O.assert_close('o', o_ref.float().cpu(), o.float().cpu(), 0.005)
        O.assert_close('ht', ht_ref.cpu(), ht.cpu(), 0.005)
        assert torch.equal(o, o_ref) and torch.equal(ht, ht_ref)   # same kernels, so in fact bit-identical


def test_static_scratch_rejects_oversized_problem():
    """Size check comes before any CUDA call, so this part also runs without a GPU."""
    _lib, lib, fn = _lib_and_fn()
    a = _lib.ChunkArgs()
    a.struct_bytes = C.sizeof(a)
    a.rows, a.H, a.HV, a.K, a.V, a.n_seq, a.n_chunks = 16384, 16, 16, 128, 128, 4, 256
    one = C.c_void_p(256)   # non-null placeholders; never dereferenced because the call is rejected
    for n in ('chunk_meta', 'seq_meta', 'q', 'k', 'v', 'g', 'beta', 'o'):
        setattr(a, n, one)
    assert fn(C.byref(a), None) == -4
    msg = lib.b200gdn_last_error().decode()
    assert 'needs' in msg and str(STATIC_BYTES) in msg
    a.rows = 0
    assert fn(C.byref(a), None) == -1
