"""The C-ABI library loads on a machine without a GPU and exports every symbol include/b200gdn.h declares;
struct layouts of the ctypes mirror match the header (checked through a tiny C program)."""
import ctypes
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), '..'))
HEADER = os.path.join(ROOT, 'include', 'b200gdn.h')


def _declared_functions():
    src = open(HEADER).read()
    src = re.sub(r'/\*.*?\*/', '', src, flags=re.S)
    return sorted(set(re.findall(r'\b(b200gdn_[a-z0-9_]+)\s*\(', src)))


def test_library_exports_every_declared_symbol():
    from b200gdn import _lib
    lib = _lib.load()
    names = _declared_functions()
    assert len(names) >= 9
    for n in names:
        assert hasattr(lib, n), f'{n} declared in include/b200gdn.h but not exported'
    assert set(_lib.EXPORTS) <= set(names)
    assert lib.b200gdn_abi_version() == _lib.ABI_VERSION


def test_struct_layouts_match_header(tmp_path):
    from b200gdn import _lib
    prog = tmp_path / 'sz.c'
    prog.write_text('#include <stdio.h>\n#include <stddef.h>\n#include "b200gdn.h"\nint main(void){'
                    'printf("%zu %zu %zu %zu %zu %zu %zu %zu %zu\\n", sizeof(b200gdn_chunk_args), sizeof(b200gdn_recurrent_args),'
                    'sizeof(b200gdn_affine_args), offsetof(b200gdn_chunk_args, chunk_meta), offsetof(b200gdn_chunk_args, dq_acc),'
                    'offsetof(b200gdn_recurrent_args, cu_seqlens), sizeof(b200gdn_prep_args), offsetof(b200gdn_prep_args, q),'
                    'offsetof(b200gdn_prep_args, partials));return 0;}\n')
    exe = tmp_path / 'sz'
    subprocess.check_call(['gcc', '-I', os.path.join(ROOT, 'include'), str(prog), '-o', str(exe)])
    got = [int(x) for x in subprocess.check_output([str(exe)]).split()]
    want = [ctypes.sizeof(_lib.ChunkArgs), ctypes.sizeof(_lib.RecurrentArgs), ctypes.sizeof(_lib.AffineArgs),
            _lib.ChunkArgs.chunk_meta.offset, _lib.ChunkArgs.dq_acc.offset, _lib.RecurrentArgs.cu_seqlens.offset,
            ctypes.sizeof(_lib.PrepArgs), _lib.PrepArgs.q.offset, _lib.PrepArgs.partials.offset]
    assert got == want


def test_argument_errors_without_gpu():
    """Argument validation happens before any CUDA call, so it can be exercised on the CPU."""
    from b200gdn import _lib
    a = _lib.ChunkArgs()
    with pytest.raises(_lib.B200GDNError, match='empty problem'):
        _lib.call('b200gdn_chunk_fwd', a, 0)
    lib = _lib.load()
    a.struct_bytes = 8
    assert lib.b200gdn_chunk_bwd(ctypes.byref(a), None) == -1
    assert b'ABI mismatch' in lib.b200gdn_last_error()
    assert lib.b200gdn_recurrent_fwd(None, None) == -1
    p = _lib.PrepArgs()
    p.struct_bytes = ctypes.sizeof(p)
    p.rows, p.H, p.HV, p.K, p.flags = 64, 2, 2, 100, _lib.PREP_L2NORM
    assert lib.b200gdn_prep_fwd(ctypes.byref(p), None) == -2 and b'are built' in lib.b200gdn_last_error()
    p.K, p.flags = 128, _lib.PREP_GATE
    assert lib.b200gdn_prep_bwd(ctypes.byref(p), None) == -1 and b'is NULL' in lib.b200gdn_last_error()
    assert lib.b200gdn_saved_bytes(16384, 16, 16, 128, 128, 256) == 16384 * 16 * (4 + 256 + 256 * 3) + 256 * 16 * 32768
    assert lib.b200gdn_bwd_workspace_bytes(64, 2, 4, 128, 128, 1) > 0


def test_product_does_not_import_oracle():
    """Nothing under the package may import, read or run the oracle."""
    pkg = os.path.join(ROOT, 'flash-linear-attention_b200')
    for d, _, files in os.walk(pkg):
        for f in files:
            if f.endswith(('.py', '.cu', '.cuh', '.h')):
                text = open(os.path.join(d, f)).read()
                assert 'oracle' not in text, os.path.join(d, f)


def test_cpu_tensor_is_rejected():
    import torch
    from b200gdn import B200GDNError, chunk_gated_delta_rule, fused_recurrent_gated_delta_rule
    q = torch.zeros(1, 64, 1, 128, dtype=torch.bfloat16)
    g = torch.zeros(1, 64, 1)
    with pytest.raises(B200GDNError, match='CUDA device only'):
        chunk_gated_delta_rule(q, q, q, g, g)
    with pytest.raises(B200GDNError, match='CUDA device only'):
        fused_recurrent_gated_delta_rule(q, q, q, g, beta=g)
