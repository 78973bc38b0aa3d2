"""The backend object really is what the reference's dispatcher calls: with the reference installed under
baseline/_ref, `fla.ops.gated_delta_rule.chunk_gated_delta_rule` on a B200 must reach B200GDNBackend's method
(spy, as tests/ops/test_gdn.py:1318-1331 does for its FlashQLA backend) and give this library's result, and fp32
inputs must fall through to the reference's own Triton path.  Runs in a child process so that the reference's
modules do not leak into the other tests."""
import os
import subprocess
import sys

import pytest

ROOT = os.path.abspath(os.path.join(os.path.dirname(__file__), '..'))
REF_INSTALL = os.path.join(ROOT, 'baseline', '_ref')

_PROBE = r'''
import sys
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, sys.argv[2])
import torch
import fla
from fla.ops.gated_delta_rule import chunk_gated_delta_rule as fla_op
import b200gdn
from b200gdn.backend import B200GDNBackend
assert b200gdn.install()
calls = []
impl = B200GDNBackend.chunk_gated_delta_rule
def spy(self, *a, **kw):
    calls.append(a[0].dtype)
    return impl(self, *a, **kw)
B200GDNBackend.chunk_gated_delta_rule = spy
dev = 'cuda'
gen = torch.Generator().manual_seed(0)
B, T, H, K = 2, 200, 2, 128
nrm = torch.nn.functional.normalize
q = nrm(torch.randn(B, T, H, K, generator=gen), dim=-1).to(dev)
k = nrm(torch.randn(B, T, H, K, generator=gen), dim=-1).to(dev)
v = torch.randn(B, T, H, K, generator=gen).to(dev)
g = torch.nn.functional.logsigmoid(torch.randn(B, T, H, generator=gen)).to(dev)
beta = torch.sigmoid(torch.randn(B, T, H, generator=gen)).to(dev)
bf = torch.bfloat16
o_disp, ht_disp = fla_op(q.to(bf), k.to(bf), v.to(bf), g, beta, output_final_state=True)
assert calls == [bf], calls                                  # dispatched to this backend
o_own, ht_own = b200gdn.chunk_gated_delta_rule(q.to(bf), k.to(bf), v.to(bf), g, beta, output_final_state=True)
assert torch.equal(o_disp, o_own) and torch.equal(ht_disp, ht_own)
o32, _ = fla_op(q, k, v, g, beta, output_final_state=True)    # fp32: declined by the verifier -> Triton path
assert calls == [bf], calls
assert o32.dtype == torch.float32
den = o32.float().square().mean().sqrt()
err = (o32.float() - o_own.float()).square().mean().sqrt() / den
assert err < 0.01, float(err)
b200gdn.uninstall()
o_stock, _ = fla_op(q.to(bf), k.to(bf), v.to(bf), g, beta, output_final_state=True)
assert calls == [bf], calls                                  # after uninstall the stock path serves bf16 again
err = (o_stock.float() - o_own.float()).square().mean().sqrt() / den
assert err < 0.005, float(err)
print('dispatch-ok', fla.__version__)
'''


@pytest.mark.gpu
@pytest.mark.skipif(not os.path.isdir(os.path.join(REF_INSTALL, 'fla')), reason='no reference install under baseline/_ref')
def test_reference_dispatcher_reaches_the_backend():
    pkg = os.path.join(ROOT, 'flash-linear-attention_b200')
    out = subprocess.run([sys.executable, '-c', _PROBE, pkg, REF_INSTALL], capture_output=True, text=True, timeout=900)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert 'dispatch-ok' in out.stdout
