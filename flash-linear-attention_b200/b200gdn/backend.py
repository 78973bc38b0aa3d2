"""Plug-in for the reference's operator-dispatch registry.

The reference dispatches ``chunk_gated_delta_rule`` through ``@dispatch('gated_delta_rule')``
(fla/ops/backends/__init__.py:160-220): registered ``BaseBackend`` objects are tried by priority; a
backend offers a method named after the dispatched function plus ``<name>_verifier`` returning
``(ok, reason)``.  ``install()`` registers this backend there exactly as FlashQLABackend is registered
(fla/ops/gated_delta_rule/backends/__init__.py:14-17) and rebinds the decode function, which has no
dispatch slot (fla/layers/gated_deltanet.py:22 imports it by name).

``fla`` is optional: without it the class derives from a local stand-in with the same attributes, so
the verifier logic can be used and tested on its own.
"""
from __future__ import annotations

import os
from typing import Optional, Tuple

import torch

from .chunk import _SUPPORTED_HEAD_DIMS, chunk_gated_delta_rule
from .fused_recurrent import fused_recurrent_gated_delta_rule

try:  # pragma: no cover - depends on the host environment
    from fla.ops.backends import BaseBackend as _Base
except Exception:  # fla not importable: same class attributes and helpers as fla/ops/backends/__init__.py:33-88
    class _Base:
        backend_type = 'base'
        package_name = None
        env_var = None
        default_enable = True
        priority = 5

        @classmethod
        def is_available(cls) -> bool:
            return True

        @classmethod
        def is_enabled(cls) -> bool:
            if cls.env_var is None:
                return True
            return os.environ.get(cls.env_var, '1' if cls.default_enable else '0') != '0'

        @classmethod
        def can_use(cls) -> bool:
            return cls.is_available() and cls.is_enabled()

        def verify(self, func_name, *args, **kwargs):
            verifier = getattr(self, f'{func_name}_verifier', None)
            if verifier is None:
                return True, None
            try:
                return verifier(*args, **kwargs)
            except Exception as e:  # a verifier that raises means "cannot handle"
                return False, str(e)


class B200GDNBackend(_Base):
    """sm_100a kernels for the gated delta rule.  Disable with ``FLA_B200_GDN=0``."""

    backend_type = 'b200_gdn'
    package_name = None
    env_var = 'FLA_B200_GDN'
    default_enable = True
    priority = 2   # ahead of flash_qla (3) and the default Triton path

    @classmethod
    def is_available(cls) -> bool:
        if not torch.cuda.is_available():
            return False
        major, _ = torch.cuda.get_device_capability()
        from ._lib import LIB_PATH
        return major == 10 and os.path.exists(LIB_PATH)

    def chunk_gated_delta_rule_verifier(
        self, q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
        use_qk_l2norm_in_kernel=False, use_beta_sigmoid_in_kernel=False, allow_neg_eigval=False,
        state_v_first=False, cu_seqlens=None, cu_seqlens_cpu=None, chunk_indices=None, cp_context=None,
        **kwargs,
    ) -> Tuple[bool, Optional[str]]:
        if not q.is_cuda:
            return False, 'inputs are not on a CUDA device'
        # the tensor-core kernels compute on bf16 operands; other dtypes go to the reference's own path, which keeps
        # their precision (the direct function would round them to bf16)
        if not (q.dtype == k.dtype == v.dtype == torch.bfloat16):
            return False, f'q/k/v dtypes {q.dtype}/{k.dtype}/{v.dtype}: only bf16 is served'
        if (q.shape[-1], v.shape[-1]) not in _SUPPORTED_HEAD_DIMS:
            return False, f'head dims K={q.shape[-1]} V={v.shape[-1]} not built'
        if q.ndim != 4 or v.ndim != 4 or g.ndim != 3 or beta.ndim != 3:
            return False, 'expected q,k [B,T,H,K], v [B,T,HV,V], g,beta [B,T,HV]'
        if v.shape[2] % q.shape[2] != 0:
            return False, 'HV must be a multiple of H'
        if 'head_first' in kwargs:
            return False, 'head_first layout'
        return True, None

    def chunk_gated_delta_rule(self, q, k, v, g, beta, scale=None, initial_state=None, output_final_state=False,
                               use_qk_l2norm_in_kernel=False, use_beta_sigmoid_in_kernel=False,
                               allow_neg_eigval=False, state_v_first=False, cu_seqlens=None, cu_seqlens_cpu=None,
                               chunk_indices=None, cp_context=None, **kwargs):
        return chunk_gated_delta_rule(
            q, k, v, g, beta, scale=scale, initial_state=initial_state, output_final_state=output_final_state,
            use_qk_l2norm_in_kernel=use_qk_l2norm_in_kernel, use_beta_sigmoid_in_kernel=use_beta_sigmoid_in_kernel,
            allow_neg_eigval=allow_neg_eigval, state_v_first=state_v_first, cu_seqlens=cu_seqlens,
            cu_seqlens_cpu=cu_seqlens_cpu, chunk_indices=chunk_indices, cp_context=cp_context, **kwargs)


_saved = {}


def install() -> bool:
    """Register the backend with the reference's registry and rebind its decode function.
    Returns False (and does nothing) when ``fla`` is not importable."""
    try:
        import fla.layers.gated_deltanet as layer_mod
        import fla.ops.gated_delta_rule as op_mod
        from fla.ops.gated_delta_rule.backends import gdr_registry
    except Exception:
        return False
    gdr_registry.register(B200GDNBackend())
    if 'layer' not in _saved:
        _saved['layer'] = layer_mod.fused_recurrent_gated_delta_rule
        _saved['op'] = op_mod.fused_recurrent_gated_delta_rule
    layer_mod.fused_recurrent_gated_delta_rule = fused_recurrent_gated_delta_rule
    op_mod.fused_recurrent_gated_delta_rule = fused_recurrent_gated_delta_rule
    return True


def uninstall() -> None:
    """Undo install()."""
    try:
        import fla.layers.gated_deltanet as layer_mod
        import fla.ops.gated_delta_rule as op_mod
        from fla.ops.gated_delta_rule.backends import gdr_registry
    except Exception:
        return
    with gdr_registry._lock:
        gdr_registry._backends.pop(B200GDNBackend.backend_type, None)
        gdr_registry._active = None
        gdr_registry._update_active_backend()
    if 'layer' in _saved:
        layer_mod.fused_recurrent_gated_delta_rule = _saved.pop('layer')
        op_mod.fused_recurrent_gated_delta_rule = _saved.pop('op')
