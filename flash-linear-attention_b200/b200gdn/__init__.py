"""b200gdn: the gated delta rule (Gated DeltaNet token mixer) on NVIDIA B200.

Drop-in replacements for ``fla.ops.gated_delta_rule.chunk_gated_delta_rule`` and
``fla.ops.gated_delta_rule.fused_recurrent_gated_delta_rule`` backed by hand-written sm_100a kernels in
``libb200gdn.so`` (C ABI: include/b200gdn.h).  There is no fallback path.
"""
from ._lib import B200GDNError, device_status, launch_count, load as load_library
from .chunk import chunk_gated_delta_rule, chunk_gdn
from .fused_recurrent import fused_recurrent_gated_delta_rule, fused_recurrent_gdn
from .cp import FLACPContext, build_cp_context, get_cp_cu_seqlens
from .backend import B200GDNBackend, install, uninstall
from .modules import FusedRMSNormGated, ShortConvolution, causal_conv1d, rms_norm_gated

__version__ = '0.1.0'
__all__ = [
    'chunk_gated_delta_rule', 'chunk_gdn', 'fused_recurrent_gated_delta_rule', 'fused_recurrent_gdn',
    'FLACPContext', 'build_cp_context', 'get_cp_cu_seqlens', 'B200GDNBackend', 'install', 'uninstall',
    'B200GDNError', 'load_library', 'launch_count', 'device_status',
    'causal_conv1d', 'ShortConvolution', 'rms_norm_gated', 'FusedRMSNormGated',
]
