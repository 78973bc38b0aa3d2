"""ctypes binding of libb200gdn.so (the C ABI declared in include/b200gdn.h).

The library is the only compute path of this package: when it cannot be loaded every operator
raises, there is no fallback.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, 'libb200gdn.so')

ABI_VERSION = 1

FWD_INTRA, FWD_SCAN, FWD_OUT = 1, 2, 4
BWD_DVLOCAL, BWD_SCAN, BWD_DQKWG, BWD_WY = 1, 2, 4, 8
REC_L2NORM, REC_GATE, REC_BETA_SIGMOID, REC_NEG_EIGVAL, REC_STATE_V_FIRST = 1, 2, 4, 8, 16

_p = C.c_void_p


class ChunkArgs(C.Structure):
    _fields_ = [
        ('struct_bytes', C.c_int32), ('rows', C.c_int32), ('H', C.c_int32), ('HV', C.c_int32),
        ('K', C.c_int32), ('V', C.c_int32), ('n_seq', C.c_int32), ('n_chunks', C.c_int32),
        ('scale', C.c_float), ('stage_mask', C.c_uint32),
        ('chunk_meta', _p), ('seq_meta', _p),
        ('q', _p), ('k', _p), ('v', _p), ('g', _p), ('beta', _p), ('h0', _p),
        ('o', _p), ('ht', _p),
        ('gamma', _p), ('A', _p), ('w', _p), ('u', _p), ('h', _p), ('v_new', _p),
        ('d_o', _p), ('dht', _p),
        ('dq', _p), ('dk', _p), ('dv', _p), ('dg', _p), ('dbeta', _p), ('dh0', _p),
        ('dh', _p), ('dv2', _p), ('dw', _p), ('dk_part', _p), ('dG', _p), ('dq_acc', _p),
        ('options', C.c_uint32), ('A_log', _p), ('dt_bias', _p), ('gate_partials', _p), ('dA_log', _p), ('ddt_bias', _p),
        ('cp_M', _p), ('cp_dM', _p), ('qk', _p), ('rstd_q', _p), ('rstd_k', _p),
    ]


class RecurrentArgs(C.Structure):
    _fields_ = [
        ('struct_bytes', C.c_int32), ('B', C.c_int32), ('T', C.c_int32), ('H', C.c_int32), ('HV', C.c_int32),
        ('K', C.c_int32), ('V', C.c_int32), ('n_seq', C.c_int32), ('scale', C.c_float), ('flags', C.c_uint32),
        ('qkv_dtype', C.c_int32),
        ('cu_seqlens', _p), ('q', _p), ('k', _p), ('v', _p), ('g', _p), ('beta', _p), ('A_log', _p),
        ('dt_bias', _p), ('h0', _p), ('o', _p), ('ht', _p), ('state_indices', _p), ('n_slots', C.c_int32),
    ]


PREP_L2NORM, PREP_GATE, PREP_BETA_SIGMOID, PREP_NEG_EIGVAL = 1, 2, 4, 8
STATE_V_FIRST = 16   # chunk passes: h0, ht, dht, dh0 stored [N,HV,V,K]
PREP_PART_ROWS = 128


class PrepArgs(C.Structure):
    _fields_ = [
        ('struct_bytes', C.c_int32), ('rows', C.c_int32), ('H', C.c_int32), ('HV', C.c_int32), ('K', C.c_int32),
        ('flags', C.c_uint32), ('qk_dtype', C.c_int32), ('gb_dtype', C.c_int32),
        ('q', _p), ('k', _p), ('g', _p), ('beta', _p), ('A_log', _p), ('dt_bias', _p),
        ('qn', _p), ('kn', _p), ('rstd_q', _p), ('rstd_k', _p), ('g_out', _p), ('beta_out', _p),
        ('dqn', _p), ('dkn', _p), ('dg', _p), ('dbeta', _p),
        ('dq', _p), ('dk', _p), ('dg_raw', _p), ('dbeta_raw', _p), ('dA_log', _p), ('ddt_bias', _p), ('partials', _p),
    ]


class AffineArgs(C.Structure):
    _fields_ = [
        ('struct_bytes', C.c_int32), ('HV', C.c_int32), ('K', C.c_int32), ('V', C.c_int32),
        ('transpose_m', C.c_int32),
        ('M', _p), ('x', _p), ('b', _p), ('out', _p),
    ]


class ConvArgs(C.Structure):
    _fields_ = [
        ('struct_bytes', C.c_int32), ('rows', C.c_int32), ('D', C.c_int32), ('W', C.c_int32),
        ('n_seq', C.c_int32), ('n_tiles', C.c_int32), ('flags', C.c_uint32), ('dtype', C.c_int32),
        ('tile_meta', _p), ('seq_meta', _p), ('x', _p), ('weight', _p), ('bias', _p), ('residual', _p),
        ('initial_state', _p), ('y', _p), ('final_state', _p),
        ('dy', _p), ('dx', _p), ('dweight', _p), ('dbias', _p), ('dinitial_state', _p), ('partials', _p),
    ]


class NormGateArgs(C.Structure):
    _fields_ = [
        ('struct_bytes', C.c_int32), ('D', C.c_int32), ('rows', C.c_int64), ('flags', C.c_uint32),
        ('dtype', C.c_int32), ('eps', C.c_float),
        ('x', _p), ('g', _p), ('weight', _p), ('bias', _p), ('y', _p), ('rstd', _p),
        ('dy', _p), ('dx', _p), ('dg', _p), ('dweight', _p), ('dbias', _p), ('partials', _p),
    ]


CONV_SILU = 1
NORM_GATE_SIGMOID = 1


class PrefixArgs(C.Structure):
    _fields_ = [
        ('struct_bytes', C.c_int32), ('HV', C.c_int32), ('K', C.c_int32), ('V', C.c_int32),
        ('n_chains', C.c_int32), ('reverse', C.c_int32), ('identity', C.c_int32),
        ('table', _p), ('M', _p), ('h', _p), ('x0', _p), ('out', _p), ('last', _p),
    ]


class FoldArgs(C.Structure):
    _fields_ = [
        ('struct_bytes', C.c_int32), ('HV', C.c_int32), ('K', C.c_int32), ('V', C.c_int32),
        ('first', C.c_int32), ('count', C.c_int32), ('step', C.c_int32),
        ('gathered', _p), ('out', _p),
    ]


EXPORTS = (
    'b200gdn_chunk_fwd', 'b200gdn_chunk_bwd', 'b200gdn_recurrent_fwd', 'b200gdn_affine_apply',
    'b200gdn_saved_bytes', 'b200gdn_bwd_workspace_bytes', 'b200gdn_last_launch_count',
    'b200gdn_abi_version', 'b200gdn_last_error', 'b200gdn_device_status', 'b200gdn_prep_fwd', 'b200gdn_prep_bwd',
    'b200gdn_selftest_wait_expiry', 'b200gdn_chunk_fwd_static', 'b200gdn_cp_fold', 'b200gdn_cp_prefix',
    'b200gdn_conv_fwd', 'b200gdn_conv_bwd', 'b200gdn_norm_gate_fwd', 'b200gdn_norm_gate_bwd', 'b200gdn_norm_gate_ctas',
)

_lib = None
_lock = threading.Lock()


class B200GDNError(RuntimeError):
    pass


def load():
    """Load the shared library once; raises if it is missing or its ABI version differs."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        if not os.path.exists(LIB_PATH):
            raise B200GDNError(
                f'{LIB_PATH} is missing: build it with `make -C flash-linear-attention_b200/csrc` '
                '(or __graft_entry__.build()). There is no fallback path.')
        lib = C.CDLL(LIB_PATH)
        for name in ('b200gdn_chunk_fwd', 'b200gdn_chunk_bwd', 'b200gdn_recurrent_fwd', 'b200gdn_affine_apply',
                     'b200gdn_prep_fwd', 'b200gdn_prep_bwd', 'b200gdn_chunk_fwd_static', 'b200gdn_cp_fold', 'b200gdn_cp_prefix',
                     'b200gdn_conv_fwd', 'b200gdn_conv_bwd', 'b200gdn_norm_gate_fwd', 'b200gdn_norm_gate_bwd'):
            fn = getattr(lib, name)
            fn.restype = C.c_int
            fn.argtypes = [C.c_void_p, C.c_void_p]
        for name in ('b200gdn_saved_bytes', 'b200gdn_bwd_workspace_bytes'):
            fn = getattr(lib, name)
            fn.restype = C.c_int64
            fn.argtypes = [C.c_int32] * 6
        lib.b200gdn_norm_gate_ctas.restype = C.c_int
        lib.b200gdn_norm_gate_ctas.argtypes = [C.c_int64]
        lib.b200gdn_last_launch_count.restype = C.c_int
        lib.b200gdn_device_status.restype = C.c_int
        lib.b200gdn_device_status.argtypes = []
        lib.b200gdn_selftest_wait_expiry.restype = C.c_int
        lib.b200gdn_selftest_wait_expiry.argtypes = [C.c_void_p]
        lib.b200gdn_abi_version.restype = C.c_int
        lib.b200gdn_last_error.restype = C.c_char_p
        if lib.b200gdn_abi_version() != ABI_VERSION:
            raise B200GDNError(f'ABI version {lib.b200gdn_abi_version()} != {ABI_VERSION}: rebuild the library')
        _lib = lib
    return _lib


_launches = 0


def launch_count() -> int:
    """Kernels enqueued through this binding since import (benchmark bookkeeping)."""
    return _launches


def call(name: str, args: C.Structure, stream: int) -> None:
    global _launches
    lib = load()
    args.struct_bytes = C.sizeof(args)
    rc = getattr(lib, name)(C.byref(args), C.c_void_p(stream))
    if rc != 0:
        raise B200GDNError(f'{name} failed ({rc}): {lib.b200gdn_last_error().decode()}')
    _launches += lib.b200gdn_last_launch_count()


def device_status() -> None:
    """Synchronise the current device and raise if a bounded wait inside one of the kernels expired since the
    last check (the flagged kernel's results are invalid)."""
    lib = load()
    rc = lib.b200gdn_device_status()
    if rc != 0:
        raise B200GDNError(f'b200gdn_device_status ({rc}): {lib.b200gdn_last_error().decode()}')


def ptr(t):
    return None if t is None else t.data_ptr()
