"""ctypes binding of ``libbsx.so``, the C-ABI CUDA library (``include/bsx.h``).

The library is the only compute path of this package: there is no CPU or
PyTorch fallback.  If the shared object is missing, :func:`lib` raises; if a call
fails, :class:`BsxError` carries the library's status and message.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, 'libbsx.so')

BSX_OK = 0
BSX_ERR_INVALID_ARG = -1
BSX_ERR_CUDA = -2
BSX_ERR_INDEX_RANGE = -3
BSX_ERR_WORKSPACE = -4
BSX_ERR_UNSUPPORTED = -5
BSX_ERR_TIMEOUT = -6
BSX_ERR_NONFINITE = -7

VECMAT_GLOBAL_ATOMICS, VECMAT_SHARED_SLICES = 0, 1
LINK_EARLY_PUSH, LINK_FETCH_AHEAD, LINK_DEFAULT = 1, 2, 3
SPK_BOOL8, SPK_F32, SPK_BITS32, SPK_LIST = 0, 1, 2, 3


class BsxError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f'bsx call failed with status {status}: {message}')
        self.status = status


class BsxConn(C.Structure):
    """Mirror of ``bsx_conn_t``."""
    _fields_ = [
        ('n_pre', C.c_int64),
        ('n_post', C.c_int64),
        ('conn_num', C.c_int64),
        ('nnz', C.c_int64),
        ('indices', C.c_void_p),
        ('indptr', C.c_void_p),
        ('indptr_is_64', C.c_int32),
        ('hetero', C.c_int32),
        ('weights', C.c_void_p),
    ]


class BsxLifParams(C.Structure):
    """Mirror of ``bsx_lif_params_t``."""
    _fields_ = [(n, C.c_float) for n in ('dt', 'decay_e', 'decay_i', 'inv_tau_m', 'cuba_gain', 'V_rest', 'V_th',
                                         'V_reset', 'R', 'I_ext', 'E_e', 'E_i')] + \
               [('ref_steps', C.c_int32), ('coba', C.c_int32), ('ext_threshold', C.c_uint32),
                ('ext_seed', C.c_uint32), ('ext_weight', C.c_float)]


class BsxNet(C.Structure):
    """Mirror of ``bsx_net_t``."""
    _fields_ = [
        ('n_global', C.c_int64), ('n_exc', C.c_int64), ('first', C.c_int64), ('n_local', C.c_int64),
        ('exc', BsxConn), ('inh', BsxConn),
        ('V', C.c_void_p), ('g_e', C.c_void_p), ('g_i', C.c_void_p), ('ref', C.c_void_p),
        ('delta_e', C.c_void_p), ('delta_i', C.c_void_p), ('bits', C.c_void_p),
        ('lists', C.c_void_p), ('ring', C.c_int32), ('delay_e', C.c_int32), ('delay_i', C.c_int32),
    ]


class BsxNetShard(C.Structure):
    """Mirror of ``bsx_net_shard_t``."""
    _fields_ = [
        ('n_global', C.c_int64), ('n_exc', C.c_int64), ('first', C.c_int64), ('n_local', C.c_int64),
        ('exc', BsxConn), ('inh', BsxConn),
        ('V', C.c_void_p), ('g_e', C.c_void_p), ('g_i', C.c_void_p), ('ref', C.c_void_p),
        ('incr_e', C.c_void_p), ('incr_i', C.c_void_p), ('bits', C.c_void_p),
        ('ring', C.c_int32), ('delay_e', C.c_int32), ('delay_i', C.c_int32), ('fixed_point', C.c_int32),
    ]


class BsxNetLinks(C.Structure):
    """Mirror of ``bsx_net_links_t``."""
    _fields_ = [('world', C.c_int32), ('rank', C.c_int32), ('blocks', C.c_int32), ('words_per_block', C.c_int32),
                ('words_per_rank', C.c_int64), ('slots', C.c_int32), ('slack', C.c_int32),
                ('spin_limit', C.c_int64), ('seq0', C.c_int64), ('inbox', C.c_void_p * 16), ('sync', C.c_void_p), ('flags', C.c_int32)]


_i64, _i32, _vp, _sz, _f32 = C.c_int64, C.c_int, C.c_void_p, C.c_size_t, C.c_float
_connp = C.POINTER(BsxConn)
_netp = C.POINTER(BsxNet)
_lifp = C.POINTER(BsxLifParams)

# name -> (restype, argtypes); every symbol include/bsx.h declares, plus the two tuning hooks of
# csrc/bsx_tuning.h (INTERNAL lists them)
SIGNATURES = {
    'bsx_version': (_i32, []),
    'bsx_last_error_string': (C.c_char_p, []),
    'bsx_status_name': (C.c_char_p, [_i32]),
    'bsx_device_count': (_i32, []),
    'bsx_read_status': (_i32, [_vp, C.POINTER(C.c_int32), _vp]),
    'bsx_host_fixed_num_indices': (_i64, [C.c_uint32, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _vp, _vp]),
    'bsx_host_gen_new': (_vp, [C.c_uint32]),
    'bsx_host_gen_free': (None, [_vp]),
    'bsx_host_gen_rows': (_i64, [_vp, _i64, _i64, _i64, _i64, _i64, _vp, _vp, _vp]),
    'bsx_host_distinct_indices': (_i64, [C.c_uint32, _i64, _i64, _i64, _vp]),
    'bsx_lognormal_weights': (_i32, [_connp, _vp, _i64, C.c_uint32, C.c_double, C.c_double, _f32, _vp, _vp]),
    'bsx_lognormal_weight_at': (_f32, [C.c_uint32, C.c_uint32, C.c_uint32, C.c_double, C.c_double, _f32]),
    'bsx_validate_conn': (_i32, [_connp, _vp, _vp]),
    'bsx_pack_spikes': (_i32, [_vp, _i32, _i64, _i64, _vp, _vp]),
    'bsx_transpose_workspace_bytes': (_sz, [_i64, _i64, _i64]),
    'bsx_transpose_build': (_i32, [_connp, _i64, _vp, _vp, _vp, _vp, _sz, _vp]),
    'bsx_permute_f32': (_i32, [_vp, _vp, _i64, _vp, _vp]),
    'bsx_event_vecmat_workspace_bytes': (_sz, [_i64, _i64]),
    'bsx_event_vecmat': (_i32, [_connp, _vp, _i32, _i64, _vp, _i32, _vp, _sz, _vp]),
    'bsx_event_vecmat_tuned': (_i32, [_connp, _vp, _i32, _i64, _vp, _i32, _vp, _sz, _i32, _i32, _vp]),
    'bsx_event_vecmat_variant': (_i32, [_connp, _i32, _i64]),
    'bsx_event_vecmat_launches': (_i32, [_connp, _i32, _i64]),
    'bsx_sliced_slices': (_i64, [_i64]),
    'bsx_sliced_build': (_i32, [_connp, _vp, _vp, _vp, _vp]),
    'bsx_event_vecmat_sliced': (_i32, [_connp, _vp, _i32, _i64, _vp, _i32, _vp]),
    'bsx_fixed_scale_workspace_bytes': (_sz, [_i64]),
    'bsx_fixed_scale_log2': (_i32, [_connp, _vp, _sz, C.POINTER(C.c_int32), _vp]),
    'bsx_event_vecmat_sliced_fixed': (_i32, [_connp, _vp, _i32, _i64, _vp, _i32, _i32, _vp]),
    'bsx_event_vecmat_chained': (_i32, [_connp, _vp, _i32, _i64, _vp, _vp, _vp]),
    'bsx_sliced_compress': (_i32, [_connp, _vp, _vp]),
    'bsx_quantize_f32': (_i32, [_vp, _i64, _i32, _vp, _vp]),
    'bsx_event_vecmat_sliced16': (_i32, [_connp, _vp, _vp, _vp, _i32, _i64, _vp, _i32, _i32, _vp]),
    'bsx_event_vecmat_static': (_i32, [_connp, _vp, _i32, _i64, _vp, _i32, _vp]),
    'bsx_float_vecmat': (_i32, [_connp, _vp, _i64, _vp, _i32, _vp, _sz, _vp]),
    'bsx_event_matvec_workspace_bytes': (_sz, [_i64, _i64]),
    'bsx_event_matvec': (_i32, [_connp, _vp, _i32, _i64, _vp, _vp, _sz, _vp]),
    'bsx_event_matvec_tuned': (_i32, [_connp, _vp, _i32, _i64, _vp, _vp, _sz, _i32, _i32, _i32, _vp]),
    'bsx_float_matvec': (_i32, [_connp, _vp, _i64, _vp, _vp]),
    'bsx_vecmat_vjp': (_i32, [_connp, _vp, _i32, _i32, _vp, _i64, _vp, _vp, _vp]),
    'bsx_vecmat_vjp_batched_workspace_bytes': (_sz, [_i64, _i64]),
    'bsx_vecmat_vjp_batched': (_i32, [_connp, _vp, _i32, _i32, _vp, _i64, _vp, _vp, _vp, _sz, _vp]),
    'bsx_dense_event_vecmat': (_i32, [_vp, _i32, _vp, _i64, _i64, _i64, _vp, _vp]),
    'bsx_dense_event_dw': (_i32, [_vp, _i32, _vp, _i64, _i64, _i64, _vp, _vp]),
    'bsx_dense_event_scalar': (_i32, [_vp, _i32, _vp, _i32, _i64, _i64, _i64, _vp, _vp, _vp]),
    'bsx_net_run': (_i32, [_netp, _lifp, _i32, _i64, _vp, _vp, _i32, _vp]),
    'bsx_net_update': (_i32, [_netp, _lifp, _i64, _vp, _vp]),
    'bsx_net_list_from_bits': (_i32, [_netp, _i64, _vp]),
    'bsx_net_list_from_bits_part': (_i32, [_netp, _i64, _i64, _i64, _i32, _vp, _vp]),
    'bsx_net_scatter_part': (_i32, [_netp, _i64, _vp, _i32, _vp]),
    'bsx_net_scatter': (_i32, [_netp, _i64, _vp]),
    'bsx_net_shard_geometry': (_i32, [_i64, C.POINTER(C.c_int32), C.POINTER(C.c_int32)]),
    'bsx_net_inbox_bytes': (_sz, [_i32, _i32, _i32, _i32]),
    'bsx_net_run_sharded': (_i32, [C.POINTER(BsxNetShard), _lifp, C.POINTER(BsxNetLinks), _i32, _i64, _vp, _vp, _vp]),
    'bsx_ipc_alloc': (_i32, [_sz, C.POINTER(C.c_void_p), _vp]),
    'bsx_ipc_open': (_i32, [_vp, C.POINTER(C.c_void_p)]),
    'bsx_ipc_close': (_i32, [_vp]),
    'bsx_ipc_free': (_i32, [_vp]),
    'bsx_drive_hash': (C.c_uint32, [C.c_uint32, C.c_uint32, C.c_uint32]),
    'bsx_fill_f32': (_i32, [_vp, _i64, _f32, _vp]),
}

INTERNAL = ('bsx_event_vecmat_tuned', 'bsx_event_matvec_tuned')

_lib = None


def lib():
    """The loaded library.  Raises if ``libbsx.so`` has not been built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f'{LIB_PATH} is missing: build it with `python -m brainstate_b200.build` '
                '(nvcc, sm_100a).  This package has no fallback implementation.')
        handle = C.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)      # AttributeError here = header/library mismatch
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(status: int) -> int:
    """Raises :class:`BsxError` for a negative status; returns it otherwise."""
    if status < 0:
        raise BsxError(int(status), lib().bsx_last_error_string().decode())
    return status


def current_stream() -> int:
    import torch
    return torch.cuda.current_stream().cuda_stream


def ptr(t) -> int | None:
    """Device address of a torch tensor (``None`` passes NULL)."""
    return None if t is None else t.data_ptr()
