"""ctypes binding of ``oracle/bsx_oracle.c`` (test infrastructure only).

``build()`` compiles ``liboracle.so`` beside the source with gcc; ``lib()`` loads
it.  See the C file for which reference lines each function restates.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, 'liboracle.so')
_SRC = os.path.join(_HERE, 'bsx_oracle.c')
_lib = None


def build(force: bool = False) -> str:
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(_SRC):
        # -march=native is avoided: the library is built on one machine and run on another.
        cmd = ['gcc', '-O3', '-fopenmp', '-fPIC', '-shared', '-o', _SO, _SRC]
        subprocess.run(cmd, check=True)
    return _SO


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_SO):
            build()
        _lib = C.CDLL(_SO)
        _lib.orc_mt_state_bytes.restype = C.c_size_t
        _lib.orc_num_threads.restype = C.c_int
    return _lib


def _p(a, t):
    return a.ctypes.data_as(C.POINTER(t)) if a is not None else None


def fixed_num_indices(seed, n_pre, n_post, K):
    out = np.empty((n_pre, K), np.int32)
    lib().orc_fixed_num_indices(C.c_uint32(seed), C.c_int64(n_pre), C.c_int64(n_post), C.c_int64(K),
                                _p(out, C.c_int32))
    return out


class MT:
    """A seeded MT19937 stream with NumPy's legacy ``randint``/``random_sample`` draws."""

    def __init__(self, seed):
        self._st = C.create_string_buffer(lib().orc_mt_state_bytes())
        lib().orc_mt_seed(self._st, C.c_uint32(seed))

    def randint(self, n_post, count):
        out = np.empty(count, np.int32)
        lib().orc_randint_fill(self._st, C.c_int64(n_post), C.c_int64(count), _p(out, C.c_int32))
        return out

    def random_sample(self, count):
        out = np.empty(count, np.float64)
        lib().orc_random_sample(self._st, C.c_int64(count), _p(out, C.c_double))
        return out


def _conn_args(idx, w, indptr, n_pre):
    idx = np.ascontiguousarray(idx, np.int32)
    w = np.ascontiguousarray(np.asarray(w, np.float32).reshape(-1))
    hetero = int(w.size == idx.size and np.ndim(w) > 0 and idx.size > 1 or (w.size == idx.size and w.size > 1))
    if w.size != idx.size:
        assert w.size == 1
        hetero = 0
    K = idx.size // max(n_pre, 1) if indptr is None else 0
    ip = None if indptr is None else np.ascontiguousarray(indptr, np.int64)
    return idx, w, hetero, K, ip


def event_vecmat_u8(spk, idx, w, n_post, indptr=None, split_rows=False):
    """``split_rows``: for timing on many cores with few vectors — the active rows of a vector are
    divided among the threads (sums then differ from the sequential order within rounding)."""
    spk = np.ascontiguousarray(spk, np.uint8)
    n_pre = spk.shape[-1]
    sb = spk.reshape(-1, n_pre)
    idx, w, hetero, K, ip = _conn_args(idx, w, indptr, n_pre)
    y = np.empty((sb.shape[0], n_post), np.float32)
    fn = lib().orc_event_vecmat_u8_par if split_rows else lib().orc_event_vecmat_u8
    fn(_p(sb, C.c_uint8), C.c_int64(sb.shape[0]), C.c_int64(n_pre), C.c_int64(n_post),
                              C.c_int64(K), _p(ip, C.c_int64), _p(idx, C.c_int32), _p(w, C.c_float),
                              C.c_int(hetero), _p(y, C.c_float))
    return y.reshape(spk.shape[:-1] + (n_post,))


def float_vecmat(x, idx, w, n_post, indptr=None, event=False):
    x = np.ascontiguousarray(x, np.float32)
    n_pre = x.shape[-1]
    xb = x.reshape(-1, n_pre)
    idx, w, hetero, K, ip = _conn_args(idx, w, indptr, n_pre)
    y = np.empty((xb.shape[0], n_post), np.float32)
    lib().orc_float_vecmat(_p(xb, C.c_float), C.c_int64(xb.shape[0]), C.c_int64(n_pre), C.c_int64(n_post),
                           C.c_int64(K), _p(ip, C.c_int64), _p(idx, C.c_int32), _p(w, C.c_float),
                           C.c_int(hetero), C.c_int(int(event)), _p(y, C.c_float))
    return y.reshape(x.shape[:-1] + (n_post,))


def float_matvec(v, idx, w, n_pre, indptr=None, event=False):
    v = np.ascontiguousarray(v, np.float32)
    n_post = v.shape[-1]
    vb = v.reshape(-1, n_post)
    idx, w, hetero, K, ip = _conn_args(idx, w, indptr, n_pre)
    y = np.empty((vb.shape[0], n_pre), np.float32)
    lib().orc_float_matvec(_p(vb, C.c_float), C.c_int64(vb.shape[0]), C.c_int64(n_pre), C.c_int64(n_post),
                           C.c_int64(K), _p(ip, C.c_int64), _p(idx, C.c_int32), _p(w, C.c_float),
                           C.c_int(hetero), C.c_int(int(event)), _p(y, C.c_float))
    return y.reshape(v.shape[:-1] + (n_pre,))


def event_matvec_u8(spk, idx, w, n_pre, indptr=None):
    spk = np.ascontiguousarray(spk, np.uint8)
    n_post = spk.shape[-1]
    sb = spk.reshape(-1, n_post)
    idx, w, hetero, K, ip = _conn_args(idx, w, indptr, n_pre)
    y = np.empty((sb.shape[0], n_pre), np.float32)
    lib().orc_event_matvec_u8(_p(sb, C.c_uint8), C.c_int64(sb.shape[0]), C.c_int64(n_pre), C.c_int64(n_post),
                              C.c_int64(K), _p(ip, C.c_int64), _p(idx, C.c_int32), _p(w, C.c_float),
                              C.c_int(hetero), _p(y, C.c_float))
    return y.reshape(spk.shape[:-1] + (n_pre,))


def transpose(idx, n_pre, n_post, indptr=None):
    """Column-major copy: ``(t_indptr int64 (n_post+1,), t_rows int32 (nnz,), t_perm int64 (nnz,))``."""
    idx = np.ascontiguousarray(idx, np.int32)
    K = idx.size // max(n_pre, 1) if indptr is None else 0
    ip = None if indptr is None else np.ascontiguousarray(indptr, np.int64)
    t_indptr = np.empty(n_post + 1, np.int64)
    t_rows = np.empty(idx.size, np.int32)
    t_perm = np.empty(idx.size, np.int64)
    lib().orc_transpose(C.c_int64(n_pre), C.c_int64(n_post), C.c_int64(K), _p(ip, C.c_int64), _p(idx, C.c_int32),
                        _p(t_indptr, C.c_int64), _p(t_rows, C.c_int32), _p(t_perm, C.c_int64))
    return t_indptr, t_rows, t_perm


def vecmat_dw(x, ct, idx, n_pre, n_post, indptr=None, event=False):
    x = np.ascontiguousarray(x, np.float32).reshape(-1, n_pre)
    ct = np.ascontiguousarray(ct, np.float32).reshape(-1, n_post)
    idx = np.ascontiguousarray(idx, np.int32)
    K = idx.size // max(n_pre, 1) if indptr is None else 0
    ip = None if indptr is None else np.ascontiguousarray(indptr, np.int64)
    dw = np.empty(idx.shape, np.float32)
    lib().orc_vecmat_dw(_p(x, C.c_float), _p(ct, C.c_float), C.c_int64(x.shape[0]), C.c_int64(n_pre),
                        C.c_int64(n_post), C.c_int64(K), _p(ip, C.c_int64), _p(idx, C.c_int32),
                        C.c_int(int(event)), _p(dw, C.c_float))
    return dw


def num_threads():
    return int(lib().orc_num_threads())


def use_all_cores():
    """Sets the OpenMP thread count to the cores this process may run on (launchers
    like torchrun export OMP_NUM_THREADS=1).  Returns the count."""
    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    lib().orc_set_threads(C.c_int(n))
    return num_threads()
