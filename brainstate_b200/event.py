"""Event-driven sparse products on the GPU: the operator layer.

This module plays the part ``brainevent`` plays under the reference's
``brainstate/nn/_event_fixedprob.py``: container types for the connectivity
(``FixedPostNumConn``, ``CSR``), the spike wrapper ``EventArray`` and the ``@``
products between them, each differentiable (reverse and forward mode) and
accepting leading batch dimensions.  All arithmetic is done by ``libbsx.so``
through its C ABI on CUDA tensors; there is no other implementation.

Reference call sites replaced (``brainstate/nn/_event_fixedprob.py``):
``:176-181`` (``FixedPostNumConn``), ``:191-196`` (``CSR``), ``:204-205``
(``with_data`` + ``x @ csr``), ``:251`` (``EventArray``).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import numpy as np
import torch

from . import _lib
from ._lib import BsxConn, check, lib, ptr

__all__ = ['EventArray', 'FixedPostNumConn', 'CSR', 'FixedPreNumConn', 'CSC', 'event_vecmat', 'float_vecmat',
           'event_matvec', 'float_matvec', 'pack_spikes', 'spike_format_of']


# The batched scatter reads the compressed form of the sliced copy (16-bit column offsets, weights
# stored in fixed point) wherever its sums are order-free; False keeps the 32-bit arrays.
PACKED_SLICES = True


def _require_cuda(t: torch.Tensor, what: str):
    if not t.is_cuda:
        raise RuntimeError(f'{what} must be a CUDA tensor: this package computes on the GPU only '
                           '(no CPU fallback exists)')


def spike_format_of(x: torch.Tensor) -> int:
    """C-ABI spike format of a tensor by dtype (bool/uint8 -> BOOL8, float32 -> F32)."""
    if x.dtype in (torch.bool, torch.uint8):
        return _lib.SPK_BOOL8
    if x.dtype == torch.float32:
        return _lib.SPK_F32
    raise TypeError(f'spikes must be bool, uint8 or float32, got {x.dtype}')


class EventArray:
    """Marks a tensor as a spike (event) vector: every nonzero entry is a unit
    event in the forward product (``brainstate/nn/_event_linear.py:82-85``)."""

    __slots__ = ('value',)

    def __init__(self, value):
        self.value = value.value if isinstance(value, EventArray) else value

    @property
    def shape(self):
        return self.value.shape

    def __matmul__(self, other):
        if isinstance(other, _SparseConn):
            return other._vecmat(self.value, event=True)
        if isinstance(other, _InDegreeConn):
            return other._gather(self.value, event=True)
        if isinstance(other, torch.Tensor):       # dense event product (EventLinear)
            from .nn._event_linear import dense_event_matmul
            return dense_event_matmul(self.value, other)
        return NotImplemented


class _Transposed:
    """Postsynaptic-major copy of a connectivity (built once on the device)."""

    def __init__(self, indptr, indices, perm, n_rows, n_cols):
        self.indptr, self.indices, self.perm = indptr, indices, perm
        self.n_rows, self.n_cols = n_rows, n_cols   # n_rows = n_post of the original


class _SparseConn:
    """Shared behaviour of the two out-degree layouts."""

    def __init__(self, data, indices: torch.Tensor, indptr: Optional[torch.Tensor], shape):
        _require_cuda(indices, 'indices')
        if indices.dtype != torch.int32:
            raise TypeError('indices must be int32')
        self.shape = (int(shape[0]), int(shape[1]))
        self.indices = indices.contiguous()
        self.indptr = None
        if indptr is not None:
            _require_cuda(indptr, 'indptr')
            if indptr.dtype not in (torch.int32, torch.int64):
                raise TypeError('indptr must be int32 or int64')
            if indptr.numel() != self.shape[0] + 1:
                raise ValueError('indptr must have n_pre + 1 entries')
            self.indptr = indptr.contiguous()
        # derived layouts (transposed copy, copies grouped by output slice) and their permuted
        # weights; ONE dict shared by reference with every ``with_data`` view, so that a layout
        # built through a view (every layer call makes one) is built once for all of them
        self._derived = {}
        self.matvec_method = 'gather'    # what ``conn @ EventArray`` uses; see ``event_matvec``
        self._set_data(data)

    # -- data ---------------------------------------------------------------
    def _set_data(self, data):
        if not isinstance(data, torch.Tensor):
            data = torch.as_tensor(np.asarray(data, dtype=np.float32), device=self.indices.device)
        _require_cuda(data, 'weights')
        if data.dtype != torch.float32:
            data = data.to(torch.float32)
        if data.dim() > 0 and data.numel() == self.indices.numel() and data.numel() > 0 \
                and tuple(data.shape) == tuple(self.indices.shape):
            self.hetero = True
        elif data.numel() == 1:
            self.hetero = False
        else:
            raise ValueError(f'weights of shape {tuple(data.shape)} match neither a scalar nor the '
                             f'indices {tuple(self.indices.shape)}')
        self.data = data

    def with_data(self, data):
        """A view of the same connectivity with other weights
        (``brainevent`` ``with_data``, used at ``_event_fixedprob.py:204``).  The view shares
        the derived layouts of the connectivity it was made from."""
        new = object.__new__(type(self))
        new.__dict__.update(self.__dict__)
        new._set_data(data)
        return new

    @property
    def nnz(self) -> int:
        return self.indices.numel()

    @property
    def conn_num(self) -> int:
        return 0 if self.indptr is not None else (self.indices.shape[-1] if self.indices.dim() == 2 else 0)

    def _struct(self, weights: Optional[torch.Tensor] = None, hetero: Optional[bool] = None) -> BsxConn:
        w = self.data if weights is None else weights
        h = self.hetero if hetero is None else hetero
        wc = w if w.is_contiguous() else w.contiguous()
        s = BsxConn()
        s.n_pre, s.n_post = self.shape
        s.conn_num = self.conn_num
        s.nnz = self.nnz
        s.indices = self.indices.data_ptr() if self.nnz else None
        s.indptr = None if self.indptr is None else self.indptr.data_ptr()
        s.indptr_is_64 = int(self.indptr is not None and self.indptr.dtype == torch.int64)
        s.hetero = int(h)
        s.weights = wc.data_ptr()
        s._keep = (wc,)            # keeps a contiguous copy alive for the call
        return s

    # -- validation / derived layouts ------------------------------------------
    def validate(self):
        """Range-checks the indices on the device; raises ``ValueError`` on a bad
        layout.  (The reference has no such check: a malformed layout aborts the
        process inside brainevent, ``_event_fixedprob.py:124-134``.)"""
        status = torch.zeros(1, dtype=torch.int32, device=self.indices.device)
        st = self._struct()
        check(lib().bsx_validate_conn(C.byref(st), ptr(status), _lib.current_stream()))
        host = C.c_int32(0)
        check(lib().bsx_read_status(ptr(status), C.byref(host), _lib.current_stream()))
        if host.value != 0:
            raise ValueError('connectivity indices out of range or malformed indptr '
                             f'({lib().bsx_status_name(host.value).decode()})')
        return self

    def transposed(self) -> _Transposed:
        """Builds (once) and returns the postsynaptic-major copy."""
        if 'transposed' not in self._derived:
            n_pre, n_post = self.shape
            dev = self.indices.device
            nnz = self.nnz
            t_indptr = torch.empty(n_post + 1, dtype=torch.int64, device=dev)
            t_indices = torch.empty(nnz, dtype=torch.int32, device=dev)
            t_perm = torch.empty(nnz, dtype=torch.int32, device=dev)
            ws_bytes = lib().bsx_transpose_workspace_bytes(n_pre, n_post, nnz)
            ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=dev)
            st = self._struct()
            check(lib().bsx_transpose_build(C.byref(st), nnz, ptr(t_indptr), ptr(t_indices), ptr(t_perm),
                                            ptr(ws), ws_bytes, _lib.current_stream()))
            self._derived['transposed'] = _Transposed(t_indptr, t_indices, t_perm, n_post, n_pre)
        return self._derived['transposed']

    def _permuted_weights(self, layout: str, weights: torch.Tensor, perm: torch.Tensor) -> torch.Tensor:
        """``weights`` (original order) re-gathered for a derived layout.  Kept until the weight
        tensor changes (new storage or an in-place update), so repeated products pay the
        4-byte-per-synapse gather once."""
        wsrc = weights.contiguous()
        key = (wsrc.data_ptr(), wsrc._version, wsrc.numel())
        cached = self._derived.get('w_' + layout)
        if cached is not None and cached[0] == key:
            return cached[1]
        out = torch.empty(self.nnz, dtype=torch.float32, device=weights.device)
        check(lib().bsx_permute_f32(ptr(wsrc), ptr(perm), self.nnz, ptr(out), _lib.current_stream()))
        self._derived['w_' + layout] = (key, out, wsrc)      # wsrc held so that its address cannot be reused
        return out

    def _transposed_struct(self, weights: torch.Tensor):
        """``bsx_conn_t`` of the transposed copy with the given (original-order) weights."""
        t = self.transposed()
        wt = self._permuted_weights('t', weights, t.perm) if self.hetero else weights.contiguous()
        s = BsxConn()
        s.n_pre, s.n_post = t.n_rows, t.n_cols
        s.conn_num = 0
        s.nnz = self.nnz
        s.indices = t.indices.data_ptr() if self.nnz else None
        s.indptr = t.indptr.data_ptr()
        s.indptr_is_64 = 1
        s.hetero = int(self.hetero)
        s.weights = wt.data_ptr()
        s._keep = (wt,)
        return s

    # -- rows grouped by output slice (for the batched scatter that keeps slices in shared memory)
    def _group_offsets(self, st: BsxConn, n_rows: int, regroup: bool):
        S = int(lib().bsx_sliced_slices(st.n_post))
        dev = self.indices.device
        s_indptr = torch.empty(n_rows * S + 1, dtype=torch.int64, device=dev)
        s_indices = s_perm = None
        if regroup:
            s_indices = torch.empty(self.nnz, dtype=torch.int32, device=dev)
            s_perm = torch.empty(self.nnz, dtype=torch.int32, device=dev)
        check(lib().bsx_sliced_build(C.byref(st), ptr(s_indptr), ptr(s_indices) if regroup else None,
                                     ptr(s_perm) if regroup else None, _lib.current_stream()))
        return s_indptr, s_indices, s_perm

    def _sliced_struct(self, weights: torch.Tensor):
        """``bsx_conn_t`` of the copy whose rows are grouped by output slice (built once); the
        regrouped weights are kept until the weight tensor changes."""
        if 'sliced' not in self._derived:
            self._derived['sliced'] = self._group_offsets(self._struct(), self.shape[0], regroup=True)
        s_indptr, s_indices, s_perm = self._derived['sliced']
        ws_ = self._permuted_weights('s', weights, s_perm) if self.hetero else weights.contiguous()
        s = BsxConn()
        s.n_pre, s.n_post = self.shape
        s.conn_num = 0
        s.nnz = self.nnz
        s.indices = s_indices.data_ptr() if self.nnz else None
        s.indptr = s_indptr.data_ptr()
        s.indptr_is_64 = 1
        s.hetero = int(self.hetero)
        s.weights = ws_.data_ptr()
        s._keep = (ws_, s_indptr, s_indices)
        return s

    def _transposed_sliced_struct(self, weights: torch.Tensor):
        """``bsx_conn_t`` of the transposed copy regrouped by output slice (of the transposed
        product, i.e. by presynaptic neuron).  Built once; its permutation is composed with the
        transposed copy's, so the weights are gathered from the original array in one pass."""
        t = self.transposed()
        n_pre, n_post = self.shape
        if 't_groups' not in self._derived:
            b = BsxConn()
            b.n_pre, b.n_post = t.n_rows, t.n_cols
            b.conn_num, b.nnz = 0, self.nnz
            b.indices = t.indices.data_ptr() if self.nnz else None
            b.indptr, b.indptr_is_64 = t.indptr.data_ptr(), 1
            b.hetero, b.weights = 0, self.data.data_ptr()
            s_indptr, s_indices, s_perm = self._group_offsets(b, t.n_rows, regroup=True)
            comp = t.perm[s_perm.long()].contiguous() if self.nnz else s_perm
            self._derived['t_groups'] = (s_indptr, s_indices, comp)
        s_indptr, s_indices, comp = self._derived['t_groups']
        wt = self._permuted_weights('ts', weights, comp) if self.hetero else weights.contiguous()
        s = BsxConn()
        s.n_pre, s.n_post = t.n_rows, t.n_cols
        s.conn_num = 0
        s.nnz = self.nnz
        s.indices = s_indices.data_ptr() if self.nnz else None
        s.indptr = s_indptr.data_ptr()
        s.indptr_is_64 = 1
        s.hetero = int(self.hetero)
        s.weights = wt.data_ptr()
        s._keep = (wt, s_indptr, s_indices)
        return s

    def _fixed_scale(self, layout: str, st: BsxConn, weights: torch.Tensor, if_settled: bool = False):
        """Scale (log2) of the fixed-point scatter over a derived layout: the largest that cannot
        overflow, from the largest column sum of ``|w|`` (one pass over the weights and a stream
        synchronisation).  Kept until the weight tensor changes.  ``if_settled``: return ``None``
        instead of recomputing once the weights have changed twice — a training loop, where a
        pass per step would cost more than the float atomics it avoids."""
        if not self.hetero:
            return 0
        wsrc = weights.contiguous()
        key = (wsrc.data_ptr(), wsrc._version, wsrc.numel())
        cached = self._derived.get('scale_' + layout)
        if cached is not None and cached[0] == key:
            return cached[1]
        misses = 0 if cached is None else cached[2] + 1
        if if_settled and misses >= 2:
            return None
        nbytes = lib().bsx_fixed_scale_workspace_bytes(st.n_post)
        ws = torch.empty(max(nbytes, 8), dtype=torch.uint8, device=self.indices.device)
        s = C.c_int32(0)
        check(lib().bsx_fixed_scale_log2(C.byref(st), ptr(ws), nbytes, C.byref(s), _lib.current_stream()))
        self._derived['scale_' + layout] = (key, int(s.value), misses)
        return int(s.value)

    def _packed(self, layout: str, st: BsxConn, weights: torch.Tensor, scale: int):
        """Compressed form of a sliced copy: 16-bit column offsets inside the slice (built once)
        and, for heterogeneous weights, the weights in ``2^-scale`` fixed point (kept until the
        weight tensor or the scale changes)."""
        dev = self.indices.device
        loc = self._derived.get('loc_' + layout)
        if loc is None:
            loc = torch.empty(max(self.nnz, 1), dtype=torch.int16, device=dev)
            check(lib().bsx_sliced_compress(C.byref(st), ptr(loc), _lib.current_stream()))
            self._derived['loc_' + layout] = loc
        q = None
        if self.hetero:
            wsrc = weights.contiguous()
            key = (wsrc.data_ptr(), wsrc._version, wsrc.numel(), scale)
            cached = self._derived.get('q_' + layout)
            if cached is not None and cached[0] == key:
                q = cached[1]
            else:
                q = torch.empty(max(self.nnz, 1), dtype=torch.int32, device=dev)
                check(lib().bsx_quantize_f32(st.weights, self.nnz, scale, ptr(q), _lib.current_stream()))
                self._derived['q_' + layout] = (key, q, wsrc)
        return loc, q

    def _sliced_call(self, layout: str, st: BsxConn, weights: torch.Tensor, scale, xb, fmt, batch, out, accumulate):
        """One launch of the scatter that keeps output slices in shared memory, over the sliced copy
        ``st`` (``layout``: ``'s'`` forward, ``'ts'`` transposed).  ``scale`` None: float sums
        (heterogeneous) over the 32-bit layout.  Otherwise order-free sums over the compressed
        layout (``PACKED_SLICES``) or the 32-bit one."""
        stream = _lib.current_stream()
        if scale is None and self.hetero:
            check(lib().bsx_event_vecmat_sliced(C.byref(st), ptr(xb), fmt, batch, ptr(out), int(accumulate), stream))
        elif PACKED_SLICES:
            loc, q = self._packed(layout, st, weights, scale or 0)
            check(lib().bsx_event_vecmat_sliced16(C.byref(st), ptr(loc), ptr(q), ptr(xb), fmt, batch, ptr(out),
                                                  int(accumulate), scale or 0, stream))
        else:
            check(lib().bsx_event_vecmat_sliced_fixed(C.byref(st), ptr(xb), fmt, batch, ptr(out), int(accumulate),
                                                      scale or 0, stream))

    @staticmethod
    def _fixed_applies(n_out: int, batch: int) -> bool:
        """The fixed-point scatter keeps output slices in shared memory: batches of 16 and more
        over at most 131 072 outputs."""
        return 16 <= batch <= 65535 and n_out <= 131072

    # -- products ------------------------------------------------------------------
    def _vecmat(self, x, event: bool, method: str = 'scatter'):
        return _VecMat.apply(x, self.data, self, event, method)

    def __rmatmul__(self, x):
        if isinstance(x, EventArray):
            return self._vecmat(x.value, event=True)
        if isinstance(x, torch.Tensor):
            return self._vecmat(x, event=False)
        return NotImplemented

    def __matmul__(self, v):
        if isinstance(v, EventArray):
            return event_matvec(self, v.value, method=self.matvec_method)
        if isinstance(v, torch.Tensor):
            return float_matvec(self, v)
        return NotImplemented


class FixedPostNumConn(_SparseConn):
    """``(weight, indices)`` with a fixed number of targets per presynaptic row
    (``brainevent.FixedPostNumConn``, ``_event_fixedprob.py:176-181``)."""

    def __init__(self, data_indices, shape):
        data, indices = data_indices
        if indices.dim() != 2 or indices.shape[0] != shape[0]:
            raise ValueError('indices must have shape (n_pre, conn_num)')
        super().__init__(data, indices, None, shape)


class CSR(_SparseConn):
    """``(weight, indices, indptr)`` compressed sparse rows
    (``brainevent.CSR``, ``_event_fixedprob.py:191-196``)."""

    def __init__(self, data_indices_indptr, shape):
        data, indices, indptr = data_indices_indptr
        if indices.dim() != 1:
            raise ValueError('CSR indices must be one-dimensional')
        super().__init__(data, indices, indptr, shape)


class _InDegreeConn:
    """Connectivity stored by POSTSYNAPTIC neuron: every column of the ``(n_pre, n_post)`` matrix
    lists its presynaptic partners (a fixed number of them, or compressed sparse columns).

    The arrays are exactly those of an out-degree layout of the transposed matrix, so the
    products run on the same kernels with the roles swapped: ``x @ conn`` is the row-gather
    ``M @ x`` over ``M = conn^T`` (every output is summed by one warp in a fixed order, hence
    deterministic), ``conn @ v`` is the scatter ``v @ M``.  ``matvec_method`` selects the
    event-driven form of ``EventArray(spk) @ conn`` (``'scatter'``, over a presynaptic-major copy
    built once) as for the out-degree containers.
    """

    def __init__(self, mirror: _SparseConn, shape):
        self.shape = (int(shape[0]), int(shape[1]))
        self._m = mirror                   # out-degree layout of the transposed matrix
        self.matvec_method = 'gather'

    data = property(lambda self: self._m.data)
    indices = property(lambda self: self._m.indices)
    indptr = property(lambda self: self._m.indptr)
    hetero = property(lambda self: self._m.hetero)
    nnz = property(lambda self: self._m.nnz)

    def with_data(self, data):
        new = object.__new__(type(self))
        new.__dict__.update(self.__dict__)
        new._m = self._m.with_data(data)
        return new

    def validate(self):
        self._m.validate()
        return self

    def _gather(self, x, event: bool):
        return _MatVec.apply(x, self._m.data, self._m, event, self.matvec_method)

    def __rmatmul__(self, x):              # x @ conn -> (…, n_post)
        if isinstance(x, EventArray):
            return self._gather(x.value, event=True)
        if isinstance(x, torch.Tensor):
            return self._gather(x, event=False)
        return NotImplemented

    def __matmul__(self, v):               # conn @ v -> (…, n_pre)
        if isinstance(v, EventArray):
            return self._m._vecmat(v.value, event=True)
        if isinstance(v, torch.Tensor):
            return self._m._vecmat(v, event=False)
        return NotImplemented


class FixedPreNumConn(_InDegreeConn):
    """``(weight, indices)`` with a fixed number of presynaptic partners per postsynaptic
    neuron: ``indices`` has shape ``(n_post, conn_num)`` with values in ``[0, n_pre)``
    (``brainevent.FixedPreNumConn``, the layout the reference's ``efferent_target='pre'``
    branch names, ``_event_fixedprob.py:123-140``)."""

    def __init__(self, data_indices, shape):
        data, indices = data_indices
        if indices.dim() != 2 or indices.shape[0] != shape[1]:
            raise ValueError('indices must have shape (n_post, conn_num)')
        super().__init__(FixedPostNumConn((data, indices), (shape[1], shape[0])), shape)


class CSC(_InDegreeConn):
    """``(weight, indices, indptr)`` compressed sparse columns: ``indptr`` has ``n_post + 1``
    entries and ``indices`` holds presynaptic ids (``brainevent.CSC``)."""

    def __init__(self, data_indices_indptr, shape):
        data, indices, indptr = data_indices_indptr
        if indptr.numel() != shape[1] + 1:
            raise ValueError('indptr must have n_post + 1 entries')
        super().__init__(CSR((data, indices, indptr), (shape[1], shape[0])), shape)


# ----------------------------------------------------------------------------
# raw calls (no autograd)
# ----------------------------------------------------------------------------

def _flatten_batch(x: torch.Tensor, n: int):
    if x.shape[-1] != n:
        raise ValueError(f'last dimension is {x.shape[-1]}, expected {n}')
    lead = tuple(x.shape[:-1])
    xb = x.reshape(-1, n)
    if not xb.is_contiguous():
        xb = xb.contiguous()
    return xb, lead


def _raw_vecmat(conn: _SparseConn, x: torch.Tensor, weights: torch.Tensor, event: bool,
                method: str = 'scatter', out: Optional[torch.Tensor] = None, accumulate: bool = False):
    _require_cuda(x, 'input')
    n_pre, n_post = conn.shape
    xb, lead = _flatten_batch(x, n_pre)
    batch = xb.shape[0]
    if out is None:
        out = torch.empty((batch, n_post), dtype=torch.float32, device=x.device)
        accumulate = False
    stream = _lib.current_stream()
    if method == 'fixed':
        # order-free sums: the fixed-point scatter where it applies, the order-fixing gather elsewhere
        if event and conn._fixed_applies(n_post, batch):
            st_s = conn._sliced_struct(weights)
            scale = conn._fixed_scale('s', st_s, weights)
            conn._sliced_call('s', st_s, weights, scale, xb, spike_format_of(xb), batch, out, accumulate)
            return out.reshape(lead + (n_post,))
        method = 'gather' if event else 'scatter'
    if event and method == 'gather':
        # deterministic post-centric form: event matvec over the transposed copy
        st = conn._transposed_struct(weights)
        fmt = spike_format_of(xb)
        ws_bytes = lib().bsx_event_matvec_workspace_bytes(batch, n_pre)
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=x.device)
        if accumulate:
            tmp = torch.empty_like(out)
            check(lib().bsx_event_matvec(C.byref(st), ptr(xb), fmt, batch, ptr(tmp), ptr(ws), ws_bytes, stream))
            out += tmp
        else:
            check(lib().bsx_event_matvec(C.byref(st), ptr(xb), fmt, batch, ptr(out), ptr(ws), ws_bytes, stream))
        return out.reshape(lead + (n_post,))
    if method not in ('scatter', 'gather', 'float'):
        raise ValueError(f"method must be 'scatter', 'gather', 'fixed' or 'float', got {method!r}")
    st = conn._struct(weights)
    if event and lib().bsx_event_vecmat_variant(C.byref(st), spike_format_of(xb), batch) == _lib.VECMAT_SHARED_SLICES:
        # a batch that fills the GPU: one launch over the copy whose rows are grouped by output slice.
        # Heterogeneous weights are summed in fixed point (order-free and faster than float atomics in
        # shared memory) unless float sums are asked for.
        st_s = conn._sliced_struct(weights)
        scale = conn._fixed_scale('s', st_s, weights, if_settled=True) if conn.hetero and method != 'float' else None
        conn._sliced_call('s', st_s, weights, scale, xb, spike_format_of(xb), batch, out, accumulate)
        return out.reshape(lead + (n_post,))
    ws_bytes = lib().bsx_event_vecmat_workspace_bytes(batch, n_pre)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=x.device)
    if event:
        fmt = spike_format_of(xb)
        check(lib().bsx_event_vecmat(C.byref(st), ptr(xb), fmt, batch, ptr(out), int(accumulate),
                                     ptr(ws), ws_bytes, stream))
    else:
        if xb.dtype != torch.float32:
            xb = xb.to(torch.float32)
        check(lib().bsx_float_vecmat(C.byref(st), ptr(xb), batch, ptr(out), int(accumulate),
                                     ptr(ws), ws_bytes, stream))
    return out.reshape(lead + (n_post,))


def event_vecmat(conn: _SparseConn, spk: torch.Tensor, method: str = 'scatter'):
    """``EventArray(spk) @ conn`` (differentiable when ``spk`` is float)."""
    return conn._vecmat(spk, event=True, method=method)


def float_vecmat(conn: _SparseConn, x: torch.Tensor):
    """``x @ conn`` for float ``x``."""
    return conn._vecmat(x, event=False)


def event_matvec(conn: _SparseConn, spk: torch.Tensor, bits: bool = False, method: str = 'gather'):
    """``conn @ EventArray(spk)``: ``y[i] = sum_k w[i,k] [spk[idx[i,k]] != 0]``.
    ``bits=True`` takes packed uint32/int32 words (``(…, ceil(n_post/32))``).

    method : ``'gather'`` walks every row and tests its targets' spike bits — deterministic,
        cost independent of the firing rate.  ``'scatter'`` is the event-driven form: the
        active postsynaptic neurons scatter along the transposed copy (built once), cost
        proportional to the events — about twice as fast at 1 % firing, slower above ≈ 3 %;
        heterogeneous sums then depend on the order of the atomic adds (last-bit differences).
        Batches that fill the GPU sum heterogeneous weights in fixed point (``bsx_fixed_scale_log2``),
        which is order-free and faster; ``'float'`` keeps float atomics there.
        ``'fixed'`` asks for order-free sums at any batch size: the fixed-point scatter for batches
        of 16 and more, the gather otherwise — as reproducible as ``'gather'``, every addend rounded
        to ``2^-scale``.
    """
    _require_cuda(spk, 'spikes')
    if method not in ('gather', 'scatter', 'fixed', 'float'):
        raise ValueError(f"method must be 'gather', 'scatter', 'fixed' or 'float', got {method!r}")
    n_pre, n_post = conn.shape
    if bits:
        words = (n_post + 31) // 32
        xb, lead = _flatten_batch(spk, words)
        fmt = _lib.SPK_BITS32
    else:
        xb, lead = _flatten_batch(spk, n_post)
        fmt = spike_format_of(xb)
    batch = xb.shape[0]
    out = torch.empty((batch, n_pre), dtype=torch.float32, device=spk.device)
    if method == 'fixed':
        if conn._fixed_applies(n_pre, batch):
            st_ts = conn._transposed_sliced_struct(conn.data)
            scale = conn._fixed_scale('ts', st_ts, conn.data)
            conn._sliced_call('ts', st_ts, conn.data, scale, xb, fmt, batch, out, False)
            return out.reshape(lead + (n_pre,))
        method = 'gather'
    if method in ('scatter', 'float'):
        st = conn._transposed_struct(conn.data)
        if lib().bsx_event_vecmat_variant(C.byref(st), fmt, batch) == _lib.VECMAT_SHARED_SLICES:
            st_ts = conn._transposed_sliced_struct(conn.data)
            scale = (conn._fixed_scale('ts', st_ts, conn.data, if_settled=True)
                     if conn.hetero and method == 'scatter' else None)
            conn._sliced_call('ts', st_ts, conn.data, scale, xb, fmt, batch, out, False)
            return out.reshape(lead + (n_pre,))
        ws_bytes = lib().bsx_event_vecmat_workspace_bytes(batch, n_post)
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=spk.device)
        check(lib().bsx_event_vecmat(C.byref(st), ptr(xb), fmt, batch, ptr(out), 0, ptr(ws), ws_bytes,
                                     _lib.current_stream()))
        return out.reshape(lead + (n_pre,))
    st = conn._struct()
    ws_bytes = lib().bsx_event_matvec_workspace_bytes(batch, n_post)
    ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=spk.device)
    check(lib().bsx_event_matvec(C.byref(st), ptr(xb), fmt, batch, ptr(out), ptr(ws), ws_bytes,
                                 _lib.current_stream()))
    return out.reshape(lead + (n_pre,))


def float_matvec(conn: _SparseConn, v: torch.Tensor, weights: Optional[torch.Tensor] = None):
    """``conn @ v`` for float ``v`` (not recorded by autograd; the in-degree containers wrap it)."""
    _require_cuda(v, 'v')
    n_pre, n_post = conn.shape
    vb, lead = _flatten_batch(v.to(torch.float32), n_post)
    out = torch.empty((vb.shape[0], n_pre), dtype=torch.float32, device=v.device)
    st = conn._struct(weights)
    check(lib().bsx_float_matvec(C.byref(st), ptr(vb), vb.shape[0], ptr(out), _lib.current_stream()))
    return out.reshape(lead + (n_pre,))


def pack_spikes(spk: torch.Tensor) -> torch.Tensor:
    """Packs ``(…, n)`` spikes into ``(…, ceil(n/32))`` int32 words (bit ``i % 32`` of word ``i // 32``)."""
    _require_cuda(spk, 'spikes')
    n = spk.shape[-1]
    xb, lead = _flatten_batch(spk, n)
    words = (n + 31) // 32
    out = torch.empty((xb.shape[0], words), dtype=torch.int32, device=spk.device)
    check(lib().bsx_pack_spikes(ptr(xb), spike_format_of(xb), xb.shape[0], n, ptr(out), _lib.current_stream()))
    return out.reshape(lead + (words,))


def _raw_vjp(conn: _SparseConn, x: torch.Tensor, weights: torch.Tensor, ct: torch.Tensor, event: bool,
             need_dx: bool, need_dw: bool):
    n_pre, n_post = conn.shape
    xb, lead = _flatten_batch(x, n_pre)
    ctb, _ = _flatten_batch(ct.to(torch.float32), n_post)
    batch = xb.shape[0]
    if xb.dtype not in (torch.bool, torch.uint8, torch.float32):
        xb = xb.to(torch.float32)
    dx = torch.empty((batch, n_pre), dtype=torch.float32, device=ct.device) if need_dx else None
    dw = None
    if need_dw:
        dw = torch.empty(conn.indices.shape if conn.hetero else (1,), dtype=torch.float32, device=ct.device)
    st = conn._struct(weights)
    if batch >= 4:      # batch-minor cotangent: one index fetch serves 64 batch lanes
        ws_bytes = lib().bsx_vecmat_vjp_batched_workspace_bytes(batch, n_post)
        ws = torch.empty(max(ws_bytes, 1), dtype=torch.uint8, device=ct.device)
        check(lib().bsx_vecmat_vjp_batched(C.byref(st), ptr(xb), spike_format_of(xb), int(event), ptr(ctb), batch,
                                           ptr(dx), ptr(dw), ptr(ws), ws_bytes, _lib.current_stream()))
    else:
        check(lib().bsx_vecmat_vjp(C.byref(st), ptr(xb), spike_format_of(xb), int(event), ptr(ctb), batch,
                                   ptr(dx), ptr(dw), _lib.current_stream()))
    if dx is not None:
        dx = dx.reshape(lead + (n_pre,))
    if dw is not None and not conn.hetero:
        dw = dw.reshape(weights.shape)
    return dx, dw


class _VecMat(torch.autograd.Function):
    """``y = x @ W`` with the reverse- and forward-mode rules the reference's tests
    pin (``brainstate/nn/_event_fixedprob_test.py:56-126``).

    ``dx = ct @ W^T`` is dense also for an event input (the gradient flows through
    the value, ``_event_linear.py:84-91``); ``dw`` uses the event indicator for the
    event product and the value for the float product.
    """

    @staticmethod
    def forward(x, weights, conn, event, method):
        return _raw_vecmat(conn, x, weights, event, method)

    @staticmethod
    def setup_context(ctx, inputs, output):
        x, weights, conn, event, method = inputs
        ctx.conn, ctx.event = conn, event
        ctx.save_for_backward(x, weights)
        ctx.save_for_forward(x, weights)
        ctx.x_differentiable = x.dtype.is_floating_point

    @staticmethod
    def backward(ctx, ct):
        x, weights = ctx.saved_tensors
        need_dx = ctx.needs_input_grad[0] and ctx.x_differentiable
        need_dw = ctx.needs_input_grad[1]
        dx, dw = _raw_vjp(ctx.conn, x, weights, ct.contiguous(), ctx.event, need_dx, need_dw)
        if dx is not None and dx.dtype != x.dtype:
            dx = dx.to(x.dtype)
        return dx, dw, None, None, None

    @staticmethod
    def jvp(ctx, x_dot, w_dot, *_):
        x, weights = ctx.saved_tensors
        conn = ctx.conn
        out = None
        if x_dot is not None:
            out = _raw_vecmat(conn, x_dot.to(torch.float32), weights, event=False)
        if w_dot is not None:
            wd = w_dot.to(torch.float32)
            term = _raw_vecmat(conn.with_data(wd), x, wd, event=ctx.event)
            out = term if out is None else out + term
        return out


class _MatVec(torch.autograd.Function):
    """``y = M @ x`` over an out-degree layout ``M`` (``y[j] = sum_k w[j,k] x[idx[j,k]]``): the
    product of the in-degree containers.  ``dx = ct @ M`` is a scatter of the cotangent,
    ``dw[j,k] = ct[j] * x[idx[j,k]]`` (the event indicator for an event input) is the weight
    cotangent of the scatter product with the operands exchanged."""

    @staticmethod
    def forward(x, weights, conn, event, method):
        c = conn.with_data(weights)
        if event:
            return event_matvec(c, x, method=method)
        return float_matvec(c, x, weights)

    @staticmethod
    def setup_context(ctx, inputs, output):
        x, weights, conn, event, method = inputs
        ctx.conn, ctx.event, ctx.method = conn, event, method
        ctx.save_for_backward(x, weights)
        ctx.save_for_forward(x, weights)
        ctx.x_differentiable = x.dtype.is_floating_point

    @staticmethod
    def backward(ctx, ct):
        x, weights = ctx.saved_tensors
        conn = ctx.conn
        ct = ct.contiguous().to(torch.float32)
        dx = dw = None
        if ctx.needs_input_grad[0] and ctx.x_differentiable:
            dx = _raw_vecmat(conn, ct, weights, event=False).to(x.dtype)
        if ctx.needs_input_grad[1]:
            xv = (x != 0).to(torch.float32) if ctx.event else x.to(torch.float32)
            _, dw = _raw_vjp(conn, ct, weights, xv, event=False, need_dx=False, need_dw=True)
        return dx, dw, None, None, None

    @staticmethod
    def jvp(ctx, x_dot, w_dot, *_):
        x, weights = ctx.saved_tensors
        conn = ctx.conn
        out = None
        if x_dot is not None:
            out = float_matvec(conn, x_dot.to(torch.float32), weights)
        if w_dot is not None:
            wd = w_dot.to(torch.float32)
            c = conn.with_data(wd)
            term = event_matvec(c, x, method=ctx.method) if ctx.event else float_matvec(c, x, wd)
            out = term if out is None else out + term
        return out
